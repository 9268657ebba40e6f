// Staging copies done by a kernel instead of the copy engine: pinned (mapped) host memory
// <-> device memory, a few tens of KB per decode step.  Inside a CUDA graph a memcpy node
// costs about 10 us of fixed latency on B200 and cuts the chain of programmatically dependent
// GEMV launches; a small kernel moves the same bytes over PCIe in 2-3 us, and the GEMV that
// follows can fill its weight ring while it runs.  No counterpart in the reference (its
// end-to-end path keeps activations on the device, benchmarks/bench_e2e.py:103-155).
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

__global__ void __launch_bounds__(256) stage_copy_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src,
                                                         size_t bytes) {
  pdl_launch_dependents();  // a dependent launch may start its own prologue now
  pdl_wait();               // launched early itself: the producer of src must be complete
  const size_t n16 = bytes >> 4;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride)
    reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
  for (size_t i = (n16 << 4) + static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < bytes; i += stride) dst[i] = src[i];
}

}  // namespace

int launch_stage_copy(void *dst, const void *src, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) return RDQ_OK;
  size_t blocks = (bytes + 256 * 16 - 1) / (256 * 16);
  if (blocks > 64) blocks = 64;
  // launched with programmatic stream serialization: the kernel may become resident while its
  // predecessor drains and waits for it inside (griddepcontrol.wait)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  uint8_t *d = static_cast<uint8_t *>(dst);
  const uint8_t *sp = static_cast<const uint8_t *>(src);
  void *params[3] = {&d, &sp, &bytes};
  RDQ_CUDA(cudaLaunchKernelExC(&cfg, reinterpret_cast<const void *>(stage_copy_kernel), params));
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
