// Staging copies done by a kernel instead of the copy engine: pinned (mapped) host memory
// <-> device memory, a few tens of KB per decode step.  Inside a CUDA graph a memcpy node
// costs about 10 us of fixed latency on B200 and cuts the chain of programmatically dependent
// GEMV launches; a small kernel moves the same bytes over PCIe in 2-3 us, and the GEMV that
// follows can fill its weight ring while it runs.  No counterpart in the reference (its
// end-to-end path keeps activations on the device, benchmarks/bench_e2e.py:103-155).
#include "rdq_kernels.cuh"

namespace rdq {

namespace {

// state: [0] CTAs done in this launch, [1] launches completed.  With a non-null `flag` (pinned
// host memory) the last CTA to finish -- after a system-scope fence behind every CTA's stores --
// writes the number of completed launches there: a host thread that polls the word sees the
// copy complete without a stream synchronisation.
__global__ void __launch_bounds__(256) stage_copy_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src,
                                                         size_t bytes, int *state, int *flag) {
  pdl_launch_dependents();  // a dependent launch may start its own prologue now
  pdl_wait();               // launched early itself: the producer of src must be complete
  // every CTA takes an equal, contiguous share (the grid has one CTA per SM, see linger())
  const size_t n16 = bytes >> 4;
  const size_t per = (n16 + gridDim.x - 1) / gridDim.x;
  const size_t lo = per * blockIdx.x, hi = lo + per < n16 ? lo + per : n16;
  if (lo >= n16 && !(blockIdx.x == 0 && (bytes & 15))) {
    if (flag == nullptr) {
      linger(1500);
      return;
    }
  } else {
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x)
      reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(src)[i];
    if (blockIdx.x == 0)
      for (size_t i = (n16 << 4) + threadIdx.x; i < bytes; i += blockDim.x) dst[i] = src[i];
  }
  if (flag != nullptr) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&state[0], 1) == static_cast<int>(gridDim.x) - 1) {
      __threadfence_system();
      const int done = state[1] + 1;
      state[1] = done;
      state[0] = 0;
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(done) : "memory");
    }
  }
}

}  // namespace

int launch_stage_copy(void *dst, const void *src, size_t bytes, int *state, int *flag, cudaStream_t stream) {
  if (bytes == 0 && flag == nullptr) return RDQ_OK;
  // One CTA per SM with the footprint that keeps a second one off the SM (pin_slot): the kernel
  // sits in a chain of GEMV launches.  Launched with programmatic stream serialization: it may
  // become resident while its predecessor drains and waits for it inside (griddepcontrol.wait).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(sm_count()));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = kSlotSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  uint8_t *d = static_cast<uint8_t *>(dst);
  const uint8_t *sp = static_cast<const uint8_t *>(src);
  void *params[5] = {&d, &sp, &bytes, &state, &flag};
  RDQ_CUDA(pin_slot(reinterpret_cast<const void *>(stage_copy_kernel), kSlotSmem));
  RDQ_CUDA(cudaLaunchKernelExC(&cfg, reinterpret_cast<const void *>(stage_copy_kernel), params));
  RDQ_CUDA(cudaGetLastError());
  return RDQ_OK;
}

}  // namespace rdq
