/*
 * rdq_b200.h -- C ABI of the B200 (sm_100a) mixed-precision linear operator.
 *
 * One shared library (librdq_b200.so) exports these entry points.  Every
 * pointer is a plain device pointer unless stated otherwise; no torch types
 * cross this boundary.  All entry points
 *   - launch on the CUDA stream handed in (a cudaStream_t passed as void*,
 *     NULL = legacy default stream) of the CURRENT device,
 *   - return 0 on success and a negative RDQ_E_* code on failure, with a
 *     human readable message available from rdq_last_error() (thread local),
 *   - may be called from several host threads; state that outlives a launch is
 *     limited to: the caller-owned scratch of the GEMVs (`workspace` idle
 *     pattern, `counters` zero between launches), per-device caches of device
 *     attributes inside the library, the device array of
 *     rdq_gemv_tiled_noalloc, and one status word per device for the GEMM.
 *     A kernel whose bounded device-side wait runs out leaves a non-zero status
 *     word behind; the rdq_*_status calls below turn that into RDQ_E_DEVICE.
 *
 * Tensor layouts are the packed-checkpoint layouts of the reference
 * (rdquant/integrations/hf_export.py:58-125), rows in permuted
 * (format-grouped) channel order NVFP4 | FP8 | FP16:
 *   w_fp4         u8  [n_fp4, K/2]   byte = (code[2j+1] << 4) | code[2j]
 *   w_fp4_scales  u8  [n_fp4, K/16]  E4M3 bits, one per 16 consecutive k
 *   w_fp8         u8  [n_fp8, K]     E4M3 bits
 *   w_fp8_scales  f32 [n_fp8]        one scale per channel
 *   w_fp16        f16 [n_fp16, K]    (bf16 accepted by rdq_dequant_packed)
 *   inv_perm      i32 [N]            y[j] = y_perm[inv_perm[j]]
 *   perm          i32 [N]            perm[inv_perm[j]] = j ; permuted row p is
 *                                    original channel perm[p]
 * Dequantised value of an NVFP4 element is LUT[code] * e4m3(block scale); the
 * `w_fp4_global_scale` argument multiplies that (reference kernels do the
 * same, rdquant/csrc/fused_gemv.cu:673-674).  Checkpoints written by
 * quantize_model store absolute block scales, so their callers pass 1.0
 * (rdquant/core/formats.py:145-159 ignores the stored global scale).
 */
#ifndef RDQ_B200_H_
#define RDQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RDQ_OK               0
#define RDQ_E_INVALID       -1  /* bad shape / alignment / null pointer        */
#define RDQ_E_UNSUPPORTED   -2  /* shape outside what the kernel family takes */
#define RDQ_E_CUDA          -3  /* a CUDA runtime call failed                 */
#define RDQ_E_DEVICE        -4  /* kernel reported a bounded wait ran out     */

#define RDQ_MAX_GEMV_M      16  /* decode GEMV accepts 1..16 activation rows  */

/* Library / build identification. */
int         rdq_version(void);
const char *rdq_last_error(void);

/*
 * Bit-exact dequantisation of one packed layer to FP16 [N, K] in ORIGINAL
 * channel order.  Replaces rdquant/inference.py:67-121
 * (_materialize_packed_groups) followed by cat()[inv_perm]
 * (rdquant/inference.py:828-841) and equals
 * QuantizedWeight.dequantize().half() (rdquant/quantize.py:50-69).
 * NVFP4: f16(LUT[code] * e4m3(scale) * global); FP8: f16(f32(e4m3) * scale);
 * FP16 group copied (fp16_is_bf16 != 0: bf16 -> f32 -> f16, round to nearest).
 * out_is_f32 != 0 writes FP32 [N, K] holding the unrounded FP32 products, which
 * is what rdquant.core.formats.dequantize returns (rdquant/core/formats.py:385-395).
 * inv_perm == NULL means identity.  K % 16 == 0 when n_fp4 > 0.
 */
int rdq_dequant_packed(const void *w_fp4, const void *w_fp4_scales,
                       float w_fp4_global_scale,
                       const void *w_fp8, const float *w_fp8_scales,
                       const void *w_fp16, int fp16_is_bf16,
                       const int32_t *inv_perm,
                       void *w_out, int out_is_f32,
                       int n_fp4, int n_fp8, int n_fp16, int K,
                       void *stream);

/*
 * Scratch rdq_gemv_tiled needs on the current device (the same for every
 * layer; N is accepted for symmetry with the reference's per-layer workspace,
 * rdquant/fused_gemv_pack.py:343-349): `*workspace_bytes` of float scratch,
 * one 16 x 16 slot per CTA of the grid (148 KB on a 148-SM GPU; every 32-bit
 * word must read 0xffffffff on first use), and
 * `*counter_bytes` of int32 counters (must start zeroed).
 */
int rdq_gemv_scratch_size(int N, size_t *workspace_bytes, size_t *counter_bytes);

/*
 * Decode GEMV, M <= 16:  y[m, perm[p]] = sum_k x[m,k] * W_perm[p,k] (+ bias).
 * One launch covers the NVFP4, FP8 and FP16 groups and scatters to original
 * channel order.  Replaces fused_mixed_gemv and the split-K family
 * (rdquant/csrc/rdquant_ops.h:75-85, :104-234; launchers
 * rdquant/csrc/fused_gemv.cu:2049-2393) and, together with the FP16 group,
 * the cat + index_select tail of rdquant/ops.py:60-66.
 *   x     f16 [M, K] row-major (ldx = K)
 *   y     f16 [M, N] row-major, every element written
 *   bias  f16 [N] in original channel order, or NULL
 *   workspace / counters: unused by this entry point (it runs the any-shape
 *     kernel, one warp per output channel, on the row-major tensors); they
 *     are the scratch of rdq_gemv_tiled.  May be NULL.
 *   flags: RDQ_GEMV_* below.
 * FP32 accumulation; NVFP4 weights enter the product as f16(LUT*scale)
 * (exact), FP8 weights as f16(e4m3) with the channel scale applied to the
 * FP32 sum.  Deterministic: repeated calls give identical bits.
 */
#define RDQ_GEMV_AUTO        0   /* default kernel choice                    */
#define RDQ_GEMV_GENERIC     1   /* force the any-shape kernel               */
#define RDQ_GEMV_PDL         16  /* launch with programmatic dependent launch:
                                    weights are prefetched before the wait on
                                    the preceding kernel, x is read after it */
#define RDQ_GEMV_TEST_TIMEOUT 64 /* tiled kernels, self-test: after its work one
                                    warp of CTA 0 waits, for a fraction of a
                                    millisecond, on a barrier nothing completes
                                    and reports the expired wait (status 9) */
int rdq_gemv_mixed(const void *x, int M,
                   const void *w_fp4, const void *w_fp4_scales,
                   float w_fp4_global_scale,
                   const void *w_fp8, const float *w_fp8_scales,
                   const void *w_fp16,
                   const int32_t *perm, const void *bias,
                   void *y,
                   int n_fp4, int n_fp8, int n_fp16, int K,
                   void *workspace, int32_t *counters,
                   int flags, void *stream);

/*
 * Tiled weight layout of the fast decode GEMV.  rdq_gemv_repack re-tiles the
 * row-major checkpoint tensors once per layer into `w_tiled`
 * (rdq_gemv_tiled_bytes bytes; 0 = shape has no tiled layout: groups must be
 * multiples of 16 rows, K must split into equal chunks of at most 2048
 * elements that are multiples of 64, and a tile may have at most 256 chunks).
 * 16 rows x one k chunk are stored as one contiguous block (rows skewed by 16
 * bytes against shared-memory bank conflicts) that is copied to shared memory
 * by a single bulk-async (TMA) copy.  Plays the role of the reference's
 * load-time
 * Marlin repack
 * (rdquant/fused_gemv_pack.py:151-172, :310-354).
 */
size_t rdq_gemv_tiled_bytes(int n_fp4, int n_fp8, int n_fp16, int K);
int rdq_gemv_repack(const void *w_fp4, const void *w_fp4_scales,
                    const void *w_fp8, const void *w_fp16,
                    void *w_tiled,
                    int n_fp4, int n_fp8, int n_fp16, int K, void *stream);

/*
 * Decode GEMV, M <= 16, on the tiled layout; same contract as rdq_gemv_mixed
 * (y[m, perm[p]] = sum_k x[m,k] * W_perm[p,k] (+ bias), FP32 accumulation,
 * deterministic).  Replaces the split-K kernels on repacked weights
 * (rdquant/csrc/rdquant_ops.h:104-234).  workspace / counters are required
 * (rdq_gemv_scratch_size).  Every 32-bit word of `workspace` must read
 * 0xffffffff on first use (the mark for "no partial sum stored"); every
 * completed launch leaves it in that state.  counters must be zero on first
 * use; counters[SM count] is a status word that stays 0 unless a bounded
 * device-side wait ran out.  Launches sharing one workspace / counters pair
 * must be ordered on one stream.
 * flags: RDQ_GEMV_PDL, RDQ_GEMV_TEST_TIMEOUT.
 */
int rdq_gemv_tiled(const void *x, int M,
                   const void *w_tiled, const float *w_fp8_scales,
                   float w_fp4_global_scale,
                   const int32_t *perm, const void *bias,
                   void *y,
                   int n_fp4, int n_fp8, int n_fp16, int K,
                   void *workspace, int32_t *counters,
                   int flags, void *stream);

/*
 * Column-parallel layers on the GPUs of one node (no counterpart in the
 * reference, which is single-GPU): the tiled GEMV with the all-gather of the
 * outputs fused into its epilogue.  Instead of y, the kernel stores its slice
 * -- y_slice[m, p] for the rows p of this rank's shard, in the shard's row
 * order -- into `n_dst` destinations: dst[d] is the place of this rank's slice
 * inside the gather buffer of GPU d (peer memory reachable by plain stores over
 * NVLink, e.g. symmetric memory; the local buffer is one of them).  When the
 * last epilogue warp of the grid has finished, it stores the launch number into
 * peer_flags[d] (this rank's flag word on GPU d) with release semantics.
 * peer_state: two zero-initialised int32 on this GPU, owned by the layer
 * ([0] warps done, [1] launches completed).  Everything else as rdq_gemv_tiled.
 *
 * rdq_peer_gather is the receiving side, one small kernel launched after the
 * layer's rdq_gemv_tiled_peer on the same stream: it waits until the flag words
 * flags[0 .. world) on this GPU all show the launch number that GEMV left in
 * peer_state[1] (bounded: about wait_ms milliseconds, then *status = 10 + the
 * rank that did not arrive and y is left untouched) and copies
 * y[i] = buffer[index[i]] for i < count (un-permute out of the gather buffer).
 * flags_pdl: RDQ_GEMV_PDL makes it take part in programmatic dependent launch.
 * Both calls are plain kernel launches: a whole decode step can be captured in
 * a CUDA graph.  No TMA or multicast access touches another GPU's memory.
 */
int rdq_gemv_tiled_peer(const void *x, int M,
                        const void *w_tiled, const float *w_fp8_scales,
                        float w_fp4_global_scale,
                        const int32_t *perm, const void *bias,
                        void *const *dst, int32_t *const *peer_flags, int n_dst,
                        int32_t *peer_state,
                        int n_fp4, int n_fp8, int n_fp16, int K,
                        void *workspace, int32_t *counters,
                        int flags, void *stream);
int rdq_peer_gather(const void *buffer, const long long *index, void *y,
                    long long count, const int32_t *flags, int world,
                    const int32_t *peer_state, int32_t *status, int wait_ms,
                    int flags_pdl, void *stream);

/*
 * rdq_gemv_tiled with an activation prologue: the kernel computes its
 * activation rows from what the preceding kernels of a decode step left in
 * global memory, instead of a separate kernel writing them first.  These are
 * the element-wise steps the reference's model code runs in PyTorch between
 * two quantized linears of a decoder block (quantized_model.py:108-190 replaces
 * only the nn.Linear modules; the norms and the MLP activation stay with the
 * host model).
 *   RDQ_XOP_ADD_RMSNORM  r = x (+ x_aux, f16 add, when x_aux is not NULL);
 *                        rows = f16(r * rsqrt(mean(r^2) + eps)) * x_weight[K];
 *                        r is written to x_out [M, K] when x_out is not NULL
 *                        (the updated residual stream; must not alias x or
 *                        x_aux, which every CTA reads)
 *   RDQ_XOP_SILU_MUL     x is [M, 2 K]; rows = f16(silu(x[:, :K])) * x[:, K:]
 * Supported while the launcher keeps the activation rows in shared memory:
 * rdq_gemv_tiled_stages_x(M, K) == 1 (M * (2 K + 16) bytes next to a ring of
 * at least three weight images; K = 9728 up to M = 2, K = 2560 up to M = 8);
 * otherwise RDQ_E_UNSUPPORTED and the caller runs rdq_add_rmsnorm /
 * rdq_silu_mul followed by rdq_gemv_tiled.  Everything else as rdq_gemv_tiled.
 */
#define RDQ_XOP_ADD_RMSNORM 1
#define RDQ_XOP_SILU_MUL 2
int rdq_gemv_tiled_stages_x(int M, int K);
int rdq_gemv_tiled_xop(int op, const void *x, const void *x_aux, const void *x_weight, void *x_out, float eps,
                       int M,
                       const void *w_tiled, const float *w_fp8_scales, float w_fp4_global_scale,
                       const int32_t *perm, const void *bias, void *y,
                       int n_fp4, int n_fp8, int n_fp16, int K,
                       void *workspace, int32_t *counters, int flags, void *stream);

/*
 * rdq_gemv_tiled for callers that cannot allocate device memory.  (No
 * counterpart in the reference.)  Some hosts of this library run where
 * cudaMalloc is off limits: serving loops that forbid allocation once they
 * are warm, code called from another framework's allocator callbacks, or a
 * runtime whose device-memory budget is fixed at start-up.  This variant takes no scratch pointers: the partial-tile slots
 * and the status word live in a device array that is part of the library image
 * (about 165 KB, held by every GPU that loads the library until the process
 * exits) and is sized for GPUs with up to 160 SMs; a larger GPU gets
 * RDQ_E_UNSUPPORTED and a message.  The call itself performs no cudaMalloc,
 * cudaFree or other allocating call.
 * The first call on each device looks up the array's device address and clears
 * it on `stream`; make that first call before any stream capture begins.  All
 * calls on a device share the one array: calls that may overlap on the GPU
 * (different streams, no ordering) race on it and must be serialised by the
 * caller.  Results are identical to rdq_gemv_tiled as long as no launch gave
 * up a wait; rdq_gemv_tiled_noalloc_status reports that and restores the array.
 * Set-up is guarded by a mutex: concurrent first calls are safe.
 */
int rdq_gemv_tiled_noalloc(const void *x, int M,
                           const void *w_tiled, const float *w_fp8_scales,
                           float w_fp4_global_scale,
                           const int32_t *perm, const void *bias,
                           void *y,
                           int n_fp4, int n_fp8, int n_fp16, int K,
                           int flags, void *stream);

/*
 * Device-side error reporting.  Every wait inside the kernels is bounded; a
 * kernel that gives one up records a code in a status word and drains instead
 * of hanging, and its results are invalid.  These calls synchronise `stream`,
 * read the status word and return RDQ_OK or RDQ_E_DEVICE (rdq_last_error()
 * names the wait).  With reset != 0 they also put the scratch back to its idle
 * state (status and flags zero, every partial-sum slot 0xffffffff), so that the
 * next launch starts clean.  None of them allocates.  The reference has no
 * counterpart: its launchers return void and check nothing
 * (rdquant/csrc/fused_gemv.cu:2049-2078).
 *   rdq_gemv_tiled_status          caller scratch of rdq_gemv_tiled
 *   rdq_gemv_tiled_noalloc_status  the library array of rdq_gemv_tiled_noalloc
 *   rdq_gemm_status                rdq_gemm_mixed / rdq_gemm_mixed_ws (one word
 *                                  per device)
 * rdq_gemm_test_timeout(1) makes later GEMM launches end with a wait that runs
 * out (self-test of this path, like RDQ_GEMV_TEST_TIMEOUT); 0 switches it off.
 */
int  rdq_gemv_tiled_status(void *workspace, int32_t *counters, int reset, void *stream);
int  rdq_gemv_tiled_noalloc_status(int reset, void *stream);
int  rdq_gemm_status(int reset, void *stream);
void rdq_gemm_test_timeout(int enable);

/*
 * Prefill GEMM, any M >= 1 (meant for M >= 16):
 *   y[m, j] = sum_k x[m,k] * W[j,k] (+ bias[j]),  j in original channel order.
 * Weight tiles are gathered by inv_perm, dequantised to FP16 into shared
 * memory and multiplied by tcgen05 kind::f16 MMAs with FP32 accumulators in
 * tensor memory.  Replaces the dense-prefill F.linear over a materialised
 * FP16 copy (rdquant/inference.py:679-687) and the 2x marlin_gemm + cat +
 * index_select path (rdquant/inference.py:620-677).
 *   x f16 [M, K], y f16 [M, N]; K % 64 == 0; inv_perm NULL = identity.
 */
int rdq_gemm_mixed(const void *x, int M,
                   const void *w_fp4, const void *w_fp4_scales,
                   float w_fp4_global_scale,
                   const void *w_fp8, const float *w_fp8_scales,
                   const void *w_fp16,
                   const int32_t *inv_perm, const void *bias,
                   void *y,
                   int n_fp4, int n_fp8, int n_fp16, int K,
                   void *stream);

/*
 * The same GEMM with caller scratch.  Problems with few output tiles (small M
 * or N) leave SMs idle; given `workspace` of at least the size
 * rdq_gemm_workspace_size reports (FP32, up to 4 x M x N), up to four CTAs share
 * the k range of a tile and a second kernel adds their sums, applies channel
 * scale and bias and writes y.  With workspace NULL (or too small) it behaves
 * like rdq_gemm_mixed.  Results may differ from the unsplit launch in the last
 * bit of the FP32 sum (different summation order); they are deterministic.
 * No counterpart in the reference (cuBLAS picks its own split there).
 */
int rdq_gemm_workspace_size(int M, int N, int K, size_t *bytes);
int rdq_gemm_mixed_ws(const void *x, int M,
                      const void *w_fp4, const void *w_fp4_scales,
                      float w_fp4_global_scale,
                      const void *w_fp8, const float *w_fp8_scales,
                      const void *w_fp16,
                      const int32_t *inv_perm, const void *bias,
                      void *y,
                      int n_fp4, int n_fp8, int n_fp16, int K,
                      void *workspace, size_t workspace_bytes, void *stream);

/*
 * Encoders: one format group of a float weight matrix -> its packed checkpoint
 * tensors, bit for bit what the reference's CPU encoders and checkpoint writer
 * produce (rdquant/core/formats.py:84-142 nvfp4_quantize, :166-193
 * fp8_quantize; rdquant/integrations/hf_export.py:81-102), plus what the
 * per-channel MSE of the format search needs (rdquant/core/formats.py:414-436
 * compute_mse_2d): row_sqerr[i] = sum_k (w[i,k] - dequant(quant(w))[i,k])^2.
 *   w        f32 (w_is_f32 != 0) or f16 [n, K], 16-byte aligned, K % 16 == 0
 *   NVFP4:   codes u8 [n, K/2], scales u8 [n, K/16] (E4M3 bits);
 *            max_scale (1 float, may be NULL) receives the largest block scale
 *            (the reference's global_scale metadata; 0 if all blocks are 0)
 *   FP8:     out u8 [n, K]; scale_out f32 [n] (may be NULL) receives the group's
 *            one scale = absmax / 448 in every entry; absmax_scratch: 1 float
 *   row_sqerr f32 [n] or NULL.
 */
int rdq_quantize_nvfp4(const void *w, int w_is_f32, int n, int K,
                       void *codes, void *scales, float *row_sqerr,
                       float *max_scale, void *stream);
int rdq_quantize_fp8(const void *w, int w_is_f32, int n, int K,
                     void *out, float *scale_out, float *row_sqerr,
                     float *absmax_scratch, void *stream);

/*
 * Decode-step glue: the small operations between the linears of a transformer
 * block at one token per sequence, as kernels that take part in programmatic
 * dependent launch like the GEMV (flags: RDQ_GEMV_PDL) -- each lets the next
 * kernel start at once, so the following GEMV fills its weight rings meanwhile,
 * and reads its inputs only after the preceding kernel has finished.  The
 * reference leaves this code to the HuggingFace model around its modules
 * (module boundary rdquant/inference.py:689-708; harness
 * benchmarks/bench_e2e.py:103-155).  All tensors f16 unless stated, row-major.
 * rdq_add_rmsnorm, rdq_rope_attn_decode, rdq_silu_mul (and rdq_peer_gather,
 * rdq_stage_copy) launch one CTA per SM, each sized so that an SM takes one of
 * them beside a GEMV's CTA and no second one, and CTAs without work stay
 * resident for a few microseconds: the tiled GEMV is fastest while every SM
 * holds exactly one CTA of each launch of the chain, and a kernel of a few CTAs
 * between two GEMVs breaks that (CTAs of the next GEMV pile up on the SMs that
 * free a slot first).
 *   rdq_add_rmsnorm     x[B,H] += delta[B,H] (delta may be NULL: no add);
 *                       out[B,H] = f16(x * rsqrt(mean(x^2) + eps)) * weight[H]
 *   rdq_qk_rope_cache   qkv[B, (nq + 2 nkv) * dh] (q heads, k heads, v heads):
 *                       per-head RMSNorm of q and k with q_norm / k_norm [dh]
 *                       (NULL: none), rotary embedding with cos / sin tables
 *                       [S, dh] (halves duplicated) at position *pos (device
 *                       int64); q -> q_out[B, nq, dh], k and v -> the caches
 *                       [B, nkv, S, dh] at row *pos
 *   rdq_attn_decode     out[B, nq * dh] = softmax(q K^T * scale) V over cache
 *                       rows 0 .. *pos, grouped-query (nq % nkv == 0), positions
 *                       split over CTAs and merged by a second small kernel;
 *                       scratch: rdq_attn_decode_scratch_size bytes (f32)
 *   rdq_rope_attn_decode  rdq_qk_rope_cache + rdq_attn_decode in ONE launch
 *                       (head_dim 64, 128 or 256, at most 16 query heads per KV
 *                       head): a CTA per (KV head, split of the rows) rotates
 *                       its query heads into shared memory, brings its K / V
 *                       rows in by cp.async tiles, and the last CTA of a KV head
 *                       to finish merges the splits.  Same rounding points as
 *                       the two separate calls (q and the new k are rounded to
 *                       f16 before use).  scratch:
 *                       rdq_rope_attn_decode_scratch_size bytes (enough for
 *                       every batch up to the B it is asked for), 16-byte
 *                       aligned, ZERO before the first call (it starts with the
 *                       arrival counters, which every call leaves at zero); not
 *                       to be shared by calls that may overlap.
 *   rdq_silu_mul        out[B,F] = silu(gate_up[B, 0:F]) * gate_up[B, F:2F]
 */
int rdq_add_rmsnorm(void *x, const void *delta, const void *weight, void *out,
                    int B, int H, float eps, int flags, void *stream);
int rdq_qk_rope_cache(const void *qkv, const void *q_norm, const void *k_norm,
                      const void *cos_table, const void *sin_table,
                      const long long *pos, void *q_out, void *k_cache,
                      void *v_cache, int B, int n_q_heads, int n_kv_heads,
                      int head_dim, int S, float eps, int flags, void *stream);
int rdq_attn_decode_scratch_size(int B, int n_q_heads, int head_dim, int S,
                                 size_t *bytes);
int rdq_attn_decode(const void *q, const void *k_cache, const void *v_cache,
                    const long long *pos, void *scratch, void *out, int B,
                    int n_q_heads, int n_kv_heads, int head_dim, int S,
                    float scale, int flags, void *stream);
int rdq_rope_attn_decode_scratch_size(int B, int n_q_heads, int n_kv_heads,
                                      int head_dim, int S, size_t *bytes);
int rdq_rope_attn_decode(const void *qkv, const void *q_norm, const void *k_norm,
                         const void *cos_table, const void *sin_table,
                         const long long *pos, void *k_cache, void *v_cache,
                         void *scratch, void *out, int B, int n_q_heads,
                         int n_kv_heads, int head_dim, int S, float scale,
                         float eps, int flags, void *stream);
int rdq_silu_mul(const void *gate_up, void *out, int B, int F, int flags,
                 void *stream);

/*
 * Copy `bytes` bytes between device-accessible buffers with a small kernel
 * rather than the copy engine: meant for the few KB of activations / results a
 * decode step moves between pinned (mapped) host memory and device memory
 * inside a CUDA graph, where a memcpy node costs ~10 us of fixed latency.
 * dst and src 16-byte aligned; either may be pinned host memory (the host
 * pointer is valid on the device under unified addressing).  No counterpart in
 * the reference, whose end-to-end path keeps activations on the device
 * (benchmarks/bench_e2e.py:103-155).
 */
int rdq_stage_copy(void *dst, const void *src, size_t bytes, void *stream);
/*
 * The same copy, followed by a completion signal the host can poll instead of
 * synchronising the stream: after a system-scope fence behind all of its
 * stores the kernel writes the number of rdq_stage_copy_signal launches
 * completed on `state` so far (1, 2, ...) to *flag.
 *   state: two device ints, zero before the first call, owned by the library
 *          between calls (CTAs done, launches completed)
 *   flag:  one int in pinned host memory (read with a volatile / acquire load)
 * A host thread that sees *flag == k may read what the k-th launch copied.
 */
int rdq_stage_copy_signal(void *dst, const void *src, size_t bytes,
                          int32_t *state, int32_t *flag, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* RDQ_B200_H_ */
