/* TEST INFRASTRUCTURE ONLY -- C restatement of the reference's CPU operator, used as the
 * timed CPU baseline of bench.py and cross-checked against oracle_np.py in the CPU tests.
 *
 * Restates rdquant/ops.py:32-68 on the reference's in-memory representation
 * (rdquant/core/formats.py:28-36): for every call it dequantises each format group from
 * int64 NVFP4 codes + float32 block scales (formats.py:145-159), float32 E4M3-valued FP8
 * data + one group scale (formats.py:196-199) and float16 data (formats.py:226-228), casts
 * the weight to float16 (ops.py:59), multiplies with float16 activations accumulating in
 * float32, concatenates, gathers by inv_perm (ops.py:62-63) and adds the bias.  Like the
 * reference it re-dequantises on every call.  Rows are spread over OpenMP threads.
 */
#include <stdint.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float kLut[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                               -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* Use `n` OpenMP threads from now on (launchers such as torchrun export OMP_NUM_THREADS=1;
 * the timed CPU baseline wants all host cores).  n <= 0 leaves the setting alone. */
void rdq_oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int rdq_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* y: float32 [M, N] in original channel order.  x: float16 bits [M, K]. */
void rdq_oracle_linear(const uint16_t *x, int M, int K,
                       const int64_t *codes4, const float *scales4, int n4,
                       const float *data8, float scale8, int n8,
                       const uint16_t *data16, int n16,
                       const int64_t *inv_perm, const float *bias,
                       float *y_perm_scratch, float *y) {
  const int N = n4 + n8 + n16;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < N; ++r) {
    float acc[16];
    for (int m = 0; m < M && m < 16; ++m) acc[m] = 0.0f;
    for (int k = 0; k < K; ++k) {
      _Float16 w;
      if (r < n4) {
        const size_t i = (size_t)r * K + k;
        w = (_Float16)(kLut[codes4[i]] * scales4[i / 16]);
      } else if (r < n4 + n8) {
        w = (_Float16)(data8[(size_t)(r - n4) * K + k] * scale8);
      } else {
        union { uint16_t u; _Float16 h; } c;
        c.u = data16[(size_t)(r - n4 - n8) * K + k];
        w = c.h;
      }
      const float wf = (float)w;
      for (int m = 0; m < M && m < 16; ++m) {
        union { uint16_t u; _Float16 h; } c;
        c.u = x[(size_t)m * K + k];
        acc[m] += wf * (float)c.h;
      }
    }
    for (int m = 0; m < M && m < 16; ++m) y_perm_scratch[(size_t)m * N + r] = acc[m];
  }
#pragma omp parallel for schedule(static)
  for (int j = 0; j < N; ++j) {
    const int64_t p = inv_perm ? inv_perm[j] : j;
    for (int m = 0; m < M && m < 16; ++m)
      y[(size_t)m * N + j] = y_perm_scratch[(size_t)m * N + p] + (bias ? bias[j] : 0.0f);
  }
}
