/* CPU restatement of the reference's fused dequantize-and-dot (TEST INFRASTRUCTURE).
 *
 * Checker and timed CPU baseline only: the test-suite, the smoke check and the
 * benchmark's CPU leg load this library; the product never does.
 *
 * It restates, in plain C with OpenMP over output rows, what the reference's
 * recognizer emits for one matched dot (eterevsky/metaljax, src/metaljax/qmm.py:2469-2501):
 *     y[m, n] = sum_k x[m, k] * deq(w)[n, k]           (transpose=True)
 * with the packed layout of src/metaljax/qmm.py:206-232 (little-endian bit
 * stream, element i at bits [i*bits, (i+1)*bits) of the uint32 words of a row),
 * the affine dequant `scales*q + biases` as one FMA per element
 * (src/metaljax/qmm.py:71-75), and the MXFP4 dequant `E2M1[q] * 2^(byte-127)`
 * (src/metaljax/qmm.py:167-173, tests/test_qmm_mxfp4.py:77-90). A CPU backend
 * fuses the reconstruction into the dot's operand loop (src/metaljax/qmm.py:11-13);
 * this is that loop: a row block of the weight is dequantized to float32 once
 * and every activation row is dotted against it with float32 accumulation.
 *
 * Activations, tables and outputs cross as raw bf16 bit patterns (uint16) or
 * float32, selected by the *_dtype arguments (0 = bf16, 2 = f32).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

static inline float bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round-to-nearest-even, NaN kept quiet */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

static inline float load_elem(const void* p, int dtype, long i) {
  return dtype == 2 ? ((const float*)p)[i] : bf16_to_f32(((const uint16_t*)p)[i]);
}

/* Use `n` threads from now on (a launcher may have pinned OMP_NUM_THREADS to 1). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* One row of the weight, dequantized to float32. */
static void dequant_row(const uint32_t* wrow, const void* scales, const void* biases,
                        int table_dtype, long row, long K, int gs, int bits, int mxfp4,
                        const uint8_t* scale_bytes, float* out) {
  const int per = 32 / bits;
  const uint32_t mask = (bits == 32) ? 0xffffffffu : ((1u << bits) - 1u);
  const long groups = K / gs;
  for (long g = 0; g < groups; ++g) {
    float s, b = 0.0f;
    if (mxfp4) {
      s = ldexpf(1.0f, (int)scale_bytes[row * groups + g] - 127);
    } else {
      s = load_elem(scales, table_dtype, row * groups + g);
      b = load_elem(biases, table_dtype, row * groups + g);
    }
    for (long k = g * gs; k < (g + 1) * gs; ++k) {
      uint32_t q = (wrow[k / per] >> ((k % per) * bits)) & mask;
      out[k] = mxfp4 ? kE2M1[q] * s : fmaf(s, (float)q, b);
    }
  }
}

/* Dequantize a whole packed weight [N, K*bits/32] into float32 [N, K]. */
int oracle_dequantize(const uint32_t* w, const void* scales, const void* biases,
                      int table_dtype, float* out, long N, long K, int gs, int bits,
                      int mxfp4) {
  const long words = K * bits / 32;
#pragma omp parallel for schedule(static)
  for (long n = 0; n < N; ++n)
    dequant_row(w + n * words, scales, biases, table_dtype, n, K, gs, bits, mxfp4,
                (const uint8_t*)scales, out + n * K);
  return 0;
}

/* y[M, N] = x[M, K] . deq(w)[N, K]^T, float32 accumulation.
 * x_dtype / y_dtype / table_dtype: 0 = bf16 bits, 2 = float32. */
int oracle_qmm(const void* x, int x_dtype, const uint32_t* w, const void* scales,
               const void* biases, int table_dtype, void* y, int y_dtype, long M, long K,
               long N, int gs, int bits, int mxfp4) {
  if (K % gs || (K * bits) % 32) return 1;
  const long words = K * bits / 32;
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * (size_t)K);
  if (!xf) return 2;
#pragma omp parallel for schedule(static)
  for (long i = 0; i < M * K; ++i) xf[i] = load_elem(x, x_dtype, i);

  enum { RB = 8 };
#pragma omp parallel
  {
    float* wf = (float*)malloc(sizeof(float) * RB * (size_t)K);
#pragma omp for schedule(dynamic, 4)
    for (long n0 = 0; n0 < N; n0 += RB) {
      const long nr = (N - n0 < RB) ? (N - n0) : RB;
      for (long r = 0; r < nr; ++r)
        dequant_row(w + (n0 + r) * words, scales, biases, table_dtype, n0 + r, K, gs, bits,
                    mxfp4, (const uint8_t*)scales, wf + r * K);
      for (long r = nr; r < RB; ++r) memset(wf + r * K, 0, sizeof(float) * (size_t)K);
      for (long m = 0; m < M; ++m) {
        const float* xr = xf + m * K;
        float acc[RB] = {0};
        for (long k = 0; k < K; ++k) {
          const float xv = xr[k];
          for (int r = 0; r < RB; ++r) acc[r] += xv * wf[r * K + k];
        }
        for (long r = 0; r < nr; ++r) {
          if (y_dtype == 2) ((float*)y)[m * N + n0 + r] = acc[r];
          else ((uint16_t*)y)[m * N + n0 + r] = f32_to_bf16(acc[r]);
        }
      }
    }
    free(wf);
  }
  free(xf);
  return 0;
}

/* Grouped form: rows [off[g], off[g+1]) of x meet expert g of w[G, N, words]. */
int oracle_qmm_ragged(const void* x, int x_dtype, const uint32_t* w, const void* scales,
                      const void* biases, int table_dtype, void* y, int y_dtype,
                      const int32_t* group_sizes, long G, long M, long K, long N, int gs,
                      int bits, int mxfp4) {
  const long words = K * bits / 32, groups = K / gs;
  const size_t xe = x_dtype == 2 ? 4 : 2, ye = y_dtype == 2 ? 4 : 2;
  const size_t te = mxfp4 ? 1 : (table_dtype == 2 ? 4 : 2);
  long lo = 0;
  for (long g = 0; g < G; ++g) {
    long n = group_sizes[g];
    if (lo + n > M) return 3;
    if (n > 0) {
      int rc = oracle_qmm((const char*)x + (size_t)lo * K * xe, x_dtype, w + g * N * words,
                          (const char*)scales + (size_t)g * N * groups * te,
                          biases ? (const char*)biases + (size_t)g * N * groups * te : 0,
                          table_dtype, (char*)y + (size_t)lo * N * ye, y_dtype, n, K, N, gs,
                          bits, mxfp4);
      if (rc) return rc;
    }
    lo += n;
  }
  if (lo < M) memset((char*)y + (size_t)lo * N * ye, 0, (size_t)(M - lo) * N * ye);
  return 0;
}
