/*
 * oracle_cpu.c - C restatement of the qwen.fused_gemm decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * The same arithmetic as oracle/oracle.py, fast enough (OpenMP over column blocks) to check the
 * CUDA library at the full benchmark sizes and to serve as the timed CPU baseline.  The shipped
 * package never links or loads this file.  The reference project has no CPU code for this path;
 * every routine follows the CUDA source lines it cites (paths inside the reference project).
 * It is pinned by tests that compare it with oracle.py, which in turn is pinned against the
 * reference's test formulas and against fixtures produced by the reference's own kernels.
 *
 * Formats: BF16 / FP16 as uint16 bit patterns; FP8 E4M3FN as uint8; NVFP4 rows are N/2 nibble
 * bytes (even column in the low nibble) followed by N/16 E4M3FN block scales
 * (src/fused_gemm/skinny_gemm.cuh:200-204).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { MODE_BF16 = 0, MODE_FP8 = 1, MODE_NVFP4 = 2 };

static float g_e4m3[256];
static int g_init = 0;
/* 2 * |value| of the E2M1 magnitudes: nibble LUT 0xC8643210 (skinny_gemm.cuh:162) */
static const float k_mag2[8] = {0.f, 1.f, 2.f, 3.f, 4.f, 6.f, 8.f, 12.f};

static void init_tables(void) {
  if (g_init) return;
  for (int c = 0; c < 256; ++c) {
    const int e = (c >> 3) & 0xF, m = c & 7;
    float v;
    if (e == 0xF && m == 7) {
      v = NAN;
    } else if (e == 0) {
      v = ldexpf((float)m, -9);
    } else {
      v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    }
    g_e4m3[c] = (c & 0x80) ? -v : v;
  }
  g_init = 1;
}

static inline float bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* round to nearest even, NaN -> 0x7FFF like __float2bfloat16 (skinny_gemm.cuh:212) */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if (f != f) return 0x7FFF;
  return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

static inline float f16_to_f32(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000) << 16;
  const int e = (h >> 10) & 0x1F;
  const uint32_t m = h & 0x3FF;
  float v;
  if (e == 0) {
    v = ldexpf((float)m, -24);
  } else if (e == 31) {
    if (m) { /* cvt.f32.f16 returns the canonical NaN 0x7FFFFFFF whatever the payload */
      const uint32_t canon = 0x7FFFFFFFu;
      memcpy(&v, &canon, 4);
      return v;
    }
    v = INFINITY;
  } else {
    v = ldexpf(1.0f + (float)m / 1024.0f, e - 15);
  }
  uint32_t u;
  memcpy(&u, &v, 4);
  u |= s;
  memcpy(&v, &u, 4);
  return v;
}

/* E2M1ScaledToFloat (skinny_gemm.cuh:161-165): float(2 mag) * (scale / 2), sign XOR-ed in */
static inline float e2m1_scaled(uint32_t nib, float s_half) {
  float f = k_mag2[nib & 7] * s_half;
  uint32_t u;
  memcpy(&u, &f, 4);
  u ^= (nib & 8u) << 28;
  memcpy(&f, &u, 4);
  return f;
}

/* exact value of W[k, c0 .. c0+cnt) as the GEMV loop sees it (skinny_gemm.cuh:106-183) */
static void decode_row(int mode, const uint8_t* w, long long pitch, int n_total, int k, int c0, int cnt, float* out) {
  const uint8_t* row = w + (long long)k * pitch;
  if (mode == MODE_BF16) {
    const uint16_t* r = (const uint16_t*)row;
    for (int i = 0; i < cnt; ++i) out[i] = bf16_to_f32(r[c0 + i]);
  } else if (mode == MODE_FP8) {
    for (int i = 0; i < cnt; ++i) out[i] = g_e4m3[row[c0 + i]];
  } else {
    for (int i = 0; i < cnt; ++i) {
      const int c = c0 + i;
      const uint32_t byte = row[c >> 1];
      const uint32_t nib = (c & 1) ? (byte >> 4) : (byte & 0xF);
      const float s_half = g_e4m3[row[(n_total >> 1) + (c >> 4)]] * 0.5f;
      out[i] = e2m1_scaled(nib, s_half);
    }
  }
}

static long long pitch_of(int mode, int n_total) {
  return mode == MODE_BF16 ? 2LL * n_total : mode == MODE_FP8 ? (long long)n_total : (long long)n_total * 9 / 16;
}

void oracle_set_num_threads(int n) { omp_set_num_threads(n > 0 ? n : 1); }

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* DequantWeightBf16 (fused_gemm.cu:203-250): columns [col_offset, col_offset + n_cols) of a stored
 * weight with `row_stride` logical columns, times w_scale[output column] (or 1), rounded to BF16. */
void oracle_dequant_bf16(int mode, const uint8_t* w, int K, int row_stride, int col_offset, int n_cols,
                         const float* w_scale, uint16_t* out) {
  init_tables();
  const long long pitch = pitch_of(mode, row_stride);
#pragma omp parallel
  {
    float* buf = (float*)malloc(sizeof(float) * (size_t)n_cols);
#pragma omp for schedule(static)
    for (int k = 0; k < K; ++k) {
      decode_row(mode, w, pitch, row_stride, k, col_offset, n_cols, buf);
      uint16_t* o = out + (long long)k * n_cols;
      if (mode == MODE_BF16) {
        const uint16_t* r = (const uint16_t*)(w + (long long)k * pitch);
        for (int i = 0; i < n_cols; ++i) o[i] = r[col_offset + i];
      } else {
        for (int i = 0; i < n_cols; ++i) o[i] = f32_to_bf16(buf[i] * (w_scale ? w_scale[i] : 1.0f));
      }
    }
    free(buf);
  }
}

/* SkinnyGemm with float64 accumulation over the exact weights (skinny_gemm.cuh:332-536);
 * w_scale multiplies the sum before the single BF16 rounding (:228).  `sums` / `mags`
 * (may be NULL) receive the float64 sum and sum of |x * w|, both after w_scale. */
void oracle_skinny_gemm(int mode, const uint16_t* x, int M, int K, const uint8_t* w, int N, const float* w_scale,
                        uint16_t* out, double* sums, double* mags) {
  init_tables();
  const long long pitch = pitch_of(mode, N);
  const int BLK = 256;
  const int nblk = (N + BLK - 1) / BLK;
#pragma omp parallel
  {
    float* wf = (float*)malloc(sizeof(float) * BLK);
    double* acc = (double*)malloc(sizeof(double) * (size_t)M * BLK);
    double* mag = (double*)malloc(sizeof(double) * (size_t)M * BLK);
#pragma omp for schedule(dynamic, 1)
    for (int b = 0; b < nblk; ++b) {
      const int c0 = b * BLK;
      const int cnt = (N - c0) < BLK ? (N - c0) : BLK;
      for (int i = 0; i < M * BLK; ++i) acc[i] = mag[i] = 0.0;
      for (int k = 0; k < K; ++k) {
        decode_row(mode, w, pitch, N, k, c0, cnt, wf);
        for (int m = 0; m < M; ++m) {
          const double xv = (double)bf16_to_f32(x[(long long)m * K + k]);
          const double xa = fabs(xv);
          double* a = acc + m * BLK;
          double* g = mag + m * BLK;
          for (int i = 0; i < cnt; ++i) {
            const double wv = (double)wf[i];
            a[i] += xv * wv;
            g[i] += xa * fabs(wv);
          }
        }
      }
      for (int m = 0; m < M; ++m) {
        for (int i = 0; i < cnt; ++i) {
          double s = acc[m * BLK + i], g = mag[m * BLK + i];
          float y = (float)s;
          if (w_scale) {
            y = y * w_scale[c0 + i];
            s *= (double)w_scale[c0 + i];
            g *= fabs((double)w_scale[c0 + i]);
          }
          out[(long long)m * N + c0 + i] = f32_to_bf16(y);
          if (sums) sums[(long long)m * N + c0 + i] = s;
          if (mags) mags[(long long)m * N + c0 + i] = g;
        }
      }
    }
    free(wf);
    free(acc);
    free(mag);
  }
}

/* The unfused chain the op replaces, as a CPU execution provider would run it:
 * DequantWeightBf16 (each weight rounded to BF16 after its w_scale) -> MatMul with FP32
 * accumulation in k order -> BF16.  This is the timed CPU baseline. */
void oracle_chain_f32(int mode, const uint16_t* x, int M, int K, const uint8_t* w, int N, const float* w_scale,
                      uint16_t* out) {
  init_tables();
  const long long pitch = pitch_of(mode, N);
  const int BLK = 512;
  const int nblk = (N + BLK - 1) / BLK;
  float* xf = (float*)malloc(sizeof(float) * (size_t)M * K);
  for (long long i = 0; i < (long long)M * K; ++i) xf[i] = bf16_to_f32(x[i]);
#pragma omp parallel
  {
    float* wf = (float*)malloc(sizeof(float) * BLK);
    float* acc = (float*)malloc(sizeof(float) * (size_t)M * BLK);
#pragma omp for schedule(dynamic, 1)
    for (int b = 0; b < nblk; ++b) {
      const int c0 = b * BLK;
      const int cnt = (N - c0) < BLK ? (N - c0) : BLK;
      for (int i = 0; i < M * BLK; ++i) acc[i] = 0.f;
      for (int k = 0; k < K; ++k) {
        decode_row(mode, w, pitch, N, k, c0, cnt, wf);
        if (mode != MODE_BF16) {
          for (int i = 0; i < cnt; ++i) wf[i] = bf16_to_f32(f32_to_bf16(wf[i] * (w_scale ? w_scale[c0 + i] : 1.0f)));
        }
        for (int m = 0; m < M; ++m) {
          const float xv = xf[(long long)m * K + k];
          float* a = acc + m * BLK;
          for (int i = 0; i < cnt; ++i) a[i] += xv * wf[i];
        }
      }
      for (int m = 0; m < M; ++m)
        for (int i = 0; i < cnt; ++i) out[(long long)m * N + c0 + i] = f32_to_bf16(acc[m * BLK + i]);
    }
    free(wf);
    free(acc);
  }
  free(xf);
}

/* `Better` (argmax_rows.cuh:27-32) */
static inline int better(float av, long long ai, float bv, long long bi) {
  if (av != av) return (bv == bv) || ai < bi;
  if (bv != bv) return 0;
  return av > bv || (av == bv && ai < bi);
}

/* ArgmaxRows (argmax_rows.cuh:55-163): dtype 0 = BF16, 1 = FP16, 2 = FP32 */
void oracle_argmax_rows(int dtype, const void* x, long long rows, long long V, int64_t* idx, float* val) {
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    float bv = 0.f;
    long long bi = -1;
    for (long long i = 0; i < V; ++i) {
      float v;
      if (dtype == 0) {
        v = bf16_to_f32(((const uint16_t*)x)[r * V + i]);
      } else if (dtype == 1) {
        v = f16_to_f32(((const uint16_t*)x)[r * V + i]);
      } else {
        v = ((const float*)x)[r * V + i];
      }
      if (bi < 0 || better(v, i, bv, bi)) {
        bv = v;
        bi = i;
      }
    }
    idx[r] = bi;
    if (val) val[r] = bv;
  }
}
