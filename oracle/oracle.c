/*
 * CPU oracle for the Winograd F(2x2,3x3) convolution path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library calls, links or loads this file; it exists so that the
 * tests, the smoke check and the CPU-baseline leg of the benchmark have an independent
 * statement of what the operator must compute.
 *
 * It restates, in plain C, the arithmetic of the openCNN operator
 *   filter transform      src/FX_m2.cu:23-47,73-86
 *   input transform       src/convolutionForward_32x64x8.cu:53-82
 *   accumulation order    src/convolutionForward_32x64x8.cu:210-257, src/outer_product.cuh
 *   output transform      src/store_and_transform_output_optSTS64.cuh:29-50
 *   layouts               src/openCNN_winograd.cu:147-153 (CHWN / CRSK), :185 (KHWN)
 *   tiling and halo       src/openCNN_winograd.cu:286-288, src/convolutionForward_32x64x8.cu:179-183
 * operation for operation, so that oc_winograd_f32() is a bit-level model of the reference
 * kernels (every rounding happens in the same place), and it adds the ground truth the
 * reference lacks: an fp64 direct cross-correlation (full and sampled) and a multithreaded
 * fp32 direct convolution that serves as the timed host baseline.
 *
 * Parity pin: the reference holds no golden vectors; this file is pinned by fixtures produced
 * by the reference's own kernels (compiled for sm_100a from their original location by
 * oracle/Makefile) and committed under tests/golden/.
 *
 * Build: see oracle/Makefile (gcc -O3 -mavx2 -mfma -ffp-contract=off -fopenmp).
 * -ffp-contract=off matters: every fused multiply-add below is an explicit fmaf().
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * Seeded synthetic tensors.  Values are a pure function of (seed, tensor id, logical
 * coordinate), so any batch slice can be generated independently and host and device
 * generators agree.  The logical coordinate of an input element is its NCHW linear index
 * with the GLOBAL image number, of a filter element its KCRS linear index.
 * ---------------------------------------------------------------------------------------- */
static inline uint64_t oc_mix(uint64_t z) {            /* splitmix64 finaliser */
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
static inline uint64_t oc_hash(uint64_t seed, uint64_t tensor, uint64_t idx) {
  return oc_mix(oc_mix(seed * 0xD1342543DE82EF95ull + tensor) ^ idx);
}
/* U(-1,1): the top 24 bits give k in [0,2^24); value (2k+1)/2^24 - 1 is exact in fp32. */
static inline float oc_uniform_pm1(uint64_t h) {
  uint32_t k = (uint32_t)(h >> 40);
  return (float)((int32_t)(2 * k + 1) - (1 << 24)) * (1.0f / 16777216.0f);
}
/* N(0,1) by Box-Muller in double from the two 32-bit halves of the hash. */
static inline double oc_normal(uint64_t h) {
  double u1 = ((double)(uint32_t)(h >> 32) + 0.5) * (1.0 / 4294967296.0);
  double u2 = ((double)(uint32_t)h + 0.5) * (1.0 / 4294967296.0);
  return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
}

/* Input in CHWN, x[((c*H+h)*W+w)*N + n], images n_offset .. n_offset+N-1 of the whole batch. */
OC_API void oc_fill_input_chwn(float *x, int N, int C, int H, int W, long n_offset, uint64_t seed) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int c = 0; c < C; ++c)
    for (int h = 0; h < H; ++h)
      for (int w = 0; w < W; ++w) {
        float *row = x + (((size_t)c * H + h) * W + w) * N;
        for (int n = 0; n < N; ++n) {
          uint64_t idx = ((((uint64_t)(n_offset + n)) * C + c) * H + h) * W + w;
          row[n] = oc_uniform_pm1(oc_hash(seed, 0, idx));
        }
      }
}
/* Filter in CRSK, g[((c*3+r)*3+s)*K + k] ~ N(0, sigma^2). */
OC_API void oc_fill_filter_crsk(float *g, int C, int K, double sigma, uint64_t seed) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c)
    for (int rs = 0; rs < 9; ++rs)
      for (int k = 0; k < K; ++k) {
        uint64_t idx = (((uint64_t)k * C + c) * 9) + rs;
        g[((size_t)c * 9 + rs) * K + k] = (float)(sigma * oc_normal(oc_hash(seed, 1, idx)));
      }
}
/* Small-integer tensors: fp32 Winograd is exact on them, so every implementation must agree
 * with the direct result bit for bit.  Inputs in {-4..4}; filters are multiples of 4 in
 * {-8,-4,0,4,8} so that the two halvings of the filter transform stay integral. */
OC_API void oc_fill_input_int(float *x, int N, int C, int H, int W, uint64_t seed) {
  size_t total = (size_t)N * C * H * W;
  for (size_t i = 0; i < total; ++i) x[i] = (float)((int)(oc_hash(seed, 2, i) % 9) - 4);
}
OC_API void oc_fill_filter_int(float *g, int C, int K, uint64_t seed) {
  size_t total = (size_t)C * 9 * K;
  for (size_t i = 0; i < total; ++i) g[i] = (float)(4 * ((int)(oc_hash(seed, 3, i) % 5) - 2));
}

/* ------------------------------------------------------------------------------------------
 * Ground truth: fp64 direct cross-correlation, 3x3, stride 1, pad 1 (no filter flip, as
 * CUDNN_CROSS_CORRELATION in src/openCNN_winograd.cu:369-372).  y in KHWN.
 * ---------------------------------------------------------------------------------------- */
OC_API void oc_direct_f64(const float *x, const float *g, double *y, int N, int C, int K, int H, int W) {
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
  for (int k = 0; k < K; ++k)
    for (int h = 0; h < H; ++h) {
      for (int w = 0; w < W; ++w) {
        double *out = y + (((size_t)k * H + h) * W + w) * N;
        for (int n = 0; n < N; ++n) out[n] = 0.0;
        for (int c = 0; c < C; ++c)
          for (int r = 0; r < 3; ++r) {
            int ih = h + r - 1;
            if (ih < 0 || ih >= H) continue;
            for (int s = 0; s < 3; ++s) {
              int iw = w + s - 1;
              if (iw < 0 || iw >= W) continue;
              double gv = (double)g[((size_t)(c * 3 + r) * 3 + s) * K + k];
              const float *in = x + (((size_t)c * H + ih) * W + iw) * N;
              for (int n = 0; n < N; ++n) out[n] += gv * (double)in[n];
            }
          }
      }
    }
}
/* Same, for a list of output positions given as KHWN linear indices. */
OC_API void oc_direct_f64_sampled(const float *x, const float *g, const int64_t *idx, int64_t count,
                                  double *out, int N, int C, int K, int H, int W) {
  (void)K;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    int64_t t = idx[i];
    int n = (int)(t % N); t /= N;
    int w = (int)(t % W); t /= W;
    int h = (int)(t % H); t /= H;
    int k = (int)t;
    double acc = 0.0;
    for (int c = 0; c < C; ++c)
      for (int r = 0; r < 3; ++r) {
        int ih = h + r - 1;
        if (ih < 0 || ih >= H) continue;
        for (int s = 0; s < 3; ++s) {
          int iw = w + s - 1;
          if (iw < 0 || iw >= W) continue;
          acc += (double)g[((size_t)(c * 3 + r) * 3 + s) * K + k] *
                 (double)x[(((size_t)c * H + ih) * W + iw) * N + n];
        }
      }
    out[i] = acc;
  }
}

/* ------------------------------------------------------------------------------------------
 * Timed host baseline: fp32 direct convolution on all cores, vectorised over the batch
 * (innermost) dimension.  The reference has no CPU implementation; this is the "port".
 * ---------------------------------------------------------------------------------------- */
OC_API void oc_direct_f32_omp(const float *restrict x, const float *restrict g, float *restrict y,
                              int N, int C, int K, int H, int W) {
#pragma omp parallel for collapse(2) schedule(dynamic, 2)
  for (int k = 0; k < K; ++k)
    for (int h = 0; h < H; ++h) {
      float *orow = y + (((size_t)k * H + h) * W) * N;
      memset(orow, 0, sizeof(float) * (size_t)W * N);
      for (int c = 0; c < C; ++c)
        for (int r = 0; r < 3; ++r) {
          int ih = h + r - 1;
          if (ih < 0 || ih >= H) continue;
          const float *irow = x + (((size_t)c * H + ih) * W) * N;
          for (int s = 0; s < 3; ++s) {
            float gv = g[((size_t)(c * 3 + r) * 3 + s) * K + k];
            int w0 = s == 0 ? 1 : 0, w1 = s == 2 ? W - 1 : W;
            /* output columns w0..w1-1 read input columns w+s-1: one contiguous run */
            float *o = orow + (size_t)w0 * N;
            const float *in = irow + (size_t)(w0 + s - 1) * N;
            size_t len = (size_t)(w1 - w0) * N;
#pragma omp simd
            for (size_t i = 0; i < len; ++i) o[i] += gv * in[i];
          }
        }
    }
}
OC_API int oc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------------------------------------------
 * Filter transform U = G g G^T, CRSK -> [C][4][4][K]   (src/FX_m2.cu:23-47, 73-86).
 * Rows first, then columns; each halved term is ((a + c) +/- b) summed in fp32 and then
 * multiplied by the double literal 0.5 before rounding back to fp32.
 * ---------------------------------------------------------------------------------------- */
static inline float oc_half_sum(float a, float c, float b) { return (float)(0.5 * (double)((a + c) + b)); }
static inline float oc_half_dif(float a, float c, float b) { return (float)(0.5 * (double)((a + c) - b)); }

OC_API void oc_filter_transform(const float *g, float *U, int C, int K) {
#pragma omp parallel for schedule(static)
  for (int c = 0; c < C; ++c)
    for (int k = 0; k < K; ++k) {
      float w[9], t[12];
      for (int i = 0; i < 9; ++i) w[i] = g[((size_t)c * 9 + i) * K + k];
      for (int j = 0; j < 3; ++j) {                      /* t = G w  (4x3) */
        t[0 + j] = w[j];
        t[3 + j] = oc_half_sum(w[j], w[6 + j], w[3 + j]);
        t[6 + j] = oc_half_dif(w[j], w[6 + j], w[3 + j]);
        t[9 + j] = w[6 + j];
      }
      for (int i = 0; i < 4; ++i) {                      /* U = t G^T (4x4) */
        const float *r = t + 3 * i;
        float *o = U + ((size_t)c * 16 + 4 * i) * K + k;
        o[0] = r[0];
        o[(size_t)K] = oc_half_sum(r[0], r[2], r[1]);
        o[2 * (size_t)K] = oc_half_dif(r[0], r[2], r[1]);
        o[3 * (size_t)K] = r[2];
      }
    }
}

/* ------------------------------------------------------------------------------------------
 * Bit-level model of the fused kernel.  x CHWN, U [C][16][K], y KHWN; square or rectangular
 * images (the reference supports H == W only; rectangles are handled the same way per axis).
 *   V = B^T d B   columns first, then rows   (src/convolutionForward_32x64x8.cu:59-80)
 *   M = sum_c V*U one FMA chain per output, c ascending from 0   (:190, :210-257)
 *   Y = A^T M A   rows first, then columns   (src/store_and_transform_output_optSTS64.cuh:29-50)
 * ---------------------------------------------------------------------------------------- */
OC_API void oc_winograd_f32(const float *restrict x, const float *restrict U, float *restrict y,
                            int N, int C, int K, int H, int W) {
  const int th = (H + 1) / 2, tw = (W + 1) / 2;
#pragma omp parallel
  {
    float *V = (float *)aligned_alloc(64, sizeof(float) * 16 * (size_t)N);
    float *M = (float *)aligned_alloc(64, sizeof(float) * 16 * (size_t)K * N);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int ty = 0; ty < th; ++ty)
      for (int tx = 0; tx < tw; ++tx) {
        memset(M, 0, sizeof(float) * 16 * (size_t)K * N);
        for (int c = 0; c < C; ++c) {
          /* input transform for all images of this (tile, channel) */
          for (int n = 0; n < N; ++n) {
            float d[16], b[16];
            for (int i = 0; i < 4; ++i)
              for (int j = 0; j < 4; ++j) {
                int ih = 2 * ty - 1 + i, iw = 2 * tx - 1 + j;
                d[4 * i + j] = (ih >= 0 && ih < H && iw >= 0 && iw < W)
                                   ? x[(((size_t)c * H + ih) * W + iw) * N + n] : 0.0f;
              }
            for (int j = 0; j < 4; ++j) {
              b[j] = d[j] - d[8 + j];
              b[4 + j] = d[4 + j] + d[8 + j];
              b[8 + j] = d[8 + j] - d[4 + j];
              b[12 + j] = d[4 + j] - d[12 + j];
            }
            for (int i = 0; i < 4; ++i) {
              V[(4 * i + 0) * (size_t)N + n] = b[4 * i + 0] - b[4 * i + 2];
              V[(4 * i + 1) * (size_t)N + n] = b[4 * i + 1] + b[4 * i + 2];
              V[(4 * i + 2) * (size_t)N + n] = b[4 * i + 2] - b[4 * i + 1];
              V[(4 * i + 3) * (size_t)N + n] = b[4 * i + 1] - b[4 * i + 3];
            }
          }
          for (int xi = 0; xi < 16; ++xi) {
            const float *u = U + ((size_t)c * 16 + xi) * K;
            const float *v = V + (size_t)xi * N;
            for (int k = 0; k < K; ++k) {
              float uk = u[k];
              float *m = M + ((size_t)xi * K + k) * N;
#pragma omp simd
              for (int n = 0; n < N; ++n) m[n] = fmaf(v[n], uk, m[n]);
            }
          }
        }
        for (int k = 0; k < K; ++k)
          for (int n = 0; n < N; ++n) {
            float m[16], a[8];
            for (int xi = 0; xi < 16; ++xi) m[xi] = M[((size_t)xi * K + k) * N + n];
            for (int j = 0; j < 4; ++j) {
              a[j] = m[j] + m[4 + j] + m[8 + j];
              a[4 + j] = m[4 + j] - m[8 + j] - m[12 + j];
            }
            for (int i = 0; i < 2; ++i) {
              int oh = 2 * ty + i;
              if (oh >= H) continue;
              float y0 = a[4 * i] + a[4 * i + 1] + a[4 * i + 2];
              float y1 = a[4 * i + 1] - a[4 * i + 2] - a[4 * i + 3];
              int ow = 2 * tx;
              y[(((size_t)k * H + oh) * W + ow) * N + n] = y0;
              if (ow + 1 < W) y[(((size_t)k * H + oh) * W + ow + 1) * N + n] = y1;
            }
          }
      }
    free(V);
    free(M);
  }
}

/* Whole operator as the reference runs it: filter transform into the workspace, then the
 * fused kernel (src/convolutionForward_32x64x8.cu:274-281). */
OC_API void oc_convolution_forward(const float *x, const float *g, float *y, float *workspace,
                                   int N, int C, int K, int H, int W) {
  oc_filter_transform(g, workspace, C, K);
  oc_winograd_f32(x, workspace, y, N, C, K, H, W);
}

/* ------------------------------------------------------------------------------------------
 * Reduced-precision operand rounding for the tensor-core path (round to nearest even).
 * ---------------------------------------------------------------------------------------- */
static inline float oc_round_bits(float v, int drop) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return v;
  uint32_t lsb = (u >> drop) & 1u;
  u += (1u << (drop - 1)) - 1u + lsb;
  u &= ~((1u << drop) - 1u);
  memcpy(&v, &u, 4);
  return v;
}
OC_API void oc_round_tf32(float *a, size_t count) { for (size_t i = 0; i < count; ++i) a[i] = oc_round_bits(a[i], 13); }
OC_API void oc_round_bf16(float *a, size_t count) { for (size_t i = 0; i < count; ++i) a[i] = oc_round_bits(a[i], 16); }

static inline float oc_round_bits(float v, int drop);

/* Model of the tensor-core path: filter and input transforms in fp32 exactly as above, each
 * transformed value rounded once to the operand type (mode 1 = TF32, 2 = BF16, 0 = none), the
 * contraction over channels exact (double), the output transform in fp32.  The device
 * accumulates in fp32 inside the tensor core, so agreement is to ~1e-5 relative, not bitwise.
 * This path has no counterpart in the reference; the model states what the kernel is meant to
 * compute so that layout or indexing mistakes cannot hide behind the quantisation error. */
OC_API void oc_winograd_tc_model(const float *restrict x, const float *restrict g, float *restrict y,
                                 int N, int C, int K, int H, int W, int mode) {
  const int th = (H + 1) / 2, tw = (W + 1) / 2;
  const int drop = mode == 1 ? 13 : 16;
  float *U = (float *)malloc(sizeof(float) * (size_t)C * 16 * K);
  oc_filter_transform(g, U, C, K);
  if (mode) for (size_t i = 0; i < (size_t)C * 16 * K; ++i) U[i] = oc_round_bits(U[i], drop);
#pragma omp parallel
  {
    float *V = (float *)aligned_alloc(64, sizeof(float) * 16 * (size_t)N);
    double *M = (double *)aligned_alloc(64, sizeof(double) * 16 * (size_t)K * N);
#pragma omp for collapse(2) schedule(dynamic, 1)
    for (int ty = 0; ty < th; ++ty)
      for (int tx = 0; tx < tw; ++tx) {
        memset(M, 0, sizeof(double) * 16 * (size_t)K * N);
        for (int c = 0; c < C; ++c) {
          for (int n = 0; n < N; ++n) {
            float d[16], b[16], v[16];
            for (int i = 0; i < 4; ++i)
              for (int j = 0; j < 4; ++j) {
                int ih = 2 * ty - 1 + i, iw = 2 * tx - 1 + j;
                d[4 * i + j] = (ih >= 0 && ih < H && iw >= 0 && iw < W)
                                   ? x[(((size_t)c * H + ih) * W + iw) * N + n] : 0.0f;
              }
            for (int j = 0; j < 4; ++j) {
              b[j] = d[j] - d[8 + j];
              b[4 + j] = d[4 + j] + d[8 + j];
              b[8 + j] = d[8 + j] - d[4 + j];
              b[12 + j] = d[4 + j] - d[12 + j];
            }
            for (int i = 0; i < 4; ++i) {
              v[4 * i + 0] = b[4 * i + 0] - b[4 * i + 2];
              v[4 * i + 1] = b[4 * i + 1] + b[4 * i + 2];
              v[4 * i + 2] = b[4 * i + 2] - b[4 * i + 1];
              v[4 * i + 3] = b[4 * i + 1] - b[4 * i + 3];
            }
            for (int xi = 0; xi < 16; ++xi) V[xi * (size_t)N + n] = mode ? oc_round_bits(v[xi], drop) : v[xi];
          }
          for (int xi = 0; xi < 16; ++xi) {
            const float *u = U + ((size_t)c * 16 + xi) * K;
            const float *v = V + (size_t)xi * N;
            for (int k = 0; k < K; ++k) {
              double uk = (double)u[k];
              double *m = M + ((size_t)xi * K + k) * N;
              for (int n = 0; n < N; ++n) m[n] += (double)v[n] * uk;
            }
          }
        }
        for (int k = 0; k < K; ++k)
          for (int n = 0; n < N; ++n) {
            float m[16], a[8];
            for (int xi = 0; xi < 16; ++xi) m[xi] = (float)M[((size_t)xi * K + k) * N + n];
            for (int j = 0; j < 4; ++j) {
              a[j] = m[j] + m[4 + j] + m[8 + j];
              a[4 + j] = m[4 + j] - m[8 + j] - m[12 + j];
            }
            for (int i = 0; i < 2; ++i) {
              int oh = 2 * ty + i;
              if (oh >= H) continue;
              float y0 = a[4 * i] + a[4 * i + 1] + a[4 * i + 2];
              float y1 = a[4 * i + 1] - a[4 * i + 2] - a[4 * i + 3];
              int ow = 2 * tx;
              y[(((size_t)k * H + oh) * W + ow) * N + n] = y0;
              if (ow + 1 < W) y[(((size_t)k * H + oh) * W + ow + 1) * N + n] = y1;
            }
          }
      }
    free(V);
    free(M);
  }
  free(U);
}

/* Error statistics of a fp32 result against a fp64 truth; returns the number of elements with
 * |a-r| > rel * max(|r|, floor_) and writes max abs error, max|r| and rms(r). */
OC_API int64_t oc_compare(const float *a, const double *r, size_t count, double rel, double floor_,
                          double *max_abs_err, double *max_ref, double *rms_ref) {
  double mx = 0, mr = 0, ss = 0;
  int64_t bad = 0;
  for (size_t i = 0; i < count; ++i) {
    double e = fabs((double)a[i] - r[i]), ar = fabs(r[i]);
    if (e > mx) mx = e;
    if (ar > mr) mr = ar;
    ss += r[i] * r[i];
    if (!(e <= rel * (ar > floor_ ? ar : floor_))) ++bad;
  }
  if (max_abs_err) *max_abs_err = mx;
  if (max_ref) *max_ref = mr;
  if (rms_ref) *rms_ref = count ? sqrt(ss / (double)count) : 0.0;
  return bad;
}
