/*
 * TEST INFRASTRUCTURE -- CPU oracle kernels.  Not part of the shipped library: only the
 * tests, the smoke check and the benchmark's CPU-baseline leg may build or call this file.
 *
 * Plain C restatement of the reference's arithmetic for the ODLA execute path.  Each
 * function names the reference source it follows (paths inside
 * alibaba/heterogeneity-aware-lowering-and-optimization).  Where the reference only calls
 * into oneDNN v1.7 (not vendored), the function restates oneDNN's documented behaviour
 * for that call site and says so: those restatements are "parity unpinned" by any
 * in-tree reference test.  The int8 convolution / GEMM with int32 accumulation has no
 * reference implementation at all; its definition is the one written here.
 *
 * Compile with -ffp-contract=off: every multiply and add must round separately so the
 * bit-exact int8 comparisons against the GPU epilogues hold.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORA_MAX_RANK 10

/* ---------------------------------------------------------------- convolution ---- */
/* Direct cross-correlation, summation order (filter row, filter col, input channel),
 * zero padding, as runtime/generic/nn/conv.cc:26-83.  `nhwc` selects NHWC data + HWIO
 * kernel (else NCHW + OIHW), the two pairs HALO emits.  Groups (absent from
 * runtime/generic, present at ODLA/platforms/dnnl/odla_dnnl.cc:1027-1041) split the
 * channels contiguously.  Rows [row_begin,row_end) of the flattened (batch*out_h) range
 * are computed, so callers can split the work over threads. */
void ora_conv2d_f32(float* out, const float* in, const float* ker, int64_t N, int64_t H,
                    int64_t W, int64_t C, int64_t P, int64_t Q, int64_t K, int64_t R, int64_t S,
                    int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t groups, int nhwc,
                    int64_t row_begin, int64_t row_end) {
  int64_t cg = C / groups, kg = K / groups;
  (void)N;
  for (int64_t row = row_begin; row < row_end; ++row) {
    int64_t b = row / P, i = row % P;
    for (int64_t c = 0; c < K; ++c) {
      int64_t g = c / kg;
      for (int64_t j = 0; j < Q; ++j) {
        float sum = 0;
        for (int64_t m = 0; m < R; ++m)
          for (int64_t n = 0; n < S; ++n)
            for (int64_t k = 0; k < cg; ++k) {
              int64_t h = i * sh - pt + m, w = j * sw - pl + n, ci = g * cg + k;
              int valid = h >= 0 && h < H && w >= 0 && w < W;
              float v = 0;
              if (valid) v = nhwc ? in[((b * H + h) * W + w) * C + ci] : in[((b * C + ci) * H + h) * W + w];
              float kv = nhwc ? ker[((m * S + n) * cg + k) * K + c] : ker[((c * cg + k) * R + m) * S + n];
              sum += v * kv;
            }
        if (nhwc) out[((b * P + i) * Q + j) * K + c] = sum;
        else out[((b * K + c) * P + i) * Q + j] = sum;
      }
    }
  }
}

/* int8 x int8 -> int32 convolution, NHWC data, HWIO kernel.  Exact integer arithmetic, so
 * summation order is irrelevant.  No reference implementation exists. */
void ora_conv2d_s8(int32_t* out, const int8_t* in, const int8_t* ker, int64_t N, int64_t H,
                   int64_t W, int64_t C, int64_t P, int64_t Q, int64_t K, int64_t R, int64_t S,
                   int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t row_begin,
                   int64_t row_end) {
  (void)N;
  int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)K);
  for (int64_t row = row_begin; row < row_end; ++row) {
    int64_t b = row / P, i = row % P;
    for (int64_t j = 0; j < Q; ++j) {
      memset(acc, 0, sizeof(int32_t) * (size_t)K);
      for (int64_t m = 0; m < R; ++m)
        for (int64_t n = 0; n < S; ++n) {
          int64_t h = i * sh - pt + m, w = j * sw - pl + n;
          if (h < 0 || h >= H || w < 0 || w >= W) continue;
          const int8_t* px = in + ((b * H + h) * W + w) * C;
          for (int64_t k = 0; k < C; ++k) {
            int32_t v = px[k];
            if (!v) continue;
            const int8_t* kr = ker + ((m * S + n) * C + k) * K;
            for (int64_t c = 0; c < K; ++c) acc[c] += v * (int32_t)kr[c];
          }
        }
      memcpy(out + ((b * P + i) * Q + j) * K, acc, sizeof(int32_t) * (size_t)K);
    }
  }
  free(acc);
}

/* The same sum with 16-bit filter values: a uint8 filter minus its zero point lies in [-255, 255].  The asymmetric
 * uint8 weights are what lib/quantizer/weights_quantizer.cc:84-182 produces for -quantize-weights=quint8
 * (q = clamp(round(w / scale + zp), 0, 255)); a product with such a filter is sum x_q * (W_u - zp), exactly, in int32. */
void ora_conv2d_s8_w16(int32_t* out, const int8_t* in, const int16_t* ker, int64_t N, int64_t H,
                       int64_t W, int64_t C, int64_t P, int64_t Q, int64_t K, int64_t R, int64_t S,
                       int64_t sh, int64_t sw, int64_t pt, int64_t pl, int64_t row_begin,
                       int64_t row_end) {
  (void)N;
  int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)K);
  for (int64_t row = row_begin; row < row_end; ++row) {
    int64_t b = row / P, i = row % P;
    for (int64_t j = 0; j < Q; ++j) {
      memset(acc, 0, sizeof(int32_t) * (size_t)K);
      for (int64_t m = 0; m < R; ++m)
        for (int64_t n = 0; n < S; ++n) {
          int64_t h = i * sh - pt + m, w = j * sw - pl + n;
          if (h < 0 || h >= H || w < 0 || w >= W) continue;
          const int8_t* px = in + ((b * H + h) * W + w) * C;
          for (int64_t k = 0; k < C; ++k) {
            int32_t v = px[k];
            if (!v) continue;
            const int16_t* kr = ker + ((m * S + n) * C + k) * K;
            for (int64_t c = 0; c < K; ++c) acc[c] += v * (int32_t)kr[c];
          }
        }
      memcpy(out + ((b * P + i) * Q + j) * K, acc, sizeof(int32_t) * (size_t)K);
    }
  }
  free(acc);
}
void ora_matmul_s8_w16(int32_t* out, const int8_t* A, const int16_t* B, int64_t M, int64_t N,
                       int64_t Kd, int ta, int tb) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      int32_t s = 0;
      for (int64_t k = 0; k < Kd; ++k) {
        int32_t a = ta ? A[k * M + i] : A[i * Kd + k];
        int32_t b = tb ? B[j * Kd + k] : B[k * N + j];
        s += a * b;
      }
      out[i * N + j] = s;
    }
}

/* -------------------------------------------------------------------- GEMM ---- */
/* out[M,N] = op(A) op(B), k ascending, as runtime/generic/math/matmul.cc:22-59. */
void ora_matmul_f32(float* out, const float* A, const float* B, int64_t M, int64_t N, int64_t Kd,
                    int ta, int tb) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float s = 0;
      for (int64_t k = 0; k < Kd; ++k) {
        float a = ta ? A[k * M + i] : A[i * Kd + k];
        float b = tb ? B[j * Kd + k] : B[k * N + j];
        s += a * b;
      }
      out[i * N + j] = s;
    }
}
/* out = alpha*out + beta*C with C holding M*N, 1, M (per row) or N (per column) elements:
 * runtime/generic/math/matmul.cc:61-110.  (odla_dnnl treats "1 or N elements" as a row
 * vector and everything else as a full matrix, ODLA/platforms/dnnl/odla_dnnl.cc:1812-1820;
 * the M-element case only exists in runtime/generic.) */
void ora_gemm_finish_f32(float* out, const float* C, int64_t M, int64_t N, int64_t c_noe,
                         float alpha, float beta) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      float r = out[i * N + j] * alpha;
      if (C) {
        float cv = c_noe == M * N ? C[i * N + j] : c_noe == 1 ? C[0] : c_noe == N ? C[j] : C[i];
        r += beta * cv;
      }
      out[i * N + j] = r;
    }
}
void ora_matmul_s8(int32_t* out, const int8_t* A, const int8_t* B, int64_t M, int64_t N,
                   int64_t Kd, int ta, int tb) {
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      int32_t s = 0;
      for (int64_t k = 0; k < Kd; ++k) {
        int32_t a = ta ? A[k * M + i] : A[i * Kd + k];
        int32_t b = tb ? B[j * Kd + k] : B[k * N + j];
        s += a * b;
      }
      out[i * N + j] = s;
    }
}

/* ------------------------------------------------------------------ pooling ---- */
/* Max pooling over NHWC (nhwc=1) or NCHW, padding acts as -infinity (lowest float):
 * runtime/generic/nn/pooling.cc:27-72. */
void ora_maxpool_f32(float* out, const float* in, int64_t N, int64_t H, int64_t W, int64_t C,
                     int64_t P, int64_t Q, int64_t R, int64_t S, int64_t sh, int64_t sw,
                     int64_t pt, int64_t pl, int nhwc) {
  for (int64_t b = 0; b < N; ++b)
    for (int64_t c = 0; c < C; ++c)
      for (int64_t i = 0; i < P; ++i)
        for (int64_t j = 0; j < Q; ++j) {
          float mx = -3.402823466e+38f;
          for (int64_t m = 0; m < R; ++m)
            for (int64_t n = 0; n < S; ++n) {
              int64_t h = i * sh - pt + m, w = j * sw - pl + n;
              if (h < 0 || h >= H || w < 0 || w >= W) continue;
              float v = nhwc ? in[((b * H + h) * W + w) * C + c] : in[((b * C + c) * H + h) * W + w];
              mx = mx > v ? mx : v;
            }
          if (nhwc) out[((b * P + i) * Q + j) * C + c] = mx;
          else out[((b * C + c) * P + i) * Q + j] = mx;
        }
}
void ora_maxpool_s8(int8_t* out, const int8_t* in, int64_t N, int64_t H, int64_t W, int64_t C,
                    int64_t P, int64_t Q, int64_t R, int64_t S, int64_t sh, int64_t sw,
                    int64_t pt, int64_t pl) {
  for (int64_t b = 0; b < N; ++b)
    for (int64_t i = 0; i < P; ++i)
      for (int64_t j = 0; j < Q; ++j)
        for (int64_t c = 0; c < C; ++c) {
          int mx = -128;
          for (int64_t m = 0; m < R; ++m)
            for (int64_t n = 0; n < S; ++n) {
              int64_t h = i * sh - pt + m, w = j * sw - pl + n;
              if (h < 0 || h >= H || w < 0 || w >= W) continue;
              int v = in[((b * H + h) * W + w) * C + c];
              mx = mx > v ? mx : v;
            }
          out[((b * P + i) * Q + j) * C + c] = (int8_t)mx;
        }
}
/* Average pooling.  odla_dnnl always asks oneDNN for dnnl::algorithm::pooling_avg and
 * drops `padding_included` (ODLA/platforms/dnnl/odla_dnnl.cc:1435-1446); in oneDNN v1.7
 * that algorithm divides by the number of in-bounds window elements.  Window elements are
 * added in (row, col) order.  Parity unpinned (oneDNN not available). */
void ora_avgpool_f32(float* out, const float* in, int64_t N, int64_t H, int64_t W, int64_t C,
                     int64_t P, int64_t Q, int64_t R, int64_t S, int64_t sh, int64_t sw,
                     int64_t pt, int64_t pl, int nhwc) {
  for (int64_t b = 0; b < N; ++b)
    for (int64_t c = 0; c < C; ++c)
      for (int64_t i = 0; i < P; ++i)
        for (int64_t j = 0; j < Q; ++j) {
          float s = 0;
          int cnt = 0;
          for (int64_t m = 0; m < R; ++m)
            for (int64_t n = 0; n < S; ++n) {
              int64_t h = i * sh - pt + m, w = j * sw - pl + n;
              if (h < 0 || h >= H || w < 0 || w >= W) continue;
              s += nhwc ? in[((b * H + h) * W + w) * C + c] : in[((b * C + c) * H + h) * W + w];
              ++cnt;
            }
          float r = s / (float)(cnt ? cnt : 1);
          if (nhwc) out[((b * P + i) * Q + j) * C + c] = r;
          else out[((b * C + c) * P + i) * Q + j] = r;
        }
}

/* ------------------------------------------------------- per-channel affine ---- */
/* Inference batch normalisation: scale*x/sqrt(var+eps) + (offset - scale*mean/sqrt(var+eps)),
 * the expression order of runtime/generic/nn/batchnorm.cc:35-49.  `inner` is the number of
 * contiguous elements per channel step (1 for NHWC, H*W for NCHW). */
void ora_batchnorm_f32(float* out, const float* in, const float* mean, const float* var,
                       const float* scale, const float* offset, float scalar_scale,
                       float scalar_offset, float eps, int64_t outer, int64_t C, int64_t inner) {
  for (int64_t c = 0; c < C; ++c) {
    float inv = 1.0f / sqrtf(var[c] + eps);
    float sc = scale ? scale[c] : scalar_scale;
    float of = offset ? offset[c] : scalar_offset;
    float cst = -sc * mean[c] * inv + of;
    for (int64_t o = 0; o < outer; ++o)
      for (int64_t i = 0; i < inner; ++i) {
        int64_t idx = (o * C + c) * inner + i;
        out[idx] = sc * in[idx] * inv + cst;
      }
  }
}

/* -------------------------------------------------------------- elementwise ---- */
/* Unary ops.  relu: runtime/generic/nn/relu.cc:22-26.  The rest exist in the reference only
 * as oneDNN eltwise calls: leaky relu / clamp ODLA/platforms/dnnl/odla_dnnl.cc:688-696,834-837
 * and odla_dnnl.h:396-411; gelu (erf form, or tanh form when use_approx)
 * odla_dnnl.cc:1868-1904; erf runtime/generic/math/erf.cc; round = nearest-even
 * (odla_dnnl.cc:635-637, oneDNN eltwise_round). */
enum {
  ORA_RELU = 0, ORA_LEAKY, ORA_CLAMP, ORA_GELU_ERF, ORA_GELU_TANH, ORA_ERF, ORA_SIGMOID, ORA_TANH,
  ORA_EXP, ORA_LOG, ORA_SQRT, ORA_RSQRT, ORA_ABS, ORA_NEG, ORA_RECIP, ORA_ROUND
};
float ora_unary_one(int op, float x, float a, float b) {
  switch (op) {
    case ORA_RELU: return x > 0 ? x : 0;
    case ORA_LEAKY: return x < 0 ? a * x : x;
    case ORA_CLAMP: return x < a ? a : (x > b ? b : x);
    case ORA_GELU_ERF: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case ORA_GELU_TANH: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(u));
    }
    case ORA_ERF: return erff(x);
    case ORA_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case ORA_TANH: return tanhf(x);
    case ORA_EXP: return expf(x);
    case ORA_LOG: return logf(x);
    case ORA_SQRT: return sqrtf(x);
    case ORA_RSQRT: return 1.0f / sqrtf(x);
    case ORA_ABS: return fabsf(x);
    case ORA_NEG: return -x;
    case ORA_RECIP: return 1.0f / x;
    case ORA_ROUND: return nearbyintf(x);
  }
  return x;
}
void ora_unary_f32(int op, float* out, const float* in, int64_t n, float a, float b) {
  for (int64_t i = 0; i < n; ++i) out[i] = ora_unary_one(op, in[i], a, b);
}

/* Binary ops with numpy-style broadcasting; shapes are already right-aligned to `rank` by
 * the caller (ODLA/platforms/dnnl/odla_dnnl.h:301-343), strides of broadcast dimensions are
 * zero as in runtime/generic/math/broadcast.h:25-43. */
enum { ORA_ADD = 0, ORA_SUB, ORA_MUL, ORA_DIV, ORA_POW, ORA_PRELU };
static float ora_binary_one(int op, float x, float y) {
  switch (op) {
    case ORA_ADD: return x + y;
    case ORA_SUB: return x - y;
    case ORA_MUL: return x * y;
    case ORA_DIV: return x / y;
    case ORA_POW: return powf(x, y);
    case ORA_PRELU: return x < 0 ? x * y : x;
  }
  return x;
}
void ora_binary_f32(int op, float* out, const float* lhs, const float* rhs, int rank,
                    const int64_t* oshape, const int64_t* lshape, const int64_t* rshape) {
  int64_t ls[ORA_MAX_RANK], rs[ORA_MAX_RANK], pos[ORA_MAX_RANK] = {0}, total = 1;
  int64_t la = 1, ra = 1;
  for (int i = rank - 1; i >= 0; --i) {
    ls[i] = lshape[i] == oshape[i] ? la : 0;
    rs[i] = rshape[i] == oshape[i] ? ra : 0;
    la *= lshape[i];
    ra *= rshape[i];
    total *= oshape[i];
  }
  for (int64_t e = 0; e < total; ++e) {
    int64_t li = 0, ri = 0;
    for (int i = 0; i < rank; ++i) { li += pos[i] * ls[i]; ri += pos[i] * rs[i]; }
    out[e] = ora_binary_one(op, lhs[li], rhs[ri]);
    for (int i = rank - 1; i >= 0; --i) {
      if (++pos[i] < oshape[i]) break;
      pos[i] = 0;
    }
  }
}

/* ------------------------------------------------------ softmax / reductions ---- */
/* Max-subtracted softmax along one axis: `outer` x `dim` x `inner`.  For the last axis this
 * is runtime/generic/nn/softmax.cc:26-49; for other axes it is the single-axis form
 * odla_dnnl requests (ODLA/platforms/dnnl/odla_dnnl.cc:1628-1648). */
void ora_softmax_f32(float* out, const float* in, int64_t outer, int64_t dim, int64_t inner,
                     int log_form) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float* x = in + o * dim * inner + i;
      float* y = out + o * dim * inner + i;
      float mx = x[0], sum = 0;
      for (int64_t d = 1; d < dim; ++d) mx = x[d * inner] > mx ? x[d * inner] : mx;
      for (int64_t d = 0; d < dim; ++d) {
        float e = expf(x[d * inner] - mx);
        y[d * inner] = e;
        sum += e;
      }
      for (int64_t d = 0; d < dim; ++d)
        y[d * inner] = log_form ? (x[d * inner] - mx) - logf(sum) : y[d * inner] / sum;
    }
}
/* Mean over ONE axis: sum in ascending index order, then one division by the extent.
 * Several axes are reduced one after the other in the order given, each pass dividing by
 * its own extent, exactly like runtime/generic/common/reduce.cc:24-59. */
void ora_reduce_mean_axis_f32(float* out, const float* in, int64_t before, int64_t dim,
                              int64_t after) {
  for (int64_t i = 0; i < before; ++i)
    for (int64_t k = 0; k < after; ++k) {
      float s = in[(i * dim) * after + k];
      for (int64_t j = 1; j < dim; ++j) s += in[(i * dim + j) * after + k];
      out[i * after + k] = s / (float)dim;
    }
}
/* Layer normalisation over the trailing `dim` elements of each of `rows` rows:
 * y = (x-mean)/sqrt(var+eps)*gamma+beta with the biased variance, the pattern HALO's
 * matcher collapses (lib/transforms/fusion.cc:71-314) and its emitter calls
 * (lib/target/generic_cpp/batchnorm.cc:100-113).  No platform in the reference runs it. */
void ora_layernorm_f32(float* out, const float* in, const float* gamma, const float* beta,
                       int64_t rows, int64_t dim, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * dim;
    float mean = 0, var = 0;
    for (int64_t d = 0; d < dim; ++d) mean += x[d];
    mean /= (float)dim;
    for (int64_t d = 0; d < dim; ++d) var += (x[d] - mean) * (x[d] - mean);
    var /= (float)dim;
    float inv = 1.0f / sqrtf(var + eps);
    for (int64_t d = 0; d < dim; ++d) {
      float v = (x[d] - mean) * inv;
      out[r * dim + d] = v * (gamma ? gamma[d] : 1.0f) + (beta ? beta[d] : 0.0f);
    }
  }
}

/* -------------------------------------------------------------- quantisation ---- */
static float ora_sat(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
/* q = saturate(round_to_nearest_even(x / scale) + zero_point): a true division, then oneDNN's
 * eltwise_round, then a saturating f32->s8/u8 reorder:
 * ODLA/platforms/dnnl/odla_dnnl_quantization.cc:61-90 (division at :77).  Scales are per
 * tensor (nscale==1) or per index of one axis (outer x nscale x inner). */
void ora_quantize_f32(void* out, const float* in, const float* scale, const int32_t* zp,
                      int64_t outer, int64_t nscale_dim, int64_t inner, int per_axis,
                      int is_unsigned) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t a = 0; a < nscale_dim; ++a)
      for (int64_t i = 0; i < inner; ++i) {
        int64_t idx = (o * nscale_dim + a) * inner + i;
        float s = scale[per_axis ? a : 0];
        float q = nearbyintf(in[idx] / s);
        if (zp) q = q + (float)zp[per_axis ? a : 0];
        if (is_unsigned) ((uint8_t*)out)[idx] = (uint8_t)ora_sat(q, 0.f, 255.f);
        else ((int8_t*)out)[idx] = (int8_t)ora_sat(q, -128.f, 127.f);
      }
}
/* Requantisation: q = saturate(round_to_nearest_even(x * inv_scale)) with inv_scale = fl(1/scale) computed by
 * the caller.  This build's definition for an odla_Quantize whose input was computed from int32
 * accumulators (the int8 workload is specified as "requantisation uses an fp32 multiplier with round-half-even"); every other
 * odla_Quantize divides, like the reference.  int8, per tensor, no zero point. */
void ora_requantize_f32(int8_t* out, const float* in, float inv_scale, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = (int8_t)ora_sat(nearbyintf(in[i] * inv_scale), -128.f, 127.f);
}
/* x = (float(q) - zero_point) * scale: odla_dnnl_quantization.cc:33-59. */
void ora_dequantize_f32(float* out, const void* in, const float* scale, const int32_t* zp,
                        int64_t outer, int64_t nscale_dim, int64_t inner, int per_axis,
                        int is_unsigned) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t a = 0; a < nscale_dim; ++a)
      for (int64_t i = 0; i < inner; ++i) {
        int64_t idx = (o * nscale_dim + a) * inner + i;
        float q = is_unsigned ? (float)((const uint8_t*)in)[idx] : (float)((const int8_t*)in)[idx];
        if (zp) q = q - (float)zp[per_axis ? a : 0];
        out[idx] = q * scale[per_axis ? a : 0];
      }
}

/* ------------------------------------------------------------- data movement ---- */
/* Generic permutation of a dense tensor (runtime/generic/math/transpose.cc). esz = bytes. */
void ora_transpose(void* out, const void* in, int rank, const int64_t* ishape, const int64_t* perm,
                   int esz) {
  int64_t istr[ORA_MAX_RANK], oshape[ORA_MAX_RANK], pos[ORA_MAX_RANK] = {0}, total = 1, a = 1;
  for (int i = rank - 1; i >= 0; --i) { istr[i] = a; a *= ishape[i]; }
  for (int i = 0; i < rank; ++i) { oshape[i] = ishape[perm[i]]; total *= oshape[i]; }
  for (int64_t e = 0; e < total; ++e) {
    int64_t src = 0;
    for (int i = 0; i < rank; ++i) src += pos[i] * istr[perm[i]];
    memcpy((char*)out + e * esz, (const char*)in + src * esz, (size_t)esz);
    for (int i = rank - 1; i >= 0; --i) {
      if (++pos[i] < oshape[i]) break;
      pos[i] = 0;
    }
  }
}
/* Copy one concat input: outer x (dim_i*inner) block placed at offset `off` of an output
 * whose axis extent is out_dim (ODLA/platforms/dnnl/odla_dnnl.cc:1331-1358). */
void ora_concat_part(void* out, const void* in, int64_t outer, int64_t in_dim, int64_t out_dim,
                     int64_t off, int64_t inner, int esz) {
  for (int64_t o = 0; o < outer; ++o)
    memcpy((char*)out + ((o * out_dim + off) * inner) * esz,
           (const char*)in + (o * in_dim * inner) * esz, (size_t)(in_dim * inner * esz));
}
/* Nearest-neighbour resize of the spatial dims.  odla_dnnl hands the tensor to oneDNN
 * resampling_nearest and ignores the coordinate mode (odla_dnnl.cc:1526-1551); oneDNN v1.7
 * picks source index round((o + 0.5) * in/out - 0.5).  Parity unpinned. */
static int64_t ora_nearest(int64_t o, int64_t in, int64_t out) {
  return (int64_t)roundf(((float)o + 0.5f) * (float)in / (float)out - 0.5f);
}
void ora_resize_nearest(void* out, const void* in, int64_t N, int64_t H, int64_t W, int64_t C,
                        int64_t P, int64_t Q, int nhwc, int esz) {
  for (int64_t b = 0; b < N; ++b)
    for (int64_t i = 0; i < P; ++i)
      for (int64_t j = 0; j < Q; ++j) {
        int64_t h = ora_nearest(i, H, P), w = ora_nearest(j, W, Q);
        h = h < 0 ? 0 : (h >= H ? H - 1 : h);
        w = w < 0 ? 0 : (w >= W ? W - 1 : w);
        for (int64_t c = 0; c < C; ++c) {
          int64_t src = nhwc ? ((b * H + h) * W + w) * C + c : ((b * C + c) * H + h) * W + w;
          int64_t dst = nhwc ? ((b * P + i) * Q + j) * C + c : ((b * C + c) * P + i) * Q + j;
          memcpy((char*)out + dst * esz, (const char*)in + src * esz, (size_t)esz);
        }
      }
}
/* Gather slices along `axis`: outer x n_idx x inner (runtime/generic/common/gather.cc). */
void ora_gather(void* out, const void* in, const int64_t* idx, int64_t outer, int64_t axis_dim,
                int64_t n_idx, int64_t inner, int esz) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t k = 0; k < n_idx; ++k) {
      int64_t id = idx[k] < 0 ? idx[k] + axis_dim : idx[k];
      memcpy((char*)out + ((o * n_idx + k) * inner) * esz,
             (const char*)in + ((o * axis_dim + id) * inner) * esz, (size_t)(inner * esz));
    }
}
/* Strided slice (runtime/generic/common/slice.cc; ODLA/platforms/dnnl/odla_dnnl.cc:455-508). */
void ora_slice(void* out, const void* in, int rank, const int64_t* ishape, const int64_t* oshape,
               const int64_t* start, const int64_t* step, int esz) {
  int64_t istr[ORA_MAX_RANK], pos[ORA_MAX_RANK] = {0}, total = 1, a = 1;
  for (int i = rank - 1; i >= 0; --i) { istr[i] = a; a *= ishape[i]; total *= oshape[i]; }
  for (int64_t e = 0; e < total; ++e) {
    int64_t src = 0;
    for (int i = 0; i < rank; ++i) src += (start[i] + pos[i] * step[i]) * istr[i];
    memcpy((char*)out + e * esz, (const char*)in + src * esz, (size_t)esz);
    for (int i = rank - 1; i >= 0; --i) {
      if (++pos[i] < oshape[i]) break;
      pos[i] = 0;
    }
  }
}

/* ---- detection post-processing ------------------------------------------------------------------------------ */
/* ONNX NonMaxSuppression, the rule odla_NMS stands for (lib/target/generic_cpp/nms.cc:22-69 emits the ONNX operator's
 * operands unchanged): per (batch, class) the candidates with score > score_threshold in descending score order (ties:
 * lower index first), each kept unless its IoU with an already kept box exceeds iou_threshold; boxes are (y1, x1, y2,
 * x2) with the corners in any order.  out: rows (batch, class, box), -1 in unused rows. */
static int ora_iou_over(const float* a, const float* b, float thr) {
  float ay1 = fminf(a[0], a[2]), ay2 = fmaxf(a[0], a[2]), ax1 = fminf(a[1], a[3]), ax2 = fmaxf(a[1], a[3]);
  float by1 = fminf(b[0], b[2]), by2 = fmaxf(b[0], b[2]), bx1 = fminf(b[1], b[3]), bx2 = fmaxf(b[1], b[3]);
  float ih = fminf(ay2, by2) - fmaxf(ay1, by1), iw = fminf(ax2, bx2) - fmaxf(ax1, bx1);
  if (ih <= 0.f || iw <= 0.f) return 0;
  float inter = ih * iw;
  float area_a = (ay2 - ay1) * (ax2 - ax1), area_b = (by2 - by1) * (bx2 - bx1);
  float uni = (area_a + area_b) - inter;
  if (uni <= 0.f) return 0;
  return inter / uni > thr;
}
/* order[]: indices sorted by (score descending, index ascending); insertion sort keeps this file free of callbacks */
static void ora_sort_desc(const float* score, int32_t* order, int64_t n) {
  for (int64_t i = 1; i < n; ++i) {
    int32_t v = order[i];
    int64_t j = i - 1;
    while (j >= 0 && (score[order[j]] < score[v] || (score[order[j]] == score[v] && order[j] > v))) { order[j + 1] = order[j]; --j; }
    order[j + 1] = v;
  }
}
void ora_nms(int64_t* out, int64_t out_rows, const float* boxes, const float* scores, int64_t B, int64_t C, int64_t N, int64_t max_per_class,
             float iou_thr, float score_thr, int32_t* order_scratch, int32_t* kept_scratch) {
  int64_t row = 0;
  for (int64_t i = 0; i < out_rows * 3; ++i) out[i] = -1;
  for (int64_t b = 0; b < B; ++b)
    for (int64_t c = 0; c < C; ++c) {
      const float* sc = scores + (b * C + c) * N;
      const float* bx = boxes + b * N * 4;
      int64_t n = 0, kept = 0;
      for (int64_t i = 0; i < N; ++i) if (sc[i] > score_thr) order_scratch[n++] = (int32_t)i;
      ora_sort_desc(sc, order_scratch, n);
      for (int64_t k = 0; k < n && kept < max_per_class; ++k) {
        int32_t i = order_scratch[k];
        int drop = 0;
        for (int64_t j = 0; j < kept && !drop; ++j) drop = ora_iou_over(bx + 4 * kept_scratch[j], bx + 4 * i, iou_thr);
        if (drop) continue;
        kept_scratch[kept++] = i;
        if (row < out_rows) { out[row * 3] = b; out[row * 3 + 1] = c; out[row * 3 + 2] = i; ++row; }
      }
    }
}
/* YOLOv3 post-processing as ODLA/platforms/odla_popart/custom_ops/postprocess.cc + codelets_nms.cpp define it: the heads
 * (NHWC after the transposition at postprocess.cc:150-152) are exponentiated (:154-156), decoded cell by cell against
 * the anchors of yolo_anchors.txt -- rows 2, 1, 0 for 13, 26, 52 cells (:170-228) -- by DecodeVertex
 * (codelets_nms.cpp:73-120), concatenated 13, 26, 52 (:232-234), and each class is walked in descending score order:
 * scores below 0.3 are skipped and a box is kept unless it overlaps the LAST kept one by more than 0.45
 * (codelets_nms.cpp:48-69).  info: [cls][N/169][5] = (y_min, x_min, y_max, x_max, score), zero beyond num[cls]. */
void ora_yolo_postprocess(float* info, uint32_t* num, const float* const* heads, const int* nchw3, const int* S3, int64_t cls, uint32_t img_w, uint32_t img_h,
                          float* boxes_scratch, float* scores_scratch, int32_t* order_scratch) {
  static const unsigned anchors[3][6] = {{10, 13, 16, 30, 33, 23}, {30, 61, 62, 45, 59, 119}, {116, 90, 156, 198, 373, 326}};
  int64_t N = 0, first[3];
  for (int i = 0; i < 3; ++i) { first[i] = N; N += (int64_t)S3[i] * S3[i] * 3; }
  const int64_t per_class = N / 169, ch = cls + 5;
  float scale = (float)fmin(416.0 / img_h, 416.0 / img_w);
  float new_h = roundf(img_h * scale), new_w = roundf(img_w * scale);
  float off_h = (float)((416 - new_h) / 2.0 / 416), off_w = (float)((416 - new_w) / 2.0 / 416);
  float sc_h = 416 / new_h, sc_w = 416 / new_w;
  for (int h = 0; h < 3; ++h) {
    const int S = S3[h];
    const unsigned* an = anchors[2 - h];
    for (int y = 0; y < S; ++y)
      for (int x = 0; x < S; ++x)
        for (int a = 0; a < 3; ++a) {
          float e[5];
          int64_t n = first[h] + ((int64_t)y * S + x) * 3 + a;
#define ORA_AT(k) expf(heads[h][nchw3[h] ? (((int64_t)(a * ch + (k))) * S + y) * S + x : ((int64_t)y * S + x) * (3 * ch) + a * ch + (k)])
          for (int k = 0; k < 5; ++k) e[k] = ORA_AT(k);
          float dx = ((e[0] / (e[0] + 1)) + x) / S;
          dx = (dx - off_w) * sc_w;
          float dy = ((e[1] / (e[1] + 1)) + y) / S;
          dy = (dy - off_h) * sc_h;
          float dw = (e[2] * an[a << 1]) / 416 * sc_w, dh = (e[3] * an[a << 1 | 1]) / 416 * sc_h;
          boxes_scratch[n * 4 + 0] = (float)((dy - dh / 2.0) * img_h);
          boxes_scratch[n * 4 + 1] = (float)((dx - dw / 2.0) * img_w);
          boxes_scratch[n * 4 + 2] = (float)((dy + dh / 2.0) * img_h);
          boxes_scratch[n * 4 + 3] = (float)((dx + dw / 2.0) * img_w);
          float conf = e[4] / (e[4] + 1);
          for (int64_t c = 0; c < cls; ++c) { float ec = ORA_AT(5 + c); scores_scratch[c * N + n] = ec / (ec + 1) * conf; }
#undef ORA_AT
        }
  }
  for (int64_t c = 0; c < cls; ++c) {
    const float* sc = scores_scratch + c * N;
    int64_t n = 0, kept = 0, last = -1;
    for (int64_t i = 0; i < N; ++i) if (!(sc[i] < 0.3f)) order_scratch[n++] = (int32_t)i;
    ora_sort_desc(sc, order_scratch, n);
    for (int64_t k = 0; k < per_class * 5; ++k) info[c * per_class * 5 + k] = 0.f;
    for (int64_t k = 0; k < n && kept < per_class; ++k) {
      int32_t i = order_scratch[k];
      if (last >= 0) {
        const float* s = boxes_scratch + 4 * last; const float* b = boxes_scratch + 4 * i;
        float y_top = fmaxf(s[0], b[0]), x_left = fmaxf(s[1], b[1]), y_bot = fminf(s[2], b[2]), x_right = fminf(s[3], b[3]);
        if (!(x_right < x_left || y_bot < y_top)) {
          float comm = (x_right - x_left) * (y_bot - y_top);
          float sa = (s[2] - s[0]) * (s[3] - s[1]), ca = (b[2] - b[0]) * (b[3] - b[1]);
          if (comm / ((sa + ca) - comm) > 0.45f) continue;
        }
      }
      last = i;
      float* o = info + (c * per_class + kept) * 5;
      for (int j = 0; j < 4; ++j) o[j] = boxes_scratch[4 * i + j];
      o[4] = sc[i];
      ++kept;
    }
    num[c] = (uint32_t)kept;
  }
}
