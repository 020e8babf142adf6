// CUDA-core kernels of libodla_b200: the memory-bound operators (pooling, soft-max, layer norm,
// element-wise, quantise / dequantise, layout moves) and a direct convolution / GEMM used where
// the tensor-core kernel does not apply (fp32 graphs, channel counts that break TMA alignment,
// grouped or NCHW convolutions).  Memory-bound kernels move 16 bytes per thread along the
// innermost (channel) dimension where the layout allows it and size their grids in multiples of
// the SM count.
#include <cstdio>

#include <algorithm>

#include "epilogue.cuh"

namespace b200 {
namespace {

int g_sm_count_cache[16] = {0};
int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 0 || dev >= 16) return 148;
  if (!g_sm_count_cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_sm_count_cache[dev] = n;
  }
  return g_sm_count_cache[dev];
}
// Grid for a grid-stride loop over `work` items with `threads` per block: enough blocks to cover
// the work, capped at 16 resident blocks per SM, rounded up to a multiple of the SM count.
int grid_for(int64_t work, int threads) {
  int sms = sm_count();
  int64_t need = (work + threads - 1) / threads;
  int64_t cap = (int64_t)sms * 16;
  if (need >= cap) return (int)cap;
  if (need <= sms) return (int)(need > 0 ? need : 1);
  return (int)(((need + sms - 1) / sms) * sms);
}
int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[odla_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return -2;
  }
  return 0;
}

// ------------------------------------------------------------ direct convolution ----
template <typename T, typename ACC>
__device__ __forceinline__ ACC mac(ACC acc, T a, T b);
template <> __device__ __forceinline__ float mac<float, float>(float acc, float a, float b) { return fmaf(a, b, acc); }
template <> __device__ __forceinline__ float mac<__half, float>(float acc, __half a, __half b) {
  return fmaf(__half2float(a), __half2float(b), acc);
}
template <> __device__ __forceinline__ float mac<__nv_bfloat16, float>(float acc, __nv_bfloat16 a, __nv_bfloat16 b) {
  return fmaf(__bfloat162float(a), __bfloat162float(b), acc);
}
template <> __device__ __forceinline__ int mac<int8_t, int>(int acc, int8_t a, int8_t b) { return acc + (int)a * (int)b; }

template <typename ACC>
__device__ __forceinline__ void store_result(const Epilogue& ep, void* y, int64_t yidx, ACC acc, int64_t row, int col,
                                             int64_t ld) {
  if (ep.out_dt == DT_S32) { ((int32_t*)y)[yidx] = (int32_t)acc; return; }
  float t = epilogue_value(ep, (float)acc, row, col, ld);
  store_from_float(y, ep.out_dt, yidx, t);
}

// One thread per output element, output channel fastest so filter reads coalesce for HWIO.
template <typename T, typename ACC>
__global__ void conv_direct_kernel(ConvGeom g, const T* __restrict__ x, const T* __restrict__ w, void* y, Epilogue ep) {
  int64_t total = (int64_t)g.N * g.P * g.Q * g.K;
  int cg = g.C / g.groups, kg = g.K / g.groups;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int k = (int)(e % g.K);
    int64_t pix = e / g.K;
    int q = (int)(pix % g.Q);
    int p = (int)((pix / g.Q) % g.P);
    int n = (int)(pix / ((int64_t)g.Q * g.P));
    int grp = k / kg;
    ACC acc = 0;
    for (int r = 0; r < g.R; ++r) {
      int h = p * g.stride_h - g.pad_t + r;
      if (h < 0 || h >= g.H) continue;
      for (int s = 0; s < g.S; ++s) {
        int ww = q * g.stride_w - g.pad_l + s;
        if (ww < 0 || ww >= g.W) continue;
        const T* xp = x + n * g.xs_n + h * g.xs_h + ww * g.xs_w + (int64_t)grp * cg * g.xs_c;
        const T* wp = w + k * g.ws_k + r * g.ws_r + s * g.ws_s;
        for (int c = 0; c < cg; ++c) acc = mac<T, ACC>(acc, xp[c * g.xs_c], wp[c * g.ws_c]);
      }
    }
    int64_t yidx = n * g.ys_n + p * g.ys_h + q * g.ys_w + k * g.ys_c;
    // Residual / full-matrix operands are addressed like a dense [pixels, K] matrix (NHWC).
    store_result<ACC>(ep, y, yidx, acc, pix, k, g.K);
  }
}

template <typename T, typename ACC>
__global__ void gemm_direct_kernel(GemmGeom g, const T* __restrict__ A, const T* __restrict__ B, void* C, Epilogue ep) {
  int64_t total = g.batch * g.M * g.N;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int n = (int)(e % g.N);
    int64_t m = (e / g.N) % g.M;
    int64_t b = e / (g.N * g.M);
    const T* a = A + b * g.a_batch + m * g.a_row;
    const T* bb = B + b * g.b_batch + n * g.b_col;
    ACC acc = 0;
    for (int64_t k = 0; k < g.K; ++k) acc = mac<T, ACC>(acc, a[k * g.a_col], bb[k * g.b_row]);
    store_result<ACC>(ep, C, e, acc, b * g.M + m, n, g.N);
  }
}

// ------------------------------------------------------------------ pooling ----
template <bool IS_MAX>
__global__ void pool_generic_kernel(PoolGeom g, int dt, const void* x, void* y) {
  int64_t total = (int64_t)g.N * g.P * g.Q * g.C;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int c = (int)(e % g.C);
    int64_t pix = e / g.C;
    int q = (int)(pix % g.Q), p = (int)((pix / g.Q) % g.P), n = (int)(pix / ((int64_t)g.Q * g.P));
    float acc = IS_MAX ? -3.402823466e+38f : 0.f;
    int cnt = 0;
    for (int r = 0; r < g.R; ++r) {
      int h = p * g.stride_h - g.pad_t + r;
      if (h < 0 || h >= g.H) continue;
      for (int s = 0; s < g.S; ++s) {
        int w = q * g.stride_w - g.pad_l + s;
        if (w < 0 || w >= g.W) continue;
        float v = load_as_float(x, dt, n * g.xs_n + h * g.xs_h + w * g.xs_w + c * g.xs_c);
        if (IS_MAX) acc = fmaxf(acc, v); else acc = __fadd_rn(acc, v);
        ++cnt;
      }
    }
    if (!IS_MAX) acc = __fdiv_rn(acc, (float)(cnt ? cnt : 1));
    store_from_float(y, dt, n * g.ys_n + p * g.ys_h + q * g.ys_w + c * g.ys_c, acc);
  }
}
// NHWC max pooling, 16 bytes per thread along C (8 halves or 16 int8 values).
template <typename VT, int VEC>
struct VecMax;
template <> struct VecMax<__half, 8> {
  static __device__ __forceinline__ void init(uint4& a) { a.x = a.y = a.z = a.w = 0xFBFFFBFFu; }
  static __device__ __forceinline__ void upd(uint4& a, const uint4& v) {
    __half2* pa = (__half2*)&a; const __half2* pv = (const __half2*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) pa[i] = __hmax2(pa[i], pv[i]);
  }
};
template <> struct VecMax<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void init(uint4& a) { a.x = a.y = a.z = a.w = 0xFF7FFF7Fu; }
  static __device__ __forceinline__ void upd(uint4& a, const uint4& v) {
    __nv_bfloat162* pa = (__nv_bfloat162*)&a; const __nv_bfloat162* pv = (const __nv_bfloat162*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) pa[i] = __hmax2(pa[i], pv[i]);
  }
};
template <> struct VecMax<int8_t, 16> {
  static __device__ __forceinline__ void init(uint4& a) { a.x = a.y = a.z = a.w = 0x80808080u; }
  static __device__ __forceinline__ void upd(uint4& a, const uint4& v) {
    a.x = __vmaxs4(a.x, v.x); a.y = __vmaxs4(a.y, v.y); a.z = __vmaxs4(a.z, v.z); a.w = __vmaxs4(a.w, v.w);
  }
};
template <> struct VecMax<float, 4> {
  static __device__ __forceinline__ void init(uint4& a) { float* f = (float*)&a; f[0] = f[1] = f[2] = f[3] = -3.402823466e+38f; }
  static __device__ __forceinline__ void upd(uint4& a, const uint4& v) {
    float* pa = (float*)&a; const float* pv = (const float*)&v;
#pragma unroll
    for (int i = 0; i < 4; ++i) pa[i] = fmaxf(pa[i], pv[i]);
  }
};
// One grid row per output row (n, p): a thread owns one 16-byte channel vector of one output pixel, so the index
// arithmetic is a single small division, consecutive threads read consecutive 16-byte pieces of the input rows, and
// the rows shared by neighbouring output rows are found in L2.
template <typename T, int VEC>
__global__ void maxpool_nhwc_vec_kernel(PoolGeom g, const T* __restrict__ x, T* __restrict__ y) {
  const int cv = g.C / VEC, row_items = g.Q * cv;
  const int rows = g.N * g.P;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const int n = row / g.P, p = row - n * g.P;
    const int h0 = p * g.stride_h - g.pad_t;
    const T* xin = x + (int64_t)n * g.H * g.W * g.C;
    T* yout = y + (int64_t)row * g.Q * g.C;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < row_items; e += gridDim.x * blockDim.x) {
      const int q = e / cv, c = (e - q * cv) * VEC;
      const int w0 = q * g.stride_w - g.pad_l;
      uint4 acc;
      VecMax<T, VEC>::init(acc);
      for (int r = 0; r < g.R; ++r) {
        const int h = h0 + r;
        if (h < 0 || h >= g.H) continue;
        const T* xr = xin + ((int64_t)h * g.W) * g.C + c;
#pragma unroll 3
        for (int s = 0; s < g.S; ++s) {
          const int w = w0 + s;
          if (w < 0 || w >= g.W) continue;
          VecMax<T, VEC>::upd(acc, *(const uint4*)(xr + (int64_t)w * g.C));
        }
      }
      *(uint4*)(yout + (int64_t)q * g.C + c) = acc;
    }
  }
}

// The same for a window known at compile time: all R*S loads of a thread are issued before the first maximum, from
// addresses clamped into the image, and a tap outside the image is replaced by the identity afterwards.  With the
// run-time window above every load waits for the one before it (the bounds tests sit between them), which makes a
// thread's life R*S trips to memory long.
template <typename T, int VEC, int R, int S>
__global__ void maxpool_nhwc_win_kernel(PoolGeom g, const T* __restrict__ x, T* __restrict__ y) {
  const int cv = g.C / VEC, row_items = g.Q * cv;
  const int rows = g.N * g.P;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const int n = row / g.P, p = row - n * g.P;
    const int h0 = p * g.stride_h - g.pad_t;
    const T* xin = x + (int64_t)n * g.H * g.W * g.C;
    T* yout = y + (int64_t)row * g.Q * g.C;
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < row_items; e += gridDim.x * blockDim.x) {
      const int q = e / cv, c = (e - q * cv) * VEC;
      const int w0 = q * g.stride_w - g.pad_l;
      uint4 v[R * S];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int h = min(max(h0 + r, 0), g.H - 1);
#pragma unroll
        for (int s2 = 0; s2 < S; ++s2) {
          const int w = min(max(w0 + s2, 0), g.W - 1);
          v[r * S + s2] = *(const uint4*)(xin + ((int64_t)h * g.W + w) * g.C + c);
        }
      }
      uint4 acc;
      VecMax<T, VEC>::init(acc);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const bool h_in = h0 + r >= 0 && h0 + r < g.H;
#pragma unroll
        for (int s2 = 0; s2 < S; ++s2)
          if (h_in && w0 + s2 >= 0 && w0 + s2 < g.W) VecMax<T, VEC>::upd(acc, v[r * S + s2]);
      }
      *(uint4*)(yout + (int64_t)q * g.C + c) = acc;
    }
  }
}

// -------------------------------------------------------------- element-wise ----
__device__ __forceinline__ float unary_one(int op, float x, float a, float b) {
  switch (op) {
    case UN_RELU: return x > 0.f ? x : 0.f;
    case UN_LEAKY: return x < 0.f ? __fmul_rn(a, x) : x;
    case UN_CLAMP: return x < a ? a : (x > b ? b : x);
    case UN_GELU_ERF: return apply_act(ACT_GELU_ERF, x, 0.f, 0.f);
    case UN_GELU_TANH: return apply_act(ACT_GELU_TANH, x, 0.f, 0.f);
    case UN_ERF: return erff(x);
    case UN_SIGMOID: return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
    case UN_TANH: return tanhf(x);
    case UN_EXP: return expf(x);
    case UN_LOG: return logf(x);
    case UN_SQRT: return __fsqrt_rn(x);
    case UN_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(x));
    case UN_ABS: return fabsf(x);
    case UN_NEG: return -x;
    case UN_RECIP: return __fdiv_rn(1.0f, x);
    case UN_ROUND: return rintf(x);
  }
  return x;
}
__global__ void unary_kernel(int op, int dt_in, int dt_out, const void* x, void* y, int64_t n, float a, float b) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    store_from_float(y, dt_out, i, unary_one(op, load_as_float(x, dt_in, i), a, b));
}
// 16-byte path for fp16 -> fp16.
__global__ void unary_h8_kernel(int op, const uint4* __restrict__ x, uint4* __restrict__ y, int64_t n8, float a, float b) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 v = x[i];
    __half* h = (__half*)&v;
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(unary_one(op, __half2float(h[j]), a, b));
    y[i] = v;
  }
}
__device__ __forceinline__ float binary_one(int op, float x, float y) {
  switch (op) {
    case BIN_ADD: return __fadd_rn(x, y);
    case BIN_SUB: return __fsub_rn(x, y);
    case BIN_MUL: return __fmul_rn(x, y);
    case BIN_DIV: return __fdiv_rn(x, y);
    case BIN_POW: return powf(x, y);
    case BIN_PRELU: return x < 0.f ? __fmul_rn(x, y) : x;
  }
  return x;
}
__global__ void binary_kernel(int op, BinaryGeom g, int dt_l, int dt_r, int dt_out, const void* l, const void* r, void* y,
                              int64_t total, int act, float act_a) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = e, li = 0, ri = 0;
    for (int d = g.rank - 1; d >= 0; --d) {
      int64_t p = rem % g.oshape[d];
      rem /= g.oshape[d];
      li += p * g.lstride[d];
      ri += p * g.rstride[d];
    }
    float v = binary_one(op, load_as_float(l, dt_l, li), load_as_float(r, dt_r, ri));
    store_from_float(y, dt_out, e, apply_act(act, v, act_a, 0.f));
  }
}
// Same-shape fp16 fast path, 16 bytes per thread.
__global__ void binary_same_h8_kernel(int op, const uint4* __restrict__ l, const uint4* __restrict__ r, uint4* __restrict__ y,
                                      int64_t n8, int act, float act_a) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 a = l[i], b = r[i];
    __half* ha = (__half*)&a;
    const __half* hb = (const __half*)&b;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      ha[j] = __float2half_rn(apply_act(act, binary_one(op, __half2float(ha[j]), __half2float(hb[j])), act_a, 0.f));
    y[i] = a;
  }
}
// Two-byte left operand and result, right operand repeating with a period (a trailing-dims broadcast such as a bias
// vector or a position table), stored in the same type or in fp32: eight elements per thread.  Same arithmetic as
// binary_kernel: one fp32 operation, one rounding to the type.
template <typename T, typename RT>
__global__ void binary_period_vec_kernel(int op, const uint4* __restrict__ l, const RT* __restrict__ r, uint4* __restrict__ y, int64_t n8, int64_t period8,
                                         int act, float act_a) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 a = l[i];
    const int64_t j = (i % period8) * 8;
    float b[8];
    if (sizeof(RT) == 4) {
      const float4 b0 = *(const float4*)((const float*)r + j), b1 = *(const float4*)((const float*)r + j + 4);
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
    } else {
      const uint4 bv = *(const uint4*)((const T*)r + j);
      const T* hb = (const T*)&bv;
#pragma unroll
      for (int k = 0; k < 8; ++k) b[k] = (float)hb[k];
    }
    T* ha = (T*)&a;
#pragma unroll
    for (int k = 0; k < 8; ++k) ha[k] = (T)apply_act(act, binary_one(op, (float)ha[k], b[k]), act_a, 0.f);
    y[i] = a;
  }
}
__global__ void channel_affine_kernel(int dt, const void* x, void* y, const float* a, const float* b, int64_t total, int64_t C,
                                      int64_t inner) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int c = (int)((e / inner) % C);
    store_from_float(y, dt, e, __fadd_rn(__fmul_rn(load_as_float(x, dt, e), a[c]), b[c]));
  }
}

// rintf(x / s) for a divisor that stays the same over a whole tensor, without a division per element: x * fl(1 / s) is
// within two units in the last place of the quotient, so its nearest integer is the quotient's unless the quotient lies
// that close to a half-integer -- only then is the division done.  Beyond +-256 both round far outside the int8 range and
// saturate alike.  `QuantDiv` holds s, fl(1 / s) and whether the shortcut is safe for this s (a normal reciprocal).
struct QuantDiv {
  float s, inv;
  bool fast;
  __device__ __forceinline__ explicit QuantDiv(float scale) {
    s = scale;
    inv = __fdiv_rn(1.0f, scale);
    fast = scale > 1e-30f && scale < 1e30f;
  }
  __device__ __forceinline__ float rint_div(float x) const {
    if (!fast) return rintf(__fdiv_rn(x, s));
    const float q = x * inv, t = rintf(q);
    if (fabsf(q) < 256.f && fabsf(fabsf(q - t) - 0.5f) < 1e-4f) return rintf(__fdiv_rn(x, s));
    return t;
  }
};

// ------------------------------------------------------ soft-max / reductions ----
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// One warp per row along a contiguous last axis.
__global__ void softmax_rows_kernel(int dt, const void* x, void* y, int64_t rows, int64_t dim, int log_form) {
  int lane = threadIdx.x & 31;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int64_t base = row * dim;
    float mx = -3.402823466e+38f;
    for (int64_t d = lane; d < dim; d += 32) mx = fmaxf(mx, load_as_float(x, dt, base + d));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int64_t d = lane; d < dim; d += 32) sum += expf(load_as_float(x, dt, base + d) - mx);
    sum = warp_sum(sum);
    float lsum = logf(sum);
    for (int64_t d = lane; d < dim; d += 32) {
      float v = load_as_float(x, dt, base + d) - mx;
      store_from_float(y, dt, base + d, log_form ? v - lsum : __fdiv_rn(expf(v), sum));
    }
  }
}
// Two-byte rows of at most 8*32*NP elements, one warp per row: every lane keeps its 16-byte pieces (8 elements each)
// in registers, so a row is read once and written once.  T is __half or __nv_bfloat16.
template <typename T> __device__ __forceinline__ float2 pair_to_float2(uint32_t u);
template <> __device__ __forceinline__ float2 pair_to_float2<__half>(uint32_t u) { return __half22float2(*(const __half2*)&u); }
template <> __device__ __forceinline__ float2 pair_to_float2<__nv_bfloat16>(uint32_t u) { return __bfloat1622float2(*(const __nv_bfloat162*)&u); }
template <typename T> __device__ __forceinline__ uint32_t float2_to_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t float2_to_pair<__half>(float a, float b) { __half2 h = __floats2half2_rn(a, b); return *(uint32_t*)&h; }
template <> __device__ __forceinline__ uint32_t float2_to_pair<__nv_bfloat16>(float a, float b) { __nv_bfloat162 h = __floats2bfloat162_rn(a, b); return *(uint32_t*)&h; }
// LPR lanes share a row (32, 16 or 8: short rows put several rows in one warp); lane l of the row holds pieces l, l + LPR, ...
template <int LPR> __device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int LPR> __device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <typename T, int NP, int LPR>
__device__ __forceinline__ void load_row_pieces(const uint4* row, int pieces, int l, bool row_ok, float (&v)[NP][8], bool (&have)[NP]) {
#pragma unroll
  for (int i = 0; i < NP; ++i) {
    const int pc = l + LPR * i;
    have[i] = row_ok && pc < pieces;
    if (have[i]) {
      const uint4 u = row[pc];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) { float2 f = pair_to_float2<T>(w[t]); v[i][2 * t] = f.x; v[i][2 * t + 1] = f.y; }
    }
  }
}
template <typename T, int NP, int LPR>
__global__ void softmax_rows_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t rows, int pieces, int log_form) {
  constexpr int RPW = 32 / LPR;  // rows per warp
  const int lane = threadIdx.x & 31, l = lane % LPR;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row0 = warp * RPW; row0 < rows; row0 += nwarps * RPW) {  // uniform across the warp: every lane reaches the shuffles
    const int64_t row = row0 + lane / LPR;
    const bool row_ok = row < rows;
    float v[NP][8];
    bool have[NP];
    load_row_pieces<T, NP, LPR>(x + row * pieces, pieces, l, row_ok, v, have);
    float mx = -3.402823466e+38f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) mx = fmaxf(mx, v[i][j]);
      }
    mx = group_max<LPR>(mx);
    float sum = 0.f;
    float e[NP][8];
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[i][j] -= mx; e[i][j] = __expf(v[i][j]); sum += e[i][j]; }
      }
    sum = group_sum<LPR>(sum);
    // The results are rounded to a two-byte type: the fast exponential (2 ulp of fp32) and one reciprocal per row instead
    // of a division per element stay far inside that rounding step.
    const float lsum = log_form ? logf(sum) : 0.f, inv = __fdiv_rn(1.0f, sum);
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          // e[][] holds exp(x - max) from the summation pass
          const float a = log_form ? v[i][2 * t] - lsum : e[i][2 * t] * inv;
          const float b = log_form ? v[i][2 * t + 1] - lsum : e[i][2 * t + 1] * inv;
          w[t] = float2_to_pair<T>(a, b);
        }
        y[row * pieces + l + LPR * i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
  }
}
template <typename T, int NP, int LPR, bool QUANT>
__global__ void layernorm_rows_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, const float* __restrict__ gamma, const float* __restrict__ beta,
                                          int64_t rows, int pieces, float eps, uint2* __restrict__ qout, const float* __restrict__ qscale) {
  const QuantDiv qd(QUANT ? qscale[0] : 1.f);
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, l = lane % LPR;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float dim = (float)(pieces * 8);
  for (int64_t row0 = warp * RPW; row0 < rows; row0 += nwarps * RPW) {
    const int64_t row = row0 + lane / LPR;
    const bool row_ok = row < rows;
    float v[NP][8];
    bool have[NP];
    load_row_pieces<T, NP, LPR>(x + row * pieces, pieces, l, row_ok, v, have);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    const float mean = group_sum<LPR>(s) / dim;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { v[i][j] -= mean; q = fmaf(v[i][j], v[i][j], q); }   // (spelled out: every instantiation rounds alike)
      }
    const float inv = 1.0f / sqrtf(group_sum<LPR>(q) / dim + eps);
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (have[i]) {
        const int d0 = (l + LPR * i) * 8;
        float gm[8], bt[8];
        if (gamma) { const float4 g0 = *(const float4*)(gamma + d0), g1 = *(const float4*)(gamma + d0 + 4); gm[0] = g0.x; gm[1] = g0.y; gm[2] = g0.z; gm[3] = g0.w; gm[4] = g1.x; gm[5] = g1.y; gm[6] = g1.z; gm[7] = g1.w; }
        if (beta) { const float4 b0 = *(const float4*)(beta + d0), b1 = *(const float4*)(beta + d0 + 4); bt[0] = b0.x; bt[1] = b0.y; bt[2] = b0.z; bt[3] = b0.w; bt[4] = b1.x; bt[5] = b1.y; bt[6] = b1.z; bt[7] = b1.w; }
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          float a = __fmul_rn(v[i][2 * t], inv), b = __fmul_rn(v[i][2 * t + 1], inv);
          if (gamma) { a = __fmul_rn(a, gm[2 * t]); b = __fmul_rn(b, gm[2 * t + 1]); }
          if (beta) { a = __fadd_rn(a, bt[2 * t]); b = __fadd_rn(b, bt[2 * t + 1]); }
          w[t] = float2_to_pair<T>(a, b);
        }
        y[row * pieces + l + LPR * i] = make_uint4(w[0], w[1], w[2], w[3]);
        if (QUANT) {   // the int8 copy quantises the values as stored (after their rounding to the two-byte type)
          uint32_t b[8];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float2 f = pair_to_float2<T>(w[t]);
            b[2 * t] = (uint32_t)(sat_s8(qd.rint_div(f.x)) & 0xff);
            b[2 * t + 1] = (uint32_t)(sat_s8(qd.rint_div(f.y)) & 0xff);
          }
          qout[row * pieces + l + LPR * i] = make_uint2(b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24), b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24));
        }
      }
  }
}
template <typename T>
bool launch_rows_vec(bool is_softmax, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim, float eps, int log_form,
                     cudaStream_t s, void* q = nullptr, const float* qscale = nullptr) {
  if ((uintptr_t)q % 8 != 0) return false;
  if (dim % 8 != 0 || dim > 8 * 32 * 8 || (uintptr_t)x % 16 != 0 || (uintptr_t)y % 16 != 0 || (uintptr_t)gamma % 16 != 0 || (uintptr_t)beta % 16 != 0) return false;
  const int pieces = (int)(dim / 8);
  const int lpr = pieces <= 8 ? 8 : (pieces <= 16 ? 16 : 32), np = (pieces + lpr - 1) / lpr;
  const int grid = grid_for(rows * lpr, 256);
#define B2_ROWS(NP, LPR)                                                                                                                      \
  do {                                                                                                                                        \
    if (is_softmax) softmax_rows_vec_kernel<T, NP, LPR><<<grid, 256, 0, s>>>((const uint4*)x, (uint4*)y, rows, pieces, log_form);             \
    else if (q) layernorm_rows_vec_kernel<T, NP, LPR, true><<<grid, 256, 0, s>>>((const uint4*)x, (uint4*)y, gamma, beta, rows, pieces, eps, (uint2*)q, qscale); \
    else layernorm_rows_vec_kernel<T, NP, LPR, false><<<grid, 256, 0, s>>>((const uint4*)x, (uint4*)y, gamma, beta, rows, pieces, eps, nullptr, nullptr); \
  } while (0)
  if (lpr == 8) B2_ROWS(1, 8);
  else if (lpr == 16) B2_ROWS(1, 16);
  else if (np <= 1) B2_ROWS(1, 32);
  else if (np <= 2) B2_ROWS(2, 32);
  else if (np <= 3) B2_ROWS(3, 32);
  else if (np <= 4) B2_ROWS(4, 32);
  else B2_ROWS(8, 32);
#undef B2_ROWS
  return true;
}
// Strided axis: one thread per (outer, inner) pair.
__global__ void softmax_strided_kernel(int dt, const void* x, void* y, int64_t outer, int64_t dim, int64_t inner, int log_form) {
  int64_t total = outer * inner;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t base = (e / inner) * dim * inner + e % inner;
    float mx = -3.402823466e+38f, sum = 0.f;
    for (int64_t d = 0; d < dim; ++d) mx = fmaxf(mx, load_as_float(x, dt, base + d * inner));
    for (int64_t d = 0; d < dim; ++d) sum += expf(load_as_float(x, dt, base + d * inner) - mx);
    float lsum = logf(sum);
    for (int64_t d = 0; d < dim; ++d) {
      float v = load_as_float(x, dt, base + d * inner) - mx;
      store_from_float(y, dt, base + d * inner, log_form ? v - lsum : __fdiv_rn(expf(v), sum));
    }
  }
}
__global__ void reduce_mean_axis_kernel(int dt_in, int dt_out, const void* x, void* y, int64_t before, int64_t dim, int64_t after) {
  int64_t total = before * after;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = e / after, k = e % after;
    float s = load_as_float(x, dt_in, (i * dim) * after + k);
    for (int64_t j = 1; j < dim; ++j) s = __fadd_rn(s, load_as_float(x, dt_in, (i * dim + j) * after + k));
    store_from_float(y, dt_out, e, __fdiv_rn(s, (float)dim));
  }
}
__global__ void layernorm_kernel(int dt, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim,
                                 float eps) {
  int lane = threadIdx.x & 31;
  int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    int64_t base = row * dim;
    float s = 0.f;
    for (int64_t d = lane; d < dim; d += 32) s += load_as_float(x, dt, base + d);
    float mean = warp_sum(s) / (float)dim;
    float v = 0.f;
    for (int64_t d = lane; d < dim; d += 32) { float t = load_as_float(x, dt, base + d) - mean; v += t * t; }
    float inv = 1.0f / sqrtf(warp_sum(v) / (float)dim + eps);
    for (int64_t d = lane; d < dim; d += 32) {
      float t = (load_as_float(x, dt, base + d) - mean) * inv;
      store_from_float(y, dt, base + d, t * (gamma ? gamma[d] : 1.f) + (beta ? beta[d] : 0.f));
    }
  }
}

// ------------------------------------------------------------- quantisation ----
__global__ void quantize_kernel(int dt_in, const void* x, void* q, const float* scale, const int* zp, int64_t total, int64_t adim,
                                int64_t inner, int per_axis, int is_unsigned) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int a = per_axis ? (int)((e / inner) % adim) : 0;
    float r = rintf(__fdiv_rn(load_as_float(x, dt_in, e), scale[a]));
    if (zp) r = __fadd_rn(r, (float)zp[a]);
    if (is_unsigned) ((uint8_t*)q)[e] = sat_u8(r); else ((int8_t*)q)[e] = sat_s8(r);
  }
}
// Per-tensor fp32 -> int8, 16 elements per thread (four 16-byte loads, one 16-byte store).
__global__ void quantize_f32_s8_vec_kernel(const float4* __restrict__ x, uint4* __restrict__ q, const float* scale, int64_t n16) {
  const QuantDiv qd(scale[0]);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 out;
    uint32_t* o = (uint32_t*)&out;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float4 v = x[i * 4 + j];
      int a = sat_s8(qd.rint_div(v.x)), b = sat_s8(qd.rint_div(v.y));
      int c = sat_s8(qd.rint_div(v.z)), d = sat_s8(qd.rint_div(v.w));
      o[j] = (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
    }
    q[i] = out;
  }
}
__global__ void requantize_kernel(int dt_in, const void* x, int8_t* q, float inv, int64_t n) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < n; e += (int64_t)gridDim.x * blockDim.x)
    q[e] = (int8_t)rne_sat_s8(__fmul_rn(load_as_float(x, dt_in, e), inv));
}
__global__ void dequantize_kernel(int dt_out, const void* q, void* x, const float* scale, const int* zp, int64_t total, int64_t adim,
                                  int64_t inner, int per_axis, int is_unsigned) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int a = per_axis ? (int)((e / inner) % adim) : 0;
    float v = is_unsigned ? (float)((const uint8_t*)q)[e] : (float)((const int8_t*)q)[e];
    if (zp) v = __fsub_rn(v, (float)zp[a]);
    store_from_float(x, dt_out, e, __fmul_rn(v, scale[a]));
  }
}
__global__ void convert_kernel(int dt_in, int dt_out, const void* x, void* y, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    if (dt_in == DT_S64 && dt_out == DT_S32) { ((int32_t*)y)[i] = (int32_t)((const long long*)x)[i]; continue; }
    if (dt_in == DT_S32 && dt_out == DT_S64) { ((long long*)y)[i] = ((const int32_t*)x)[i]; continue; }
    store_from_float(y, dt_out, i, load_as_float(x, dt_in, i));
  }
}
// fp32 -> fp16, 8 elements per thread.
__global__ void convert_f32_f16_vec_kernel(const float4* __restrict__ x, uint4* __restrict__ y, int64_t n8) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    float4 a = x[2 * i], b = x[2 * i + 1];
    uint4 o;
    __half2* h = (__half2*)&o;
    h[0] = __floats2half2_rn(a.x, a.y); h[1] = __floats2half2_rn(a.z, a.w);
    h[2] = __floats2half2_rn(b.x, b.y); h[3] = __floats2half2_rn(b.z, b.w);
    y[i] = o;
  }
}

// ------------------------------------------------------------- data movement ----
template <typename T>
__global__ void move_kernel(MoveGeom g, const T* __restrict__ x, T* __restrict__ y, int64_t total) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = e, si = g.in_offset, di = g.out_offset;
    for (int d = g.rank - 1; d >= 0; --d) {
      int64_t p = rem % g.oshape[d];
      rem /= g.oshape[d];
      si += p * g.istride[d];
      di += p * g.ostride[d];
    }
    y[di] = x[si];
  }
}
template <typename T>
__global__ void pad_channels_kernel(const T* __restrict__ x, uint4* __restrict__ y, int64_t pixels, int C) {
  constexpr int CP = 32 / (int)sizeof(T);
  for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < pixels; p += (int64_t)gridDim.x * blockDim.x) {
    uint4 out[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    T* o = (T*)out;
    const T* in = x + p * C;
#pragma unroll
    for (int c = 0; c < CP; ++c)
      if (c < C) o[c] = in[c];
    y[2 * p] = out[0];
    y[2 * p + 1] = out[1];
  }
}
template <typename T>
__global__ void stem_widen_kernel(const T* __restrict__ x, uint4* __restrict__ y, int N, int H, int W, int C, int Q) {
  constexpr int PER = 16 / (int)sizeof(T);       // elements per 16-byte piece
  constexpr int PIECES = 32 / PER;                // pieces per widened pixel (32 elements)
  const int64_t total = (int64_t)N * H * Q * PIECES;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int piece = (int)(e % PIECES);
    const int64_t wp = e / PIECES;               // (n*H + h)*Q + q
    const int q = (int)(wp % Q);
    const int64_t nh = wp / Q;
    uint4 out = make_uint4(0, 0, 0, 0);
    T* o = (T*)&out;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int el = piece * PER + i, pix = 2 * q - 4 + (el >> 2), c = el & 3;
      if (pix >= 0 && pix < W && c < C) o[i] = x[(nh * W + pix) * C + c];
    }
    y[e] = out;
  }
}
// Pads every pixel to CP channels (8 or 16 bytes) and every image row with `lp` zero pixels on the left and zeros up
// to Wp pixels on the right.
template <typename T, int CP>
__global__ void stem_pad_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int W, int C, int lp, int Wp) {
  static_assert(sizeof(T) * CP == 4 || sizeof(T) * CP == 8 || sizeof(T) * CP == 16, "a padded pixel is 4, 8 or 16 bytes");
  const int64_t total = rows * Wp;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int wp = (int)(e % Wp);
    const int64_t row = e / Wp;
    const int w = wp - lp;
    __align__(16) T px[CP];
#pragma unroll
    for (int c = 0; c < CP; ++c) px[c] = 0;
    if (w >= 0 && w < W) {
#pragma unroll
      for (int c = 0; c < CP; ++c) if (c < C) px[c] = x[(row * W + w) * C + c];
    }
    if (sizeof(T) * CP == 4) *(uint32_t*)(y + e * CP) = *(const uint32_t*)px;
    else if (sizeof(T) * CP == 8) *(uint2*)(y + e * CP) = *(const uint2*)px;
    else *(uint4*)(y + e * CP) = *(const uint4*)px;
  }
}
template <typename T>
__global__ void resize_nearest_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int H, int W, int C, int P, int Q, int nhwc) {
  int64_t total = (int64_t)N * P * Q * C;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int c, q, p, n;
    if (nhwc) { c = (int)(e % C); q = (int)((e / C) % Q); p = (int)((e / ((int64_t)C * Q)) % P); n = (int)(e / ((int64_t)C * Q * P)); }
    else { q = (int)(e % Q); p = (int)((e / Q) % P); c = (int)((e / ((int64_t)Q * P)) % C); n = (int)(e / ((int64_t)Q * P * C)); }
    int h = (int)roundf(((float)p + 0.5f) * (float)H / (float)P - 0.5f);
    int w = (int)roundf(((float)q + 0.5f) * (float)W / (float)Q - 0.5f);
    h = min(max(h, 0), H - 1);
    w = min(max(w, 0), W - 1);
    int64_t src = nhwc ? (((int64_t)n * H + h) * W + w) * C + c : (((int64_t)n * C + c) * H + h) * W + w;
    y[e] = x[src];
  }
}
template <typename T>
__global__ void gather_kernel(const T* __restrict__ x, const void* idx, int idx_dt, T* __restrict__ y, int64_t outer, int64_t axis_dim,
                              int64_t n_idx, int64_t inner) {
  int64_t total = outer * n_idx * inner;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = e % inner, k = (e / inner) % n_idx, o = e / (inner * n_idx);
    int64_t id = idx_dt == DT_S64 ? ((const long long*)idx)[k] : (int64_t)((const int32_t*)idx)[k];
    if (id < 0) id += axis_dim;
    id = id < 0 ? 0 : (id >= axis_dim ? axis_dim - 1 : id);
    y[e] = x[(o * axis_dim + id) * inner + i];
  }
}

}  // namespace

// ----------------------------------------------------------------- launchers ----
int conv_simt(const ConvGeom& g, int in_dt, const void* x, const void* w, void* y, const Epilogue& ep, cudaStream_t s) {
  int64_t total = (int64_t)g.N * g.P * g.Q * g.K;
  if (total <= 0) return 0;
  int grid = grid_for(total, 256);
  switch (in_dt) {
    case DT_F32: conv_direct_kernel<float, float><<<grid, 256, 0, s>>>(g, (const float*)x, (const float*)w, y, ep); break;
    case DT_F16: conv_direct_kernel<__half, float><<<grid, 256, 0, s>>>(g, (const __half*)x, (const __half*)w, y, ep); break;
    case DT_BF16: conv_direct_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, y, ep); break;
    case DT_S8: conv_direct_kernel<int8_t, int><<<grid, 256, 0, s>>>(g, (const int8_t*)x, (const int8_t*)w, y, ep); break;
    default: return -1;
  }
  return check_launch();
}
int gemm_simt(const GemmGeom& g, int in_dt, const void* A, const void* B, void* C, const Epilogue& ep, cudaStream_t s) {
  int64_t total = g.batch * g.M * g.N;
  if (total <= 0) return 0;
  int grid = grid_for(total, 256);
  switch (in_dt) {
    case DT_F32: gemm_direct_kernel<float, float><<<grid, 256, 0, s>>>(g, (const float*)A, (const float*)B, C, ep); break;
    case DT_F16: gemm_direct_kernel<__half, float><<<grid, 256, 0, s>>>(g, (const __half*)A, (const __half*)B, C, ep); break;
    case DT_BF16: gemm_direct_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(g, (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, C, ep); break;
    case DT_S8: gemm_direct_kernel<int8_t, int><<<grid, 256, 0, s>>>(g, (const int8_t*)A, (const int8_t*)B, C, ep); break;
    default: return -1;
  }
  return check_launch();
}
static dim3 pool_grid(const PoolGeom& g, int vec) {
  const int row_items = g.Q * (g.C / vec);
  const int gx = (row_items + 255) / 256;
  int64_t gy = (int64_t)g.N * g.P;
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)(gx > 0 ? gx : 1), (unsigned)gy);
}
int pool2d(const PoolGeom& g, int dt, bool is_max, const void* x, void* y, cudaStream_t s) {
  int64_t total = (int64_t)g.N * g.P * g.Q * g.C;
  if (total <= 0) return 0;
  bool nhwc_dense = g.xs_c == 1 && g.xs_w == g.C && g.xs_h == (int64_t)g.W * g.C && g.ys_c == 1 && g.ys_w == g.C &&
                    g.ys_h == (int64_t)g.Q * g.C && g.ys_n == (int64_t)g.P * g.Q * g.C && g.xs_n == (int64_t)g.H * g.W * g.C;
  bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0);
  if (is_max && nhwc_dense && aligned && g.H >= 1 && g.W >= 1 && ((g.R == 3 && g.S == 3) || (g.R == 2 && g.S == 2)) && !getenv("ODLA_B200_POOL_RUNTIME_WINDOW")) {
#define B2_POOL_WIN(T, V)                                                                                                          \
    do {                                                                                                                           \
      if (g.R == 3) maxpool_nhwc_win_kernel<T, V, 3, 3><<<pool_grid(g, V), 256, 0, s>>>(g, (const T*)x, (T*)y);                    \
      else maxpool_nhwc_win_kernel<T, V, 2, 2><<<pool_grid(g, V), 256, 0, s>>>(g, (const T*)x, (T*)y);                             \
      return check_launch();                                                                                                       \
    } while (0)
    if (dt == DT_F16 && g.C % 8 == 0) B2_POOL_WIN(__half, 8);
    if (dt == DT_BF16 && g.C % 8 == 0) B2_POOL_WIN(__nv_bfloat16, 8);
    if (dt == DT_S8 && g.C % 16 == 0) B2_POOL_WIN(int8_t, 16);
    if (dt == DT_F32 && g.C % 4 == 0) B2_POOL_WIN(float, 4);
#undef B2_POOL_WIN
  }
  if (is_max && nhwc_dense && aligned) {
    if (dt == DT_F16 && g.C % 8 == 0) { maxpool_nhwc_vec_kernel<__half, 8><<<pool_grid(g, 8), 256, 0, s>>>(g, (const __half*)x, (__half*)y); return check_launch(); }
    if (dt == DT_BF16 && g.C % 8 == 0) { maxpool_nhwc_vec_kernel<__nv_bfloat16, 8><<<pool_grid(g, 8), 256, 0, s>>>(g, (const __nv_bfloat16*)x, (__nv_bfloat16*)y); return check_launch(); }
    if (dt == DT_S8 && g.C % 16 == 0) { maxpool_nhwc_vec_kernel<int8_t, 16><<<pool_grid(g, 16), 256, 0, s>>>(g, (const int8_t*)x, (int8_t*)y); return check_launch(); }
    if (dt == DT_F32 && g.C % 4 == 0) { maxpool_nhwc_vec_kernel<float, 4><<<pool_grid(g, 4), 256, 0, s>>>(g, (const float*)x, (float*)y); return check_launch(); }
  }
  if (is_max) pool_generic_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(g, dt, x, y);
  else pool_generic_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(g, dt, x, y);
  return check_launch();
}
int unary(int op, int dt_in, int dt_out, const void* x, void* y, int64_t n, float a, float b, cudaStream_t s) {
  if (n <= 0) return 0;
  if (dt_in == DT_F16 && dt_out == DT_F16 && n % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
    unary_h8_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>(op, (const uint4*)x, (uint4*)y, n / 8, a, b);
    return check_launch();
  }
  unary_kernel<<<grid_for(n, 256), 256, 0, s>>>(op, dt_in, dt_out, x, y, n, a, b);
  return check_launch();
}
int binary(int op, const BinaryGeom& g, int dt_l, int dt_r, int dt_out, const void* l, const void* r, void* y, int act, float act_a,
           cudaStream_t s) {
  int64_t total = 1;
  bool same = true;
  int64_t acc = 1;
  for (int d = g.rank - 1; d >= 0; --d) {
    total *= g.oshape[d];
    if (g.oshape[d] != 1 && (g.lstride[d] != acc || g.rstride[d] != acc)) same = false;
    acc *= g.oshape[d];
  }
  if (total <= 0) return 0;
  if (same && dt_l == DT_F16 && dt_r == DT_F16 && dt_out == DT_F16 && total % 8 == 0 && (uintptr_t)l % 16 == 0 &&
      (uintptr_t)r % 16 == 0 && (uintptr_t)y % 16 == 0) {
    binary_same_h8_kernel<<<grid_for(total / 8, 256), 256, 0, s>>>(op, (const uint4*)l, (const uint4*)r, (uint4*)y, total / 8, act, act_a);
    return check_launch();
  }
  // left operand dense, right operand a broadcast over the leading dims (zero strides there, dense strides after)
  if ((dt_out == DT_F16 || dt_out == DT_BF16) && dt_l == dt_out && (dt_r == dt_out || dt_r == DT_F32) && total % 8 == 0 && (uintptr_t)l % 16 == 0 &&
      (uintptr_t)r % 16 == 0 && (uintptr_t)y % 16 == 0) {
    bool l_dense = true, r_suffix = true, in_suffix = true;
    int64_t dense = 1, period = 1;
    for (int d = g.rank - 1; d >= 0; --d) {
      if (g.oshape[d] == 1) continue;
      if (g.lstride[d] != dense) l_dense = false;
      if (in_suffix && g.rstride[d] == dense) period = dense * g.oshape[d];
      else { in_suffix = false; if (g.rstride[d] != 0) r_suffix = false; }
      dense *= g.oshape[d];
    }
    if (l_dense && r_suffix && period % 8 == 0 && period >= 8) {
      const int grid = grid_for(total / 8, 256);
      if (dt_out == DT_F16 && dt_r == DT_F16) binary_period_vec_kernel<__half, __half><<<grid, 256, 0, s>>>(op, (const uint4*)l, (const __half*)r, (uint4*)y, total / 8, period / 8, act, act_a);
      else if (dt_out == DT_F16) binary_period_vec_kernel<__half, float><<<grid, 256, 0, s>>>(op, (const uint4*)l, (const float*)r, (uint4*)y, total / 8, period / 8, act, act_a);
      else if (dt_r == DT_BF16) binary_period_vec_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(op, (const uint4*)l, (const __nv_bfloat16*)r, (uint4*)y, total / 8, period / 8, act, act_a);
      else binary_period_vec_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(op, (const uint4*)l, (const float*)r, (uint4*)y, total / 8, period / 8, act, act_a);
      return check_launch();
    }
  }
  binary_kernel<<<grid_for(total, 256), 256, 0, s>>>(op, g, dt_l, dt_r, dt_out, l, r, y, total, act, act_a);
  return check_launch();
}
int channel_affine(int dt, const void* x, void* y, const float* a, const float* b, int64_t outer, int64_t C, int64_t inner, cudaStream_t s) {
  int64_t total = outer * C * inner;
  if (total <= 0) return 0;
  channel_affine_kernel<<<grid_for(total, 256), 256, 0, s>>>(dt, x, y, a, b, total, C, inner);
  return check_launch();
}
// fp32 rows of up to 32 * NP elements, one warp per row: the row is read once into registers (lane l holds elements
// l, l + 32, ...), reduced with shuffles and written once.  Same arithmetic as softmax_rows_kernel / layernorm_kernel.
template <int NP, bool SOFTMAX>
__global__ void rows_f32_reg_kernel(const float* __restrict__ x, float* __restrict__ y, const float* __restrict__ gamma, const float* __restrict__ beta,
                                    int64_t rows, int dim, float eps, int log_form) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp; row < rows; row += nwarps) {
    const float* xr = x + row * dim;
    float* yr = y + row * dim;
    float v[NP];
#pragma unroll
    for (int i = 0; i < NP; ++i) { const int d = lane + 32 * i; v[i] = d < dim ? xr[d] : 0.f; }
    if (SOFTMAX) {
      float mx = -3.402823466e+38f;
#pragma unroll
      for (int i = 0; i < NP; ++i) if (lane + 32 * i < dim) mx = fmaxf(mx, v[i]);
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NP; ++i) if (lane + 32 * i < dim) sum += expf(v[i] - mx);
      sum = warp_sum(sum);
      const float lsum = logf(sum);
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) { const float t = v[i] - mx; yr[d] = log_form ? t - lsum : __fdiv_rn(expf(t), sum); }
      }
    } else {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < NP; ++i) if (lane + 32 * i < dim) s += v[i];
      const float mean = warp_sum(s) / (float)dim;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < NP; ++i) if (lane + 32 * i < dim) { const float t = v[i] - mean; q += t * t; }
      const float inv = 1.0f / sqrtf(warp_sum(q) / (float)dim + eps);
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int d = lane + 32 * i;
        if (d < dim) { const float t = (v[i] - mean) * inv; yr[d] = t * (gamma ? gamma[d] : 1.f) + (beta ? beta[d] : 0.f); }
      }
    }
  }
}
static bool launch_rows_f32(bool is_softmax, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim, float eps,
                            int log_form, cudaStream_t s) {
  if (dim > 2048) return false;
  const int grid = grid_for(rows * 32, 128);
#define B2_ROWS32(NP)                                                                                                                              \
  do {                                                                                                                                             \
    if (is_softmax) rows_f32_reg_kernel<NP, true><<<grid, 128, 0, s>>>((const float*)x, (float*)y, gamma, beta, rows, (int)dim, eps, log_form);     \
    else rows_f32_reg_kernel<NP, false><<<grid, 128, 0, s>>>((const float*)x, (float*)y, gamma, beta, rows, (int)dim, eps, log_form);               \
  } while (0)
  if (dim <= 128) B2_ROWS32(4);
  else if (dim <= 512) B2_ROWS32(16);
  else if (dim <= 1024) B2_ROWS32(32);
  else B2_ROWS32(64);
#undef B2_ROWS32
  return true;
}
int softmax(int dt, const void* x, void* y, int64_t outer, int64_t dim, int64_t inner, bool log_form, cudaStream_t s) {
  if (outer * dim * inner <= 0) return 0;
  if (inner == 1 && dt == DT_F32 && launch_rows_f32(true, x, y, nullptr, nullptr, outer, dim, 0.f, log_form, s)) return check_launch();
  if (inner == 1 && dt == DT_F16 && launch_rows_vec<__half>(true, x, y, nullptr, nullptr, outer, dim, 0.f, log_form, s)) return check_launch();
  if (inner == 1 && dt == DT_BF16 && launch_rows_vec<__nv_bfloat16>(true, x, y, nullptr, nullptr, outer, dim, 0.f, log_form, s)) return check_launch();
  if (inner == 1) softmax_rows_kernel<<<grid_for(outer * 32, 256), 256, 0, s>>>(dt, x, y, outer, dim, log_form);
  else softmax_strided_kernel<<<grid_for(outer * inner, 128), 128, 0, s>>>(dt, x, y, outer, dim, inner, log_form);
  return check_launch();
}
// Mean along one axis with 16-byte loads across the kept inner axis: a thread owns VEC neighbouring outputs and adds
// their `dim` terms one after the other (left to right, fp32, one division at the end), so every output is computed
// exactly as by the scalar kernel; only the memory accesses change.  IN = float, __half, __nv_bfloat16 or int8_t (int8
// terms are dequantised on the fly: fl(q * in_scale), the value a Dequantize node in front would have produced).
template <typename IN> struct RedVec { static constexpr int N = 16 / (int)sizeof(IN); };
template <typename IN> __device__ __forceinline__ void red_load(const IN* p, float in_scale, float (&f)[RedVec<IN>::N]) {
  const uint4 u = *(const uint4*)p;
  if constexpr (sizeof(IN) == 4) { const float* v = (const float*)&u; for (int i = 0; i < 4; ++i) f[i] = v[i]; }
  else if constexpr (sizeof(IN) == 1) { const int8_t* v = (const int8_t*)&u; for (int i = 0; i < 16; ++i) f[i] = __fmul_rn((float)v[i], in_scale); }
  else { const IN* v = (const IN*)&u; for (int i = 0; i < 8; ++i) f[i] = (float)v[i]; }
}
template <typename IN>
__global__ void reduce_mean_axis_vec_kernel(int dt_out, const IN* __restrict__ x, void* __restrict__ y, int64_t before, int64_t dim, int64_t after, float in_scale) {
  constexpr int VEC = RedVec<IN>::N;
  const int64_t av = after / VEC, total = before * av;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = e / av, k = (e - i * av) * VEC;
    const IN* p = x + (i * dim) * after + k;
    float s[VEC], t[VEC];
    red_load<IN>(p, in_scale, s);
    for (int64_t j = 1; j < dim; ++j) {
      red_load<IN>(p + j * after, in_scale, t);
#pragma unroll
      for (int q = 0; q < VEC; ++q) s[q] = __fadd_rn(s[q], t[q]);
    }
    const float d = (float)dim;
#pragma unroll
    for (int q = 0; q < VEC; ++q) store_from_float(y, dt_out, i * after + k + q, __fdiv_rn(s[q], d));
  }
}
// Two adjacent axes of D1 x D2 (a global average pool: 7 x 7) in one pass, with the arithmetic of the two single-axis
// passes: per second-axis index the first axis is summed left to right and divided, those quotients are summed left to
// right and divided.  All D1 * D2 loads of a thread are independent, so they overlap instead of waiting in a loop.
template <typename IN, int D1, int D2>
__global__ void reduce_mean_two_axes_kernel(int dt_out, const IN* __restrict__ x, void* __restrict__ y, int64_t before, int64_t after, float in_scale) {
  constexpr int VEC = RedVec<IN>::N;
  const int64_t av = after / VEC, total = before * av;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i = e / av, k = (e - i * av) * VEC;
    const IN* p = x + i * (D1 * D2) * after + k;
    float u[VEC];
#pragma unroll
    for (int w = 0; w < D2; ++w) {
      float s[VEC], t[VEC];
      red_load<IN>(p + (int64_t)w * after, in_scale, s);
#pragma unroll
      for (int h = 1; h < D1; ++h) {
        red_load<IN>(p + ((int64_t)h * D2 + w) * after, in_scale, t);
#pragma unroll
        for (int q = 0; q < VEC; ++q) s[q] = __fadd_rn(s[q], t[q]);
      }
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        const float m = __fdiv_rn(s[q], (float)D1);
        u[q] = w == 0 ? m : __fadd_rn(u[q], m);
      }
    }
#pragma unroll
    for (int q = 0; q < VEC; ++q) store_from_float(y, dt_out, i * after + k + q, __fdiv_rn(u[q], (float)D2));
  }
}
int reduce_mean_two_axes(int dt_in, int dt_out, const void* x, void* y, int64_t before, int64_t d1, int64_t d2, int64_t after, cudaStream_t s, float in_scale) {
  const int esz = dt_in == DT_F32 ? 4 : (dt_in == DT_S8 ? 1 : 2), vec = 16 / esz;
  if (d1 != 7 || d2 != 7 || after % vec != 0 || (uintptr_t)x % 16 != 0 || before * after <= 0) return 1;   // not taken: the caller runs the two passes
  if (!(dt_in == DT_F32 || dt_in == DT_F16 || dt_in == DT_BF16 || dt_in == DT_S8)) return 1;
  const int grid = grid_for(before * (after / vec), 128);
  if (dt_in == DT_F32) reduce_mean_two_axes_kernel<float, 7, 7><<<grid, 128, 0, s>>>(dt_out, (const float*)x, y, before, after, in_scale);
  else if (dt_in == DT_F16) reduce_mean_two_axes_kernel<__half, 7, 7><<<grid, 128, 0, s>>>(dt_out, (const __half*)x, y, before, after, in_scale);
  else if (dt_in == DT_BF16) reduce_mean_two_axes_kernel<__nv_bfloat16, 7, 7><<<grid, 128, 0, s>>>(dt_out, (const __nv_bfloat16*)x, y, before, after, in_scale);
  else reduce_mean_two_axes_kernel<int8_t, 7, 7><<<grid, 128, 0, s>>>(dt_out, (const int8_t*)x, y, before, after, in_scale);
  return check_launch();
}
__global__ void reduce_mean_axis_s8_kernel(int dt_out, const int8_t* x, void* y, int64_t before, int64_t dim, int64_t after, float in_scale) {
  int64_t total = before * after;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    int64_t i = e / after, k = e % after;
    float s = __fmul_rn((float)x[(i * dim) * after + k], in_scale);
    for (int64_t j = 1; j < dim; ++j) s = __fadd_rn(s, __fmul_rn((float)x[(i * dim + j) * after + k], in_scale));
    store_from_float(y, dt_out, e, __fdiv_rn(s, (float)dim));
  }
}
int reduce_mean_axis(int dt_in, int dt_out, const void* x, void* y, int64_t before, int64_t dim, int64_t after, cudaStream_t s, float in_scale) {
  if (before * after <= 0) return 0;
  const int esz = dt_in == DT_F32 ? 4 : (dt_in == DT_S8 ? 1 : 2), vec = 16 / esz;
  if ((dt_in == DT_F32 || dt_in == DT_F16 || dt_in == DT_BF16 || dt_in == DT_S8) && after % vec == 0 && (uintptr_t)x % 16 == 0) {
    const int64_t work = before * (after / vec);
    const int grid = grid_for(work, 128);
    if (dt_in == DT_F32) reduce_mean_axis_vec_kernel<float><<<grid, 128, 0, s>>>(dt_out, (const float*)x, y, before, dim, after, in_scale);
    else if (dt_in == DT_F16) reduce_mean_axis_vec_kernel<__half><<<grid, 128, 0, s>>>(dt_out, (const __half*)x, y, before, dim, after, in_scale);
    else if (dt_in == DT_BF16) reduce_mean_axis_vec_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(dt_out, (const __nv_bfloat16*)x, y, before, dim, after, in_scale);
    else reduce_mean_axis_vec_kernel<int8_t><<<grid, 128, 0, s>>>(dt_out, (const int8_t*)x, y, before, dim, after, in_scale);
    return check_launch();
  }
  if (dt_in == DT_S8) reduce_mean_axis_s8_kernel<<<grid_for(before * after, 128), 128, 0, s>>>(dt_out, (const int8_t*)x, y, before, dim, after, in_scale);
  else reduce_mean_axis_kernel<<<grid_for(before * after, 128), 128, 0, s>>>(dt_in, dt_out, x, y, before, dim, after);
  return check_launch();
}
int layernorm(int dt, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim, float eps, cudaStream_t s) {
  if (rows * dim <= 0) return 0;
  if (dt == DT_F16 && launch_rows_vec<__half>(false, x, y, gamma, beta, rows, dim, eps, 0, s)) return check_launch();
  if (dt == DT_BF16 && launch_rows_vec<__nv_bfloat16>(false, x, y, gamma, beta, rows, dim, eps, 0, s)) return check_launch();
  if (dt == DT_F32 && launch_rows_f32(false, x, y, gamma, beta, rows, dim, eps, 0, s)) return check_launch();
  layernorm_kernel<<<grid_for(rows * 32, 256), 256, 0, s>>>(dt, x, y, gamma, beta, rows, dim, eps);
  return check_launch();
}
int quantize(int dt_in, const void* x, void* q, const float* scale, const int* zp, int64_t outer, int64_t adim, int64_t inner,
             bool per_axis, bool is_unsigned, cudaStream_t s);
int layernorm_quantize(int dt, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim, float eps, void* q,
                       const float* scale, cudaStream_t s) {
  if (rows * dim <= 0) return 0;
  if (dt == DT_F16 && launch_rows_vec<__half>(false, x, y, gamma, beta, rows, dim, eps, 0, s, q, scale)) return check_launch();
  if (dt == DT_BF16 && launch_rows_vec<__nv_bfloat16>(false, x, y, gamma, beta, rows, dim, eps, 0, s, q, scale)) return check_launch();
  // rows the vector kernel does not take: the two passes one after the other
  if (int rc = layernorm(dt, x, y, gamma, beta, rows, dim, eps, s)) return rc;
  return quantize(dt, y, q, scale, nullptr, 1, 1, rows * dim, false, false, s);
}
// Per-tensor two-byte float -> int8, 16 elements per thread (two 16-byte loads, one 16-byte store).
template <typename T>
__global__ void quantize_h_s8_vec_kernel(const uint4* __restrict__ x, uint4* __restrict__ q, const float* scale, int64_t n16) {
  const QuantDiv qd(scale[0]);
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    uint4 out;
    uint32_t* o = (uint32_t*)&out;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint4 u = x[i * 2 + h];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const float2 f0 = pair_to_float2<T>(w[2 * t]), f1 = pair_to_float2<T>(w[2 * t + 1]);
        const int a = sat_s8(qd.rint_div(f0.x)), b = sat_s8(qd.rint_div(f0.y));
        const int c = sat_s8(qd.rint_div(f1.x)), d = sat_s8(qd.rint_div(f1.y));
        o[2 * h + t] = (uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8) | ((uint32_t)(c & 0xff) << 16) | ((uint32_t)(d & 0xff) << 24);
      }
    }
    q[i] = out;
  }
}
int quantize(int dt_in, const void* x, void* q, const float* scale, const int* zp, int64_t outer, int64_t adim, int64_t inner,
             bool per_axis, bool is_unsigned, cudaStream_t s) {
  int64_t total = outer * adim * inner;
  if (total <= 0) return 0;
  if (dt_in == DT_F32 && !per_axis && !zp && !is_unsigned && total % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)q % 16 == 0) {
    quantize_f32_s8_vec_kernel<<<grid_for(total / 16, 256), 256, 0, s>>>((const float4*)x, (uint4*)q, scale, total / 16);
    return check_launch();
  }
  if ((dt_in == DT_F16 || dt_in == DT_BF16) && !per_axis && !zp && !is_unsigned && total % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)q % 16 == 0) {
    if (dt_in == DT_F16) quantize_h_s8_vec_kernel<__half><<<grid_for(total / 16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)q, scale, total / 16);
    else quantize_h_s8_vec_kernel<__nv_bfloat16><<<grid_for(total / 16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)q, scale, total / 16);
    return check_launch();
  }
  quantize_kernel<<<grid_for(total, 256), 256, 0, s>>>(dt_in, x, q, scale, zp, total, adim, inner, per_axis, is_unsigned);
  return check_launch();
}
// Per-tensor int8 -> float storage type, 16 elements per thread: x = fl(float(q) * scale), one rounding to the storage type.
template <typename OUT>
__global__ void dequantize_s8_vec_kernel(const uint4* __restrict__ q, OUT* __restrict__ x, const float* __restrict__ scale, int64_t n16) {
  const float s = scale[0];
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 u = q[i];
    const int8_t* b = (const int8_t*)&u;
    if constexpr (sizeof(OUT) == 4) {
      float4* o = (float4*)(x + i * 16);
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = make_float4(__fmul_rn((float)b[4 * k], s), __fmul_rn((float)b[4 * k + 1], s), __fmul_rn((float)b[4 * k + 2], s), __fmul_rn((float)b[4 * k + 3], s));
    } else {
      __align__(16) OUT h[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) h[k] = (OUT)__fmul_rn((float)b[k], s);
      uint4* o = (uint4*)(x + i * 16);
      o[0] = ((const uint4*)h)[0];
      o[1] = ((const uint4*)h)[1];
    }
  }
}
// Requantisation of a value computed from int32 accumulators: q = sat(rne(x * inv)), 16 elements per thread.
template <typename IN>
__global__ void requantize_vec_kernel(const IN* __restrict__ x, uint4* __restrict__ q, float inv, int64_t n16) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    float f[16];
    if constexpr (sizeof(IN) == 4) {
      const float4* p = (const float4*)(x + i * 16);
#pragma unroll
      for (int k = 0; k < 4; ++k) { const float4 v = p[k]; f[4 * k] = v.x; f[4 * k + 1] = v.y; f[4 * k + 2] = v.z; f[4 * k + 3] = v.w; }
    } else {
      const uint4* p = (const uint4*)(x + i * 16);
      const uint4 a = p[0], b = p[1];
      const IN* ha = (const IN*)&a; const IN* hb = (const IN*)&b;
#pragma unroll
      for (int k = 0; k < 8; ++k) { f[k] = (float)ha[k]; f[8 + k] = (float)hb[k]; }
    }
    uint4 out;
    uint32_t* o = (uint32_t*)&out;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t w = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) w |= ((uint32_t)rne_sat_s8(__fmul_rn(f[4 * k + b], inv)) & 0xffu) << (8 * b);
      o[k] = w;
    }
    q[i] = out;
  }
}
int requantize(int dt_in, const void* x, void* q, float inv_scale, int64_t n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)q % 16 == 0 && (dt_in == DT_F32 || dt_in == DT_F16 || dt_in == DT_BF16)) {
    const int grid = grid_for(n / 16, 256);
    if (dt_in == DT_F32) requantize_vec_kernel<float><<<grid, 256, 0, s>>>((const float*)x, (uint4*)q, inv_scale, n / 16);
    else if (dt_in == DT_F16) requantize_vec_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, (uint4*)q, inv_scale, n / 16);
    else requantize_vec_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (uint4*)q, inv_scale, n / 16);
    return check_launch();
  }
  requantize_kernel<<<grid_for(n, 256), 256, 0, s>>>(dt_in, x, (int8_t*)q, inv_scale, n);
  return check_launch();
}
int dequantize(int dt_out, const void* q, void* x, const float* scale, const int* zp, int64_t outer, int64_t adim, int64_t inner,
               bool per_axis, bool is_unsigned, cudaStream_t s) {
  int64_t total = outer * adim * inner;
  if (total <= 0) return 0;
  if (!per_axis && !zp && !is_unsigned && total % 16 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)x % 16 == 0 &&
      (dt_out == DT_F32 || dt_out == DT_F16 || dt_out == DT_BF16)) {
    const int grid = grid_for(total / 16, 256);
    if (dt_out == DT_F32) dequantize_s8_vec_kernel<float><<<grid, 256, 0, s>>>((const uint4*)q, (float*)x, scale, total / 16);
    else if (dt_out == DT_F16) dequantize_s8_vec_kernel<__half><<<grid, 256, 0, s>>>((const uint4*)q, (__half*)x, scale, total / 16);
    else dequantize_s8_vec_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const uint4*)q, (__nv_bfloat16*)x, scale, total / 16);
    return check_launch();
  }
  dequantize_kernel<<<grid_for(total, 256), 256, 0, s>>>(dt_out, q, x, scale, zp, total, adim, inner, per_axis, is_unsigned);
  return check_launch();
}
int convert(int dt_in, int dt_out, const void* x, void* y, int64_t n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (dt_in == DT_F32 && dt_out == DT_F16 && n % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {
    convert_f32_f16_vec_kernel<<<grid_for(n / 8, 256), 256, 0, s>>>((const float4*)x, (uint4*)y, n / 8);
    return check_launch();
  }
  // two-byte -> fp32 (an fp16 / bf16 graph whose API outputs are fp32): four values per thread, as one long row
  if ((dt_in == DT_F16 || dt_in == DT_BF16) && dt_out == DT_F32 && n % 4 == 0 && n < (1 << 30) && (uintptr_t)x % 8 == 0 && (uintptr_t)y % 16 == 0)
    return convert_rows(dt_in, dt_out, x, y, 1, n, n, s);
  convert_kernel<<<grid_for(n, 256), 256, 0, s>>>(dt_in, dt_out, x, y, n);
  return check_launch();
}
__global__ void convert_rows_kernel(int dt_in, int dt_out, const void* x, void* y, int64_t rows, int64_t K, int64_t Kp) {
  const int64_t total = rows * K;
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / K, k = e - r * K;
    store_from_float(y, dt_out, e, load_as_float(x, dt_in, r * Kp + k));
  }
}
// Two-byte rows of pitch Kp -> dense fp32 rows of K.  Neighbouring threads write neighbouring floats (a warp's store is
// one contiguous run): four values per thread as one 16-byte store when the rows allow it, one value per thread otherwise.
template <typename IN>
__global__ void convert_rows_h_f32_v4_kernel(const IN* __restrict__ x, float4* __restrict__ y, int64_t total4, int K4, int64_t Kp) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total4; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / K4;
    const int k = (int)(e - r * K4) * 4;
    const uint2 u = *(const uint2*)(x + r * Kp + k);
    const IN* h = (const IN*)&u;
    y[e] = make_float4((float)h[0], (float)h[1], (float)h[2], (float)h[3]);
  }
}
template <typename IN>
__global__ void convert_rows_h_f32_flat_kernel(const IN* __restrict__ x, float* __restrict__ y, int64_t total, int K, int64_t Kp) {
  for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / K;
    y[e] = (float)x[r * Kp + (e - r * K)];
  }
}
int convert_rows(int dt_in, int dt_out, const void* x, void* y, int64_t rows, int64_t K, int64_t Kp, cudaStream_t s) {
  if (rows * K <= 0) return 0;
  if ((dt_in == DT_F16 || dt_in == DT_BF16) && dt_out == DT_F32 && K < (1 << 30)) {
    const bool v4 = K % 4 == 0 && Kp % 4 == 0 && (uintptr_t)x % 8 == 0 && (uintptr_t)y % 16 == 0;
    if (v4) {
      const int64_t total4 = rows * (K / 4);
      const int grid = grid_for(total4, 256);
      if (dt_in == DT_F16) convert_rows_h_f32_v4_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, (float4*)y, total4, (int)(K / 4), Kp);
      else convert_rows_h_f32_v4_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (float4*)y, total4, (int)(K / 4), Kp);
    } else {
      const int grid = grid_for(rows * K, 256);
      if (dt_in == DT_F16) convert_rows_h_f32_flat_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, (float*)y, rows * K, (int)K, Kp);
      else convert_rows_h_f32_flat_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (float*)y, rows * K, (int)K, Kp);
    }
    return check_launch();
  }
  convert_rows_kernel<<<grid_for(rows * K, 256), 256, 0, s>>>(dt_in, dt_out, x, y, rows, K, Kp);
  return check_launch();
}
// ---- range profiling: min / max per tensor and per channel (last axis) ----
// A float maps to an unsigned key that orders the same way (sign bit flipped for positives, all bits for negatives).
__device__ __forceinline__ unsigned range_key(float f) { const unsigned b = __float_as_uint(f); return (b & 0x80000000u) ? ~b : (b | 0x80000000u); }
__global__ void range_reset_kernel(unsigned* stats, int64_t channels) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < 2 + 2 * channels; i += (int64_t)gridDim.x * blockDim.x)
    stats[i] = (i == 0 || (i >= 2 && i < 2 + channels)) ? 0xffffffffu : 0u;   // minima start at the largest key, maxima at the smallest
}
// A block takes a contiguous run of rows; thread t keeps channels t, t + 256, ... (up to 16 of them) in registers and
// publishes them with one atomic pair per channel at the end.
__global__ void range_minmax_kernel(int dt, const void* __restrict__ x, int64_t rows, int channels, unsigned* __restrict__ stats) {
  const int64_t per_block = (rows + gridDim.x - 1) / gridDim.x, r0 = blockIdx.x * per_block, r1 = min(rows, r0 + per_block);
  for (int c0 = 0; c0 < channels; c0 += 16 * blockDim.x) {
    float mn[16], mx[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) { mn[k] = 3.402823466e+38f; mx[k] = -3.402823466e+38f; }
    for (int64_t r = r0; r < r1; ++r) {
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int c = c0 + threadIdx.x + k * blockDim.x;
        if (c < channels) { const float v = load_as_float(x, dt, r * channels + c); mn[k] = fminf(mn[k], v); mx[k] = fmaxf(mx[k], v); }
      }
    }
    if (r1 > r0) {
#pragma unroll
      for (int k = 0; k < 16; ++k) {
        const int c = c0 + threadIdx.x + k * blockDim.x;
        if (c < channels) {
          atomicMin(stats + 2 + c, range_key(mn[k])); atomicMax(stats + 2 + channels + c, range_key(mx[k]));
          atomicMin(stats, range_key(mn[k])); atomicMax(stats + 1, range_key(mx[k]));
        }
      }
    }
  }
}
int range_stats_reset(unsigned* stats, int64_t channels, cudaStream_t s) {
  range_reset_kernel<<<grid_for(2 + 2 * channels, 256), 256, 0, s>>>(stats, channels);
  return check_launch();
}
int range_minmax(int dt, const void* x, int64_t count, int64_t channels, unsigned* stats, cudaStream_t s) {
  if (count <= 0 || channels <= 0 || count % channels != 0 || channels > (1 << 30)) return 0;
  if (dt != DT_F32 && dt != DT_F16 && dt != DT_BF16) return 0;
  const int64_t rows = count / channels;
  int grid = (int)std::min<int64_t>(rows, (int64_t)sm_count() * 8);
  range_minmax_kernel<<<grid > 0 ? grid : 1, 256, 0, s>>>(dt, x, rows, (int)channels, stats);
  return check_launch();
}
// out[b][n][k] = in[b][k][n]: the last two axes swapped, through 32 x 32 shared-memory tiles so that both the reads
// (along n) and the writes (along k) are contiguous.
template <typename T>
__global__ void transpose_last2_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t in_off, int64_t out_off, int N, int K, int tiles_n, int tiles_k) {
  __shared__ T tile[32][33];
  const int64_t b = blockIdx.x / (tiles_n * tiles_k);
  const int t = (int)(blockIdx.x % (tiles_n * tiles_k));
  const int n0 = (t % tiles_n) * 32, k0 = (t / tiles_n) * 32;
  const T* src = x + in_off + b * (int64_t)N * K;
  T* dst = y + out_off + b * (int64_t)N * K;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int k = k0 + r, n = n0 + threadIdx.x;
    if (k < K && n < N) tile[r][threadIdx.x] = src[(int64_t)k * N + n];
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int n = n0 + r, k = k0 + threadIdx.x;
    if (n < N && k < K) dst[(int64_t)n * K + k] = tile[threadIdx.x][r];
  }
}
template <typename T>
static bool launch_transpose_last2(const MoveGeom& g, const void* x, void* y, cudaStream_t s) {
  // canonical rank 2 or 3: out [B][N][K] dense, in strides {N*K, 1, N}
  const int r = g.rank;
  if (r != 2 && r != 3) return false;
  const int64_t N = g.oshape[r - 2], K = g.oshape[r - 1], B = r == 3 ? g.oshape[0] : 1;
  if (g.ostride[r - 1] != 1 || g.ostride[r - 2] != K || g.istride[r - 2] != 1 || g.istride[r - 1] != N) return false;
  if (r == 3 && (g.ostride[0] != N * K || g.istride[0] != N * K)) return false;
  if (N > (1 << 30) || K > (1 << 30)) return false;
  const int tn = (int)((N + 31) / 32), tk = (int)((K + 31) / 32);
  const int64_t blocks = B * tn * tk;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return false;
  transpose_last2_kernel<T><<<(unsigned)blocks, dim3(32, 8), 0, s>>>((const T*)x, (T*)y, g.in_offset, g.out_offset, (int)N, (int)K, tn, tk);
  return true;
}
int move(const MoveGeom& g0, int esz, const void* x, void* y, cudaStream_t s) {
  MoveGeom g = g0;
  // Canonical form first: axes of extent 1 dropped, neighbours that are contiguous on both sides merged.
  {
    int r = 0;
    for (int d = 0; d < g.rank; ++d) {
      if (g.oshape[d] == 1 && g.rank > 1) continue;
      if (r > 0 && g.istride[r - 1] == g.istride[d] * g.oshape[d] && g.ostride[r - 1] == g.ostride[d] * g.oshape[d]) {
        g.oshape[r - 1] *= g.oshape[d];
        g.istride[r - 1] = g.istride[d];
        g.ostride[r - 1] = g.ostride[d];
        continue;
      }
      g.oshape[r] = g.oshape[d]; g.istride[r] = g.istride[d]; g.ostride[r] = g.ostride[d];
      ++r;
    }
    if (r == 0) { g.oshape[0] = 1; g.istride[0] = 1; g.ostride[0] = 1; r = 1; }
    g.rank = r;
  }
  if (g.rank >= 2 && g.istride[g.rank - 1] != 1) {
    bool done = esz == 1 ? launch_transpose_last2<uint8_t>(g, x, y, s) : esz == 2 ? launch_transpose_last2<uint16_t>(g, x, y, s)
              : esz == 4 ? launch_transpose_last2<uint32_t>(g, x, y, s) : esz == 8 ? launch_transpose_last2<uint64_t>(g, x, y, s) : false;
    if (done) return check_launch();
  }
  // When the innermost axis is contiguous on both sides (a head split / merge, a concat along an outer axis), move
  // the widest power-of-two unit up to 16 bytes that divides every stride, offset and the innermost extent.
  if (g.rank >= 1 && g.istride[g.rank - 1] == 1 && g.ostride[g.rank - 1] == 1) {
    for (int unit = 16; unit > esz; unit /= 2) {
      const int v = unit / esz;
      bool ok = unit % esz == 0 && g.oshape[g.rank - 1] % v == 0 && g.in_offset % v == 0 && g.out_offset % v == 0 &&
                (uintptr_t)x % unit == 0 && (uintptr_t)y % unit == 0;
      for (int d = 0; d + 1 < g.rank && ok; ++d) ok = g.istride[d] % v == 0 && g.ostride[d] % v == 0;
      if (!ok) continue;
      g.oshape[g.rank - 1] /= v;
      for (int d = 0; d + 1 < g.rank; ++d) { g.istride[d] /= v; g.ostride[d] /= v; }
      g.in_offset /= v; g.out_offset /= v;
      esz = unit;
      break;
    }
  }
  int64_t total = 1;
  for (int d = 0; d < g.rank; ++d) total *= g.oshape[d];
  if (total <= 0) return 0;
  int grid = grid_for(total, 256);
  switch (esz) {
    case 16: move_kernel<uint4><<<grid, 256, 0, s>>>(g, (const uint4*)x, (uint4*)y, total); break;
    case 1: move_kernel<uint8_t><<<grid, 256, 0, s>>>(g, (const uint8_t*)x, (uint8_t*)y, total); break;
    case 2: move_kernel<uint16_t><<<grid, 256, 0, s>>>(g, (const uint16_t*)x, (uint16_t*)y, total); break;
    case 4: move_kernel<uint32_t><<<grid, 256, 0, s>>>(g, (const uint32_t*)x, (uint32_t*)y, total); break;
    case 8: move_kernel<uint64_t><<<grid, 256, 0, s>>>(g, (const uint64_t*)x, (uint64_t*)y, total); break;
    default: return -1;
  }
  return check_launch();
}
int pad_channels(int esz, const void* x, void* y, int64_t pixels, int C, int Cp, cudaStream_t s) {
  if (pixels <= 0) return 0;
  if (Cp * esz != 32 || C > Cp || (uintptr_t)y % 16 != 0) return -1;
  int grid = grid_for(pixels, 256);
  if (esz == 1) pad_channels_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint4*)y, pixels, C);
  else if (esz == 2) pad_channels_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint4*)y, pixels, C);
  else return -1;
  return check_launch();
}
int stem_widen(int esz, const void* x, void* y, int N, int H, int W, int C, int Q, cudaStream_t s) {
  int64_t total = (int64_t)N * H * Q * (32 * esz / 16);
  if (total <= 0) return 0;
  if (C > 4 || (uintptr_t)y % 16 != 0) return -1;
  int grid = grid_for(total, 256);
  if (esz == 1) stem_widen_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint4*)y, N, H, W, C, Q);
  else if (esz == 2) stem_widen_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint4*)y, N, H, W, C, Q);
  else return -1;
  return check_launch();
}
int stem_pad(int esz, const void* x, void* y, int N, int H, int W, int C, int pixel_bytes, int lp, int Wp, cudaStream_t s) {
  int64_t rows = (int64_t)N * H, total = rows * Wp;
  if (total <= 0) return 0;
  const int cp = pixel_bytes / esz;
  if (C > cp || (uintptr_t)y % 16 != 0) return -1;
  int grid = grid_for(total, 256);
  if (esz == 1 && cp == 4) stem_pad_kernel<uint8_t, 4><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, rows, W, C, lp, Wp);
  else if (esz == 1 && cp == 8) stem_pad_kernel<uint8_t, 8><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, rows, W, C, lp, Wp);
  else if (esz == 1 && cp == 16) stem_pad_kernel<uint8_t, 16><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, rows, W, C, lp, Wp);
  else if (esz == 2 && cp == 4) stem_pad_kernel<uint16_t, 4><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, rows, W, C, lp, Wp);
  else if (esz == 2 && cp == 8) stem_pad_kernel<uint16_t, 8><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, rows, W, C, lp, Wp);
  else return -1;
  return check_launch();
}
int resize_nearest(int esz, const void* x, void* y, int N, int H, int W, int C, int P, int Q, bool nhwc, cudaStream_t s) {
  int64_t total = (int64_t)N * P * Q * C;
  if (total <= 0) return 0;
  if (nhwc && ((int64_t)C * esz) % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {  // whole 16-byte pieces of a pixel per thread
    const int C16 = (int)((int64_t)C * esz / 16);
    resize_nearest_kernel<uint4><<<grid_for((int64_t)N * P * Q * C16, 256), 256, 0, s>>>((const uint4*)x, (uint4*)y, N, H, W, C16, P, Q, 1);
    return check_launch();
  }
  int grid = grid_for(total, 256);
  switch (esz) {
    case 1: resize_nearest_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, N, H, W, C, P, Q, nhwc); break;
    case 2: resize_nearest_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, N, H, W, C, P, Q, nhwc); break;
    case 4: resize_nearest_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)x, (uint32_t*)y, N, H, W, C, P, Q, nhwc); break;
    default: return -1;
  }
  return check_launch();
}
int gather(int esz, const void* x, const void* idx, int idx_dt, void* y, int64_t outer, int64_t axis_dim, int64_t n_idx, int64_t inner,
           cudaStream_t s) {
  int64_t total = outer * n_idx * inner;
  if (total <= 0) return 0;
  if ((inner * esz) % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0) {  // rows are copied in 16-byte pieces
    const int64_t inner16 = inner * esz / 16;
    gather_kernel<uint4><<<grid_for(outer * n_idx * inner16, 256), 256, 0, s>>>((const uint4*)x, idx, idx_dt, (uint4*)y, outer, axis_dim, n_idx, inner16);
    return check_launch();
  }
  int grid = grid_for(total, 256);
  switch (esz) {
    case 1: gather_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, idx, idx_dt, (uint8_t*)y, outer, axis_dim, n_idx, inner); break;
    case 2: gather_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)x, idx, idx_dt, (uint16_t*)y, outer, axis_dim, n_idx, inner); break;
    case 4: gather_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)x, idx, idx_dt, (uint32_t*)y, outer, axis_dim, n_idx, inner); break;
    default: return -1;
  }
  return check_launch();
}

}  // namespace b200
