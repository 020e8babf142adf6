// Device helpers shared by the CUDA-core and tensor-core kernels: typed loads/stores and the
// accumulator epilogue.  Every floating-point step uses the *_rn intrinsics so the compiler
// cannot contract a multiply and an add into one fused operation; the int8 path depends on
// that to match a node-by-node fp32 evaluation bit for bit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "kernels.h"

namespace b200 {

__device__ __forceinline__ float load_as_float(const void* p, int dt, int64_t i) {
  switch (dt) {
    case DT_F32: return ((const float*)p)[i];
    case DT_F16: return __half2float(((const __half*)p)[i]);
    case DT_BF16: return __bfloat162float(((const __nv_bfloat16*)p)[i]);
    case DT_S8: return (float)((const int8_t*)p)[i];
    case DT_U8: return (float)((const uint8_t*)p)[i];
    case DT_S32: return (float)((const int32_t*)p)[i];
    case DT_S64: return (float)((const long long*)p)[i];
  }
  return 0.f;
}
__device__ __forceinline__ int8_t sat_s8(float r) {  // r already rounded to an integer value
  r = fminf(fmaxf(r, -128.f), 127.f);
  return (int8_t)(int)r;
}
// sat(rne(x)) to int8 in one instruction (cvt.rni.sat.s8.f32); the result sits in the low byte.
__device__ __forceinline__ int rne_sat_s8(float x) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ uint8_t sat_u8(float r) {
  r = fminf(fmaxf(r, 0.f), 255.f);
  return (uint8_t)(int)r;
}
__device__ __forceinline__ void store_from_float(void* p, int dt, int64_t i, float v) {
  switch (dt) {
    case DT_F32: ((float*)p)[i] = v; break;
    case DT_F16: ((__half*)p)[i] = __float2half_rn(v); break;
    case DT_BF16: ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v); break;
    case DT_S8: ((int8_t*)p)[i] = sat_s8(rintf(v)); break;
    case DT_U8: ((uint8_t*)p)[i] = sat_u8(rintf(v)); break;
    case DT_S32: ((int32_t*)p)[i] = (int32_t)v; break;
    case DT_S64: ((long long*)p)[i] = (long long)v; break;
  }
}

__device__ __forceinline__ float apply_act(int act, float t, float a, float b) {
  switch (act) {
    case ACT_RELU: return t > 0.f ? t : 0.f;
    case ACT_LEAKY: return t < 0.f ? __fmul_rn(a, t) : t;
    case ACT_CLAMP: return t < a ? a : (t > b ? b : t);
    case ACT_GELU_ERF: return __fmul_rn(__fmul_rn(0.5f, t), __fadd_rn(1.0f, erff(__fmul_rn(t, 0.70710678118654752440f))));
    case ACT_GELU_TANH: {
      float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
      return 0.5f * t * (1.0f + tanhf(u));
    }
  }
  return t;
}

// The same activation over N register-resident values with the dispatch outside the loop, so that the N
// evaluations (an erf or tanh each, for GELU) are independent instruction streams the scheduler can interleave.
template <int N>
__device__ __forceinline__ void apply_act_all(int act, float (&v)[N], float a, float b) {
  switch (act) {
    case ACT_RELU:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = apply_act(ACT_RELU, v[j], a, b);
      break;
    case ACT_LEAKY:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = apply_act(ACT_LEAKY, v[j], a, b);
      break;
    case ACT_CLAMP:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = apply_act(ACT_CLAMP, v[j], a, b);
      break;
    case ACT_GELU_ERF:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = apply_act(ACT_GELU_ERF, v[j], a, b);
      break;
    case ACT_GELU_TANH:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = apply_act(ACT_GELU_TANH, v[j], a, b);
      break;
    default: break;
  }
}

// Steps that depend only on the column (output channel), applied to t = (float)acc.
__device__ __forceinline__ float epilogue_value(const Epilogue& ep, float t, int64_t row, int col, int64_t ld) {
  if (ep.mul) t = __fmul_rn(t, ep.mul[col]);
  if (ep.alpha != 1.f) t = __fmul_rn(t, ep.alpha);
  if (ep.add1) t = __fadd_rn(t, ep.add1[col]);
  if (ep.add2) t = __fadd_rn(t, ep.add2[col]);
  if (ep.add_full) t = __fadd_rn(t, __fmul_rn(ep.beta_full, load_as_float(ep.add_full, ep.add_full_dt, row * ld + col)));
  if (ep.act_first) t = apply_act(ep.act, t, ep.act_a, ep.act_b);
  if (ep.res) {
    float r = load_as_float(ep.res, ep.res_dt, row * ld + col);
    if (ep.res_dt == DT_S8) r = __fmul_rn(r, ep.res_scale);
    t = __fadd_rn(t, r);
  }
  if (!ep.act_first) t = apply_act(ep.act, t, ep.act_a, ep.act_b);
  if (ep.out_dt == DT_S8) t = ep.out_multiply ? __fmul_rn(t, ep.out_inv) : __fdiv_rn(t, ep.out_scale);
  return t;
}

}  // namespace b200
