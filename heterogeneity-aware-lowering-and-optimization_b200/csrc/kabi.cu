// Raw kernel entry points of the C ABI (declared in include/odla_b200.h): thin wrappers that
// let a caller that already holds device memory run one kernel without building a graph.
#include <cstdio>
#include <cstdlib>

#include "common.h"

using namespace b200;

extern "C" int odla_b200_conv_umma(const odla_b200_conv_desc* d, const void* x, const void* w, const float* mul, const float* add,
                                   const void* residual, void* y, void* stream) {
  if (!d || !x || !w || !y) return -1;
  if (visible_devices() <= 0) {
    fprintf(stderr, "[odla_b200] odla_b200_conv_umma: no CUDA device (there is no CPU fallback)\n");
    return -2;
  }
  int in_dt = d->dtype == 0 ? DT_F16 : d->dtype == 1 ? DT_BF16 : d->dtype == 2 ? DT_S8 : -1;
  if (in_dt < 0) return -1;
  UmmaConv c{d->n, d->h, d->w, d->c, d->k, d->r, d->s, d->p, d->q, d->stride_h, d->stride_w, d->pad_top, d->pad_left, in_dt};
  if (!umma_conv_supported(c)) return -1;
  Epilogue ep;
  ep.mul = mul;
  ep.add1 = add;
  ep.res = residual;
  ep.res_dt = d->res_kind == 0 ? in_dt : d->res_kind == 1 ? DT_F32 : DT_S8;
  if (ep.res_dt == DT_S8 && d->res_kind == 0) ep.res_dt = DT_S8;
  ep.res_scale = d->res_scale;
  ep.act = d->act == 1 ? ACT_RELU : d->act == 2 ? ACT_LEAKY : ACT_NONE;
  ep.act_a = d->alpha;
  switch (d->out_kind) {
    case 0: ep.out_dt = in_dt == DT_S8 ? DT_F32 : in_dt; break;
    case 1: ep.out_dt = DT_F32; break;
    case 2: ep.out_dt = DT_S8; ep.out_scale = d->out_scale; ep.out_inv = 1.0f / d->out_scale; ep.out_multiply = d->out_multiply != 0; break;
    case 3: if (in_dt != DT_S8) return -1; ep.out_dt = DT_S32; break;
    default: return -1;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int* status = nullptr;
  if (cudaMalloc((void**)&status, kStatusBytes) != cudaSuccess) return -2;
  cudaMemsetAsync(status, 0, kStatusBytes, (cudaStream_t)stream);
  UmmaLaunch* L = umma_conv_prepare(c, x, w, y, ep, status, sms);
  if (!L) { cudaFree(status); return -2; }
  int rc = umma_conv_run(L, (cudaStream_t)stream);
  int host_status[2] = {0, 0};
  if (rc == 0 && cudaMemcpyAsync(host_status, status, sizeof(host_status), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess) rc = -2;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) rc = -2;
  umma_conv_destroy(L);
  if (getenv("ODLA_B200_DEBUG_TS")) {
    // only meaningful in a build with UMMA_DEBUG_TS: block 0's timeline (ns) and the cycles it spent in each wait
    unsigned long long ts[124];
    cudaMemcpy(ts, (char*)status + 32, sizeof(ts), cudaMemcpyDeviceToHost);
    fprintf(stderr, "ts(ns rel. to kernel entry): sync=%lld tfull0=%lld epi0_end=%lld teardown=%lld | cycles %lld\n", (long long)(ts[0] - ts[7]),
            (long long)(ts[4] - ts[7]), (long long)(ts[5] - ts[7]), (long long)(ts[6] - ts[7]), (long long)(ts[16 + 6] - ts[16 + 7]));
    static const char* site[8] = {"", "producer<-empty", "mma<-tempty", "mma<-full", "epi<-tfull", "loader<-box_free", "epi<-box_full", "storer<-box_done"};
    for (int code = 1; code < 8; ++code) {
      const unsigned long long* c4 = ts + 28 + code * 4;  // ts[] starts at status + 32 bytes = 4 words
      fprintf(stderr, "  wait %-18s %10llu %10llu %10llu %10llu\n", site[code], c4[0], c4[1], c4[2], c4[3]);
    }
  }
  if (rc == 0 && host_status[0] != 0) {
    fprintf(stderr, "[odla_b200] odla_b200_conv_umma: bounded wait expired (code %d, block %d)\n", host_status[0], host_status[1]);
    cudaFree(status);
    return -3;
  }
  cudaFree(status);
  return rc;
}

// Raw fused attention over device pointers (see AttnLaunch in kernels.h): dtype 0 = fp16, 1 = bf16.  Synchronous.
// Returns 0, -1 (unsupported arguments), -2 (CUDA failure) or -3 (a bounded wait inside the kernel expired).
extern "C" int odla_b200_attention(int dtype, const void* q, const void* k, const void* v, void* y, long long batch, int heads, int positions, int channels,
                                   float scale, int merge_heads, void* stream) {
  if (!q || !k || !v || !y || batch <= 0 || heads <= 0) return -1;
  if (visible_devices() <= 0) {
    fprintf(stderr, "[odla_b200] odla_b200_attention: no CUDA device (there is no CPU fallback)\n");
    return -2;
  }
  const int dt = dtype == 0 ? DT_F16 : dtype == 1 ? DT_BF16 : -1;
  if (dt < 0 || !attn_supported(dt, positions, channels)) return -1;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int* status = nullptr;
  if (cudaMalloc((void**)&status, kStatusBytes) != cudaSuccess) return -2;
  cudaMemsetAsync(status, 0, kStatusBytes, (cudaStream_t)stream);
  AttnLaunch* L = attn_prepare(dt, q, k, v, y, batch, heads, scale, merge_heads != 0, status, sms);
  if (!L) { cudaFree(status); return -2; }
  int rc = attn_run(L, (cudaStream_t)stream);
  int host_status[2] = {0, 0};
  if (rc == 0 && cudaMemcpyAsync(host_status, status, sizeof(host_status), cudaMemcpyDeviceToHost, (cudaStream_t)stream) != cudaSuccess) rc = -2;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) rc = -2;
  attn_destroy(L);
  cudaFree(status);
  if (rc == 0 && host_status[0] != 0) {
    fprintf(stderr, "[odla_b200] odla_b200_attention: bounded wait expired (code %d, block %d)\n", host_status[0], host_status[1]);
    return -3;
  }
  return rc;
}
