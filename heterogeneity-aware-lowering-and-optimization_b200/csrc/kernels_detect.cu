// Detection post-processing: odla_NMS (ODLA/include/ODLA/ops/odla_ops_nn.h:504-507) and odla_PostProcess
// (odla_ops_nn.h:757-759).
//
// Greedy non-maximum suppression is a walk over the candidates in descending score order; sorting them first is what
// a CPU does.  Here one CTA owns one (batch, class) problem and repeats: block-wide arg-max over the candidates that
// are still eligible (score, then the lower index on a tie -- the order a stable descending sort gives), record it,
// strike what it suppresses.  That is the same walk without the sort, costs one pass over the scores per SELECTED box
// (a few dozen for real detectors) and needs no scratch beyond a bit mask in shared memory.
//
//   mode 0  odla_NMS: the ONNX NonMaxSuppression rule the reference's emitter maps to it
//           (lib/target/generic_cpp/nms.cc:22-69): boxes [B, N, 4] as (y1, x1, y2, x2) in any corner order, scores
//           [B, C, N]; a candidate is dropped for good once its IoU with ANY selected box exceeds the threshold.
//   mode 1  the rule of the reference's YOLOv3 post-processing vertex
//           (ODLA/platforms/odla_popart/custom_ops/codelets_nms.cpp:23-71): a candidate is compared with the LAST selected
//           box only, scores below the threshold are skipped, boxes are (y_min, x_min, y_max, x_max).
//
// Every floating-point step uses the *_rn intrinsics in the order of the CPU oracle, so both pick the same boxes.
#include <cstdio>

#include "epilogue.cuh"

namespace b200 {

namespace {

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[odla_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return -2;
  }
  return 0;
}

struct Cand { float score; int idx; };
__device__ __forceinline__ bool better(const Cand& a, const Cand& b) { return a.score > b.score || (a.score == b.score && a.idx < b.idx); }
__device__ __forceinline__ Cand warp_best(Cand c) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Cand d;
    d.score = __shfl_xor_sync(0xffffffffu, c.score, o);
    d.idx = __shfl_xor_sync(0xffffffffu, c.idx, o);
    if (d.idx >= 0 && (c.idx < 0 || better(d, c))) c = d;
  }
  return c;
}
__device__ __forceinline__ void load_box(const void* boxes, int dt, int64_t i, float (&b)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) b[k] = load_as_float(boxes, dt, i * 4 + k);
}
// IoU > threshold, ONNX form: corners in any order, empty unions never suppress.
__device__ __forceinline__ bool overlaps_onnx(const float (&a)[4], const float (&b)[4], float thr) {
  const float ay1 = fminf(a[0], a[2]), ay2 = fmaxf(a[0], a[2]), ax1 = fminf(a[1], a[3]), ax2 = fmaxf(a[1], a[3]);
  const float by1 = fminf(b[0], b[2]), by2 = fmaxf(b[0], b[2]), bx1 = fminf(b[1], b[3]), bx2 = fmaxf(b[1], b[3]);
  const float ih = __fsub_rn(fminf(ay2, by2), fmaxf(ay1, by1)), iw = __fsub_rn(fminf(ax2, bx2), fmaxf(ax1, bx1));
  if (ih <= 0.f || iw <= 0.f) return false;
  const float inter = __fmul_rn(ih, iw);
  const float area_a = __fmul_rn(__fsub_rn(ay2, ay1), __fsub_rn(ax2, ax1)), area_b = __fmul_rn(__fsub_rn(by2, by1), __fsub_rn(bx2, bx1));
  const float uni = __fsub_rn(__fadd_rn(area_a, area_b), inter);
  if (uni <= 0.f) return false;
  return __fdiv_rn(inter, uni) > thr;
}
// The reference vertex's test (codelets_nms.cpp:32-46).
__device__ __forceinline__ bool overlaps_yolo(const float (&s)[4], const float (&c)[4], float thr) {
  const float y_top = fmaxf(s[0], c[0]), x_left = fmaxf(s[1], c[1]), y_bot = fminf(s[2], c[2]), x_right = fminf(s[3], c[3]);
  if (x_right < x_left || y_bot < y_top) return false;
  const float comm = __fmul_rn(__fsub_rn(x_right, x_left), __fsub_rn(y_bot, y_top));
  const float sa = __fmul_rn(__fsub_rn(s[2], s[0]), __fsub_rn(s[3], s[1])), ca = __fmul_rn(__fsub_rn(c[2], c[0]), __fsub_rn(c[3], c[1]));
  return __fdiv_rn(comm, __fsub_rn(__fadd_rn(sa, ca), comm)) > thr;
}

// grid = problems (batch x class); sel[p][k] = k-th selected box of problem p, cnt[p] = how many.
template <int MODE>
__global__ void greedy_nms_kernel(const void* __restrict__ boxes, int box_dt, const void* __restrict__ scores, int score_dt, int C, int N, int max_sel,
                                  float iou_thr, float score_thr, int* __restrict__ sel, int* __restrict__ cnt) {
  extern __shared__ uint32_t alive[];          // MODE 0: one bit per candidate
  __shared__ Cand warp_c[32];
  __shared__ Cand chosen;
  const int p = blockIdx.x, b = p / C;
  const int64_t sbase = (int64_t)p * N, bbase = (int64_t)b * N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if (MODE == 0) {
    for (int w = threadIdx.x; w < (N + 31) / 32; w += blockDim.x) {
      uint32_t m = 0;
      for (int j = 0; j < 32; ++j) { const int i = w * 32 + j; if (i < N && load_as_float(scores, score_dt, sbase + i) > score_thr) m |= 1u << j; }
      alive[w] = m;
    }
    __syncthreads();
  }
  Cand last; last.score = 0.f; last.idx = -1;
  float lb[4] = {0.f, 0.f, 0.f, 0.f};
  int n_sel = 0;
  while (n_sel < max_sel) {
    Cand best; best.score = 0.f; best.idx = -1;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
      bool ok;
      Cand c; c.idx = i;
      if (MODE == 0) {
        ok = (alive[i >> 5] >> (i & 31)) & 1u;
        if (!ok) continue;
        c.score = load_as_float(scores, score_dt, sbase + i);
      } else {
        c.score = load_as_float(scores, score_dt, sbase + i);
        ok = !(c.score < score_thr);
        // after the last selected one in (score descending, index ascending) order, and not overlapping it
        if (ok && last.idx >= 0) {
          ok = better(last, c);
          if (ok) { float cb[4]; load_box(boxes, box_dt, bbase + i, cb); ok = !overlaps_yolo(lb, cb, iou_thr); }
        }
        if (!ok) continue;
      }
      if (best.idx < 0 || better(c, best)) best = c;
    }
    best = warp_best(best);
    if (lane == 0) warp_c[warp] = best;
    __syncthreads();
    if (warp == 0) {
      Cand c = lane < nwarps ? warp_c[lane] : Cand{0.f, -1};
      c = warp_best(c);
      if (lane == 0) chosen = c;
    }
    __syncthreads();
    last = chosen;
    if (last.idx < 0) break;
    if (threadIdx.x == 0) sel[(int64_t)p * max_sel + n_sel] = last.idx;
    ++n_sel;
    load_box(boxes, box_dt, bbase + last.idx, lb);
    if (MODE == 0) {
      // strike the selected box and everything it suppresses; each thread owns whole mask words
      for (int w = threadIdx.x; w < (N + 31) / 32; w += blockDim.x) {
        uint32_t m = alive[w];
        if (!m) continue;
        for (int j = 0; j < 32; ++j) {
          if (!((m >> j) & 1u)) continue;
          const int i = w * 32 + j;
          bool kill = i == last.idx;
          if (!kill) { float cb[4]; load_box(boxes, box_dt, bbase + i, cb); kill = overlaps_onnx(lb, cb, iou_thr); }
          if (kill) m &= ~(1u << j);
        }
        alive[w] = m;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) cnt[p] = n_sel;
}

// Selections of all problems in (batch, class, selection order) order -> rows (batch, class, box) of the output,
// at most `rows`; the rest is filled with -1.
__global__ void nms_emit_kernel(const int* __restrict__ sel, const int* __restrict__ cnt, int problems, int C, int max_sel, int rows, int out64, void* out) {
  __shared__ int start[1025];
  if (threadIdx.x == 0) { int s = 0; for (int p = 0; p < problems; ++p) { start[p] = s; s += cnt[p]; } start[problems] = s; }
  __syncthreads();
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    int v[3] = {-1, -1, -1};
    if (r < start[problems]) {
      int lo = 0, hi = problems;   // the problem whose range holds row r
      while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (start[mid] <= r) lo = mid; else hi = mid; }
      v[0] = lo / C; v[1] = lo % C; v[2] = sel[(int64_t)lo * max_sel + (r - start[lo])];
    }
    for (int k = 0; k < 3; ++k) { if (out64) ((long long*)out)[r * 3 + k] = v[k]; else ((int*)out)[r * 3 + k] = v[k]; }
  }
}

// YOLOv3 head decoding as the reference's DecodeVertex does it (codelets_nms.cpp:73-120) after exponentiating the whole
// head (postprocess.cc, expInPlace): boxes become (y_min, x_min, y_max, x_max) in pixels of the original image,
// objectness e/(e+1), class scores e/(e+1) * objectness.  One thread per (cell, anchor).
__global__ void yolo_decode_kernel(const void* __restrict__ head, int dt, int nchw, int S, int cls, int first, int N, const unsigned* __restrict__ anchors6,
                                   const unsigned* __restrict__ img_w, const unsigned* __restrict__ img_h, float* __restrict__ boxes, float* __restrict__ scores) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= S * S * 3) return;
  const int a = t % 3, x = (t / 3) % S, y = t / (3 * S);
  const int ch = cls + 5;
  auto at = [&](int k) {
    const int c = a * ch + k;
    const int64_t i = nchw ? ((int64_t)c * S + y) * S + x : ((int64_t)y * S + x) * (3 * ch) + c;
    return expf(load_as_float(head, dt, i));
  };
  const unsigned ow = *img_w, oh = *img_h;
  const float scale = (float)fmin(416.0 / oh, 416.0 / ow);
  const float nh = roundf(oh * scale), nw = roundf(ow * scale);
  const float off_h = (float)((416 - nh) / 2.0 / 416), off_w = (float)((416 - nw) / 2.0 / 416);
  const float sc_h = 416 / nh, sc_w = 416 / nw;
  const float e0 = at(0), e1 = at(1), e2 = at(2), e3 = at(3), e4 = at(4);
  float dx = ((e0 / (e0 + 1)) + x) / S;
  dx = (dx - off_w) * sc_w;
  float dy = ((e1 / (e1 + 1)) + y) / S;
  dy = (dy - off_h) * sc_h;
  const float dw = (e2 * anchors6[a << 1]) / 416 * sc_w, dh = (e3 * anchors6[a << 1 | 1]) / 416 * sc_h;
  const int n = first + t;
  boxes[n * 4 + 0] = (float)((dy - dh / 2.0) * oh);
  boxes[n * 4 + 1] = (float)((dx - dw / 2.0) * ow);
  boxes[n * 4 + 2] = (float)((dy + dh / 2.0) * oh);
  boxes[n * 4 + 3] = (float)((dx + dw / 2.0) * ow);
  const float conf = e4 / (e4 + 1);
  for (int c = 0; c < cls; ++c) { const float e = at(5 + c); scores[(int64_t)c * N + n] = e / (e + 1) * conf; }
}
// selected_info[c][k] = (y_min, x_min, y_max, x_max, score) of class c's k-th selection, zeros beyond the count.
__global__ void yolo_emit_kernel(const int* __restrict__ sel, const int* __restrict__ cnt, const float* __restrict__ boxes, const float* __restrict__ scores,
                                 int cls, int N, int per_class, float* __restrict__ info, unsigned* __restrict__ num) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < cls) num[t] = (unsigned)cnt[t];
  if (t >= cls * per_class) return;
  const int c = t / per_class, k = t % per_class;
  float v[5] = {0.f, 0.f, 0.f, 0.f, 0.f};
  if (k < cnt[c]) {
    const int i = sel[c * per_class + k];
    for (int j = 0; j < 4; ++j) v[j] = boxes[i * 4 + j];
    v[4] = scores[(int64_t)c * N + i];
  }
  for (int j = 0; j < 5; ++j) info[t * 5 + j] = v[j];
}

}  // namespace

int nms(int B, int C, int N, int max_sel, float iou_thr, float score_thr, int box_dt, const void* boxes, int score_dt, const void* scores, int out_rows,
        int out64, void* out, int* sel, int* cnt, cudaStream_t s) {
  if (B * C <= 0 || out_rows <= 0) return 0;
  if (B * C > 1024 || N > 1500000) return -1;
  if (N > 0 && max_sel > 0) {
    greedy_nms_kernel<0><<<B * C, 256, ((N + 31) / 32) * 4, s>>>(boxes, box_dt, scores, score_dt, C, N, max_sel, iou_thr, score_thr, sel, cnt);
    if (int rc = check_launch()) return rc;
  } else if (cudaMemsetAsync(cnt, 0, sizeof(int) * B * C, s) != cudaSuccess) return -2;
  nms_emit_kernel<<<1, 256, 0, s>>>(sel, cnt, B * C, C, max_sel > 0 ? max_sel : 1, out_rows, out64, out);
  return check_launch();
}

int yolo_postprocess(int cls, const int* S3, const void* const* heads, int dt, const int* nchw3, const unsigned* anchors18, const unsigned* img_w,
                     const unsigned* img_h, float* boxes, float* scores, int* sel, int* cnt, float* info, unsigned* num, cudaStream_t s) {
  int N = 0, first[3];
  for (int i = 0; i < 3; ++i) { first[i] = N; N += S3[i] * S3[i] * 3; }
  const int per_class = N / 169;
  for (int i = 0; i < 3; ++i) {
    const int threads = S3[i] * S3[i] * 3;
    // the coarsest head (stride 32) uses the largest anchors: rows 2, 1, 0 of the anchor table for 13, 26, 52
    yolo_decode_kernel<<<(threads + 127) / 128, 128, 0, s>>>(heads[i], dt, nchw3[i], S3[i], cls, first[i], N, anchors18 + 6 * (2 - i), img_w, img_h, boxes, scores);
    if (int rc = check_launch()) return rc;
  }
  greedy_nms_kernel<1><<<cls, 256, 0, s>>>(boxes, DT_F32, scores, DT_F32, cls, N, per_class, 0.45f, 0.3f, sel, cnt);
  if (int rc = check_launch()) return rc;
  yolo_emit_kernel<<<(cls * per_class + 127) / 128, 128, 0, s>>>(sel, cnt, boxes, scores, cls, N, per_class, info, num);
  return check_launch();
}

}  // namespace b200
