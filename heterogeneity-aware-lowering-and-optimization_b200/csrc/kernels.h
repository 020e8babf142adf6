// Launchers of the CUDA kernels.  Every launcher enqueues on `stream` and returns 0, or a
// negative code (-1 bad argument, -2 CUDA error).  Pointers are device pointers.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

namespace b200 {

// Size of the device status block every tensor-core launch is given: word 0 = code of the wait that expired, word 1 =
// the CTA; a debug build (UMMA_DEBUG_TS) also keeps time stamps and per-site wait counters up to byte 512.
constexpr size_t kStatusBytes = 1024;

// Storage element types of tensors held in HBM.
enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2, DT_S8 = 3, DT_U8 = 4, DT_S32 = 5, DT_S64 = 6 };

enum { ACT_NONE = 0, ACT_RELU = 1, ACT_LEAKY = 2, ACT_CLAMP = 3, ACT_GELU_ERF = 4, ACT_GELU_TANH = 5 };

// Epilogue applied to every accumulator of a convolution / GEMM, in this fixed order and with
// every fp32 operation rounded separately (no fused multiply-add), so that the int8 path
// reproduces a node-by-node fp32 evaluation of the quantised graph bit for bit:
//   t = (float)acc
//   if mul        : t = t * mul[col]
//   if alpha != 1 : t = t * alpha
//   if add1       : t = t + add1[col]          (convolution bias, or beta*C of a Gemm)
//   if add2       : t = t + add2[col]          (the per-channel Add that carries a folded BN)
//   if add_full   : t = t + beta_full * add_full[row, col]     (Gemm with a full-matrix C)
//   if act_first  : t = act(t)
//   if res        : t = t + (res_dt == DT_S8 ? (float)res * res_scale : (float)res)
//   if !act_first : t = act(t)
//   store         : float types round to nearest even; DT_S8 stores sat(rne(t / out_scale)), or
//                   sat(rne(t * out_inv)) when out_multiply is set (requantisation of a value that
//                   comes from int32 accumulators); DT_S32 stores the raw accumulator (int8 inputs only).
struct Epilogue {
  const float* mul = nullptr;
  float alpha = 1.f;
  const float* add1 = nullptr;
  const float* add2 = nullptr;
  const void* add_full = nullptr;  // same storage type as the float mode of the graph
  int add_full_dt = DT_F32;
  float beta_full = 1.f;
  const void* res = nullptr;
  int res_dt = DT_F32;
  float res_scale = 1.f;
  int act = ACT_NONE;
  int act_first = 0;
  float act_a = 0.f, act_b = 0.f;
  int out_dt = DT_F32;
  float out_scale = 1.f;
  float out_inv = 1.f;   // fl(1 / out_scale)
  int out_multiply = 0;
  // int32 accumulators proven (from the filter values) to stay inside (-2^22, 2^22): the tensor-core epilogue may then
  // convert them to fp32 with an integer add and a floating-point subtract instead of a conversion instruction.
  int acc_small = 0;
};

// 2-d convolution geometry.  Data is addressed through element strides so NHWC and NCHW share
// the SIMT kernel: x[n*xs_n + h*xs_h + w*xs_w + c*xs_c], same for y; the filter is
// w[k*ws_k + c*ws_c + r*ws_r + s*ws_s].
struct ConvGeom {
  int N, H, W, C, K, R, S, P, Q, stride_h, stride_w, pad_t, pad_l, groups;
  int64_t xs_n, xs_h, xs_w, xs_c, ys_n, ys_h, ys_w, ys_c, ws_k, ws_c, ws_r, ws_s;
};

// Direct convolution on the CUDA cores; in_dt = DT_F32, DT_F16, DT_BF16 (fp32 accumulate, k
// ascending within taps in (r,s,c) order) or DT_S8 (int32 accumulate); the filter has the same
// type as the input.  Fallback for shapes the tensor-core kernel does not take.
int conv_simt(const ConvGeom& g, int in_dt, const void* x, const void* w, void* y, const Epilogue& ep,
              cudaStream_t stream);

// Batched GEMM on the CUDA cores: C[b] = op(A[b]) op(B[b]); element strides given; epilogue col =
// n index.  A/B same storage type (as conv_simt).  b_batch_stride may be 0 (shared B).
struct GemmGeom {
  int64_t batch, M, N, K;
  int64_t a_row, a_col, a_batch;  // A element (m,k) at m*a_row + k*a_col
  int64_t b_row, b_col, b_batch;  // B element (k,n) at k*b_row + n*b_col
};
int gemm_simt(const GemmGeom& g, int in_dt, const void* A, const void* B, void* C, const Epilogue& ep,
              cudaStream_t stream);

// ---- tensor-core path (kernels_umma.cu) ----
// NHWC implicit-GEMM convolution: x [N,H,W,C], w repacked to [K][R*S*C] (K-major), y [N,P,Q,K].
// A 1x1/stride-1 convolution with H=W=1 is a plain GEMM, which is how Gemm uses it.
struct UmmaConv {
  int N, H, W, C, K, R, S, P, Q, stride_h, stride_w, pad_t, pad_l;
  int in_dt;  // DT_F16, DT_BF16 or DT_S8
  // Optional byte strides of the W and H dimensions of x (0 = dense NHWC).  A W stride smaller than C*elemsize
  // describes overlapping pixels: each position reads C contiguous elements starting x_w_stride bytes after
  // the previous one (the widened-pixel stem without a materialised copy).
  long long x_w_stride = 0, x_h_stride = 0, x_n_stride = 0;
  // Batched GEMM (attention): w holds `w_batches` matrices [K][C] back to back and output rows
  // [b*rows_per_batch, (b+1)*rows_per_batch) use matrix b.  rows_per_batch must be a multiple of 128.
  int w_batches = 0, rows_per_batch = 0;
  // Batched GEMM whose matrices are stored [C][K] (the reduction outermost, e.g. attention probabilities x V): the
  // tensor cores read B "MN-major" straight from that layout, no transposed copy.  Needs K == 64 two-byte columns
  // (one 128-byte swizzle span) and C a multiple of 64.
  int w_n_major = 0;
  // Permuted store (attention head split / merge folded into the GEMM): the output rows are (b, s) [mode 1] or
  // (b, h, s) [mode 2] with s < store_S, the columns are head h x store_D [mode 1] or store_D [mode 2], and element
  // (b, h, s, d) goes to y[b][h][s][d] (mode 1: [B,S,NH*D] -> [B,NH,S,D]) or y[b][s][h][d] (mode 2: [B,NH,S,D] -> [B,S,NH,D]).
  int store_mode = 0, store_S = 0, store_NH = 0, store_D = 0;
  // Row pitch of y in elements when it is wider than K (0 = K): lets an output with rows that are not 16-byte
  // multiples use the TMA-store epilogue; columns K .. y_pitch-1 receive unspecified values.
  int y_pitch = 0;
  // Filter terms: w holds [K][w_terms * R*S][C] and the accumulator is the sum over the terms, each walking the same
  // R x S window of x.  A filter whose values do not fit the operand type is split into terms that do (uint8 weights
  // minus their zero point span [-255, 255]: two or three int8 terms).  0 and 1 both mean a single term.
  int w_terms = 0;
};
// True when the tensor-core kernel can run this problem.
bool umma_conv_supported(const UmmaConv& p);
// Whether a launch with p.store_mode != 0 can store through the permuted tensor map (staged epilogue, one head = one box).
bool umma_store_perm_ok(const UmmaConv& p, const Epilogue& ep, const void* y);
// Opaque prepared launch (tensor maps live in it).  Create once at plan time.
struct UmmaLaunch;
UmmaLaunch* umma_conv_prepare(const UmmaConv& p, const void* x, const void* w, void* y, const Epilogue& ep,
                              int* status_word, int device_sms);
int umma_conv_run(UmmaLaunch* l, cudaStream_t stream);
void umma_conv_destroy(UmmaLaunch* l);

// Fused attention for one shape family: softmax(scale * Q K^T) V over `batch * heads` heads of 128 positions x 64
// channels, q / k / v laid out [batch][heads][128][64] in a two-byte type; the result is stored in the same layout or,
// with merge_heads, as [batch][128][heads][64].  The scores stay in tensor memory.
struct AttnLaunch;
bool attn_supported(int dt, int64_t positions, int64_t channels);
AttnLaunch* attn_prepare(int dt, const void* q, const void* k, const void* v, void* y, int64_t batch, int heads, float scale, bool merge_heads,
                         int* status_word, int device_sms);
int attn_run(AttnLaunch* l, cudaStream_t stream);
void attn_destroy(AttnLaunch* l);

// ---- memory-bound kernels (kernels_simt.cu) ----
struct PoolGeom {
  int N, H, W, C, P, Q, R, S, stride_h, stride_w, pad_t, pad_l;
  int64_t xs_n, xs_h, xs_w, xs_c, ys_n, ys_h, ys_w, ys_c;
};
int pool2d(const PoolGeom& g, int dt, bool is_max, const void* x, void* y, cudaStream_t stream);

enum { UN_RELU = 0, UN_LEAKY, UN_CLAMP, UN_GELU_ERF, UN_GELU_TANH, UN_ERF, UN_SIGMOID, UN_TANH, UN_EXP,
       UN_LOG, UN_SQRT, UN_RSQRT, UN_ABS, UN_NEG, UN_RECIP, UN_ROUND, UN_IDENTITY };
int unary(int op, int dt_in, int dt_out, const void* x, void* y, int64_t n, float a, float b, cudaStream_t stream);

enum { BIN_ADD = 0, BIN_SUB, BIN_MUL, BIN_DIV, BIN_POW, BIN_PRELU };
// Broadcasting binary op; shapes right-aligned to `rank` (<= 8); lhs/rhs strides are 0 on
// broadcast dimensions.  Optional fused activation afterwards (ACT_*).
struct BinaryGeom {
  int rank;
  int64_t oshape[8], lstride[8], rstride[8];
};
int binary(int op, const BinaryGeom& g, int dt_l, int dt_r, int dt_out, const void* l, const void* r, void* y,
           int act, float act_a, cudaStream_t stream);

// y = x * a[c] + b[c] over (outer, C, inner) with fp32 a, b.
int channel_affine(int dt, const void* x, void* y, const float* a, const float* b, int64_t outer, int64_t C,
                   int64_t inner, cudaStream_t stream);

int softmax(int dt, const void* x, void* y, int64_t outer, int64_t dim, int64_t inner, bool log_form,
            cudaStream_t stream);
// Mean over one axis, sum in ascending order then a single division (bit-reproducible).
int reduce_mean_axis(int dt_in, int dt_out, const void* x, void* y, int64_t before, int64_t dim, int64_t after,
                     cudaStream_t stream, float in_scale = 1.f);
// Two adjacent axes (d1, then d2) in one launch with the same arithmetic as two reduce_mean_axis passes; returns 1
// without launching when the shape is not one it serves (7 x 7, 16-byte channel vectors).
int reduce_mean_two_axes(int dt_in, int dt_out, const void* x, void* y, int64_t before, int64_t d1, int64_t d2, int64_t after, cudaStream_t stream,
                         float in_scale = 1.f);  // in_scale: dequantisation scale of an int8 input
int layernorm(int dt, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim,
              float eps, cudaStream_t stream);
// The same, also writing q = sat(rne(y / scale[0])) as int8 for the rounded two-byte result y (what a per-tensor
// odla_Quantize of y gives); dt must be DT_F16 or DT_BF16.
int layernorm_quantize(int dt, const void* x, void* y, const float* gamma, const float* beta, int64_t rows, int64_t dim, float eps, void* q,
                       const float* scale, cudaStream_t stream);

// q = sat(rne(x / scale[a]) + zp[a]); x = (q - zp[a]) * scale[a]; (outer, adim, inner) split.
int quantize(int dt_in, const void* x, void* q, const float* scale, const int* zp, int64_t outer, int64_t adim,
             int64_t inner, bool per_axis, bool is_unsigned, cudaStream_t stream);
// Per-tensor int8 requantisation q = sat(rne(x * inv_scale)).
int requantize(int dt_in, const void* x, void* q, float inv_scale, int64_t n, cudaStream_t stream);
int dequantize(int dt_out, const void* q, void* x, const float* scale, const int* zp, int64_t outer,
               int64_t adim, int64_t inner, bool per_axis, bool is_unsigned, cudaStream_t stream);

// Type conversion between storage types (float<->float, int<->float with saturation to int8).
int convert(int dt_in, int dt_out, const void* x, void* y, int64_t n, cudaStream_t stream);
// y[r][0..K) = x[r][0..K) for rows of pitch Kp (>= K) in x and K in y, with the same type conversion.
int convert_rows(int dt_in, int dt_out, const void* x, void* y, int64_t rows, int64_t K, int64_t Kp, cudaStream_t stream);

// Generic gather-style movement: out[e] = in[src(e)] with src given by per-dimension strides and
// an element offset (covers transpose, slice, concat parts, broadcast).  esz in bytes.
struct MoveGeom {
  int rank;
  int64_t oshape[8], istride[8], ostride[8];
  int64_t in_offset, out_offset;
};
int move(const MoveGeom& g, int esz, const void* x, void* y, cudaStream_t stream);
// out[pixel][0..Cp) = in[pixel][0..C) followed by zeros; Cp*esz must be 32 (one thread writes one pixel as
// two 16-byte stores).  Gives few-channel inputs (an RGB image) rows that TMA can address.
int pad_channels(int esz, const void* x, void* y, int64_t pixels, int C, int Cp, cudaStream_t stream);
// Stride-2 stem helper: y[n][h][q][8*4] gathers, for every output column q, the eight input pixels
// 2q-4 .. 2q+3 (C <= 4 channels each, zero outside the image or beyond C) so that a (R x S) stride-2
// convolution over few channels becomes an (R x 1) convolution over 32 channels with unit column
// stride.  esz is 1 or 2 bytes; one thread writes 16 bytes.
int stem_widen(int esz, const void* x, void* y, int N, int H, int W, int C, int Q, cudaStream_t stream);
// y[n][h][lp + w][cp] = x[n][h][w][0..C) (zeros elsewhere), cp = pixel_bytes / esz channels (pixel_bytes 8 or 16), rows of
// Wp pixels: an image with zero columns on both sides from which overlapping windows of 64 bytes can be read at
// 16-byte steps (every pixel at 16-byte pixels, every second one at 8-byte pixels).
int stem_pad(int esz, const void* x, void* y, int N, int H, int W, int C, int pixel_bytes, int lp, int Wp, cudaStream_t stream);
int resize_nearest(int esz, const void* x, void* y, int N, int H, int W, int C, int P, int Q, bool nhwc,
                   cudaStream_t stream);
// out[o, k, :] = in[o, idx[k], :]; idx int32 or int64.
int gather(int esz, const void* x, const void* idx, int idx_dt, void* y, int64_t outer, int64_t axis_dim,
           int64_t n_idx, int64_t inner, cudaStream_t stream);

// Running minimum / maximum of a dense float tensor (fp32 / fp16 / bf16) whose last axis has `channels` entries:
// stats[0], stats[1] = whole tensor, stats[2 + c], stats[2 + channels + c] = channel c, all as order-preserving
// unsigned keys (range_key_init / range_key_decode) updated with atomicMin / atomicMax, so calls accumulate.
int range_minmax(int dt, const void* x, int64_t count, int64_t channels, unsigned* stats, cudaStream_t stream);
int range_stats_reset(unsigned* stats, int64_t channels, cudaStream_t stream);
inline float range_key_decode(unsigned k) { unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k; float f; memcpy(&f, &b, 4); return f; }

// Greedy non-maximum suppression (odla_NMS): boxes [B, N, 4] (y1, x1, y2, x2), scores [B, C, N]; `out` gets out_rows rows
// (batch, class, box) as int32 or int64, -1 beyond the selected ones.  sel [B*C*max_sel] and cnt [B*C] are scratch.
int nms(int B, int C, int N, int max_sel, float iou_thr, float score_thr, int box_dt, const void* boxes, int score_dt, const void* scores, int out_rows,
        int out64, void* out, int* sel, int* cnt, cudaStream_t stream);
// YOLOv3 post-processing (odla_PostProcess): three heads [1, 3*(cls+5), S, S] (nchw) or [1, S, S, 3*(cls+5)] with
// S = 13, 26, 52 -> info [cls, N/169, 5] (y_min, x_min, y_max, x_max, score) and num [cls]; boxes [N, 4], scores [cls, N],
// sel [cls * N/169] and cnt [cls] are scratch, anchors18 the 3 x 6 anchor table in device memory.
int yolo_postprocess(int cls, const int* S3, const void* const* heads, int dt, const int* nchw3, const unsigned* anchors18, const unsigned* img_w,
                     const unsigned* img_h, float* boxes, float* scores, int* sel, int* cnt, float* info, unsigned* num, cudaStream_t stream);

}  // namespace b200
