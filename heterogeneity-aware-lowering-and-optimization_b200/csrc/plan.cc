// Planning and execution.
//
// The recorded graph is turned, once per (GPU, shard batch), into a flat launch list:
//   1. analysis   - use counts, which values carry the batch, which chains fold into a
//                   convolution / GEMM epilogue (per-channel Add that carries a folded BN, residual
//                   Add, Relu/LeakyRelu/Clamp/Gelu, Quantize) and which Dequantize nodes are
//                   absorbed by their consumers (int8 operands, int8 residuals);
//   2. placement  - liveness-based offsets inside one arena per plan;
//   3. emission   - constants are converted / repacked on the host and uploaded once, tensor maps
//                   are encoded, and each entry becomes a closure that enqueues its kernel.
// odla_ExecuteComputation then shards dim 0 of every argument over the replicas (one per GPU,
// weights replicated), and per GPU enqueues host-to-device copies, the launch list (replayed as a
// CUDA graph when possible) and the copies of the output shards, on that GPU's own stream.  No
// collective is involved: every op of a shardable graph is independent across the batch.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <set>
#include <thread>

#include "common.h"

namespace b200 {

int visible_devices() {
  static int n = [] {
    int c = 0;
    if (cudaGetDeviceCount(&c) != cudaSuccess) { cudaGetLastError(); return 0; }
    return c;
  }();
  return n;
}

Plan::~Plan() {
  cudaSetDevice(device);
  if (graph) cudaGraphExecDestroy(graph);
  for (auto& l : launches) l.fn = nullptr;
  for (auto* u : umma) umma_conv_destroy(u);
  for (auto* a : attn) attn_destroy(a);
  for (void* p : extra_allocs) cudaFree(p);
  if (arena) cudaFree(arena);
  if (status) cudaFree(status);
}

namespace {

typedef const _odla_value* V;

// ---- host-side numeric helpers (constants are converted before upload) ----
uint16_t f2h(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  uint32_t s = (u >> 16) & 0x8000; int32_t e = (int32_t)((u >> 23) & 0xff) - 127 + 15; uint32_t m = u & 0x7fffff;
  if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(s | 0x7c00 | (m ? 0x200 : 0));
  if (e >= 31) return (uint16_t)(s | 0x7c00);
  if (e <= 0) {
    if (e < -10) return (uint16_t)s;
    m |= 0x800000; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return (uint16_t)(s | r);
  }
  uint32_t r = ((uint32_t)e << 10) | (m >> 13), rem = m & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) ++r;
  return (uint16_t)(s | r);
}
float h2f(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff, u;
  if (e == 0) {
    if (m == 0) u = s << 31;
    else { int k = 0; while (!(m & 0x400)) { m <<= 1; ++k; } u = (s << 31) | ((uint32_t)(127 - 15 - k + 1) << 23) | ((m & 0x3ff) << 13); }
  } else if (e == 31) u = (s << 31) | 0x7f800000u | (m << 13);
  else u = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}
uint16_t f2bf(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffff) > 0x7f800000) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fff + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}
float bf2f(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }

int api_dt(odla_element_type t) {  // storage type that holds an API element type verbatim
  switch (t) {
    case ODLA_FLOAT32: return DT_F32;
    case ODLA_FLOAT16: return DT_F16;
    case ODLA_BFLOAT16: return DT_BF16;
    case ODLA_INT8: case ODLA_QINT8: return DT_S8;
    case ODLA_UINT8: case ODLA_QUINT8: case ODLA_BOOL: return DT_U8;
    case ODLA_INT32: case ODLA_QINT32: case ODLA_UINT32: return DT_S32;
    case ODLA_INT64: case ODLA_UINT64: return DT_S64;
    default: return -1;
  }
}
// Reads constant `v` (any supported element type) as fp32.
std::vector<float> const_as_f32(V v) {
  int64_t n = numel(v->type.shape);
  std::vector<float> r((size_t)n);
  switch (api_dt(v->type.element_type)) {
    case DT_F32: memcpy(r.data(), v->host, sizeof(float) * (size_t)n); break;
    case DT_F16: for (int64_t i = 0; i < n; ++i) r[i] = h2f(((const uint16_t*)v->host)[i]); break;
    case DT_BF16: for (int64_t i = 0; i < n; ++i) r[i] = bf2f(((const uint16_t*)v->host)[i]); break;
    case DT_S8: for (int64_t i = 0; i < n; ++i) r[i] = ((const int8_t*)v->host)[i]; break;
    case DT_U8: for (int64_t i = 0; i < n; ++i) r[i] = ((const uint8_t*)v->host)[i]; break;
    case DT_S32: for (int64_t i = 0; i < n; ++i) r[i] = (float)((const int32_t*)v->host)[i]; break;
    case DT_S64: for (int64_t i = 0; i < n; ++i) r[i] = (float)((const int64_t*)v->host)[i]; break;
    default: break;
  }
  return r;
}
std::vector<uint8_t> f32_to_storage(const std::vector<float>& f, int dt) {
  std::vector<uint8_t> out(f.size() * (size_t)storage_size(dt));
  switch (dt) {
    case DT_F32: memcpy(out.data(), f.data(), out.size()); break;
    case DT_F16: for (size_t i = 0; i < f.size(); ++i) ((uint16_t*)out.data())[i] = f2h(f[i]); break;
    case DT_BF16: for (size_t i = 0; i < f.size(); ++i) ((uint16_t*)out.data())[i] = f2bf(f[i]); break;
    case DT_S8: for (size_t i = 0; i < f.size(); ++i) ((int8_t*)out.data())[i] = (int8_t)std::max(-128.f, std::min(127.f, std::nearbyint(f[i]))); break;
    case DT_U8: for (size_t i = 0; i < f.size(); ++i) ((uint8_t*)out.data())[i] = (uint8_t)std::max(0.f, std::min(255.f, std::nearbyint(f[i]))); break;
    case DT_S32: for (size_t i = 0; i < f.size(); ++i) ((int32_t*)out.data())[i] = (int32_t)f[i]; break;
    case DT_S64: for (size_t i = 0; i < f.size(); ++i) ((int64_t*)out.data())[i] = (int64_t)f[i]; break;
  }
  return out;
}

// A fused convolution / GEMM: root node plus the chain folded into its epilogue.
struct Fused {
  V root = nullptr, out = nullptr;
  bool int8 = false;
  V x = nullptr;            // data operand actually read (int8 source when int8)
  V x_scale = nullptr;      // per-tensor activation scale (int8)
  V w = nullptr;            // constant weights actually read (int8 source when int8)
  V w_scale = nullptr;      // per-tensor or per-output-channel weight scale (int8)
  V w_zp = nullptr;         // per-tensor zero point of asymmetric uint8 weights (the filter is W_u - zp)
  V add_const = nullptr;    // per-channel Add operand
  V res = nullptr;          // residual tensor actually read
  V res_scale = nullptr;    // Dequantize scale when the residual is int8
  int act = ACT_NONE; float act_a = 0, act_b = 0; bool act_first = false;
  V quant_scale = nullptr;  // absorbed Quantize
  float scalar_mul = 1.f;   // a following Mul by a scalar constant, folded into alpha
  // attention head split ([B*S, NH*D] -> Reshape -> Transpose(0,2,1,3) = [B,NH,S,D], mode 1) or merge ([B,NH,S,D] ->
  // Transpose(0,2,1,3) = [B,S,NH,D], mode 2) folded into the Gemm's store
  int perm_mode = 0;
  int64_t perm_S = 0, perm_NH = 0, perm_D = 0;
  bool has_scalar_mul = false;
};

struct Item {               // one launch-list entry before emission
  V out = nullptr;          // value it materialises
  std::vector<V> reads;     // materialised values it reads (after alias resolution)
  const Fused* fused = nullptr;
  V extra_out = nullptr;    // a second value the same launch writes (the int8 copy a LayerNorm makes for a following Quantize)
  // fused attention: this item is the context product; the scores product and the soft-max in front of it have no
  // items of their own, their operands are read here
  V attn_q = nullptr, attn_k = nullptr;
  float attn_scale = 1.f;
};

class Builder {
 public:
  Builder(_odla_computation* c, Plan* p, int64_t full_batch, int64_t shard, int64_t shard_start)
      : c_(c), p_(p), B_(full_batch), b_(shard), start_(shard_start) {}
  odla_status run();

 private:
  _odla_computation* c_;
  Plan* p_;
  int64_t B_, b_, start_;
  std::map<V, int> users_;
  std::map<V, std::vector<V>> consumers_;
  std::map<V, bool> carries_batch_;
  std::map<V, bool> from_acc_;         // computed from int32 accumulators through element-wise ops only
  std::map<V, V> fused_into_;          // node -> root of the chain that swallowed it
  std::set<V> merged_;                 // Quantize nodes written by their producer's launch (see Item::extra_out)
  std::map<V, std::unique_ptr<Fused>> fused_;  // by root
  std::map<V, int> dq_unabsorbed_;     // Dequantize node -> number of consumers that need it in memory
  std::map<V, V> alias_;               // reshape output -> source
  std::map<V, int> dt_;                // storage type of materialised values
  std::map<V, int64_t> pitch_;          // internal row pitch (elements) of an output whose rows TMA could not store otherwise
  std::vector<Item> items_;
  std::map<std::pair<V, int>, void*> const_cache_;
  std::string err_;
  odla_status err_status_ = ODLA_SUCCESS;

  odla_status fail(odla_status s, const std::string& m) { if (err_.empty()) { err_ = m; err_status_ = s; } B2_ERR("%s", m.c_str()); return s; }
  int FS() const { return c_->float_mode; }
  V resolve(V v) const { auto it = alias_.find(v); while (it != alias_.end()) { v = it->second; it = alias_.find(v); } return v; }
  // shape of `v` inside this shard
  odla_value_shape shape(V v) const {
    odla_value_shape s = v->type.shape;
    auto it = carries_batch_.find(v);
    if (it != carries_batch_.end() && it->second && B_ != b_ && s.size > 0) s.dims[0] = s.dims[0] / B_ * b_;
    return s;
  }
  int64_t count(V v) const { return numel(shape(v)); }
  int storage_of(V v) const {
    if (is_float_type(v->type.element_type)) return FS();
    return api_dt(v->type.element_type);
  }
  void* dev_ptr(V v) const {
    v = resolve(v);
    auto it = p_->slots.find(v);
    if (it == p_->slots.end() || it->second.offset < 0) return nullptr;
    return p_->arena + it->second.offset;
  }
  void* upload(const void* host, size_t bytes) {
    void* d = nullptr;
    if (inject_fault("alloc") || cudaMalloc(&d, bytes ? bytes : 16) != cudaSuccess) { fail(ODLA_MEM_ERROR, "constant allocation failed"); return nullptr; }
    p_->extra_allocs.push_back(d);
    if (bytes && cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) { fail(ODLA_FAILURE, "constant upload failed"); return nullptr; }
    p_->const_bytes += (int64_t)bytes;
    return d;
  }
  void* const_dev(V v, int dt) {  // constant converted to storage type dt, uploaded once
    auto key = std::make_pair(v, dt);
    auto it = const_cache_.find(key);
    if (it != const_cache_.end()) return it->second;
    void* d;
    if (api_dt(v->type.element_type) == dt) d = upload(v->host, (size_t)(numel(v->type.shape) * storage_size(dt)));
    else { auto bytes = prepared(v, "dt" + std::to_string(dt), [&] { return f32_to_storage(const_as_f32(v), dt); }); d = upload(bytes->data(), bytes->size()); }
    const_cache_[key] = d;
    return d;
  }
  float* upload_f32(const std::vector<float>& f) { return (float*)upload(f.data(), f.size() * sizeof(float)); }
  // The bytes of constant `v` in form `form`: taken from the computation's prepared set, or produced by `make` and
  // added to it (other replicas' plans and a stored executable reuse them).
  std::shared_ptr<std::vector<uint8_t>> prepared(V v, const std::string& form, const std::function<std::vector<uint8_t>()>& make) {
    const std::string key = std::to_string(v->index) + "|" + form;
    {
      std::lock_guard<std::mutex> lock(c_->prepared_mutex);
      auto it = c_->prepared.find(key);
      if (it != c_->prepared.end()) { ++c_->prepared_hits; return it->second; }
    }
    auto blob = std::make_shared<std::vector<uint8_t>>(make());
    std::lock_guard<std::mutex> lock(c_->prepared_mutex);
    ++c_->prepared_misses;
    c_->prepared[key] = blob;
    return blob;
  }

  odla_status analyse();
  void try_fuse(V root);
  odla_status place();
  odla_status emit();
  void try_attention(Item& it, const Fused& f);
  odla_status emit_fused(const Item& it);
  odla_status emit_plain(const Item& it);
  void add_launch(const char* op, V out, double flops, double bytes, std::function<int(cudaStream_t)> fn) {
    Launch l; l.op = op; l.name = out->name; l.flops = flops; l.bytes = bytes; l.fn = std::move(fn);
    l.out_v = out;
    if (dt_.count(out) && !pitch_.count(out) && p_->slots.count(out)) {
      const odla_value_shape sh = shape(out);
      l.out_ptr = dev_ptr(out); l.out_dt = dt_[out]; l.out_count = count(out); l.out_channels = sh.size ? sh.dims[sh.size - 1] : 1;
    }
    p_->launches.push_back(std::move(l));
  }
  double tensor_bytes(V v) const { return (double)count(v) * storage_size(dt_.count(resolve(v)) ? dt_.at(resolve(v)) : storage_of(v)); }
};

bool is_per_tensor_dq(V v) {
  return v && v->kind == OP_DEQUANTIZE && !v->in[2] && numel(v->in[1]->type.shape) == 1 &&
         (v->in[0]->type.element_type == ODLA_INT8);
}

odla_status Builder::analyse() {
  // users / consumers
  for (auto& n : c_->nodes)
    for (auto i : n->in)
      if (i) { users_[i]++; consumers_[i].push_back(n.get()); }
  // batch propagation and shardability
  for (auto& n : c_->nodes) {
    V v = n.get();
    bool cb = v->kind == OP_ARG;
    for (auto i : v->in) if (i && carries_batch_[i]) cb = true;
    carries_batch_[v] = cb;
  }
  if (B_ != b_) {
    for (auto& n : c_->nodes) {
      V v = n.get();
      if (!carries_batch_[v]) continue;
      if (v->type.shape.size == 0 || v->type.shape.dims[0] % B_ != 0) return fail(ODLA_INTERNAL_LOGIC_ERR, "value '" + v->name + "' does not scale with the batch");
    }
  }
  // fusion roots
  for (auto& n : c_->nodes)
    if (n->kind == OP_CONV || n->kind == OP_GEMM) try_fuse(n.get());
  // Values that come from int32 accumulators: an int8-path Conv/Gemm result and any element-wise
  // (unary / binary / reshape) function of one.  Quantising such a value is a requantisation and
  // multiplies by fl(1/s); every other Quantize divides like the reference.
  for (auto& n : c_->nodes) {
    V v = n.get();
    bool t = false;
    if ((v->kind == OP_CONV || v->kind == OP_GEMM) && fused_.count(v)) t = fused_[v]->int8;
    else if (v->kind == OP_UNARY || v->kind == OP_BINARY || v->kind == OP_RESHAPE)
      for (auto i : v->in) if (i && from_acc_[i]) t = true;
    from_acc_[v] = t;
  }
  // which Dequantize nodes still need to exist in memory
  for (auto& n : c_->nodes) {
    V v = n.get();
    if (v->kind != OP_DEQUANTIZE) continue;
    int need = v->is_output ? 1 : 0;
    for (V cons : consumers_[v]) {
      bool absorbed = false;
      auto fi = fused_into_.find(cons);
      V root = cons->kind == OP_CONV || cons->kind == OP_GEMM ? cons : (fi != fused_into_.end() ? fi->second : nullptr);
      if (root && fused_.count(root)) {
        const Fused& f = *fused_[root];
        if (f.int8 && (root->in[0] == v || root->in[1] == v) && cons == root) absorbed = true;
        if (f.res_scale && cons != root && (cons->in[0] == v || cons->in[1] == v) && f.res == v->in[0]) absorbed = true;
      }
      // ReduceMean dequantises int8 terms as it reads them
      if (cons->kind == OP_REDUCE_MEAN && cons->in[0] == v && is_per_tensor_dq(v) && !getenv("ODLA_B200_NO_DQ_REDUCE")) absorbed = true;
      if (!absorbed) ++need;
    }
    dq_unabsorbed_[v] = need;
  }
  // launch items in topological order
  for (auto& n : c_->nodes) {
    V v = n.get();
    if (v->kind == OP_CONST) continue;
    if (v->kind == OP_ARG) {
      dt_[v] = storage_of(v);
      // A float argument that only feeds Quantize nodes is quantised straight from the caller's element type
      // (no conversion pass over the input; the values are the same numbers in either type).
      bool only_q = is_float_type(v->type.element_type) && !consumers_[v].empty() && !v->is_output;
      for (V cons : consumers_[v]) if (cons->kind != OP_QUANTIZE || cons->in[0] != v) only_q = false;
      if (only_q && api_dt(v->type.element_type) >= 0) dt_[v] = api_dt(v->type.element_type);
      continue;
    }
    if (v->kind == OP_RESHAPE) { alias_[v] = v->in[0]; continue; }
    if (merged_.count(v)) continue;
    auto fi = fused_into_.find(v);
    if (fi != fused_into_.end() && fused_[fi->second]->out != v) continue;  // swallowed, not the chain end
    if (v->kind == OP_DEQUANTIZE && dq_unabsorbed_[v] == 0) continue;
    Item it;
    it.out = v;
    V root = (v->kind == OP_CONV || v->kind == OP_GEMM) ? v : (fi != fused_into_.end() ? fi->second : nullptr);
    if (root && fused_.count(root)) {
      const Fused* f = fused_[root].get();
      it.fused = f;
      it.reads.push_back(f->x);
      if (f->w->kind != OP_CONST) it.reads.push_back(f->w);
      if (f->res) it.reads.push_back(f->res);
      if (root->kind == OP_GEMM && root->in[2] && root->in[2]->kind != OP_CONST) it.reads.push_back(root->in[2]);
      dt_[v] = f->quant_scale ? DT_S8 : FS();
      // softmax(scale * Q K^T) V with heads of 128 positions x 64 channels: one launch, the scores stay on chip
      if (root->kind == OP_GEMM) try_attention(it, *f);
    } else {
      for (auto i : v->in) {
        if (!i || i->kind == OP_CONST) continue;
        const bool through_dq = v->kind == OP_REDUCE_MEAN && i == v->in[0] && i->kind == OP_DEQUANTIZE && dq_unabsorbed_[i] == 0;
        it.reads.push_back(through_dq ? i->in[0] : i);
      }
      dt_[v] = storage_of(v);
      // LayerNorm over a two-byte tensor whose result is also wanted as int8 (the input of an int8 Gemm; the float
      // copy feeds the residual): the row kernel writes both, the Quantize launch and its pass over the tensor go.
      if (v->kind == OP_LAYERNORM && (dt_[v] == DT_F16 || dt_[v] == DT_BF16) && !getenv("ODLA_B200_NO_LN_QUANT")) {
        const auto& sh = v->type.shape;
        int64_t dim = 1;
        for (int i = sh.size - (int)v->ia[0]; i < sh.size; ++i) if (i >= 0) dim *= sh.dims[i];
        for (V cons : consumers_[v]) {
          if (cons->kind != OP_QUANTIZE || cons->in[0] != v || cons->in[2] || !cons->in[1] || cons->in[1]->kind != OP_CONST) continue;
          if (numel(cons->in[1]->type.shape) != 1 || cons->type.element_type != ODLA_INT8 || fused_into_.count(cons)) continue;
          if (dim % 8 != 0 || dim > 2048 || dim < 8) continue;
          it.extra_out = cons;
          merged_.insert(cons);
          dt_[cons] = DT_S8;
          break;
        }
      }
    }
    items_.push_back(std::move(it));
  }
  // reshape of a constant has no producer item: treat as constant view
  return ODLA_SUCCESS;
}

void Builder::try_fuse(V root) {
  auto f = std::make_unique<Fused>();
  f->root = root;
  f->x = root->in[0];
  f->w = root->in[1];
  int64_t K;  // output channels / columns
  if (root->kind == OP_CONV) K = root->ia[0] ? root->type.shape.dims[3] : root->type.shape.dims[1];
  else K = root->type.shape.dims[root->type.shape.size - 1];
  bool channel_last = root->kind == OP_GEMM || root->ia[0];
  // int8 operands
  V xin = root->in[0], win = root->in[1];
  const bool w_s8 = win && win->kind == OP_DEQUANTIZE && !win->in[2] && win->in[0]->kind == OP_CONST && win->in[0]->type.element_type == ODLA_INT8 &&
                    (numel(win->in[1]->type.shape) == 1 || numel(win->in[1]->type.shape) == K);
  // asymmetric uint8 weights as -quantize-weights=quint8 leaves them (lib/quantizer/weights_quantizer.cc:84-182): one
  // scale and one zero point per tensor
  const bool w_u8 = win && win->kind == OP_DEQUANTIZE && win->in[2] && win->in[2]->kind == OP_CONST && numel(win->in[2]->type.shape) == 1 &&
                    win->in[0]->kind == OP_CONST && (win->in[0]->type.element_type == ODLA_UINT8 || win->in[0]->type.element_type == ODLA_QUINT8) &&
                    win->in[1]->kind == OP_CONST && numel(win->in[1]->type.shape) == 1;
  if (is_per_tensor_dq(xin) && (w_s8 || w_u8) && channel_last && (root->kind == OP_CONV ? root->ia[1] == 1 : root->type.shape.size == 2)) {
    f->int8 = true;
    f->x = xin->in[0];
    f->x_scale = xin->in[1];
    f->w = win->in[0];
    f->w_scale = win->in[1];
    if (w_u8) f->w_zp = win->in[2];
  }
  V cur = root;
  fused_into_[root] = root;
  while (channel_last) {
    if (cur->is_output || users_[cur] != 1) break;
    V nxt = consumers_[cur][0];
    if (fused_into_.count(nxt)) break;  // already folded into another root's epilogue
    if (nxt->kind == OP_BINARY && nxt->ia[0] == BIN_ADD) {
      V other = nxt->in[0] == cur ? nxt->in[1] : nxt->in[0];
      if (other == cur) break;
      const auto& os = other->type.shape;
      bool per_channel = other->kind == OP_CONST && numel(os) == K && os.dims[os.size - 1] == K;
      bool same_shape = numel(other->type.shape) == numel(cur->type.shape) && other->kind != OP_CONST;
      if (per_channel && !f->add_const && !f->res && f->act == ACT_NONE) f->add_const = other;
      // the residual must exist before this root launches: when two convolutions feed one Add
      // (projection shortcut), the later one takes the Add and reads the earlier one's result
      else if (same_shape && !f->res && (is_per_tensor_dq(other) ? other->in[0] : other)->index < root->index) {
        if (is_per_tensor_dq(other)) { f->res = other->in[0]; f->res_scale = other->in[1]; }
        else f->res = other;
        if (f->act != ACT_NONE) f->act_first = true;
      } else break;
    } else if (nxt->kind == OP_BINARY && nxt->ia[0] == BIN_MUL && !f->int8 && !f->add_const && !f->res && f->act == ACT_NONE && !f->has_scalar_mul &&
               !root->in[2] && (nxt->in[0] == cur ? nxt->in[1] : nxt->in[0])->kind == OP_CONST &&
               numel((nxt->in[0] == cur ? nxt->in[1] : nxt->in[0])->type.shape) == 1 && (nxt->in[0] == cur ? nxt->in[1] : nxt->in[0]) != cur) {
      // Gemm / Conv without bias followed by a multiplication by a scalar constant (the 1/sqrt(d) of attention)
      f->scalar_mul = const_as_f32(nxt->in[0] == cur ? nxt->in[1] : nxt->in[0])[0];
      f->has_scalar_mul = true;
    } else if (nxt->kind == OP_UNARY && f->act == ACT_NONE &&
               (nxt->ia[0] == UN_RELU || nxt->ia[0] == UN_LEAKY || nxt->ia[0] == UN_CLAMP || nxt->ia[0] == UN_GELU_ERF || nxt->ia[0] == UN_GELU_TANH)) {
      f->act = nxt->ia[0] == UN_RELU ? ACT_RELU : nxt->ia[0] == UN_LEAKY ? ACT_LEAKY : nxt->ia[0] == UN_CLAMP ? ACT_CLAMP
               : nxt->ia[0] == UN_GELU_ERF ? ACT_GELU_ERF : ACT_GELU_TANH;
      f->act_a = nxt->fa[0];
      f->act_b = nxt->fa[1];
    } else if (nxt->kind == OP_QUANTIZE && !nxt->in[2] && numel(nxt->in[1]->type.shape) == 1 && nxt->type.element_type == ODLA_INT8) {
      f->quant_scale = nxt->in[1];
      fused_into_[nxt] = root;
      cur = nxt;
      break;
    } else break;
    fused_into_[nxt] = root;
    cur = nxt;
  }
  // A Gemm whose only consumer is the head split / merge of attention stores straight into the permuted tensor.
  if (root->kind == OP_GEMM && channel_last && !f->quant_scale && !f->res && !cur->is_output && users_[cur] == 1 && !getenv("ODLA_B200_NO_PERM_STORE")) {
    auto is_head_swap = [](V t) {
      return t->kind == OP_TRANSPOSE && t->ia.size() == 4 && t->ia[0] == 0 && t->ia[1] == 2 && t->ia[2] == 1 && t->ia[3] == 3;
    };
    V nxt = consumers_[cur][0];
    const auto& cs = cur->type.shape;
    if (nxt->kind == OP_RESHAPE && cs.size == 2 && nxt->type.shape.size == 4 && !nxt->is_output && users_[nxt] == 1 && !fused_into_.count(nxt)) {
      V t = consumers_[nxt][0];
      const auto& rs = nxt->type.shape;  // [B, S, NH, D]
      if (is_head_swap(t) && !fused_into_.count(t) && rs.dims[0] * rs.dims[1] == cs.dims[0] && rs.dims[2] * rs.dims[3] == cs.dims[1]) {
        f->perm_mode = 1; f->perm_S = rs.dims[1]; f->perm_NH = rs.dims[2]; f->perm_D = rs.dims[3];
        fused_into_[nxt] = root;
        fused_into_[t] = root;
        cur = t;
      }
    } else if (is_head_swap(nxt) && cs.size == 4 && !fused_into_.count(nxt)) {  // [B, NH, S, D]
      f->perm_mode = 2; f->perm_NH = cs.dims[1]; f->perm_S = cs.dims[2]; f->perm_D = cs.dims[3];
      fused_into_[nxt] = root;
      cur = nxt;
    }
  }
  f->out = cur;
  fused_[root] = std::move(f);
}

// First-fit free-list allocator over byte offsets (1 KiB granularity).
struct Arena {
  std::vector<std::pair<int64_t, int64_t>> free_;  // (offset, size), sorted by offset
  int64_t top = 0;
  static int64_t round(int64_t b) { return (b + 1023) / 1024 * 1024; }
  int64_t alloc(int64_t bytes) {
    bytes = round(bytes ? bytes : 1);
    int best = -1;
    for (size_t i = 0; i < free_.size(); ++i)
      if (free_[i].second >= bytes && (best < 0 || free_[i].second < free_[best].second)) best = (int)i;
    if (best >= 0) {
      int64_t off = free_[best].first;
      if (free_[best].second == bytes) free_.erase(free_.begin() + best);
      else { free_[best].first += bytes; free_[best].second -= bytes; }
      return off;
    }
    // grow: merge with a trailing free block if it touches the top
    if (!free_.empty() && free_.back().first + free_.back().second == top) {
      int64_t off = free_.back().first;
      top = off + bytes;
      free_.pop_back();
      return off;
    }
    int64_t off = top;
    top += bytes;
    return off;
  }
  void release(int64_t off, int64_t bytes) {
    bytes = round(bytes ? bytes : 1);
    auto it = std::lower_bound(free_.begin(), free_.end(), std::make_pair(off, (int64_t)0));
    it = free_.insert(it, {off, bytes});
    if (it + 1 != free_.end() && it->first + it->second == (it + 1)->first) { it->second += (it + 1)->second; free_.erase(it + 1); }
    if (it != free_.begin() && (it - 1)->first + (it - 1)->second == it->first) { (it - 1)->second += it->second; free_.erase(it); }
  }
};


odla_status Builder::place() {
  Arena arena;
  // last use of every materialised value (index into items_; outputs and arguments live to the end)
  std::map<V, int> last;
  for (size_t i = 0; i < items_.size(); ++i)
    for (V r : items_[i].reads) last[resolve(r)] = (int)i;
  // A channels-last convolution that ends the graph with an odd channel count (YOLO's 255-channel heads) has rows
  // that are not 16-byte multiples, which would push it off the TMA-store epilogue.  When only the output conversion
  // reads it, its internal rows are padded to the next multiple of 8 channels and the conversion drops the padding.
  for (auto& it : items_) {
    V v = it.out;
    if (!it.fused || it.fused->root->kind != OP_CONV || !it.fused->root->ia[0] || !v->is_output || users_[v] != 0 || alias_.count(v)) continue;
    if (!(dt_[v] == DT_F16 || dt_[v] == DT_BF16) || api_dt(v->type.element_type) == dt_[v] || getenv("ODLA_B200_NO_PITCH")) continue;
    // only where the tensor-core kernel with the staged epilogue is certain to run
    if (getenv("ODLA_B200_NO_UMMA") || getenv("ODLA_B200_DIRECT_EPILOGUE") || it.fused->root->ia[1] != 1 || it.fused->res) continue;
    {
      const auto& xs = it.fused->root->in[0]->type.shape;
      const int64_t cin_bytes = xs.dims[xs.size - 1] * 2;
      if (cin_bytes % 16 != 0 || cin_bytes < 32) continue;
    }
    const auto& sh = v->type.shape;
    const int64_t K = sh.dims[sh.size - 1];
    bool aliased = false;
    for (auto& kv : alias_) if (resolve(kv.first) == v) aliased = true;
    if ((K * 2) % 16 != 0 && !aliased) pitch_[v] = (K + 7) / 8 * 8;
  }
  auto bytes_of = [&](V v) {
    auto pi = pitch_.find(v);
    if (pi != pitch_.end()) { const auto& sh = v->type.shape; return count(v) / sh.dims[sh.size - 1] * pi->second * storage_size(dt_[v]); }
    return count(v) * storage_size(dt_[v]);
  };
  for (V a : c_->args) {
    Slot s; s.dt = dt_[a]; s.bytes = bytes_of(a); s.offset = arena.alloc(s.bytes);
    p_->slots[a] = s;
  }
  std::set<V> outputs;
  for (V o : c_->outs) outputs.insert(resolve(o));
  for (size_t i = 0; i < items_.size(); ++i) {
    V v = items_[i].out;
    Slot s; s.dt = dt_[v]; s.bytes = bytes_of(v); s.offset = arena.alloc(s.bytes);
    p_->slots[v] = s;
    if (V e = items_[i].extra_out) {   // allocated while this item's inputs are still held: the launch writes it too
      Slot se; se.dt = dt_[e]; se.bytes = bytes_of(e); se.offset = arena.alloc(se.bytes);
      p_->slots[e] = se;
      if (!last.count(e) && !outputs.count(e)) arena.release(se.offset, se.bytes);
    }
    for (V r : items_[i].reads) {
      V rr = resolve(r);
      if (rr->kind == OP_ARG || rr->kind == OP_CONST || outputs.count(rr)) continue;
      auto li = last.find(rr);
      if (li != last.end() && li->second == (int)i) {
        auto& sl = p_->slots[rr];
        if (sl.offset >= 0) arena.release(sl.offset, sl.bytes);
        li->second = -1;  // released once even if read twice by this item
      }
    }
    if (!last.count(v) && !outputs.count(v)) arena.release(s.offset, s.bytes);  // never read: reuse at once
  }
  // staging for arguments / outputs whose API element type differs from the storage type
  for (V a : c_->args) {
    Plan::Io io; io.v = a; io.slot = p_->slots[a].offset;
    io.api_bytes = count(a) * elem_size(a->type.element_type);
    io.per_shard = true;
    io.user_offset = B_ ? numel(a->type.shape) / B_ * start_ * elem_size(a->type.element_type) : 0;
    io.stage = api_dt(a->type.element_type) == dt_[a] ? io.slot : arena.alloc(io.api_bytes);
    p_->inputs.push_back(io);
  }
  for (V o : c_->outs) {
    Plan::Io io; io.v = o;
    V r = resolve(o);
    io.api_bytes = count(o) * elem_size(o->type.element_type);
    io.per_shard = carries_batch_[o];
    io.user_offset = io.per_shard && B_ ? numel(o->type.shape) / B_ * start_ * elem_size(o->type.element_type) : 0;
    if (r->kind == OP_CONST) io.const_host = r->host;
    else {
      io.slot = p_->slots[r].offset;
      io.stage = api_dt(o->type.element_type) == dt_[r] ? io.slot : arena.alloc(io.api_bytes);
    }
    p_->outputs.push_back(io);
  }
  p_->arena_bytes = arena.top;
  if (inject_fault("alloc") || cudaMalloc((void**)&p_->arena, (size_t)std::max<int64_t>(p_->arena_bytes, 1024)) != cudaSuccess)
    return fail(ODLA_MEM_ERROR, "arena allocation failed");
  if (cudaMalloc((void**)&p_->status, kStatusBytes) != cudaSuccess) return fail(ODLA_MEM_ERROR, "status word allocation failed");
  cudaMemset(p_->status, 0, kStatusBytes);
  return ODLA_SUCCESS;
}

// Recognises Gemm(Softmax(Mul(Gemm(q, k^T), scale), last axis), v) whose intermediates have no other reader, in the one
// shape family the fused kernel serves; on success the items of the scores product and of the soft-max are taken out
// of the launch list and `it` (the context product) reads q, k and v itself.
void Builder::try_attention(Item& it, const Fused& f) {
  if (getenv("ODLA_B200_NO_ATTENTION") || getenv("ODLA_B200_NO_UMMA")) return;
  const int fs = FS();
  if (fs != DT_F16 && fs != DT_BF16) return;
  V root = f.root;
  auto plain = [](const Fused& g) { return !g.int8 && !g.add_const && !g.res && g.act == ACT_NONE && !g.quant_scale; };
  if (!plain(f) || f.has_scalar_mul || root->ia[0] != 0 || root->ia[1] != 0 || root->fa[0] != 1.f || (root->in[2] && root->fa[1] != 0.f)) return;
  if (!f.w || f.w->kind == OP_CONST || (f.perm_mode != 0 && f.perm_mode != 2)) return;
  V sm = resolve(f.x);
  if (!sm || sm->kind != OP_SOFTMAX || sm->ia[1] != 0 || users_[sm] != 1 || sm->is_output) return;
  const auto& ps = sm->type.shape;
  if (ps.size != 4 || (sm->ia[0] != 3 && sm->ia[0] != -1)) return;
  V sc_out = resolve(sm->in[0]);
  if (!sc_out || users_[sc_out] != 1 || sc_out->is_output) return;
  auto fi = fused_into_.find(sc_out);
  V sc_root = sc_out->kind == OP_GEMM ? sc_out : (fi != fused_into_.end() ? fi->second : nullptr);
  if (!sc_root || sc_root->kind != OP_GEMM || !fused_.count(sc_root)) return;
  const Fused& g = *fused_[sc_root];
  if (g.out != sc_out || !plain(g) || g.perm_mode != 0 || sc_root->ia[0] != 0 || sc_root->ia[1] == 0 || (sc_root->in[2] && sc_root->fa[1] != 0.f)) return;
  if (!g.w || g.w->kind == OP_CONST) return;
  V q = resolve(g.x), k = resolve(g.w), v = resolve(f.w);
  const auto &qs = q->type.shape, &ks = k->type.shape, &vs = v->type.shape;
  if (qs.size != 4 || ks.size != 4 || vs.size != 4) return;
  const int64_t B = qs.dims[0], NH = qs.dims[1], S = qs.dims[2], D = qs.dims[3];
  if (!attn_supported(fs, S, D)) return;
  for (int d = 0; d < 4; ++d) if (ks.dims[d] != qs.dims[d] || vs.dims[d] != qs.dims[d]) return;
  if (ps.dims[0] != B || ps.dims[1] != NH || ps.dims[2] != S || ps.dims[3] != S) return;
  if (f.perm_mode == 2 && (f.perm_NH != NH || f.perm_S != S || f.perm_D != D)) return;
  if (dt_[q] != fs || dt_[k] != fs || dt_[v] != fs || alias_.count(q) || alias_.count(k) || alias_.count(v)) return;
  if (pitch_.count(q) || pitch_.count(k) || pitch_.count(v)) return;
  // the two earlier launches go; nothing else reads what they would have written
  size_t removed = 0;
  for (size_t i = items_.size(); i-- > 0;)
    if (items_[i].out == sm || items_[i].out == sc_out) { items_.erase(items_.begin() + (long)i); ++removed; }
  if (removed != 2) { B2_WARN("attention pattern at '%s' matched but its producers were not separate launches", root->name.c_str()); }
  it.attn_q = q;
  it.attn_k = k;
  it.attn_scale = sc_root->fa[0] * g.scalar_mul;
  it.reads.clear();
  it.reads.push_back(q); it.reads.push_back(k); it.reads.push_back(v);
}

odla_status Builder::emit_fused(const Item& it) {
  if (it.attn_q) {
    const Fused& f = *it.fused;
    const auto& qs = it.attn_q->type.shape;
    const int64_t B = shape(it.attn_q).dims[0], NH = qs.dims[1], S = qs.dims[2], D = qs.dims[3];
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p_->device);
    AttnLaunch* al = attn_prepare(FS(), dev_ptr(it.attn_q), dev_ptr(it.attn_k), dev_ptr(f.w), dev_ptr(f.out), B, (int)NH, it.attn_scale, f.perm_mode == 2,
                                  p_->status, sms);
    if (!al) return fail(ODLA_FAILURE, "'" + f.root->name + "': fused attention could not be prepared");
    p_->attn.push_back(al);
    const double flops = 2.0 * 2.0 * (double)B * NH * S * S * D;
    const double bytes = 4.0 * (double)B * NH * S * D * storage_size(FS());
    add_launch("attention", f.out, flops, bytes, [al](cudaStream_t s) { return attn_run(al, s); });
    return ODLA_SUCCESS;
  }
  const Fused& f = *it.fused;
  V root = f.root;
  int in_dt = f.int8 ? DT_S8 : FS();
  if (dt_[resolve(f.x)] != in_dt) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + root->name + "': operand storage type does not match the compute type");
  if (in_dt == DT_U8 || in_dt == DT_S32 || in_dt == DT_S64) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + root->name + "': integer convolution needs Dequantize operands");
  const void* x = dev_ptr(f.x);
  void* y = dev_ptr(f.out);
  int64_t K = root->kind == OP_CONV ? (root->ia[0] ? root->type.shape.dims[3] : root->type.shape.dims[1])
                                    : root->type.shape.dims[root->type.shape.size - 1];
  Epilogue ep;
  std::vector<int> wint;   // int8 path: the filter as integers
  int w_terms = 1;         // ... and how many int8 terms they need
  if (f.int8) {
    auto sx = const_as_f32(f.x_scale), sw = const_as_f32(f.w_scale);
    std::vector<float> m((size_t)K);
    for (int64_t k = 0; k < K; ++k) m[k] = sx[0] * sw[sw.size() == 1 ? 0 : k];
    ep.mul = upload_f32(m);
    // Integer filter values: int8 as they are, uint8 minus the zero point (a 9-bit range that is split into int8 terms).
    const int64_t wn = numel(f.w->type.shape);
    wint.resize((size_t)wn);
    if (f.w_zp) {
      const int zp = (int)const_as_f32(f.w_zp)[0];
      for (int64_t i = 0; i < wn; ++i) wint[(size_t)i] = (int)((const uint8_t*)f.w->host)[i] - zp;
      int lo = 0, hi = 0;
      for (int v : wint) { lo = std::min(lo, v); hi = std::max(hi, v); }
      while (lo < -128 * w_terms || hi > 127 * w_terms) ++w_terms;
    } else {
      for (int64_t i = 0; i < wn; ++i) wint[(size_t)i] = ((const int8_t*)f.w->host)[i];
    }
    // |accumulator| <= 128 * sum |w[k,:]| (activations lie in [-128, 127]); below 2^22 for every output channel the
    // epilogue can convert the accumulators without the conversion pipe.
    if (f.w->kind == OP_CONST && !getenv("ODLA_B200_NO_ACC_SMALL")) {
      const int* wq = wint.data();
      const int64_t n = wn;
      // filters are [.., K] (HWIO) and Gemm weights [Kd, N] or, transposed, [N, Kd]: the output channel is the last
      // axis unless the Gemm's B is transposed
      const bool k_last = !(root->kind == OP_GEMM && root->ia[1] != 0);
      std::vector<int64_t> sum((size_t)K, 0);
      if (n % K == 0) {
        const int64_t inner = n / K;
        for (int64_t i = 0; i < n; ++i) sum[(size_t)(k_last ? i % K : i / inner)] += std::abs((int)wq[i]);
        int64_t worst = 0;
        for (int64_t k = 0; k < K; ++k) worst = std::max(worst, sum[(size_t)k]);
        ep.acc_small = worst * 128 < (1ll << 22) ? 1 : 0;
      }
    }
  }
  if (f.add_const) ep.add2 = (const float*)const_dev(f.add_const, DT_F32);
  if (f.res) {
    ep.res = dev_ptr(f.res);
    ep.res_dt = dt_[resolve(f.res)];
    if (f.res_scale) ep.res_scale = const_as_f32(f.res_scale)[0];
    else if (ep.res_dt == DT_S8 || ep.res_dt == DT_U8) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + root->name + "': integer residual without Dequantize");
  }
  ep.act = f.act; ep.act_a = f.act_a; ep.act_b = f.act_b; ep.act_first = f.act_first;
  ep.out_dt = dt_[f.out];
  if (f.quant_scale) {
    ep.out_scale = const_as_f32(f.quant_scale)[0];
    ep.out_inv = 1.0f / ep.out_scale;
    ep.out_multiply = f.int8 ? 1 : 0;  // the chain hangs off int32 accumulators exactly when its root is an int8 kernel
  }
  if (f.has_scalar_mul) ep.alpha = f.scalar_mul;
  bool allow_umma = !getenv("ODLA_B200_NO_UMMA");
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, p_->device);

  if (root->kind == OP_CONV) {
    bool nhwc = root->ia[0] != 0;
    int groups = (int)root->ia[1];
    odla_value_shape xs = shape(root->in[0]), os = shape(root);
    const odla_value_shape& ws = root->in[1]->type.shape;
    if (f.w->kind != OP_CONST) return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': convolution filters must be constants");
    ConvGeom g{};
    g.N = (int)xs.dims[0];
    g.H = (int)(nhwc ? xs.dims[1] : xs.dims[2]); g.W = (int)(nhwc ? xs.dims[2] : xs.dims[3]); g.C = (int)(nhwc ? xs.dims[3] : xs.dims[1]);
    g.R = (int)(nhwc ? ws.dims[0] : ws.dims[2]); g.S = (int)(nhwc ? ws.dims[1] : ws.dims[3]); g.K = (int)K;
    g.P = (int)(nhwc ? os.dims[1] : os.dims[2]); g.Q = (int)(nhwc ? os.dims[2] : os.dims[3]);
    g.stride_h = (int)root->ia[2]; g.stride_w = (int)root->ia[3]; g.pad_t = (int)root->ia[4]; g.pad_l = (int)root->ia[5];
    g.groups = groups;
    int cg = g.C / groups;
    if (root->in[2]) {
      if (root->in[2]->kind != OP_CONST) return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': convolution bias must be a constant");
      ep.add1 = (const float*)const_dev(root->in[2], DT_F32);
    }
    double flops = 2.0 * g.N * g.P * g.Q * (double)K * g.R * g.S * cg;
    double bytes = tensor_bytes(f.x) + tensor_bytes(f.out) + (double)numel(ws) * storage_size(in_dt) + (f.res ? tensor_bytes(f.res) : 0);
    UmmaConv uc{g.N, g.H, g.W, g.C, g.K, g.R, g.S, g.P, g.Q, g.stride_h, g.stride_w, g.pad_t, g.pad_l, in_dt};
    // A few-channel input (the RGB stem) has pixels TMA cannot address (rows must be 16-byte
    // multiples of at least 32 bytes): copy it once into a channel-padded scratch tensor (32 bytes
    // per pixel, zeros in the tail, zero filter taps to match) and run the tensor-core kernel on that.
    int Cp = g.C;
    const void* x_umma = x;
    void* padded = nullptr;
    bool overlap = false;   // ... read through overlapping tensor-map strides instead of a materialised copy
    bool widened = false;   // stride-2 stem rewritten as an (R x 1) convolution over widened pixels (8 input pixels each)
    int wide_c = 32, wide_cp = 4;  // channels of a widened pixel / of each input pixel inside it
    const bool small_c = allow_umma && nhwc && groups == 1 && (in_dt == DT_F16 || in_dt == DT_BF16 || in_dt == DT_S8) && !umma_conv_supported(uc) &&
                         g.C * storage_size(in_dt) < 32;
    // Widened pixels: output column q reads the S input pixels from q*stride_w - pad_l on.  With pixels padded to
    // 16 / stride_w bytes those taps lie inside one 64-byte window that starts 16 bytes after the window of column
    // q-1, so the column taps collapse into the channel axis: an (R x S) convolution over few channels becomes an
    // (R x 1) convolution over 64-byte "widened pixels" with unit column stride.
    int wide_pb = 8, wide_lp = 4, wide_Wp = 0, wide_gq = 1;   // pixel bytes, zero pixels on the left, padded row length, columns per group (overlapping form)
    if (small_c && (g.stride_w == 1 || g.stride_w == 2) && g.S <= 4 * g.stride_w && g.C * storage_size(in_dt) <= 16 / g.stride_w &&
        !getenv("ODLA_B200_NO_WIDEN")) {
      const int esz0 = storage_size(in_dt);
      UmmaConv uw = uc;
      uw.W = g.Q; uw.C = 64 / esz0; uw.S = 1; uw.stride_w = 1; uw.pad_l = 0;
      // First choice: no widened copy at all.  A pre-pass pads every pixel to 16 / stride_w bytes and every row with
      // pad_l zero pixels on the left (and enough on the right); the widened pixel of column q is then the 64
      // contiguous bytes that start 16 bytes after the one of column q-1, which a tensor map with a W stride smaller
      // than the pixel size describes directly.  If the driver refuses such a map, a stride-2 stem falls back to a
      // materialised widened copy, others to plain channel padding.
      if (umma_conv_supported(uw) && !getenv("ODLA_B200_NO_OVERLAP")) {
        int pb = 16 / g.stride_w;
        // Column groups: gq neighbouring output columns share one window (their taps span (gq-1)*stride_w + S
        // pixels) and become gq*K "channels" of one output pixel -- the same bytes in memory.  That divides the number
        // of rows the TMA unit has to deliver, which is what bounds a stem, by gq and gives the tensor pipe gq times
        // wider instructions.  A group's window starts every gq*stride_w pixels, so pixels may be narrower than
        // 16/stride_w bytes as long as that distance stays a multiple of 16 bytes: int8 RGB pixels take 4 bytes, which
        // halves the window (and the number of tensor-core instructions per tile) against 8-byte pixels.
        int gq = 1;
        if (!f.res && !getenv("ODLA_B200_NO_COLUMN_GROUPS"))
          for (int cand = 4; cand >= 2 && gq == 1; cand /= 2) {
            if (g.Q % cand != 0 || (int64_t)cand * K > 256) continue;
            int px = 4;
            while (px < g.C * esz0) px *= 2;
            for (; px <= 16 / g.stride_w; px *= 2)
              if ((cand * g.stride_w * px) % 16 == 0 && ((cand - 1) * g.stride_w + g.S) * px <= 128 && !getenv("ODLA_B200_WIDE_PIXELS")) break;
            if (px > 16 / g.stride_w) { px = 16 / g.stride_w; if ((cand - 1) * g.stride_w + g.S > 128 / px) continue; }
            gq = cand; pb = px;
          }
        int win_bytes = 64;
        if (gq > 1) { const int need = ((gq - 1) * g.stride_w + g.S) * pb; win_bytes = need > 64 ? 128 : (need > 32 ? 64 : 32); }
        const int wp = win_bytes / pb;
        int Wp = std::max(g.pad_l + g.W, (g.Q / gq - 1) * gq * g.stride_w + wp);
        { const int unit = 16 / pb > 1 ? 16 / pb : 1; Wp = (Wp + unit - 1) / unit * unit; }  // rows are 16-byte multiples for every pixel size
        UmmaConv uo = uw;
        uo.C = win_bytes / esz0;
        uo.W = g.Q / gq; uo.Q = g.Q / gq; uo.K = (int)(K * gq);
        uo.x_w_stride = (long long)gq * g.stride_w * pb;
        uo.x_h_stride = (long long)Wp * pb;
        uo.x_n_stride = uo.x_h_stride * g.H;
        void* padbuf = nullptr;
        size_t pbytes = (size_t)uo.x_n_stride * g.N + 256;
        if (umma_conv_supported(uo) && !inject_fault("alloc") && cudaMalloc(&padbuf, pbytes) == cudaSuccess) {
          Epilogue probe_ep;
          probe_ep.out_dt = DT_F32;
          UmmaLaunch* probe = umma_conv_prepare(uo, padbuf, padbuf, padbuf, probe_ep, p_->status, sms);
          if (probe) {
            umma_conv_destroy(probe);
            p_->extra_allocs.push_back(padbuf);
            padded = padbuf;
            x_umma = padded;
            uc = uo;
            widened = true;
            overlap = true;
            wide_c = uo.C;
            wide_pb = pb; wide_cp = pb / esz0; wide_lp = g.pad_l; wide_Wp = Wp; wide_gq = gq;
            if (gq > 1) {
              // per-channel vectors repeat for every column of the group
              auto tile = [&](const std::vector<float>& v) { std::vector<float> t; t.reserve(v.size() * gq); for (int r = 0; r < gq; ++r) t.insert(t.end(), v.begin(), v.end()); return upload_f32(t); };
              if (ep.mul) { auto sx = const_as_f32(f.x_scale), sw = const_as_f32(f.w_scale); std::vector<float> m((size_t)K); for (int64_t k = 0; k < K; ++k) m[k] = sx[0] * sw[sw.size() == 1 ? 0 : k]; ep.mul = tile(m); }
              if (ep.add1) ep.add1 = tile(const_as_f32(root->in[2]));
              if (ep.add2) ep.add2 = tile(const_as_f32(f.add_const));
            }
          } else {
            cudaFree(padbuf);
          }
        } else cudaGetLastError();
      }
      // Second choice (stride 2, at most 4 channels, taps within 2q-4 .. 2q+3): gather the eight pixels x 4 channels
      // of every output column into a materialised 32-channel tensor.
      if (!widened && g.stride_w == 2 && g.C <= 4 && g.pad_l <= 4 && g.S - g.pad_l <= 4) {
        UmmaConv um = uw;
        um.C = 32;
        if (umma_conv_supported(um)) {
          size_t pbytes = (size_t)g.N * g.H * g.Q * 32 * esz0;
          if (inject_fault("alloc") || cudaMalloc(&padded, pbytes ? pbytes : 32) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
          p_->extra_allocs.push_back(padded);
          x_umma = padded;
          uc = um;
          widened = true;
          wide_c = 32; wide_cp = 4; wide_lp = 4;
        }
      }
    }
    if (small_c && !widened) {
      UmmaConv up = uc;
      up.C = 32 / storage_size(in_dt);
      if (umma_conv_supported(up)) {
        Cp = up.C;
        size_t pbytes = (size_t)g.N * g.H * g.W * 32;
        if (inject_fault("alloc") || cudaMalloc(&padded, pbytes ? pbytes : 32) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
        p_->extra_allocs.push_back(padded);
        x_umma = padded;
        uc = up;
      }
    }
    if (allow_umma && nhwc && groups == 1 && umma_conv_supported(uc)) {
      // filters HWIO -> [K][R*S*C] so that each output channel's taps are contiguous (K-major B operand)
      char form[256];
      snprintf(form, sizeof(form), "conv_kmajor dt%d w%d gq%d wc%d cp%d lp%d pl%d sw%d Cp%d", in_dt, widened ? 1 : 0, wide_gq, wide_c, wide_cp, wide_lp, g.pad_l, g.stride_w, Cp);
      if (w_terms > 1) {
        if (widened || Cp != g.C) return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': asymmetric uint8 filters over fewer than 32 bytes of channels");
        uc.w_terms = w_terms;
        snprintf(form + strlen(form), sizeof(form) - strlen(form), " terms%d", w_terms);
      }
      if (f.w_zp) snprintf(form + strlen(form), sizeof(form) - strlen(form), " zp%d", (int)const_as_f32(f.w_zp)[0]);
      auto wb = prepared(f.w, form, [&] {
        if (w_terms > 1) {
          // [K][terms * R*S][C] int8: term t holds clamp(remainder, -128, 127) of every filter value
          const int64_t rs = (int64_t)g.R * g.S;
          std::vector<uint8_t> out((size_t)(K * w_terms * rs * g.C));
          for (int64_t t2 = 0; t2 < rs; ++t2)
            for (int64_t c = 0; c < g.C; ++c)
              for (int64_t k = 0; k < K; ++k) {
                int rem = wint[(size_t)((t2 * g.C + c) * K + k)];
                for (int t = 0; t < w_terms; ++t) {
                  const int part = std::max(-128, std::min(127, rem));
                  rem -= part;
                  out[(size_t)(((k * w_terms + t) * rs + t2) * g.C + c)] = (uint8_t)(int8_t)part;
                }
              }
          return out;
        }
        auto wf = f.int8 ? std::vector<float>(wint.begin(), wint.end()) : const_as_f32(f.w);
        int64_t rs = (int64_t)g.R * g.S;
        std::vector<float> w2;
        if (widened) {
          // [gq*K][R][wide_c]: element el of a window is pixel el / cp, channel el % cp; the window starts wide_lp pixels
          // left of column (q - q % gq) * stride_w, the taps of the group's column j start pad_l - j*stride_w pixels left
          // of it: filter column = el / cp - wide_lp + pad_l - j * stride_w
          w2.assign((size_t)(K * wide_gq * g.R * wide_c), 0.f);
          for (int j = 0; j < wide_gq; ++j)
            for (int64_t r = 0; r < g.R; ++r)
              for (int el = 0; el < wide_c; ++el) {
                int sc = el / wide_cp - wide_lp + g.pad_l - j * g.stride_w, c = el % wide_cp;
                if (sc < 0 || sc >= g.S || c >= g.C) continue;
                for (int64_t k = 0; k < K; ++k) w2[(size_t)(((j * K + k) * g.R + r) * wide_c + el)] = wf[(size_t)(((r * g.S + sc) * g.C + c) * K + k)];
              }
        } else {
          w2.assign((size_t)(K * rs * Cp), 0.f);
          for (int64_t t = 0; t < rs; ++t)
            for (int64_t c = 0; c < g.C; ++c)
              for (int64_t k = 0; k < K; ++k) w2[(size_t)((k * rs + t) * Cp + c)] = wf[(size_t)((t * g.C + c) * K + k)];
        }
        return f32_to_storage(w2, in_dt);
      });
      void* wd = upload(wb->data(), wb->size());
      if (!wd) return err_status_;
      if (pitch_.count(f.out)) uc.y_pitch = (int)pitch_[f.out];
      UmmaLaunch* ul = umma_conv_prepare(uc, x_umma, wd, y, ep, p_->status, sms);
      if (!ul) return fail(ODLA_FAILURE, "'" + root->name + "': tensor-map encoding failed");
      p_->umma.push_back(ul);
      if (padded) {
        int esz = storage_size(in_dt), C0 = g.C;
        int64_t pixels = (int64_t)g.N * g.H * g.W;
        ConvGeom gg = g;
        bool wide = widened, ov = overlap;
        const int pbb = wide_pb, lpp = wide_lp, Wpp = wide_Wp;
        double scratch_bytes = ov ? 2.0 * g.N * g.H * (double)Wpp * pbb : wide ? 2.0 * g.N * g.H * g.Q * 32 * esz : 2.0 * pixels * 32;
        add_launch("conv_umma", f.out, flops, bytes + scratch_bytes, [=](cudaStream_t s) {
          int rc = ov ? stem_pad(esz, x, padded, gg.N, gg.H, gg.W, C0, pbb, lpp, Wpp, s)
                      : wide ? stem_widen(esz, x, padded, gg.N, gg.H, gg.W, C0, gg.Q, s) : pad_channels(esz, x, padded, pixels, C0, Cp, s);
          return rc ? rc : umma_conv_run(ul, s);
        });
        p_->launches.back().n_kernels = 2;
      } else {
        add_launch("conv_umma", f.out, flops, bytes, [ul](cudaStream_t s) { return umma_conv_run(ul, s); });
      }
      return ODLA_SUCCESS;
    }
    if (f.w_zp) return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': asymmetric uint8 filters need the tensor-core path (NHWC, one group, 16-byte channel rows)");
    const void* wd = const_dev(f.w, in_dt);
    if (!wd) return err_status_;
    if (nhwc) {
      g.xs_c = 1; g.xs_w = g.C; g.xs_h = (int64_t)g.W * g.C; g.xs_n = (int64_t)g.H * g.W * g.C;
      g.ys_c = 1; g.ys_w = g.K; g.ys_h = (int64_t)g.Q * g.K; g.ys_n = (int64_t)g.P * g.Q * g.K;
      g.ws_k = 1; g.ws_c = g.K; g.ws_s = (int64_t)cg * g.K; g.ws_r = (int64_t)g.S * cg * g.K;
    } else {
      g.xs_w = 1; g.xs_h = g.W; g.xs_c = (int64_t)g.H * g.W; g.xs_n = (int64_t)g.C * g.H * g.W;
      g.ys_w = 1; g.ys_h = g.Q; g.ys_c = (int64_t)g.P * g.Q; g.ys_n = (int64_t)g.K * g.P * g.Q;
      g.ws_s = 1; g.ws_r = g.S; g.ws_c = (int64_t)g.R * g.S; g.ws_k = (int64_t)cg * g.R * g.S;
      if (f.res || ep.add_full) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + root->name + "': NCHW chain fused unexpectedly");
    }
    add_launch("conv_simt", f.out, flops, bytes, [=](cudaStream_t s) { return conv_simt(g, in_dt, x, wd, y, ep, s); });
    return ODLA_SUCCESS;
  }

  // ---- Gemm ----
  V A = root->in[0], Bv = root->in[1], C = root->in[2];
  odla_value_shape as = shape(A);
  odla_value_shape bs = f.w->kind == OP_CONST ? f.w->type.shape : shape(Bv);
  bool ta = root->ia[0] != 0, tb = root->ia[1] != 0;
  float alpha = root->fa[0], beta = root->fa[1];
  int ra = as.size, rb = bs.size;
  int64_t batch = 1, bbatch = 1;
  for (int i = 0; i < ra - 2; ++i) batch *= as.dims[i];
  for (int i = 0; i < rb - 2; ++i) bbatch *= bs.dims[i];
  int64_t ar = as.dims[ra - 2], ac = as.dims[ra - 1], br = bs.dims[rb - 2], bc = bs.dims[rb - 1];
  int64_t M = ta ? ac : ar, Kd = ta ? ar : ac, N = tb ? br : bc;
  if ((tb ? bc : br) != Kd) return fail(ODLA_INVALID_PARAM, "'" + root->name + "': Gemm inner dimensions differ");
  if (bbatch != batch && bbatch != 1) return fail(ODLA_INVALID_PARAM, "'" + root->name + "': Gemm batch dimensions differ");
  if (count(root) != batch * M * N) return fail(ODLA_INVALID_PARAM, "'" + root->name + "': Gemm output_dims do not match the operands");
  ep.alpha = alpha * f.scalar_mul;
  if (C && beta != 0.f) {
    int64_t cn = C->kind == OP_CONST ? numel(C->type.shape) : count(C);
    if (C->kind == OP_CONST && (cn == 1 || cn == N)) {
      auto cf = const_as_f32(C);
      std::vector<float> v((size_t)N);
      for (int64_t j = 0; j < N; ++j) v[j] = beta * cf[cn == 1 ? 0 : j];
      ep.add1 = upload_f32(v);
    } else if (cn == batch * M * N) {
      if (C->kind == OP_CONST) { ep.add_full = const_dev(C, DT_F32); ep.add_full_dt = DT_F32; }
      else { ep.add_full = dev_ptr(C); ep.add_full_dt = dt_[resolve(C)]; }
      ep.beta_full = beta;
    } else return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': Gemm C must be a constant scalar / row vector or a full matrix");
  }
  double flops = 2.0 * batch * M * N * Kd;
  double bytes = tensor_bytes(f.x) + tensor_bytes(f.out) + (double)(br * bc * bbatch) * storage_size(in_dt);
  // Head split / merge folded into the store.  When the tensor-core kernel cannot store through the permuted map
  // (fp32 graphs, a sequence that does not fill 128-row boxes, ...) the product goes to scratch and is moved.
  void* y_final = y;
  MoveGeom perm_move{};
  bool perm_via_move = false;
  auto set_store = [&](UmmaConv& u) { u.store_mode = f.perm_mode; u.store_S = (int)f.perm_S; u.store_NH = (int)f.perm_NH; u.store_D = (int)f.perm_D; };
  if (f.perm_mode) {
    bool direct = false;
    if (allow_umma && !ta) {
      UmmaConv probe{1, 1, (int)(batch * M), (int)Kd, (int)N, 1, 1, 1, (int)(batch * M), 1, 1, 0, 0, in_dt};
      if (f.w->kind != OP_CONST) { probe.w_batches = (int)batch; probe.rows_per_batch = (int)M; }
      set_store(probe);
      const bool shape_ok = f.w->kind == OP_CONST ? bbatch == 1
                                                  : (bbatch == batch && batch > 1 && M % 128 == 0 && (in_dt == DT_F16 || in_dt == DT_BF16) && dt_[resolve(f.w)] == in_dt);
      direct = shape_ok && batch * M < (1ll << 31) && umma_conv_supported(probe) && umma_store_perm_ok(probe, ep, y);
    }
    if (!direct) {
      void* tmp = nullptr;
      if (cudaMalloc(&tmp, (size_t)std::max<int64_t>(count(root) * storage_size(dt_[f.out]), 16)) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
      p_->extra_allocs.push_back(tmp);
      y = tmp;
      perm_via_move = true;
      // scratch is [B][X][Y][D] row-major (X, Y = S, NH for a split; NH, S for a merge); the result swaps X and Y
      const int64_t X = f.perm_mode == 1 ? f.perm_S : f.perm_NH, Yd = f.perm_mode == 1 ? f.perm_NH : f.perm_S, D = f.perm_D;
      const int64_t Bn = count(root) / (X * Yd * D);
      perm_move.rank = 4;
      perm_move.oshape[0] = Bn; perm_move.oshape[1] = Yd; perm_move.oshape[2] = X; perm_move.oshape[3] = D;
      perm_move.istride[0] = X * Yd * D; perm_move.istride[1] = D; perm_move.istride[2] = Yd * D; perm_move.istride[3] = 1;
      perm_move.ostride[0] = X * Yd * D; perm_move.ostride[1] = X * D; perm_move.ostride[2] = D; perm_move.ostride[3] = 1;
    }
  }
  const bool store_direct = f.perm_mode && !perm_via_move;
  const int out_esz = storage_size(dt_[f.out]);
  // wraps a launch so that the scratch result is moved into place afterwards
  auto with_move = [&](std::function<int(cudaStream_t)> fn) -> std::function<int(cudaStream_t)> {
    if (!perm_via_move) return fn;
    const void* src = y;
    return [=](cudaStream_t s) { int rc = fn(s); return rc ? rc : move(perm_move, out_esz, src, y_final, s); };
  };
  if (allow_umma && !ta && f.w->kind == OP_CONST && bbatch == 1) {
    int64_t Mt = batch * M;
    UmmaConv uc{1, 1, (int)Mt, (int)Kd, (int)N, 1, 1, 1, (int)Mt, 1, 1, 0, 0, in_dt};
    if (store_direct) set_store(uc);
    if (Mt < (1ll << 31) && umma_conv_supported(uc)) {
      if (w_terms > 1) uc.w_terms = w_terms;
      auto wb = prepared(f.w, std::string("gemm_kmajor dt") + std::to_string(in_dt) + (tb ? " t" : " n") + " terms" + std::to_string(w_terms) +
                                  (f.w_zp ? " zp" + std::to_string((int)const_as_f32(f.w_zp)[0]) : std::string()), [&] {
        if (w_terms > 1) {
          // [N][terms][Kd] int8
          std::vector<uint8_t> out((size_t)(N * w_terms * Kd));
          for (int64_t n = 0; n < N; ++n)
            for (int64_t k = 0; k < Kd; ++k) {
              int rem = wint[(size_t)(tb ? n * Kd + k : k * N + n)];
              for (int t = 0; t < w_terms; ++t) {
                const int part = std::max(-128, std::min(127, rem));
                rem -= part;
                out[(size_t)((n * w_terms + t) * Kd + k)] = (uint8_t)(int8_t)part;
              }
            }
          return out;
        }
        auto wf = f.int8 ? std::vector<float>(wint.begin(), wint.end()) : const_as_f32(f.w);
        std::vector<float> w2;
        if (tb) w2 = wf;  // already [N][K]
        else { w2.resize(wf.size()); for (int64_t k = 0; k < Kd; ++k) for (int64_t n = 0; n < N; ++n) w2[(size_t)(n * Kd + k)] = wf[(size_t)(k * N + n)]; }
        return f32_to_storage(w2, in_dt);
      });
      void* wd = upload(wb->data(), wb->size());
      if (!wd) return err_status_;
      UmmaLaunch* ul = umma_conv_prepare(uc, x, wd, y, ep, p_->status, sms);
      if (!ul) return fail(ODLA_FAILURE, "'" + root->name + "': tensor-map encoding failed");
      p_->umma.push_back(ul);
      add_launch("gemm_umma", f.out, flops, bytes, with_move([ul](cudaStream_t s) { return umma_conv_run(ul, s); }));
      if (perm_via_move) p_->launches.back().n_kernels = 2;
      return ODLA_SUCCESS;
    }
  }
  // Batched product of two run-time tensors (attention scores and context): one tensor-core launch whose B
  // operand changes with the batch.  A [batch, K, 64] operand is read in place (MN-major); any other [batch, K, N]
  // operand is transposed into scratch first, because B is otherwise read K-major.
  if (allow_umma && !ta && f.w->kind != OP_CONST && bbatch == batch && batch > 1 && M % 128 == 0 && (in_dt == DT_F16 || in_dt == DT_BF16) &&
      dt_[resolve(f.w)] == in_dt && batch * M < (1ll << 31)) {
    UmmaConv uc{1, 1, (int)(batch * M), (int)Kd, (int)N, 1, 1, 1, (int)(batch * M), 1, 1, 0, 0, in_dt};
    uc.w_batches = (int)batch;
    uc.rows_per_batch = (int)M;
    if (store_direct) set_store(uc);
    // a [batch, K, 64] operand (attention probabilities x V) is read as it lies; other widths are transposed first
    if (!tb && N == 64 && Kd % 64 == 0 && !getenv("ODLA_B200_NO_N_MAJOR")) uc.w_n_major = 1;
    if (umma_conv_supported(uc)) {
      const void* bsrc = dev_ptr(f.w);
      void* bt = nullptr;
      MoveGeom mg{};
      if (!tb && !uc.w_n_major) {
        if (cudaMalloc(&bt, (size_t)(batch * N * Kd * storage_size(in_dt))) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
        p_->extra_allocs.push_back(bt);
        mg.rank = 3;
        mg.oshape[0] = batch; mg.oshape[1] = N; mg.oshape[2] = Kd;
        mg.istride[0] = Kd * N; mg.istride[1] = 1; mg.istride[2] = N;
        mg.ostride[0] = N * Kd; mg.ostride[1] = Kd; mg.ostride[2] = 1;
      }
      UmmaLaunch* ul = umma_conv_prepare(uc, x, bt ? bt : bsrc, y, ep, p_->status, sms);
      if (!ul) return fail(ODLA_FAILURE, "'" + root->name + "': tensor-map encoding failed");
      p_->umma.push_back(ul);
      int esz = storage_size(in_dt);
      add_launch("gemm_umma", f.out, flops, bytes, with_move([=](cudaStream_t s) {
        if (bt) { int rc = move(mg, esz, bsrc, bt, s); if (rc) return rc; }
        return umma_conv_run(ul, s);
      }));
      p_->launches.back().n_kernels = (bt ? 2 : 1) + (perm_via_move ? 1 : 0);
      return ODLA_SUCCESS;
    }
  }
  if (f.w_zp) return fail(ODLA_UNSUPPORTED_OP, "'" + root->name + "': asymmetric uint8 weights need the tensor-core path (rows of 16-byte multiples)");
  GemmGeom g{};
  g.batch = batch; g.M = M; g.N = N; g.K = Kd;
  g.a_row = ta ? 1 : ac; g.a_col = ta ? ac : 1; g.a_batch = ar * ac;
  g.b_row = tb ? 1 : bc; g.b_col = tb ? bc : 1; g.b_batch = bbatch == 1 ? 0 : br * bc;
  const void* bp;
  if (f.w->kind == OP_CONST) bp = const_dev(f.w, in_dt);
  else {
    if (dt_[resolve(f.w)] != in_dt) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + root->name + "': Gemm operand types differ");
    bp = dev_ptr(f.w);
  }
  if (!bp) return err_status_;
  add_launch("gemm_simt", f.out, flops, bytes, with_move([=](cudaStream_t s) { return gemm_simt(g, in_dt, x, bp, y, ep, s); }));
  if (perm_via_move) p_->launches.back().n_kernels = 2;
  return ODLA_SUCCESS;
}

odla_status Builder::emit_plain(const Item& it) {
  V v = it.out;
  void* y = dev_ptr(v);
  int odt = dt_[v];
  // operand pointer + storage type; constants are uploaded (float constants as fp32 unless `want` says otherwise)
  auto operand = [&](V o, int* dt, int want = -1) -> const void* {
    V r = resolve(o);
    if (r->kind == OP_CONST) {
      int d = want >= 0 ? want : (is_float_type(r->type.element_type) ? DT_F32 : api_dt(r->type.element_type));
      *dt = d;
      return const_dev(r, d);
    }
    *dt = dt_[r];
    return dev_ptr(r);
  };
  odla_value_shape os = shape(v);
  double out_bytes = tensor_bytes(v);
  switch (v->kind) {
    case OP_MAXPOOL: case OP_AVGPOOL: {
      V xin = v->in[0];
      int xdt; const void* x = operand(xin, &xdt, odt);
      if (xdt != odt) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': pooling changes the storage type");
      bool nhwc = v->ia[0] != 0;
      odla_value_shape xs = shape(xin);
      PoolGeom g{};
      g.N = (int)xs.dims[0];
      g.H = (int)(nhwc ? xs.dims[1] : xs.dims[2]); g.W = (int)(nhwc ? xs.dims[2] : xs.dims[3]); g.C = (int)(nhwc ? xs.dims[3] : xs.dims[1]);
      g.P = (int)(nhwc ? os.dims[1] : os.dims[2]); g.Q = (int)(nhwc ? os.dims[2] : os.dims[3]);
      g.R = (int)v->ia[1]; g.S = (int)v->ia[2]; g.stride_h = (int)v->ia[3]; g.stride_w = (int)v->ia[4]; g.pad_t = (int)v->ia[5]; g.pad_l = (int)v->ia[6];
      if (nhwc) {
        g.xs_c = 1; g.xs_w = g.C; g.xs_h = (int64_t)g.W * g.C; g.xs_n = (int64_t)g.H * g.W * g.C;
        g.ys_c = 1; g.ys_w = g.C; g.ys_h = (int64_t)g.Q * g.C; g.ys_n = (int64_t)g.P * g.Q * g.C;
      } else {
        g.xs_w = 1; g.xs_h = g.W; g.xs_c = (int64_t)g.H * g.W; g.xs_n = (int64_t)g.C * g.H * g.W;
        g.ys_w = 1; g.ys_h = g.Q; g.ys_c = (int64_t)g.P * g.Q; g.ys_n = (int64_t)g.C * g.P * g.Q;
      }
      bool is_max = v->kind == OP_MAXPOOL;
      if (!is_max && (odt == DT_S8 || odt == DT_U8)) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + v->name + "': average pooling of integers");
      add_launch(is_max ? "maxpool" : "avgpool", v, 0, tensor_bytes(xin) + out_bytes, [=](cudaStream_t s) { return pool2d(g, odt, is_max, x, y, s); });
      return ODLA_SUCCESS;
    }
    case OP_BATCHNORM: {
      int xdt; const void* x = operand(v->in[0], &xdt);
      bool nhwc = v->ia[0] != 0;
      int64_t C = nhwc ? os.dims[os.size - 1] : os.dims[1], inner = 1;
      if (!nhwc) for (int i = 2; i < os.size; ++i) inner *= os.dims[i];
      int64_t outer = count(v) / (C * inner);
      auto mean = const_as_f32(v->in[1]), var = const_as_f32(v->in[2]);
      std::vector<float> a((size_t)C), b((size_t)C);
      std::vector<float> sc = v->in[3] ? const_as_f32(v->in[3]) : std::vector<float>(), of = v->in[4] ? const_as_f32(v->in[4]) : std::vector<float>();
      for (int64_t c = 0; c < C; ++c) {
        float inv = 1.0f / std::sqrt(var[c] + v->fa[0]);
        float s = v->in[3] ? sc[c] : v->fa[1], o = v->in[4] ? of[c] : v->fa[2];
        a[c] = s * inv;
        b[c] = -s * mean[c] * inv + o;
      }
      const float* ad = upload_f32(a); const float* bd = upload_f32(b);
      if (xdt != odt) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': batchnorm changes the storage type");
      add_launch("batchnorm", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return channel_affine(odt, x, y, ad, bd, outer, C, inner, s); });
      return ODLA_SUCCESS;
    }
    case OP_UNARY: {
      int xdt; const void* x = operand(v->in[0], &xdt);
      int op = (int)v->ia[0]; float a = v->fa[0], b = v->fa[1]; int64_t n = count(v);
      add_launch("unary", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return unary(op, xdt, odt, x, y, n, a, b, s); });
      return ODLA_SUCCESS;
    }
    case OP_BINARY: {
      int ldt, rdt; const void* l = operand(v->in[0], &ldt); const void* r = operand(v->in[1], &rdt);
      odla_value_shape ls = resolve(v->in[0])->kind == OP_CONST ? v->in[0]->type.shape : shape(v->in[0]);
      odla_value_shape rs = resolve(v->in[1])->kind == OP_CONST ? v->in[1]->type.shape : shape(v->in[1]);
      if (os.size > 8) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': rank above 8");
      BinaryGeom g{};
      g.rank = os.size;
      int64_t la = 1, ra = 1;
      for (int d = os.size - 1; d >= 0; --d) {
        int li = d - (os.size - ls.size), ri = d - (os.size - rs.size);
        int64_t ld = li >= 0 ? ls.dims[li] : 1, rd = ri >= 0 ? rs.dims[ri] : 1;
        g.oshape[d] = os.dims[d];
        g.lstride[d] = ld == os.dims[d] ? la : 0;
        g.rstride[d] = rd == os.dims[d] ? ra : 0;
        if (os.dims[d] == 1) { g.lstride[d] = g.rstride[d] = 0; }
        la *= ld; ra *= rd;
      }
      // keep dense strides for size-1 dims out of the "same shape" test: recompute with 0 allowed
      int op = (int)v->ia[0];
      add_launch("binary", v, 0, out_bytes * 3, [=](cudaStream_t s) { return binary(op, g, ldt, rdt, odt, l, r, y, ACT_NONE, 0.f, s); });
      return ODLA_SUCCESS;
    }
    case OP_SOFTMAX: {
      int xdt; const void* x = operand(v->in[0], &xdt);
      int axis = (int)v->ia[0]; bool lg = v->ia[1] != 0;
      int64_t outer = 1, inner = 1, dim = os.dims[axis];
      for (int i = 0; i < axis; ++i) outer *= os.dims[i];
      for (int i = axis + 1; i < os.size; ++i) inner *= os.dims[i];
      if (xdt != odt) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': softmax changes the storage type");
      add_launch("softmax", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return softmax(odt, x, y, outer, dim, inner, lg, s); });
      return ODLA_SUCCESS;
    }
    case OP_REDUCE_MEAN: {
      V xin = v->in[0];
      float in_scale = 1.f;
      if (xin->kind == OP_DEQUANTIZE && dq_unabsorbed_.count(xin) && dq_unabsorbed_[xin] == 0 && is_per_tensor_dq(xin)) {
        in_scale = const_as_f32(xin->in[1])[0];   // the first pass reads the int8 tensor and scales each term as Dequantize would
        xin = xin->in[0];
      }
      int xdt; const void* x = operand(xin, &xdt);
      odla_value_shape xs = shape(v->in[0]);
      std::vector<int64_t> d(xs.dims, xs.dims + xs.size);
      struct Pass { const void* src; void* dst; int sdt, ddt; int64_t before, dim, after; };
      std::vector<Pass> passes;
      const void* cur = x; int cdt = xdt;
      size_t n_axes = v->ia.size() - 1;
      if (n_axes == 0) return fail(ODLA_INVALID_PARAM, "'" + v->name + "': ReduceMean without axes");
      for (size_t k = 0; k < n_axes; ++k) {
        int64_t a = v->ia[1 + k], before = 1, after = 1;
        for (int64_t i = 0; i < (int64_t)d.size(); ++i) { if (i < a) before *= d[i]; else if (i > a) after *= d[i]; }
        bool lastp = k + 1 == n_axes;
        void* dst = y; int ddt = odt;
        if (!lastp) {  // intermediate passes keep fp32 so that the order of roundings equals the reference's
          void* t = nullptr;
          if (cudaMalloc(&t, (size_t)(before * after * 4)) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
          p_->extra_allocs.push_back(t);
          dst = t; ddt = DT_F32;
        }
        passes.push_back({cur, dst, cdt, ddt, before, d[a], after});
        d[a] = 1; cur = dst; cdt = ddt;
      }
      // two adjacent axes in rising order (a global average pool): one launch when the kernel serves the shape
      const bool adjacent = n_axes == 2 && v->ia[2] == v->ia[1] + 1 && passes[0].after == passes[1].dim * passes[1].after &&
                            passes[1].before == passes[0].before && !getenv("ODLA_B200_REDUCE_TWO_PASSES");
      const int vec = cdt == DT_F32 && xdt == DT_F32 ? 4 : (xdt == DT_S8 ? 16 : (xdt == DT_F32 ? 4 : 8));
      const bool one_launch = adjacent && passes[0].dim == 7 && passes[1].dim == 7 && passes[1].after % vec == 0;
      add_launch("reduce_mean", v, 0, tensor_bytes(xin) + out_bytes, [=](cudaStream_t s) {
        if (adjacent) {
          int r = reduce_mean_two_axes(passes[0].sdt, passes[1].ddt, passes[0].src, passes[1].dst, passes[0].before, passes[0].dim, passes[1].dim, passes[1].after, s, in_scale);
          if (r <= 0) return r;
        }
        bool first = true;
        for (auto& p : passes) { int r = reduce_mean_axis(p.sdt, p.ddt, p.src, p.dst, p.before, p.dim, p.after, s, first ? in_scale : 1.f); if (r) return r; first = false; }
        return 0;
      });
      p_->launches.back().n_kernels = one_launch ? 1 : (int)passes.size();
      return ODLA_SUCCESS;
    }
    case OP_LAYERNORM: {
      int xdt; const void* x = operand(v->in[0], &xdt);
      int64_t dim = 1; for (int i = os.size - (int)v->ia[0]; i < os.size; ++i) dim *= os.dims[i];
      int64_t rows = count(v) / dim;
      const float* g = v->in[1] ? (const float*)const_dev(v->in[1], DT_F32) : nullptr;
      const float* b = v->in[2] ? (const float*)const_dev(v->in[2], DT_F32) : nullptr;
      float eps = v->fa[0];
      if (xdt != odt) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': layernorm changes the storage type");
      if (V qv = it.extra_out) {
        void* q = dev_ptr(qv);
        const float* qs = (const float*)const_dev(qv->in[1], DT_F32);
        if (!q || !qs) return err_status_;
        add_launch("layernorm", v, 0, 2 * out_bytes + tensor_bytes(qv), [=](cudaStream_t s) { return layernorm_quantize(odt, x, y, g, b, rows, dim, eps, q, qs, s); });
        return ODLA_SUCCESS;
      }
      add_launch("layernorm", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return layernorm(odt, x, y, g, b, rows, dim, eps, s); });
      return ODLA_SUCCESS;
    }
    case OP_QUANTIZE: case OP_DEQUANTIZE: {
      bool q = v->kind == OP_QUANTIZE;
      int xdt; const void* x = operand(v->in[0], &xdt);
      const float* sc = (const float*)const_dev(v->in[1], DT_F32);
      const int* zp = v->in[2] ? (const int*)const_dev(v->in[2], DT_S32) : nullptr;
      int64_t ns = numel(v->in[1]->type.shape);
      bool per_axis = ns > 1;
      int64_t outer = 1, adim = 1, inner = count(v);
      if (per_axis) {
        int axis = (int)v->ia[0];
        if (os.dims[axis] != ns) return fail(ODLA_INVALID_PARAM, "'" + v->name + "': scale count differs from the axis extent");
        outer = 1; inner = 1; adim = os.dims[axis];
        for (int i = 0; i < axis; ++i) outer *= os.dims[i];
        for (int i = axis + 1; i < os.size; ++i) inner *= os.dims[i];
      }
      if (q && from_acc_[v->in[0]] && !per_axis && !zp && odt == DT_S8) {
        float inv = 1.0f / const_as_f32(v->in[1])[0];
        int64_t n = count(v);
        add_launch("requantize", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return requantize(xdt, x, y, inv, n, s); });
      } else if (q) {
        bool uns = odt == DT_U8;
        add_launch("quantize", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return quantize(xdt, x, y, sc, zp, outer, adim, inner, per_axis, uns, s); });
      } else {
        if (xdt != DT_S8 && xdt != DT_U8) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + v->name + "': Dequantize input must be int8 / uint8");
        bool uns = xdt == DT_U8;
        add_launch("dequantize", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return dequantize(odt, x, y, sc, zp, outer, adim, inner, per_axis, uns, s); });
      }
      return ODLA_SUCCESS;
    }
    case OP_TRANSPOSE: {
      int xdt; const void* x = operand(v->in[0], &xdt, odt);
      odla_value_shape xs = shape(v->in[0]);
      if (xs.size > 8) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': rank above 8");
      int64_t istr[ODLA_MAX_DIMENSION], a = 1;
      for (int i = xs.size - 1; i >= 0; --i) { istr[i] = a; a *= xs.dims[i]; }
      MoveGeom g{};
      g.rank = xs.size;
      a = 1;
      for (int i = xs.size - 1; i >= 0; --i) { g.oshape[i] = xs.dims[v->ia[i]]; g.istride[i] = istr[v->ia[i]]; g.ostride[i] = a; a *= g.oshape[i]; }
      int esz = storage_size(odt);
      add_launch("transpose", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return move(g, esz, x, y, s); });
      return ODLA_SUCCESS;
    }
    case OP_CONCAT: {
      int axis = (int)v->ia[0];
      int64_t outer = 1, inner = 1, off = 0;
      for (int i = 0; i < axis; ++i) outer *= os.dims[i];
      for (int i = axis + 1; i < os.size; ++i) inner *= os.dims[i];
      struct Part { const void* x; MoveGeom g; };
      std::vector<Part> parts;
      for (V in : v->in) {
        int xdt; const void* x = operand(in, &xdt, odt);
        if (xdt != odt) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': concat inputs have different storage types");
        odla_value_shape is = resolve(in)->kind == OP_CONST ? in->type.shape : shape(in);
        MoveGeom g{};
        g.rank = 3;
        g.oshape[0] = outer; g.oshape[1] = is.dims[axis]; g.oshape[2] = inner;
        g.istride[0] = is.dims[axis] * inner; g.istride[1] = inner; g.istride[2] = 1;
        g.ostride[0] = os.dims[axis] * inner; g.ostride[1] = inner; g.ostride[2] = 1;
        g.out_offset = off * inner;
        off += is.dims[axis];
        parts.push_back({x, g});
      }
      int esz = storage_size(odt);
      add_launch("concat", v, 0, 2 * out_bytes, [=](cudaStream_t s) {
        for (auto& p : parts) { int r = move(p.g, esz, p.x, y, s); if (r) return r; }
        return 0;
      });
      p_->launches.back().n_kernels = (int)parts.size();
      return ODLA_SUCCESS;
    }
    case OP_RESIZE: {
      int xdt; const void* x = operand(v->in[0], &xdt, odt);
      odla_value_shape xs = shape(v->in[0]);
      // No layout argument exists: a tensor whose dim 1 is unchanged while dim 2 or 3 changes is NCHW.
      bool nchw = xs.dims[1] == os.dims[1] && (xs.dims[2] != os.dims[2] || xs.dims[3] != os.dims[3]);
      if (!nchw && xs.dims[3] != os.dims[3]) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': resize must keep the channel extent");
      if (xs.dims[0] != os.dims[0]) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': resize must keep the batch extent");
      int N = (int)xs.dims[0], H = (int)(nchw ? xs.dims[2] : xs.dims[1]), W = (int)(nchw ? xs.dims[3] : xs.dims[2]), C = (int)(nchw ? xs.dims[1] : xs.dims[3]);
      int P = (int)(nchw ? os.dims[2] : os.dims[1]), Q = (int)(nchw ? os.dims[3] : os.dims[2]);
      int esz = storage_size(odt);
      add_launch("resize", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return resize_nearest(esz, x, y, N, H, W, C, P, Q, !nchw, s); });
      return ODLA_SUCCESS;
    }
    case OP_GATHER: {
      int xdt, idt; const void* x = operand(v->in[0], &xdt, odt); const void* idx = operand(v->in[1], &idt);
      if (idt != DT_S32 && idt != DT_S64) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + v->name + "': gather indices must be int32 or int64");
      odla_value_shape xs = resolve(v->in[0])->kind == OP_CONST ? v->in[0]->type.shape : shape(v->in[0]);
      int axis = (int)v->ia[0];
      int64_t outer = 1, inner = 1, adim = xs.dims[axis];
      for (int i = 0; i < axis; ++i) outer *= xs.dims[i];
      for (int i = axis + 1; i < xs.size; ++i) inner *= xs.dims[i];
      int64_t n_idx = resolve(v->in[1])->kind == OP_CONST ? numel(v->in[1]->type.shape) : count(v->in[1]);
      int esz = storage_size(odt);
      add_launch("gather", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return gather(esz, x, idx, idt, y, outer, adim, n_idx, inner, s); });
      return ODLA_SUCCESS;
    }
    case OP_SLICE: {
      int xdt; const void* x = operand(v->in[0], &xdt, odt);
      odla_value_shape xs = shape(v->in[0]);
      if (xs.size > 8) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': rank above 8");
      MoveGeom g{};
      g.rank = xs.size;
      int64_t a = 1, oa = 1;
      for (int i = xs.size - 1; i >= 0; --i) {
        g.oshape[i] = os.dims[i];
        g.istride[i] = a * v->ia[xs.size + i];
        g.in_offset += v->ia[i] * a;
        g.ostride[i] = oa;
        a *= xs.dims[i]; oa *= os.dims[i];
      }
      int esz = storage_size(odt);
      add_launch("slice", v, 0, 2 * out_bytes, [=](cudaStream_t s) { return move(g, esz, x, y, s); });
      return ODLA_SUCCESS;
    }
    case OP_NMS: {
      int bdt, sdt; const void* boxes = operand(v->in[0], &bdt); const void* scores = operand(v->in[1], &sdt);
      const auto& ss = v->in[1]->type.shape;
      const int B = (int)ss.dims[0], C = (int)ss.dims[1], N = (int)ss.dims[2], rows = (int)os.dims[0];
      const int max_sel = (int)std::min<int64_t>(v->ia[0] > 0 ? v->ia[0] : rows, std::max(N, 1));
      if ((int64_t)B * C > 1024) return fail(ODLA_UNSUPPORTED_OP, "'" + v->name + "': more than 1024 (batch, class) pairs");
      int* scratch = nullptr;
      if (cudaMalloc((void**)&scratch, sizeof(int) * ((size_t)B * C * std::max(max_sel, 1) + (size_t)B * C)) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
      p_->extra_allocs.push_back(scratch);
      int* cnt = scratch + (size_t)B * C * std::max(max_sel, 1);
      const float iou = v->fa[0], thr = v->fa[1];
      const int out64 = odt == DT_S64;
      add_launch("nms", v, 0, tensor_bytes(v->in[0]) + tensor_bytes(v->in[1]) + out_bytes,
                 [=](cudaStream_t s) { return nms(B, C, N, max_sel, iou, thr, bdt, boxes, sdt, scores, rows, out64, y, scratch, cnt, s); });
      p_->launches.back().n_kernels = 2;
      return ODLA_SUCCESS;
    }
    case OP_POSTPROCESS: {
      const int cls = (int)v->ia[0];
      int wdt, hdt; const void* iw = operand(v->in[0], &wdt); const void* ih = operand(v->in[1], &hdt);
      if (wdt != DT_S32 || hdt != DT_S32) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + v->name + "': the image extents are 32-bit integers");
      struct Heads { const void* p[3]; int S[3], nchw[3]; } hd{};
      int hdt0 = -1;
      for (int i = 0; i < 3; ++i) {
        int dt; hd.p[i] = operand(v->in[2 + i], &dt);
        if (hdt0 >= 0 && dt != hdt0) return fail(ODLA_UNSUPPORTED_DATATYPE, "'" + v->name + "': heads of different storage types");
        hdt0 = dt;
        const auto& s = v->in[2 + i]->type.shape;
        hd.nchw[i] = s.dims[2] == s.dims[3] && s.dims[1] == 3 * (cls + 5) ? 1 : 0;
        hd.S[i] = (int)s.dims[2];
      }
      const int N = 3 * (hd.S[0] * hd.S[0] + hd.S[1] * hd.S[1] + hd.S[2] * hd.S[2]), per_class = N / 169;
      static const unsigned anchors[18] = {10, 13, 16, 30, 33, 23, 30, 61, 62, 45, 59, 119, 116, 90, 156, 198, 373, 326};  // yolo_anchors.txt
      const unsigned* anc = (const unsigned*)upload(anchors, sizeof(anchors));
      // scratch: boxes [N,4], scores [cls,N], selections, counts, fp32 result (when the storage type is narrower)
      const size_t f_boxes = (size_t)N * 4, f_scores = (size_t)cls * N, f_info = (size_t)cls * per_class * 5;
      char* scratch = nullptr;
      const size_t bytes = 4 * (f_boxes + f_scores + f_info + (size_t)cls * per_class + 2 * (size_t)cls);
      if (!anc || cudaMalloc((void**)&scratch, bytes) != cudaSuccess) return fail(ODLA_MEM_ERROR, "scratch allocation failed");
      p_->extra_allocs.push_back(scratch);
      float* boxes = (float*)scratch; float* scores = boxes + f_boxes; float* info32 = scores + f_scores;
      int* sel = (int*)(info32 + f_info); int* cnt = sel + (size_t)cls * per_class; unsigned* num = (unsigned*)(cnt + cls);
      p_->pp_counts[v] = num;
      const int dt = hdt0; const int64_t n_info = (int64_t)f_info;
      add_launch("postprocess", v, 0, tensor_bytes(v->in[2]) + tensor_bytes(v->in[3]) + tensor_bytes(v->in[4]) + out_bytes, [=](cudaStream_t s) {
        float* info = odt == DT_F32 ? (float*)y : info32;
        int rc = yolo_postprocess(cls, hd.S, hd.p, dt, hd.nchw, anc, (const unsigned*)iw, (const unsigned*)ih, boxes, scores, sel, cnt, info, num, s);
        if (rc || odt == DT_F32) return rc;
        return convert(DT_F32, odt, info32, y, n_info, s);
      });
      p_->launches.back().n_kernels = 5 + (odt == DT_F32 ? 0 : 1);
      return ODLA_SUCCESS;
    }
    case OP_POSTPROCESS_NUM: {
      auto it2 = p_->pp_counts.find(v->in[0]);
      if (it2 == p_->pp_counts.end()) return fail(ODLA_INTERNAL_LOGIC_ERR, "'" + v->name + "': its PostProcess has not been planned");
      const void* src = it2->second;
      const size_t nb = (size_t)count(v) * 4;
      add_launch("postprocess_num", v, 0, 2.0 * nb, [=](cudaStream_t s) { return cudaMemcpyAsync(y, src, nb, cudaMemcpyDeviceToDevice, s) == cudaSuccess ? 0 : -2; });
      p_->launches.back().n_kernels = 0;
      return ODLA_SUCCESS;
    }
    case OP_CAST: {
      int xdt; const void* x = operand(v->in[0], &xdt);
      int64_t n = count(v);
      add_launch("cast", v, 0, tensor_bytes(v->in[0]) + out_bytes, [=](cudaStream_t s) { return convert(xdt, odt, x, y, n, s); });
      return ODLA_SUCCESS;
    }
    default: break;
  }
  return fail(ODLA_UNSUPPORTED_OP, std::string("no kernel for op '") + op_name(v->kind) + "' (value '" + v->name + "')");
}

odla_status Builder::emit() {
  // argument conversions first
  for (auto& io : p_->inputs) {
    if (io.stage == io.slot) continue;
    const void* src = p_->arena + io.stage; void* dst = p_->arena + io.slot;
    int sdt = api_dt(io.v->type.element_type), ddt = dt_[io.v];
    int64_t n = count(io.v);
    add_launch("convert_in", io.v, 0, (double)io.api_bytes + (double)n * storage_size(ddt), [=](cudaStream_t s) { return convert(sdt, ddt, src, dst, n, s); });
  }
  for (auto& it : items_) {
    odla_status st = it.fused ? emit_fused(it) : emit_plain(it);
    if (st != ODLA_SUCCESS) return st;
    if (!err_.empty()) return err_status_;
  }
  for (auto& io : p_->outputs) {
    if (io.const_host || io.stage == io.slot) continue;
    V r = resolve(io.v);
    const void* src = p_->arena + io.slot; void* dst = p_->arena + io.stage;
    int sdt = dt_[r], ddt = api_dt(io.v->type.element_type);
    int64_t n = count(io.v);
    Launch l; l.op = "convert_out"; l.name = io.v->name; l.bytes = (double)io.api_bytes + (double)n * storage_size(sdt);
    auto pi = pitch_.find(r);
    if (pi != pitch_.end()) {
      const auto& sh = r->type.shape;
      const int64_t K = sh.dims[sh.size - 1], Kp = pi->second, rows = n / K;
      l.fn = [=](cudaStream_t s) { return convert_rows(sdt, ddt, src, dst, rows, K, Kp, s); };
    } else
    l.fn = [=](cudaStream_t s) { return convert(sdt, ddt, src, dst, n, s); };
    p_->launches.push_back(std::move(l));
  }
  return ODLA_SUCCESS;
}

odla_status Builder::run() {
  for (V a : c_->args) if (api_dt(a->type.element_type) < 0) return fail(ODLA_UNSUPPORTED_DATATYPE, "argument '" + a->name + "' has an unsupported element type");
  odla_status s = analyse();
  if (s != ODLA_SUCCESS) return s;
  s = place();
  if (s != ODLA_SUCCESS) return s;
  s = emit();
  if (s != ODLA_SUCCESS) return s;
  return err_.empty() ? ODLA_SUCCESS : err_status_;
}

// dim 0 can be split across GPUs only when no op mixes rows of the batch.
bool graph_shardable(_odla_computation* c, int64_t* batch_out) {
  if (c->args.empty()) return false;
  int64_t B = c->args[0]->type.shape.size ? c->args[0]->type.shape.dims[0] : 1;
  *batch_out = B;
  if (B <= 0) return false;  // an empty batch cannot be split
  for (V a : c->args) if (a->type.shape.size == 0 || a->type.shape.dims[0] != B) return false;
  std::map<V, bool> cb;
  for (auto& n : c->nodes) {
    V v = n.get();
    bool b = v->kind == OP_ARG;
    for (auto i : v->in) if (i && cb[i]) b = true;
    cb[v] = b;
    if (!b) continue;
    const auto& s = v->type.shape;
    if (s.size == 0 || s.dims[0] % B != 0) return false;
    // An operand that does not depend on the arguments (a constant, or a function of constants) but spans the whole
    // batch extent would have to be offset by the shard's first row; such graphs run unsharded instead.
    auto spans_batch = [&](V o) {
      if (!o || cb[o]) return false;
      const auto& os = o->type.shape;
      return s.dims[0] > 1 && os.size == s.size && os.dims[0] == s.dims[0];
    };
    if (v->kind == OP_BINARY || v->kind == OP_CONCAT)
      for (auto i : v->in) if (spans_batch(i)) return false;
    // (a Gemm's right operand has the reduction, not the batch, as its first dimension -- a [2048, 1000] classifier
    // under a batch of 2048 is not a constant that spans the batch; its left operand and its addend are aligned with the rows)
    if (v->kind == OP_GEMM && (spans_batch(v->in[0]) || (v->in.size() > 2 && spans_batch(v->in[2])))) return false;
    switch (v->kind) {
      case OP_NMS: case OP_POSTPROCESS: case OP_POSTPROCESS_NUM: return false;   // rows of the result are not rows of the batch
      case OP_TRANSPOSE: if (v->ia[0] != 0) return false; break;
      case OP_SOFTMAX: if (v->ia[0] == 0) return false; break;
      case OP_REDUCE_MEAN: for (size_t k = 1; k < v->ia.size(); ++k) if (v->ia[k] == 0) return false; break;
      case OP_CONCAT: if (v->ia[0] == 0) return false; break;
      case OP_LAYERNORM: if ((int)v->ia[0] >= s.size) return false; break;
      case OP_SLICE: if (v->ia[0] != 0 || s.dims[0] != v->in[0]->type.shape.dims[0]) return false; break;
      case OP_GATHER: if (cb[v->in[0]] && v->ia[0] == 0) return false; break;
      case OP_QUANTIZE: case OP_DEQUANTIZE: if (numel(v->in[1]->type.shape) > 1 && v->ia[0] == 0) return false; break;
      case OP_GEMM: if (v->in[1] && cb[v->in[1]] && v->type.shape.size == 2) return false; if (v->ia[0] && v->type.shape.size == 2) return false; break;
      case OP_RESHAPE: {
        // rows stay whole only if the per-row element count is the same integer before and after
        const auto& is = v->in[0]->type.shape;
        if (is.size == 0 || is.dims[0] % B != 0) return false;
        break;
      }
      default: break;
    }
  }
  for (V o : c->outs) if (cb[o] && (o->type.shape.size == 0 || o->type.shape.dims[0] % B != 0)) return false;
  return true;
}

}  // namespace

void destroy_replicas(std::vector<Replica>& reps) {
  for (auto& r : reps) {
    cudaSetDevice(r.device);
    r.plan.reset();
    if (r.host_status) cudaFreeHost(r.host_status);
    if (r.ev_begin) cudaEventDestroy(r.ev_begin);
    if (r.ev_end) cudaEventDestroy(r.ev_end);
    if (r.stream) cudaStreamDestroy(r.stream);
  }
  reps.clear();
}

// One replica's share of an execute: which GPU, which rows of dim 0.
struct Shard { int device; int64_t start, rows; };

// How `run_batch` rows of a graph are split: an even split over the GPUs (the first `run_batch % G` GPUs take one row
// more), and within a GPU over S sub-batches (ODLA_BATCHES_PER_STEP), each with its own stream, so that one
// sub-batch's host-to-device copy runs under another's kernels.  Needs no device: the arithmetic is tested on the host.
static std::vector<Shard> shard_layout(_odla_computation* c, int visible, int64_t B, int64_t run_batch) {
  int want = c->n_gpus > 0 ? c->n_gpus : visible;
  int G = c->shardable ? (int)std::min<int64_t>(std::min(want, visible), std::max<int64_t>(run_batch, 1)) : 1;
  if (G < 1) G = 1;
  int S = c->sub_batches > 0 ? c->sub_batches : (getenv("ODLA_B200_SUBBATCHES") ? atoi(getenv("ODLA_B200_SUBBATCHES")) : 1);
  if (!c->shardable || S < 1) S = 1;
  while (S > 1 && (int64_t)G * S > run_batch) --S;
  const int devices = G;
  G *= S;
  // Within a GPU the sub-batches grow geometrically by `growth` (1 = even), so that each one's input copy still fits
  // under the kernels of the smaller one before it while the first, exposed, copy is short.
  // Measured on ResNet-50 (B = 256, inputs 300 KB and outputs 4 KB per image): two sub-batches of 64 and 192 rows beat
  // 128 + 128 by 4 %; when the outputs are the larger transfer the last sub-batch's copy-out is the exposed one and
  // the split stays even.
  double growth = 1.0;
  {
    double in_bytes = 0, out_bytes = 0;
    for (auto a : c->args) in_bytes += (double)numel(a->type.shape) * elem_size(a->type.element_type);
    for (auto o : c->outs) out_bytes += (double)numel(o->type.shape) * elem_size(o->type.element_type);
    if (in_bytes > 4 * out_bytes) growth = 3.0;
    if (getenv("ODLA_B200_SUBBATCH_GROWTH")) growth = atof(getenv("ODLA_B200_SUBBATCH_GROWTH"));
  }
  std::vector<int64_t> rows((size_t)G, 0);
  for (int d = 0; d < devices; ++d) {
    const int64_t share = run_batch / devices + (d < run_batch % devices ? 1 : 0);
    int64_t* r = &rows[(size_t)d * S];
    double wsum = 0, w = 1;
    for (int k = 0; k < S; ++k) { wsum += w; w *= growth > 0 ? growth : 1.0; }
    int64_t given = 0;
    w = 1;
    for (int k = 0; k < S; ++k) {
      r[k] = k + 1 == S ? share - given : std::max<int64_t>(1, (int64_t)(share * (w / wsum)));
      if (given + r[k] > share - (S - 1 - k)) r[k] = std::max<int64_t>(1, share - (S - 1 - k) - given);  // leave a row for each later sub-batch
      given += r[k];
      w *= growth > 0 ? growth : 1.0;
    }
    if (growth == 1.0) for (int k = 0; k < S; ++k) r[k] = share / S + (k < share % S ? 1 : 0);
  }
  std::vector<Shard> out((size_t)G);
  int64_t start = 0;
  for (int i = 0; i < G; ++i) {
    out[(size_t)i].device = (c->first_device + i / S) % std::max(visible, 1);
    out[(size_t)i].rows = c->shardable ? rows[(size_t)i] : B;
    out[(size_t)i].start = start;
    start += out[(size_t)i].rows;
  }
  return out;
}

// Builds the replicas (streams, arenas, constant pools, launch lists) that run `run_batch` rows of a graph
// recorded with `B` rows in dim 0.
static odla_status build_replicas(_odla_computation* c, int visible, int64_t B, int64_t run_batch, std::vector<Replica>& reps) {
  const std::vector<Shard> layout = shard_layout(c, visible, B, run_batch);
  const int G = (int)layout.size();
  reps.resize((size_t)G);
  // any failure below releases what the replicas built so far own (streams, events, pinned status words, plans)
  struct Guard { std::vector<Replica>& r; bool armed = true; ~Guard() { if (armed) destroy_replicas(r); } } guard{reps};
  for (int i = 0; i < G; ++i) {
    Replica& r = reps[i];
    r.device = layout[(size_t)i].device;
    r.shard_batch = layout[(size_t)i].rows;
    r.shard_start = layout[(size_t)i].start;
    B2_CUDA("setdevice", cudaSetDevice(r.device), ODLA_FAILURE);
    B2_CUDA("stream", cudaStreamCreateWithFlags(&r.stream, cudaStreamNonBlocking), ODLA_FAILURE);
    B2_CUDA("event", cudaEventCreate(&r.ev_begin), ODLA_FAILURE);
    B2_CUDA("event", cudaEventCreate(&r.ev_end), ODLA_FAILURE);
    B2_CUDA("alloc", cudaMallocHost((void**)&r.host_status, 256), ODLA_MEM_ERROR);
    memset(r.host_status, 0, 256);
    r.plan = std::make_unique<Plan>();
    r.plan->device = r.device;
    r.plan->batch = r.shard_batch;
    Builder b(c, r.plan.get(), c->shardable ? B : r.shard_batch, r.shard_batch, r.shard_start);
    odla_status s = b.run();
    if (s != ODLA_SUCCESS) return s;
    B2_INFO("GPU %d: rows [%lld,%lld), %zu launches, arena %.1f MiB, constants %.1f MiB", r.device, (long long)r.shard_start,
            (long long)(r.shard_start + r.shard_batch), r.plan->launches.size(), r.plan->arena_bytes / 1048576.0, r.plan->const_bytes / 1048576.0);
  }
  // peer access between every pair, for device-resident outputs gathered over NVLink
  for (int i = 0; i < G; ++i)
    for (int j = 0; j < G; ++j) {
      if (i == j || reps[i].device == reps[j].device) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, reps[i].device, reps[j].device);
      if (can) { cudaSetDevice(reps[i].device); cudaError_t e = cudaDeviceEnablePeerAccess(reps[j].device, 0); if (e != cudaSuccess) cudaGetLastError(); }
    }
  guard.armed = false;
  return ODLA_SUCCESS;
}

odla_status ensure_planned(_odla_computation* c) {
  std::lock_guard<std::recursive_mutex> plan_lock(c->plan_mutex);
  if (c->planned) return ODLA_SUCCESS;
  int visible = visible_devices();
  if (visible <= 0) {
    B2_ERR("no CUDA device is visible: libodla_b200 has no CPU fallback");
    return ODLA_FAILURE;
  }
  if (odla_status qs = apply_quant_table(c)) return qs;
  destroy_replicas(c->replicas);
  for (auto& kv : c->batch_replicas) destroy_replicas(kv.second);
  c->batch_replicas.clear();
  for (auto& lane : c->lanes) {
    for (auto& kv : lane->batch_replicas) destroy_replicas(kv.second);
    lane->batch_replicas.clear();
  }
  int64_t B = 1;
  c->shardable = graph_shardable(c, &B);
  c->graph_batch = B;
  odla_status s = build_replicas(c, visible, B, B, c->replicas);
  if (s != ODLA_SUCCESS) return s;
  c->planned = true;
  return ODLA_SUCCESS;
}

// The replicas that run `run_batch` rows (ODLA_RUN_BATCH_SIZE) on lane `lane`; plans for other batch sizes than the
// recorded one, and every plan of a lane other than 0, are built on first use and kept.
odla_status replicas_for_batch(_odla_computation* c, int64_t run_batch, int lane, std::vector<Replica>** out) {
  std::lock_guard<std::recursive_mutex> plan_lock(c->plan_mutex);
  odla_status s = ensure_planned(c);
  if (s != ODLA_SUCCESS) return s;
  const bool whole = run_batch <= 0 || run_batch == c->graph_batch;
  if (whole && lane == 0) { *out = &c->replicas; return ODLA_SUCCESS; }
  if (!whole) {
    if (!c->shardable) { B2_ERR("ODLA_RUN_BATCH_SIZE needs a graph whose dim 0 is an independent batch"); return ODLA_UNSUPPORTED_OP; }
    if (run_batch > c->graph_batch) { B2_ERR("ODLA_RUN_BATCH_SIZE %lld exceeds the recorded batch %lld", (long long)run_batch, (long long)c->graph_batch); return ODLA_INVALID_PARAM; }
  }
  if (lane < 0 || lane > (int)c->lanes.size()) { B2_ERR("context lane %d does not exist", lane); return ODLA_INTERNAL_LOGIC_ERR; }
  std::map<int64_t, std::vector<Replica>>& plans = lane == 0 ? c->batch_replicas : c->lanes[(size_t)lane - 1]->batch_replicas;
  const int64_t rows = whole ? c->graph_batch : run_batch;
  auto it = plans.find(rows);
  if (it == plans.end()) {
    std::vector<Replica> reps;
    s = build_replicas(c, visible_devices(), c->graph_batch, rows, reps);
    if (s != ODLA_SUCCESS) return s;
    it = plans.emplace(rows, std::move(reps)).first;
  }
  *out = &it->second;
  return ODLA_SUCCESS;
}

namespace {
// Which device owns `p`, or -1 for host memory.
int pointer_device(const void* p) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return -1; }
  if (at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) return at.device;
  return -1;
}
int run_launches(Replica& r, _odla_context* ctx, bool use_graph, long long* n_launched) {
  Plan& p = *r.plan;
  if (ctx->profiling) {
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    for (auto& l : p.launches) {
      cudaEventRecord(a, r.stream);
      int rc = inject_fault("launch") ? -2 : l.fn(r.stream);
      cudaEventRecord(b, r.stream);
      if (rc) { cudaEventDestroy(a); cudaEventDestroy(b); return rc; }
      cudaEventSynchronize(b);
      float ms = 0; cudaEventElapsedTime(&ms, a, b);
      l.prof_ms += ms; l.prof_n++;
      *n_launched += l.n_kernels;
    }
    cudaEventDestroy(a); cudaEventDestroy(b);
    return 0;
  }
  if (ctx->range_profiling) {
    // plain launches, each followed by a min / max pass over what it left in memory (allocated on first use)
    auto stats_for = [&](unsigned*& st, int64_t channels) {
      if (st) return true;
      if (cudaMalloc((void**)&st, sizeof(unsigned) * (size_t)(2 + 2 * channels)) != cudaSuccess) { st = nullptr; cudaGetLastError(); return false; }
      p.extra_allocs.push_back(st);
      return range_stats_reset(st, channels, r.stream) == 0;
    };
    p.input_range_stats.resize(p.inputs.size(), nullptr);
    for (size_t i = 0; i < p.inputs.size(); ++i) {
      const auto& io = p.inputs[i];
      const auto& sl = p.slots[io.v];
      if (sl.dt != DT_F32 && sl.dt != DT_F16 && sl.dt != DT_BF16) continue;
      const auto& sh = io.v->type.shape;
      const int64_t ch = sh.size ? sh.dims[sh.size - 1] : 1, n = sl.bytes / storage_size(sl.dt);
      // an argument that is converted on the device is measured in its API type at the staging slot
      const bool staged = io.stage != io.slot;
      const int dt = staged ? DT_F32 : sl.dt;
      const int64_t cnt = staged ? io.api_bytes / 4 : n;
      if (staged && io.v->type.element_type != ODLA_FLOAT32) continue;
      if (!stats_for(p.input_range_stats[i], ch)) return -2;
      if (range_minmax(dt, p.arena + io.stage, cnt, ch, p.input_range_stats[i], r.stream)) return -2;
    }
    for (auto& l : p.launches) {
      int rc = l.fn(r.stream);
      if (rc) return rc;
      *n_launched += l.n_kernels;
      if (!l.out_ptr || (l.out_dt != DT_F32 && l.out_dt != DT_F16 && l.out_dt != DT_BF16)) continue;
      if (!stats_for(l.range_stats, l.out_channels)) return -2;
      if (range_minmax(l.out_dt, l.out_ptr, l.out_count, l.out_channels, l.range_stats, r.stream)) return -2;
    }
    return 0;
  }
  if (use_graph && !p.graph && !p.graph_failed && !p.launches.empty()) {
    cudaGraph_t g = nullptr;
    bool ok = cudaStreamBeginCapture(r.stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
    if (ok) {
      int rc = 0;
      for (auto& l : p.launches) { rc = l.fn(r.stream); if (rc) break; }
      cudaError_t e = cudaStreamEndCapture(r.stream, &g);
      ok = rc == 0 && e == cudaSuccess && g;
      if (ok) ok = cudaGraphInstantiate(&p.graph, g, 0) == cudaSuccess;
      if (g) cudaGraphDestroy(g);
    }
    if (!ok) { cudaGetLastError(); p.graph = nullptr; p.graph_failed = true; B2_WARN("CUDA graph capture refused on GPU %d; using plain launches", r.device); }
  }
  if (inject_fault("launch")) return -2;
  if (use_graph && p.graph) {
    if (cudaGraphLaunch(p.graph, r.stream) != cudaSuccess) return -2;
    for (auto& l : p.launches) *n_launched += l.n_kernels;
    return 0;
  }
  for (auto& l : p.launches) {
    int rc = l.fn(r.stream);
    if (rc) return rc;
    *n_launched += l.n_kernels;
  }
  return 0;
}
}  // namespace

// Enqueues one replica's share of an execute on its own stream: input copies, the launch list, output copies, the
// status read-back and the two events that time it.  Nothing here waits for the GPU.
static odla_status enqueue_replica(Replica& r, size_t index, _odla_context* ctx, bool use_graph, long long* launched) {
  Plan& p = *r.plan;
  auto fail_here = [&](odla_status s, const char* what) { B2_ERR("GPU %d: %s failed", r.device, what); return s; };
  if (cudaSetDevice(r.device) != cudaSuccess) return fail_here(ODLA_FAILURE, "cudaSetDevice");
  cudaEventRecord(r.ev_begin, r.stream);
  for (auto& io : p.inputs) {
    const char* src = (const char*)ctx->in.find(io.v)->second + io.user_offset;  // every argument is bound (checked by the caller)
    int pd = pointer_device(src);
    cudaError_t e;
    if (inject_fault("h2d")) e = cudaErrorUnknown;
    else if (pd >= 0 && pd != r.device) e = cudaMemcpyPeerAsync(p.arena + io.stage, r.device, src, pd, (size_t)io.api_bytes, r.stream);
    else e = cudaMemcpyAsync(p.arena + io.stage, src, (size_t)io.api_bytes, pd >= 0 ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, r.stream);
    if (e != cudaSuccess) return fail_here(ODLA_FAILURE, "input copy");
  }
  // With contexts on several lanes in flight, this execute's kernels start behind the kernels of the execute that was
  // enqueued before it on this GPU (its input copies above do not wait): interleaving two executes layer by layer
  // would only evict each other's activations from L2.
  _odla_computation* c = ctx->comp;
  const bool chained = c && c->multi_lane.load() && !ctx->profiling && !ctx->range_profiling;
  int rc;
  if (chained) {
    _odla_computation::ChainLink* link;
    {
      std::lock_guard<std::mutex> map_lock(c->chain_mutex);
      auto& slot = c->chain[r.device];
      if (!slot) slot.reset(new _odla_computation::ChainLink());
      link = slot.get();
    }
    std::lock_guard<std::mutex> order(link->enqueue);   // wait + launches + record of one execute stay together
    if (!link->last) {
      if (cudaEventCreateWithFlags(&link->last, cudaEventDisableTiming) != cudaSuccess) return fail_here(ODLA_FAILURE, "event creation");
    } else if (cudaStreamWaitEvent(r.stream, link->last, 0) != cudaSuccess) return fail_here(ODLA_FAILURE, "cudaStreamWaitEvent");
    rc = run_launches(r, ctx, use_graph, launched);
    cudaEventRecord(link->last, r.stream);
  } else rc = run_launches(r, ctx, use_graph, launched);
  if (rc) return fail_here(ODLA_FAILURE, "kernel launch");
  for (auto& io : p.outputs) {
    auto bound = ctx->out.find(io.v);
    if (bound == ctx->out.end()) continue;
    if (!io.per_shard && index != 0) continue;  // a value that does not depend on the batch: the first replica writes it
    char* dst = (char*)bound->second + io.user_offset;
    int pd = pointer_device(dst);
    cudaError_t e;
    if (inject_fault("d2h")) e = cudaErrorUnknown;
    else if (io.const_host) {
      e = cudaMemcpyAsync(dst, io.const_host, (size_t)io.api_bytes, pd >= 0 ? cudaMemcpyHostToDevice : cudaMemcpyHostToHost, r.stream);
    } else if (pd >= 0 && pd != r.device) {
      e = inject_fault("peer") ? cudaErrorUnknown : cudaMemcpyPeerAsync(dst, pd, p.arena + io.stage, r.device, (size_t)io.api_bytes, r.stream);
    } else e = cudaMemcpyAsync(dst, p.arena + io.stage, (size_t)io.api_bytes, pd >= 0 ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost, r.stream);
    if (e != cudaSuccess) return fail_here(ODLA_FAILURE, "output copy");
  }
  cudaMemcpyAsync(r.host_status, p.status, sizeof(int) * 4, cudaMemcpyDeviceToHost, r.stream);
  cudaEventRecord(r.ev_end, r.stream);
  return ODLA_SUCCESS;
}

odla_status execute(_odla_computation* c, _odla_context* ctx) {
  for (V a : c->args)
    if (!ctx->in.count(a)) { B2_ERR("argument '%s' is not bound", a->name.c_str()); return ODLA_INVALID_PARAM; }
  odla_status result = ODLA_SUCCESS;
  long long launched = 0;
  std::vector<Replica>* reps_p = nullptr;
  if (odla_status rs = replicas_for_batch(c, ctx->run_batch, ctx->lane, &reps_p)) return rs;
  std::vector<Replica>& reps = *reps_p;
  std::vector<char> started(reps.size(), 0);
  // Enqueue everything on every GPU, then wait.  With more than one GPU each GPU is fed by a host thread of its own:
  // a copy from pageable host memory blocks the calling thread until it is staged, and eight GPUs fed from one
  // thread would start one after the other.  A failure stops that GPU's enqueuing; what started is drained below.
  bool several_devices = false;
  for (auto& r : reps) if (r.device != reps[0].device) several_devices = true;
  if (several_devices && !getenv("ODLA_B200_INJECT") && !ctx->profiling && !getenv("ODLA_B200_SERIAL_ENQUEUE")) {
    std::map<int, std::vector<size_t>> by_device;
    for (size_t i = 0; i < reps.size(); ++i) by_device[reps[i].device].push_back(i);
    std::vector<std::thread> workers;
    std::vector<odla_status> st(by_device.size(), ODLA_SUCCESS);
    std::vector<long long> nl(by_device.size(), 0);
    size_t w = 0;
    for (auto& kv : by_device) {
      const std::vector<size_t>* idx = &kv.second;
      odla_status* s_out = &st[w];
      long long* n_out = &nl[w];
      ++w;
      workers.emplace_back([&, idx, s_out, n_out] {
        for (size_t i : *idx) {
          started[i] = 1;
          *s_out = enqueue_replica(reps[i], i, ctx, c->use_graph, n_out);
          if (*s_out != ODLA_SUCCESS) break;
        }
      });
    }
    for (auto& t : workers) t.join();
    for (size_t k = 0; k < st.size(); ++k) { if (st[k] != ODLA_SUCCESS && result == ODLA_SUCCESS) result = st[k]; launched += nl[k]; }
  } else {
    for (size_t i = 0; i < reps.size() && result == ODLA_SUCCESS; ++i) {
      started[i] = 1;
      result = enqueue_replica(reps[i], i, ctx, c->use_graph, &launched);
    }
  }
  if (result != ODLA_SUCCESS) cudaGetLastError();
  float worst = 0.f;
  for (size_t i = 0; i < reps.size(); ++i) {
    if (!started[i]) continue;
    Replica& r = reps[i];
    cudaSetDevice(r.device);
    cudaError_t e = cudaStreamSynchronize(r.stream);
    if (e != cudaSuccess) { B2_ERR("GPU %d: stream synchronise failed: %s", r.device, cudaGetErrorString(e)); if (result == ODLA_SUCCESS) result = ODLA_FAILURE; continue; }
    if (result == ODLA_SUCCESS) {
      float ms = 0.f;
      if (cudaEventElapsedTime(&ms, r.ev_begin, r.ev_end) == cudaSuccess) worst = std::max(worst, ms); else cudaGetLastError();
      if (r.host_status[0] != 0) {
        B2_ERR("GPU %d: a bounded wait inside a kernel expired (code %d, detail %d)", r.device, r.host_status[0], r.host_status[1]);
        cudaMemsetAsync(r.plan->status, 0, kStatusBytes, r.stream);
        cudaStreamSynchronize(r.stream);
        result = ODLA_TIMEOUT;
      }
    }
  }
  if (result == ODLA_SUCCESS) { ctx->last_ms = worst; ctx->last_launches = launched; }
  return result;
}

}  // namespace b200

using namespace b200;
// The whole-batch replicas of the lane `ctx` executes on (lane 0's while that lane has built none yet).
static std::vector<Replica>& context_replicas(odla_context ctx) {
  _odla_computation* c = ctx->comp;
  std::lock_guard<std::recursive_mutex> plan_lock(c->plan_mutex);
  if (ctx->lane > 0 && ctx->lane <= (int)c->lanes.size()) {
    auto& plans = c->lanes[(size_t)ctx->lane - 1]->batch_replicas;
    auto it = plans.find(c->graph_batch);
    if (it != plans.end()) return it->second;
  }
  return c->replicas;
}
extern "C" {
float odla_b200_LastExecuteDeviceMs(odla_context ctx) { return ctx ? ctx->last_ms : -1.f; }
long long odla_b200_LastExecuteLaunches(odla_context ctx) { return ctx ? ctx->last_launches : 0; }
odla_status odla_b200_SetProfiling(odla_context ctx, int enabled) {
  if (!ctx) return ODLA_INVALID_PARAM;
  ctx->profiling = enabled != 0;
  if (enabled && ctx->comp)
    for (auto& r : context_replicas(ctx))
      if (r.plan) for (auto& l : r.plan->launches) { l.prof_ms = 0; l.prof_n = 0; }
  return ODLA_SUCCESS;
}
int odla_b200_GetProfile(odla_context ctx, odla_b200_profile_entry* entries, int capacity) {
  if (!ctx || !ctx->comp) return 0;
  std::vector<Replica>& reps = context_replicas(ctx);
  if (reps.empty() || !reps[0].plan) return 0;
  auto& ls = reps[0].plan->launches;
  for (int i = 0; i < (int)ls.size() && i < capacity && entries; ++i) {
    memset(&entries[i], 0, sizeof(entries[i]));
    snprintf(entries[i].op, sizeof(entries[i].op), "%s", ls[i].op.c_str());
    snprintf(entries[i].name, sizeof(entries[i].name), "%s", ls[i].name.c_str());
    entries[i].total_ms = ls[i].prof_ms; entries[i].launches = ls[i].prof_n;
    entries[i].flops = ls[i].flops; entries[i].bytes = ls[i].bytes;
  }
  return (int)ls.size();
}
odla_status odla_b200_SetRangeProfiling(odla_context ctx, int enabled) {
  if (!ctx) return ODLA_INVALID_PARAM;
  ctx->range_profiling = enabled != 0;
  return ODLA_SUCCESS;
}
int odla_b200_GetQuantTable(odla_context ctx, odla_value_quant_info* records, int capacity) {
  if (!ctx || !ctx->comp) return 0;
  _odla_computation* c = ctx->comp;
  // name -> (min, max, per-channel min / max), merged over every replica (each saw its own rows of the batch)
  struct R { float mn = 3.402823466e+38f, mx = -3.402823466e+38f; std::vector<float> cmn, cmx; const _odla_value* v = nullptr; };
  std::map<const _odla_value*, R> seen;
  std::vector<const _odla_value*> order;
  auto take = [&](const _odla_value* v, unsigned* dev, int64_t channels, int device) {
    if (!dev || !v) return;
    std::vector<unsigned> h((size_t)(2 + 2 * channels));
    cudaSetDevice(device);
    if (cudaMemcpy(h.data(), dev, h.size() * sizeof(unsigned), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return; }
    if (h[0] == 0xffffffffu && h[1] == 0u) return;   // never updated
    if (!seen.count(v)) order.push_back(v);
    R& r = seen[v];
    r.v = v;
    r.mn = std::min(r.mn, range_key_decode(h[0])); r.mx = std::max(r.mx, range_key_decode(h[1]));
    if (r.cmn.empty()) { r.cmn.assign((size_t)channels, 3.402823466e+38f); r.cmx.assign((size_t)channels, -3.402823466e+38f); }
    for (int64_t k = 0; k < channels && k < (int64_t)r.cmn.size(); ++k) {
      r.cmn[(size_t)k] = std::min(r.cmn[(size_t)k], range_key_decode(h[(size_t)(2 + k)]));
      r.cmx[(size_t)k] = std::max(r.cmx[(size_t)k], range_key_decode(h[(size_t)(2 + channels + k)]));
    }
  };
  auto scan = [&](std::vector<Replica>& reps) {
    for (auto& rep : reps) {
      if (!rep.plan) continue;
      cudaSetDevice(rep.device);
      cudaStreamSynchronize(rep.stream);
      Plan& p = *rep.plan;
      for (size_t i = 0; i < p.inputs.size() && i < p.input_range_stats.size(); ++i) {
        const auto& sh = p.inputs[i].v->type.shape;
        take(p.inputs[i].v, p.input_range_stats[i], sh.size ? sh.dims[sh.size - 1] : 1, rep.device);
      }
      for (auto& l : p.launches) take(l.out_v, l.range_stats, l.out_channels, rep.device);
    }
  };
  scan(c->replicas);
  for (auto& kv : c->batch_replicas) scan(kv.second);
  for (auto& lane : c->lanes)
    for (auto& kv : lane->batch_replicas) scan(kv.second);
  // Reshape results share their source's memory: give them a per-value record under their own name
  std::vector<std::pair<const _odla_value*, const _odla_value*>> aliases;
  for (auto& n : c->nodes) {
    if (n->kind != OP_RESHAPE) continue;
    const _odla_value* src = n->in[0];
    while (src && src->kind == OP_RESHAPE) src = src->in[0];
    if (src && seen.count(src)) aliases.push_back({n.get(), src});
  }
  int n_rec = 0;
  auto emit = [&](const _odla_value* v, int ch_idx, float scale, float mn, float mx) {
    if (records && n_rec < capacity) {
      odla_value_quant_info q{};
      q.value_id = (odla_value_id)v->name.c_str(); q.ch_idx = ch_idx; q.scale = scale; q.offset = 0.f; q.min = mn; q.max = mx;
      records[n_rec] = q;
    }
    ++n_rec;
  };
  auto sym = [](float mn, float mx) { const float a = std::max(std::fabs(mn), std::fabs(mx)); return a > 0.f ? a / 127.f : 1.f; };
  // layout of utils/halo_pgq.py:309-327: one record per value with ch_idx = -channels, then one per channel
  for (const _odla_value* v : order) {
    const R& r = seen[v];
    const int chs = v->type.shape.size >= 3 ? (int)r.cmn.size() : 1;   // channel-wise ranges for image-like tensors only
    emit(v, -chs, sym(r.mn, r.mx), r.mn, r.mx);
    if (chs > 1) for (int k = 0; k < chs; ++k) emit(v, k, 0.f, r.cmn[(size_t)k], r.cmx[(size_t)k]);
  }
  for (auto& a : aliases) { const R& r = seen[a.second]; emit(a.first, -1, sym(r.mn, r.mx), r.mn, r.mx); }
  return n_rec;
}
int odla_b200_PlanShards(odla_computation c, long long run_batch, int visible_devices, int* device, long long* start, long long* rows, int capacity) {
  if (!c || visible_devices < 1) return 0;
  int64_t B = 1;
  // the same decisions ensure_planned takes, on a scratch copy of the two fields they write
  const bool was_shardable = c->shardable;
  c->shardable = graph_shardable(c, &B);
  if (run_batch <= 0) run_batch = B;
  const std::vector<Shard> layout = shard_layout(c, visible_devices, B, run_batch);
  c->shardable = was_shardable;
  for (size_t i = 0; i < layout.size() && (int)i < capacity; ++i) {
    if (device) device[i] = layout[i].device;
    if (start) start[i] = layout[i].start;
    if (rows) rows[i] = layout[i].rows;
  }
  return (int)layout.size();
}
int odla_b200_DescribePlan(odla_computation c, char* buf, int capacity) {
  if (!c) return 0;
  if (ensure_planned(c) != ODLA_SUCCESS) return 0;
  std::string s;
  char line[256];
  for (auto& r : c->replicas) {
    snprintf(line, sizeof(line), "gpu %d rows [%lld,%lld) arena %lld bytes\n", r.device, (long long)r.shard_start, (long long)(r.shard_start + r.shard_batch), (long long)r.plan->arena_bytes);
    s += line;
    for (auto& l : r.plan->launches) { snprintf(line, sizeof(line), "  %-12s %s\n", l.op.c_str(), l.name.c_str()); s += line; }
  }
  if (buf && capacity > 0) { snprintf(buf, (size_t)capacity, "%s", s.c_str()); }
  return (int)s.size() + 1;
}
}
