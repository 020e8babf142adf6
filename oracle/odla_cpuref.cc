// TEST INFRASTRUCTURE -- libodla_cpuref.so, a CPU ODLA platform used as the oracle.
//
// It implements the same ODLA C ABI as libodla_b200.so (include/odla_b200.h) on top of the
// plain-C kernels in oracle/kernels.c, so one model description can be run through both
// libraries and the results compared.  It is not part of the shipped library: only tests, the
// smoke check and the benchmark's CPU-baseline leg may load it.
//
// Execution model: like ODLA/platforms/dnnl/odla_dnnl.cc:60-72,133-159 each op builder
// appends one closure to the computation and odla_ExecuteComputation replays the list, then
// copies outputs into the bound host pointers.  All floating-point tensors are held as fp32.
//
// When the shared object built from the reference's own runtime/generic sources is available
// (oracle/_ref/libhalo_rt_generic.so, or $ODLA_CPUREF_REFLIB) its _sn_rt_* kernels are used for
// fp32 convolution, max-pooling, soft-max (last axis), matmul and relu, so those results come
// from the reference's code; odla_cpuref_UsesReference() tells which.
//
// int8 rule (this build's definition; the reference has no int8 execution): a Conv or Gemm
// whose data operand is odla_Dequantize(int8, per-tensor scale) and whose weight operand is
// odla_Dequantize(int8, per-tensor or per-output-channel scale), both without zero point -- or
// odla_Dequantize(uint8, per-tensor scale, per-tensor zero point), the asymmetric weights of
// -quantize-weights=quint8, taken as W_u - zp -- is computed exactly in integers and scaled once: out = float(acc_int32) * (s_in * s_w[k]), the
// product s_in*s_w[k] rounded to fp32 first.  Everything after that (bias add, residual add,
// relu) is ordinary node-by-node fp32 arithmetic.  A value "comes from accumulators" if it is such a
// Conv/Gemm result or an element-wise (unary / binary / reshape) function of one; odla_Quantize of
// such a value (per-tensor scale, no zero point, int8) is a requantisation and multiplies by
// fl(1/s): q = sat(rne(x * fl(1/s))).  Every other odla_Quantize divides, q = sat(rne(x / s)), as
// ODLA/platforms/dnnl/odla_dnnl_quantization.cc:77 does.
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "../include/odla_b200.h"

extern "C" {
void ora_conv2d_f32(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int, int64_t, int64_t);
void ora_conv2d_s8(int32_t*, const int8_t*, const int8_t*, int64_t, int64_t, int64_t, int64_t,
                   int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                   int64_t, int64_t);
void ora_matmul_f32(float*, const float*, const float*, int64_t, int64_t, int64_t, int, int);
void ora_gemm_finish_f32(float*, const float*, int64_t, int64_t, int64_t, float, float);
void ora_matmul_s8(int32_t*, const int8_t*, const int8_t*, int64_t, int64_t, int64_t, int, int);
void ora_conv2d_s8_w16(int32_t*, const int8_t*, const int16_t*, int64_t, int64_t, int64_t, int64_t,
                       int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t);
void ora_matmul_s8_w16(int32_t*, const int8_t*, const int16_t*, int64_t, int64_t, int64_t, int, int);
void ora_maxpool_f32(float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                     int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int);
void ora_maxpool_s8(int8_t*, const int8_t*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int64_t, int64_t, int64_t, int64_t, int64_t, int64_t);
void ora_avgpool_f32(float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                     int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int);
void ora_batchnorm_f32(float*, const float*, const float*, const float*, const float*, const float*,
                       float, float, float, int64_t, int64_t, int64_t);
void ora_unary_f32(int, float*, const float*, int64_t, float, float);
void ora_binary_f32(int, float*, const float*, const float*, int, const int64_t*, const int64_t*,
                    const int64_t*);
void ora_softmax_f32(float*, const float*, int64_t, int64_t, int64_t, int);
void ora_reduce_mean_axis_f32(float*, const float*, int64_t, int64_t, int64_t);
void ora_layernorm_f32(float*, const float*, const float*, const float*, int64_t, int64_t, float);
void ora_quantize_f32(void*, const float*, const float*, const int32_t*, int64_t, int64_t, int64_t,
                      int, int);
void ora_requantize_f32(int8_t*, const float*, float, int64_t);
void ora_dequantize_f32(float*, const void*, const float*, const int32_t*, int64_t, int64_t,
                        int64_t, int, int);
void ora_transpose(void*, const void*, int, const int64_t*, const int64_t*, int);
void ora_concat_part(void*, const void*, int64_t, int64_t, int64_t, int64_t, int64_t, int);
void ora_resize_nearest(void*, const void*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                        int, int);
void ora_gather(void*, const void*, const int64_t*, int64_t, int64_t, int64_t, int64_t, int);
void ora_nms(int64_t*, int64_t, const float*, const float*, int64_t, int64_t, int64_t, int64_t, float, float, int32_t*, int32_t*);
void ora_yolo_postprocess(float*, uint32_t*, const float* const*, const int*, const int*, int64_t, uint32_t, uint32_t, float*, float*, int32_t*);
void ora_slice(void*, const void*, int, const int64_t*, const int64_t*, const int64_t*,
               const int64_t*, int);
}
enum { U_RELU = 0, U_LEAKY, U_CLAMP, U_GELU_ERF, U_GELU_TANH, U_ERF, U_SIGMOID, U_TANH, U_EXP, U_LOG,
       U_SQRT, U_RSQRT, U_ABS, U_NEG, U_RECIP, U_ROUND };
enum { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_POW, B_PRELU };

// ---- optional kernels compiled from the reference's runtime/generic sources ----
namespace {
struct RefLib {
  void (*conv_nhwc)(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int64_t) = nullptr;
  void (*maxpool_nhwc)(float*, const float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                       int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                       int64_t) = nullptr;
  void (*softmax)(float*, const float*, const int64_t*, int32_t, int32_t, int64_t) = nullptr;
  void (*matmul)(float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t, bool,
                 bool) = nullptr;
  void (*relu)(float*, const float*, int64_t) = nullptr;
  bool ok = false;
};
RefLib& reflib() {
  static RefLib r;
  static bool tried = false;
  if (tried) return r;
  tried = true;
  if (getenv("ODLA_CPUREF_NO_REFLIB")) return r;
  std::string path;
  if (const char* e = getenv("ODLA_CPUREF_REFLIB")) path = e;
  else {
    Dl_info info;
    if (dladdr((void*)&reflib, &info) && info.dli_fname) {
      path = info.dli_fname;
      auto p = path.rfind('/');
      path = (p == std::string::npos ? std::string(".") : path.substr(0, p)) + "/_ref/libhalo_rt_generic.so";
    }
  }
  void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
  if (!h) return r;
  r.conv_nhwc = (decltype(r.conv_nhwc))dlsym(h, "_sn_rt_conv2d_f32_nhwc");
  r.maxpool_nhwc = (decltype(r.maxpool_nhwc))dlsym(h, "_sn_rt_poolingmax_f32_nhwc");
  r.softmax = (decltype(r.softmax))dlsym(h, "_sn_rt_softmax_f32");
  r.matmul = (decltype(r.matmul))dlsym(h, "_sn_rt_matmul_f32");
  r.relu = (decltype(r.relu))dlsym(h, "_sn_rt_relu_f32");
  r.ok = r.conv_nhwc && r.maxpool_nhwc && r.softmax && r.matmul && r.relu;
  return r;
}
int n_threads() {
  static int n = [] {
    if (const char* e = getenv("ODLA_CPUREF_THREADS")) return std::max(1, atoi(e));
    return (int)std::max(1u, std::thread::hardware_concurrency());
  }();
  return n;
}
// Run fn(begin,end) over [0,total) split across the host threads.
void parallel_for(int64_t total, const std::function<void(int64_t, int64_t)>& fn) {
  int nt = (int)std::min<int64_t>(n_threads(), total);
  if (nt <= 1) { fn(0, total); return; }
  std::vector<std::thread> th;
  for (int t = 0; t < nt; ++t) {
    int64_t b = total * t / nt, e = total * (t + 1) / nt;
    th.emplace_back([=, &fn] { fn(b, e); });
  }
  for (auto& t : th) t.join();
}
float half_to_float(uint16_t h) {
  uint32_t s = (h >> 15) & 1, e = (h >> 10) & 0x1f, m = h & 0x3ff, u;
  if (e == 0) {
    if (m == 0) u = s << 31;
    else { int k = 0; while (!(m & 0x400)) { m <<= 1; ++k; } u = (s << 31) | ((127 - 15 - k + 1) << 23) | ((m & 0x3ff) << 13); }
  } else if (e == 31) u = (s << 31) | 0x7f800000u | (m << 13);
  else u = (s << 31) | ((e - 15 + 127) << 23) | (m << 13);
  float f; memcpy(&f, &u, 4); return f;
}
uint16_t float_to_half(float f) {  // round to nearest even
  uint32_t u; memcpy(&u, &f, 4);
  uint32_t s = (u >> 16) & 0x8000; int32_t e = ((u >> 23) & 0xff) - 127 + 15; uint32_t m = u & 0x7fffff;
  if (((u >> 23) & 0xff) == 0xff) return s | 0x7c00 | (m ? 0x200 : 0);
  if (e >= 31) return s | 0x7c00;
  if (e <= 0) {
    if (e < -10) return s;
    m |= 0x800000; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (r & 1))) ++r;
    return s | r;
  }
  uint32_t r = (e << 10) | (m >> 13), rem = m & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) ++r;
  return s | r;
}
float bf16_to_float(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f; }
uint16_t float_to_bf16(float f) {
  uint32_t u; memcpy(&u, &f, 4);
  if ((u & 0x7fffffff) > 0x7f800000) return (u >> 16) | 0x40;
  u += 0x7fff + ((u >> 16) & 1);
  return u >> 16;
}
int elem_size(odla_element_type t) {
  switch (t) {
    case ODLA_INT8: case ODLA_UINT8: case ODLA_QINT8: case ODLA_QUINT8: case ODLA_BOOL: return 1;
    case ODLA_INT16: case ODLA_UINT16: case ODLA_FLOAT16: case ODLA_BFLOAT16: return 2;
    case ODLA_INT32: case ODLA_UINT32: case ODLA_FLOAT32: case ODLA_QINT32: return 4;
    case ODLA_INT64: case ODLA_UINT64: case ODLA_FLOAT64: return 8;
    default: return 0;
  }
}
bool is_float(odla_element_type t) { return t == ODLA_FLOAT32 || t == ODLA_FLOAT16 || t == ODLA_BFLOAT16; }
int64_t numel(const odla_value_shape& s) { int64_t n = 1; for (int i = 0; i < s.size; ++i) n *= s.dims[i]; return n; }
}  // namespace

// Internal storage type: floats are always fp32; integers keep their width.
struct _odla_value {
  std::string name;
  odla_value_type api_type;        // what the caller declared
  odla_element_type store;         // ODLA_FLOAT32 for every float tensor
  std::vector<uint8_t> buf;
  bool is_arg = false, is_const = false;
  // producer info used by the int8 rule
  odla_value dq_src = nullptr, dq_scale = nullptr; bool dq_zp = false; int dq_axis = -1;
  odla_value dq_zp_value = nullptr;   // the zero-point operand itself (asymmetric uint8 weights)
  std::vector<int32_t> acc;        // int32 accumulators of the last int8 Conv/Gemm (for tests)
  bool from_acc = false;           // computed from int32 accumulators through element-wise ops only
  float* f() { return (float*)buf.data(); }
  int64_t n() const { return numel(api_type.shape); }
  const odla_value_shape& shape() const { return api_type.shape; }
};
struct _odla_computation {
  std::vector<std::unique_ptr<_odla_value>> vals;
  std::vector<std::function<void()>> ops;
  std::vector<odla_value> args, outs;
  std::map<std::string, odla_value> by_name;
  std::string error;
};
struct _odla_context {
  odla_computation comp;
  std::map<odla_value, const void*> in;
  std::map<odla_value, void*> out;
};
struct _odla_device { int idx; };

static thread_local odla_computation g_comp = nullptr;

static odla_value new_value(odla_element_type et, const odla_value_shape& shape, const odla_value_id id) {
  auto v = std::make_unique<_odla_value>();
  static int anon = 0;
  v->name = id ? std::string((const char*)id) : ("_anon" + std::to_string(anon++));
  v->api_type.element_type = et;
  v->api_type.shape = shape;
  if (shape.size == 0) { v->api_type.shape.size = 1; v->api_type.shape.dims[0] = 1; }  // odla_dnnl.cc:181-190
  v->store = is_float(et) ? ODLA_FLOAT32 : et;
  v->buf.resize((size_t)(numel(v->api_type.shape) * elem_size(v->store)));
  odla_value r = v.get();
  g_comp->by_name[v->name] = r;
  g_comp->vals.push_back(std::move(v));
  return r;
}
static void load_external(odla_value v, const void* src) {  // caller memory -> internal storage
  int64_t n = v->n();
  if (v->api_type.element_type == ODLA_FLOAT16) { auto* s = (const uint16_t*)src; for (int64_t i = 0; i < n; ++i) v->f()[i] = half_to_float(s[i]); }
  else if (v->api_type.element_type == ODLA_BFLOAT16) { auto* s = (const uint16_t*)src; for (int64_t i = 0; i < n; ++i) v->f()[i] = bf16_to_float(s[i]); }
  else memcpy(v->buf.data(), src, v->buf.size());
}
static void store_external(odla_value v, void* dst) {
  int64_t n = v->n();
  if (v->api_type.element_type == ODLA_FLOAT16) { auto* d = (uint16_t*)dst; for (int64_t i = 0; i < n; ++i) d[i] = float_to_half(v->f()[i]); }
  else if (v->api_type.element_type == ODLA_BFLOAT16) { auto* d = (uint16_t*)dst; for (int64_t i = 0; i < n; ++i) d[i] = float_to_bf16(v->f()[i]); }
  else memcpy(dst, v->buf.data(), v->buf.size());
}
static odla_value fail(const char* msg) {
  fprintf(stderr, "[odla_cpuref] %s\n", msg);
  if (g_comp && g_comp->error.empty()) g_comp->error = msg;
  odla_value_shape s{1, {1}};
  return new_value(ODLA_FLOAT32, s, nullptr);
}
static std::vector<int64_t> read_indices(odla_value v) {
  std::vector<int64_t> r((size_t)v->n());
  for (int64_t i = 0; i < v->n(); ++i)
    r[i] = v->store == ODLA_INT64 ? ((int64_t*)v->buf.data())[i] : v->store == ODLA_INT32 ? ((int32_t*)v->buf.data())[i] : (int64_t)v->f()[i];
  return r;
}

extern "C" {
int odla_cpuref_UsesReference(void) { return reflib().ok ? 1 : 0; }
int odla_cpuref_Threads(void) { return n_threads(); }
// Copies the int32 accumulators the int8 rule produced for value `name` (0 if none).
long long odla_cpuref_GetAccumulators(odla_computation c, const char* name, int32_t* dst, long long cap) {
  auto it = c->by_name.find(name);
  if (it == c->by_name.end()) return 0;
  auto& a = it->second->acc;
  if (dst) memcpy(dst, a.data(), sizeof(int32_t) * (size_t)std::min<long long>(cap, (long long)a.size()));
  return (long long)a.size();
}
// Copies the fp32/int internal storage of any value after an execution (for layer-wise tests).
long long odla_cpuref_GetValueData(odla_computation c, const char* name, void* dst, long long cap_bytes) {
  auto it = c->by_name.find(name);
  if (it == c->by_name.end()) return 0;
  auto& b = it->second->buf;
  if (dst) memcpy(dst, b.data(), (size_t)std::min<long long>(cap_bytes, (long long)b.size()));
  return (long long)b.size();
}

const char* odla_GetVersionString() { return "odla_cpuref 0.5 (oracle)"; }
odla_status odla_SetLogLevel(odla_log_level) { return ODLA_SUCCESS; }
odla_status odla_SetLogger(odla_logging_func) { return ODLA_SUCCESS; }
odla_logging_func odla_GetLogger() { return nullptr; }

odla_status odla_CreateComputation(odla_computation* c) { *c = new _odla_computation(); g_comp = *c; return ODLA_SUCCESS; }
odla_status odla_DestroyComputation(odla_computation c) { if (g_comp == c) g_comp = nullptr; delete c; return ODLA_SUCCESS; }
odla_status odla_SetComputationItem(odla_computation, odla_item_type, odla_item_value) { return ODLA_SUCCESS; }
odla_status odla_CreateContext(odla_context* ctx) { *ctx = new _odla_context{g_comp, {}, {}}; return ODLA_SUCCESS; }
odla_status odla_DestroyContext(odla_context ctx) { delete ctx; return ODLA_SUCCESS; }
odla_status odla_SetContextItem(odla_context, odla_item_type, odla_item_value) { return ODLA_SUCCESS; }
odla_status odla_GetNumOfArgsFromComputation(const odla_computation c, odla_uint32* n) { *n = (odla_uint32)c->args.size(); return ODLA_SUCCESS; }
odla_status odla_GetArgFromComputationByIdx(const odla_computation c, const odla_uint32 i, odla_value* v) {
  if (i >= c->args.size()) return ODLA_INVALID_PARAM; *v = c->args[i]; return ODLA_SUCCESS; }
odla_status odla_GetNumOfOutputsFromComputation(const odla_computation c, odla_uint32* n) { *n = (odla_uint32)c->outs.size(); return ODLA_SUCCESS; }
odla_status odla_GetOutputFromComputationByIdx(const odla_computation c, const odla_uint32 i, odla_value* v) {
  if (i >= c->outs.size()) return ODLA_INVALID_PARAM; *v = c->outs[i]; return ODLA_SUCCESS; }
odla_status odla_GetValueType(const odla_value v, odla_value_type* t) { *t = v->api_type; return ODLA_SUCCESS; }
odla_status odla_GetValueId(const odla_value v, odla_value_id* id) { *id = (odla_value_id)v->name.c_str(); return ODLA_SUCCESS; }
odla_status odla_GetRuntimeShape(odla_context, odla_value v, odla_value_shape* s) { *s = v->shape(); return ODLA_SUCCESS; }
odla_status odla_SetValueAsOutput(odla_value v) { g_comp->outs.push_back(v); return ODLA_SUCCESS; }
odla_status odla_SetValuesAsOutput(odla_values vs) { for (size_t i = 0; i < vs.size; ++i) g_comp->outs.push_back(vs.values[i]); return ODLA_SUCCESS; }
odla_status odla_BindToArgument(odla_value v, const odla_void* p, odla_context ctx) { ctx->in[v] = p; return ODLA_SUCCESS; }
odla_status odla_BindToArgumentById(const odla_value_id id, const odla_void* p, odla_context ctx) {
  auto it = ctx->comp->by_name.find((const char*)id); if (it == ctx->comp->by_name.end()) return ODLA_INVALID_PARAM;
  return odla_BindToArgument(it->second, p, ctx); }
odla_status odla_BindToOutput(odla_value v, odla_void* p, odla_context ctx) { ctx->out[v] = p; return ODLA_SUCCESS; }
odla_status odla_BindToOutputById(const odla_value_id id, odla_void* p, odla_context ctx) {
  auto it = ctx->comp->by_name.find((const char*)id); if (it == ctx->comp->by_name.end()) return ODLA_INVALID_PARAM;
  return odla_BindToOutput(it->second, p, ctx); }
odla_status odla_ExecuteComputation(const odla_computation c, const odla_context ctx, const odla_compute_mode, odla_device) {
  if (!c->error.empty()) return ODLA_UNSUPPORTED_OP;
  for (auto a : c->args) { auto it = ctx->in.find(a); if (it == ctx->in.end()) return ODLA_INVALID_PARAM; load_external(a, it->second); }
  for (auto& op : c->ops) op();
  for (auto o : c->outs) { auto it = ctx->out.find(o); if (it != ctx->out.end()) store_external(o, it->second); }
  return ODLA_SUCCESS;
}
odla_status odla_AllocateDevice(odla_vendor, odla_device_name, odla_int32 idx, odla_device* d) { *d = new _odla_device{idx}; return ODLA_SUCCESS; }
odla_status odla_DestroyDevice(odla_device d) { delete d; return ODLA_SUCCESS; }
odla_status odla_SetCurrentDevice(odla_device) { return ODLA_SUCCESS; }

odla_value odla_CreateArgument(const odla_value_type t, const odla_value_id id) {
  odla_value v = new_value(t.element_type, t.shape, id); v->is_arg = true; g_comp->args.push_back(v); return v; }
odla_value odla_CreateConstant(const odla_value_type t, const odla_void* p, const odla_value_id id) {
  odla_value v = new_value(t.element_type, t.shape, id); v->is_const = true; load_external(v, p); return v; }

// Asymmetric uint8 weights (per-tensor scale and zero point): the integer rule applies to W_u - zp.
static bool is_u8_weight(odla_value w) {
  return w->dq_src && w->dq_zp && w->dq_zp_value && w->dq_src->store == ODLA_UINT8 && w->dq_scale->n() == 1 && w->dq_zp_value->n() == 1;
}
static std::vector<int16_t> u8_weight_minus_zp(odla_value w) {
  odla_value zp = w->dq_zp_value;
  int32_t z = zp->store == ODLA_INT8 ? ((int8_t*)zp->buf.data())[0] : zp->store == ODLA_UINT8 ? ((uint8_t*)zp->buf.data())[0] : ((int32_t*)zp->buf.data())[0];
  std::vector<int16_t> r((size_t)w->dq_src->n());
  for (size_t i = 0; i < r.size(); ++i) r[i] = (int16_t)((int32_t)((uint8_t*)w->dq_src->buf.data())[i] - z);
  return r;
}
// ---- convolution: argument meaning as ODLA/include/ODLA/ops/odla_ops_nn.h:213-219 ----
odla_value odla_Conv(odla_value in, odla_memory_layout il, odla_uint32 group, odla_value ker, odla_memory_layout kl,
                     const odla_uint32* st, const odla_uint32* dil, const odla_uint32* pf, const odla_uint32* pb,
                     odla_value bias, odla_value_shape od, const odla_value_id id) {
  (void)pb;
  if (in->shape().size != 4) return fail("Conv: only 2-d convolution");
  if (dil && (dil[0] != 1 || dil[1] != 1)) return fail("Conv: dilation must be 1");  // odla_dnnl.cc:1070
  bool nhwc = il == ODLA_CHANNELS_LAST;
  if (!((nhwc && kl == ODLA_SIO) || (!nhwc && kl == ODLA_OIS))) return fail("Conv: layout pair not supported");
  const auto& is = in->shape(); const auto& ks = ker->shape();
  int64_t N = is.dims[0], H = nhwc ? is.dims[1] : is.dims[2], W = nhwc ? is.dims[2] : is.dims[3], C = nhwc ? is.dims[3] : is.dims[1];
  int64_t R = nhwc ? ks.dims[0] : ks.dims[2], S = nhwc ? ks.dims[1] : ks.dims[3], K = nhwc ? ks.dims[3] : ks.dims[0];
  int64_t P = nhwc ? od.dims[1] : od.dims[2], Q = nhwc ? od.dims[2] : od.dims[3];
  int64_t sh = st[0], sw = st[1], pt = pf[0], pl = pf[1], g = group ? group : 1;
  odla_value out = new_value(ODLA_FLOAT32, od, id);
  const bool u8w = is_u8_weight(ker);
  bool int_path = in->dq_src && ker->dq_src && !in->dq_zp && (u8w || (!ker->dq_zp && ker->dq_src->store == ODLA_INT8)) && in->dq_src->store == ODLA_INT8 &&
                  in->dq_scale->n() == 1 && nhwc && g == 1;
  if (int_path) {
    odla_value xq = in->dq_src, wq = ker->dq_src, sx = in->dq_scale, sw_ = ker->dq_scale;
    out->from_acc = true;
    g_comp->ops.push_back([=] {
      out->acc.resize((size_t)out->n());
      std::vector<int16_t> w16;
      if (u8w) w16 = u8_weight_minus_zp(ker);
      parallel_for(N * P, [&](int64_t b, int64_t e) {
        if (u8w) ora_conv2d_s8_w16(out->acc.data(), (int8_t*)xq->buf.data(), w16.data(), N, H, W, C, P, Q, K, R, S, sh, sw, pt, pl, b, e);
        else ora_conv2d_s8(out->acc.data(), (int8_t*)xq->buf.data(), (int8_t*)wq->buf.data(), N, H, W, C, P, Q, K, R, S, sh, sw, pt, pl, b, e); });
      for (int64_t i = 0; i < out->n(); ++i) {
        float m = sx->f()[0] * sw_->f()[sw_->n() == 1 ? 0 : i % K];
        float v = (float)out->acc[i] * m;
        if (bias) v = v + bias->f()[i % K];
        out->f()[i] = v;
      }
    });
    return out;
  }
  g_comp->ops.push_back([=] {
    if (nhwc && g == 1 && reflib().ok) {
      parallel_for(N, [&](int64_t b, int64_t e) {
        reflib().conv_nhwc(out->f() + b * P * Q * K, in->f() + b * H * W * C, ker->f(), e - b, H, W, C, P, Q, K, R, S, sh, sw, pt, 0, pl, 0); });
    } else {
      parallel_for(N * P, [&](int64_t b, int64_t e) { ora_conv2d_f32(out->f(), in->f(), ker->f(), N, H, W, C, P, Q, K, R, S, sh, sw, pt, pl, g, nhwc, b, e); });
    }
    if (bias) {
      int64_t inner = nhwc ? 1 : P * Q;
      for (int64_t i = 0; i < out->n(); ++i) out->f()[i] += bias->f()[(i / inner) % K];
    }
  });
  return out;
}

// ---- Gemm: alpha*op(A)*op(B) + beta*C; rank>2 is batched (odla_dnnl.cc:1730-1866) ----
odla_value odla_Gemm(odla_value A, odla_bool ta, odla_value B, odla_bool tb, odla_float32 alpha, odla_float32 beta,
                     odla_value C, odla_value_shape od, const odla_value_id id) {
  const auto& as = A->shape(); const auto& bs = B->shape();
  int ra = as.size, rb = bs.size;
  if (ra < 2 || rb < 2) return fail("Gemm: rank < 2");
  int64_t batch = 1; for (int i = 0; i < ra - 2; ++i) batch *= as.dims[i];
  int64_t bbatch = 1; for (int i = 0; i < rb - 2; ++i) bbatch *= bs.dims[i];
  int64_t ar = as.dims[ra - 2], ac = as.dims[ra - 1], br = bs.dims[rb - 2], bc = bs.dims[rb - 1];
  int64_t M = ta ? ac : ar, Kd = ta ? ar : ac, N = tb ? br : bc;
  if ((tb ? bc : br) != Kd) return fail("Gemm: inner dimensions differ");
  if (bbatch != batch && bbatch != 1) return fail("Gemm: batch dimensions differ");
  odla_value out = new_value(ODLA_FLOAT32, od, id);
  if (out->n() != batch * M * N) return fail("Gemm: output_dims do not match operands");
  const bool u8w = is_u8_weight(B);
  bool int_path = A->dq_src && B->dq_src && !A->dq_zp && (u8w || (!B->dq_zp && B->dq_src->store == ODLA_INT8)) && A->dq_src->store == ODLA_INT8 &&
                  A->dq_scale->n() == 1 && batch == 1;
  if (int_path) {
    odla_value aq = A->dq_src, bq = B->dq_src, sa = A->dq_scale, sb = B->dq_scale;
    out->from_acc = true;
    g_comp->ops.push_back([=] {
      out->acc.resize((size_t)out->n());
      if (u8w) { auto w16 = u8_weight_minus_zp(B); ora_matmul_s8_w16(out->acc.data(), (int8_t*)aq->buf.data(), w16.data(), M, N, Kd, ta, tb); }
      else ora_matmul_s8(out->acc.data(), (int8_t*)aq->buf.data(), (int8_t*)bq->buf.data(), M, N, Kd, ta, tb);
      for (int64_t i = 0; i < out->n(); ++i) {
        float m = sa->f()[0] * sb->f()[sb->n() == 1 ? 0 : i % N];
        out->f()[i] = (float)out->acc[i] * m;
      }
      ora_gemm_finish_f32(out->f(), (C && beta != 0) ? C->f() : nullptr, M, N, C ? C->n() : 0, alpha, beta);
    });
    return out;
  }
  g_comp->ops.push_back([=] {
    parallel_for(batch, [&](int64_t b0, int64_t b1) {
      for (int64_t b = b0; b < b1; ++b) {
        const float* bp = B->f() + (bbatch == 1 ? 0 : b * br * bc);
        if (reflib().ok && !(ta && tb)) reflib().matmul(out->f() + b * M * N, A->f() + b * ar * ac, bp, ar, ac, br, bc, ta, tb);
        else ora_matmul_f32(out->f() + b * M * N, A->f() + b * ar * ac, bp, M, N, Kd, ta, tb);
        int64_t cn = C ? C->n() : 0;
        const float* cp = (C && beta != 0) ? C->f() : nullptr;
        if (cp && cn == batch * M * N && batch > 1) { cp += b * M * N; cn = M * N; }
        ora_gemm_finish_f32(out->f() + b * M * N, cp, M, N, cn, alpha, beta);
      }
    });
  });
  return out;
}
odla_value odla_BatchMatMul(odla_value A, odla_bool ta, odla_value B, odla_bool tb, odla_value_shape od, const odla_value_id id) {
  return odla_Gemm(A, ta, B, tb, 1.f, 0.f, nullptr, od, id);
}

static odla_value pool(bool is_max, odla_value in, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st,
                       const odla_uint32* pf, odla_value_shape od, const odla_value_id id) {
  if (in->shape().size != 4) return fail("Pool: only 2-d pooling");
  bool nhwc = il == ODLA_CHANNELS_LAST;
  const auto& is = in->shape();
  int64_t N = is.dims[0], H = nhwc ? is.dims[1] : is.dims[2], W = nhwc ? is.dims[2] : is.dims[3], C = nhwc ? is.dims[3] : is.dims[1];
  int64_t P = nhwc ? od.dims[1] : od.dims[2], Q = nhwc ? od.dims[2] : od.dims[3];
  int64_t R = win[0], S = win[1], sh = st[0], sw = st[1], pt = pf[0], pl = pf[1];
  odla_value out = new_value(in->api_type.element_type, od, id);
  g_comp->ops.push_back([=] {
    if (in->store == ODLA_INT8) {
      if (!is_max || !nhwc) { fprintf(stderr, "[odla_cpuref] int8 pooling: NHWC max only\n"); return; }
      ora_maxpool_s8((int8_t*)out->buf.data(), (int8_t*)in->buf.data(), N, H, W, C, P, Q, R, S, sh, sw, pt, pl);
    } else if (is_max) {
      if (nhwc && reflib().ok) reflib().maxpool_nhwc(out->f(), in->f(), N, H, W, C, P, Q, R, S, sh, sw, pt, 0, pl, 0);
      else ora_maxpool_f32(out->f(), in->f(), N, H, W, C, P, Q, R, S, sh, sw, pt, pl, nhwc);
    } else ora_avgpool_f32(out->f(), in->f(), N, H, W, C, P, Q, R, S, sh, sw, pt, pl, nhwc);
  });
  return out;
}
odla_value odla_MaxPool(odla_value in, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st, const odla_uint32* pf,
                        const odla_uint32*, odla_value_shape od, const odla_value_id id) { return pool(true, in, il, win, st, pf, od, id); }
odla_value odla_AveragePool(odla_value in, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st, const odla_uint32* pf,
                            const odla_uint32*, odla_bool, odla_value_shape od, const odla_value_id id) { return pool(false, in, il, win, st, pf, od, id); }

odla_value odla_BatchNormalization(odla_value in, odla_memory_layout il, odla_value mean, odla_value var, odla_float32 eps,
                                   odla_value scale, odla_value offset, odla_float32 ss, odla_float32 so, const odla_value_id id) {
  const auto& is = in->shape();
  bool nhwc = il == ODLA_CHANNELS_LAST;
  int64_t C = nhwc ? is.dims[is.size - 1] : is.dims[1];
  int64_t inner = 1; if (!nhwc) for (int i = 2; i < is.size; ++i) inner *= is.dims[i];
  int64_t outer = in->n() / (C * inner);
  odla_value out = new_value(ODLA_FLOAT32, is, id);
  g_comp->ops.push_back([=] { ora_batchnorm_f32(out->f(), in->f(), mean->f(), var->f(), scale ? scale->f() : nullptr,
                                                offset ? offset->f() : nullptr, ss, so, eps, outer, C, inner); });
  return out;
}

static odla_value unary(int op, odla_value in, float a, float b, const odla_value_id id) {
  odla_value out = new_value(ODLA_FLOAT32, in->shape(), id);
  out->from_acc = in->from_acc;
  g_comp->ops.push_back([=] {
    if (op == U_RELU && reflib().ok) reflib().relu(out->f(), in->f(), in->n());
    else ora_unary_f32(op, out->f(), in->f(), in->n(), a, b);
  });
  return out;
}
odla_value odla_Relu(odla_value x, const odla_value_id id) { return unary(U_RELU, x, 0, 0, id); }
odla_value odla_LeakyRelu(odla_value x, odla_float32 a, const odla_value_id id) { return unary(U_LEAKY, x, a, 0, id); }
odla_value odla_Clamp(odla_value x, odla_float32 lo, odla_float32 hi, const odla_value_id id) { return unary(U_CLAMP, x, lo, hi, id); }
odla_value odla_Gelu(odla_value x, odla_bool approx, const odla_value_id id) { return unary(approx ? U_GELU_TANH : U_GELU_ERF, x, 0, 0, id); }
odla_value odla_Erf(odla_value x, const odla_value_id id) { return unary(U_ERF, x, 0, 0, id); }
odla_value odla_Sigmoid(odla_value x, const odla_value_id id) { return unary(U_SIGMOID, x, 0, 0, id); }
odla_value odla_Tanh(odla_value x, const odla_value_id id) { return unary(U_TANH, x, 0, 0, id); }
odla_value odla_Exp(odla_value x, const odla_value_id id) { return unary(U_EXP, x, 0, 0, id); }
odla_value odla_Log(odla_value x, const odla_value_id id) { return unary(U_LOG, x, 0, 0, id); }
odla_value odla_Sqrt(odla_value x, const odla_value_id id) { return unary(U_SQRT, x, 0, 0, id); }
odla_value odla_Rsqrt(odla_value x, const odla_value_id id) { return unary(U_RSQRT, x, 0, 0, id); }
odla_value odla_Abs(odla_value x, const odla_value_id id) { return unary(U_ABS, x, 0, 0, id); }
odla_value odla_Neg(odla_value x, const odla_value_id id) { return unary(U_NEG, x, 0, 0, id); }
odla_value odla_Reciprocal(odla_value x, const odla_value_id id) { return unary(U_RECIP, x, 0, 0, id); }
odla_value odla_Round(odla_value x, const odla_value_id id) { return unary(U_ROUND, x, 0, 0, id); }

static odla_value binary(int op, odla_value l, odla_value r, const odla_value_id id) {
  int rank = std::max(l->shape().size, r->shape().size);
  std::vector<int64_t> ls(rank, 1), rs(rank, 1), os(rank);
  for (int i = 0; i < l->shape().size; ++i) ls[rank - l->shape().size + i] = l->shape().dims[i];
  for (int i = 0; i < r->shape().size; ++i) rs[rank - r->shape().size + i] = r->shape().dims[i];
  odla_value_shape osh; osh.size = rank;
  for (int i = 0; i < rank; ++i) {
    if (ls[i] != rs[i] && ls[i] != 1 && rs[i] != 1) return fail("binary op: shapes do not broadcast");
    os[i] = std::max(ls[i], rs[i]); osh.dims[i] = os[i];
  }
  odla_value out = new_value(ODLA_FLOAT32, osh, id);
  out->from_acc = l->from_acc || r->from_acc;
  g_comp->ops.push_back([=] { ora_binary_f32(op, out->f(), l->f(), r->f(), rank, os.data(), ls.data(), rs.data()); });
  return out;
}
odla_value odla_Add(odla_value l, odla_value r, const odla_value_id id) { return binary(B_ADD, l, r, id); }
odla_value odla_Sub(odla_value l, odla_value r, const odla_value_id id) { return binary(B_SUB, l, r, id); }
odla_value odla_Mul(odla_value l, odla_value r, const odla_value_id id) { return binary(B_MUL, l, r, id); }
odla_value odla_Div(odla_value l, odla_value r, const odla_value_id id) { return binary(B_DIV, l, r, id); }
odla_value odla_Pow(odla_value l, odla_value r, const odla_value_id id) { return binary(B_POW, l, r, id); }
odla_value odla_PRelu(odla_value l, odla_value r, const odla_value_id id) { return binary(B_PRELU, l, r, id); }

static odla_value softmax(odla_value in, int axis, bool log_form, const odla_value_id id) {
  const auto& s = in->shape();
  if (axis < 0) axis += s.size;
  int64_t outer = 1, inner = 1, dim = s.dims[axis];
  for (int i = 0; i < axis; ++i) outer *= s.dims[i];
  for (int i = axis + 1; i < s.size; ++i) inner *= s.dims[i];
  odla_value out = new_value(ODLA_FLOAT32, s, id);
  bool last = axis == s.size - 1;
  g_comp->ops.push_back([=] {
    if (last && !log_form && reflib().ok) reflib().softmax(out->f(), in->f(), in->shape().dims, axis, in->shape().size, in->n());
    else ora_softmax_f32(out->f(), in->f(), outer, dim, inner, log_form);
  });
  return out;
}
odla_value odla_Softmax(odla_value in, odla_int32 axis, const odla_value_id id) { return softmax(in, axis, false, id); }
odla_value odla_LogSoftmax(odla_value in, odla_int32 axis, const odla_value_id id) { return softmax(in, axis, true, id); }

odla_value odla_ReduceMean(odla_value in, odla_size_t na, const odla_uint32* axes, odla_bool, odla_value_shape od, const odla_value_id id) {
  std::vector<int64_t> dims(in->shape().dims, in->shape().dims + in->shape().size);
  std::vector<uint32_t> ax(axes, axes + na);
  odla_value out = new_value(ODLA_FLOAT32, od, id);
  g_comp->ops.push_back([=] {
    std::vector<int64_t> d = dims;
    std::vector<float> cur(in->f(), in->f() + in->n()), nxt;
    for (uint32_t a : ax) {
      int64_t before = 1, after = 1;
      for (size_t i = 0; i < d.size(); ++i) { if (i < a) before *= d[i]; else if (i > a) after *= d[i]; }
      nxt.assign((size_t)(before * after), 0.f);
      ora_reduce_mean_axis_f32(nxt.data(), cur.data(), before, d[a], after);
      d[a] = 1; cur.swap(nxt);
    }
    memcpy(out->f(), cur.data(), sizeof(float) * cur.size());
  });
  return out;
}
odla_value odla_LayerNorm(odla_value in, odla_int32 na, const odla_int32* axes, odla_float32 eps, odla_value scale, odla_value offset,
                          const odla_value_id id) {
  const auto& s = in->shape();
  int first = s.size;
  for (int i = 0; i < na; ++i) first = std::min(first, axes[i] < 0 ? axes[i] + s.size : axes[i]);
  if (first != s.size - na) return fail("LayerNorm: axes must be the trailing dimensions");
  int64_t dim = 1; for (int i = first; i < s.size; ++i) dim *= s.dims[i];
  odla_value out = new_value(ODLA_FLOAT32, s, id);
  g_comp->ops.push_back([=] { ora_layernorm_f32(out->f(), in->f(), scale ? scale->f() : nullptr, offset ? offset->f() : nullptr, in->n() / dim, dim, eps); });
  return out;
}

static void axis_split(const odla_value_shape& s, int axis, int64_t nscale, int64_t* outer, int64_t* adim, int64_t* inner, int* per_axis) {
  *per_axis = nscale > 1;
  if (!*per_axis) { *outer = 1; *adim = 1; *inner = numel(s); return; }
  if (axis < 0) axis += s.size;
  *outer = 1; *inner = 1; *adim = s.dims[axis];
  for (int i = 0; i < axis; ++i) *outer *= s.dims[i];
  for (int i = axis + 1; i < s.size; ++i) *inner *= s.dims[i];
}
odla_value odla_Quantize(odla_value in, odla_value scale, odla_value zp, odla_int32 axis, odla_element_type tt, const odla_value_id id) {
  if (tt != ODLA_INT8 && tt != ODLA_UINT8) return fail("Quantize: target must be int8 or uint8");  // odla_dnnl_quantization.cc:68
  int64_t outer, adim, inner; int per_axis;
  axis_split(in->shape(), axis, scale->n(), &outer, &adim, &inner, &per_axis);
  odla_value out = new_value(tt, in->shape(), id);
  const bool requant = in->from_acc && !zp && scale->n() == 1 && tt == ODLA_INT8;
  g_comp->ops.push_back([=] {
    if (requant) { ora_requantize_f32((int8_t*)out->buf.data(), in->f(), 1.0f / scale->f()[0], in->n()); return; }
    std::vector<int32_t> z;
    if (zp) { z.resize((size_t)zp->n()); for (int64_t i = 0; i < zp->n(); ++i) z[i] = zp->store == ODLA_INT8 ? ((int8_t*)zp->buf.data())[i] : zp->store == ODLA_UINT8 ? ((uint8_t*)zp->buf.data())[i] : ((int32_t*)zp->buf.data())[i]; }
    ora_quantize_f32(out->buf.data(), in->f(), scale->f(), zp ? z.data() : nullptr, outer, adim, inner, per_axis, tt == ODLA_UINT8);
  });
  return out;
}
odla_value odla_Dequantize(odla_value in, odla_value scale, odla_value zp, odla_int32 axis, odla_element_type tt, const odla_value_id id) {
  if (!is_float(tt)) return fail("Dequantize: target must be a float type");
  int64_t outer, adim, inner; int per_axis;
  axis_split(in->shape(), axis, scale->n(), &outer, &adim, &inner, &per_axis);
  odla_value out = new_value(ODLA_FLOAT32, in->shape(), id);
  out->dq_src = in; out->dq_scale = scale; out->dq_zp = zp != nullptr; out->dq_axis = axis; out->dq_zp_value = zp;
  g_comp->ops.push_back([=] {
    std::vector<int32_t> z;
    if (zp) { z.resize((size_t)zp->n()); for (int64_t i = 0; i < zp->n(); ++i) z[i] = zp->store == ODLA_INT8 ? ((int8_t*)zp->buf.data())[i] : zp->store == ODLA_UINT8 ? ((uint8_t*)zp->buf.data())[i] : ((int32_t*)zp->buf.data())[i]; }
    ora_dequantize_f32(out->f(), in->buf.data(), scale->f(), zp ? z.data() : nullptr, outer, adim, inner, per_axis, in->store == ODLA_UINT8);
  });
  return out;
}

odla_value odla_Reshape(odla_value in, odla_value_shape od, const odla_value_id id) {
  odla_value out = new_value(in->api_type.element_type, od, id);
  if (out->n() != in->n()) return fail("Reshape: element count differs");
  out->from_acc = in->from_acc;
  g_comp->ops.push_back([=] { memcpy(out->buf.data(), in->buf.data(), in->buf.size()); });
  return out;
}
odla_value odla_Transpose(odla_value in, odla_value_shape perm, odla_value_shape od, const odla_value_id id) {
  odla_value out = new_value(in->api_type.element_type, od, id);
  std::vector<int64_t> p(perm.dims, perm.dims + perm.size);
  g_comp->ops.push_back([=] { ora_transpose(out->buf.data(), in->buf.data(), in->shape().size, in->shape().dims, p.data(), elem_size(in->store)); });
  return out;
}
odla_value odla_Concat(odla_values ins, odla_int32 axis, odla_value_shape od, const odla_value_id id) {
  if (ins.size == 0) return fail("Concat: no inputs");
  odla_value first = ins.values[0];
  if (axis < 0) axis += first->shape().size;
  odla_value out = new_value(first->api_type.element_type, od, id);
  std::vector<odla_value> v(ins.values, ins.values + ins.size);
  g_comp->ops.push_back([=] {
    int64_t outer = 1, inner = 1, off = 0;
    for (int i = 0; i < axis; ++i) outer *= od.dims[i];
    for (int i = axis + 1; i < od.size; ++i) inner *= od.dims[i];
    for (auto x : v) { ora_concat_part(out->buf.data(), x->buf.data(), outer, x->shape().dims[axis], od.dims[axis], off, inner, elem_size(x->store)); off += x->shape().dims[axis]; }
  });
  return out;
}
odla_value odla_Resize(odla_value in, odla_interpolation_mode interp, odla_resize_coordinate_mode, odla_uint32, odla_value_shape od, const odla_value_id id) {
  if (interp != ODLA_NEAREST || in->shape().size != 4) return fail("Resize: only nearest, rank 4");
  const auto& s = in->shape();
  // A tensor whose channel extent is unchanged and last is treated as NHWC, else NCHW.
  bool nhwc = s.dims[3] == od.dims[3] && !(s.dims[1] == od.dims[1] && s.dims[2] != od.dims[2]);
  if (s.dims[1] == od.dims[1] && s.dims[3] != od.dims[3]) nhwc = false;
  int64_t N = s.dims[0], H = nhwc ? s.dims[1] : s.dims[2], W = nhwc ? s.dims[2] : s.dims[3], C = nhwc ? s.dims[3] : s.dims[1];
  int64_t P = nhwc ? od.dims[1] : od.dims[2], Q = nhwc ? od.dims[2] : od.dims[3];
  odla_value out = new_value(in->api_type.element_type, od, id);
  g_comp->ops.push_back([=] { ora_resize_nearest(out->buf.data(), in->buf.data(), N, H, W, C, P, Q, nhwc, elem_size(in->store)); });
  return out;
}
odla_value odla_Gather(odla_value in, odla_value idx, odla_int32 axis, odla_value_shape od, const odla_value_id id) {
  const auto& s = in->shape();
  if (axis < 0) axis += s.size;
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < axis; ++i) outer *= s.dims[i];
  for (int i = axis + 1; i < s.size; ++i) inner *= s.dims[i];
  odla_value out = new_value(in->api_type.element_type, od, id);
  g_comp->ops.push_back([=] { auto ids = read_indices(idx); ora_gather(out->buf.data(), in->buf.data(), ids.data(), outer, in->shape().dims[axis], (int64_t)ids.size(), inner, elem_size(in->store)); });
  return out;
}
odla_value odla_Slice(odla_value in, const odla_int32* start, const odla_int32* end, const odla_int32* stride, odla_value_shape od, const odla_value_id id) {
  (void)end;
  int rank = in->shape().size;
  std::vector<int64_t> st(start, start + rank), sp(rank, 1);
  if (stride) for (int i = 0; i < rank; ++i) sp[i] = stride[i];
  odla_value out = new_value(in->api_type.element_type, od, id);
  g_comp->ops.push_back([=] { ora_slice(out->buf.data(), in->buf.data(), rank, in->shape().dims, out->shape().dims, st.data(), sp.data(), elem_size(in->store)); });
  return out;
}
odla_value odla_NMS(odla_value boxes, odla_value scores, odla_uint32 max_num_outputs, odla_float32 iou, odla_float32 thr, odla_value_type ot, const odla_value_id id) {
  const auto& ss = scores->shape();
  if (boxes->shape().size != 3 || ss.size != 3) return fail("NMS: boxes [B,N,4], scores [B,C,N]");
  int64_t B = ss.dims[0], C = ss.dims[1], N = ss.dims[2], rows = ot.shape.dims[0];
  odla_value out = new_value(ot.element_type, ot.shape, id);
  g_comp->ops.push_back([=] {
    std::vector<int64_t> r((size_t)rows * 3);
    std::vector<int32_t> order((size_t)N + 1), kept((size_t)N + 1);
    ora_nms(r.data(), rows, boxes->f(), scores->f(), B, C, N, max_num_outputs ? (int64_t)max_num_outputs : rows, iou, thr, order.data(), kept.data());
    for (size_t i = 0; i < r.size(); ++i) { if (out->store == ODLA_INT64) ((int64_t*)out->buf.data())[i] = r[i]; else ((int32_t*)out->buf.data())[i] = (int32_t)r[i]; }
  });
  return out;
}
odla_values odla_PostProcess(odla_value iw, odla_value ih, odla_value b13, odla_value b26, odla_value b52, const odla_value_id id) {
  odla_values res{};
  std::string base = id ? (const char*)id : "postprocess", n0 = base + "0", n1 = base + "1";
  odla_value heads[3] = {b13, b26, b52};
  int S3[3], nchw3[3];
  int64_t chn = 0;
  for (int i = 0; i < 3; ++i) {
    const auto& s = heads[i]->shape();
    nchw3[i] = s.dims[2] == s.dims[3] && s.dims[1] % 3 == 0 && s.dims[1] / 3 > 5 && s.dims[1] != s.dims[2];
    S3[i] = (int)s.dims[2];
    chn = nchw3[i] ? s.dims[1] : s.dims[3];
  }
  const int64_t cls = chn / 3 - 5, N = 3 * ((int64_t)S3[0] * S3[0] + (int64_t)S3[1] * S3[1] + (int64_t)S3[2] * S3[2]);
  odla_value_shape s0{3, {cls, N / 169, 5}}, s1{1, {cls}};
  odla_value info = new_value(ODLA_FLOAT32, s0, (const odla_value_id)n0.c_str());
  odla_value num = new_value(ODLA_UINT32, s1, (const odla_value_id)n1.c_str());
  std::vector<int> S(S3, S3 + 3), L(nchw3, nchw3 + 3);
  g_comp->ops.push_back([=] {
    const float* hp[3] = {b13->f(), b26->f(), b52->f()};
    std::vector<float> bx((size_t)N * 4), sc((size_t)cls * N);
    std::vector<int32_t> order((size_t)N + 1);
    ora_yolo_postprocess(info->f(), (uint32_t*)num->buf.data(), hp, L.data(), S.data(), cls, *(uint32_t*)iw->buf.data(), *(uint32_t*)ih->buf.data(), bx.data(), sc.data(), order.data());
  });
  res.size = 2; res.values[0] = info; res.values[1] = num;
  return res;
}
odla_value odla_Cast(odla_value in, odla_element_type tt, const odla_value_id id) {
  odla_value out = new_value(tt, in->shape(), id);
  g_comp->ops.push_back([=] {
    for (int64_t i = 0; i < in->n(); ++i) {
      double v = in->store == ODLA_FLOAT32 ? in->f()[i] : in->store == ODLA_INT32 ? ((int32_t*)in->buf.data())[i] : in->store == ODLA_INT64 ? (double)((int64_t*)in->buf.data())[i]
                 : in->store == ODLA_INT8 ? ((int8_t*)in->buf.data())[i] : in->store == ODLA_UINT8 ? ((uint8_t*)in->buf.data())[i] : 0;
      switch (out->store) {
        case ODLA_FLOAT32: out->f()[i] = (float)v; break;
        case ODLA_INT32: ((int32_t*)out->buf.data())[i] = (int32_t)v; break;
        case ODLA_INT64: ((int64_t*)out->buf.data())[i] = (int64_t)v; break;
        case ODLA_INT8: ((int8_t*)out->buf.data())[i] = (int8_t)std::max(-128.0, std::min(127.0, std::nearbyint(v))); break;  // saturating, odla_dnnl_cast.cc:232-276
        case ODLA_UINT8: ((uint8_t*)out->buf.data())[i] = (uint8_t)std::max(0.0, std::min(255.0, std::nearbyint(v))); break;
        default: break;
      }
    }
  });
  return out;
}
}  // extern "C"
