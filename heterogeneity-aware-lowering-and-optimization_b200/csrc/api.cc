// The ODLA C entry points of libodla_b200.so: graph recording, binding, property bags, device and
// logging functions.  Builders only record nodes (compile mode, like odla_dnnl's add_op in
// ODLA/platforms/dnnl/odla_dnnl.cc:60-72); planning and kernel launches live in plan.cc.
//
// Error convention: the generated model code never checks the odla_value returned by an op
// builder (lib/target/generic_cpp/generic_cxx_codegen.cc:775-800 only checks odla_status
// results), so a failing builder logs, remembers the first error in the computation, and
// returns a non-NULL poison value; odla_CreateContext / odla_ExecuteComputation then report it.
// No C++ exception crosses the ABI.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <set>
#include <mutex>

#include "common.h"

namespace b200 {

static odla_log_level g_level = ODLA_LOG_LEVEL_WARN;
static void default_logger(const char* file, int line, const char* func, odla_log_level lvl, const char* msg) {
  static const char* names[] = {"OFF", "FATAL", "ERROR", "WARN", "INFO", "DEBUG", "TRACE"};
  const char* base = strrchr(file, '/');
  fprintf(stderr, "[odla_b200 %s] %s:%d %s: %s\n", names[lvl], base ? base + 1 : file, line, func, msg);
}
static odla_logging_func g_logger = default_logger;

void log_msg(const char* file, int line, const char* func, odla_log_level lvl, const char* fmt, ...) {
  if (lvl > g_level || !g_logger) return;
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_logger(file, line, func, lvl, buf);
}

bool inject_fault(const char* site) {
  static std::mutex mu;
  static std::string spec_site;
  static long target = -1, count = 0;
  static bool parsed = false;
  std::lock_guard<std::mutex> lk(mu);
  const char* e = getenv("ODLA_B200_INJECT");
  if (!e) { parsed = false; return false; }
  if (!parsed || spec_site.empty()) {
    std::string s(e);
    auto at = s.find('@');
    spec_site = s.substr(0, at);
    target = at == std::string::npos ? 1 : atol(s.c_str() + at + 1);
    count = 0;
    parsed = true;
  }
  if (spec_site != site) return false;
  return ++count == target;
}

const char* op_name(OpKind k) {
  static const char* n[] = {"arg", "const", "conv", "gemm", "maxpool", "avgpool", "batchnorm", "unary", "binary",
                            "softmax", "reduce_mean", "layernorm", "quantize", "dequantize", "reshape", "transpose",
                            "concat", "resize", "gather", "slice", "cast", "nms", "postprocess", "postprocess_num"};
  return n[k];
}
int elem_size(odla_element_type t) {
  switch (t) {
    case ODLA_INT8: case ODLA_UINT8: case ODLA_QINT8: case ODLA_QUINT8: case ODLA_BOOL: return 1;
    case ODLA_INT16: case ODLA_UINT16: case ODLA_QINT16: case ODLA_QUINT16: case ODLA_FLOAT16: case ODLA_BFLOAT16: return 2;
    case ODLA_INT32: case ODLA_UINT32: case ODLA_QINT32: case ODLA_QUINT32: case ODLA_FLOAT32: return 4;
    case ODLA_INT64: case ODLA_UINT64: case ODLA_QINT64: case ODLA_QUINT64: case ODLA_FLOAT64: return 8;
    default: return 0;
  }
}
bool is_float_type(odla_element_type t) { return t == ODLA_FLOAT32 || t == ODLA_FLOAT16 || t == ODLA_BFLOAT16; }
int64_t numel(const odla_value_shape& s) {
  int64_t n = 1;
  for (int i = 0; i < s.size; ++i) n *= s.dims[i];
  return n;
}
int storage_size(int dt) {
  switch (dt) {
    case DT_F32: case DT_S32: return 4;
    case DT_F16: case DT_BF16: return 2;
    case DT_S8: case DT_U8: return 1;
    case DT_S64: return 8;
  }
  return 0;
}

thread_local int g_current_device = -1;
// The computation op builders append to; set by odla_CreateComputation on the calling thread,
// the same implicit contract as ODLA/platforms/dnnl/odla_dnnl.cc:55-59,98-105.
static thread_local odla_computation g_comp = nullptr;

static odla_value add_node(OpKind kind, odla_element_type et, const odla_value_shape& shape, const odla_value_id id,
                           std::vector<odla_value> in, std::vector<int64_t> ia = {}, std::vector<float> fa = {}) {
  if (!g_comp) {
    B2_ERR("op builder called with no current computation (call odla_CreateComputation first)");
    return nullptr;
  }
  auto v = std::make_unique<_odla_value>();
  v->name = id ? std::string((const char*)id) : ("_v" + std::to_string(g_comp->nodes.size()));
  v->type.element_type = et;
  v->type.shape = shape;
  if (shape.size == 0) {  // scalars become [1], ODLA/platforms/dnnl/odla_dnnl.cc:181-190
    v->type.shape.size = 1;
    v->type.shape.dims[0] = 1;
  }
  v->kind = kind;
  v->in = std::move(in);
  v->ia = std::move(ia);
  v->fa = std::move(fa);
  v->index = (int)g_comp->nodes.size();
  for (auto i : v->in)
    if (i && i->poison) v->poison = true;
  odla_value r = v.get();
  g_comp->by_name[v->name] = r;
  g_comp->nodes.push_back(std::move(v));
  g_comp->planned = false;
  return r;
}
static odla_value fail_node(odla_status st, const odla_value_id id, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  B2_ERR("%s", buf);
  if (!g_comp) return nullptr;
  if (g_comp->first_error.empty()) {
    g_comp->first_error = buf;
    g_comp->error_status = st;
  }
  odla_value_shape s;
  s.size = 1;
  s.dims[0] = 1;
  odla_value v = add_node(OP_CONST, ODLA_FLOAT32, s, id, {});
  v->poison = true;
  return v;
}
static bool any_null(std::initializer_list<odla_value> vs) {
  for (auto v : vs)
    if (!v) return true;
  return false;
}

}  // namespace b200

using namespace b200;

_odla_computation::~_odla_computation() {
  b200::destroy_replicas(replicas);
  for (auto& kv : batch_replicas) b200::destroy_replicas(kv.second);
  for (auto& lane : lanes)
    for (auto& kv : lane->batch_replicas) b200::destroy_replicas(kv.second);
  for (auto& kv : chain) {
    if (!kv.second || !kv.second->last) continue;
    if (cudaSetDevice(kv.first) == cudaSuccess) cudaEventDestroy(kv.second->last);
    else cudaGetLastError();
  }
}

extern "C" {

// ------------------------------------------------------------- log / version ----
odla_status odla_SetLogLevel(odla_log_level level) { g_level = level; return ODLA_SUCCESS; }
odla_status odla_SetLogger(odla_logging_func logger) { g_logger = logger ? logger : default_logger; return ODLA_SUCCESS; }
odla_logging_func odla_GetLogger() { return g_logger; }
const char* odla_GetVersionString() { return "odla_b200 0.5.0 (ODLA 0.5, sm_100a)"; }

// ------------------------------------------------------------------- devices ----
int odla_b200_DeviceCount(void) { return visible_devices(); }

odla_status odla_AllocateDevice(odla_vendor, odla_device_name name, odla_int32 idx, odla_device* device) {
  if (!device) return ODLA_INVALID_PARAM;
  if (name != ODLA_DEVICE_DEFAULT && name != ODLA_DEVICE_NVIDIA_GPU) return ODLA_UNSUPPORTED_DEVICE_TYPE;
  int n = visible_devices();
  if (n > 0 && (idx < 0 || idx >= n)) return ODLA_INVALID_PARAM;
  *device = new _odla_device{idx};
  return ODLA_SUCCESS;
}
odla_status odla_DestroyDevice(odla_device device) { delete device; return ODLA_SUCCESS; }
odla_status odla_SetCurrentDevice(odla_device device) {
  if (!device) return ODLA_INVALID_PARAM;
  g_current_device = device->index;
  return ODLA_SUCCESS;
}
// Every item answers ODLA_SUCCESS, as tests/ODLA/device_test.cc:63-89 in the reference expects;
// utilisation and power need NVML, which this library does not load, and read as zero.
odla_status odla_GetDeviceInfo(odla_device device, odla_device_info info, odla_scalar_value* out) {
  if (!device || !out) return ODLA_INVALID_PARAM;
  static char uuid[64], version[32];
  int n = visible_devices();
  cudaDeviceProp prop;
  bool have = n > 0 && cudaGetDeviceProperties(&prop, device->index) == cudaSuccess;
  size_t free_b = 0, total_b = 0;
  switch (info) {
    case ODLA_DEVICE_INFO_ODLA_LIB_VERSION: out->data_type = ODLA_STRING; out->val_str = odla_GetVersionString(); break;
    case ODLA_DEVICE_INFO_DEV_COUNT: out->data_type = ODLA_INT32; out->val_int32 = n; break;
    case ODLA_DEVICE_INFO_DEV_INDEX: out->data_type = ODLA_INT32; out->val_int32 = device->index; break;
    case ODLA_DEVICE_INFO_DEV_TYPE: out->data_type = ODLA_STRING; out->val_str = have ? "NVIDIA GPU" : "none"; break;
    case ODLA_DEVICE_INFO_DEV_UUID:
      out->data_type = ODLA_STRING;
      uuid[0] = 0;
      if (have) for (int i = 0; i < 16; ++i) snprintf(uuid + 2 * i, 3, "%02x", (unsigned char)prop.uuid.bytes[i]);
      out->val_str = uuid;
      break;
    case ODLA_DEVICE_INFO_PROCESSOR_UTIL: case ODLA_DEVICE_INFO_MEMORY_UTIL: case ODLA_DEVICE_INFO_POWER_USAGE:
    case ODLA_DEVICE_INFO_POWER_LIMIT: out->data_type = ODLA_FLOAT32; out->val_fp32 = 0.f; break;
    case ODLA_DEVICE_INFO_TOTAL_MEMORY: out->data_type = ODLA_UINT64; out->val_uint64 = have ? prop.totalGlobalMem : 0; break;
    case ODLA_DEVICE_INFO_USED_MEMORY:
      out->data_type = ODLA_UINT64;
      if (have && cudaSetDevice(device->index) == cudaSuccess && cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) out->val_uint64 = total_b - free_b;
      else out->val_uint64 = 0;
      break;
    case ODLA_DEVICE_INFO_DRIVER_VERSION: case ODLA_DEVICE_INFO_SDK_VERSION: {
      int v = 0;
      if (info == ODLA_DEVICE_INFO_DRIVER_VERSION) cudaDriverGetVersion(&v); else cudaRuntimeGetVersion(&v);
      snprintf(version, sizeof(version), "%d.%d", v / 1000, (v % 1000) / 10);
      out->data_type = ODLA_STRING;
      out->val_str = version;
      break;
    }
    default: return ODLA_INVALID_PARAM;
  }
  return ODLA_SUCCESS;
}

// -------------------------------------------------------------------- memory ----
odla_status odla_AllocateDeviceMemory(odla_void** p, odla_size_t size) {
  if (!p) return ODLA_INVALID_PARAM;
  B2_CUDA("alloc", cudaMalloc(p, size), ODLA_MEM_ERROR);
  return ODLA_SUCCESS;
}
odla_status odla_FreeDeviceMemory(odla_void* p) { B2_CUDA("free", cudaFree(p), ODLA_MEM_ERROR); return ODLA_SUCCESS; }
odla_status odla_AllocateHostMemory(odla_void** p, odla_size_t size) {
  if (!p) return ODLA_INVALID_PARAM;
  B2_CUDA("alloc", cudaMallocHost(p, size), ODLA_MEM_ERROR);
  return ODLA_SUCCESS;
}
odla_status odla_FreeHostMemory(odla_void* p) { B2_CUDA("free", cudaFreeHost(p), ODLA_MEM_ERROR); return ODLA_SUCCESS; }
odla_status odla_CopyMemory(odla_void* dst, odla_void* src, odla_size_t size, odla_memcpy_type type) {
  cudaMemcpyKind k = type == ODLA_MEMCPY_H2H ? cudaMemcpyHostToHost : type == ODLA_MEMCPY_H2D ? cudaMemcpyHostToDevice
                   : type == ODLA_MEMCPY_D2H ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  B2_CUDA("copy", cudaMemcpy(dst, src, size, k), ODLA_FAILURE);
  return ODLA_SUCCESS;
}

// ------------------------------------------------------ computation / context ----
odla_status odla_CreateComputation(odla_computation* computation) {
  if (!computation) return ODLA_INVALID_PARAM;
  *computation = new _odla_computation();
  g_comp = *computation;
  if (g_current_device >= 0) (*computation)->first_device = g_current_device;
  if (const char* e = getenv("ODLA_B200_DEVICE")) (*computation)->first_device = atoi(e);
  if (const char* e = getenv("ODLA_B200_NUM_GPUS")) (*computation)->n_gpus = atoi(e);
  if (const char* e = getenv("ODLA_B200_GRAPH")) (*computation)->use_graph = atoi(e) != 0;
  return ODLA_SUCCESS;
}
odla_status odla_DestroyComputation(odla_computation computation) {
  if (!computation) return ODLA_SUCCESS;
  if (g_comp == computation) g_comp = nullptr;
  // Callers may destroy the computation before its contexts, even right after an asynchronous execute
  // (ODLA/platforms/odla_popart/test/odla_compute_test.cc:302-309): wait for that work and detach the contexts.
  std::set<odla_context> ctxs;
  {
    std::lock_guard<std::mutex> lock(computation->ctx_mutex);
    ctxs.swap(computation->contexts);
  }
  for (odla_context ctx : ctxs) {
    if (ctx->worker.joinable()) ctx->worker.join();
    ctx->comp = nullptr;
  }
  delete computation;
  return ODLA_SUCCESS;
}
// Property keys follow ODLA/include/ODLA/odla_compute.h:41-70.  Boolean and integer items are
// passed as pointers to bool / int, the way the generated code does
// (lib/target/generic_cpp/generic_cxx_codegen.cc:612-648); unknown keys are refused like
// ODLA/platforms/dnnl/odla_dnnl.cc:84-96 does.
odla_status odla_SetComputationItem(odla_computation c, odla_item_type type, odla_item_value value) {
  if (!c) return ODLA_INVALID_PARAM;
  switch (type) {
    case ODLA_FP16_MODE: if (value && *(bool*)value) c->float_mode = DT_F16; else if (c->float_mode == DT_F16) c->float_mode = DT_F32; break;
    case ODLA_BF16_MODE: {
      int m = value ? *(int*)value : 0;
      if (m != BF16_DISABLE) c->float_mode = DT_BF16; else if (c->float_mode == DT_BF16) c->float_mode = DT_F32;
      break;
    }
    case ODLA_USE_DATA_TYPE: {
      odla_element_type t = value ? *(odla_element_type*)value : ODLA_FLOAT32;
      if (t == ODLA_FLOAT16) c->float_mode = DT_F16;
      else if (t == ODLA_BFLOAT16) c->float_mode = DT_BF16;
      else if (t == ODLA_FLOAT32) c->float_mode = DT_F32;
      else return ODLA_UNSUPPORTED_DATATYPE;
      break;
    }
    case ODLA_PROCESSOR_NUM: c->n_gpus = value ? *(int*)value : 0; break;
    case ODLA_AGGREGATE_OPS: c->use_graph = value ? *(bool*)value : true; break;
    case ODLA_QUANT_TABLE_SIZE: c->quant_table.resize(value ? (size_t)*(int*)value : 0); break;
    case ODLA_QUANT_TABLE:
      // `value` is the first of ODLA_QUANT_TABLE_SIZE records; the value ids are copied so the table need not outlive the call
      if (value && !c->quant_table.empty()) {
        memcpy(c->quant_table.data(), value, sizeof(odla_value_quant_info) * c->quant_table.size());
        for (auto& rec : c->quant_table) {
          if (!rec.value_id) continue;
          c->quant_names.emplace_back((const char*)rec.value_id);
          rec.value_id = (odla_value_id)c->quant_names.back().c_str();
        }
        if (c->quant_applied) B2_WARN("ODLA_QUANT_TABLE set after the computation was planned: ignored");
        c->planned = false;
      }
      break;
    case ODLA_BATCHES_PER_STEP:  // sub-batches one execute is pipelined over (copy of one under the kernels of another)
      c->sub_batches = value ? *(int*)value : 0;
      break;
    // Generated code for a dynamic-batch model sets all four of these (generic_cxx_codegen.cc, EmitComputationItems);
    // the run batch size of this library is ODLA_RUN_BATCH_SIZE on the context, so they carry no information here.
    case ODLA_DYNAMIC_BATCH: case ODLA_MIN_BATCH_SIZE: case ODLA_MAX_BATCH_SIZE: case ODLA_OPT_BATCH_SIZE:
    case ODLA_USE_SIM_MODE: case ODLA_LOAD_ENGINE_MODE: case ODLA_ENABLE_ENGINE_CACHE:
    case ODLA_CACHE_DIR:
      B2_INFO("computation item %d accepted and ignored", (int)type);
      return ODLA_SUCCESS;
    default:
      B2_ERR("unsupported computation item %d", (int)type);
      return ODLA_FAILURE;
  }
  c->planned = false;
  return ODLA_SUCCESS;
}
odla_status odla_CreateContext(odla_context* context) {
  if (!context) return ODLA_INVALID_PARAM;
  if (!g_comp) { B2_ERR("odla_CreateContext: no current computation"); return ODLA_FAILURE; }
  if (!g_comp->first_error.empty()) {
    B2_ERR("computation has a build error: %s", g_comp->first_error.c_str());
    return g_comp->error_status;
  }
  *context = new _odla_context();
  (*context)->comp = g_comp;
  {
    // The first context takes lane 0; each further one takes the free lane with the lowest number (a lane of its
    // own: it may then execute while the others do), or shares the least used one when all are taken.
    std::lock_guard<std::mutex> lock(g_comp->ctx_mutex);
    int max_lanes = 2;
    if (const char* e = getenv("ODLA_B200_CONTEXT_LANES")) max_lanes = std::max(1, std::min(8, atoi(e)));
    std::vector<int> users((size_t)max_lanes, 0);
    for (auto* other : g_comp->contexts) users[(size_t)std::min(other->lane, max_lanes - 1)]++;
    int lane = 0;
    for (int k = 1; k < max_lanes; ++k) if (users[(size_t)k] < users[(size_t)lane]) lane = k;
    if (lane > 0) {
      std::lock_guard<std::recursive_mutex> plan_lock(g_comp->plan_mutex);
      while ((int)g_comp->lanes.size() < lane) g_comp->lanes.emplace_back(new b200::Lane());
      g_comp->multi_lane.store(true);
    }
    (*context)->lane = lane;
    g_comp->contexts.insert(*context);
  }
  return ODLA_SUCCESS;
}
odla_status odla_DestroyContext(odla_context context) {
  if (!context) return ODLA_SUCCESS;
  if (context->worker.joinable()) context->worker.join();  // an asynchronous execute still owns the bindings
  if (context->comp) {
    std::lock_guard<std::mutex> lock(context->comp->ctx_mutex);
    context->comp->contexts.erase(context);
  }
  delete context;
  return ODLA_SUCCESS;
}
// ODLA_RUN_BATCH_SIZE: `value` points to an int, as for the TensorRT platform (ODLA/platforms/tensorrt/odla_tensorrt.cc:284-301).
// ODLA_ASYNC_CALLBACK_FUNC / _ARG: `value` is the function pointer / the argument itself, as for the PopART
// platform (ODLA/platforms/odla_popart/odla_compute.cc:85-100); the callback is int (*)(void* arg, odla_status).
odla_status odla_SetContextItem(odla_context context, odla_item_type type, odla_item_value value) {
  if (!context) return ODLA_INVALID_PARAM;
  if (context->worker.joinable()) context->worker.join();
  switch (type) {
    case ODLA_RUN_BATCH_SIZE: {
      if (!value) return ODLA_INVALID_PARAM;
      int bs = *(int*)value;
      if (bs < 0) return ODLA_FAILURE;
      context->run_batch = bs;
      return ODLA_SUCCESS;
    }
    case ODLA_ASYNC_CALLBACK_FUNC: context->async_fn = (int (*)(void*, odla_status))value; return ODLA_SUCCESS;
    case ODLA_ASYNC_CALLBACK_ARG: context->async_arg = (void*)value; return ODLA_SUCCESS;
    default: break;
  }
  B2_ERR("unsupported context item %d", (int)type);
  return ODLA_FAILURE;
}
odla_status odla_GetNumOfArgsFromComputation(const odla_computation c, odla_uint32* n) {
  if (!c || !n) return ODLA_INVALID_PARAM;
  *n = (odla_uint32)c->args.size();
  return ODLA_SUCCESS;
}
odla_status odla_GetArgFromComputationByIdx(const odla_computation c, const odla_uint32 i, odla_value* v) {
  if (!c || !v || i >= c->args.size()) return ODLA_INVALID_PARAM;
  *v = c->args[i];
  return ODLA_SUCCESS;
}
odla_status odla_GetNumOfOutputsFromComputation(const odla_computation c, odla_uint32* n) {
  if (!c || !n) return ODLA_INVALID_PARAM;
  *n = (odla_uint32)c->outs.size();
  return ODLA_SUCCESS;
}
odla_status odla_GetOutputFromComputationByIdx(const odla_computation c, const odla_uint32 i, odla_value* v) {
  if (!c || !v || i >= c->outs.size()) return ODLA_INVALID_PARAM;
  *v = c->outs[i];
  return ODLA_SUCCESS;
}
odla_status odla_SetValueShapeInfo(odla_value, odla_item_type, odla_value_shape) { return ODLA_SUCCESS; }
odla_status odla_GetRuntimeShape(odla_context context, odla_value value, odla_value_shape* shape) {
  if (!value || !shape) return ODLA_INVALID_PARAM;
  *shape = value->type.shape;
  // with ODLA_RUN_BATCH_SIZE set, dim 0 of a batched value follows it
  if (context && context->run_batch > 0 && context->comp && context->comp->planned && context->comp->shardable && shape->size > 0 &&
      context->comp->graph_batch > 0 && shape->dims[0] % context->comp->graph_batch == 0 && value->kind != OP_CONST)
    shape->dims[0] = shape->dims[0] / context->comp->graph_batch * context->run_batch;
  return ODLA_SUCCESS;
}
odla_status odla_GetValueType(const odla_value value, odla_value_type* type) {
  if (!value || !type) return ODLA_INVALID_PARAM;
  *type = value->type;
  return ODLA_SUCCESS;
}
odla_status odla_GetValueId(const odla_value value, odla_value_id* id) {
  if (!value || !id) return ODLA_INVALID_PARAM;
  *id = (odla_value_id)value->name.c_str();
  return ODLA_SUCCESS;
}
odla_status odla_SetValueAsOutput(odla_value value) {
  if (!value || !g_comp) return ODLA_INVALID_PARAM;
  value->is_output = true;
  g_comp->outs.push_back(value);
  g_comp->planned = false;
  return ODLA_SUCCESS;
}
odla_status odla_SetValuesAsOutput(odla_values values) {
  for (size_t i = 0; i < values.size; ++i) {
    odla_status s = odla_SetValueAsOutput(values.values[i]);
    if (s != ODLA_SUCCESS) return s;
  }
  return ODLA_SUCCESS;
}
odla_status odla_BindToArgument(odla_value value, const odla_void* data, odla_context ctx) {
  if (!value || !ctx || !data) return ODLA_INVALID_PARAM;
  if (value->kind != OP_ARG) { B2_ERR("odla_BindToArgument: '%s' is not an argument", value->name.c_str()); return ODLA_INVALID_PARAM; }
  ctx->in[value] = data;
  return ODLA_SUCCESS;
}
odla_status odla_BindToArgumentById(const odla_value_id id, const odla_void* data, odla_context ctx) {
  if (!ctx || !ctx->comp || !id) return ODLA_INVALID_PARAM;
  auto it = ctx->comp->by_name.find((const char*)id);
  if (it == ctx->comp->by_name.end()) { B2_ERR("odla_BindToArgumentById: unknown value '%s'", (const char*)id); return ODLA_INVALID_PARAM; }
  return odla_BindToArgument(it->second, data, ctx);
}
odla_status odla_BindToOutput(odla_value value, odla_void* data, odla_context ctx) {
  if (!value || !ctx || !data) return ODLA_INVALID_PARAM;
  if (!value->is_output) { B2_ERR("odla_BindToOutput: '%s' was not marked as an output", value->name.c_str()); return ODLA_INVALID_PARAM; }
  ctx->out[value] = data;
  return ODLA_SUCCESS;
}
odla_status odla_BindToOutputById(const odla_value_id id, odla_void* data, odla_context ctx) {
  if (!ctx || !ctx->comp || !id) return ODLA_INVALID_PARAM;
  auto it = ctx->comp->by_name.find((const char*)id);
  if (it == ctx->comp->by_name.end()) { B2_ERR("odla_BindToOutputById: unknown value '%s'", (const char*)id); return ODLA_INVALID_PARAM; }
  return odla_BindToOutput(it->second, data, ctx);
}
static odla_status execute_locked(odla_computation c, odla_context ctx) {
  // Contexts of one computation may be driven from different threads.  Those on one lane share that lane's per-GPU
  // arenas and streams and are serialised here; contexts on different lanes run side by side.
  std::mutex* lane_mutex = &c->exec_mutex;
  {
    std::lock_guard<std::recursive_mutex> plan_lock(c->plan_mutex);
    if (ctx->lane > 0 && ctx->lane <= (int)c->lanes.size()) lane_mutex = &c->lanes[(size_t)ctx->lane - 1]->exec_mutex;
  }
  std::lock_guard<std::mutex> lock(*lane_mutex);
  odla_status s = ensure_planned(c);
  if (s != ODLA_SUCCESS) return s;
  return execute(c, ctx);
}
// Returns once the work is handed to a worker thread; when it has finished (outputs written) the context's
// callback, if set, is called with its argument and the status -- the shape of the PopART platform's asynchronous
// execute (ODLA/platforms/odla_popart/odla_compute.cc:262-291).  Bindings must not change until then; the next
// execute / item / destroy call on the context waits for it, and odla_b200_WaitContext returns its status.
odla_status odla_AsyncExecuteComputation(const odla_computation c, const odla_context ctx, const odla_compute_mode mode, odla_device) {
  if (!c || !ctx) return ODLA_INVALID_PARAM;
  if (mode == ODLA_COMPUTE_TRAINING) return ODLA_UNSUPPORTED_OP;
  if (!c->first_error.empty()) { B2_ERR("computation has a build error: %s", c->first_error.c_str()); return c->error_status; }
  if (ctx->worker.joinable()) ctx->worker.join();
  for (auto a : c->args)
    if (!ctx->in.count(a)) { B2_ERR("argument '%s' is not bound", a->name.c_str()); return ODLA_INVALID_PARAM; }
  ctx->async_status = ODLA_SUCCESS;
  try {
    ctx->worker = std::thread([c, ctx]() {
      odla_status s = execute_locked(c, ctx);
      ctx->async_status = s;
      if (ctx->async_fn) ctx->async_fn(ctx->async_arg, s);
    });
  } catch (...) {
    B2_ERR("could not start a worker thread");
    return ODLA_FAILURE;
  }
  return ODLA_SUCCESS;
}
int odla_b200_ContextLane(odla_context ctx) { return ctx ? ctx->lane : -1; }
odla_status odla_b200_WaitContext(odla_context ctx) {
  if (!ctx) return ODLA_INVALID_PARAM;
  if (ctx->worker.joinable()) ctx->worker.join();
  return ctx->async_status;
}
odla_status odla_ExecuteComputation(const odla_computation c, const odla_context ctx, const odla_compute_mode mode, odla_device) {
  if (!c || !ctx) return ODLA_INVALID_PARAM;
  if (mode == ODLA_COMPUTE_TRAINING) return ODLA_UNSUPPORTED_OP;
  if (ctx->worker.joinable()) ctx->worker.join();
  if (!c->first_error.empty()) { B2_ERR("computation has a build error: %s", c->first_error.c_str()); return c->error_status; }
  return execute_locked(c, ctx);
}
// The executable is the planned computation itself; these two exist so callers written against
// the TensorRT platform's compile/launch pair (ODLA/platforms/tensorrt/odla_tensorrt.cc:561-701)
// link and run.
odla_status odla_CompileComputation(const odla_computation c, const odla_device, odla_executable* exe) {
  if (!c || !exe) return ODLA_INVALID_PARAM;
  if (!c->first_error.empty()) return c->error_status;
  odla_status s = ensure_planned(c);
  *exe = (odla_executable)c;
  return s;
}
odla_status odla_LaunchExecutable(odla_executable exe, odla_context ctx) {
  return odla_ExecuteComputation((odla_computation)exe, ctx, ODLA_COMPUTE_INFERENCE, nullptr);
}
odla_status odla_DestroyExecutable(odla_executable) { return ODLA_SUCCESS; }

// ------------------------------------------------------------ leaf values ----
odla_value odla_CreateArgument(const odla_value_type type, const odla_value_id id) {
  odla_value v = add_node(OP_ARG, type.element_type, type.shape, id, {});
  if (v) g_comp->args.push_back(v);
  return v;
}
odla_value odla_CreateConstant(const odla_value_type type, const odla_void* data, const odla_value_id id) {
  if (!data) return fail_node(ODLA_INVALID_PARAM, id, "odla_CreateConstant: null data pointer");
  odla_value v = add_node(OP_CONST, type.element_type, type.shape, id, {});
  if (v) v->host = data;
  return v;
}

// ------------------------------------------------------------------- nn ops ----
odla_value odla_Conv(odla_value input, odla_memory_layout il, odla_uint32 group, odla_value kernel, odla_memory_layout kl,
                     const odla_uint32* strides, const odla_uint32* dilations, const odla_uint32* pf, const odla_uint32* pb,
                     odla_value bias, odla_value_shape od, const odla_value_id id) {
  if (any_null({input, kernel}) || !strides || !pf || !pb) return fail_node(ODLA_INVALID_PARAM, id, "odla_Conv: null operand");
  if (input->type.shape.size != 4 || kernel->type.shape.size != 4 || od.size != 4)
    return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Conv: only 2-d convolution (rank-4 tensors) is supported");
  if (dilations && (dilations[0] != 1 || dilations[1] != 1))
    return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Conv: dilation must be 1");
  bool nhwc = il == ODLA_CHANNELS_LAST;
  if (!((nhwc && kl == ODLA_SIO) || (il == ODLA_CHANNELS_FIRST && kl == ODLA_OIS)))
    return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Conv: supported layout pairs are CHANNELS_LAST+SIO and CHANNELS_FIRST+OIS");
  if (group == 0) group = 1;
  return add_node(OP_CONV, input->type.element_type == ODLA_INT8 ? ODLA_INT32 : input->type.element_type, od, id,
                  {input, kernel, bias},
                  {nhwc, group, strides[0], strides[1], pf[0], pf[1], pb[0], pb[1]});
}
odla_value odla_Gemm(odla_value A, odla_bool ta, odla_value B, odla_bool tb, odla_float32 alpha, odla_float32 beta, odla_value C,
                     odla_value_shape od, const odla_value_id id) {
  if (any_null({A, B})) return fail_node(ODLA_INVALID_PARAM, id, "odla_Gemm: null operand");
  if (A->type.shape.size < 2 || B->type.shape.size < 2) return fail_node(ODLA_INVALID_PARAM, id, "odla_Gemm: operands need rank >= 2");
  return add_node(OP_GEMM, A->type.element_type, od, id, {A, B, C}, {ta != 0, tb != 0}, {alpha, beta});
}
odla_value odla_BatchMatMul(odla_value A, odla_bool ta, odla_value B, odla_bool tb, odla_value_shape od, const odla_value_id id) {
  return odla_Gemm(A, ta, B, tb, 1.f, 0.f, nullptr, od, id);
}
static odla_value pool_node(OpKind kind, odla_value input, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st,
                            const odla_uint32* pf, const odla_uint32* pb, int included, odla_value_shape od, const odla_value_id id) {
  if (!input || !win || !st || !pf || !pb) return fail_node(ODLA_INVALID_PARAM, id, "pooling: null operand");
  if (input->type.shape.size != 4) return fail_node(ODLA_UNSUPPORTED_OP, id, "pooling: only 2-d pooling is supported");
  return add_node(kind, input->type.element_type, od, id, {input},
                  {il == ODLA_CHANNELS_LAST, win[0], win[1], st[0], st[1], pf[0], pf[1], pb[0], pb[1], included});
}
odla_value odla_MaxPool(odla_value input, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st, const odla_uint32* pf,
                        const odla_uint32* pb, odla_value_shape od, const odla_value_id id) {
  return pool_node(OP_MAXPOOL, input, il, win, st, pf, pb, 0, od, id);
}
odla_value odla_AveragePool(odla_value input, odla_memory_layout il, const odla_uint32* win, const odla_uint32* st, const odla_uint32* pf,
                            const odla_uint32* pb, odla_bool included, odla_value_shape od, const odla_value_id id) {
  return pool_node(OP_AVGPOOL, input, il, win, st, pf, pb, included != 0, od, id);
}
odla_value odla_BatchNormalization(odla_value input, odla_memory_layout il, odla_value mean, odla_value var, odla_float32 eps,
                                   odla_value scale, odla_value offset, odla_float32 ss, odla_float32 so, const odla_value_id id) {
  if (any_null({input, mean, var})) return fail_node(ODLA_INVALID_PARAM, id, "odla_BatchNormalization: null operand");
  for (odla_value c : {mean, var, scale, offset})
    if (c && c->kind != OP_CONST) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_BatchNormalization: statistics must be constants");
  return add_node(OP_BATCHNORM, input->type.element_type, input->type.shape, id, {input, mean, var, scale, offset},
                  {il == ODLA_CHANNELS_LAST}, {eps, ss, so});
}
static odla_value unary_node(int op, odla_value x, float a, float b, const odla_value_id id, const char* what) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "%s: null operand", what);
  return add_node(OP_UNARY, x->type.element_type, x->type.shape, id, {x}, {op}, {a, b});
}
odla_value odla_Relu(odla_value x, const odla_value_id id) { return unary_node(UN_RELU, x, 0, 0, id, "odla_Relu"); }
odla_value odla_LeakyRelu(odla_value x, odla_float32 alpha, const odla_value_id id) { return unary_node(UN_LEAKY, x, alpha, 0, id, "odla_LeakyRelu"); }
odla_value odla_Clamp(odla_value x, odla_float32 lo, odla_float32 hi, const odla_value_id id) { return unary_node(UN_CLAMP, x, lo, hi, id, "odla_Clamp"); }
odla_value odla_Gelu(odla_value x, odla_bool approx, const odla_value_id id) { return unary_node(approx ? UN_GELU_TANH : UN_GELU_ERF, x, 0, 0, id, "odla_Gelu"); }
odla_value odla_Erf(odla_value x, const odla_value_id id) { return unary_node(UN_ERF, x, 0, 0, id, "odla_Erf"); }
odla_value odla_Sigmoid(odla_value x, const odla_value_id id) { return unary_node(UN_SIGMOID, x, 0, 0, id, "odla_Sigmoid"); }
odla_value odla_Tanh(odla_value x, const odla_value_id id) { return unary_node(UN_TANH, x, 0, 0, id, "odla_Tanh"); }
odla_value odla_Exp(odla_value x, const odla_value_id id) { return unary_node(UN_EXP, x, 0, 0, id, "odla_Exp"); }
odla_value odla_Log(odla_value x, const odla_value_id id) { return unary_node(UN_LOG, x, 0, 0, id, "odla_Log"); }
odla_value odla_Sqrt(odla_value x, const odla_value_id id) { return unary_node(UN_SQRT, x, 0, 0, id, "odla_Sqrt"); }
odla_value odla_Rsqrt(odla_value x, const odla_value_id id) { return unary_node(UN_RSQRT, x, 0, 0, id, "odla_Rsqrt"); }
odla_value odla_Abs(odla_value x, const odla_value_id id) { return unary_node(UN_ABS, x, 0, 0, id, "odla_Abs"); }
odla_value odla_Neg(odla_value x, const odla_value_id id) { return unary_node(UN_NEG, x, 0, 0, id, "odla_Neg"); }
odla_value odla_Reciprocal(odla_value x, const odla_value_id id) { return unary_node(UN_RECIP, x, 0, 0, id, "odla_Reciprocal"); }
odla_value odla_Round(odla_value x, const odla_value_id id) { return unary_node(UN_ROUND, x, 0, 0, id, "odla_Round"); }

// Binary ops broadcast numpy style with right-aligned dimensions
// (ODLA/platforms/dnnl/odla_dnnl.h:301-343).
static odla_value binary_node(int op, odla_value l, odla_value r, const odla_value_id id, const char* what) {
  if (any_null({l, r})) return fail_node(ODLA_INVALID_PARAM, id, "%s: null operand", what);
  const auto &ls = l->type.shape, &rs = r->type.shape;
  odla_value_shape os;
  os.size = ls.size > rs.size ? ls.size : rs.size;
  for (int i = 0; i < os.size; ++i) {
    int li = i - (os.size - ls.size), ri = i - (os.size - rs.size);
    int64_t a = li >= 0 ? ls.dims[li] : 1, b = ri >= 0 ? rs.dims[ri] : 1;
    if (a != b && a != 1 && b != 1) return fail_node(ODLA_INVALID_PARAM, id, "%s: shapes do not broadcast", what);
    os.dims[i] = a > b ? a : b;
  }
  return add_node(OP_BINARY, l->type.element_type, os, id, {l, r}, {op});
}
odla_value odla_Add(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_ADD, l, r, id, "odla_Add"); }
odla_value odla_Sub(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_SUB, l, r, id, "odla_Sub"); }
odla_value odla_Mul(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_MUL, l, r, id, "odla_Mul"); }
odla_value odla_Div(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_DIV, l, r, id, "odla_Div"); }
odla_value odla_Pow(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_POW, l, r, id, "odla_Pow"); }
odla_value odla_PRelu(odla_value l, odla_value r, const odla_value_id id) { return binary_node(BIN_PRELU, l, r, id, "odla_PRelu"); }

static odla_value softmax_node(odla_value x, int axis, int log_form, const odla_value_id id) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "odla_Softmax: null operand");
  int rank = x->type.shape.size;
  if (axis < 0) axis += rank;
  if (axis < 0 || axis >= rank) return fail_node(ODLA_INVALID_PARAM, id, "odla_Softmax: axis out of range");
  return add_node(OP_SOFTMAX, x->type.element_type, x->type.shape, id, {x}, {axis, log_form});
}
odla_value odla_Softmax(odla_value x, odla_int32 axis, const odla_value_id id) { return softmax_node(x, axis, 0, id); }
odla_value odla_LogSoftmax(odla_value x, odla_int32 axis, const odla_value_id id) { return softmax_node(x, axis, 1, id); }

odla_value odla_ReduceMean(odla_value x, odla_size_t n_axes, const odla_uint32* axes, odla_bool keep, odla_value_shape od,
                           const odla_value_id id) {
  if (!x || (n_axes && !axes)) return fail_node(ODLA_INVALID_PARAM, id, "odla_ReduceMean: null operand");
  std::vector<int64_t> ia{keep != 0};
  for (size_t i = 0; i < n_axes; ++i) {
    if ((int)axes[i] >= x->type.shape.size) return fail_node(ODLA_INVALID_PARAM, id, "odla_ReduceMean: axis out of range");
    ia.push_back(axes[i]);
  }
  return add_node(OP_REDUCE_MEAN, x->type.element_type, od, id, {x}, ia);
}
odla_value odla_LayerNorm(odla_value x, odla_int32 n_axes, const odla_int32* axes, odla_float32 eps, odla_value scale, odla_value offset,
                          const odla_value_id id) {
  if (!x || n_axes <= 0 || !axes) return fail_node(ODLA_INVALID_PARAM, id, "odla_LayerNorm: null operand");
  int rank = x->type.shape.size, first = rank;
  for (int i = 0; i < n_axes; ++i) {
    int a = axes[i] < 0 ? axes[i] + rank : axes[i];
    if (a < first) first = a;
  }
  if (first != rank - n_axes) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_LayerNorm: axes must be the trailing dimensions");
  for (odla_value c : {scale, offset})
    if (c && c->kind != OP_CONST) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_LayerNorm: scale/offset must be constants");
  return add_node(OP_LAYERNORM, x->type.element_type, x->type.shape, id, {x, scale, offset}, {n_axes}, {eps});
}

// ----------------------------------------------------------- quantisation ----
odla_value odla_Quantize(odla_value x, odla_value scale, odla_value zp, odla_int32 axis, odla_element_type target, const odla_value_id id) {
  if (any_null({x, scale})) return fail_node(ODLA_INVALID_PARAM, id, "odla_Quantize: null operand");
  if (target != ODLA_INT8 && target != ODLA_UINT8 && target != ODLA_QINT8 && target != ODLA_QUINT8)
    return fail_node(ODLA_UNSUPPORTED_DATATYPE, id, "odla_Quantize: target type must be int8 or uint8");  // odla_dnnl_quantization.cc:68
  if (scale->kind != OP_CONST || (zp && zp->kind != OP_CONST)) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Quantize: scale and zero point must be constants");
  if (axis < 0) axis += x->type.shape.size;
  return add_node(OP_QUANTIZE, (target == ODLA_INT8 || target == ODLA_QINT8) ? ODLA_INT8 : ODLA_UINT8, x->type.shape, id, {x, scale, zp}, {axis});
}
odla_value odla_Dequantize(odla_value x, odla_value scale, odla_value zp, odla_int32 axis, odla_element_type target, const odla_value_id id) {
  if (any_null({x, scale})) return fail_node(ODLA_INVALID_PARAM, id, "odla_Dequantize: null operand");
  if (!is_float_type(target)) return fail_node(ODLA_UNSUPPORTED_DATATYPE, id, "odla_Dequantize: target type must be a float type");
  if (scale->kind != OP_CONST || (zp && zp->kind != OP_CONST)) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Dequantize: scale and zero point must be constants");
  if (axis < 0) axis += x->type.shape.size;
  return add_node(OP_DEQUANTIZE, target, x->type.shape, id, {x, scale, zp}, {axis});
}

// ----------------------------------------------------------- data movement ----
odla_value odla_Reshape(odla_value x, odla_value_shape od, const odla_value_id id) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "odla_Reshape: null operand");
  if (numel(od) != numel(x->type.shape)) return fail_node(ODLA_INVALID_PARAM, id, "odla_Reshape: element count differs");
  return add_node(OP_RESHAPE, x->type.element_type, od, id, {x});
}
odla_value odla_Transpose(odla_value x, odla_value_shape perm, odla_value_shape od, const odla_value_id id) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "odla_Transpose: null operand");
  if (perm.size != x->type.shape.size) return fail_node(ODLA_INVALID_PARAM, id, "odla_Transpose: permutation rank differs");
  std::vector<int64_t> p(perm.dims, perm.dims + perm.size);
  return add_node(OP_TRANSPOSE, x->type.element_type, od, id, {x}, p);
}
odla_value odla_Concat(odla_values inputs, odla_int32 axis, odla_value_shape od, const odla_value_id id) {
  if (inputs.size == 0) return fail_node(ODLA_INVALID_PARAM, id, "odla_Concat: no inputs");
  std::vector<odla_value> in(inputs.values, inputs.values + inputs.size);
  for (auto v : in)
    if (!v) return fail_node(ODLA_INVALID_PARAM, id, "odla_Concat: null operand");
  if (axis < 0) axis += od.size;
  return add_node(OP_CONCAT, in[0]->type.element_type, od, id, in, {axis});
}
odla_value odla_Resize(odla_value x, odla_interpolation_mode interp, odla_resize_coordinate_mode mode, odla_uint32 mask,
                       odla_value_shape od, const odla_value_id id) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "odla_Resize: null operand");
  if (interp != ODLA_NEAREST || x->type.shape.size != 4) return fail_node(ODLA_UNSUPPORTED_OP, id, "odla_Resize: only nearest-neighbour on rank-4 tensors");
  return add_node(OP_RESIZE, x->type.element_type, od, id, {x}, {interp, mode, mask});
}
odla_value odla_Gather(odla_value x, odla_value idx, odla_int32 axis, odla_value_shape od, const odla_value_id id) {
  if (any_null({x, idx})) return fail_node(ODLA_INVALID_PARAM, id, "odla_Gather: null operand");
  if (axis < 0) axis += x->type.shape.size;
  return add_node(OP_GATHER, x->type.element_type, od, id, {x, idx}, {axis});
}
odla_value odla_Slice(odla_value x, const odla_int32* start, const odla_int32* end, const odla_int32* stride, odla_value_shape od,
                      const odla_value_id id) {
  if (!x || !start || !end) return fail_node(ODLA_INVALID_PARAM, id, "odla_Slice: null operand");
  int rank = x->type.shape.size;
  std::vector<int64_t> ia;
  for (int i = 0; i < rank; ++i) ia.push_back(start[i]);
  for (int i = 0; i < rank; ++i) ia.push_back(stride ? stride[i] : 1);
  return add_node(OP_SLICE, x->type.element_type, od, id, {x}, ia);
}
// ODLA/include/ODLA/ops/odla_ops_nn.h:504-507.  The emitter maps ONNX NonMaxSuppression to it
// (lib/target/generic_cpp/nms.cc:22-69) with the result typed [max_num_outputs, 3]: rows (batch, class, box), -1 in rows
// that no selection fills.  boxes [B, N, 4], scores [B, C, N]; at most max_num_outputs boxes per (batch, class).
odla_value odla_NMS(odla_value boxes, odla_value scores, odla_uint32 max_num_outputs, odla_float32 iou_threshold, odla_float32 score_threshold,
                    odla_value_type output_value_type, const odla_value_id id) {
  if (any_null({boxes, scores})) return fail_node(ODLA_INVALID_PARAM, id, "odla_NMS: null operand");
  const auto& bs = boxes->type.shape; const auto& ss = scores->type.shape;
  if (bs.size != 3 || ss.size != 3 || bs.dims[2] != 4 || bs.dims[0] != ss.dims[0] || bs.dims[1] != ss.dims[2])
    return fail_node(ODLA_INVALID_PARAM, id, "odla_NMS: boxes must be [B, N, 4] and scores [B, C, N]");
  if (output_value_type.element_type != ODLA_INT32 && output_value_type.element_type != ODLA_INT64)
    return fail_node(ODLA_UNSUPPORTED_DATATYPE, id, "odla_NMS: the result is int32 or int64");
  if (output_value_type.shape.size != 2 || output_value_type.shape.dims[1] != 3)
    return fail_node(ODLA_INVALID_PARAM, id, "odla_NMS: the result is [rows, 3]");
  return add_node(OP_NMS, output_value_type.element_type, output_value_type.shape, id, {boxes, scores}, {(int64_t)max_num_outputs}, {iou_threshold, score_threshold});
}
// ODLA/include/ODLA/ops/odla_ops_nn.h:757-759; semantics of the only implementation the reference has
// (ODLA/platforms/odla_popart/custom_ops/postprocess.cc, codelets_nms.cpp): YOLOv3 heads at 13, 26 and 52 cells, batch 1,
// decoded against the 9 anchors, per class a greedy suppression at IoU 0.45 / score 0.3 -> selected_info
// [classes, N/169, 5] (y_min, x_min, y_max, x_max, score) and selected_num [classes].
odla_values odla_PostProcess(odla_value orig_img_w, odla_value orig_img_h, odla_value bb13, odla_value bb26, odla_value bb52, const odla_value_id id) {
  odla_values out{};
  const std::string base = id ? std::string((const char*)id) : std::string("postprocess");
  const std::string n0 = base + "0", n1 = base + "1";
  auto failed = [&](odla_status st, const char* msg) { out.size = 2; out.values[0] = fail_node(st, (const odla_value_id)n0.c_str(), "%s", msg); out.values[1] = out.values[0]; return out; };
  if (any_null({orig_img_w, orig_img_h, bb13, bb26, bb52})) return failed(ODLA_INVALID_PARAM, "odla_PostProcess: null operand");
  int64_t ch = -1;
  const int want[3] = {13, 26, 52};
  odla_value heads[3] = {bb13, bb26, bb52};
  for (int i = 0; i < 3; ++i) {
    const auto& s = heads[i]->type.shape;
    if (s.size != 4 || s.dims[0] != 1) return failed(ODLA_INVALID_PARAM, "odla_PostProcess: heads are rank 4 with batch 1");
    const bool nchw = s.dims[2] == want[i] && s.dims[3] == want[i], nhwc = s.dims[1] == want[i] && s.dims[2] == want[i];
    if (!nchw && !nhwc) return failed(ODLA_INVALID_PARAM, "odla_PostProcess: heads must have 13, 26 and 52 cells");
    const int64_t c = nchw ? s.dims[1] : s.dims[3];
    if ((ch >= 0 && c != ch) || c % 3 != 0 || c / 3 <= 5) return failed(ODLA_INVALID_PARAM, "odla_PostProcess: heads must have 3 * (classes + 5) channels");
    ch = c;
  }
  const int64_t cls = ch / 3 - 5, N = 3 * (13 * 13 + 26 * 26 + 52 * 52);
  odla_value_shape s0{3, {cls, N / 169, 5}}, s1{1, {cls}};
  odla_value info = add_node(OP_POSTPROCESS, ODLA_FLOAT32, s0, (const odla_value_id)n0.c_str(), {orig_img_w, orig_img_h, bb13, bb26, bb52}, {cls});
  odla_value num = add_node(OP_POSTPROCESS_NUM, ODLA_UINT32, s1, (const odla_value_id)n1.c_str(), {info}, {cls});
  out.size = 2; out.values[0] = info; out.values[1] = num;
  return out;
}
odla_value odla_Cast(odla_value x, odla_element_type target, const odla_value_id id) {
  if (!x) return fail_node(ODLA_INVALID_PARAM, id, "odla_Cast: null operand");
  return add_node(OP_CAST, target, x->type.shape, id, {x}, {target});
}

}  // extern "C"
