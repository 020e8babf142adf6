// Internal definitions of libodla_b200.so: the recorded graph, the launch plan and the
// per-GPU replicas.  The opaque ODLA handle types are defined here, privately, in the same
// spirit as ODLA/platforms/dnnl/odla_dnnl.h:43-108 and
// ODLA/platforms/tensorrt/odla_tensorrt.h:183-312 in the reference.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <deque>
#include <functional>
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "../../include/odla_b200.h"
#include "kernels.h"

namespace b200 {

// ---------------------------------------------------------------- logging ----
void log_msg(const char* file, int line, const char* func, odla_log_level lvl, const char* fmt, ...);
#define B2_LOG(lvl, ...) ::b200::log_msg(__FILE__, __LINE__, __func__, lvl, __VA_ARGS__)
#define B2_ERR(...) B2_LOG(ODLA_LOG_LEVEL_ERROR, __VA_ARGS__)
#define B2_WARN(...) B2_LOG(ODLA_LOG_LEVEL_WARN, __VA_ARGS__)
#define B2_INFO(...) B2_LOG(ODLA_LOG_LEVEL_INFO, __VA_ARGS__)
#define B2_DEBUG(...) B2_LOG(ODLA_LOG_LEVEL_DEBUG, __VA_ARGS__)

// Host-side fault injection for tests: the environment variable ODLA_B200_INJECT holds
// "<site>@<n>" with site one of h2d, launch, d2h, peer, alloc; the n-th call (1-based) of
// that site reports cudaErrorUnknown without touching the device.
bool inject_fault(const char* site);

// Evaluates a CUDA runtime call; on failure logs and makes the enclosing function return `ret`.
#define B2_CUDA(site, expr, ret)                                                        \
  do {                                                                                  \
    cudaError_t e__ = ::b200::inject_fault(site) ? cudaErrorUnknown : (expr);           \
    if (e__ != cudaSuccess) {                                                           \
      B2_ERR("CUDA call failed (%s): %s -> %s", site, #expr, cudaGetErrorString(e__));  \
      return ret;                                                                       \
    }                                                                                   \
  } while (0)

// ------------------------------------------------------------ graph nodes ----
enum OpKind {
  OP_ARG, OP_CONST, OP_CONV, OP_GEMM, OP_MAXPOOL, OP_AVGPOOL, OP_BATCHNORM, OP_UNARY, OP_BINARY,
  OP_SOFTMAX, OP_REDUCE_MEAN, OP_LAYERNORM, OP_QUANTIZE, OP_DEQUANTIZE, OP_RESHAPE, OP_TRANSPOSE,
  OP_CONCAT, OP_RESIZE, OP_GATHER, OP_SLICE, OP_CAST, OP_NMS, OP_POSTPROCESS, OP_POSTPROCESS_NUM
};
const char* op_name(OpKind k);

int elem_size(odla_element_type t);
bool is_float_type(odla_element_type t);
int64_t numel(const odla_value_shape& s);
int storage_size(int dt);  // bytes per element of a DT_* storage type

}  // namespace b200

struct _odla_value {
  std::string name;
  odla_value_type type;            // as seen through the API (shape includes the batch)
  b200::OpKind kind = b200::OP_ARG;
  std::vector<odla_value> in;      // operands (may hold nullptr for absent optionals)
  std::vector<int64_t> ia;         // integer attributes, meaning depends on kind
  std::vector<float> fa;           // float attributes
  const void* host = nullptr;      // caller-owned constant data (read at plan time only)
  int index = 0;                   // position in the computation's node list
  bool is_output = false;
  bool poison = false;             // produced by a failed builder call
};

namespace b200 {

// One entry of the launch list.  `fn` issues exactly the kernels of this entry on `stream`.
struct Launch {
  std::string op;     // kernel family
  std::string name;   // id of the value it materialises
  double flops = 0, bytes = 0;
  int n_kernels = 1;
  // returns 0 on success
  std::function<int(cudaStream_t)> fn;
  // profiling accumulators
  double prof_ms = 0;
  long long prof_n = 0;
  // what the entry leaves in memory, for range profiling (out_ptr == nullptr: not a dense tensor of out_count elements)
  const _odla_value* out_v = nullptr;
  const void* out_ptr = nullptr;
  int out_dt = 0;
  int64_t out_count = 0, out_channels = 1;
  unsigned* range_stats = nullptr;   // device: [2 + 2 * out_channels] order-preserving keys of min / max, whole tensor then per channel
};

// Where a value lives inside a replica's arena.
struct Slot {
  int64_t offset = -1, bytes = 0;
  int dt = DT_F32;                 // storage type
  bool constant = false;           // lives in the constant pool instead of the arena
};

// A plan specialised for one batch size on one GPU.
struct Plan {
  int64_t batch = 0;               // extent of dim 0 this plan was built for
  int device = 0;
  std::vector<Launch> launches;
  std::map<const _odla_value*, Slot> slots;
  char* arena = nullptr;           // activations and staging
  int64_t arena_bytes = 0;
  char* consts = nullptr;          // converted / repacked constants
  int64_t const_bytes = 0;
  int* status = nullptr;           // device status block (kStatusBytes): word 0 non-zero when a bounded wait expired
  std::vector<void*> extra_allocs; // uploaded constants and scratch
  std::vector<UmmaLaunch*> umma;   // prepared tensor-core launches (own their tensor maps)
  std::vector<AttnLaunch*> attn;   // prepared fused-attention launches
  std::map<const _odla_value*, unsigned*> pp_counts;  // odla_PostProcess: where a node's per-class counts are on the device
  cudaGraphExec_t graph = nullptr; // captured launch list (optional)
  bool graph_failed = false;       // capture was tried and refused: stay on plain launches
  // How arguments enter and outputs leave the arena.  `stage` is where the caller's bytes land
  // (API element type); it equals `slot` when no conversion kernel is needed.
  struct Io {
    const _odla_value* v = nullptr;
    int64_t slot = -1, stage = -1;
    int64_t api_bytes = 0;         // bytes of this shard in the API element type
    bool per_shard = true;         // false: independent of the batch, identical on every GPU
    int64_t user_offset = 0;       // byte offset of this shard inside the caller's buffer
    const void* const_host = nullptr;  // output that is a constant: copied straight from here
  };
  std::vector<Io> inputs, outputs;
  std::vector<unsigned*> input_range_stats;  // per input, like Launch::range_stats
  ~Plan();
};

struct Replica {
  int device = 0;
  int64_t shard_start = 0, shard_batch = 0;  // rows [start, start+batch) of dim 0
  int* host_status = nullptr;      // pinned copy of the plan's device status word
  std::unique_ptr<Plan> plan;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev_begin = nullptr, ev_end = nullptr;
};

}  // namespace b200

struct _odla_context;
namespace b200 {
// A further set of arenas, streams and plans for one computation, so that a second context can be in flight while the
// first one runs (its input copy under the other's kernels).  Lane 0 is the computation's own `replicas`.
struct Lane {
  std::map<int64_t, std::vector<Replica>> batch_replicas;  // keyed by the rows an execute runs (the recorded batch included)
  std::mutex exec_mutex;
};
}  // namespace b200
struct _odla_computation {
  std::vector<std::unique_ptr<_odla_value>> nodes;
  std::vector<odla_value> args, outs;
  std::map<std::string, odla_value> by_name;
  std::string first_error;         // first builder failure; reported at context/execute time
  odla_status error_status = ODLA_SUCCESS;
  // properties (odla_SetComputationItem)
  int float_mode = b200::DT_F32;         // DT_F32, DT_F16 (ODLA_FP16_MODE) or DT_BF16 (ODLA_BF16_MODE)
  int n_gpus = 0;                  // ODLA_PROCESSOR_NUM; 0 = all visible
  bool use_graph = true;           // ODLA_AGGREGATE_OPS / ODLA_B200_GRAPH
  int first_device = 0;
  int sub_batches = 0;             // ODLA_BATCHES_PER_STEP: replicas per GPU; 0 = environment / 1
  std::vector<odla_value_quant_info> quant_table;
  std::deque<std::string> quant_names;   // owns the value ids the table's records point to
  bool quant_applied = false;      // the table has been folded into the graph (quant_table.cc)
  std::vector<std::unique_ptr<std::vector<uint8_t>>> owned_consts;  // data of constants the library synthesised
  // Constants in the form the kernels read them (converted to the storage type, filters repacked K-major, ...), keyed
  // by "<node index>|<form>".  Filled by the first plan, shared by every replica's plan after it, written into and
  // read back from a stored executable so that a loaded one skips the conversions.
  std::map<std::string, std::shared_ptr<std::vector<uint8_t>>> prepared;
  std::mutex prepared_mutex;
  long long prepared_hits = 0, prepared_misses = 0;
  // built lazily at first context / execute
  bool planned = false;
  bool shardable = true;           // dim 0 of every argument/output is an independent batch
  std::vector<b200::Replica> replicas;
  int64_t graph_batch = 1;         // dim 0 of the recorded graph
  std::map<int64_t, std::vector<b200::Replica>> batch_replicas;  // plans for other run batch sizes (ODLA_RUN_BATCH_SIZE)
  std::mutex exec_mutex;           // executions that share lane 0's arenas: one at a time
  // Contexts are spread over `lanes` + 1 sets of arenas (ODLA_B200_CONTEXT_LANES, default 2): contexts on different
  // lanes execute concurrently, contexts that share a lane take turns.  lanes[k - 1] belongs to lane k.
  std::vector<std::unique_ptr<b200::Lane>> lanes;
  std::atomic<bool> multi_lane{false};
  std::recursive_mutex plan_mutex; // guards planning: `planned`, `replicas`, `batch_replicas`, every lane's plans
  // Kernels of concurrent executes run one execute after the other on each GPU (only copies overlap kernels): each
  // execute's launches wait for the event the previous execute recorded behind its own.
  struct ChainLink { std::mutex enqueue; cudaEvent_t last = nullptr; };
  std::mutex chain_mutex;          // guards the map, not the links
  std::map<int, std::unique_ptr<ChainLink>> chain;   // per device
  std::mutex ctx_mutex;            // guards `contexts`
  std::set<_odla_context*> contexts;  // live contexts created for this computation
  ~_odla_computation();
};

struct _odla_context {
  odla_computation comp = nullptr;
  std::map<const _odla_value*, const void*> in;
  std::map<const _odla_value*, void*> out;
  float last_ms = -1.f;
  long long last_launches = 0;
  bool profiling = false;
  bool range_profiling = false;    // accumulate min / max of every materialised value (odla_b200_SetRangeProfiling)
  int64_t run_batch = 0;           // ODLA_RUN_BATCH_SIZE; 0 = the recorded batch
  int lane = 0;                    // which set of arenas this context executes on
  // odla_AsyncExecuteComputation: one worker at a time per context
  std::thread worker;
  int (*async_fn)(void*, odla_status) = nullptr;
  void* async_arg = nullptr;
  odla_status async_status = ODLA_SUCCESS;
};

struct _odla_device {
  int index = 0;
};

namespace b200 {
// Rewrites the graph according to comp->quant_table (once).  Defined in quant_table.cc.
odla_status apply_quant_table(_odla_computation* comp);
// Builds replicas and plans for `comp` (idempotent).  Defined in plan.cc.
odla_status ensure_planned(_odla_computation* comp);
odla_status execute(_odla_computation* comp, _odla_context* ctx);
void destroy_replicas(std::vector<Replica>& reps);
int visible_devices();
extern thread_local int g_current_device;  // set by odla_SetCurrentDevice, -1 = unset
}  // namespace b200
