// odla_b200_reduce_mean_noalloc: mean over several axes for callers that must not allocate.
//
// Who needs it: a host runtime that reserved all device memory for its own pool when it started
// (so a cudaMalloc made on its behalf fails), and serving loops with a latency bound that cannot
// afford cudaMalloc / cudaFree, which take the driver's allocator lock and synchronise the device.
// The graph path (odla_ReduceMean) allocates its intermediate buffers with cudaMalloc when the plan
// is built; this entry point keeps them in a fixed array that is part of the library image instead.
//
// The array below exists once per GPU that loads the library and stays resident until the process
// exits.  Its name is only a host-side handle: the device address is looked up with
// cudaGetSymbolAddress the first time the entry point runs on a device (with that device current)
// and cached.  That first call therefore does driver work; make it before starting a stream
// capture.  Every later call only enqueues kernels.
#include <atomic>
#include <cstdio>

#include "../../include/odla_b200.h"
#include "kernels.h"

namespace {

// Two halves, used alternately by consecutive reduction passes: 2 x 1 Mi floats = 8 MiB per GPU.
constexpr long long kHalfFloats = 1ll << 20;
static __device__ __align__(256) float g_reduce_scratch[2 * kHalfFloats];

constexpr int kMaxDevices = 64;
std::atomic<float*> g_scratch_addr[kMaxDevices];   // zero-initialised; two threads that race on a first call store the same address

// Device address of the scratch array on the current device, or nullptr (error already printed).
float* scratch_on_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fprintf(stderr, "[odla_b200] reduce_mean_noalloc: no usable current CUDA device\n");
    return nullptr;
  }
  float* cached = g_scratch_addr[dev].load(std::memory_order_acquire);
  if (!cached) {
    float* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_reduce_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "[odla_b200] reduce_mean_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_addr[dev].store(p, std::memory_order_release);
    cached = p;
  }
  return cached;
}

}  // namespace

extern "C" int odla_b200_reduce_mean_noalloc(const void* x, void* y, int dtype, const long long* dims, int rank, const int* axes, int n_axes,
                                             void* stream) {
  using namespace b200;
  if (!x || !y || !dims || !axes || rank < 1 || rank > ODLA_MAX_DIMENSION || n_axes < 1 || n_axes > rank) return -1;
  const int dt = dtype == 0 ? DT_F32 : dtype == 1 ? DT_F16 : dtype == 2 ? DT_BF16 : -1;
  if (dt < 0) return -1;
  if (x == y) return -1;  // a pass reads rows that another block of the same pass would already have overwritten
  for (int k = 0; k < n_axes; ++k)
    for (int j = 0; j < k; ++j)
      if (axes[j] == axes[k]) return -1;  // an axis can be reduced once
  long long d[ODLA_MAX_DIMENSION];
  for (int i = 0; i < rank; ++i) {
    if (dims[i] < 1) return -1;
    d[i] = dims[i];
  }
  // Every pass but the last writes an fp32 intermediate into one half of the fixed array; refuse
  // shapes whose intermediates do not fit, before anything is enqueued.
  {
    long long t[ODLA_MAX_DIMENSION];
    for (int i = 0; i < rank; ++i) t[i] = d[i];
    for (int k = 0; k + 1 < n_axes; ++k) {
      if (axes[k] < 0 || axes[k] >= rank) return -1;
      t[axes[k]] = 1;
      long long n = 1;
      for (int i = 0; i < rank; ++i) n *= t[i];
      if (n > kHalfFloats) {
        fprintf(stderr,
                "[odla_b200] reduce_mean_noalloc: an intermediate of %lld floats exceeds the fixed scratch of %lld floats per pass; "
                "use odla_ReduceMean (which allocates) or reduce fewer rows per call\n",
                n, kHalfFloats);
        return -1;
      }
    }
    if (axes[n_axes - 1] < 0 || axes[n_axes - 1] >= rank) return -1;
  }
  float* scratch = n_axes > 1 ? scratch_on_current_device() : nullptr;
  if (n_axes > 1 && !scratch) return -2;
  const void* src = x;
  int sdt = dt;
  for (int k = 0; k < n_axes; ++k) {
    const int a = axes[k];
    long long before = 1, after = 1;
    for (int i = 0; i < a; ++i) before *= d[i];
    for (int i = a + 1; i < rank; ++i) after *= d[i];
    const bool last = k + 1 == n_axes;
    void* dst = last ? y : (void*)(scratch + (k & 1) * kHalfFloats);
    const int ddt = last ? dt : DT_F32;
    // Nothing in the array has to start from zero: a pass overwrites every element the next pass reads.
    int rc = reduce_mean_axis(sdt, ddt, src, dst, before, d[a], after, (cudaStream_t)stream);
    if (rc) return rc;
    d[a] = 1;
    src = dst;
    sdt = ddt;
  }
  return 0;
}
