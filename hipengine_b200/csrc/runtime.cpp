// Native host runtime: validated graph launches, a per-bucket graph-exec cache and a launch-sequence helper.
//
//   he_cycle_launch      one captured CUDA graph = one speculative cycle or one decode step; the control block is
//                        validated first, so a stale or corrupted descriptor is refused on the host instead of
//                        becoming a device fault.
//   he_graph_cache_*     (key -> cudaGraphExec_t) map with hit / miss counters, so the steady-state decode loop
//                        is "look up bucket, launch" without crossing back into Python object code.
//   he_launch_sequence   launches several graphs back to back on one stream in a single native call (the role of
//                        the reference's launch-batch shim, hipengine/kernels/hip_gfx1100/runtime/
//                        laguna_launch_batch.hip, and of its PM4 graph submitter: replay with minimal host work).
// No device code here: every kernel lives in the .cu files.
#include <cuda_runtime.h>

#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "he_cycle_abi.h"

#define HE_API extern "C" __attribute__((visibility("default")))

namespace {
std::atomic<uint64_t> g_launches{0};
std::mutex g_mu;
struct Entry { cudaGraphExec_t exec; uint64_t hits; };
std::unordered_map<uint64_t, Entry> g_cache;
uint64_t g_hits = 0, g_misses = 0;
}  // namespace

HE_API int he_cycle_control_size(void) { return (int)sizeof(HeCycleControlV1); }
HE_API int he_cycle_result_size(void) { return (int)sizeof(HeCycleResultV1); }

// 0 when the block is acceptable, otherwise a negative code naming the first failed check.
HE_API int he_cycle_validate(const HeCycleControlV1* c) {
  if (c == nullptr) return -1;
  if (c->magic != HE_CYCLE_MAGIC) return -2;
  if (c->version != HE_CYCLE_VERSION) return -3;
  if (c->struct_bytes != sizeof(HeCycleControlV1)) return -4;
  if (c->mode != HE_MODE_CHAIN) return -5;
  if (c->n_requests < 1 || c->n_requests > HE_CYCLE_MAX_REQUESTS) return -6;
  if (c->depth > HE_CYCLE_MAX_DEPTH) return -7;
  const uint32_t known = HE_STAGE_PROPOSE | HE_STAGE_VERIFY | HE_STAGE_ACCEPT | HE_STAGE_COMMIT |
                         HE_STAGE_UPDATE_CURSORS | HE_STAGE_DECODE_STEP;
  if (c->stage_mask == 0 || (c->stage_mask & ~known) != 0) return -8;
  // a decode step carries no speculative stages and no depth; a speculative cycle must verify what it proposes
  if ((c->stage_mask & HE_STAGE_DECODE_STEP) && (c->stage_mask != HE_STAGE_DECODE_STEP || c->depth != 0)) return -9;
  if ((c->stage_mask & HE_STAGE_PROPOSE) && !(c->stage_mask & HE_STAGE_VERIFY)) return -10;
  if ((c->stage_mask & HE_STAGE_COMMIT) && !(c->stage_mask & HE_STAGE_ACCEPT)) return -11;
  if ((c->stage_mask & HE_STAGE_VERIFY) && c->depth == 0) return -12;
  return 0;
}

HE_API int he_cycle_launch(const HeCycleControlV1* c, void* graph_exec, void* stream, HeCycleResultV1* out) {
  if (out == nullptr) return -1;
  std::memset(out, 0, sizeof(*out));
  const int v = he_cycle_validate(c);
  if (v != 0 || graph_exec == nullptr) {
    out->rc = v != 0 ? v : -13;
    return out->rc;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_exec), s);
  if (e != cudaSuccess) {
    out->rc = (int)e;
    return out->rc;
  }
  out->launches = ++g_launches;
  if (c->wait) {
    if (c->n_accept != 0) {
      e = cudaMemcpyAsync(out->n_accept, reinterpret_cast<const void*>(c->n_accept), sizeof(int32_t) * c->n_requests,
                          cudaMemcpyDeviceToHost, s);
      if (e != cudaSuccess) { out->rc = (int)e; return out->rc; }
    }
    if (c->status_word != 0) {
      e = cudaMemcpyAsync(&out->device_status, reinterpret_cast<const void*>(c->status_word), sizeof(int32_t),
                          cudaMemcpyDeviceToHost, s);
      if (e != cudaSuccess) { out->rc = (int)e; return out->rc; }
    }
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { out->rc = (int)e; return out->rc; }
  }
  return 0;
}

// ---- graph-exec cache (the execs are owned by the caller; the cache only maps keys to them)
HE_API int he_graph_cache_put(uint64_t key, void* graph_exec) {
  if (graph_exec == nullptr) return -1;
  std::lock_guard<std::mutex> lk(g_mu);
  g_cache[key] = Entry{reinterpret_cast<cudaGraphExec_t>(graph_exec), 0};
  return 0;
}
HE_API void* he_graph_cache_get(uint64_t key) {
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_cache.find(key);
  if (it == g_cache.end()) { ++g_misses; return nullptr; }
  ++g_hits;
  ++it->second.hits;
  return it->second.exec;
}
HE_API int he_graph_cache_erase(uint64_t key) {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_cache.erase(key) ? 0 : -1;
}
HE_API void he_graph_cache_clear(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_cache.clear();
}
HE_API void he_graph_cache_stats(uint64_t* entries, uint64_t* hits, uint64_t* misses) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (entries) *entries = g_cache.size();
  if (hits) *hits = g_hits;
  if (misses) *misses = g_misses;
}
// look up `key` and launch it; -2 when the bucket has not been captured yet
HE_API int he_graph_cache_launch(uint64_t key, void* stream) {
  void* exec = he_graph_cache_get(key);
  if (exec == nullptr) return -2;
  cudaError_t e = cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return (int)e;
  ++g_launches;
  return 0;
}

// launch n graphs back to back on one stream; returns 0 or the first error (index in *failed_at)
HE_API int he_launch_sequence(void* const* graph_execs, int n, void* stream, int* failed_at) {
  if (graph_execs == nullptr || n < 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  for (int i = 0; i < n; ++i) {
    if (graph_execs[i] == nullptr) { if (failed_at) *failed_at = i; return -13; }
    cudaError_t e = cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(graph_execs[i]), s);
    if (e != cudaSuccess) { if (failed_at) *failed_at = i; return (int)e; }
    ++g_launches;
  }
  return 0;
}
HE_API uint64_t he_native_graph_launches(void) { return g_launches.load(); }

// ---------------------------------------------------------------- bounds words of the "checked" library variant
// Every .cu file of a build with -DHE_BOUNDS_CHECK=1 registers a reader of its device-side bounds word here (static
// initialiser); he_bounds_status() asks them all.  Returns -1 in the product build (no readers), else the first
// non-zero code found (out4 = {code, site, index, limit}) or 0; `reset` clears what was read.
namespace {
typedef int (*HeBoundsReader)(int* out4, int reset);
HeBoundsReader g_bounds_readers[64];
int g_n_bounds_readers = 0;
}  // namespace

extern "C" __attribute__((visibility("default"))) void he_bounds_register_reader(HeBoundsReader fn) {
  if (g_n_bounds_readers < 64) g_bounds_readers[g_n_bounds_readers++] = fn;
}

HE_API int he_bounds_status(int* out4, int reset) {
  if (g_n_bounds_readers == 0) return -1;
  int first[4] = {0, 0, 0, 0};
  for (int i = 0; i < g_n_bounds_readers; ++i) {
    int w[4] = {0, 0, 0, 0};
    const int rc = g_bounds_readers[i](w, reset);
    if (rc < 0) return -2;
    if (rc != 0 && first[0] == 0) std::memcpy(first, w, sizeof(first));
  }
  if (out4 != nullptr) std::memcpy(out4, first, sizeof(first));
  return first[0];
}
