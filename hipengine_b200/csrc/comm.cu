// Peer-memory collectives for tensor-parallel decode: push all-reduce fused with the residual add.
//
// Every rank owns one "symmetric" region (same layout on all ranks, mapped into every peer through CUDA IPC):
//     data  [2 phases][world][max_rows * width] fp32   -- slot (phase, src) is written only by rank `src`
//     flags [2 phases][world][MAX_CTAS] uint32          -- epoch stamps, one per (phase, src rank, CTA)
// One call = one kernel on every rank:
//     1. CTA c copies its slice of the local partial rows into slot (phase, me) of EVERY rank (plain
//        st.global over NVLink for peers), fences at system scope, then stamps flag (phase, me, c) on every rank;
//     2. CTA c waits -- bounded -- until the stamps of all ranks for slice c show this call's epoch;
//     3. CTA c sums the world slots of slice c in rank order (so all ranks compute bit-identical sums and the
//        replicated residual stream cannot drift apart) and adds the sum to the fp32 residual rows.
// The epoch lives in device memory and is advanced by the kernel itself, so a captured CUDA graph can be
// replayed without any host-side argument patching.  Phases alternate per call: a rank can run at most one
// call ahead of its slowest peer (it needs that peer's stamps to finish a call), so two phases are enough.
// A wait that runs out records HE_ERR_WAIT_TIMEOUT in the status word and the CTA leaves without touching the
// residual; the context stays usable and the host sees the failure on its next status check.
// The reference engine is single-device: no counterpart there.
#include "common.cuh"
#include "peer_comm.cuh"

using namespace he;

namespace {

constexpr int COMM_MAX_CTAS = 64;
constexpr int COMM_MAX_WORLD = 8;

struct CommArgs {
  float* data[COMM_MAX_WORLD];        // data region of every rank (peer-mapped), indexed by rank
  uint32_t* flags[COMM_MAX_WORLD];    // flag region of every rank
  uint32_t* epoch;                    // [COMM_MAX_CTAS] local per-CTA call counters
  const float* partial;               // [rows][width] local partial products
  float* resid;                       // [rows][ld_resid] residual stream, updated in place (may be null)
  float* out;                         // optional: reduced rows stored here instead of / as well as resid
  long long ld_resid, ld_out;
  int rows, width, slot_floats;       // slot_floats = max_rows * width
  int world, rank;
  int* status;
  unsigned wait_limit;                // polls before giving up
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cg4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

__global__ void __launch_bounds__(256) comm_push_reduce_kernel(const CommArgs a) {
  __shared__ int ok_s;
  const int c = blockIdx.x, n_cta = gridDim.x;
  // Programmatic dependent launch: this grid is already resident when the producer of `partial` drains, and the
  // kernel after it (a GEMV) may start prefetching its weights while the CTAs below wait for the peers' stamps.
  // Nothing -- not even the epoch -- is read before the wait: with chained early launches only the wait orders this
  // grid after ALL earlier kernels of the stream.
  pdl_launch();
  pdl_wait();
  const uint32_t epoch = a.epoch[c] + 1;
  const int phase = epoch & 1;
  const int total = a.rows * a.width;              // floats in flight this call (multiple of 4)
  const int per = (((total + n_cta - 1) / n_cta) + 3) & ~3;
  const int lo = min(total, c * per), hi = min(total, lo + per);
  const size_t slot_me = ((size_t)phase * a.world + a.rank) * a.slot_floats;
  // 1. push my slice to every rank
  for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(a.partial + i);
    for (int r = 0; r < a.world; ++r) *reinterpret_cast<float4*>(a.data[r] + slot_me + i) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < a.world)
    st_release_sys(a.flags[threadIdx.x] + ((size_t)phase * a.world + a.rank) * COMM_MAX_CTAS + c, epoch);
  // 2. bounded wait for every rank's stamp of this slice
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < a.world) {
    const uint32_t* f = a.flags[a.rank] + ((size_t)phase * a.world + threadIdx.x) * COMM_MAX_CTAS + c;
    unsigned polls = 0;
    // stamps only grow; "epoch or later" also accepts a peer that is already one call ahead on this phase
    while ((int)(ld_acquire_sys(f) - epoch) < 0) {
      if (++polls > a.wait_limit) {
        ok_s = 0;
        if (a.status != nullptr) atomicCAS(a.status, 0, HE_ERR_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  // 3. reduce in rank order + residual add
  if (ok_s) {
    const float* mine = a.data[a.rank] + (size_t)phase * a.world * a.slot_floats;
    for (int i = lo + threadIdx.x * 4; i < hi; i += blockDim.x * 4) {
      float4 s = ld_cg4(mine + i);
      for (int r = 1; r < a.world; ++r) {
        const float4 v = ld_cg4(mine + (size_t)r * a.slot_floats + i);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      const int row = i / a.width, col = i % a.width;
      if (a.out != nullptr) *reinterpret_cast<float4*>(a.out + (size_t)row * a.ld_out + col) = s;
      if (a.resid != nullptr) {
        float4* hp = reinterpret_cast<float4*>(a.resid + (size_t)row * a.ld_resid + col);
        float4 h = *hp;
        h.x += s.x; h.y += s.y; h.z += s.z; h.w += s.w;
        *hp = h;
      }
    }
  }
  if (threadIdx.x == 0) a.epoch[c] = epoch;
}

}  // namespace

// ---- symmetric region management (set-up time only)
HE_API int he_comm_alloc(long long bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
HE_API int he_comm_free(void* p) { return (int)cudaFree(p); }
HE_API int he_comm_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
HE_API int he_comm_ipc_get(void* p, void* handle_out) {
  return (int)cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle_out), p);
}
HE_API int he_comm_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
HE_API int he_comm_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

HE_API int he_comm_max_ctas() { return COMM_MAX_CTAS; }
HE_API int he_comm_args_size() { return (int)sizeof(CommArgs); }

// All-reduce of `rows x width` fp32 partial rows over the ranks, fused with resid += sum (and/or out = sum).
HE_API int he_comm_push_reduce(const CommArgs* args, int n_ctas, cudaStream_t stream) {
  const CommArgs& a = *args;
  if (a.rows <= 0) return 0;
  if (a.world < 1 || a.world > COMM_MAX_WORLD || a.rank < 0 || a.rank >= a.world) return -HE_ERR_BAD_ARG;
  if (a.width % 4 != 0 || (long long)a.rows * a.width > a.slot_floats) return -HE_ERR_BAD_ARG;
  if (n_ctas < 1 || n_ctas > COMM_MAX_CTAS) return -HE_ERR_BAD_ARG;
  cudaError_t e = launch_pdl(comm_push_reduce_kernel, dim3(n_ctas), dim3(256), 0, stream, a);
  if (e != cudaSuccess) return (int)e;
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Collectives over the same receive regions as the decode GEMV's push epilogue (peer_comm.cuh).
namespace {

// Stand-alone consumer of a push: resid rows += sum over ranks of the pushed partial rows (rank order).  Used where
// the next reader of the residual is not a GEMV with a reduce prologue (MoE routing, tensor-core batches, NextN).
__global__ void __launch_bounds__(256) comm_reduce_in_kernel(const HeGemvComm c, float* resid, long long ld_resid,
                                                             int rows, int* status) {
  pdl_launch();
  pdl_wait();
  const uint32_t tag = *reinterpret_cast<volatile uint32_t*>(c.state);
  const int parity = (int)((tag - 1u) & 1u);
  const uint2* mine = c.recv[c.rank] + (size_t)parity * c.world * c.slot_floats;
  const int total = rows * c.width;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 8; i < total; i += gridDim.x * blockDim.x * 8) {
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < c.world; ++q) {
      float v[8];
      ll_load8(mine + (size_t)q * c.slot_floats + i, tag, c.wait_limit, status, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] = q == 0 ? v[e] : s[e] + v[e];
    }
    const int row = i / c.width, col = i % c.width;
    float4* hp = reinterpret_cast<float4*>(resid + (size_t)row * ld_resid + col);
    float4 h0 = hp[0], h1 = hp[1];
    h0.x += s[0]; h0.y += s[1]; h0.z += s[2]; h0.w += s[3];
    h1.x += s[4]; h1.y += s[5]; h1.z += s[6]; h1.w += s[7];
    hp[0] = h0;
    hp[1] = h1;
  }
}

// Stand-alone producer: pushes `rows` fp32 rows (any producer's output, e.g. the MoE expert sum) to every rank.
__global__ void __launch_bounds__(256) comm_push_rows_kernel(const HeGemvComm c, const float* partial, int rows) {
  pdl_launch();
  pdl_wait();
  const uint32_t seq0 = *reinterpret_cast<volatile uint32_t*>(c.state);
  const size_t off = ((size_t)(seq0 & 1u) * c.world + c.rank) * c.slot_floats;
  const int total = rows * c.width;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const float v = partial[i];
    for (int q = 0; q < c.world; ++q) ll_store(c.recv[q] + off + i, v, seq0 + 1u);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(c.state + 1, 1u);
    if (prev == gridDim.x - 1) {
      c.state[1] = 0;
      *reinterpret_cast<volatile uint32_t*>(c.state) = seq0 + 1u;
    }
  }
}

// Vocab-parallel greedy head: every rank has the (max, id) of its own vocabulary shard per row; one CTA pushes its
// pairs to every rank, waits (bounded) for the others and keeps the best pair: larger value, lower token id on exact
// ties -- what a single argmax over the concatenated logits returns.  A region word is one (value, id) pair; this
// exchange is ordered by the region's stamps (fence + flag), not by tags.
__global__ void __launch_bounds__(64) comm_argmax_merge_kernel(const HeGemvComm c, const float* loc_val,
                                                               const long long* loc_idx, int vocab_off, int rows,
                                                               long long* out_ids, int* status) {
  __shared__ int ok_s;
  pdl_launch();
  pdl_wait();
  const uint32_t seq0 = *reinterpret_cast<volatile uint32_t*>(c.state);
  const int parity = (int)(seq0 & 1u);
  const int t = threadIdx.x;
  if (t < rows) {
    const uint2 word = make_uint2(__float_as_uint(loc_val[t]), (uint32_t)((int)loc_idx[t] + vocab_off));
    const size_t off = ((size_t)parity * c.world + c.rank) * c.slot_floats + (size_t)t;
    for (int q = 0; q < c.world; ++q) c.recv[q][off] = word;
  }
  if (t == 0) ok_s = 1;
  __threadfence_system();
  __syncthreads();
  if (t < c.world) st_release_sys_u32(c.flags[t] + parity * c.world + c.rank, seq0 + 1u);
  if (t < c.world) {
    const uint32_t* f = c.flags[c.rank] + parity * c.world + t;
    unsigned polls = 0;
    while ((int)(ld_acquire_sys_u32(f) - (seq0 + 1u)) < 0) {
      if (++polls > c.wait_limit) {
        ok_s = 0;
        if (status != nullptr) atomicCAS(status, 0, HE_ERR_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (t < rows && ok_s) {
    const uint2* mine = c.recv[c.rank] + (size_t)parity * c.world * c.slot_floats + (size_t)t;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int q = 0; q < c.world; ++q) {
      uint2 p;
      asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(p.x), "=r"(p.y) : "l"(mine + (size_t)q * c.slot_floats));
      const float pv = __uint_as_float(p.x);
      const int id = (int)p.y;
      if (pv > bv || (pv == bv && id < bi)) { bv = pv; bi = id; }
    }
    out_ids[t] = bi == 0x7fffffff ? 0 : bi;
  }
  if (t == 0) *reinterpret_cast<volatile uint32_t*>(c.state) = seq0 + 1u;
}

int comm_valid(const HeGemvComm& c, int rows) {
  if (c.world < 2 || c.world > GEMV_MAX_WORLD || c.rank < 0 || c.rank >= c.world || c.state == nullptr) return 0;
  if (c.width % 8 != 0 && c.width != 1) return 0;
  if ((long long)rows * c.width > c.slot_floats) return 0;
  for (int q = 0; q < c.world; ++q)
    if (c.recv[q] == nullptr || c.flags[q] == nullptr) return 0;
  return 1;
}

}  // namespace

HE_API int he_gemv_comm_size() { return (int)sizeof(HeGemvComm); }

HE_API int he_comm_reduce_in(const HeGemvComm* comm, void* resid, long long ld_resid, int rows, void* status,
                             cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!comm_valid(*comm, rows) || ld_resid % 4 != 0) return -HE_ERR_BAD_ARG;
  const int n8 = rows * comm->width / 8;
  int grid = (n8 + 255) / 256;
  if (grid > 32) grid = 32;
  if (grid < 1) grid = 1;
  cudaError_t e = launch_pdl(comm_reduce_in_kernel, dim3(grid), dim3(256), 0, stream, *comm, (float*)resid, ld_resid,
                             rows, (int*)status);
  if (e != cudaSuccess) return (int)e;
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_comm_push_rows(const HeGemvComm* comm, const void* partial, int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!comm_valid(*comm, rows)) return -HE_ERR_BAD_ARG;
  const int n1 = rows * comm->width;
  int grid = (n1 + 255) / 256;
  if (grid > 64) grid = 64;
  cudaError_t e = launch_pdl(comm_push_rows_kernel, dim3(grid), dim3(256), 0, stream, *comm, (const float*)partial,
                             rows);
  if (e != cudaSuccess) return (int)e;
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_comm_argmax_merge(const HeGemvComm* comm, const void* loc_val, const void* loc_idx, int vocab_off,
                                int rows, void* out_ids, void* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > 64 || comm->width != 1 || !comm_valid(*comm, rows)) return -HE_ERR_BAD_ARG;
  cudaError_t e = launch_pdl(comm_argmax_merge_kernel, dim3(1), dim3(64), 0, stream, *comm, (const float*)loc_val,
                             (const long long*)loc_idx, vocab_off, rows, (long long*)out_ids, (int*)status);
  if (e != cudaSuccess) return (int)e;
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Sequence-parallel prefill: the fp32 residual is sharded by M-tiles (tile tm of `mt` rows belongs to rank
// tm % world).  After a reduce-scatter GEMM has completed a rank's rows, this kernel normalises them and writes the
// bf16 result into EVERY rank's activation buffer (RMSNorm + all-gather as peer stores of whole rows), then stamps
// its flag on every rank; the consumers (gemm_wq_sm100.cu, all-gather wait) read the rows from local memory once the
// stamp of the rows' owner is there.  mode 1 copies the fp32 rows instead (gathering the residual itself at the end
// of a forward pass).  The reference engine is single-device: no counterpart there.
namespace {

struct SpPushArgs {
  void* dst[GEMV_MAX_WORLD];        // every rank's destination rows (bf16 [T][ld_dst] or fp32 for mode 1)
  uint32_t* flags[GEMV_MAX_WORLD];  // every rank's stamp array [world]
  uint32_t* state;                  // local: [0] epoch of the last completed push, [1] CTAs done
  const float* h;
  const float* norm_w;
  long long ld_h, ld_dst;
  float eps;
  int T, H, mt, world, rank, mode;
};

constexpr int SP_MAXG = 4;   // 8-element groups per thread: rows of up to 256 * 4 * 8 = 8192 columns

__global__ void __launch_bounds__(256) sp_norm_push_kernel(const SpPushArgs a) {
  __shared__ float red[33];
  const int W = a.world;
  const int tiles_m = (a.T + a.mt - 1) / a.mt;
  const int owned_tiles = tiles_m > a.rank ? (tiles_m - a.rank + W - 1) / W : 0;
  const int n_groups = a.H / 8;
  for (int j = blockIdx.x; j < owned_tiles * a.mt; j += gridDim.x) {
    const int m = (a.rank + W * (j / a.mt)) * a.mt + j % a.mt;
    if (m >= a.T) continue;                           // uniform across the CTA
    const float* hr = a.h + (size_t)m * a.ld_h;
    float v[SP_MAXG][8];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < SP_MAXG; ++u) {
      const int g = u * 256 + (int)threadIdx.x;
      if (g < n_groups) {
        const float4 x0 = *reinterpret_cast<const float4*>(hr + (size_t)g * 8);
        const float4 x1 = *reinterpret_cast<const float4*>(hr + (size_t)g * 8 + 4);
        v[u][0] = x0.x; v[u][1] = x0.y; v[u][2] = x0.z; v[u][3] = x0.w;
        v[u][4] = x1.x; v[u][5] = x1.y; v[u][6] = x1.z; v[u][7] = x1.w;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[u][e] * v[u][e];
      }
    }
    float inv = 1.f;
    if (a.mode == 0) {
      ss = block_sum(ss, red);
      inv = rsqrtf(ss / (float)a.H + a.eps);
    }
#pragma unroll
    for (int u = 0; u < SP_MAXG; ++u) {
      const int g = u * 256 + (int)threadIdx.x;
      if (g < n_groups) {
        if (a.mode == 0) {
          const float4 w0 = __ldg(reinterpret_cast<const float4*>(a.norm_w + (size_t)g * 8));
          const float4 w1 = __ldg(reinterpret_cast<const float4*>(a.norm_w + (size_t)g * 8 + 4));
          const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          uint4 pk;
          uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[u][2 * e] * inv * wv[2 * e], v[u][2 * e + 1] * inv * wv[2 * e + 1]);
            pw[e] = *reinterpret_cast<uint32_t*>(&h2);
          }
          for (int q = 0; q < W; ++q)
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.dst[q]) + (size_t)m * a.ld_dst + (size_t)g * 8) = pk;
        } else {
          for (int q = 0; q < W; ++q) {
            if (q == a.rank) continue;                 // the local rows are the source
            float* d = reinterpret_cast<float*>(a.dst[q]) + (size_t)m * a.ld_dst + (size_t)g * 8;
            *reinterpret_cast<float4*>(d) = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
            *reinterpret_cast<float4*>(d + 4) = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
          }
        }
      }
    }
  }
  // every row of this CTA is stored; the last CTA of the grid publishes the push on every rank
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(a.state + 1, 1u);
    if (prev == gridDim.x - 1) {
      a.state[1] = 0;
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.state) + 1u;
      __threadfence_system();
      for (int q = 0; q < W; ++q) st_release_sys_u32(a.flags[q] + a.rank, epoch);
      *reinterpret_cast<volatile uint32_t*>(a.state) = epoch;
    }
  }
}

// Stream-ordered wait for the stamps of all ranks (for consumers that are not the all-gather GEMM).
__global__ void sp_wait_kernel(const uint32_t* flags, const uint32_t* state, int world, unsigned limit, int* status) {
  const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(state);
  if ((int)threadIdx.x < world) {
    unsigned polls = 0;
    while ((int)(ld_acquire_sys_u32(flags + threadIdx.x) - want) < 0) {
      if (++polls > limit) {
        if (status != nullptr) atomicCAS(status, 0, HE_ERR_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
}

}  // namespace

HE_API int he_sp_push_args_size() { return (int)sizeof(SpPushArgs); }

HE_API int he_sp_norm_push(const SpPushArgs* args, int num_sms, cudaStream_t stream) {
  const SpPushArgs& a = *args;
  if (a.T <= 0) return 0;
  if (a.world < 1 || a.world > GEMV_MAX_WORLD || a.rank < 0 || a.rank >= a.world || a.mt <= 0) return -HE_ERR_BAD_ARG;
  if (a.H % 8 != 0 || a.H > 256 * SP_MAXG * 8 || a.state == nullptr || a.h == nullptr) return -HE_ERR_BAD_ARG;
  if (a.mode == 0 && a.norm_w == nullptr) return -HE_ERR_BAD_ARG;
  for (int q = 0; q < a.world; ++q)
    if (a.dst[q] == nullptr || a.flags[q] == nullptr) return -HE_ERR_BAD_ARG;
  const int tiles_m = (a.T + a.mt - 1) / a.mt;
  const int owned = tiles_m > a.rank ? (tiles_m - a.rank + a.world - 1) / a.world : 0;
  int grid = owned * a.mt;
  if (grid > 4 * num_sms) grid = 4 * num_sms;
  if (grid < 1) grid = 1;
  sp_norm_push_kernel<<<grid, 256, 0, stream>>>(a);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_sp_wait(const void* flags, const void* state, int world, unsigned limit, void* status,
                      cudaStream_t stream) {
  if (world < 1 || world > GEMV_MAX_WORLD) return -HE_ERR_BAD_ARG;
  sp_wait_kernel<<<1, 32, 0, stream>>>((const uint32_t*)flags, (const uint32_t*)state, world, limit, (int*)status);
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// Reduce-scatter of token-ordered partial rows into the row-sharded residual (expert parallelism on top of the
// sequence-parallel residual): every rank holds partial[T][H] fp32 -- the weighted outputs of ITS experts for every
// token -- and each row's sum over ranks belongs to the row's owner (tile tm of mt rows -> rank tm % world).
//   push   : rows owned by another rank go as bf16 into that rank's stage [src][owned row index][H] (peer stores of
//            whole rows); the last CTA fences and stamps flags[owner][me];
//   reduce : the owner waits (bounded) for the world-1 stamps and adds local fp32 partial + the staged rows (rank
//            order, fp32) into its residual rows.
namespace {

struct SpRowsArgs {
  __nv_bfloat16* stage[GEMV_MAX_WORLD];   // every rank's stage
  uint32_t* flags[GEMV_MAX_WORLD];        // every rank's stamp array [world]
  uint32_t* state;                        // local: [0] epoch of the last completed push, [1] CTAs done
  const float* partial;                   // local [T][ld_p]
  float* resid;                           // local [T][ld_h]: owned rows are updated
  long long ld_p, ld_h;
  int T, H, mt, world, rank, rows_cap;    // rows_cap: stage rows per source
  unsigned wait_limit;
  int* status;
};

__device__ __forceinline__ int sp_owned_index(int m, int mt, int W) { return (m / mt / W) * mt + m % mt; }

__global__ void __launch_bounds__(256) sp_rows_push_kernel(const SpRowsArgs a) {
  const int W = a.world, n8 = a.H / 8;
  for (int m = blockIdx.x; m < a.T; m += gridDim.x) {
    const int owner = (m / a.mt) % W;
    if (owner == a.rank) continue;
    __nv_bfloat16* dst = a.stage[owner] + ((size_t)a.rank * a.rows_cap + sp_owned_index(m, a.mt, W)) * a.H;
    const float* src = a.partial + (size_t)m * a.ld_p;
    for (int g = threadIdx.x; g < n8; g += blockDim.x) {
      const float4 x0 = *reinterpret_cast<const float4*>(src + (size_t)g * 8);
      const float4 x1 = *reinterpret_cast<const float4*>(src + (size_t)g * 8 + 4);
      uint4 pk;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
      __nv_bfloat162 h0 = __floats2bfloat162_rn(x0.x, x0.y), h1 = __floats2bfloat162_rn(x0.z, x0.w);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(x1.x, x1.y), h3 = __floats2bfloat162_rn(x1.z, x1.w);
      pw[0] = *reinterpret_cast<uint32_t*>(&h0); pw[1] = *reinterpret_cast<uint32_t*>(&h1);
      pw[2] = *reinterpret_cast<uint32_t*>(&h2); pw[3] = *reinterpret_cast<uint32_t*>(&h3);
      *reinterpret_cast<uint4*>(dst + (size_t)g * 8) = pk;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned prev = atomicAdd(a.state + 1, 1u);
    if (prev == gridDim.x - 1) {
      a.state[1] = 0;
      const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.state) + 1u;
      __threadfence_system();
      for (int q = 0; q < W; ++q) st_release_sys_u32(a.flags[q] + a.rank, epoch);
      *reinterpret_cast<volatile uint32_t*>(a.state) = epoch;
    }
  }
}

__global__ void __launch_bounds__(256) sp_rows_reduce_kernel(const SpRowsArgs a) {
  const int W = a.world, n8 = a.H / 8;
  const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(a.state);
  if ((int)threadIdx.x < W) {
    unsigned polls = 0;
    while ((int)(ld_acquire_sys_u32(a.flags[a.rank] + threadIdx.x) - want) < 0) {
      if (++polls > a.wait_limit) {
        if (a.status != nullptr) atomicCAS(a.status, 0, HE_ERR_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  const int tiles_m = (a.T + a.mt - 1) / a.mt;
  const int owned_tiles = tiles_m > a.rank ? (tiles_m - a.rank + W - 1) / W : 0;
  for (int j = blockIdx.x; j < owned_tiles * a.mt; j += gridDim.x) {
    const int m = (a.rank + W * (j / a.mt)) * a.mt + j % a.mt;
    if (m >= a.T) continue;
    const float* loc = a.partial + (size_t)m * a.ld_p;
    float* hr = a.resid + (size_t)m * a.ld_h;
    for (int g = threadIdx.x; g < n8; g += blockDim.x) {
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int q = 0; q < W; ++q) {                 // rank order; the local contribution is exact fp32
        if (q == a.rank) {
          const float4 x0 = *reinterpret_cast<const float4*>(loc + (size_t)g * 8);
          const float4 x1 = *reinterpret_cast<const float4*>(loc + (size_t)g * 8 + 4);
          s[0] += x0.x; s[1] += x0.y; s[2] += x0.z; s[3] += x0.w;
          s[4] += x1.x; s[5] += x1.y; s[6] += x1.z; s[7] += x1.w;
        } else {
          uint4 v;
          const __nv_bfloat16* sp = a.stage[a.rank] + ((size_t)q * a.rows_cap + j) * a.H + (size_t)g * 8;
          asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(sp));
          const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t2 = __bfloat1622float2(hv[e]);
            s[2 * e] += t2.x;
            s[2 * e + 1] += t2.y;
          }
        }
      }
      float4* hp = reinterpret_cast<float4*>(hr + (size_t)g * 8);
      float4 h0 = hp[0], h1 = hp[1];
      h0.x += s[0]; h0.y += s[1]; h0.z += s[2]; h0.w += s[3];
      h1.x += s[4]; h1.y += s[5]; h1.z += s[6]; h1.w += s[7];
      hp[0] = h0;
      hp[1] = h1;
    }
  }
}

}  // namespace

HE_API int he_sp_rows_args_size() { return (int)sizeof(SpRowsArgs); }

// phases bit 0: push, bit 1: reduce (3 in production; emulated ranks of one GPU run all pushes before any reduce).
HE_API int he_sp_rows_reduce_scatter(const SpRowsArgs* args, int phases, int num_sms, cudaStream_t stream) {
  const SpRowsArgs& a = *args;
  if (a.T <= 0) return 0;
  if (a.world < 1 || a.world > GEMV_MAX_WORLD || a.rank < 0 || a.rank >= a.world || a.mt <= 0 || a.H % 8 != 0)
    return -HE_ERR_BAD_ARG;
  const int tiles_m = (a.T + a.mt - 1) / a.mt;
  if (((tiles_m + a.world - 1) / a.world) * a.mt > a.rows_cap) return -HE_ERR_BAD_ARG;
  for (int q = 0; q < a.world; ++q)
    if (a.stage[q] == nullptr || a.flags[q] == nullptr) return -HE_ERR_BAD_ARG;
  int grid = a.T < 4 * num_sms ? a.T : 4 * num_sms;
  if (phases & 1) {
    sp_rows_push_kernel<<<grid, 256, 0, stream>>>(a);
    HE_LAUNCH_CHECK();
  }
  if (phases & 2) {
    sp_rows_reduce_kernel<<<grid, 256, 0, stream>>>(a);
    HE_LAUNCH_CHECK();
  }
  return 0;
}
