// Speculative decoding (MTP / NextN chain): device-side accept and commit bookkeeping.
//
// A verify batch holds, per request, the chain [t0, d1 .. dK]: the last committed token followed by K draft
// tokens.  The target model scores all K+1 rows in one forward; row i yields the distribution of the token
// that follows chain position i.
//   greedy  : accept d_{i+1} while it equals argmax(row i); the argmax of the first mismatching row (or of
//             row K) is the bonus token, so a cycle emits n+1 tokens, n = accepted drafts.
//   sampled : exact speculative sampling -- accept d with probability min(1, p(d)/q(d)); on rejection draw from
//             normalize(max(0, p - q)); after K acceptances draw the bonus from p_K.  A null q means the draft
//             was chosen greedily (q is a point mass), so the rule becomes "accept with probability p(d), else
//             draw from p with d removed".
// The commit kernel then moves the per-request cursors: tokens <- bonus, positions += n+1, and publishes the
// journal row whose recurrent state must become the live state (row n of the chain).
// Behavioural references: hipengine/kernels/hip_gfx1100/speculative/dflash_accept.hip (greedy chain accept),
// sampled_accept.hip and hipengine/speculative/sampling.py:135-339 (exact law), dflash_commit.hip (cursor commit).
#include "common.cuh"

using namespace he;

namespace {

// one thread per request
__global__ void spec_accept_greedy_kernel(const long long* __restrict__ draft, const long long* __restrict__ target,
                                          int R, int K, int* __restrict__ n_accept, long long* __restrict__ out,
                                          const int* __restrict__ max_emit) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  int n = 0;
  while (n < K && draft[(size_t)r * K + n] == target[(size_t)r * (K + 1) + n]) ++n;
  if (max_emit != nullptr) n = min(n, max(0, max_emit[r] - 1));   // never emit past the request's token budget
  n_accept[r] = n;
  for (int i = 0; i <= K; ++i) {
    long long v = -1;
    if (i < n) v = draft[(size_t)r * K + i];
    else if (i == n) v = target[(size_t)r * (K + 1) + n];
    out[(size_t)r * (K + 1) + i] = v;
  }
}

__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long ctr) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (ctr + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)((z >> 40) + 1) * (1.0f / 16777217.0f);   // (0, 1)
}

struct SampledArgs {
  const float* p_logits;     // [R][K+1][V] target logits
  const float* q_logits;     // [R][K][V] draft logits, or null for a greedy draft
  const long long* draft;    // [R][K]
  const float* temperature;  // [R]
  const unsigned long long* seed;     // [R]
  const unsigned long long* counter;  // [R]
  int* n_accept;             // [R]
  long long* out;            // [R][K+1]
  int R, K, V;
};

// one CTA (1024 threads) per request; walks the chain serially.
__global__ void __launch_bounds__(1024) spec_accept_sampled_kernel(const SampledArgs a) {
  __shared__ float red[33];
  __shared__ float scan[1024];
  __shared__ int pick_s;
  const int r = blockIdx.x, tid = threadIdx.x, V = a.V, K = a.K;
  const float invT = 1.f / fmaxf(a.temperature[r], 1e-6f);
  const unsigned long long seed = a.seed[r], ctr0 = a.counter[r];
  int n = 0;
  long long emitted = -1;
  for (int i = 0; i <= K; ++i) {
    const float* pl = a.p_logits + ((size_t)r * (K + 1) + i) * V;
    const float* ql = (a.q_logits != nullptr && i < K) ? a.q_logits + ((size_t)r * K + i) * V : nullptr;
    // softmax statistics of p (and q)
    float pm = -INFINITY, qm = -INFINITY;
    for (int v = tid; v < V; v += 1024) {
      pm = fmaxf(pm, pl[v] * invT);
      if (ql != nullptr) qm = fmaxf(qm, ql[v] * invT);
    }
    pm = block_max(pm, red);
    if (ql != nullptr) qm = block_max(qm, red);
    float ps = 0.f, qs = 0.f;
    for (int v = tid; v < V; v += 1024) {
      ps += __expf(pl[v] * invT - pm);
      if (ql != nullptr) qs += __expf(ql[v] * invT - qm);
    }
    ps = block_sum(ps, red);
    if (ql != nullptr) qs = block_sum(qs, red);
    const long long d = i < K ? a.draft[(size_t)r * K + i] : -1;
    bool accept = false;
    if (i < K) {
      const float pd = __expf(pl[d] * invT - pm) / ps;
      const float qd = ql != nullptr ? __expf(ql[d] * invT - qm) / qs : 1.f;
      const float u = uniform01(seed, ctr0 + 2 * i);
      accept = u * qd <= pd;      // u <= min(1, p/q)
    }
    if (accept) {
      ++n;
      continue;
    }
    // draw from the residual (i < K) or from p itself (bonus row): weights w_v = max(0, p_v - q_v)
    auto weight = [&](int v) -> float {
      const float pv = __expf(pl[v] * invT - pm) / ps;
      if (i >= K) return pv;
      const float qv = ql != nullptr ? __expf(ql[v] * invT - qm) / qs : (v == (int)d ? 1.f : 0.f);
      return fmaxf(0.f, pv - qv);
    };
    const int per = (V + 1023) / 1024;
    const int v0 = tid * per, v1 = min(V, v0 + per);
    float local = 0.f;
    for (int v = v0; v < v1; ++v) local += weight(v);
    scan[tid] = local;
    __syncthreads();
    // inclusive scan over the 1024 per-thread sums (Hillis-Steele; tiny compared with the vocabulary passes)
    for (int off = 1; off < 1024; off <<= 1) {
      const float t = tid >= off ? scan[tid - off] : 0.f;
      __syncthreads();
      scan[tid] += t;
      __syncthreads();
    }
    const float total = scan[1023];
    const float target_mass = uniform01(seed, ctr0 + 2 * i + 1) * total;
    if (tid == 0) pick_s = -1;
    __syncthreads();
    const float before = tid > 0 ? scan[tid - 1] : 0.f;
    if (total > 0.f && target_mass > before && target_mass <= scan[tid]) {
      float run = before;
      int pick = v1 - 1;
      for (int v = v0; v < v1; ++v) {
        run += weight(v);
        if (run >= target_mass) { pick = v; break; }
      }
      pick_s = pick;
    }
    __syncthreads();
    if (pick_s < 0) {
      // degenerate residual (p == q everywhere up to rounding): fall back to the mode of p
      float best = -INFINITY;
      int bi = 0;
      for (int v = tid; v < V; v += 1024)
        if (pl[v] > best) { best = pl[v]; bi = v; }
      const float bm = block_max(best, red);
      if (best == bm) atomicMax(&pick_s, bi);
      __syncthreads();
    }
    emitted = pick_s;
    break;
  }
  if (tid == 0) {
    a.n_accept[r] = n;
    for (int i = 0; i <= K; ++i) {
      long long v = -1;
      if (i < n) v = a.draft[(size_t)r * K + i];
      else if (i == n) v = emitted;
      a.out[(size_t)r * (K + 1) + i] = v;
    }
  }
}

// one thread per request: cursors and the journal row to publish
__global__ void spec_commit_kernel(const int* __restrict__ n_accept, const long long* __restrict__ out, int R, int K,
                                   long long* __restrict__ tokens, int* __restrict__ pos, int* __restrict__ ctx_len,
                                   int* __restrict__ commit_row, int* __restrict__ hidden_row) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const int n = n_accept[r];
  tokens[r] = out[(size_t)r * (K + 1) + n];
  pos[r] += n + 1;
  if (ctx_len != nullptr) ctx_len[r] = pos[r] + 1;
  if (commit_row != nullptr) commit_row[r] = r * (K + 1) + n;
  if (hidden_row != nullptr) hidden_row[r] = r * (K + 1) + n;
}

// dst[r][:] = src[rows[r]][:]  (fp32 rows; hidden hand-off to the next draft cycle)
__global__ void gather_rows_f32_kernel(const float* __restrict__ src, long long lds, const int* __restrict__ rows,
                                       float* __restrict__ dst, long long ldd, int H) {
  const int r = blockIdx.x;
  const float* s = src + (size_t)rows[r] * lds;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4)
    *reinterpret_cast<float4*>(dst + (size_t)r * ldd + i) = *reinterpret_cast<const float4*>(s + i);
}

}  // namespace

HE_API int he_spec_accept_greedy(const void* draft, const void* target, int R, int K, void* n_accept, void* out,
                                 const void* max_emit, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (K < 1 || K > 16) return -HE_ERR_BAD_ARG;
  spec_accept_greedy_kernel<<<(R + 63) / 64, 64, 0, stream>>>((const long long*)draft, (const long long*)target, R, K,
                                                              (int*)n_accept, (long long*)out, (const int*)max_emit);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_spec_accept_sampled(const SampledArgs* args, cudaStream_t stream) {
  if (args->R <= 0) return 0;
  if (args->K < 1 || args->K > 16 || args->V < 2) return -HE_ERR_BAD_ARG;
  spec_accept_sampled_kernel<<<args->R, 1024, 0, stream>>>(*args);
  HE_LAUNCH_CHECK();
  return 0;
}
HE_API int he_spec_sampled_args_size() { return (int)sizeof(SampledArgs); }

HE_API int he_spec_commit(const void* n_accept, const void* out, int R, int K, void* tokens, void* pos, void* ctx_len,
                          void* commit_row, void* hidden_row, cudaStream_t stream) {
  if (R <= 0) return 0;
  spec_commit_kernel<<<(R + 63) / 64, 64, 0, stream>>>((const int*)n_accept, (const long long*)out, R, K,
                                                       (long long*)tokens, (int*)pos, (int*)ctx_len, (int*)commit_row,
                                                       (int*)hidden_row);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_gather_rows_f32(const void* src, long long lds, const void* rows, void* dst, long long ldd, int R, int H,
                              cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H % 4 != 0) return -HE_ERR_BAD_ARG;
  gather_rows_f32_kernel<<<R, 256, 0, stream>>>((const float*)src, lds, (const int*)rows, (float*)dst, ldd, H);
  HE_LAUNCH_CHECK();
  return 0;
}
