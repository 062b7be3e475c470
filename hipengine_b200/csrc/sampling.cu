// Output-head reductions and the on-device sampler.
//
//  * argmax over fp32 logits rows in two stages; ties resolve to the lowest token id
//    (hipengine/generation/sampling.py:1733; kernels hipengine/kernels/hip_gfx1100/linear/lm_head.hip).
//  * sampler: temperature -> top-k -> top-p -> min-p -> seeded draw, one CTA per row.  Instead of the
//    reference's full-vocabulary sort (sampler_sort_tiles/merge/scan in sampling/sampler.hip, scratch
//    rows*(24*vocab) bytes) the kept set is found by bisection on a probability threshold, which needs no
//    scratch memory at all; the draw walks the kept tokens in id order, so results are deterministic
//    for a given (seed, counter).
//  * top-N logprobs (N <= 32) by repeated masked argmax.
#include "common.cuh"

using namespace he;

namespace {

struct MaxIdx {
  float v;
  int i;
};

__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ MaxIdx warp_argmax(MaxIdx m) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx t;
    t.v = __shfl_xor_sync(0xffffffffu, m.v, o);
    t.i = __shfl_xor_sync(0xffffffffu, m.i, o);
    m = better(m, t);
  }
  return m;
}

__device__ MaxIdx block_argmax(MaxIdx m, MaxIdx* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  m = warp_argmax(m);
  __syncthreads();
  if (lane == 0) sh[warp] = m;
  __syncthreads();
  MaxIdx t;
  t.v = -INFINITY;
  t.i = 0x7fffffff;
  if (lane < nw) t = sh[lane];
  return warp_argmax(t);
}

constexpr int AM_PARTS = 64;

// grid (AM_PARTS, R)
__global__ void __launch_bounds__(256) argmax_stage1(const float* __restrict__ logits, long long stride, int V,
                                                     float* __restrict__ pv, int* __restrict__ pi) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  __shared__ MaxIdx sh[32];
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * stride;
  const int per = (V + AM_PARTS - 1) / AM_PARTS;
  const int b = blockIdx.x * per, e = min(V, b + per);
  MaxIdx m;
  m.v = -INFINITY;
  m.i = 0x7fffffff;
  for (int i = b + threadIdx.x; i < e; i += blockDim.x) {
    MaxIdx c;
    c.v = row[i];
    c.i = i;
    m = better(m, c);
  }
  m = block_argmax(m, sh);
  if (threadIdx.x == 0) {
    pv[r * AM_PARTS + blockIdx.x] = m.v;
    pi[r * AM_PARTS + blockIdx.x] = m.i;
  }
}

// grid R, block 64
__global__ void argmax_stage2(const float* __restrict__ pv, const int* __restrict__ pi, long long* __restrict__ out,
                              float* __restrict__ out_val) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  __shared__ MaxIdx sh[32];
  const int r = blockIdx.x;
  MaxIdx m;
  m.v = pv[r * AM_PARTS + threadIdx.x];
  m.i = pi[r * AM_PARTS + threadIdx.x];
  m = block_argmax(m, sh);
  if (threadIdx.x == 0) {
    out[r] = m.i == 0x7fffffff ? 0 : m.i;
    if (out_val != nullptr) out_val[r] = m.v;
  }
}

// ---- counter-based RNG: SplitMix64 finaliser over (seed, counter) -> uniform in [0, 1)
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (counter + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

struct SampleParams {
  float temperature;
  int top_k;
  float top_p;
  float min_p;
  unsigned long long seed;
  unsigned long long counter;
};

// grid R, block 1024.  out_id[r], out_logprob[r] (log-softmax of the *processed* distribution at T).
__global__ void __launch_bounds__(1024) sample_rows_kernel(const float* __restrict__ logits, long long stride, int V,
                                                           const SampleParams* __restrict__ params,
                                                           long long* __restrict__ out_id,
                                                           float* __restrict__ out_logprob) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  __shared__ float red[33];
  __shared__ MaxIdx shm[32];
  __shared__ float scan[1024];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * stride;
  const SampleParams sp = params[r];
  // greedy rows
  MaxIdx m;
  m.v = -INFINITY;
  m.i = 0x7fffffff;
  for (int i = tid; i < V; i += blockDim.x) {
    MaxIdx c;
    c.v = row[i];
    c.i = i;
    m = better(m, c);
  }
  m = block_argmax(m, shm);
  const float mx = m.v;
  if (sp.temperature <= 0.f) {
    if (tid == 0) {
      out_id[r] = m.i;
      if (out_logprob != nullptr) out_logprob[r] = 0.f;
    }
    return;
  }
  const float invT = 1.f / sp.temperature;
  float z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) z += __expf((row[i] - mx) * invT);
  z = block_sum(z, red);
  // Threshold t on x_i = (logit_i - max)/T; the kept set is {x_i >= t}.  count(t) and mass(t) both fall as t
  // rises, so  t* = max(t_k, t_p)  is the largest t with  count(t) >= k  OR  mass(t) >= top_p * z.
  const bool need_k = sp.top_k > 0 && sp.top_k < V;
  const bool need_p = sp.top_p > 0.f && sp.top_p < 1.f;
  float thr = -INFINITY;
  if (need_k || need_p) {
    float lo = -100.f, hi = 1e-3f;
    for (int it = 0; it < 40; ++it) {
      const float mid = 0.5f * (lo + hi);
      float cnt = 0.f, mass = 0.f;
      for (int i = tid; i < V; i += blockDim.x) {
        const float x = (row[i] - mx) * invT;
        if (x >= mid) { cnt += 1.f; mass += __expf(x); }
      }
      cnt = block_sum(cnt, red);
      mass = block_sum(mass, red);
      const bool pred = (need_k && cnt >= (float)sp.top_k) || (need_p && mass >= sp.top_p * z);
      if (pred) lo = mid; else hi = mid;
    }
    thr = lo;
  }
  if (sp.min_p > 0.f) thr = fmaxf(thr, logf(sp.min_p));
  const float tau = thr == -INFINITY ? 0.f : __expf(thr) * (1.f - 1e-6f);
  // kept mass and draw
  float mass = 0.f;
  for (int i = tid; i < V; i += blockDim.x) {
    const float e = __expf((row[i] - mx) * invT);
    if (e >= tau) mass += e;
  }
  const float my_mass = mass;
  const float total = block_sum(mass, red);
  const float u = uniform01(sp.seed, sp.counter) * total;
  // inclusive scan of per-thread masses in *interleaved* ownership order is not id order; to keep the draw in
  // id order, re-own contiguous ranges: thread t covers ids [t*per, (t+1)*per).
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int b = tid * per, e_ = min(V, b + per);
  float cm = 0.f;
  for (int i = b; i < e_; ++i) {
    const float e = __expf((row[i] - mx) * invT);
    if (e >= tau) cm += e;
  }
  scan[tid] = cm;
  __syncthreads();
  (void)my_mass;
  if (tid == 0) {
    float run = 0.f;
    int owner = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (run + scan[t] > u && scan[t] > 0.f) { owner = t; break; }
      run += scan[t];
    }
    if (owner < 0) {  // numerical tail: fall back to the last thread holding mass
      run = 0.f;
      for (int t = 0; t < (int)blockDim.x; ++t) if (scan[t] > 0.f) owner = t;
      for (int t = 0; t < owner; ++t) run += scan[t];
    }
    int pick = m.i;
    const int ob = owner * per, oe = min(V, ob + per);
    int last_kept = -1;
    for (int i = ob; i < oe; ++i) {
      const float e = __expf((row[i] - mx) * invT);
      if (e >= tau) {
        last_kept = i;
        run += e;
        if (run > u) { pick = i; last_kept = -2; break; }
      }
    }
    if (last_kept >= 0) pick = last_kept;
    out_id[r] = pick;
    if (out_logprob != nullptr) out_logprob[r] = (row[pick] - mx) * invT - logf(total);
  }
}

// Top-N (N<=32) ids + log-softmax values per row by repeated masked argmax.  grid R, block 1024.
__global__ void __launch_bounds__(1024) topn_logprobs_kernel(const float* __restrict__ logits, long long stride,
                                                             int V, int N, float temperature,
                                                             const long long* __restrict__ chosen,
                                                             int* __restrict__ top_ids, float* __restrict__ top_lp,
                                                             float* __restrict__ chosen_lp) {
  __shared__ float red[33];
  __shared__ MaxIdx shm[32];
  __shared__ int taken[32];
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * stride;
  const float invT = temperature > 0.f ? 1.f / temperature : 1.f;
  MaxIdx m;
  m.v = -INFINITY;
  m.i = 0x7fffffff;
  for (int i = tid; i < V; i += blockDim.x) {
    MaxIdx c;
    c.v = row[i];
    c.i = i;
    m = better(m, c);
  }
  m = block_argmax(m, shm);
  const float mx = m.v;
  float z = 0.f;
  for (int i = tid; i < V; i += blockDim.x) z += __expf((row[i] - mx) * invT);
  z = block_sum(z, red);
  const float lz = logf(z);
  if (tid == 0 && chosen_lp != nullptr && chosen != nullptr) chosen_lp[r] = (row[chosen[r]] - mx) * invT - lz;
  for (int k = 0; k < N; ++k) {
    MaxIdx b;
    b.v = -INFINITY;
    b.i = 0x7fffffff;
    for (int i = tid; i < V; i += blockDim.x) {
      bool skip = false;
      for (int j = 0; j < k; ++j) skip |= (taken[j] == i);
      if (!skip) {
        MaxIdx c;
        c.v = row[i];
        c.i = i;
        b = better(b, c);
      }
    }
    b = block_argmax(b, shm);
    if (tid == 0) {
      taken[k] = b.i;
      top_ids[r * N + k] = b.i;
      top_lp[r * N + k] = (b.v - mx) * invT - lz;
    }
    __syncthreads();
  }
}

// softcap in place: x = cap * tanh(x / cap)
__global__ void softcap_kernel(float* x, long long n, float cap) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

}  // namespace

// scratch: pv float[R*64], pi int[R*64] supplied by the caller.
HE_API int he_argmax_rows(const void* logits, long long stride, int R, int V, void* pv, void* pi, void* out_ids,
                          void* out_val, cudaStream_t stream) {
  if (R <= 0) return 0;
  dim3 g1(AM_PARTS, R);
  (void)launch_pdl(argmax_stage1, dim3(g1), dim3(256), 0, stream, (const float*)logits, stride, V, (float*)pv, (int*)pi);
  HE_LAUNCH_CHECK();
  (void)launch_pdl(argmax_stage2, dim3(R), dim3(AM_PARTS), 0, stream, (const float*)pv, (const int*)pi, (long long*)out_ids, (float*)out_val);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_sample_rows(const void* logits, long long stride, int R, int V, const void* params, void* out_ids,
                          void* out_logprob, cudaStream_t stream) {
  if (R <= 0) return 0;
  (void)launch_pdl(sample_rows_kernel, dim3(R), dim3(1024), 0, stream, (const float*)logits, stride, V, (const SampleParams*)params,
                                             (long long*)out_ids, (float*)out_logprob);
  HE_LAUNCH_CHECK();
  return 0;
}
HE_API int he_sample_params_size() { return (int)sizeof(SampleParams); }

HE_API int he_topn_logprobs(const void* logits, long long stride, int R, int V, int N, float temperature,
                            const void* chosen, void* top_ids, void* top_lp, void* chosen_lp, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (N < 0 || N > 32) return -HE_ERR_BAD_ARG;
  topn_logprobs_kernel<<<R, 1024, 0, stream>>>((const float*)logits, stride, V, N, temperature,
                                               (const long long*)chosen, (int*)top_ids, (float*)top_lp,
                                               (float*)chosen_lp);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_softcap(void* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  (void)launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (float*)x, n, cap);
  HE_LAUNCH_CHECK();
  return 0;
}
