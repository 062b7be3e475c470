// Paged GQA decode attention: split-K partial pass + reduce with the fused sigmoid output gate.
//
// One CTA owns (row, kv head, key span) and serves all G = H/Hkv query heads of that kv head from one
// read of the K/V pages, writing un-normalised partial outputs plus (max, sum) to a scratch buffer;
// a second small kernel merges the spans, applies sigmoid(gate) and stores bf16.
// Behavioural reference: the split-K producers/reducers in
// hipengine/kernels/hip_gfx1100/attention/paged_attn_decode.hip (chunk = KV block, reduce_threads = head_dim,
// gate fused in the reducer) and the live-span oracle hipengine/kernels/cpu_reference/ops.py:2895-2997.
// KV cache layout: [n_pages][2 (k,v)][Hkv][PAGE][D] bf16, addressed through block_table[slot][pos / PAGE].
#include "common.cuh"

using namespace he;

struct AttnDecArgs {
  const __nv_bfloat16* q;     // [R][H][D]
  const __nv_bfloat16* gate;  // [R][H][D] or null
  const __nv_bfloat16* kv_cache;
  const int* block_table;     // [n_slots][max_pages]
  const int* slot;            // [R]
  const int* ctx_len;         // [R] keys visible to the row (its own token included)
  float* partial;             // [R][H][max_splits][D + 2]
  __nv_bfloat16* out;         // [R][H*D]
  int R, H, Hkv, D, page, max_pages;
  int split_len, max_splits;
  int window;                 // > 0: only the last `window` keys are visible
  float scale;
};

namespace {

constexpr int NWARP = 8;

template <int D, int G>
__global__ void __launch_bounds__(256) attn_decode_split_kernel(const AttnDecArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int sp = blockIdx.x, hk = blockIdx.y, r = blockIdx.z;
  pdl_wait();
  pdl_launch();
  const int ctx = a.ctx_len[r];
  const int start = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int k0 = start + sp * a.split_len;
  if (k0 >= ctx) return;
  const int n = min(a.split_len, ctx - k0);
  float* q_s = smem;                       // [G][D]
  float* sc = q_s + G * D;                 // [G][split_len]
  float* red = sc + G * a.split_len;       // [NWARP][G][D]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = a.block_table + (size_t)a.slot[r] * a.max_pages;

  for (int i = tid; i < G * D; i += 256) {
    const int g = i / D, d = i % D;
    q_s[i] = bf16_to_f32(a.q[((size_t)r * a.H + hk * G + g) * D + d]) * a.scale;
  }
  __syncthreads();

  // ---- phase 1: scores.  8 lanes per key; lane `sub` owns 16-byte chunks sub, sub+8, ...
  {
    const int sub = lane & 7, grp = lane >> 3;
#pragma unroll 2
    for (int t0 = warp * 4; t0 < n; t0 += NWARP * 4) {
      const int tk = t0 + grp;
      float acc[G];
#pragma unroll
      for (int g = 0; g < G; ++g) acc[g] = 0.f;
      if (tk < n) {
        const int pos = k0 + tk;
        const int pg = bt[pos / a.page];
        const __nv_bfloat16* kr = a.kv_cache + ((((size_t)pg * 2 + 0) * a.Hkv + hk) * a.page + (pos % a.page)) * D;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          const int ch = sub + 8 * c;
          const uint4 kv = ldg128(kr + ch * 8);
          const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
          float kf[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(k2[e]);
            kf[2 * e] = f.x; kf[2 * e + 1] = f.y;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(q_s + g * D + ch * 8);
            const float4 qb = *reinterpret_cast<const float4*>(q_s + g * D + ch * 8 + 4);
            acc[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x + kf[5] * qb.y +
                      kf[6] * qb.z + kf[7] * qb.w;
          }
        }
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float v = acc[g];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        if (sub == 0 && tk < n) sc[g * a.split_len + tk] = v;
      }
    }
  }
  __syncthreads();

  // ---- phase 2: per-head softmax statistics inside the span (warp g handles head g)
  float* part_base = a.partial + (((size_t)r * a.H + hk * G) * a.max_splits + sp) * (D + 2);
  for (int g = warp; g < G; g += NWARP) {
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, sc[g * a.split_len + i]);
    m = warp_max(m);
    float l = 0.f;
    for (int i = lane; i < n; i += 32) {
      const float p = __expf(sc[g * a.split_len + i] - m);
      sc[g * a.split_len + i] = p;
      l += p;
    }
    l = warp_sum(l);
    if (lane == 0) {
      float* pb = part_base + (size_t)g * a.max_splits * (D + 2);
      pb[D] = m;
      pb[D + 1] = l;
    }
  }
  __syncthreads();

  // ---- phase 3: P·V.  A warp step covers TPS keys; a lane owns CPL 16-byte chunks of its key's V row.
  constexpr int NCH = D / 8;
  constexpr int CPL = NCH >= 32 ? NCH / 32 : 1;
  constexpr int TPS = NCH >= 32 ? 1 : 32 / NCH;
  float acc[G][CPL * 8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < CPL * 8; ++e) acc[g][e] = 0.f;
  const int tgrp = NCH >= 32 ? 0 : lane / NCH;
  const int ch0 = NCH >= 32 ? lane : lane % NCH;
#pragma unroll 2
  for (int t0 = warp * TPS; t0 < n; t0 += NWARP * TPS) {
    const int tk = t0 + tgrp;
    if (tk < n) {
      const int pos = k0 + tk;
      const int pg = bt[pos / a.page];
      const __nv_bfloat16* vr = a.kv_cache + ((((size_t)pg * 2 + 1) * a.Hkv + hk) * a.page + (pos % a.page)) * D;
      float p[G];
#pragma unroll
      for (int g = 0; g < G; ++g) p[g] = sc[g * a.split_len + tk];
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const uint4 vv = ldg128(vr + (ch0 + 32 * c) * 8);
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(v2[e]);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            acc[g][c * 8 + 2 * e] += p[g] * f.x;
            acc[g][c * 8 + 2 * e + 1] += p[g] * f.y;
          }
        }
      }
    }
  }
  if constexpr (TPS > 1) {
#pragma unroll
    for (int off = NCH; off < 32; off <<= 1)
#pragma unroll
      for (int g = 0; g < G; ++g)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], off);
  }
  if (tgrp == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int c = 0; c < CPL; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[((size_t)warp * G + g) * D + (ch0 + 32 * c) * 8 + e] = acc[g][c * 8 + e];
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 256) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) s += red[(size_t)w * G * D + i];
    const int g = i / D, d = i % D;
    part_base[(size_t)g * a.max_splits * (D + 2) + d] = s;
  }
}

// grid (H, R), block D.  Split statistics are staged in shared memory first, so the accumulation over splits
// is a stream of independent loads instead of a chain of dependent ones.
__global__ void attn_decode_reduce_kernel(const AttnDecArgs a) {
  extern __shared__ float wsm[];     // [max_splits] softmax weights of the splits
  __shared__ float red[33];
  const int h = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  const int D = a.D;
  pdl_wait();
  pdl_launch();
  const int ctx = a.ctx_len[r];
  const int start = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  // never past what the split kernel wrote (its grid is max_splits wide) nor past wsm[]: a context longer than
  // split_len * max_splits is the caller's error and is reduced over the first max_splits splits only
  const int ns = min((ctx - start + a.split_len - 1) / a.split_len, a.max_splits);
  const float* pb = a.partial + ((size_t)r * a.H + h) * a.max_splits * (D + 2);
  float m = -INFINITY;
  for (int s = d; s < ns; s += blockDim.x) {
    const float ms = pb[(size_t)s * (D + 2) + D];
    wsm[s] = ms;
    m = fmaxf(m, ms);
  }
  m = block_max(m, red);
  float den = 0.f;
  for (int s = d; s < ns; s += blockDim.x) {
    const float w = __expf(wsm[s] - m);
    wsm[s] = w;
    den += w * pb[(size_t)s * (D + 2) + D + 1];
  }
  den = block_sum(den, red);      // barriers inside also publish wsm[]
  float n4[4] = {0.f, 0.f, 0.f, 0.f};
  int s = 0;
  for (; s + 4 <= ns; s += 4) {
#pragma unroll
    for (int u = 0; u < 4; ++u) n4[u] += wsm[s + u] * pb[(size_t)(s + u) * (D + 2) + d];
  }
  for (; s < ns; ++s) n4[0] += wsm[s] * pb[(size_t)s * (D + 2) + d];
  const float num = (n4[0] + n4[1]) + (n4[2] + n4[3]);
  float o = den > 0.f ? num / den : 0.f;
  if (a.gate != nullptr) {
    // the reference rounds the attention output to bf16 before the gate multiply (cpu_reference/ops.py:2250)
    o = bf16_to_f32(f32_to_bf16(o)) * sigmoid_f(bf16_to_f32(a.gate[((size_t)r * a.H + h) * D + d]));
  }
  a.out[(size_t)r * a.H * D + (size_t)h * D + d] = f32_to_bf16(o);
}

template <int D, int G>
int launch_split(const AttnDecArgs& a, cudaStream_t stream) {
  const size_t smem = ((size_t)G * D + (size_t)G * a.split_len + (size_t)NWARP * G * D) * sizeof(float);
  // the attribute belongs to the (function, device) pair: remember the largest value set per device
  static size_t configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_split_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = smem;
  }
  dim3 grid(a.max_splits, a.Hkv, a.R);
  cudaError_t le = launch_pdl(attn_decode_split_kernel<D, G>, grid, dim3(256), smem, stream, a);
  if (le != cudaSuccess) return (int)le;
  return 0;
}

template <int D>
int dispatch_g(const AttnDecArgs& a, cudaStream_t stream) {
  switch (a.H / a.Hkv) {
    case 1: return launch_split<D, 1>(a, stream);
    case 2: return launch_split<D, 2>(a, stream);
    case 3: return launch_split<D, 3>(a, stream);
    case 4: return launch_split<D, 4>(a, stream);
    case 6: return launch_split<D, 6>(a, stream);
    case 8: return launch_split<D, 8>(a, stream);
    default: return -HE_ERR_BAD_ARG;
  }
}

}  // namespace

// Scratch needed by he_attn_decode: R*H*max_splits*(D+2) floats, supplied by the caller in args->partial.
HE_API int he_attn_decode(const AttnDecArgs* args, cudaStream_t stream) {
  const AttnDecArgs& a = *args;
  if (a.R <= 0) return 0;
  if (a.H % a.Hkv != 0 || a.split_len <= 0 || a.max_splits <= 0) return -HE_ERR_BAD_ARG;
  int rc;
  switch (a.D) {
    case 64: rc = dispatch_g<64>(a, stream); break;
    case 128: rc = dispatch_g<128>(a, stream); break;
    case 256: rc = dispatch_g<256>(a, stream); break;
    case 512: rc = dispatch_g<512>(a, stream); break;
    default: return -HE_ERR_BAD_ARG;
  }
  if (rc != 0) return rc;
  dim3 grid(a.H, a.R);
  cudaError_t le = launch_pdl(attn_decode_reduce_kernel, grid, dim3(a.D), (size_t)a.max_splits * sizeof(float),
                              stream, a);
  if (le != cudaSuccess) return (int)le;
  return 0;
}
HE_API int he_attn_dec_args_size() { return (int)sizeof(AttnDecArgs); }

// ------------------------------------------------------------------------------------------------
// Allocation-free variant (declared in attn_decode_noalloc.h; no counterpart in the reference engine).
// The split-K partials go to a fixed array inside this module's device image instead of a caller
// buffer, for callers that must not allocate: during or between stream captures, when the KV pool
// owns all remaining device memory, or when calling the C symbols without a tensor framework.
// One array per device, shared by all calls: calls that may overlap on the device race on it.
#include "attn_decode_noalloc.h"

static __device__ __align__(256) float g_noalloc_partial[HE_ATTN_NOALLOC_MAX_FLOATS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};  // address of g_noalloc_partial on each device, once looked up
}  // namespace

HE_API long long he_attn_decode_noalloc_capacity(void) { return (long long)HE_ATTN_NOALLOC_MAX_FLOATS; }

HE_API int he_attn_decode_noalloc(const AttnDecArgs* args, cudaStream_t stream) {
  if (args == nullptr) return -HE_ERR_BAD_ARG;
  if (args->R <= 0) return 0;
  if (args->H <= 0 || args->max_splits <= 0 || args->D <= 0) return -HE_ERR_BAD_ARG;
  const unsigned long long need =
      (unsigned long long)args->R * args->H * (unsigned long long)args->max_splits * (unsigned long long)(args->D + 2);
  if (need > (unsigned long long)HE_ATTN_NOALLOC_MAX_FLOATS) return -HE_ERR_BAD_ARG;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return -HE_ERR_BAD_ARG;
  if (g_noalloc_ptr[dev] == nullptr) {
    // Set-up, once per device with that device current.  Do this before any stream capture begins.
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_partial);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return (int)cudaErrorInvalidSymbol;
    g_noalloc_ptr[dev] = ptr;
  }
  AttnDecArgs a = *args;
  a.partial = g_noalloc_ptr[dev];
  return he_attn_decode(&a, stream);
}
