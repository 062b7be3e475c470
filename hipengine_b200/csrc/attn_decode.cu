// Paged GQA decode attention: split-K partial pass + reduce with the fused sigmoid output gate.
//
// One CTA owns (row, kv head, key span) and serves all G = H/Hkv query heads of that kv head from one
// read of the K/V pages, writing un-normalised partial outputs plus (max, sum) to a scratch buffer;
// a second small kernel merges the spans, applies sigmoid(gate) and stores bf16.
// Behavioural reference: the split-K producers/reducers in
// hipengine/kernels/hip_gfx1100/attention/paged_attn_decode.hip (chunk = KV block, reduce_threads = head_dim,
// gate fused in the reducer) and the live-span oracle hipengine/kernels/cpu_reference/ops.py:2895-2997.
// KV cache layout: [n_pages][2 (k,v)][Hkv][PAGE][D] bf16, addressed through block_table[slot][pos / PAGE].
#include <cstdlib>

#include "common.cuh"
#include "sm100.cuh"

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
  int* status;                // optional status word: a bounded wait that gave up records its code here
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
        const int pg = bt[HE_INDEX_OK(pos / a.page, a.max_pages, HE_SITE_ATTN_DECODE_PAGE) ? pos / a.page : 0];
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
      const int pg = bt[HE_INDEX_OK(pos / a.page, a.max_pages, HE_SITE_ATTN_DECODE_PAGE) ? pos / a.page : 0];
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

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core split kernel.  Same contract as attn_decode_split_kernel (one CTA per (row, kv head, key span), partial
// outputs + (max, sum) per span), built so that the K/V bytes of a span are touched exactly once on every level:
//   producer warp  : streams whole KV pages (16 keys x D) row by row with 1-D bulk copies into a ring of stages of
//                    64 keys (rows padded by 16 bytes, which makes every ldmatrix conflict-free); first all K tiles
//                    of the span, then all V tiles, so V is already in flight while the softmax statistics run;
//   phase 1        : S = Q K^T with mma.sync m16n8k16 (the G <= 8 query heads of the group are the rows of the M
//                    tile; warp w takes the w-th page of every stage), scores to shared memory;
//   phase 2        : per-head max / sum over the span, P = exp(S - max) as bf16 rows in shared memory;
//   phase 3        : O = P V, warp w owns D/4 output columns and walks every stage.
// Reads of shared memory equal the bytes copied in; the span's keys never pass through registers as scalars.
namespace mma_dec {

constexpr int NCONS = 4;                    // consumer warps
constexpr int NTHREADS = (NCONS + 1) * 32;  // + one producer warp
constexpr int TILE_KEYS = 64;
constexpr int MAX_STAGES = 5;        // barrier slots
constexpr int RING_STAGES = 2;       // stages in use: with two stages (~68 KB for head_dim 256) three CTAs share an SM
                                     // and hide each other's phase changes; one CTA with a five-stage ring left the
                                     // SM at 8 % warp occupancy and 20 % of DRAM bandwidth

template <int D>
__host__ __device__ constexpr int pitch() { return D * 2 + 16; }
// ring depth: one stage per tile the span has (K and V), at most five, and what ~170 KB of shared memory hold
template <int D>
__host__ __device__ inline int stages_for(int split_len) {
  const int uses = 2 * ((split_len + TILE_KEYS - 1) / TILE_KEYS);
  const int fit = (170 * 1024) / (TILE_KEYS * pitch<D>());
  const int cap = fit < RING_STAGES ? fit : RING_STAGES;
  return uses < cap ? uses : cap;
}
template <int D>
__host__ __device__ inline size_t smem_bytes(int G, int split_len) {
  return (size_t)stages_for<D>(split_len) * TILE_KEYS * pitch<D>() + 8 * (size_t)pitch<D>() +
         8 * ((size_t)split_len * 2 + 16) + (size_t)G * split_len * 4 + 2 * MAX_STAGES * 8 + 16;
}

__device__ __forceinline__ void ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
// D (16x8 fp32) += A (16x16 bf16, rows 8..15 zero: a1 = a3 = 0) * B (16x8 bf16)
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bulk_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(sm100::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCONS * 32) : "memory"); }

template <int D, int G>
__global__ void __launch_bounds__(NTHREADS) attn_decode_mma_kernel(const AttnDecArgs a) {
  static_assert(G <= 8 && D % 64 == 0, "group of <= 8 query heads, head_dim a multiple of 64");
  extern __shared__ __align__(128) uint8_t smem_raw[];
  constexpr int PITCH = pitch<D>();
  constexpr int STAGE = TILE_KEYS * PITCH;
  const int sp = blockIdx.x, hk = blockIdx.y, r = blockIdx.z;
  pdl_wait();
  pdl_launch();
  const int ctx = a.ctx_len[r];
  const int start = (a.window > 0 && ctx > a.window) ? ctx - a.window : 0;
  const int k0 = start + sp * a.split_len;
  if (k0 >= ctx) return;
  const int n = min(a.split_len, ctx - k0);
  const int ntile = (n + TILE_KEYS - 1) / TILE_KEYS;
  const int NST = stages_for<D>(a.split_len);
  const int PP = a.split_len * 2 + 16;                 // pitch of a P row (bytes)
  uint8_t* ring = smem_raw;
  uint8_t* q_s = ring + (size_t)NST * STAGE;           // [8][PITCH] bf16 rows (rows >= G zero)
  uint8_t* p_s = q_s + 8 * PITCH;                      // [8][PP] bf16 rows
  float* sc = reinterpret_cast<float*>(p_s + 8 * (size_t)PP);     // [G][split_len]
  uint64_t* full = reinterpret_cast<uint64_t*>(sc + (size_t)G * a.split_len);
  uint64_t* empty = full + MAX_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + MAX_STAGES);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = a.block_table + (size_t)a.slot[r] * a.max_pages;

  if (tid == 0) {
    for (int s = 0; s < NST; ++s) {
      sm100::mbar_init(&full[s], 1);
      sm100::mbar_init(&empty[s], NCONS);
    }
    *abort_flag = 0;
    sm100::mbar_fence_init();
  }
  __syncthreads();

  if (warp == NCONS) {
    // ------------------------------------------------------------ producer: K tiles, then V tiles
    int s = 0;
    uint32_t ph = 0;
    for (int u = 0; u < 2 * ntile; ++u) {
      if (!sm100::mbar_wait(&empty[s], ph ^ 1u, abort_flag, a.status, 401)) break;
      const int kv = u < ntile ? 0 : 1, tile = u < ntile ? u : u - ntile;
      if (lane == 0) sm100::mbar_expect_tx(&full[s], (uint32_t)(TILE_KEYS * D * 2));
      __syncwarp();
#pragma unroll
      for (int h2 = 0; h2 < TILE_KEYS / 32; ++h2) {
        const int row = lane + 32 * h2;
        // rows past the span re-read its last key: finite values that the zero probabilities then ignore
        const int pos = k0 + min(tile * TILE_KEYS + row, n - 1);
        const int pg = bt[HE_INDEX_OK(pos / a.page, a.max_pages, HE_SITE_ATTN_DECODE_PAGE) ? pos / a.page : 0];
        const __nv_bfloat16* src =
            a.kv_cache + ((((size_t)pg * 2 + kv) * a.Hkv + hk) * a.page + (pos % a.page)) * D;
        bulk_row(ring + (size_t)s * STAGE + (size_t)row * PITCH, src, D * 2, &full[s]);
      }
      if (++s == NST) {
        s = 0;
        ph ^= 1u;
      }
    }
    return;
  }

  // ------------------------------------------------------------ consumers
  // Q rows of the group as bf16 (rows >= G and the P rows >= G stay zero)
  for (int i = tid; i < 8 * (PITCH / 16); i += NCONS * 32) {
    const int g = i / (PITCH / 16), c = i % (PITCH / 16);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (g < G && c < D / 8) v = *reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.H + hk * G + g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + (size_t)g * PITCH + c * 16) = v;
  }
  for (int i = tid; i < (8 - G) * (PP / 16); i += NCONS * 32) {
    const int g = G + i / (PP / 16), c = i % (PP / 16);
    *reinterpret_cast<uint4*>(p_s + (size_t)g * PP + c * 16) = make_uint4(0u, 0u, 0u, 0u);
  }
  cons_sync();

  int s = 0;
  uint32_t ph = 0;
  bool ok = true;
  // ---- phase 1: scores of 16 keys per warp and stage
  {
    // ldmatrix row addresses: Q (x2: k 0-7 | k 8-15 of rows 0-7), K (x4: keys 0-7 | 8-15, each k-lo | k-hi)
    const uint32_t q_addr = sm100::smem_u32(q_s) + (lane & 7) * PITCH + ((lane >> 3) & 1) * 16;
    const int k_row = warp * 16 + ((lane >> 4) & 1) * 8 + (lane & 7);
    const int k_col = ((lane >> 3) & 1) * 16;
    for (int t = 0; t < ntile && ok; ++t) {
      if (!sm100::mbar_wait(&full[s], ph, abort_flag, a.status, 402)) { ok = false; break; }
      const int key0 = t * TILE_KEYS + warp * 16;      // first key of this warp's page, relative to the span
      if (key0 < n) {
        const uint32_t k_addr = sm100::smem_u32(ring + (size_t)s * STAGE) + k_row * PITCH + k_col;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int ks = 0; ks < D / 16; ++ks) {
          uint32_t a0, a2, b0, b1, b2, b3;
          ldsm_x2(q_addr + ks * 32, a0, a2);
          ldsm_x4(k_addr + ks * 32, b0, b1, b2, b3);
          mma_16816(s0, a0, a2, b0, b1);
          mma_16816(s1, a0, a2, b2, b3);
        }
        const int g = lane >> 2, kc = 2 * (lane & 3);
        if (g < G) {
          float* row = sc + (size_t)g * a.split_len + key0;
          const float NEG = -INFINITY;
          row[kc] = key0 + kc < n ? s0[0] * a.scale : NEG;
          row[kc + 1] = key0 + kc + 1 < n ? s0[1] * a.scale : NEG;
          row[8 + kc] = key0 + 8 + kc < n ? s1[0] * a.scale : NEG;
          row[8 + kc + 1] = key0 + 8 + kc + 1 < n ? s1[1] * a.scale : NEG;
        }
      }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&empty[s]);
      if (++s == NST) {
        s = 0;
        ph ^= 1u;
      }
    }
  }
  cons_sync();
  if (*abort_flag) return;

  // ---- phase 2: per-head softmax statistics of the span, P as bf16 rows
  const int n16 = (n + 15) & ~15;                       // keys covered by the live pages
  float* part_base = a.partial + (((size_t)r * a.H + hk * G) * a.max_splits + sp) * (D + 2);
  for (int g = warp; g < G; g += NCONS) {
    const float* srow = sc + (size_t)g * a.split_len;
    __nv_bfloat16* prow = reinterpret_cast<__nv_bfloat16*>(p_s + (size_t)g * PP);
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, srow[i]);
    m = warp_max(m);
    float l = 0.f;
    for (int i = lane; i < n16; i += 32) {
      const float p = i < n ? __expf(srow[i] - m) : 0.f;
      prow[i] = f32_to_bf16(p);
      l += p;
    }
    l = warp_sum(l);
    if (lane == 0) {
      float* pb = part_base + (size_t)g * a.max_splits * (D + 2);
      pb[D] = m;
      pb[D + 1] = l;
    }
  }
  cons_sync();

  // ---- phase 3: O[:, warp's D/4 columns] = P V over every stage
  constexpr int DW = D / NCONS;                          // output columns per warp
  constexpr int NB = DW / 8;                             // 8-column blocks per warp
  float o[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  {
    const uint32_t p_addr = sm100::smem_u32(p_s) + (lane & 7) * PP + ((lane >> 3) & 1) * 16;
    // V (x4.trans): keys 0-7 | 8-15 of column block j, then of block j + 1
    const int v_row = ((lane >> 3) & 1) * 8 + (lane & 7);
    const int v_col = (warp * DW + ((lane >> 4) & 1) * 8) * 2;
    for (int t = 0; t < ntile && ok; ++t) {
      if (!sm100::mbar_wait(&full[s], ph, abort_flag, a.status, 403)) { ok = false; break; }
      const uint32_t v_base = sm100::smem_u32(ring + (size_t)s * STAGE) + v_row * PITCH + v_col;
#pragma unroll
      for (int kk = 0; kk < TILE_KEYS / 16; ++kk) {
        const int key0 = t * TILE_KEYS + kk * 16;
        if (key0 < n) {
          uint32_t a0, a2;
          ldsm_x2(p_addr + key0 * 2, a0, a2);
#pragma unroll
          for (int j = 0; j < NB; j += 2) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(v_base + kk * 16 * PITCH + j * 16, b0, b1, b2, b3);
            mma_16816(o[j], a0, a2, b0, b1);
            mma_16816(o[j + 1], a0, a2, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) sm100::mbar_arrive(&empty[s]);
      if (++s == NST) {
        s = 0;
        ph ^= 1u;
      }
    }
  }
  if (!ok) return;
  const int g = lane >> 2;
  if (g < G) {
    float* pb = part_base + (size_t)g * a.max_splits * (D + 2) + warp * DW + 2 * (lane & 3);
#pragma unroll
    for (int j = 0; j < NB; ++j) *reinterpret_cast<float2*>(pb + j * 8) = make_float2(o[j][0], o[j][1]);
  }
}

}  // namespace mma_dec

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

// HE_ATTN_DECODE=scalar keeps the CUDA-core split kernel (for comparisons).
bool mma_decode_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HE_ATTN_DECODE");
    v = (e != nullptr && e[0] == 's') ? 0 : 1;
  }
  return v != 0;
}

template <int D, int G>
int launch_split_mma(const AttnDecArgs& a, cudaStream_t stream) {
  const size_t smem = mma_dec::smem_bytes<D>(G, a.split_len);
  static size_t configured[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mma_dec::attn_decode_mma_kernel<D, G>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = smem;
  }
  dim3 grid(a.max_splits, a.Hkv, a.R);
  cudaError_t le = launch_pdl(mma_dec::attn_decode_mma_kernel<D, G>, grid, dim3(mma_dec::NTHREADS), smem, stream, a);
  if (le != cudaSuccess) return (int)le;
  return 0;
}

template <int D, int G>
int launch_split(const AttnDecArgs& a, cudaStream_t stream) {
  if constexpr (D >= 128 && G <= 8) {
    // tensor-core kernel: whole 16-key pages, spans that are a multiple of 16 keys, rings that fit shared memory
    if (mma_decode_enabled() && a.page == 16 && a.split_len % 16 == 0 &&
        mma_dec::smem_bytes<D>(G, a.split_len) <= 220 * 1024)
      return launch_split_mma<D, G>(a, stream);
  }
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
