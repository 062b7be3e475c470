// Gated DeltaNet prefill scan in chunked (WY) form on the tensor cores.
//
// The recurrence  S_t = g_t S_{t-1} + k_t d_t^T,  d_t = beta_t (v_t - (g_t S_{t-1})^T k_t),  o_t = S_t^T q_t
// (hipengine/kernels/cpu_reference/ops.py:1967-2012; chunked algebra oracle :2015-2141) is evaluated 16 tokens at
// a time.  With G_t = prod_{s<=t} g_s inside the chunk (kept as log-sums, ratios G_t/G_j <= 1 for j <= t):
//     A_tj = beta_t (G_t/G_j)(k_t.k_j), j < t          (strictly lower 16x16)
//     (I + A) [U | W] = [beta*V | beta*G*K]             (forward substitution, one thread per column)
//     D = U - W S_0                                     (the 16 delta rows)
//     O = (G*Q) S_0 + P D,  P_tj = (G_t/G_j)(q_t.k_j), j <= t
//     S_16 = G_16 S_0 + Kt^T D,  Kt_j = (G_16/G_j) k_j
// All matrix products run as mma.sync m16n8k8 TF32 (fp32 accumulate) from shared memory; the state slice stays in
// shared memory for the whole segment.  One CTA = (segment, V head, 32-column slice of the state), 4 warps; the
// next chunk's K / Q / V rows are fetched with cp.async while the current chunk computes.
// Used for prefill segments without a state journal; decode rows, verify chains and short segments keep the
// serial kernel in gdn.cu.  V head h reads K head h % G (GGUF order).
#include "common.cuh"

using namespace he;

namespace {

constexpr int CK = 16;          // tokens per chunk
constexpr int NST = 2;          // chunk buffers: the next chunk's rows are in flight while one computes (a third stage measured no gain)
constexpr int DK = 128;         // state rows (key dim)
constexpr int LDK = DK + 16;    // row stride (floats) of K / Q / W / transposed S: conflict-free 128-bit fragment reads
constexpr int LDA = CK + 1;

// Fragment convention for the 128-deep products (K K^T, Q K^T, Q S_0, W S_0): the k index is relabelled so that the
// four k values a lane feeds into two consecutive m16n8k8 steps are contiguous in memory (k0 + 4t .. k0 + 4t + 3,
// one 128-bit load); A and B use the same relabelling, so the product is unchanged.  Operands go in as raw fp32 bit
// patterns (the tensor core drops the low mantissa bits).
__device__ __forceinline__ uint4 ld4(const float* p) { return *reinterpret_cast<const uint4*>(p); }

struct GdnChunkArgs {
  const float* qkv;       // [T][C] prepared conv output: q | k | v (q, k normalised)
  const float* decay;     // [T][Hv]
  const float* beta;      // [T][Hv]
  float* state;           // [n_slots][Hv][128][128]
  const int* seg_start;   // [n_seg+1]
  const int* seg_slot;    // [n_seg]
  float* out;             // [T][Hv][128]
  int C, G, Hv, T, n_seg;
  int write_state;
};

__device__ __forceinline__ uint32_t tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <int NV>
struct Smem {
  static constexpr int LDS_ = NV + 8;   // row stride of S / V / D: conflict-free B-fragment reads
  float K[NST][CK][LDK];
  float Q[NST][CK][LDK];
  float V[NST][CK][LDS_];
  float St[NV][LDK];       // state slice, transposed: St[n][k]
  float W[CK][LDK];
  float D[CK][LDS_];       // delta rows
  float A[CK][LDA];
  float P[CK][LDA];
  float Tm[CK][LDA];       // (I + A)^-1
  float b[NST][CK];        // inclusive log-decay sums of the chunk
  float bt[NST][CK];       // beta
};

// grid (n_seg, Hv, DV/NV), block 128.  NV = 32 or 16 state columns per CTA: the narrower slice doubles the CTAs
// (and repeats the K K^T / Q K^T / inverse work per slice), which pays when one sequence is all there is.
template <int NV>
__global__ void __launch_bounds__(128) gdn_chunk_kernel(const GdnChunkArgs p) {
  constexpr int NT = NV / 8;              // n-tiles of the state slice
  constexpr int QT = NT / 2;              // n-tiles of Q S_0 per warp (warps 2 and 3)
  extern __shared__ __align__(16) uint8_t smem_raw[];
  Smem<NV>& sm = *reinterpret_cast<Smem<NV>*>(smem_raw);
  const int sg = blockIdx.x, h = blockIdx.y, sl = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int kh = h % p.G;
  const int s0 = p.seg_start[sg], s1 = p.seg_start[sg + 1];
  const int n_chunks = (s1 - s0 + CK - 1) / CK;
  float* Sg = p.state + (((size_t)p.seg_slot[sg] * p.Hv + h) * DK) * 128 + sl * NV;
  const size_t q_off = (size_t)kh * DK, k_off = (size_t)p.G * DK + (size_t)kh * DK;
  const size_t v_off = (size_t)2 * p.G * DK + (size_t)h * 128 + sl * NV;

  for (int i = tid; i < DK * (NV / 4); i += 128) {
    const int r = i / (NV / 4), c4 = (i % (NV / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(Sg + (size_t)r * 128 + c4);
    sm.St[c4][r] = v.x; sm.St[c4 + 1][r] = v.y; sm.St[c4 + 2][r] = v.z; sm.St[c4 + 3][r] = v.w;
  }

  auto prefetch = [&](int chunk, int buf) {
    const int c0 = s0 + chunk * CK;
    for (int i = tid; i < CK * (DK / 4); i += 128) {
      const int tt = i / (DK / 4), d4 = (i % (DK / 4)) * 4;
      const int tok = c0 + tt;
      const bool ok = tok < s1;
      const float* row = p.qkv + (size_t)(ok ? tok : s0) * p.C;
      cp_async16(&sm.K[buf][tt][d4], row + k_off + d4, ok ? 16 : 0);
      cp_async16(&sm.Q[buf][tt][d4], row + q_off + d4, ok ? 16 : 0);
    }
    for (int i = tid; i < CK * (NV / 4); i += 128) {
      const int tt = i / (NV / 4), d4 = (i % (NV / 4)) * 4;
      const int tok = c0 + tt;
      const bool ok = tok < s1;
      cp_async16(&sm.V[buf][tt][d4], p.qkv + (size_t)(ok ? tok : s0) * p.C + v_off + d4, ok ? 16 : 0);
    }
    cp_async_commit();
  };
  // The per-token decay / beta of a chunk are loaded one chunk ahead into registers (lanes 0..15 of warp 0) and
  // turned into the inclusive log-decay prefix at the end of the previous iteration, so that their global-load
  // latency is off the critical path.  Tokens past the segment end act as identity steps (decay 1, beta 0).
  float nd = 1.f, nbeta = 0.f;
  auto load_scalars = [&](int chunk) {
    if (tid < CK) {
      const int tok = s0 + chunk * CK + tid;
      const bool ok = tok < s1;
      nd = ok ? p.decay[(size_t)tok * p.Hv + h] : 1.f;
      nbeta = ok ? p.beta[(size_t)tok * p.Hv + h] : 0.f;
    }
  };
  auto store_scalars = [&](int buf) {
    if (tid < CK) {
      float lg = __logf(fmaxf(nd, 1e-37f));
#pragma unroll
      for (int o = 1; o < CK; o <<= 1) {
        const float v = __shfl_up_sync(0x0000ffffu, lg, o, CK);
        if (tid >= o) lg += v;
      }
      sm.b[buf][tid] = lg;
      sm.bt[buf][tid] = nbeta;
    }
  };

  // every warp keeps its 32 rows of the state slice in registers, in accumulator-fragment layout, for the whole
  // segment; shared memory only holds the copy the other warps read as a B operand
  float sreg[2][NT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int m0 = warp * 32 + mt * 16, n0 = nt * 8;
      sreg[mt][nt][0] = Sg[(size_t)(m0 + g) * 128 + n0 + 2 * t];
      sreg[mt][nt][1] = Sg[(size_t)(m0 + g) * 128 + n0 + 2 * t + 1];
      sreg[mt][nt][2] = Sg[(size_t)(m0 + g + 8) * 128 + n0 + 2 * t];
      sreg[mt][nt][3] = Sg[(size_t)(m0 + g + 8) * 128 + n0 + 2 * t + 1];
    }
  if (n_chunks > 0) {
    prefetch(0, 0);
    load_scalars(0);
    store_scalars(0);
  }
  if (NST > 2 && n_chunks > 1) prefetch(1, 1);
  float qs[QT][4];                         // warps 2,3: Q S_0 for their n-tiles
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int buf = ch % NST;
    if (NST > 2 && ch + 1 < n_chunks) cp_async_wait_1();   // all but the newest group (chunk ch+1) has landed
    else cp_async_wait_all();
    __syncthreads();                       // chunk data + previous state update visible to everyone
    if (ch + NST - 1 < n_chunks) prefetch(ch + NST - 1, (ch + NST - 1) % NST);
    if (ch + 1 < n_chunks) load_scalars(ch + 1);
    float (*K_)[LDK] = sm.K[buf];
    float (*Q_)[LDK] = sm.Q[buf];
    const float* b = sm.b[buf];
    const float* bt = sm.bt[buf];

    // ---- phase 1: warps 0,1: A = tril(beta G-ratio K K^T, -1), then warp 0 inverts (I + A);
    //               warps 2,3: P = tril(G-ratio Q K^T) and Q S_0 for two n-tiles each (shared Q fragments)
    if (warp < 2) {
      const int nt = warp;
      // legacy mma.sync has a long result latency on this part: four independent accumulation chains per tile
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f},
            c3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < DK; kk += 32) {
        const uint4 alo = ld4(&K_[g][kk + 4 * t]), ahi = ld4(&K_[g + 8][kk + 4 * t]);
        const uint4 bb = ld4(&K_[nt * 8 + g][kk + 4 * t]);
        const uint4 alo2 = ld4(&K_[g][kk + 16 + 4 * t]), ahi2 = ld4(&K_[g + 8][kk + 16 + 4 * t]);
        const uint4 bb2 = ld4(&K_[nt * 8 + g][kk + 16 + 4 * t]);
        mma_tf32(c0, alo.x, ahi.x, alo.y, ahi.y, bb.x, bb.y);
        mma_tf32(c1, alo.z, ahi.z, alo.w, ahi.w, bb.z, bb.w);
        mma_tf32(c2, alo2.x, ahi2.x, alo2.y, ahi2.y, bb2.x, bb2.y);
        mma_tf32(c3, alo2.z, ahi2.z, alo2.w, ahi2.w, bb2.z, bb2.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        c0[e] += c2[e];
        c1[e] += c3[e];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = g + (e >> 1) * 8, j = nt * 8 + 2 * t + (e & 1);
        sm.A[i][j] = j < i ? bt[i] * __expf(b[i] - b[j]) * (c0[e] + c1[e]) : 0.f;
      }
      asm volatile("bar.sync 1, 64;" ::: "memory");       // A complete (warps 0 and 1 only)
      if (warp == 0 && lane < CK) {
        // column `lane` of Tm = (I + A)^-1 by forward substitution; stored in P's sibling array sm.Tm
        float x[CK];
#pragma unroll
        for (int i = 0; i < CK; ++i) {
          float r = i == lane ? 1.f : 0.f;
#pragma unroll
          for (int m = 0; m < i; ++m) r -= sm.A[i][m] * x[m];
          x[i] = r;
          sm.Tm[i][lane] = r;
        }
      }
    } else {
      const int nt = warp - 2;
      float c0[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int q2 = 0; q2 < QT; ++q2)
#pragma unroll
        for (int e = 0; e < 4; ++e) qs[q2][e] = 0.f;
      const int n0 = nt * QT * 8;
      float c1[4] = {0.f, 0.f, 0.f, 0.f};
      float qs2[QT][4], qs3[QT][4], qs4[QT][4];     // extra chains of Q S_0, folded into qs[] after the loop
#pragma unroll
      for (int q2 = 0; q2 < QT; ++q2)
#pragma unroll
        for (int e = 0; e < 4; ++e) qs2[q2][e] = qs3[q2][e] = qs4[q2][e] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DK; kk += 32) {
        const uint4 alo = ld4(&Q_[g][kk + 4 * t]), ahi = ld4(&Q_[g + 8][kk + 4 * t]);
        const uint4 bk = ld4(&K_[nt * 8 + g][kk + 4 * t]);
        const uint4 alo2 = ld4(&Q_[g][kk + 16 + 4 * t]), ahi2 = ld4(&Q_[g + 8][kk + 16 + 4 * t]);
        const uint4 bk2 = ld4(&K_[nt * 8 + g][kk + 16 + 4 * t]);
        mma_tf32(c0, alo.x, ahi.x, alo.y, ahi.y, bk.x, bk.y);
        mma_tf32(c1, alo.z, ahi.z, alo.w, ahi.w, bk.z, bk.w);
        mma_tf32(c0, alo2.x, ahi2.x, alo2.y, ahi2.y, bk2.x, bk2.y);
        mma_tf32(c1, alo2.z, ahi2.z, alo2.w, ahi2.w, bk2.z, bk2.w);
#pragma unroll
        for (int q2 = 0; q2 < QT; ++q2) {
          const uint4 bs = ld4(&sm.St[n0 + q2 * 8 + g][kk + 4 * t]);
          const uint4 bs2 = ld4(&sm.St[n0 + q2 * 8 + g][kk + 16 + 4 * t]);
          mma_tf32(qs[q2], alo.x, ahi.x, alo.y, ahi.y, bs.x, bs.y);
          mma_tf32(qs2[q2], alo.z, ahi.z, alo.w, ahi.w, bs.z, bs.w);
          mma_tf32(qs3[q2], alo2.x, ahi2.x, alo2.y, ahi2.y, bs2.x, bs2.y);
          mma_tf32(qs4[q2], alo2.z, ahi2.z, alo2.w, ahi2.w, bs2.z, bs2.w);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) c0[e] += c1[e];
#pragma unroll
      for (int q2 = 0; q2 < QT; ++q2)
#pragma unroll
        for (int e = 0; e < 4; ++e) qs[q2][e] += qs2[q2][e] + (qs3[q2][e] + qs4[q2][e]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = g + (e >> 1) * 8, j = nt * 8 + 2 * t + (e & 1);
        sm.P[i][j] = j <= i ? __expf(b[i] - b[j]) * c0[e] : 0.f;
      }
    }
    __syncthreads();

    // ---- phase 2: [U | W] = Tm [beta V | beta G K]: warp w -> W n-tiles 4w..4w+3 (to shared) and U n-tile w (regs)
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    {
      uint32_t ta[2][4];
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        ta[ks][0] = tf32(sm.Tm[g][ks * 8 + t]);
        ta[ks][1] = tf32(sm.Tm[g + 8][ks * 8 + t]);
        ta[ks][2] = tf32(sm.Tm[g][ks * 8 + t + 4]);
        ta[ks][3] = tf32(sm.Tm[g + 8][ks * 8 + t + 4]);
      }
      float sc_lo[2], sc_hi[2], bt_lo[2], bt_hi[2];     // row scales of the right-hand sides for tokens ks*8+t, +4
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        bt_lo[ks] = bt[ks * 8 + t];
        bt_hi[ks] = bt[ks * 8 + t + 4];
        sc_lo[ks] = bt_lo[ks] * __expf(b[ks * 8 + t]);
        sc_hi[ks] = bt_hi[ks] * __expf(b[ks * 8 + t + 4]);
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const int n0 = (warp * 4 + q4) * 8;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          mma_tf32(c, ta[ks][0], ta[ks][1], ta[ks][2], ta[ks][3], tf32(K_[ks * 8 + t][n0 + g] * sc_lo[ks]),
                   tf32(K_[ks * 8 + t + 4][n0 + g] * sc_hi[ks]));
        *reinterpret_cast<float2*>(&sm.W[g][n0 + 2 * t]) = make_float2(c[0], c[1]);
        *reinterpret_cast<float2*>(&sm.W[g + 8][n0 + 2 * t]) = make_float2(c[2], c[3]);
      }
      if (warp < NT) {
        const int n0 = warp * 8;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          mma_tf32(u, ta[ks][0], ta[ks][1], ta[ks][2], ta[ks][3], tf32(sm.V[buf][ks * 8 + t][n0 + g] * bt_lo[ks]),
                   tf32(sm.V[buf][ks * 8 + t + 4][n0 + g] * bt_hi[ks]));
      }
    }
    __syncthreads();

    // ---- phase 3: D = U - W S_0   (warp w -> columns [8w, 8w+8)), two accumulation chains
    if (warp < NT) {
      const int n0 = warp * 8;
      float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
      float c2[4] = {0.f, 0.f, 0.f, 0.f}, c3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < DK; kk += 32) {
        const uint4 alo = ld4(&sm.W[g][kk + 4 * t]), ahi = ld4(&sm.W[g + 8][kk + 4 * t]);
        const uint4 bs = ld4(&sm.St[n0 + g][kk + 4 * t]);
        const uint4 alo2 = ld4(&sm.W[g][kk + 16 + 4 * t]), ahi2 = ld4(&sm.W[g + 8][kk + 16 + 4 * t]);
        const uint4 bs2 = ld4(&sm.St[n0 + g][kk + 16 + 4 * t]);
        mma_tf32(c0, alo.x, ahi.x, alo.y, ahi.y, bs.x, bs.y);
        mma_tf32(c1, alo.z, ahi.z, alo.w, ahi.w, bs.z, bs.w);
        mma_tf32(c2, alo2.x, ahi2.x, alo2.y, ahi2.y, bs2.x, bs2.y);
        mma_tf32(c3, alo2.z, ahi2.z, alo2.w, ahi2.w, bs2.z, bs2.w);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        c0[e] += c2[e];
        c1[e] += c3[e];
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = g + (e >> 1) * 8, j = n0 + 2 * t + (e & 1);
        sm.D[i][j] = u[e] - (c0[e] + c1[e]);
      }
    }
    __syncthreads();

    // ---- phase 4a (warps 2,3): O = G*(Q S_0) + P D for their two n-tiles
    if (warp >= 2) {
      const int c0t = s0 + ch * CK;
      uint32_t pa[2][4];
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        pa[ks][0] = tf32(sm.P[g][ks * 8 + t]);
        pa[ks][1] = tf32(sm.P[g + 8][ks * 8 + t]);
        pa[ks][2] = tf32(sm.P[g][ks * 8 + t + 4]);
        pa[ks][3] = tf32(sm.P[g + 8][ks * 8 + t + 4]);
      }
      const float g_lo = __expf(b[g]), g_hi = __expf(b[g + 8]);
#pragma unroll
      for (int q2 = 0; q2 < QT; ++q2) {
        const int n0 = ((warp - 2) * QT + q2) * 8;
        float c[4] = {qs[q2][0] * g_lo, qs[q2][1] * g_lo, qs[q2][2] * g_hi, qs[q2][3] * g_hi};
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          mma_tf32(c, pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], tf32(sm.D[ks * 8 + t][n0 + g]),
                   tf32(sm.D[ks * 8 + t + 4][n0 + g]));
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int tok = c0t + g + hh * 8;
          if (tok < s1)
            *reinterpret_cast<float2*>(p.out + ((size_t)tok * p.Hv + h) * 128 + sl * NV + n0 + 2 * t) =
                make_float2(c[hh * 2], c[hh * 2 + 1]);
        }
      }
    }
    // ---- phase 4b: S <- G_16 S_0 + Kt^T D   (warp w owns state rows [32w, 32w+32))
    {
      const float bl = b[CK - 1];
      const float gall = __expf(bl);
      float e_lo[2], e_hi[2];          // exp(b_16 - b_j) for the token columns this lane feeds: j = ks*8 + t, +4
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
        e_lo[ks] = __expf(bl - b[ks * 8 + t]);
        e_hi[ks] = __expf(bl - b[ks * 8 + t + 4]);
      }
      uint32_t ka[2][2][4];          // [mt][ks]: scaled K^T fragments of this warp's two 16-row tiles
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const int m0 = warp * 32 + mt * 16;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          const int j0 = ks * 8;
          ka[mt][ks][0] = tf32(K_[j0 + t][m0 + g] * e_lo[ks]);
          ka[mt][ks][1] = tf32(K_[j0 + t][m0 + g + 8] * e_lo[ks]);
          ka[mt][ks][2] = tf32(K_[j0 + t + 4][m0 + g] * e_hi[ks]);
          ka[mt][ks][3] = tf32(K_[j0 + t + 4][m0 + g + 8] * e_hi[ks]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int n0 = nt * 8;
        uint32_t db[2][2];
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          db[ks][0] = tf32(sm.D[ks * 8 + t][n0 + g]);
          db[ks][1] = tf32(sm.D[ks * 8 + t + 4][n0 + g]);
        }
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const int m0 = warp * 32 + mt * 16;
          float (&c)[4] = sreg[mt][nt];
#pragma unroll
          for (int e = 0; e < 4; ++e) c[e] *= gall;
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)
            mma_tf32(c, ka[mt][ks][0], ka[mt][ks][1], ka[mt][ks][2], ka[mt][ks][3], db[ks][0], db[ks][1]);
          // publish the rows this warp owns for the next chunk's B-operand reads
          sm.St[n0 + 2 * t][m0 + g] = c[0];
          sm.St[n0 + 2 * t + 1][m0 + g] = c[1];
          sm.St[n0 + 2 * t][m0 + g + 8] = c[2];
          sm.St[n0 + 2 * t + 1][m0 + g + 8] = c[3];
        }
      }
    }
    if (ch + 1 < n_chunks) store_scalars((ch + 1) % NST);
  }
  __syncthreads();
  if (p.write_state) {
    for (int i = tid; i < DK * (NV / 4); i += 128) {
      const int r = i / (NV / 4), c4 = (i % (NV / 4)) * 4;
      *reinterpret_cast<float4*>(Sg + (size_t)r * 128 + c4) =
          make_float4(sm.St[c4][r], sm.St[c4 + 1][r], sm.St[c4 + 2][r], sm.St[c4 + 3][r]);
    }
  }
}



// Chunked tensor-core scan.  Same arguments as he_gdn_scan minus the journal; state size must be 128.
template <int NV>
int launch_chunk(const GdnChunkArgs& a, cudaStream_t stream) {
  const size_t smem = sizeof(Smem<NV>);
  // set per call (cheap): the attribute belongs to the (function, device) pair, not to the process
  cudaError_t e = cudaFuncSetAttribute(gdn_chunk_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(a.n_seg, a.Hv, 128 / NV);
  gdn_chunk_kernel<NV><<<grid, 128, smem, stream>>>(a);
  HE_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// Chunked tensor-core scan.  Same arguments as he_gdn_scan minus the journal; state size must be 128.
HE_API int he_gdn_scan_chunked(const GdnChunkArgs* args, cudaStream_t stream) {
  if (args->T <= 0 || args->n_seg <= 0) return 0;
  if (args->C != 2 * args->G * 128 + args->Hv * 128) return -HE_ERR_BAD_ARG;
  static const int nv_env = []() { const char* e = getenv("HE_GDN_NV"); return e ? atoi(e) : 0; }();
  // 16-column slices double the CTAs but repeat the per-chunk K K^T / inverse work; measured equal to 32 columns on a
  // single 4096-token sequence, so the wider slice is the default (HE_GDN_NV=16 selects the narrow one)
  // ... unless the grid would leave most SMs idle (few heads: a tensor-parallel shard), where more CTAs win
  int sms = 148;
  {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool narrow = nv_env == 16 || (nv_env == 0 && (long long)args->n_seg * args->Hv * 4 <= sms);
  return narrow ? launch_chunk<16>(*args, stream) : launch_chunk<32>(*args, stream);
}
HE_API int he_gdn_chunk_args_size() { return (int)sizeof(GdnChunkArgs); }
