// Causal paged GQA prefill attention (append-then-attend) with the fused sigmoid output gate.
//
// Flash-style single pass: a CTA owns 64 query rows of one head (4 warps x 16 rows), streams 32-key tiles of
// K and V out of the paged cache with cp.async (double buffered), keeps running max / sum per row and the
// 16 x D output accumulator in registers.  Tensor-core path: mma.sync m16n8k16 bf16 with fp32 accumulation
// (the projections, which are >98% of prefill FLOPs, run on tcgen05; this kernel is bounded by the softmax
// pipeline, not by the MMA rate).  The queries of one segment sit at consecutive positions
// pos0 .. pos0+T-1 and attend keys 0 .. their own position (optionally only the last `window` keys).
// Behavioural reference: hipengine/kernels/hip_gfx1100/attention/paged_attn_decode.hip (prefill_gqa_gate_*
// kernels) and the oracle hipengine/kernels/cpu_reference/ops.py:2144-2256 (output rounded to bf16 before the
// gate multiply).
#include "common.cuh"

using namespace he;

namespace {

constexpr int BM = 64;       // query rows per CTA
constexpr int BN = 32;       // keys per tile
constexpr int NTHR = 128;

struct PrefillArgs {
  const __nv_bfloat16* q;      // [T][H][D]
  const __nv_bfloat16* gate;   // [T][H][D] or null
  const __nv_bfloat16* kv;     // [n_pages][2][Hkv][page][D]
  const int* block_table;      // row of this segment's slot: [max_pages]
  __nv_bfloat16* out;          // [T][H*D]
  int T, H, Hkv, page, pos0, window;
  float scale_log2;            // scale * log2(e)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int D>
__global__ void __launch_bounds__(NTHR) flash_prefill_kernel(const PrefillArgs a) {
  constexpr int LDS = D + 8;                 // padded row stride (elements) -> conflict-free ldmatrix
  extern __shared__ __align__(16) __nv_bfloat16 sm[];
  __nv_bfloat16* sQ = sm;                    // [BM][LDS]
  __nv_bfloat16* sK = sQ + BM * LDS;         // [2][BN][LDS]
  __nv_bfloat16* sV = sK + 2 * BN * LDS;     // [2][BN][LDS]

  const int qt = gridDim.x - 1 - blockIdx.x; // heavy (late) tiles first
  const int h = blockIdx.y, hk = h / (a.H / a.Hkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int t0 = qt * BM;
  const int rows = min(BM, a.T - t0);
  const int q_pos_last = a.pos0 + t0 + rows - 1;
  const int kv_end = q_pos_last + 1;                                   // keys [0, kv_end)
  int kv_begin = 0;
  if (a.window > 0) kv_begin = max(0, a.pos0 + t0 - a.window + 1) / BN * BN;
  const int n_tiles = (kv_end - kv_begin + BN - 1) / BN;

  auto load_kv = [&](int tile, int buf) {
    const int k0 = kv_begin + tile * BN;
    constexpr int CH = D / 8;                                          // 16-byte chunks per row
    for (int i = tid; i < BN * CH; i += NTHR) {
      const int r = i / CH, ch = i % CH;
      const int p = k0 + r;
      const bool valid = p < kv_end;
      const int pc = valid ? p : kv_end - 1;
      const int pg = a.block_table[pc / a.page];
      const size_t base = ((((size_t)pg * 2) * a.Hkv + hk) * a.page + (pc % a.page)) * D + ch * 8;
      const size_t vofs = (size_t)a.Hkv * a.page * D;
      cp_async16(sK + ((size_t)buf * BN + r) * LDS + ch * 8, a.kv + base, valid);
      cp_async16(sV + ((size_t)buf * BN + r) * LDS + ch * 8, a.kv + base + vofs, valid);
    }
  };

  // Q tile (rows past T are zero)
  {
    constexpr int CH = D / 8;
    for (int i = tid; i < BM * CH; i += NTHR) {
      const int r = i / CH, ch = i % CH;
      const bool valid = r < rows;
      const size_t src = ((size_t)(t0 + (valid ? r : 0)) * a.H + h) * D + ch * 8;
      cp_async16(sQ + (size_t)r * LDS + ch * 8, a.q + src, valid);
    }
  }
  load_kv(0, 0);
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int qrow0 = a.pos0 + t0 + warp * 16 + g;       // position of this thread's first row (second is +8)

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < n_tiles) load_kv(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    // ---- S = Q K^T  (16 x 32 per warp)
    float sacc[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
    const __nv_bfloat16* kb = sK + (size_t)buf * BN * LDS;
#pragma unroll
    for (int kk = 0; kk < D / 32; ++kk) {               // 32 d per step = two k16 steps
      uint32_t qa0[4], qa1[4];
      const __nv_bfloat16* qp = sQ + (size_t)(warp * 16 + (lane & 15)) * LDS + kk * 32 + (lane >> 4) * 8;
      ldmatrix_x4(qa0, qp);
      ldmatrix_x4(qa1, qp + 16);
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) {
        uint32_t kf[4];
        ldmatrix_x4(kf, kb + (size_t)(j * 8 + (lane & 7)) * LDS + kk * 32 + (lane >> 3) * 8);
        mma_bf16(sacc[j], qa0, kf[0], kf[1]);
        mma_bf16(sacc[j], qa1, kf[2], kf[3]);
      }
    }

    // ---- mask + online softmax (rows g and g+8 of this warp's 16)
    const int k0 = kv_begin + tile * BN;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + j * 8 + 2 * c + (e & 1);
        const int qp = qrow0 + (e >> 1) * 8;
        bool ok = key <= qp && key < kv_end;
        if (a.window > 0) ok = ok && key > qp - a.window;
        const float v = ok ? sacc[j][e] * a.scale_log2 : -INFINITY;
        sacc[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float corr[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      corr[r] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= corr[r];
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pa[BN / 16][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mref = m_run[e >> 1];
        p[e] = (mref == -INFINITY) ? 0.f : exp2f(sacc[j][e] - mref);
        rs[e >> 1] += p[e];
      }
      pa[j >> 1][(j & 1) * 2] = pack_bf16(p[0], p[1]);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
    }
    l_run[0] += rs[0];
    l_run[1] += rs[1];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1];
    }

    // ---- O += P V   (P: 16 x 32, V: 32 x D)
    const __nv_bfloat16* vb = sV + (size_t)buf * BN * LDS;
#pragma unroll
    for (int ks = 0; ks < BN / 16; ++ks) {
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {                 // two n8 tiles per ldmatrix.x4.trans
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vb + (size_t)(ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LDS + i * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * i], pa[ks], vf[0], vf[1]);
        mma_bf16(o[2 * i + 1], pa[ks], vf[2], vf[3]);
      }
    }
    __syncthreads();
  }

  // ---- epilogue: normalise, round to bf16, gate, store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + r * 8;
    if (row >= rows) continue;
    const int t = t0 + row;
    const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int d = i * 8 + 2 * c;
      float v0 = o[i][r * 2] * inv, v1 = o[i][r * 2 + 1] * inv;
      if (a.gate != nullptr) {
        const __nv_bfloat162 gt = *reinterpret_cast<const __nv_bfloat162*>(a.gate + ((size_t)t * a.H + h) * D + d);
        const float2 gf = __bfloat1622float2(gt);
        v0 = bf16_to_f32(f32_to_bf16(v0)) * sigmoid_f(gf.x);
        v1 = bf16_to_f32(f32_to_bf16(v1)) * sigmoid_f(gf.y);
      }
      *reinterpret_cast<__nv_bfloat162*>(a.out + (size_t)t * a.H * D + (size_t)h * D + d) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

template <int D>
int launch(const PrefillArgs& a, cudaStream_t stream) {
  const size_t smem = (size_t)(BM + 4 * BN) * (D + 8) * sizeof(__nv_bfloat16);
  // set per call (cheap): the attribute belongs to the (function, device) pair, not to the process
  cudaError_t e = cudaFuncSetAttribute(flash_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((a.T + BM - 1) / BM, a.H);
  flash_prefill_kernel<D><<<grid, NTHR, smem, stream>>>(a);
  HE_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// One segment: T query rows at positions pos0 .. pos0+T-1 of the request whose block-table row is `block_table_row`.
HE_API int he_flash_prefill(const void* q, const void* gate, const void* kv_cache, const void* block_table_row,
                            void* out, int T, int H, int Hkv, int D, int page, int pos0, float scale, int window,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % Hkv != 0) return -HE_ERR_BAD_ARG;
  PrefillArgs a;
  a.q = (const __nv_bfloat16*)q; a.gate = (const __nv_bfloat16*)gate; a.kv = (const __nv_bfloat16*)kv_cache;
  a.block_table = (const int*)block_table_row; a.out = (__nv_bfloat16*)out;
  a.T = T; a.H = H; a.Hkv = Hkv; a.page = page; a.pos0 = pos0; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  switch (D) {
    case 64: return launch<64>(a, stream);
    case 128: return launch<128>(a, stream);
    case 256: return launch<256>(a, stream);
    default: return -HE_ERR_BAD_ARG;
  }
}
