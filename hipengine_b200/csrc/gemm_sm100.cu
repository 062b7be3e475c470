// Tensor-core GEMM for sm_100a: C[M][N] = A[M][K] * B[N][K]^T with bf16 operands and fp32 accumulation in
// tensor memory (TMEM).  Persistent, warp-specialised:
//   warp 0     : TMA producer  (cp.async.bulk.tensor, 128-byte swizzled K-major tiles, 4-stage ring)
//   warp 1     : MMA issuer    (one elected thread issues tcgen05.mma 128x256x16; owns the TMEM allocation)
//   warps 2..5 : epilogue      (tcgen05.ld 32 lanes x 32 columns -> bf16/fp32 -> global; optional fused
//                               residual add or act(gate)*up)
// Two 256-column accumulators (all 512 TMEM columns) alternate between tiles so the epilogue of tile i
// overlaps the main loop of tile i+1.  Tiles are walked M-fastest so CTAs running at the same time share
// the weight tile in L2.  This is the projection engine for prefill / verify / wide decode
// (roles of hipengine/kernels/hip_gfx1100/quant/gguf_q4_k_prefill.hip and gguf_q8_0_prefill.hip in the
// reference, which use 16x16x16 WMMA with one wave per block).
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_BYTES = BN * BK * 2;   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int ACC_COLS = BN;           // fp32 columns per accumulator
constexpr int TMEM_COLS = 512;
constexpr int NTHREADS = 192;
constexpr int NTHREADS_FUSED = 320;    // + 4 collective warps (fused GEMM -> all-reduce kernel)

// Quantised-B mode (QM): the weight stays in its GGUF-derived device layout (Q4_K 144-byte blocks, Q6_K 224-byte
// blocks, Q8_0 int8 + scale planes) all the way into shared memory.  One extra warp streams raw block bytes with
// 2-D byte-typed TMA boxes into a small ring ("q-stages"); eight unpack warps expand each 64-column slice to bf16
// straight into the 128-byte-swizzled K-major operand stage that the MMA issuer reads, so DRAM and L2 only ever see
// 4.5 / 6.6 / 8.5 bits per weight and no bf16 copy of the weight exists anywhere.
//   Q4_K : q-stage = one 256-column super-block per row (144 B): 4 k-blocks per q-stage
//   Q6_K : q-stage = one 128-column half block per row (ql 64 B + qh 32 B + scales/d 32 B): 2 k-blocks
//   Q8_0 : q-stage = 128 columns per row (128 B int8 + the 16-byte scale group of the 256-aligned range): 2 k-blocks
constexpr int STAGES_Q = 3;            // A / dequantised-B ring depth in QM
constexpr int QSTAGES = 2;             // raw-block ring depth
constexpr int Q_STAGE_BYTES = BN * 144;
constexpr int N_UNPACK_WARPS = 8;
constexpr int NTHREADS_FUSED_Q = NTHREADS_FUSED + 32 * (1 + N_UNPACK_WARPS);

struct GemmArgs {
  void* C;
  long long ldc;        // elements
  const float* resid;   // unused (reserved)
  int M, N, K;
  int epi;              // 0: bf16 store, 1: fp32 store, 2: fp32 += (C is fp32, in place)
  int* status;
  // grouped mode (MoE experts): M-tile tm multiplies rows [tm*BM, +BM) of A with the weight block
  // B[tile_group[tm] * N .. +N); a negative group marks an unused tile.  Null for a plain GEMM.
  const int* tile_group;
  // split-K (small M, few output tiles): the K range is cut into k_splits pieces handled by different CTAs, which
  // add their partial tiles into the fp32 C with atomics (epi 3).  1 = off.
  int k_splits;
  long long split_stride;   // epi 4: split ks stores its fp32 partial tile at C + ks * split_stride (elements)
  int qtype;                // QM kernels: HE_Q4_K / HE_Q6_K / HE_Q8_0
  int kb_per;               // k-blocks per split when > 0 (set by the split-K launchers), else derived from k_splits
};

// Fused GEMM -> all-reduce -> residual add over peer memory (tensor-parallel row-parallel projections).
// Every rank owns one symmetric region, mapped into all peers:
//     stage  [world src][owned_cap][BM*BN] bf16 : partial tiles pushed by rank `src` for the tiles this rank owns
//     result [max_tiles][BM*BN] bf16            : reduced tiles, written by each tile's owner into every rank
//     flags  arrive[max_tiles][world][4] u32, then done[max_tiles][4] u32 : epoch stamps per 32-row tile quarter
// Tile t (M-fastest index) is owned by rank t % world.  One kernel per rank runs three phases; all
// synchronisation is per warp (phase 1: the four epilogue warps; phases 2 and 3: four extra "collective" warps that
// run beside the GEMM pipeline for the whole kernel; each warp handles one 32-row quarter of a tile):
//   1. the GEMM epilogue stores its partial quarter straight into the owner's stage slot (peer stores for remote
//      owners), fences at system scope and stamps arrive[t][me][q] on the owner;
//   2. for each owned tile, wait (bounded) for the world stamps of the quarter, sum the slots in rank order in
//      fp32, store the bf16 result into every rank's result region and stamp done[t][q] there;
//   3. for each tile, wait (bounded) for done[t][q] locally and add the result rows into the fp32 residual.
// The transfers of phase 1 overlap the MMAs of later tiles.  The epoch lives in device memory and is advanced by the
// last CTA to leave, so the kernel can be replayed from a CUDA graph.  `phases` (bit 0/1/2) selects which phases a
// launch runs: 7 in production; a single-GPU test runs the phases of several emulated ranks as separate launches
// (1,1,..,2,2,..,4,4,..) so that no launch ever waits for a later one.
constexpr int FUSE_MAX_WORLD = 8;
constexpr int TILE_ELEMS = 128 * 256;

struct FuseArgs {
  __nv_bfloat16* stage[FUSE_MAX_WORLD];
  __nv_bfloat16* result[FUSE_MAX_WORLD];
  uint32_t* flags[FUSE_MAX_WORLD];
  uint32_t* sync;         // local [2]: epoch of the last finished call, CTAs that have left the current call
  float* resid;           // local fp32 [M][ld_resid]: resid += all-reduced product
  long long ld_resid;
  int world, rank, max_tiles, owned_cap, phases;
  unsigned wait_limit;
  // 1: one-hop form for small worlds.  Every rank stores its partial tiles into ALL ranks' stage buffers
  // (stage [2 epoch parities][world src][max_tiles][BM*BN], owned_cap = max_tiles) and every rank reduces every tile
  // itself, straight into its residual: (world-1) x the link traffic of the owner form at world > 2, the same at
  // world = 2, but one flag hop instead of two and no result buffer.  Two parities because a rank may be one call
  // ahead of a peer that still reads the previous call's tiles.
  int direct;
  int reserved;
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// resid[0..3] += v, no return value: the add happens at the L2, so the adder never waits for the old value
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Whole-warp probe: true when the n stamps p[lane * stride] (lanes < n) have all reached `epoch` (stamps only grow).
__device__ __forceinline__ bool warp_stamps_ready(const uint32_t* p, int n, int stride, uint32_t epoch) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  if (lane < n) ok = (int)(ld_acquire_sys_u32(p + (size_t)lane * stride) - epoch) >= 0;
  return __all_sync(0xffffffffu, ok);
}

// Phase 2 for one warp: quarter q of owned tile mn -- sum the world stage slots in rank order, store the bf16 result
// into every rank, stamp done[mn][q] everywhere.  The quarter is 32 rows x 256 columns = 1024 16-byte groups.
__device__ __forceinline__ void fuse_reduce_quarter(const FuseArgs* f, int mn, int q, uint32_t epoch) {
  const int lane = threadIdx.x & 31, W = f->world;
  const size_t q_off = (size_t)q * 32 * 256;
  const __nv_bfloat16* src0 = f->stage[f->rank] + (size_t)(mn / W) * TILE_ELEMS + q_off;
  const size_t src_stride = (size_t)f->owned_cap * TILE_ELEMS;
  const size_t dst_off = (size_t)mn * TILE_ELEMS + q_off;
#pragma unroll 1
  for (int it0 = 0; it0 < 32; it0 += 4) {
    float acc[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
    // two ranks' slots in flight at a time (8 independent 16-byte loads per lane); the sums stay in rank order
    for (int r = 0; r < W; r += 2) {
      const bool two = r + 1 < W;
      uint4 v[4], v2[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const size_t o = (size_t)((it0 + u) * 32 + lane) * 8;
        v[u] = ld_cg_u4(src0 + (size_t)r * src_stride + o);
        v2[u] = two ? ld_cg_u4(src0 + (size_t)(r + 1) * src_stride + o) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
        const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&v2[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t2 = __bfloat1622float2(hv[e]);
          acc[u][2 * e] += t2.x;
          acc[u][2 * e + 1] += t2.y;
        }
        if (two) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t2 = __bfloat1622float2(hw[e]);
            acc[u][2 * e] += t2.x;
            acc[u][2 * e + 1] += t2.y;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint4 pk;
      uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 h2 = __floats2bfloat162_rn(acc[u][2 * e], acc[u][2 * e + 1]);
        pw[e] = *reinterpret_cast<uint32_t*>(&h2);
      }
      const size_t e0 = (size_t)((it0 + u) * 32 + lane) * 8;
      for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(f->result[r] + dst_off + e0) = pk;
    }
  }
  __threadfence_system();
  __syncwarp();
  if (lane < W) st_release_sys_u32(f->flags[lane] + (size_t)f->max_tiles * W * 4 + (size_t)mn * 4 + q, epoch);
}

// Phase 3 for one warp: resid rows of quarter q of tile mn += reduced tile.  Lane = row of the quarter (the tile is
// fragment-major, so the 32 lanes read 512 contiguous bytes per column group); 16 column groups in flight; the adds
// are vector red.add, each lane covering one full 32-byte sector of its row.
__device__ __forceinline__ void fuse_add_quarter(const FuseArgs* f, int mn, int q, int tiles_m, int M, int N) {
  const int lane = threadIdx.x & 31;
  const int tm = mn % tiles_m, tn = mn / tiles_m;
  const __nv_bfloat16* res = f->result[f->rank] + (size_t)mn * TILE_ELEMS + (size_t)q * 8192 + lane * 8;
  const int row = tm * 128 + q * 32 + lane;
  const int col0 = tn * 256;
  const bool live = row < M;
  float* hrow = f->resid + (size_t)(live ? row : 0) * f->ld_resid + col0;
#pragma unroll 1
  for (int cg0 = 0; cg0 < 32; cg0 += 16) {
    if (col0 + cg0 * 8 >= N) break;
    uint4 v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u)
      v[u] = (live && col0 + (cg0 + u) * 8 < N) ? ld_cg_u4(res + (size_t)(cg0 + u) * 256) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      if (live && col0 + (cg0 + u) * 8 < N) {
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
        const float2 a0 = __bfloat1622float2(hv[0]), a1 = __bfloat1622float2(hv[1]);
        const float2 a2 = __bfloat1622float2(hv[2]), a3 = __bfloat1622float2(hv[3]);
        float* hp = hrow + (cg0 + u) * 8;
        red_add_f32x4(hp, a0.x, a0.y, a1.x, a1.y);
        red_add_f32x4(hp + 4, a2.x, a2.y, a3.x, a3.y);
      }
    }
  }
}

// One-hop form, one warp: resid rows of quarter q of tile mn += bf16(sum over ranks of the stage slots), ranks in
// order.  Lane = row of the quarter, 8 column groups in flight per rank slot, vector red.add into the residual.
__device__ __forceinline__ void fuse_direct_quarter(const FuseArgs* f, int mn, int q, int tiles_m, int M, int N,
                                                    uint32_t epoch) {
  const int lane = threadIdx.x & 31, W = f->world;
  const int tm = mn % tiles_m, tn = mn / tiles_m;
  const size_t slot_stride = (size_t)f->owned_cap * TILE_ELEMS;
  const __nv_bfloat16* src = f->stage[f->rank] + (size_t)(epoch & 1u) * W * slot_stride + (size_t)mn * TILE_ELEMS +
                             (size_t)q * 8192 + lane * 8;
  const int row = tm * 128 + q * 32 + lane;
  const int col0 = tn * 256;
  const bool live = row < M;
  float* hrow = f->resid + (size_t)(live ? row : 0) * f->ld_resid + col0;
#pragma unroll 1
  for (int cg0 = 0; cg0 < 32; cg0 += 8) {
    if (col0 + cg0 * 8 >= N) break;
    float acc[8][8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
    for (int r = 0; r < W; ++r) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = (live && col0 + (cg0 + u) * 8 < N) ? ld_cg_u4(src + (size_t)r * slot_stride + (size_t)(cg0 + u) * 256)
                                                  : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t2 = __bfloat1622float2(hv[e]);
          acc[u][2 * e] += t2.x;
          acc[u][2 * e + 1] += t2.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (live && col0 + (cg0 + u) * 8 < N) {
        // round the sum to bf16 first: the same value the owner form broadcasts, so both forms agree bit for bit
        float s8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) s8[e] = __bfloat162float(__float2bfloat16_rn(acc[u][e]));
        float* hp = hrow + (cg0 + u) * 8;
        red_add_f32x4(hp, s8[0], s8[1], s8[2], s8[3]);
        red_add_f32x4(hp + 4, s8[4], s8[5], s8[6], s8[7]);
      }
    }
  }
}

struct __align__(8) Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t bfull[STAGES];     // QM: dequantised B slice of the stage is in place (one arrive per unpack warp)
  uint64_t qfull[QSTAGES];    // QM: raw blocks of the q-stage have landed (TMA bytes)
  uint64_t qempty[QSTAGES];   // QM: every unpack warp is done with the q-stage
  uint32_t tmem_base;
  int abort_flag;
};

// ---------------------------------------------------------------- in-pipeline dequantisation (QM)
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ __nv_bfloat162 bf162_bits(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }
__device__ __forceinline__ uint32_t bits_bf162(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Four small unsigned integers (< 128), one per byte of `b4`, become two bf16x2 registers holding
// (q - sub) * s + add.  A byte q under the high byte 0x43 is the bf16 number 128 + q exactly, so the integer
// reaches bf16 with one byte permute and one subtract; the scale and offset are applied by a single fused
// multiply-add (one rounding).
__device__ __forceinline__ void bytes4_to_bf16(uint32_t b4, __nv_bfloat162 sub, __nv_bfloat162 s, __nv_bfloat162 add,
                                               uint32_t& o01, uint32_t& o23) {
  const uint32_t MAGIC = 0x43434343u;
  const __nv_bfloat162 v0 = __hsub2(bf162_bits(prmt_b32(b4, MAGIC, 0x5140u)), sub);
  const __nv_bfloat162 v1 = __hsub2(bf162_bits(prmt_b32(b4, MAGIC, 0x7362u)), sub);
  o01 = bits_bf162(__hfma2(v0, s, add));
  o23 = bits_bf162(__hfma2(v1, s, add));
}

// 16-byte chunk `chunk` (0..7) of row `row` in a K-major operand tile with the 128-byte swizzle.
__device__ __forceinline__ void st_b_chunk(uint8_t* bstage, int row, int chunk, uint4 v) {
  *reinterpret_cast<uint4*>(bstage + (size_t)row * 128 + (size_t)((chunk ^ (row & 7)) << 4)) = v;
}

// Q4_K: thread `ut` (0..255) owns weight row `ut` of the tile; k-block c (0..3) of the staged super-block is the 32
// nibble bytes [16 + 32c, +32) of the 144-byte block: low nibbles = columns 0..31, high nibbles = columns 32..63.
__device__ __forceinline__ void unpack_q4k(const uint8_t* qst, uint8_t* bstage, int ut, int c) {
  const uint8_t* blk = qst + (size_t)ut * 144;
  const uint4 meta = *reinterpret_cast<const uint4*>(blk);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&meta.x));
  uint32_t scw, mnw;   // bytes 0,1: 6-bit scale / min of sub-blocks 2c, 2c+1
  if (c < 2) {
    scw = (meta.y & 0x3F3F3F3Fu) >> (16 * c);
    mnw = (meta.z & 0x3F3F3F3Fu) >> (16 * c);
  } else {
    scw = ((meta.w & 0x0F0F0F0Fu) | ((meta.y >> 2) & 0x30303030u)) >> (16 * (c - 2));
    mnw = (((meta.w >> 4) & 0x0F0F0F0Fu) | ((meta.z >> 2) & 0x30303030u)) >> (16 * (c - 2));
  }
  const __nv_bfloat162 s_lo = __float2bfloat162_rn(dd.x * (float)(scw & 0xFFu));
  const __nv_bfloat162 s_hi = __float2bfloat162_rn(dd.x * (float)((scw >> 8) & 0xFFu));
  const __nv_bfloat162 m_lo = __float2bfloat162_rn(-dd.y * (float)(mnw & 0xFFu));
  const __nv_bfloat162 m_hi = __float2bfloat162_rn(-dd.y * (float)((mnw >> 8) & 0xFFu));
  const __nv_bfloat162 k128 = bf162_bits(0x43004300u);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint4 qv = *reinterpret_cast<const uint4*>(blk + 16 + 32 * c + 16 * half);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
    uint32_t lo[8], hi[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      bytes4_to_bf16(w[i] & 0x0F0F0F0Fu, k128, s_lo, m_lo, lo[2 * i], lo[2 * i + 1]);
      bytes4_to_bf16((w[i] >> 4) & 0x0F0F0F0Fu, k128, s_hi, m_hi, hi[2 * i], hi[2 * i + 1]);
    }
    st_b_chunk(bstage, ut, 2 * half, make_uint4(lo[0], lo[1], lo[2], lo[3]));
    st_b_chunk(bstage, ut, 2 * half + 1, make_uint4(lo[4], lo[5], lo[6], lo[7]));
    st_b_chunk(bstage, ut, 4 + 2 * half, make_uint4(hi[0], hi[1], hi[2], hi[3]));
    st_b_chunk(bstage, ut, 4 + 2 * half + 1, make_uint4(hi[4], hi[5], hi[6], hi[7]));
  }
}

// Q6_K: the q-stage holds half `h` of each row's block as three dense regions: ql [BN][64], qh [BN][32],
// tail [BN][32] (16 int8 scales, d).  k-block cb (0 / 1) of the half takes the low / high nibbles of the 64 ql bytes
// and bit pairs 4cb.. of qh.  A task is (row, 16 ql bytes) = 16 consecutive columns; 4 tasks per thread.
__device__ __forceinline__ void unpack_q6k(const uint8_t* qst, uint8_t* bstage, int ut, int cb, int h) {
  const __nv_bfloat162 k160 = bf162_bits(0x43204320u);   // 128 + 32: the stored value is q + 32
  const __nv_bfloat162 zero = bf162_bits(0u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = ut + 256 * i, row = id >> 2, j = id & 3;
    const uint4 la = *reinterpret_cast<const uint4*>(qst + (size_t)row * 64 + j * 16);
    const uint4 hq = *reinterpret_cast<const uint4*>(qst + BN * 64 + (size_t)row * 32 + (j & 1) * 16);
    const uint8_t* tail = qst + BN * 96 + (size_t)row * 32;
    const int qt = 2 * cb + (j >> 1);
    const float d = __half2float(*reinterpret_cast<const __half*>(tail + 16));
    const float sc = (float)reinterpret_cast<const int8_t*>(tail)[h * 8 + 2 * qt + (j & 1)];
    const __nv_bfloat162 s = __float2bfloat162_rn(d * sc);
    const uint32_t lw[4] = {la.x, la.y, la.z, la.w}, hw[4] = {hq.x, hq.y, hq.z, hq.w};
    uint32_t o[8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint32_t nib = (cb ? (lw[u] >> 4) : lw[u]) & 0x0F0F0F0Fu;
      const uint32_t q4 = nib | (((hw[u] >> (2 * qt)) & 0x03030303u) << 4);
      bytes4_to_bf16(q4, k160, s, zero, o[2 * u], o[2 * u + 1]);
    }
    st_b_chunk(bstage, row, 2 * j, make_uint4(o[0], o[1], o[2], o[3]));
    st_b_chunk(bstage, row, 2 * j + 1, make_uint4(o[4], o[5], o[6], o[7]));
  }
}

// Q8_0: the q-stage holds 128 int8 columns per row ([BN][128]) and the 16-byte group of eight fp16 scales of the
// 256-aligned column range ([BN][16]); `par` = which half of that range this q-stage is.  A task is (row, 16 int8).
__device__ __forceinline__ void unpack_q80(const uint8_t* qst, uint8_t* bstage, int ut, int cb, int par) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int id = ut + 256 * i, row = id >> 2, j = id & 3;
    const uint4 qv = *reinterpret_cast<const uint4*>(qst + (size_t)row * 128 + cb * 64 + j * 16);
    const float d =
        __half2float(reinterpret_cast<const __half*>(qst + BN * 128 + (size_t)row * 16)[par * 4 + cb * 2 + (j >> 1)]);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
    uint32_t o[8];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float f0 = d * (float)(int8_t)(w[u] & 0xFFu), f1 = d * (float)(int8_t)((w[u] >> 8) & 0xFFu);
      const float f2 = d * (float)(int8_t)((w[u] >> 16) & 0xFFu), f3 = d * (float)(int8_t)(w[u] >> 24);
      o[2 * u] = bits_bf162(__floats2bfloat162_rn(f0, f1));
      o[2 * u + 1] = bits_bf162(__floats2bfloat162_rn(f2, f3));
    }
    st_b_chunk(bstage, row, 2 * j, make_uint4(o[0], o[1], o[2], o[3]));
    st_b_chunk(bstage, row, 2 * j + 1, make_uint4(o[4], o[5], o[6], o[7]));
  }
}

__device__ __forceinline__ int q_kb_per_stage(int qtype) { return qtype == HE_Q4_K ? 4 : 2; }

template <bool FUSE, bool QM>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmQ1,
                                          const CUtensorMap& tmQ2, const GemmArgs& g, const FuseArgs* f) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int NST = QM ? STAGES_Q : STAGES;
  uint8_t* qring = smem + NST * STAGE_BYTES;                     // QM only: QSTAGES x Q_STAGE_BYTES
  Barriers* bar = reinterpret_cast<Barriers*>(smem + NST * STAGE_BYTES + (QM ? QSTAGES * Q_STAGE_BYTES : 0));
  volatile int* abort_flag = &bar->abort_flag;
  constexpr int WARP_Q = FUSE ? 10 : 6;                          // QM: raw-block producer warp, then the unpack warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + BM - 1) / BM, tiles_n = (g.N + BN - 1) / BN;
  const int ksp = g.k_splits > 1 ? g.k_splits : 1;
  const int n_tiles = (FUSE && !(f->phases & 1)) ? 0 : tiles_m * tiles_n * ksp;
  const int k_blocks_all = (g.K + BK - 1) / BK;
  // k-blocks per split (the last split may get fewer); in QM the launcher makes it a multiple of 4, so that every
  // split starts on a 256-column boundary (whole q-stages)
  const int kb_per = g.kb_per > 0 ? g.kb_per : (k_blocks_all + ksp - 1) / ksp;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&bar->full[s], 1);
      mbar_init(&bar->empty[s], 1);
      mbar_init(&bar->bfull[s], N_UNPACK_WARPS);
    }
    for (int s = 0; s < QSTAGES; ++s) {
      mbar_init(&bar->qfull[s], 1);
      mbar_init(&bar->qempty[s], N_UNPACK_WARPS);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar->acc_full[a], 1);
      mbar_init(&bar->acc_empty[a], 4);   // one arrive per epilogue warp
    }
    bar->abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bar->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bar->tmem_base;
  uint32_t fuse_epoch = 0;
  if constexpr (FUSE) fuse_epoch = *reinterpret_cast<volatile uint32_t*>(f->sync) + 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (A, and B when it is bf16)
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      if constexpr (!QM) tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int ks = tile % ksp, mn = tile / ksp;
        const int tm = mn % tiles_m, tn = mn / tiles_m;
        int b_row0 = tn * BN;
        if (g.tile_group != nullptr) {
          const int grp = __ldg(g.tile_group + tm);
          if (grp < 0) continue;
          b_row0 += grp * g.N;
        }
        const int kb0 = ks * kb_per, kb1 = min(k_blocks_all, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % NST;
          const uint32_t ph = (it / NST) & 1;
          if (!mbar_wait(&bar->empty[s], ph ^ 1, abort_flag, g.status, 101)) break;
          mbar_expect_tx(&bar->full[s], QM ? A_BYTES : STAGE_BYTES);
          uint8_t* sa = smem + s * STAGE_BYTES;
          tma_load_2d(sa, &tmA, &bar->full[s], kb * BK, tm * BM);
          if constexpr (!QM) tma_load_2d(sa + A_BYTES, &tmB, &bar->full[s], kb * BK, b_row0);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        if (g.tile_group != nullptr && __ldg(g.tile_group + (tile / ksp) % tiles_m) < 0) continue;
        const int kb0 = (tile % ksp) * kb_per, kb1 = min(k_blocks_all, kb0 + kb_per);
        const int k_blocks = kb1 - kb0;
        const int acc = tcount & 1;
        const uint32_t acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&bar->acc_empty[acc], acc_ph ^ 1, abort_flag, g.status, 102)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % NST;
          const uint32_t ph = (it / NST) & 1;
          if (!mbar_wait(&bar->full[s], ph, abort_flag, g.status, 103)) break;
          if constexpr (QM) {
            if (!mbar_wait(&bar->bfull[s], ph, abort_flag, g.status, 105)) break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            const uint64_t da = umma_desc_k_sw128(a_addr + k * UK * 2);
            const uint64_t db = umma_desc_k_sw128(b_addr + k * UK * 2);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bar->empty[s]);   // frees the smem stage once these MMAs have read it
        }
        if (*abort_flag) break;
        umma_commit(&bar->acc_full[acc]);
        ++tcount;
      }
    }
  } else if (QM && warp == WARP_Q) {
    // ------------------------------------------------------------ raw-block producer (QM)
    if (elect_one()) {
      tma_prefetch_desc(&tmB);
      const int kbq = q_kb_per_stage(g.qtype);
      uint32_t qit = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int ks = tile % ksp, mn = tile / ksp;
        const int tm = mn % tiles_m, tn = mn / tiles_m;
        int b_row0 = tn * BN;
        if (g.tile_group != nullptr) {
          const int grp = __ldg(g.tile_group + tm);
          if (grp < 0) continue;
          b_row0 += grp * g.N;
        }
        const int kb0 = ks * kb_per, kb1 = min(k_blocks_all, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; kb += kbq, ++qit) {
          const int qs = qit % QSTAGES;
          const uint32_t ph = (qit / QSTAGES) & 1;
          if (!mbar_wait(&bar->qempty[qs], ph ^ 1, abort_flag, g.status, 106)) break;
          uint8_t* dst = qring + qs * Q_STAGE_BYTES;
          uint64_t* fb = &bar->qfull[qs];
          const int qi = kb / kbq;                      // q-stage index along K
          if (g.qtype == HE_Q4_K) {
            mbar_expect_tx(fb, BN * 144);
            tma_load_2d(dst, &tmB, fb, qi * 144, b_row0);
          } else if (g.qtype == HE_Q6_K) {
            const int sb = qi >> 1, h = qi & 1;
            mbar_expect_tx(fb, BN * 128);
            tma_load_2d(dst, &tmB, fb, sb * 224 + 64 * h, b_row0);
            tma_load_2d(dst + BN * 64, &tmQ1, fb, sb * 224 + 128 + 32 * h, b_row0);
            tma_load_2d(dst + BN * 96, &tmQ2, fb, sb * 224 + 192, b_row0);
          } else {
            mbar_expect_tx(fb, BN * 144);
            tma_load_2d(dst, &tmB, fb, qi * 128, b_row0);
            tma_load_2d(dst + BN * 128, &tmQ1, fb, g.K + 16 * (qi >> 1), b_row0);
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (QM && warp > WARP_Q) {
    // ------------------------------------------------------------ unpack warps (QM): raw blocks -> bf16 operand stage
    const int ut = (int)threadIdx.x - (WARP_Q + 1) * 32;
    const int kbq = q_kb_per_stage(g.qtype);
    uint32_t it = 0, qit = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      if (g.tile_group != nullptr && __ldg(g.tile_group + (tile / ksp) % tiles_m) < 0) continue;
      const int kb0 = (tile % ksp) * kb_per, kb1 = min(k_blocks_all, kb0 + kb_per);
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; kb += kbq, ++qit) {
        const int qs = qit % QSTAGES;
        if (!mbar_wait(&bar->qfull[qs], (qit / QSTAGES) & 1, abort_flag, g.status, 107)) { ok = false; break; }
        const uint8_t* qst = qring + qs * Q_STAGE_BYTES;
        const int qi = kb / kbq;
        for (int c = 0; c < kbq; ++c, ++it) {
          const int s = it % NST;
          if (!mbar_wait(&bar->empty[s], ((it / NST) & 1) ^ 1, abort_flag, g.status, 108)) { ok = false; break; }
          uint8_t* bstage = smem + s * STAGE_BYTES + A_BYTES;
          if (g.qtype == HE_Q4_K) unpack_q4k(qst, bstage, ut, c);
          else if (g.qtype == HE_Q6_K) unpack_q6k(qst, bstage, ut, c, qi & 1);
          else unpack_q80(qst, bstage, ut, c, qi & 1);
          fence_proxy_async_smem();      // the tensor core reads the stage through the async proxy
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar->bfull[s]);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar->qempty[qs]);
      }
      if (!ok || *abort_flag) break;
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;              // TMEM lane quarter this warp may touch
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const int mn = tile / ksp;
      const int tm = mn % tiles_m, tn = mn / tiles_m;
      if (g.tile_group != nullptr && __ldg(g.tile_group + tm) < 0) continue;
      const int ks_e = tile % ksp;
      const bool empty_split = ks_e * kb_per >= k_blocks_all;
      const int acc = tcount & 1;
      const uint32_t acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait(&bar->acc_full[acc], acc_ph, abort_flag, g.status, 104)) break;
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if constexpr (FUSE) {
          // partial quarter -> the owner's stage slot; rows and columns past M / N are zeros (zero-filled operand
          // tiles), so the whole tile is stored and no bound is needed
          uint4 pk[4];
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk[v]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]),
                                                        __uint_as_float(r[v * 8 + 2 * e + 1]));
              pw[e] = *reinterpret_cast<uint32_t*>(&h2);
            }
          }
          // fragment-major tile layout: 16-byte group (quarter q, column group cg = 4c + v, row lane) sits at
          // q * 8192 + (cg * 32 + lane) * 8, so every store instruction of the warp covers 512 contiguous bytes
          // (full lines on the link) instead of 32 pieces 512 bytes apart
          const size_t in_tile = (size_t)q * 8192 + ((size_t)(c * 4) * 32 + lane) * 8;
          if (f->direct) {
            const size_t off = (((size_t)(fuse_epoch & 1u) * f->world + f->rank) * f->owned_cap + mn) * TILE_ELEMS +
                               in_tile;
            for (int pr = 0; pr < f->world; ++pr) {
              __nv_bfloat16* dst = f->stage[pr] + off;
#pragma unroll
              for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(dst + v * 256) = pk[v];
            }
          } else {
            const int owner = mn % f->world, oi = mn / f->world;
            __nv_bfloat16* dst = f->stage[owner] + ((size_t)f->rank * f->owned_cap + oi) * TILE_ELEMS + in_tile;
#pragma unroll
            for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(dst + v * 256) = pk[v];
          }
        } else
        if (row < g.M && col0 < g.N) {
          const int ncols = min(32, g.N - col0);
          if (g.epi == 0) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + (size_t)row * g.ldc + col0;
            if (ncols == 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 pk;
                uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]),
                                                           __uint_as_float(r[v * 8 + 2 * e + 1]));
                  pw[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + v * 8) = pk;
              }
            } else {
              for (int e = 0; e < ncols; ++e) dst[e] = __float2bfloat16_rn(__uint_as_float(r[e]));
            }
          } else {
            float* dst = reinterpret_cast<float*>(g.C) + (size_t)row * g.ldc + col0 +
                         (g.epi == 4 ? (size_t)ks_e * (size_t)g.split_stride : (size_t)0);
            const bool vec = ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
            if ((g.epi == 1 || g.epi == 4) && vec) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                reinterpret_cast<float4*>(dst)[v] =
                    make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                __uint_as_float(r[4 * v + 3]));
            } else if (g.epi == 2 && vec) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = reinterpret_cast<float4*>(dst)[v];
                o.x += __uint_as_float(r[4 * v]); o.y += __uint_as_float(r[4 * v + 1]);
                o.z += __uint_as_float(r[4 * v + 2]); o.w += __uint_as_float(r[4 * v + 3]);
                reinterpret_cast<float4*>(dst)[v] = o;
              }
            } else if (g.epi == 1 || g.epi == 4) {
              for (int e = 0; e < ncols; ++e) dst[e] = __uint_as_float(r[e]);
            } else if (g.epi == 2) {
              for (int e = 0; e < ncols; ++e) dst[e] += __uint_as_float(r[e]);
            } else if (!empty_split) {
              for (int e = 0; e < ncols; ++e) atomicAdd(dst + e, __uint_as_float(r[e]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->acc_empty[acc]);
      if constexpr (FUSE) {
        __threadfence_system();
        __syncwarp();
        if (f->direct) {
          if (lane < f->world)
            st_release_sys_u32(f->flags[lane] + ((size_t)mn * f->world + f->rank) * 4 + q, fuse_epoch);
        } else if (lane == 0) {
          st_release_sys_u32(f->flags[mn % f->world] + ((size_t)mn * f->world + f->rank) * 4 + q, fuse_epoch);
        }
      }
      ++tcount;
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------ collective warps 6..9 (fused kernel only)
    // Warp 6+q reduces quarter q of the tiles this rank owns (phase 2) and adds quarter q of this CTA's share of
    // all tiles into the residual (phase 3) while the other warps keep the tensor cores busy.  It takes whichever
    // unit has its stamps, and gives up after wait_limit polls without progress.
    if constexpr (FUSE) {
      const int q = warp - 6;
      const int tiles_mn = tiles_m * tiles_n;
      const int W = f->world;
      int p2_next = ((f->phases & 2) && !f->direct) ? f->rank + (int)blockIdx.x * W : tiles_mn;
      int p3_next = (f->phases & 4) ? (int)blockIdx.x : tiles_mn;
      uint32_t* my_flags = f->flags[f->rank];
      const size_t done_off = (size_t)f->max_tiles * W * 4;
      unsigned stall = 0;
      while (p2_next < tiles_mn || p3_next < tiles_mn) {
        if (p2_next < tiles_mn && warp_stamps_ready(my_flags + (size_t)p2_next * W * 4 + q, W, 4, fuse_epoch)) {
          fuse_reduce_quarter(f, p2_next, q, fuse_epoch);
          p2_next += gridDim.x * W;
          stall = 0;
        } else if (p3_next < tiles_mn && f->direct &&
                   warp_stamps_ready(my_flags + (size_t)p3_next * W * 4 + q, W, 4, fuse_epoch)) {
          fuse_direct_quarter(f, p3_next, q, tiles_m, g.M, g.N, fuse_epoch);
          p3_next += gridDim.x;
          stall = 0;
        } else if (p3_next < tiles_mn && !f->direct &&
                   warp_stamps_ready(my_flags + done_off + (size_t)p3_next * 4 + q, 1, 1, fuse_epoch)) {
          fuse_add_quarter(f, p3_next, q, tiles_m, g.M, g.N);
          p3_next += gridDim.x;
          stall = 0;
        } else {
          if (++stall > f->wait_limit || *abort_flag) {
            if (lane == 0 && g.status != nullptr) atomicCAS(g.status, 0, HE_ERR_WAIT_TIMEOUT);
            break;
          }
          __nanosleep(128);
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if constexpr (FUSE) {
    // the last CTA to leave a launch that ran the final phase publishes the new epoch for the next launch
    if (threadIdx.x == 0 && (f->phases & 4)) {
      __threadfence();
      const unsigned prev = atomicAdd(f->sync + 1, 1u);
      if (prev == gridDim.x - 1) {
        f->sync[1] = 0;
        f->sync[0] = fuse_epoch;
        __threadfence();
      }
    }
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs g) {
  gemm_body<false, false>(tmA, tmB, tmB, tmB, g, nullptr);
}

__global__ void __launch_bounds__(NTHREADS_FUSED, 1)
gemm_bf16_allreduce_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const GemmArgs g, const __grid_constant__ FuseArgs f) {
  gemm_body<true, false>(tmA, tmB, tmB, tmB, g, &f);
}

// The fused pipeline with the weight read in its quantised device layout (tmQ0..2: byte-typed maps over the rows;
// the stand-alone quantised GEMM lives in gemm_wq_sm100.cu).
__global__ void __launch_bounds__(NTHREADS_FUSED_Q, 1)
gemm_q_allreduce_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ0,
                        const __grid_constant__ CUtensorMap tmQ1, const __grid_constant__ CUtensorMap tmQ2,
                        const GemmArgs g, const __grid_constant__ FuseArgs f) {
  gemm_body<true, true>(tmA, tmQ0, tmQ1, tmQ2, g, &f);
}

// ---------------------------------------------------------------- host side: tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 row-major [rows][cols] with row stride `ld` elements; box = {BK cols, box_rows rows}; 128B swizzle.
int make_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -HE_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * 2) % 16 != 0) return -HE_ERR_BAD_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

// Byte-typed 2-D map over quantised weight rows: [rows][row_bytes] uint8, box = {box_bytes, BN rows}, no swizzle.
int make_byte_map(CUtensorMap* m, const void* ptr, long long rows, long long row_bytes, int box_bytes) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -HE_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || row_bytes % 16 != 0 || box_bytes % 16 != 0) return -HE_ERR_BAD_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)BN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

struct QMaps {
  CUtensorMap m[3];
};

// Maps for the raw-block boxes of each type (see the q-stage table at the top of the file).
int make_qmaps(QMaps* q, const void* B, int qtype, long long rows, int K) {
  if (K % 256 != 0) return -HE_ERR_BAD_ARG;
  int rc;
  if (qtype == HE_Q4_K) {
    const long long rb = (long long)(K >> 8) * 144;
    rc = make_byte_map(&q->m[0], B, rows, rb, 144);
    q->m[1] = q->m[0];
    q->m[2] = q->m[0];
    return rc;
  }
  if (qtype == HE_Q6_K) {
    const long long rb = (long long)(K >> 8) * 224;
    if ((rc = make_byte_map(&q->m[0], B, rows, rb, 64)) != 0) return rc;
    if ((rc = make_byte_map(&q->m[1], B, rows, rb, 32)) != 0) return rc;
    q->m[2] = q->m[1];
    return 0;
  }
  if (qtype == HE_Q8_0) {
    const long long rb = (long long)K + (((K >> 4) + 15) / 16) * 16;
    if ((rc = make_byte_map(&q->m[0], B, rows, rb, 128)) != 0) return rc;
    if ((rc = make_byte_map(&q->m[1], B, rows, rb, 16)) != 0) return rc;
    q->m[2] = q->m[1];
    return 0;
  }
  return -HE_ERR_BAD_ARG;
}

constexpr size_t SMEM_Q = STAGES_Q * STAGE_BYTES + QSTAGES * Q_STAGE_BYTES + sizeof(Barriers) + 1024;

}  // namespace

// C[M][N] = A[M][K] (bf16, row stride lda) * B[N][K]^T (bf16, row stride ldb).
// epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate into C.  `status` (device int, may be null) receives a
// non-zero code if a bounded wait inside the kernel gave up.
HE_API int he_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc, int M,
                        int N, int K, int epi, void* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 != 0) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmB, B, N, K, ldb, BN);
  if (rc != 0) return rc;
  GemmArgs g = {};
  g.C = C; g.ldc = ldc; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = epi; g.status = (int*)status;
  g.tile_group = nullptr;
  g.k_splits = 1;
  g.split_stride = 0;
  g.qtype = 0;
  g.kb_per = 0;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
  // the attribute is per device: set it on every call (cheap) rather than once per process
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_bf16_kernel<<<grid, NTHREADS, smem, stream>>>(tmA, tmB, g);
  HE_LAUNCH_CHECK();
  return 0;
}

// resid[M][N] (fp32) += sum over ranks of A_rank[M][K] * B_rank[N][K]^T: the GEMM, the all-reduce over peer memory
// and the residual add in one kernel per rank (see FuseArgs).  Every rank of the group must issue the same sequence
// of calls with the same M and N.  `fuse` is a host copy of FuseArgs.
HE_API int he_gemm_fuse_args_size() { return (int)sizeof(FuseArgs); }
HE_API int he_gemm_fuse_tile_elems() { return TILE_ELEMS; }
HE_API int he_gemm_fuse_tiles(int M, int N) { return ((M + BM - 1) / BM) * ((N + BN - 1) / BN); }

HE_API int he_gemm_bf16_allreduce(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                                  const FuseArgs* fuse, void* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const FuseArgs& f = *fuse;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (K % 8 != 0 || N % 8 != 0) return -HE_ERR_BAD_ARG;
  if (f.world < 1 || f.world > FUSE_MAX_WORLD || f.rank < 0 || f.rank >= f.world) return -HE_ERR_BAD_ARG;
  if (tiles > f.max_tiles || (f.direct ? tiles : (tiles + f.world - 1) / f.world) > f.owned_cap)
    return -HE_ERR_BAD_ARG;
  if (f.resid == nullptr || (reinterpret_cast<uintptr_t>(f.resid) & 15) != 0 || f.ld_resid % 4 != 0 || f.ld_resid < N)
    return -HE_ERR_BAD_ARG;
  if ((f.phases & 7) == 0 || f.sync == nullptr) return -HE_ERR_BAD_ARG;
  for (int r = 0; r < f.world; ++r)
    if (f.stage[r] == nullptr || f.result[r] == nullptr || f.flags[r] == nullptr) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmB, B, N, K, ldb, BN);
  if (rc != 0) return rc;
  GemmArgs g = {};
  g.C = nullptr; g.ldc = 0; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = 5; g.status = (int*)status;
  g.tile_group = nullptr;
  g.k_splits = 1;
  g.split_stride = 0;
  g.qtype = 0;
  g.kb_per = 0;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  // every CTA must be resident at once (CTAs of one rank wait for tiles of CTAs on other ranks): one CTA per SM
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_bf16_allreduce_kernel<<<grid, NTHREADS_FUSED, smem, stream>>>(tmA, tmB, g, f);
  HE_LAUNCH_CHECK();
  return 0;
}

// Grouped GEMM for MoE experts: rows [tm*128, +128) of A use weight block B[tile_group[tm]*N .. +N) of the
// stacked matrix B[n_groups*N][K]; tile_group (device, ceil(M/128) ints) holds -1 for unused tiles, which are
// skipped.  C[M][N] rows follow A.  M is the padded upper bound of sorted rows.
HE_API int he_gemm_bf16_grouped(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                                int M, int N, int K, int n_groups, const int* tile_group, int epi, void* status,
                                int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || n_groups <= 0) return 0;
  if (K % 8 != 0 || tile_group == nullptr) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmB, B, (long long)n_groups * N, K, ldb, BN);
  if (rc != 0) return rc;
  GemmArgs g = {};
  g.C = C; g.ldc = ldc; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = epi; g.status = (int*)status;
  g.tile_group = tile_group;
  g.k_splits = 1;
  g.split_stride = 0;
  g.qtype = 0;
  g.kb_per = 0;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_bf16_kernel<<<grid, NTHREADS, smem, stream>>>(tmA, tmB, g);
  HE_LAUNCH_CHECK();
  return 0;
}

// C[M][N] (fp32) += A[M][K] * B[N][K]^T with the K range split over CTAs and atomic accumulation: for small M and
// few output tiles (decode batches of 9..128 rows against a 5120-wide output) this is what lets all SMs stream
// the weight instead of one CTA per 256 output columns.  C must already hold the value to add to (e.g. the
// residual stream).  k_splits <= 0 picks a split that gives about one tile per SM.
namespace {
// out[m][n] (+)= sum over splits, in split order (deterministic).  mode 0: fp32 store, 1: fp32 add in place.
__global__ void splitk_reduce_kernel(const float* __restrict__ part, long long split_stride, int k_splits,
                                     float* __restrict__ out, long long ldo, int M, int N, int mode) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= (long long)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  float4 s = *reinterpret_cast<const float4*>(part + (size_t)m * N + n);
  for (int k = 1; k < k_splits; ++k) {
    const float4 v = *reinterpret_cast<const float4*>(part + (size_t)k * split_stride + (size_t)m * N + n);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  float4* o = reinterpret_cast<float4*>(out + (size_t)m * ldo + n);
  if (mode == 1) {
    const float4 h = *o;
    s.x += h.x; s.y += h.y; s.z += h.z; s.w += h.w;
  }
  *o = s;
}
}  // namespace

// Deterministic split-K: partial tiles go to `partials` ([k_splits][M][N] fp32, caller scratch of at least
// he_gemm_splitk_scratch_floats(M, N, K) floats), then one pass sums them in split order into `out`
// (mode 0: store, 1: add in place -- the residual add).  Same use as he_gemm_bf16_splitk, bit-reproducible.
HE_API long long he_gemm_splitk_plan(int M, int N, int K, int num_sms) {
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int k_blocks = (K + BK - 1) / BK;
  int k_splits = (num_sms + tiles - 1) / tiles;
  if (k_splits > k_blocks) k_splits = k_blocks;
  if (k_splits < 1) k_splits = 1;
  const int kb_per = (k_blocks + k_splits - 1) / k_splits;
  return (k_blocks + kb_per - 1) / kb_per;
}

HE_API int he_gemm_bf16_splitk_det(const void* A, long long lda, const void* B, long long ldb, void* partials,
                                   void* out, long long ldo, int M, int N, int K, int mode, void* status,
                                   int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 != 0 || N % 4 != 0) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmB, B, N, K, ldb, BN);
  if (rc != 0) return rc;
  const int k_splits = (int)he_gemm_splitk_plan(M, N, K, num_sms);
  GemmArgs g = {};
  g.C = partials; g.ldc = N; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = 4; g.status = (int*)status;
  g.tile_group = nullptr;
  g.k_splits = k_splits;
  g.split_stride = (long long)M * N;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int total = tiles * k_splits;
  gemm_bf16_kernel<<<total < num_sms ? total : num_sms, NTHREADS, smem, stream>>>(tmA, tmB, g);
  HE_LAUNCH_CHECK();
  const long long n4 = ((long long)M * N + 3) / 4;
  splitk_reduce_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>((const float*)partials, g.split_stride,
                                                                        k_splits, (float*)out, ldo, M, N, mode);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_gemm_bf16_splitk(const void* A, long long lda, const void* B, long long ldb, void* C, long long ldc,
                               int M, int N, int K, int k_splits, void* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 8 != 0) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA, tmB;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmB, B, N, K, ldb, BN);
  if (rc != 0) return rc;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int k_blocks = (K + BK - 1) / BK;
  if (k_splits <= 0) k_splits = (num_sms + tiles - 1) / tiles;
  if (k_splits > k_blocks) k_splits = k_blocks;
  if (k_splits < 1) k_splits = 1;
  const int kb_per = (k_blocks + k_splits - 1) / k_splits;
  k_splits = (k_blocks + kb_per - 1) / kb_per;            // no empty split
  GemmArgs g = {};
  g.C = C; g.ldc = ldc; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = 3; g.status = (int*)status;
  g.tile_group = nullptr;
  g.k_splits = k_splits;
  g.split_stride = 0;
  const size_t smem = STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int total = tiles * k_splits;
  const int grid = total < num_sms ? total : num_sms;
  gemm_bf16_kernel<<<grid, NTHREADS, smem, stream>>>(tmA, tmB, g);
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------- quantised-weight entry points
// The fused GEMM -> all-reduce -> residual add of he_gemm_bf16_allreduce with a quantised weight.
HE_API int he_gemm_q_allreduce(const void* A, long long lda, const void* B, int qtype, long long b_rows, int M, int N,
                               int K, const FuseArgs* fuse, void* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const FuseArgs& f = *fuse;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (N % 8 != 0) return -HE_ERR_BAD_ARG;
  if (f.world < 1 || f.world > FUSE_MAX_WORLD || f.rank < 0 || f.rank >= f.world) return -HE_ERR_BAD_ARG;
  if (tiles > f.max_tiles || (f.direct ? tiles : (tiles + f.world - 1) / f.world) > f.owned_cap)
    return -HE_ERR_BAD_ARG;
  if (f.resid == nullptr || (reinterpret_cast<uintptr_t>(f.resid) & 15) != 0 || f.ld_resid % 4 != 0 || f.ld_resid < N)
    return -HE_ERR_BAD_ARG;
  if ((f.phases & 7) == 0 || f.sync == nullptr) return -HE_ERR_BAD_ARG;
  for (int r = 0; r < f.world; ++r)
    if (f.stage[r] == nullptr || f.result[r] == nullptr || f.flags[r] == nullptr) return -HE_ERR_BAD_ARG;
  CUtensorMap tmA;
  QMaps q;
  int rc = make_map(&tmA, A, M, K, lda, BM);
  if (rc != 0) return rc;
  rc = make_qmaps(&q, B, qtype, b_rows, K);
  if (rc != 0) return rc;
  GemmArgs g = {};
  g.C = nullptr; g.ldc = 0; g.resid = nullptr; g.M = M; g.N = N; g.K = K; g.epi = 5; g.status = (int*)status;
  g.tile_group = nullptr;
  g.k_splits = 1;
  g.split_stride = 0;
  g.qtype = qtype;
  g.kb_per = 0;
  cudaError_t e = cudaFuncSetAttribute(gemm_q_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)SMEM_Q);
  if (e != cudaSuccess) return (int)e;
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_q_allreduce_kernel<<<grid, NTHREADS_FUSED_Q, SMEM_Q, stream>>>(tmA, q.m[0], q.m[1], q.m[2], g, f);
  HE_LAUNCH_CHECK();
  return 0;
}
