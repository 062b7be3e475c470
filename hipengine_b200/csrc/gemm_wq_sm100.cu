// Tensor-core GEMM over a QUANTISED weight for sm_100a: C[M][N] = X[M][K] * W[N][K]^T with W kept in its
// GGUF-derived device layout (Q4_K 144-byte blocks, Q6_K 224-byte blocks, Q8_0 int8 + scale planes).
//
// The product is computed transposed, D^T[128 weight rows][mt activation rows], so that the WEIGHT is the MMA's
// A operand -- and tcgen05.mma can take A from tensor memory.  Raw block bytes arrive in shared memory by
// byte-typed TMA boxes; sixteen unpack warps turn each 64-column slice of a weight row into 32 packed bf16x2
// registers and store them with tcgen05.st straight into a TMEM operand stage (row = TMEM lane).  The expanded
// weight therefore never exists in shared or global memory: DRAM and L2 see 4.5 / 6.6 / 8.5 bits per weight, and
// shared-memory bandwidth is left to the activation tiles.  Roles (24 warps):
//   warp 0      : TMA producer of activation tiles X[mt][64] (128-byte swizzle, 5-stage ring)
//   warp 1      : MMA issuer (tcgen05.mma 128 x mt x 16, A from TMEM, B from smem); owns the TMEM allocation
//   warp 2      : TMA producer of raw weight blocks (one 256-column super-block of 128 rows per q-stage, 3 stages)
//   warps 4..7  : epilogue (tcgen05.ld, transposed store: lane = weight row n, register = activation row m, so a
//                 store instruction of a warp covers 32 consecutive n of one output row)
//   warps 8..23 : unpack, four sets of four warps; set g expands k-block g of every super-block into TMEM
//                 operand stage g (thread = weight row), so four k-blocks are in flight
// TMEM (512 columns): two accumulators of 192 fp32 columns (epilogue of tile i overlaps the main loop of
// tile i+1) + four operand stages of 32 columns.
// Counterparts in the reference: hipengine/kernels/hip_gfx1100/quant/gguf_q4_k_prefill.hip:170-296 (raw 144-byte
// blocks read inside the matrix-core loop), gguf_q8_0_prefill.hip, and the grouped expert form
// quant/gguf_q4_k_selected_prefill.hip.
#include <cstdlib>
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int WN = 128;                  // weight rows per tile (the MMA's M)
constexpr int MT_MAX = 192;              // activation rows per tile (the MMA's N), multiple of 16
constexpr int BK = 64, UK = 16;
constexpr int XSTAGES = 5;                          // activation ring depth (stage = mt x 64 bf16, <= 24 KB); seven
                                                    // stages (with three raw-block stages) measured slower in pair mode
constexpr int QSTAGES_MAX = 12;                     // raw-block ring: as many stages as shared memory holds, up to 12
constexpr int SMEM_BUDGET = 224 * 1024;             // dynamic shared memory the rings may use
constexpr int N_SETS = 4;                           // unpack sets == TMEM operand stages == k-blocks per q-stage
constexpr int N_UNPACK_WARPS = 16;
constexpr int WARP_UNPACK0 = 8;
constexpr int NTHREADS_WQ = (WARP_UNPACK0 + N_UNPACK_WARPS) * 32;   // 768
constexpr int TMEM_COLS = 512;
constexpr int D_COLS = MT_MAX;                      // column stride between the two accumulators (tiles > 64 rows)
constexpr int D_COLS_SMALL = 64;                    // ... for tiles of <= 64 activation rows
constexpr int A_STAGE_COLS = 32;                    // 64 bf16 per lane
constexpr int A_DEPTH_MAX = 3;                      // operand stages per unpack set (small tiles); 1 for large tiles
constexpr int A_STAGES_MAX = N_SETS * A_DEPTH_MAX;  // 12 x 32 columns + 2 x 64 = 512
constexpr int X_KB_WIDE = 4;                        // k-blocks per activation stage when the tile is small

struct WqArgs {
  void* C;
  long long ldc;            // elements
  int M, N, K;
  int epi;                  // 0: bf16 store, 1: fp32 store, 2: fp32 +=, 4: fp32 split-K partial store
  int qtype;                // HE_Q4_K / HE_Q6_K / HE_Q8_0
  int mt;                   // activation rows per tile: multiple of 16, <= MT_MAX (128 in grouped mode)
  int k_splits;             // >= 1
  int sb_per;               // super-blocks (256 columns) per split
  long long split_stride;   // epi 4: split ks stores at C + ks * split_stride
  int pair;                 // 1: a work unit is one weight tile against two neighbouring M-tiles (see TileCoord)
  const int* tile_group;    // grouped mode: M-tile tm uses weight rows [tile_group[tm] * N, +N); < 0 skips the tile
  int* status;
  long long* dbg;           // optional cycle counters of CTA 0 (he_gemm_q_debug_counters), null in normal use
  // ring geometry, set by the launcher: few activation rows leave room for a deep raw-block ring, which is what
  // hides DRAM latency when the weight is streamed once (decode batches)
  int x_stage_bytes;        // x_kb * mt * 128 rounded up to 1 KB
  int x_kb;                 // 64-column k-blocks per activation stage: 4 (a whole super-block) for tiles of <= 48
                            // rows, else 1.  With few rows an MMA batch lasts tens of cycles, so a ring of single
                            // k-blocks would be bound by the round trip of its own barriers, not by bandwidth
  int a_depth;              // operand stages per unpack set: 3 for tiles of <= 64 rows (the accumulators need only
                            // 2 x 64 TMEM columns then), else 1; a set expands super-block i + 1 .. i + depth - 1
                            // while the MMAs of super-block i are still in flight
  int q_stage_bytes;        // 128 rows x bytes per super-block row, rounded up to 1 KB
  int q_stages;
  // all-gather -> GEMM (sequence-parallel activations): the rows of M-tile tm were written into the local activation
  // buffer by rank tm % ag_world (peer stores of its norm kernel, then a stamp in ag_flags[that rank]); the activation
  // producer waits -- bounded -- for the stamp of a tile's owner before the first load of the tile, so the GEMM
  // starts on the rows that are already here while the others are still crossing the links.  ag_world 0: off.
  const uint32_t* ag_flags;   // local [ag_world]
  const uint32_t* ag_epoch;   // local: the stamp value this call waits for
  int ag_world;
  unsigned ag_wait_limit;
};

// GEMM -> reduce-scatter -> residual add (sequence-parallel residual): M-tile tm belongs to rank tm % world.
// Every rank owns one symmetric region, mapped into all peers:
//     stage  [world src][slots][128 x MT_MAX] bf16 : partial tiles pushed by rank `src` for the tiles this rank owns
//                                                    (slot = (tm / world) * tiles_n + tn)
//     flags  [slots][world][4] u32                 : epoch stamps per (tile, source rank, 32-row quarter)
// Phase 1 (epilogue warps): the partial quarter goes straight into the owner's stage slot as bf16 (peer stores for
// remote owners, fragment-major so a warp's store instruction covers 512 contiguous bytes), then a system fence and
// the stamp.  Phase 2 (two collective warps per CTA, beside the pipeline for the whole kernel): for each owned
// (tile, quarter) wait -- bounded -- for the world stamps, sum the slots in rank order in fp32 and add into the local
// fp32 residual rows: bf16 on the wire, fp32 accumulation, no rounding of the sum.  The epoch lives in device memory
// and is advanced by the last CTA to leave, so the kernel replays from CUDA graphs.  `phases` (bit 0 / 1) selects
// the phases a launch runs: 3 in production; a single-GPU test runs the phases of several emulated ranks as
// separate launches (all phase 1, then all phase 2) so that no launch waits for a later one.
constexpr int RS_MAX_WORLD = 8;
constexpr int RS_TILE_ELEMS = WN * MT_MAX;
struct WqFuse {
  __nv_bfloat16* stage[RS_MAX_WORLD];
  uint32_t* flags[RS_MAX_WORLD];
  uint32_t* sync;           // local [2]: epoch of the last finished call, CTAs that have left the current call
  float* resid;             // local fp32 [M][ld_resid]; only rows of owned tiles are touched
  long long ld_resid;
  int world, rank, slots, phases;
  unsigned wait_limit;
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

struct __align__(8) WqBarriers {
  uint64_t x_full[XSTAGES];
  uint64_t x_empty[XSTAGES];
  uint64_t q_full[QSTAGES_MAX];
  uint64_t q_empty[QSTAGES_MAX];
  uint64_t a_full[A_STAGES_MAX];
  uint64_t a_empty[A_STAGES_MAX];
  uint64_t d_full[2];
  uint64_t d_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// ---------------------------------------------------------------- register-level dequantisation
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t bits_bf162(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Packed fp32 pair helpers: sm_100 issues two fp32 FMAs as one instruction on a 64-bit register pair.
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
// Role cycle counters (he_gemm_q_debug_counters) exist only in builds with -DHE_WQ_PROFILE=1: the product build
// folds every `prof` flag to false, so the hot loops carry no extra registers or branches.
#ifdef HE_WQ_PROFILE
#define HE_WQ_PROF_ON true
#else
#define HE_WQ_PROF_ON false
#endif

#ifndef HE_WQ_SCALAR_FMA
#define HE_WQ_SCALAR_FMA 0
#endif
__device__ __forceinline__ uint32_t fma2_to_bf162(__half2 v, uint64_t s2, uint64_t c2) {
  const float2 f = __half22float2(v);
#if HE_WQ_SCALAR_FMA
  float s, c, unused;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(s), "=f"(unused) : "l"(s2));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(c), "=f"(unused) : "l"(c2));
  return bits_bf162(__floats2bfloat162_rn(fmaf(f.x, s, c), fmaf(f.y, s, c)));
#else
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack_f2(f.x, f.y)), "l"(s2), "l"(c2));
  float d0, d1;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
  return bits_bf162(__floats2bfloat162_rn(d0, d1));
#endif
}

// Four unsigned bytes v of `b4` become two bf16x2 registers holding bf16(v * s + off) with a single rounding.  A byte
// under the high byte 0x64 is the fp16 number 1024 + v exactly, so ONE byte permute makes two operands; the
// half -> float conversions and the FMAs run on the FMA pipe, which leaves the integer pipe (the busier one here) with
// one instruction per pair and one packing conversion per pair:
//     (1024 + v) * s + (off - 1024 s) = v * s + off.
// `s2` = (s, s) and `c2` = (off - 1024 s) twice are per sub-block constants.  The sum is exact in fp32 up to the
// rounding of the constant (2^-14 s), so the result is the reference dequantisation (fp32) rounded once to bf16.
__device__ __forceinline__ void bytes4_to_bf16(uint32_t b4, uint64_t s2, uint64_t c2, uint32_t& o01, uint32_t& o23) {
  const uint32_t MAGIC = 0x64646464u;
  const uint32_t p0 = prmt_b32(b4, MAGIC, 0x5140u), p1 = prmt_b32(b4, MAGIC, 0x7362u);
  o01 = fma2_to_bf162(*reinterpret_cast<const __half2*>(&p0), s2, c2);
  o23 = fma2_to_bf162(*reinterpret_cast<const __half2*>(&p1), s2, c2);
}
__device__ __forceinline__ uint64_t dup_f2(float v) { return pack_f2(v, v); }

// Q4_K, k-block c (0..3) of the super-block at `blk` (144 bytes): the 32 nibble bytes [16 + 32c, +32); low
// nibbles are columns 0..31 (sub-block 2c), high nibbles columns 32..63 (sub-block 2c+1).  r[j] = columns 2j, 2j+1.
__device__ __forceinline__ void unpack_q4k(const uint8_t* blk, int c, uint32_t (&r)[32]) {
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
  // high nibbles are used in place (byte = 16 q): their scale is s / 16, exact
  const float s_lo = dd.x * (float)(scw & 0xFFu), s_hi = 0.0625f * dd.x * (float)((scw >> 8) & 0xFFu);
  const uint64_t s2_lo = dup_f2(s_lo), s2_hi = dup_f2(s_hi);
  const uint64_t c2_lo = dup_f2(-dd.y * (float)(mnw & 0xFFu) - 1024.f * s_lo);
  const uint64_t c2_hi = dup_f2(-dd.y * (float)((mnw >> 8) & 0xFFu) - 1024.f * s_hi);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint4 qv = *reinterpret_cast<const uint4*>(blk + 16 + 32 * c + 16 * half);
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // word i of this half holds columns 16*half + 4i .. +3 (low nibbles) and 32 + the same (high nibbles)
      bytes4_to_bf16(w[i] & 0x0F0F0F0Fu, s2_lo, c2_lo, r[8 * half + 2 * i], r[8 * half + 2 * i + 1]);
      bytes4_to_bf16(w[i] & 0xF0F0F0F0u, s2_hi, c2_hi, r[16 + 8 * half + 2 * i], r[16 + 8 * half + 2 * i + 1]);
    }
  }
}

// Q6_K, k-block c of the 224-byte block [ql 128][qh 64][scales 16][d]: half = c >> 1, cb = c & 1.  Columns
// 32t + l (t = 0, 1) of the k-block are element (half, qt = 2cb + t, l): ql byte half*64 + 32t + l (low nibble when
// cb = 0, high when cb = 1), qh byte 128 + half*32 + l bits [2qt, 2qt+2), scale index half*8 + 2qt + (l >> 4).
__device__ __forceinline__ void unpack_q6k(const uint8_t* blk, int c, uint32_t (&r)[32]) {
  const int half = c >> 1, cb = c & 1;
  const float d = __half2float(*reinterpret_cast<const __half*>(blk + 208));
  const uint32_t scw = *reinterpret_cast<const uint32_t*>(blk + 192 + half * 8 + 4 * cb);   // 4 int8 scales
  const uint4 h0 = *reinterpret_cast<const uint4*>(blk + 128 + half * 32);
  const uint4 h1 = *reinterpret_cast<const uint4*>(blk + 128 + half * 32 + 16);
  const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int sh = 4 * cb + 2 * t;   // = 2 * qt
#pragma unroll
    for (int u = 0; u < 2; ++u) {    // l = 16u .. 16u+15 share one scale
      const uint4 la = *reinterpret_cast<const uint4*>(blk + half * 64 + 32 * t + 16 * u);
      const uint32_t lw[4] = {la.x, la.y, la.z, la.w};
      const float sv = d * (float)(int8_t)(scw >> (8 * (2 * t + u)));   // weight = sv * (stored - 32)
      const uint64_t s2 = dup_f2(sv), c2 = dup_f2(-1056.f * sv);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // the two high bits land on bits 4..5 of every byte with one shift (left or right by |sh - 4|)
        const uint32_t hsh = sh >= 4 ? (hw[4 * u + i] >> (sh - 4)) : (hw[4 * u + i] << (4 - sh));
        const uint32_t q6 = ((cb ? (lw[i] >> 4) : lw[i]) & 0x0F0F0F0Fu) | (hsh & 0x30303030u);
        bytes4_to_bf16(q6, s2, c2, r[16 * t + 8 * u + 2 * i], r[16 * t + 8 * u + 2 * i + 1]);
      }
    }
  }
}

// Q8_0, k-block c of a 256-column range staged as two 128-byte-swizzled planes [2][128 rows][128 int8] and one
// plane [128 rows][8 fp16 scales]; `row` is the row inside the tile.
__device__ __forceinline__ void unpack_q80(const uint8_t* qst, int row, int c, uint32_t (&r)[32]) {
  const uint8_t* plane = qst + (size_t)(c >> 1) * (WN * 128) + (size_t)row * 128;
  const uint32_t scw = *reinterpret_cast<const uint32_t*>(qst + 2 * WN * 128 + (size_t)row * 16 + 4 * c);
  const __half2 sc2 = *reinterpret_cast<const __half2*>(&scw);
  // the byte with its sign bit flipped is q + 128: weight = d * (v - 128), exact in fp32
  const float d0 = __low2float(sc2), d1 = __high2float(sc2);
  const uint64_t s2[2] = {dup_f2(d0), dup_f2(d1)}, c2[2] = {dup_f2(-1152.f * d0), dup_f2(-1152.f * d1)};
#pragma unroll
  for (int j = 0; j < 4; ++j) {      // 16-byte chunk j of the k-block = chunk 4*(c&1) + j of the 128-byte row
    const int chunk = 4 * (c & 1) + j;
    const uint4 qv = *reinterpret_cast<const uint4*>(plane + ((chunk ^ (row & 7)) << 4));
    const uint32_t w[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      bytes4_to_bf16(w[i] ^ 0x80808080u, s2[j >> 1], c2[j >> 1], r[8 * j + 2 * i], r[8 * j + 2 * i + 1]);
  }
}

// Cursor of a ring whose depth is a runtime value: stage index and phase bit advance without divisions.
struct RingCursor {
  int s = 0;
  uint32_t ph = 0;
  __device__ __forceinline__ void next(int depth) {
    if (++s == depth) {
      s = 0;
      ph ^= 1u;
    }
  }
};

__device__ __forceinline__ int q_row_bytes(int qtype) { return qtype == HE_Q4_K ? 144 : (qtype == HE_Q6_K ? 224 : 272); }

// Tile walk shared by every role: tile index -> (split, m-tile, n-tile); M-fastest so that CTAs running at the
// same time share the weight tile in L2.
// In pair mode a work unit is one weight tile against TWO neighbouring M-tiles (tm, tm + 1): the weight tile is
// expanded once and every operand stage feeds two MMAs, one per accumulator, which halves the expansion work per
// FLOP.  `ntile` is 2 there (1 for the last unit of an odd tile count) and 1 otherwise.
struct TileCoord {
  int ks, tm, tn, b_row0, sb0, sb1, ntile;
  bool skip;
};

__device__ __forceinline__ TileCoord tile_coord(const WqArgs& g, int tile, int tiles_m, int sb_all) {
  TileCoord t;
  const int ksp = g.k_splits;
  t.ks = tile % ksp;
  const int mn = tile / ksp;
  if (g.pair) {
    const int units_m = (tiles_m + 1) >> 1;
    t.tm = (mn % units_m) * 2;
    t.tn = mn / units_m;
    t.ntile = min(2, tiles_m - t.tm);
  } else {
    t.tm = mn % tiles_m;
    t.tn = mn / tiles_m;
    t.ntile = 1;
  }
  t.b_row0 = t.tn * WN;
  t.skip = false;
  if (g.tile_group != nullptr) {
    const int grp = __ldg(g.tile_group + t.tm);
    t.skip = grp < 0;
    t.b_row0 += (grp < 0 ? 0 : grp) * g.N;
  }
  t.sb0 = t.ks * g.sb_per;
  t.sb1 = min(sb_all, t.sb0 + g.sb_per);
  return t;
}

constexpr int WARP_COLL = WARP_UNPACK0 + N_UNPACK_WARPS;   // second collective warp of the reduce-scatter form
constexpr int NTHREADS_WQ_RS = NTHREADS_WQ + 32;

// Phase 2 of the reduce-scatter form for one warp: quarter q of owned tile (tm, tn).  Lane = weight row (output
// column n); each 16-byte group holds 8 consecutive activation rows m of that column.
__device__ __forceinline__ void rs_reduce_quarter(const WqArgs& g, const WqFuse& f, int tm, int tn, int tiles_n,
                                                  int q) {
  const int lane = threadIdx.x & 31, W = f.world;
  const int slot = (tm / W) * tiles_n + tn;
  const __nv_bfloat16* src0 = f.stage[f.rank] + (size_t)slot * RS_TILE_ELEMS + (size_t)q * 32 * MT_MAX;
  const size_t src_stride = (size_t)f.slots * RS_TILE_ELEMS;
  const int n = tn * WN + q * 32 + lane;
  const int m0 = tm * g.mt;
  const int m_lim = min(g.mt, g.M - m0);
  if (n >= g.N) return;
  float* hcol = f.resid + (size_t)m0 * f.ld_resid + n;
#pragma unroll 1
  for (int gi0 = 0; gi0 * 8 < m_lim; gi0 += 4) {
    float acc[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
    for (int r = 0; r < W; ++r) {           // rank order: every owner sums the same way
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        v[u] = (gi0 + u) * 8 < m_lim ? ld_cg_u4(src0 + (size_t)r * src_stride + ((size_t)(gi0 + u) * 32 + lane) * 8)
                                     : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t2 = __bfloat1622float2(hv[e]);
          acc[u][2 * e] += t2.x;
          acc[u][2 * e + 1] += t2.y;
        }
      }
    }
    // fire-and-forget adds (performed at the L2, no value comes back): the warp never waits for the old residual,
    // and an instruction of the warp covers 32 consecutive columns of one row
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int m = (gi0 + u) * 8 + e;
        if (m < m_lim)
          asm volatile("red.global.add.f32 [%0], %1;" ::"l"(hcol + (size_t)m * f.ld_resid), "f"(acc[u][e]) : "memory");
      }
  }
}

template <bool RS, bool SMALL>
__device__ __forceinline__ void gemm_wq_body(const CUtensorMap& tmX, const CUtensorMap& tmQ0, const CUtensorMap& tmQ1,
                                             const WqArgs& g, const WqFuse* f) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* qring = smem + XSTAGES * g.x_stage_bytes;
  WqBarriers* bar = reinterpret_cast<WqBarriers*>(qring + g.q_stages * g.q_stage_bytes);
  const int QS = g.q_stages;
  volatile int* abort_flag = &bar->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt = g.mt;
  const int tiles_m = (g.M + mt - 1) / mt, tiles_n = (g.N + WN - 1) / WN;
  const int units_m = g.pair ? (tiles_m + 1) >> 1 : tiles_m;
  const int n_tiles = (RS && !(f->phases & 1)) ? 0 : units_m * tiles_n * g.k_splits;   // work units
  const int sb_all = g.K >> 8;

  if (threadIdx.x == 0) {
    for (int s = 0; s < XSTAGES; ++s) {
      mbar_init(&bar->x_full[s], 1);
      mbar_init(&bar->x_empty[s], 1);
    }
    for (int s = 0; s < QS; ++s) {
      mbar_init(&bar->q_full[s], 1);
      mbar_init(&bar->q_empty[s], N_UNPACK_WARPS);
    }
    // large tiles: one barrier pair per operand stage (a k-block, filled by the 4 warps of a set); small tiles: one
    // pair per slot of a whole super-block (filled by all 16 warps), so that the MMA issuer -- a single thread, and
    // the critical path when an MMA batch lasts tens of cycles -- waits and commits once per super-block
    for (int s = 0; s < A_STAGES_MAX; ++s) {
      mbar_init(&bar->a_full[s], SMALL ? N_UNPACK_WARPS : N_UNPACK_WARPS / N_SETS);
      mbar_init(&bar->a_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bar->d_full[a], 1);
      mbar_init(&bar->d_empty[a], 4);
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
  // compile-time ring geometry (see WqArgs::x_kb / a_depth): the MMA issuer's index arithmetic is on the critical
  // path when tiles are small, so no runtime divisors
  constexpr int AD = SMALL ? A_DEPTH_MAX : 1, XKB = SMALL ? X_KB_WIDE : 1;
  constexpr int d_cols = SMALL ? D_COLS_SMALL : D_COLS;   // accumulator stride
  constexpr int a_col0 = 2 * d_cols;                      // first operand-stage column
  uint32_t rs_epoch = 0;
  if constexpr (RS) rs_epoch = *reinterpret_cast<volatile uint32_t*>(f->sync) + 1;

  if (warp == 0) {
    // ------------------------------------------------------------ activation tiles
    if (elect_one()) {
      tma_prefetch_desc(&tmX);
      uint32_t it = 0;
      uint32_t ag_seen = 0;                     // owners whose rows are known to have arrived
      const uint32_t ag_want = g.ag_world > 0 ? *reinterpret_cast<const volatile uint32_t*>(g.ag_epoch) : 0u;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const TileCoord t = tile_coord(g, tile, tiles_m, sb_all);
        if (t.skip) continue;
        for (int j = 0; j < t.ntile && g.ag_world > 0; ++j) {
          const int owner = (t.tm + j) % g.ag_world;
          if (!(ag_seen & (1u << owner))) {
            unsigned polls = 0;
            while ((int)(ld_acquire_sys_u32(g.ag_flags + owner) - ag_want) < 0) {
              if (++polls > g.ag_wait_limit) {
                if (g.status != nullptr) atomicCAS(g.status, 0, HE_ERR_WAIT_TIMEOUT);
                break;
              }
              __nanosleep(100);
            }
            asm volatile("fence.proxy.async;" ::: "memory");   // rows written by a peer, read next by TMA
            ag_seen |= 1u << owner;
          }
        }
        // a stage holds XKB k-blocks of one M-tile (XKB > 1 only with one tile per unit)
        for (int kb = 4 * t.sb0; kb < 4 * t.sb1 && !*abort_flag; kb += XKB)
          for (int j = 0; j < t.ntile; ++j, ++it) {
            const int s = it % XSTAGES;
            if (!mbar_wait(&bar->x_empty[s], ((it / XSTAGES) & 1) ^ 1, abort_flag, g.status, 301)) break;
            mbar_expect_tx(&bar->x_full[s], (uint32_t)(XKB * mt * BK * 2));
            for (int u = 0; u < XKB; ++u)
              tma_load_2d(smem + s * g.x_stage_bytes + u * mt * BK * 2, &tmX, &bar->x_full[s], (kb + u) * BK,
                          (t.tm + j) * mt);
          }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ raw weight blocks
    if (elect_one()) {
      tma_prefetch_desc(&tmQ0);
      const uint32_t rb = (uint32_t)q_row_bytes(g.qtype);
      uint32_t qit = 0;
      RingCursor qc;
      const bool qprof = HE_WQ_PROF_ON && g.dbg != nullptr && blockIdx.x == 0;
      long long c_qe = 0, c_qall = qprof ? clock64() : 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const TileCoord t = tile_coord(g, tile, tiles_m, sb_all);
        if (t.skip) continue;
        for (int sb = t.sb0; sb < t.sb1; ++sb, ++qit, qc.next(QS)) {
          const int qs = qc.s;
          long long p0 = qprof ? clock64() : 0;
          if (!mbar_wait(&bar->q_empty[qs], qc.ph ^ 1u, abort_flag, g.status, 302)) break;
          if (qprof) c_qe += clock64() - p0;
          uint8_t* dst = qring + qs * g.q_stage_bytes;
          uint64_t* fb = &bar->q_full[qs];
          mbar_expect_tx(fb, WN * rb);
          if (g.qtype == HE_Q8_0) {
            tma_load_2d(dst, &tmQ0, fb, sb * 256, t.b_row0);
            tma_load_2d(dst + WN * 128, &tmQ0, fb, sb * 256 + 128, t.b_row0);
            tma_load_2d(dst + 2 * WN * 128, &tmQ1, fb, g.K + 16 * sb, t.b_row0);
          } else {
            tma_load_2d(dst, &tmQ0, fb, sb * (int)rb, t.b_row0);
          }
        }
        if (*abort_flag) break;
      }
      if (qprof) { g.dbg[16] = c_qe; g.dbg[17] = clock64() - c_qall; g.dbg[18] = qit; }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = umma_idesc_bf16(WN, mt);
      uint32_t it = 0, ait = 0, ucount = 0;
      uint32_t par = 0;                         // bit b: parity of the completed uses of accumulator b
      const bool mprof = HE_WQ_PROF_ON && g.dbg != nullptr && blockIdx.x == 0;
      long long c_af = 0, c_xf = 0, c_de = 0, c_all = mprof ? clock64() : 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const TileCoord t = tile_coord(g, tile, tiles_m, sb_all);
        if (t.skip) continue;
        // pair mode: tile j of the unit accumulates in buffer j; otherwise units alternate between the buffers so
        // that the epilogue of one overlaps the main loop of the next
        const int acc0 = g.pair ? 0 : (int)(ucount & 1);
        bool ok = true;
        long long d0 = mprof ? clock64() : 0;
        for (int j = 0; j < t.ntile && ok; ++j)
          ok = mbar_wait(&bar->d_empty[acc0 + j], ((par >> (acc0 + j)) & 1) ^ 1, abort_flag, g.status, 303);
        if (!ok) break;
        if (mprof) c_de += clock64() - d0;
        tc_fence_after();
        const int n_kb = 4 * (t.sb1 - t.sb0);
        if constexpr (SMALL) {
          // one super-block per iteration: slot sbi % AD of the operand ring, one activation stage (4 k-blocks)
          const uint32_t d_tmem = tmem_base + acc0 * d_cols;
          for (int sb = 0; sb < t.sb1 - t.sb0 && ok; ++sb, ait += N_SETS, ++it) {
            const uint32_t sbi = ait / N_SETS;
            const int slot = (int)(sbi % AD), s = it % XSTAGES;
            long long m0 = 0;
            if (mprof) m0 = clock64();
            if (!mbar_wait(&bar->a_full[slot], (sbi / AD) & 1, abort_flag, g.status, 305)) { ok = false; break; }
            if (mprof) { c_af += clock64() - m0; m0 = clock64(); }
            if (!mbar_wait(&bar->x_full[s], (it / XSTAGES) & 1, abort_flag, g.status, 304)) { ok = false; break; }
            if (mprof) c_xf += clock64() - m0;
            tc_fence_after();
            const uint32_t x_addr = smem_u32(smem + s * g.x_stage_bytes);
            const uint32_t a_tmem = tmem_base + a_col0 + slot * (N_SETS * A_STAGE_COLS);
#pragma unroll
            for (int c = 0; c < N_SETS; ++c)
#pragma unroll
              for (int k = 0; k < BK / UK; ++k)
                umma_f16_ts(d_tmem, a_tmem + c * A_STAGE_COLS + k * (UK / 2),
                            umma_desc_k_sw128(x_addr + c * mt * BK * 2 + k * UK * 2), idesc,
                            (sb > 0 || c > 0 || k > 0) ? 1u : 0u);
            umma_commit(&bar->x_empty[s]);
            umma_commit(&bar->a_empty[slot]);
          }
        } else {
        for (int kb = 0; kb < n_kb && ok; ++kb, ++ait) {
            // operand stage of k-block c of the unit-spanning super-block count sbi: set c, slot sbi % AD
            const uint32_t sbi = ait / N_SETS;
            const int a = (int)(ait % N_SETS) + N_SETS * (int)(sbi % AD);
            long long m0 = 0;
            if (mprof) m0 = clock64();
            if (!mbar_wait(&bar->a_full[a], (sbi / AD) & 1, abort_flag, g.status, 305)) { ok = false; break; }
            if (mprof) c_af += clock64() - m0;
            const uint32_t a_tmem = tmem_base + a_col0 + a * A_STAGE_COLS;
            const int u = kb % XKB;           // k-block inside the activation stage
            for (int j = 0; j < t.ntile; ++j) {
              const int s = it % XSTAGES;
              if (mprof) m0 = clock64();
              if (u == 0 && !mbar_wait(&bar->x_full[s], (it / XSTAGES) & 1, abort_flag, g.status, 304)) {
                ok = false;
                break;
              }
              if (mprof) c_xf += clock64() - m0;
              tc_fence_after();
              const uint32_t x_addr = smem_u32(smem + s * g.x_stage_bytes + u * mt * BK * 2);
              const uint32_t d_tmem = tmem_base + (acc0 + j) * d_cols;
  #pragma unroll
              for (int k = 0; k < BK / UK; ++k)
                umma_f16_ts(d_tmem, a_tmem + k * (UK / 2), umma_desc_k_sw128(x_addr + k * UK * 2), idesc,
                            (kb > 0 || k > 0) ? 1u : 0u);
              if (u == XKB - 1) {
                umma_commit(&bar->x_empty[s]);  // the smem stage is free once these MMAs have read it
                ++it;
              }
            }
            umma_commit(&bar->a_empty[a]);    // ... and so is the TMEM operand stage
          }
        }
        if (!ok || *abort_flag) break;
        for (int j = 0; j < t.ntile; ++j) {
          umma_commit(&bar->d_full[acc0 + j]);
          par ^= 1u << (acc0 + j);
        }
        ++ucount;
      }
      if (mprof) {
        g.dbg[8] = c_af; g.dbg[9] = c_xf; g.dbg[10] = c_de; g.dbg[11] = clock64() - c_all; g.dbg[12] = ait;
      }
    }
  } else if (warp >= WARP_UNPACK0 && warp < WARP_COLL) {
    // ------------------------------------------------------------ unpack: raw blocks -> bf16 operand in TMEM
    const int set = (warp - WARP_UNPACK0) >> 2;          // k-block of every super-block this warp expands
    const int row = (warp & 3) * 32 + lane;              // weight row in the tile == TMEM lane
    const uint32_t a_tmem0 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + a_col0 + set * A_STAGE_COLS;
    const uint32_t rb = (uint32_t)q_row_bytes(g.qtype);
    uint32_t qit = 0;
    RingCursor qc;
    bool ok = true;
    const bool prof = HE_WQ_PROF_ON && g.dbg != nullptr && blockIdx.x == 0 && warp == WARP_UNPACK0;
    long long c_q = 0, c_math = 0, c_a = 0, c_st = 0, t0 = 0, t1;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const TileCoord t = tile_coord(g, tile, tiles_m, sb_all);
      if (t.skip) continue;
      for (int sb = t.sb0; sb < t.sb1; ++sb, ++qit, qc.next(QS)) {
        const int qs = qc.s;
        if (prof) t0 = clock64();
        if (!mbar_wait(&bar->q_full[qs], qc.ph, abort_flag, g.status, 306)) { ok = false; break; }
        if (prof) { t1 = clock64(); c_q += t1 - t0; t0 = t1; }
        const uint8_t* qst = qring + qs * g.q_stage_bytes;
        uint32_t r[32];
        if (g.qtype == HE_Q4_K) unpack_q4k(qst + (size_t)row * 144, set, r);
        else if (g.qtype == HE_Q6_K) unpack_q6k(qst + (size_t)row * 224, set, r);
        else unpack_q80(qst, row, set, r);
        // the set's operand stages are reused every AD super-blocks: wait until the MMAs that read this one
        // AD super-blocks ago are done
        const int a = SMALL ? (int)(qit % AD) : set + N_SETS * (int)(qit % AD);
        if (prof) { t1 = clock64(); c_math += t1 - t0; t0 = t1; }
        if (!mbar_wait(&bar->a_empty[a], ((qit / AD) & 1) ^ 1, abort_flag, g.status, 307)) { ok = false; break; }
        if (prof) { t1 = clock64(); c_a += t1 - t0; t0 = t1; }
        tc_fence_after();
        tmem_st_32x32(a_tmem0 + (qit % AD) * (N_SETS * A_STAGE_COLS), r);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bar->a_full[a]);
          mbar_arrive(&bar->q_empty[qs]);
        }
        if (prof) { t1 = clock64(); c_st += t1 - t0; }
      }
    }
    if (prof && lane == 0) {
      g.dbg[0] = c_q; g.dbg[1] = c_math; g.dbg[2] = c_a; g.dbg[3] = c_st; g.dbg[4] = qit;
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------ epilogue (warps 4..7): transposed store
    const int q = warp & 3;
    uint32_t ucount = 0;
    uint32_t par = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
      const TileCoord t = tile_coord(g, tile, tiles_m, sb_all);
      if (t.skip) continue;
      for (int j = 0; j < t.ntile; ++j) {
      const int acc = g.pair ? j : (int)(ucount & 1);
      const int tmj = t.tm + j;                              // the M-tile held by this accumulator
      if (!mbar_wait(&bar->d_full[acc], (par >> acc) & 1, abort_flag, g.status, 308)) { ok = false; break; }
      par ^= 1u << acc;
      tc_fence_after();
      const int n = t.tn * WN + q * 32 + lane;               // output column of this thread
      const bool n_ok = n < g.N;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * d_cols;
      const int m0 = tmj * mt;
      const int m_lim = min(mt, g.M - m0);                   // live activation rows of this tile
#pragma unroll 1
      for (int c = 0; c * 32 < m_lim; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int jn = min(32, m_lim - c * 32);
        if constexpr (RS) {
          // partial quarter -> the owner's stage slot, bf16, fragment-major (16-byte group gi = 4c + v of lane l at
          // (gi * 32 + l) * 8): a store instruction of the warp covers 512 contiguous bytes on the link
          const int W = f->world, owner = tmj % W;
          const int slot = (tmj / W) * tiles_n + t.tn;
          __nv_bfloat16* dst = f->stage[owner] + ((size_t)f->rank * f->slots + slot) * RS_TILE_ELEMS +
                               (size_t)q * 32 * MT_MAX + ((size_t)(c * 4) * 32 + lane) * 8;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 pk;
            uint32_t* pw = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * e]),
                                                        __uint_as_float(r[v * 8 + 2 * e + 1]));
              pw[e] = *reinterpret_cast<uint32_t*>(&h2);
            }
            if (v * 8 < jn) *reinterpret_cast<uint4*>(dst + (size_t)v * 256) = pk;
          }
        } else
        if (n_ok) {
          if (g.epi == 0) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(g.C) + (size_t)(m0 + c * 32) * g.ldc + n;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < jn) dst[(size_t)j * g.ldc] = __float2bfloat16_rn(__uint_as_float(r[j]));
          } else {
            float* dst = reinterpret_cast<float*>(g.C) + (size_t)(m0 + c * 32) * g.ldc + n +
                         (g.epi == 4 ? (size_t)t.ks * (size_t)g.split_stride : (size_t)0);
            if (g.epi == 2) {
              // one CTA owns the tile, so each element gets exactly one add (order-free, reproducible); the add is
              // performed at the L2 and nothing comes back, so the warp never waits for the old value
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < jn)
                  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)j * g.ldc), "f"(__uint_as_float(r[j]))
                               : "memory");
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j < jn) dst[(size_t)j * g.ldc] = __uint_as_float(r[j]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar->d_empty[acc]);
      if constexpr (RS) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int W = f->world;
          const int slot = (tmj / W) * tiles_n + t.tn;
          st_release_sys_u32(f->flags[tmj % W] + ((size_t)slot * W + f->rank) * 4 + q, rs_epoch);
        }
      }
      }
      ++ucount;
    }
  } else if (RS && (warp == 3 || warp == WARP_COLL)) {
    // ------------------------------------------------------------ collective warps (reduce-scatter form only)
    // Units = (owned tile, quarter); this CTA's two warps take units b*2 + {0,1}, + 2*grid, ... and reduce whichever
    // has its world stamps; they give up after wait_limit polls without progress.
    if constexpr (RS) {
      if (f->phases & 2) {
        const int W = f->world;
        const int owned_m = tiles_m > f->rank ? (tiles_m - f->rank + W - 1) / W : 0;
        const int n_units = owned_m * tiles_n * 4;
        const uint32_t* my_flags = f->flags[f->rank];
        unsigned stall = 0;
        int u = (int)blockIdx.x * 2 + (warp == 3 ? 0 : 1);
        while (u < n_units) {
          const int q = u & 3, ot = u >> 2;
          const int tm = f->rank + W * (ot % owned_m), tn = ot / owned_m;
          const int slot = (tm / W) * tiles_n + tn;
          bool ready = true;
          if (lane < W) ready = (int)(ld_acquire_sys_u32(my_flags + ((size_t)slot * W + lane) * 4 + q) - rs_epoch) >= 0;
          if (__all_sync(0xffffffffu, ready)) {
            rs_reduce_quarter(g, *f, tm, tn, tiles_n, q);
            u += 2 * (int)gridDim.x;
            stall = 0;
          } else {
            if (++stall > f->wait_limit || *abort_flag) {
              if (lane == 0 && g.status != nullptr) atomicCAS(g.status, 0, HE_ERR_WAIT_TIMEOUT);
              break;
            }
            __nanosleep(200);
          }
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
  if constexpr (RS) {
    // the last CTA to leave a launch that ran the final phase publishes the new epoch for the next launch
    if (threadIdx.x == 0 && (f->phases & 2)) {
      __threadfence();
      const unsigned prev = atomicAdd(f->sync + 1, 1u);
      if (prev == gridDim.x - 1) {
        f->sync[1] = 0;
        f->sync[0] = rs_epoch;
        __threadfence();
      }
    }
  }
}

__global__ void __launch_bounds__(NTHREADS_WQ, 1)
gemm_wq_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmQ0,
               const __grid_constant__ CUtensorMap tmQ1, const WqArgs g) {
  gemm_wq_body<false, false>(tmX, tmQ0, tmQ1, g, nullptr);
}

__global__ void __launch_bounds__(NTHREADS_WQ, 1)
gemm_wq_small_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmQ0,
                     const __grid_constant__ CUtensorMap tmQ1, const WqArgs g) {
  gemm_wq_body<false, true>(tmX, tmQ0, tmQ1, g, nullptr);
}

__global__ void __launch_bounds__(NTHREADS_WQ_RS, 1)
gemm_wq_rs_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmQ0,
                  const __grid_constant__ CUtensorMap tmQ1, const WqArgs g, const __grid_constant__ WqFuse f) {
  gemm_wq_body<true, false>(tmX, tmQ0, tmQ1, g, &f);
}

// out[m][n] (+)= sum over splits, in split order (deterministic).  mode 0: fp32 store, 1: fp32 add in place.
__global__ void wq_splitk_reduce_kernel(const float* __restrict__ part, long long split_stride, int k_splits,
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

// ---------------------------------------------------------------- host side
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

// Activations: bf16 row-major [rows][cols], row stride ld elements; box {64 columns, box_rows}, 128-byte swizzle.
int make_x_map(CUtensorMap* m, const void* ptr, long long rows, long long cols, long long ld, int box_rows) {
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

// Raw weight rows as bytes: [rows][row_bytes] uint8; box {box_bytes, 128 rows}.
int make_q_map(CUtensorMap* m, const void* ptr, long long rows, long long row_bytes, int box_bytes, bool swizzle128) {
  EncodeTiledFn enc = get_encode();
  if (enc == nullptr) return -HE_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || row_bytes % 16 != 0 || box_bytes % 16 != 0) return -HE_ERR_BAD_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)WN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 1000 + (int)r;
}

int make_q_maps(CUtensorMap* q0, CUtensorMap* q1, const void* B, int qtype, long long rows, int K) {
  int rc;
  if (qtype == HE_Q4_K) {
    rc = make_q_map(q0, B, rows, (long long)(K >> 8) * 144, 144, false);
    *q1 = *q0;
    return rc;
  }
  if (qtype == HE_Q6_K) {
    rc = make_q_map(q0, B, rows, (long long)(K >> 8) * 224, 224, false);
    *q1 = *q0;
    return rc;
  }
  if (qtype == HE_Q8_0) {
    const long long rb = (long long)K + (((K >> 4) + 15) / 16) * 16;
    if ((rc = make_q_map(q0, B, rows, rb, 128, true)) != 0) return rc;
    return make_q_map(q1, B, rows, rb, 16, false);
  }
  return -HE_ERR_BAD_ARG;
}

constexpr size_t SMEM_WQ = (size_t)SMEM_BUDGET + sizeof(WqBarriers) + 1024;

// HE_GEMMQ_PAIR=0 turns the two-tiles-per-weight-tile mode off (for comparisons).
bool pair_mode_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HE_GEMMQ_PAIR");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// HE_GEMMQ_SMALL=0 turns the deep-ring variant for tiles of <= 48 rows off (for comparisons).
bool small_mode_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("HE_GEMMQ_SMALL");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

int pick_mt(int M, bool grouped) {
  if (grouped) return 128;
  if (M >= MT_MAX) return MT_MAX;
  return (M + 15) & ~15;
}

long long* g_debug_counters = nullptr;

int launch_wq(const void* A, long long lda, int a_cols, const void* B, int qtype, long long b_rows, WqArgs g,
              int num_sms, cudaStream_t stream, const WqFuse* fuse = nullptr) {
  if (g.K % 256 != 0) return -HE_ERR_BAD_ARG;
  if (a_cols <= 0 || a_cols > g.K || a_cols % 8 != 0) return -HE_ERR_BAD_ARG;
  const int row_bytes = qtype == HE_Q4_K ? 144 : (qtype == HE_Q6_K ? 224 : 272);
  g.dbg = g_debug_counters;
  const bool small = small_mode_enabled() && g.mt <= 48 && g.tile_group == nullptr && fuse == nullptr;
  g.x_kb = small ? X_KB_WIDE : 1;
  g.a_depth = small ? A_DEPTH_MAX : 1;
  g.x_stage_bytes = (g.x_kb * g.mt * BK * 2 + 1023) & ~1023;
  g.q_stage_bytes = (WN * row_bytes + 1023) & ~1023;
  {
    const int tiles_m0 = (g.M + g.mt - 1) / g.mt;
    g.pair = (pair_mode_enabled() && g.tile_group == nullptr && g.k_splits == 1 && tiles_m0 >= 2) ? 1 : 0;
  }
  g.q_stages = (SMEM_BUDGET - XSTAGES * g.x_stage_bytes) / g.q_stage_bytes;
  if (g.q_stages > QSTAGES_MAX) g.q_stages = QSTAGES_MAX;
  if (g.q_stages < 2) return -HE_ERR_BAD_ARG;
  CUtensorMap tmX, q0, q1;
  int rc = make_x_map(&tmX, A, g.M, a_cols, lda, g.mt);
  if (rc != 0) return rc;
  rc = make_q_maps(&q0, &q1, B, qtype, b_rows, g.K);
  if (rc != 0) return rc;
  const int tiles_m = (g.M + g.mt - 1) / g.mt;
  const long long tiles = (long long)(g.pair ? (tiles_m + 1) / 2 : tiles_m) * ((g.N + WN - 1) / WN) * g.k_splits;
  const int grid = (int)(tiles < num_sms ? tiles : num_sms);
  if (fuse != nullptr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wq_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_WQ);
    if (e != cudaSuccess) return (int)e;
    // CTAs of this kernel wait for stamps written by CTAs of other ranks, so the whole grid has to be resident at
    // once: refuse a grid the device cannot hold (the caller then takes GEMM + library collective); the waits stay
    // bounded either way
    static int resident_per_sm[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (resident_per_sm[dev] == 0) {
      int n = 0;
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemm_wq_rs_kernel, NTHREADS_WQ_RS, SMEM_WQ);
      if (e != cudaSuccess) return (int)e;
      resident_per_sm[dev] = n > 0 ? n : -1;
    }
    if (resident_per_sm[dev] < 0 || (long long)grid > (long long)resident_per_sm[dev] * num_sms) return -HE_ERR_BAD_ARG;
    gemm_wq_rs_kernel<<<grid, NTHREADS_WQ_RS, SMEM_WQ, stream>>>(tmX, q0, q1, g, *fuse);
  } else if (small) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wq_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)SMEM_WQ);
    if (e != cudaSuccess) return (int)e;
    gemm_wq_small_kernel<<<grid, NTHREADS_WQ, SMEM_WQ, stream>>>(tmX, q0, q1, g);
  } else {
    cudaError_t e = cudaFuncSetAttribute(gemm_wq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_WQ);
    if (e != cudaSuccess) return (int)e;
    gemm_wq_kernel<<<grid, NTHREADS_WQ, SMEM_WQ, stream>>>(tmX, q0, q1, g);
  }
  HE_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// Developer aid (builds with -DHE_WQ_PROFILE=1, a no-op otherwise): with a device array of >= 32 int64 set here, CTA 0
// of every following quantised GEMM records the
// cycles its roles spent waiting ([0..4] one unpack warp: raw-block wait, expansion, operand-stage wait, TMEM store,
// super-blocks; [8..12] MMA issuer: operand wait, activation wait, accumulator wait, total, k-blocks; [16..18] raw
// block producer: free-stage wait, total, stages).  Null (the default) turns it off.
HE_API void he_gemm_q_debug_counters(void* dev_i64x32) { g_debug_counters = (long long*)dev_i64x32; }

// C[M][N] = A[M][K] (bf16) * W[N][K]^T where W is `b_rows` rows in the device layout of `qtype` (Q4_K / Q6_K / Q8_0),
// expanded to bf16 inside the pipeline.  epi: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate into C.
// `a_cols` (<= K, multiple of 8) is the number of columns A really has: columns up to K read as zeros (weights whose
// K was padded to a whole number of 256-column blocks).  With `tile_group` (device, ceil(M/128) ints) the call is the
// grouped form: 128-row M-tile tm uses weight rows [tile_group[tm] * N, +N); negative entries skip the tile.
HE_API int he_gemm_q(const void* A, long long lda, int a_cols, const void* B, int qtype, long long b_rows, void* C,
                     long long ldc, int M, int N, int K, int epi, const int* tile_group, void* status, int num_sms,
                     cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  WqArgs g = {};
  g.C = C; g.ldc = ldc; g.M = M; g.N = N; g.K = K; g.epi = epi; g.qtype = qtype;
  g.mt = pick_mt(M, tile_group != nullptr);
  g.k_splits = 1;
  g.sb_per = K >> 8;
  g.split_stride = 0;
  g.tile_group = tile_group;
  g.status = (int*)status;
  return launch_wq(A, lda, a_cols, B, qtype, b_rows, g, num_sms, stream);
}

// Split plan of the deterministic split-K form: about one tile per SM, every split a whole number of 256-column
// super-blocks and none empty.  Low 32 bits: split count; high 32 bits: super-blocks per split.
HE_API long long he_gemm_q_splitk_plan(int M, int N, int K, int num_sms) {
  const int mt = pick_mt(M, false);
  const int tiles = ((M + mt - 1) / mt) * ((N + WN - 1) / WN);
  const int sb_all = K >> 8;
  // cost of a plan = rounds of work items per CTA x super-blocks per item (+1 per round for the tile change-over)
  int k_splits = 1, sb_per = sb_all;
  long long best = -1;
  for (int ks = 1; ks <= sb_all && ks <= 32; ++ks) {
    const int per = (sb_all + ks - 1) / ks;
    const int ks_eff = (sb_all + per - 1) / per;
    const long long items = (long long)tiles * ks_eff;
    const long long rounds = (items + num_sms - 1) / num_sms;
    const long long cost = rounds * (per + 1);
    if (best < 0 || cost < best) {
      best = cost;
      k_splits = ks_eff;
      sb_per = per;
    }
  }
  return ((long long)sb_per << 32) | (long long)k_splits;
}

// out[M][N] (fp32) = (mode 0) or += (mode 1) A * W^T for few rows: the K range is split over CTAs so that every SM
// streams a share of the quantised weight; partial tiles go to `partials` ([k_splits][M][N] fp32, caller scratch)
// and are summed in split order (bit-reproducible).
HE_API int he_gemm_q_splitk_det(const void* A, long long lda, const void* B, int qtype, long long b_rows,
                                void* partials, void* out, long long ldo, int M, int N, int K, int mode, void* status,
                                int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (N % 4 != 0 || K % 256 != 0) return -HE_ERR_BAD_ARG;
  const long long plan = he_gemm_q_splitk_plan(M, N, K, num_sms);
  WqArgs g = {};
  g.C = partials; g.ldc = N; g.M = M; g.N = N; g.K = K; g.epi = 4; g.qtype = qtype;
  g.mt = pick_mt(M, false);
  g.k_splits = (int)(plan & 0xffffffffll);
  g.sb_per = (int)(plan >> 32);
  if (g.k_splits == 1) {
    // enough tiles to fill the GPU without splitting: one CTA owns each output tile, so it stores (or adds, one add
    // per element: order-free) straight into `out` and no reduction pass runs
    g.C = out; g.ldc = ldo; g.epi = mode == 1 ? 2 : 1;
    g.status = (int*)status;
    return launch_wq(A, lda, K, B, qtype, b_rows, g, num_sms, stream);
  }
  g.split_stride = (long long)M * N;
  g.tile_group = nullptr;
  g.status = (int*)status;
  const int rc = launch_wq(A, lda, K, B, qtype, b_rows, g, num_sms, stream);
  if (rc != 0) return rc;
  const long long n4 = ((long long)M * N + 3) / 4;
  wq_splitk_reduce_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>((const float*)partials, g.split_stride,
                                                                           g.k_splits, (float*)out, ldo, M, N, mode);
  HE_LAUNCH_CHECK();
  return 0;
}

// The plain quantised GEMM with the all-gather wait of sequence-parallel activations (see WqArgs::ag_flags): A's rows
// of M-tile tm (tiles of he_gemm_q_mt(M) rows) were written by rank tm % ag_world, which then stamped ag_flags[rank]
// with the value found in *ag_epoch.
HE_API int he_gemm_q_mt(int M) { return pick_mt(M, false); }

HE_API int he_gemm_q_ag(const void* A, long long lda, int a_cols, const void* B, int qtype, long long b_rows, void* C,
                        long long ldc, int M, int N, int K, int epi, const void* ag_flags, const void* ag_epoch,
                        int ag_world, unsigned ag_wait_limit, void* status, int num_sms, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (ag_world < 1 || ag_world > RS_MAX_WORLD || ag_flags == nullptr || ag_epoch == nullptr) return -HE_ERR_BAD_ARG;
  WqArgs g = {};
  g.C = C; g.ldc = ldc; g.M = M; g.N = N; g.K = K; g.epi = epi; g.qtype = qtype;
  g.mt = pick_mt(M, false);
  g.k_splits = 1;
  g.sb_per = K >> 8;
  g.status = (int*)status;
  g.ag_flags = (const uint32_t*)ag_flags;
  g.ag_epoch = (const uint32_t*)ag_epoch;
  g.ag_world = ag_world;
  g.ag_wait_limit = ag_wait_limit;
  return launch_wq(A, lda, a_cols, B, qtype, b_rows, g, num_sms, stream);
}

// resid[owned rows][N] (fp32) += sum over ranks of A_rank[M][K] * W_rank[N][K]^T for the M-tiles this rank owns (tile
// tm of he_gemm_q_mt(M) rows belongs to rank tm % world): the GEMM and the reduce-scatter over peer memory in one
// kernel per rank (see WqFuse).  Every rank issues the same calls with the same M and N.
HE_API int he_gemm_q_fuse_args_size() { return (int)sizeof(WqFuse); }
HE_API int he_gemm_q_rs_tile_elems() { return RS_TILE_ELEMS; }

HE_API int he_gemm_q_reduce_scatter(const void* A, long long lda, const void* B, int qtype, long long b_rows, int M,
                                    int N, int K, const WqFuse* fuse, void* status, int num_sms,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const WqFuse& f = *fuse;
  const int mt = pick_mt(M, false);
  const int tiles_m = (M + mt - 1) / mt, tiles_n = (N + WN - 1) / WN;
  if (f.world < 1 || f.world > RS_MAX_WORLD || f.rank < 0 || f.rank >= f.world) return -HE_ERR_BAD_ARG;
  if (((tiles_m + f.world - 1) / f.world) * tiles_n > f.slots) return -HE_ERR_BAD_ARG;
  if (f.resid == nullptr || f.ld_resid < N || (f.phases & 3) == 0 || f.sync == nullptr) return -HE_ERR_BAD_ARG;
  for (int r = 0; r < f.world; ++r)
    if (f.stage[r] == nullptr || f.flags[r] == nullptr) return -HE_ERR_BAD_ARG;
  WqArgs g = {};
  g.C = nullptr; g.ldc = 0; g.M = M; g.N = N; g.K = K; g.epi = 5; g.qtype = qtype;
  g.mt = mt;
  g.k_splits = 1;
  g.sb_per = K >> 8;
  g.status = (int*)status;
  return launch_wq(A, lda, K, B, qtype, b_rows, g, num_sms, stream, fuse);
}
