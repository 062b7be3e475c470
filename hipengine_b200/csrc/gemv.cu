// Quantized GEMV for decode (1..8 activation rows): Q4_K / Q6_K / Q8_0 / F32 / F16 / BF16 weights.
//
// One launch = weight stream + [activation prologue] + [dot products] + [epilogue]:
//   weight stream : every warp owns a ring of shared-memory slots and keeps the next row chunks in flight
//                   with cp.async.bulk (1-D bulk copies completing on an mbarrier), so DRAM latency is hidden
//                   without spending registers, and the first copies are issued before the activation
//                   prologue runs.
//   prologue      : every CTA loads the activation rows, optionally applies RMSNorm (fp32 statistics, the
//                   weight used directly) and quantises them to int8 per 32 elements into shared memory.
//   dot products  : a warp works on rg rows x 32/rg blocks at a time, one lane per (row, 256-element block);
//                   nibble unpack in registers, dp4a against the int8 activations, per-sub-block fp32 scaling.
//   epilogue      : fp32/bf16 store, fp32 residual add in place, or act(gate)*up for gate/up pairs.
// Up to four weight segments (e.g. attn_qkv + attn_gate + ssm_alpha + ssm_beta) share one launch.
//
// Behavioural reference: the decode GEMV family in hipengine/kernels/hip_gfx1100/quant/gguf_q4_k_gemv.hip
// (Q8_1 activation quantize + integer dot) and the oracle hipengine/kernels/cpu_reference/ops.py:466-537.
#include <cstdlib>
#include "common.cuh"
#include "gemv_rows.cuh"
#include "peer_comm.cuh"
#include "sm100.cuh"

using namespace he;
using hegemv::SmemView;

struct HeGemvSeg {
  const void* w;
  const void* w2;
  void* out;
  long long out_stride;
  int n_rows;
  int qtype;
  int qtype2;
  int epi;  // 0: f32 store, 1: bf16 store, 2: f32 +=, 3: silu(g)*u -> bf16, 4: gelu_tanh(g)*u -> bf16
};

struct HeGemvArgs {
  HeGemvSeg seg[4];
  int n_seg;
  int K;
  int R;
  int x_dtype;  // 0 f32, 1 bf16
  const void* x;
  long long x_stride;
  const float* norm_w;
  float eps;
  int n_slots;      // ring depth per warp (set by the launcher)
  int rg;           // weight rows per work item: 2, 4 or 8 (set by the launcher); 32/rg blocks per staged unit
  int slot_bytes;   // bytes of one ring slot = rg * row_stride
  int* status;      // device status word (may be null)
  HeGemvComm comm;  // mode 0: unused
  // Optional image of the normalised + quantised activation rows in exactly the kernel's shared-memory layout
  // (he_gemv_prequant): the CTAs copy it instead of each running the prologue over all R rows.  With several rows the
  // per-CTA prologue (R x K elements and a block reduction per row, in every CTA of every launch) costs more than
  // the dot products of the small projections.
  const uint8_t* x_image;
};

namespace {

constexpr int MAX_SLOTS = 4;

__device__ __forceinline__ void load8(const void* x, int dtype, size_t off, float (&v)[8]) {
  if (dtype == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off);
    const float4 a = __ldg(p), b = __ldg(p + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + off));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
}

// Quantise 8 consecutive activations (4 neighbouring lanes form one 32-wide block) into shared memory.
__device__ __forceinline__ void quant_store(const SmemView& s, int K, int r, int g, bool valid, float (&v)[8]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float d = amax / 127.f;
  const float inv = d > 0.f ? 1.f / d : 0.f;
  int q[8];
  int qsum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    q[i] = __float2int_rn(v[i] * inv);
    qsum += q[i];
  }
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
  if (valid) {
    const uint32_t p0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t p1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2*>(s.xq + (size_t)r * s.xq_row + (size_t)(g >> 5) * hegemv::XQ_STRIDE + (g & 31) * 8) =
        make_uint2(p0, p1);
    if ((g & 3) == 0) {
      s.dx[(size_t)r * s.sc_row + (g >> 2)] = d;
      s.sx[(size_t)r * s.sc_row + (g >> 2)] = d * (float)qsum;
    }
  }
}

// (optional RMSNorm) + per-32 int8 quantisation.  With a norm and K <= 8192 the row is read once and kept in
// registers between the statistics and the quantisation.
template <int R, bool COMM>
__device__ void prologue(const HeGemvArgs& a, const SmemView& s, float* red) {
  const int K = a.K;
  const int n_groups = K / 8;
  constexpr int MAXG = 4;
  const int nthr = (int)blockDim.x;
  const bool one_pass = a.norm_w != nullptr && n_groups <= MAXG * nthr;
  // reduce mode (the launcher admits it only with the one-pass prologue and fp32 rows): the rows are the residual
  // stream, to which the partial rows pushed by every rank are added before anything else happens
  const bool rin = COMM && (a.comm.mode & 2) != 0;
  __shared__ int last_cta_s;
  uint32_t rin_tag = 0;
  int parity = 0;
  if (rin) {
    rin_tag = *reinterpret_cast<volatile uint32_t*>(a.comm.state);     // tag of the push being consumed
    parity = (int)((rin_tag - 1u) & 1u);
  }
  for (int r = 0; r < R; ++r) {
    const size_t base = (size_t)r * a.x_stride;
    if (one_pass) {
      float v[MAXG][8];
      float ss = 0.f;
#pragma unroll
      for (int u = 0; u < MAXG; ++u) {
        const int g = u * nthr + (int)threadIdx.x;
        if (g < n_groups) {
          load8(a.x, a.x_dtype, base + (size_t)g * 8, v[u]);
          if (rin) {
            const uint2* pp = a.comm.recv[a.comm.rank] + (size_t)parity * a.comm.world * a.comm.slot_floats +
                              (size_t)r * a.comm.width + (size_t)g * 8;
            for (int q = 0; q < a.comm.world; ++q, pp += a.comm.slot_floats) {   // rank order: replicas agree
              float pv[8];
              ll_load8(pp, rin_tag, a.comm.wait_limit, a.status, pv);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[u][i] += pv[i];
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) ss += v[u][i] * v[u][i];
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[u][i] = 0.f;
        }
      }
      ss = block_sum(ss, red);
      const float inv_rms = rsqrtf(ss / (float)K + a.eps);
      if (threadIdx.x == 0) s.inv_rms[r] = inv_rms;
      if (rin) {
        // every thread of this CTA has read row r (the barriers inside block_sum); the last CTA of the grid to get
        // here is the only one that may overwrite the row with the reduced residual
        if (threadIdx.x == 0) {
          const unsigned prev = atomicAdd(a.comm.state + 2 + r, 1u);
          last_cta_s = prev == gridDim.x - 1;
          if (last_cta_s) a.comm.state[2 + r] = 0;
        }
        __syncthreads();
        if (last_cta_s) {
          float* xw = const_cast<float*>(reinterpret_cast<const float*>(a.x)) + base;
#pragma unroll
          for (int u = 0; u < MAXG; ++u) {
            const int g = u * nthr + (int)threadIdx.x;
            if (g < n_groups) {
              reinterpret_cast<float4*>(xw + (size_t)g * 8)[0] = make_float4(v[u][0], v[u][1], v[u][2], v[u][3]);
              reinterpret_cast<float4*>(xw + (size_t)g * 8)[1] = make_float4(v[u][4], v[u][5], v[u][6], v[u][7]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < MAXG; ++u) {
        const int g = u * nthr + (int)threadIdx.x;
        if (u * nthr < n_groups) {  // uniform across the CTA
          const bool valid = g < n_groups;
          if (valid) {
            const float4* wp = reinterpret_cast<const float4*>(a.norm_w + (size_t)g * 8);
            const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
            v[u][0] *= inv_rms * w0.x; v[u][1] *= inv_rms * w0.y; v[u][2] *= inv_rms * w0.z; v[u][3] *= inv_rms * w0.w;
            v[u][4] *= inv_rms * w1.x; v[u][5] *= inv_rms * w1.y; v[u][6] *= inv_rms * w1.z; v[u][7] *= inv_rms * w1.w;
          }
          quant_store(s, K, r, g, valid, v[u]);
        }
      }
      continue;
    }
    float inv_rms = 1.f;
    if (a.norm_w != nullptr) {
      float ss = 0.f;
      for (int g = threadIdx.x; g < n_groups; g += blockDim.x) {
        float v[8];
        load8(a.x, a.x_dtype, base + (size_t)g * 8, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
      }
      ss = block_sum(ss, red);
      inv_rms = rsqrtf(ss / (float)K + a.eps);
    }
    if (threadIdx.x == 0) s.inv_rms[r] = inv_rms;
    for (int g0 = 0; g0 < n_groups; g0 += blockDim.x) {
      const int g = g0 + threadIdx.x;
      const bool valid = g < n_groups;
      float v[8];
      if (valid) {
        load8(a.x, a.x_dtype, base + (size_t)g * 8, v);
        if (a.norm_w != nullptr) {
          const float4* wp = reinterpret_cast<const float4*>(a.norm_w + (size_t)g * 8);
          const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
          v[0] *= inv_rms * w0.x; v[1] *= inv_rms * w0.y; v[2] *= inv_rms * w0.z; v[3] *= inv_rms * w0.w;
          v[4] *= inv_rms * w1.x; v[5] *= inv_rms * w1.y; v[6] *= inv_rms * w1.z; v[7] *= inv_rms * w1.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
      quant_store(s, K, r, g, valid, v);
    }
  }
  __syncthreads();
}



// ---------------------------------------------------------------- work decomposition (32-bit arithmetic only)
// An item is rg = 1 << rg_shift weight rows.  Plain segments: rows [rg*i, rg*i + rg).  Gate/up pair segments:
// rg/2 gate rows [i*rg/2, ...) in row slots t < rg/2 and the same rows of the up weight in t >= rg/2.
__device__ __forceinline__ int seg_items(const HeGemvSeg& sg, int rg_shift) {
  const int sh = sg.epi >= 3 ? rg_shift - 1 : rg_shift;
  return (sg.n_rows + (1 << sh) - 1) >> sh;
}

struct ItemLoc {
  int si;     // segment
  int row0;   // first row of the item inside the segment
};

__device__ __forceinline__ ItemLoc locate(const HeGemvArgs& a, int item, int rg_shift) {
  ItemLoc L;
  L.si = 0;
  while (L.si < a.n_seg - 1) {
    const int cnt = seg_items(a.seg[L.si], rg_shift);
    if (item < cnt) break;
    item -= cnt;
    ++L.si;
  }
  L.row0 = item << (a.seg[L.si].epi >= 3 ? rg_shift - 1 : rg_shift);
  return L;
}

// Row slot t (0..rg-1) of an item: which weight, which quant type, which row (clamped), and whether it is real.
struct RowRef {
  const uint8_t* w;
  int qt;
  int n;
  bool valid;
};

__device__ __forceinline__ RowRef row_of(const HeGemvArgs& a, const ItemLoc& L, int t, int rg) {
  const HeGemvSeg& sg = a.seg[L.si];
  RowRef r;
  if (sg.epi >= 3) {
    const int hp = rg >> 1;
    const bool up = t >= hp;
    r.w = reinterpret_cast<const uint8_t*>(up ? sg.w2 : sg.w);
    r.qt = up ? sg.qtype2 : sg.qtype;
    r.n = L.row0 + (up ? t - hp : t);
  } else {
    r.w = reinterpret_cast<const uint8_t*>(sg.w);
    r.qt = sg.qtype;
    r.n = L.row0 + t;
  }
  r.valid = r.n < sg.n_rows;
  if (!r.valid) r.n = sg.n_rows - 1;
  return r;
}

// Bytes one row contributes to a staged unit of `nblk` 256-element blocks (float weights are not staged).
__device__ __forceinline__ uint32_t unit_bytes(int qt, int nblk) {
  if (qt == HE_Q4_K) return (uint32_t)nblk * 144;
  if (qt == HE_Q6_K) return (uint32_t)nblk * 224;
  if (qt == HE_Q8_0) return (uint32_t)nblk * 272;
  return 0;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(sm100::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ float apply_act(float g, int epi) { return epi == 3 ? silu_f(g) : gelu_tanh_f(g); }

// One CTA per activation row: (optional RMSNorm) + per-32 int8 quantisation of row blockIdx.x into `image`, which has
// the layout of gemv_kernel's shared-memory activation area for R rows (xq | dx | sx | inv_rms).
__global__ void __launch_bounds__(512) gemv_prequant_kernel(const void* __restrict__ x, int x_dtype, long long x_stride,
                                                            const float* __restrict__ norm_w, float eps, int K, int R,
                                                            uint8_t* __restrict__ image) {
  __shared__ float red[33];
  const int r = blockIdx.x, nb = K >> 8, n_groups = K / 8;
  // let the consumer GEMV start right away (it only prefetches weights until its own wait, which this grid's
  // completion releases), then wait: the rows come from the previous kernel, and the image may still be read by it
  pdl_launch();
  pdl_wait();
  SmemView s;
  s.xq_row = nb * hegemv::XQ_STRIDE;
  s.sc_row = nb * 8;
  s.xq = reinterpret_cast<int8_t*>(image);
  s.dx = reinterpret_cast<float*>(image + (size_t)R * s.xq_row);
  s.sx = s.dx + (size_t)R * s.sc_row;
  s.inv_rms = s.sx + (size_t)R * s.sc_row;
  const size_t base = (size_t)r * x_stride;
  float inv_rms = 1.f;
  if (norm_w != nullptr) {
    float ss = 0.f;
    for (int g = threadIdx.x; g < n_groups; g += blockDim.x) {
      float v[8];
      load8(x, x_dtype, base + (size_t)g * 8, v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = block_sum(ss, red);
    inv_rms = rsqrtf(ss / (float)K + eps);
  }
  if (threadIdx.x == 0) s.inv_rms[r] = inv_rms;
  for (int g0 = 0; g0 < n_groups; g0 += blockDim.x) {
    const int g = g0 + threadIdx.x;
    const bool valid = g < n_groups;
    float v[8];
    if (valid) {
      load8(x, x_dtype, base + (size_t)g * 8, v);
      if (norm_w != nullptr) {
        const float4* wp = reinterpret_cast<const float4*>(norm_w + (size_t)g * 8);
        const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
        v[0] *= inv_rms * w0.x; v[1] *= inv_rms * w0.y; v[2] *= inv_rms * w0.z; v[3] *= inv_rms * w0.w;
        v[4] *= inv_rms * w1.x; v[5] *= inv_rms * w1.y; v[6] *= inv_rms * w1.z; v[7] *= inv_rms * w1.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
    }
    quant_store(s, K, r, g, valid, v);
  }
}

// Cursor over this warp's units: item index (global), unit within item, ring slot and its phase parity.
struct Cursor {
  int item;     // global item id
  int uk;       // unit within the item
  int slot;
  uint32_t parity;
  int left;     // units still to visit
};

// COMM = false compiles the tensor-parallel push / reduce paths out (the single-GPU kernel carries none of their
// registers or branches).
// P2 (batches of 2+ rows, no peer communication): a lane owns half a block of TWO weight rows of the staged unit
// instead of one block of one row, so every activation word it loads serves two rows (see gemv_rows.cuh).
template <int R, int NW, bool COMM, bool P2>
__global__ void __launch_bounds__(NW * 32, 1) gemv_kernel(const __grid_constant__ HeGemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[33];
  __shared__ __align__(8) uint64_t bars[NW][MAX_SLOTS];
  __shared__ int abort_flag;

  const int K = a.K, nb = K >> 8;
  const int rg = a.rg, rg_shift = 31 - __clz(rg), BQ = 32 >> rg_shift, bq_shift = 5 - rg_shift;
  SmemView s;
  s.xq_row = nb * hegemv::XQ_STRIDE;
  s.sc_row = nb * 8;
  s.xq = reinterpret_cast<int8_t*>(smem);
  s.dx = reinterpret_cast<float*>(smem + (size_t)R * s.xq_row);
  s.sx = s.dx + (size_t)R * s.sc_row;
  s.inv_rms = s.sx + (size_t)R * s.sc_row;
  const uint32_t x_bytes = ((uint32_t)R * s.xq_row + (uint32_t)R * s.sc_row * 8 + 64 + 127) & ~127u;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* ring = smem + x_bytes + (uint32_t)warp * a.n_slots * a.slot_bytes;
  const int row_stride = a.slot_bytes >> rg_shift;

  if (threadIdx.x == 0) abort_flag = 0;
  if (lane == 0) {
    for (int i = 0; i < a.n_slots; ++i) sm100::mbar_init(&bars[warp][i], 1);
    sm100::mbar_fence_init();
  }
  __syncthreads();

  int total_items = 0;
  for (int i = 0; i < a.n_seg; ++i) total_items += seg_items(a.seg[i], rg_shift);
  const int upi = (nb + BQ - 1) >> bq_shift;                 // staged units per item
  const int gw = warp * gridDim.x + blockIdx.x;             // global warp id, CTA-first: item i starts on CTA i % grid
  const int tw = gridDim.x * NW;                            // total warps
  const int my_items = gw < total_items ? (total_items - gw + tw - 1) / tw : 0;
  const int my_units = my_items * upi;

  auto advance = [&](Cursor& c) {
    if (++c.uk == upi) { c.uk = 0; c.item += tw; }
    if (++c.slot == a.n_slots) { c.slot = 0; c.parity ^= 1u; }
    --c.left;
  };

  // Warp-collective: stage the unit under the producer cursor, then advance it.
  Cursor pc{gw, 0, 0, 0u, my_units};
  ItemLoc pL = locate(a, gw < total_items ? gw : 0, rg_shift);
  auto issue = [&]() {
    if (pc.left <= 0) return;
    if (pc.uk == 0 && pc.item != gw) pL = locate(a, pc.item, rg_shift);
    const int blk0 = pc.uk << bq_shift, nblk = min(BQ, nb - blk0);
    uint64_t* bar = &bars[warp][pc.slot];
    RowRef rr;
    uint32_t bytes = 0;
    if (lane < rg) {
      rr = row_of(a, pL, lane, rg);
      bytes = unit_bytes(rr.qt, nblk);
    }
    uint32_t total = bytes;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);   // rg <= 8 lanes carry bytes
    total = __shfl_sync(0xffffffffu, total, 0);
    if (lane == 0) {
      if (total > 0) sm100::mbar_expect_tx(bar, total);
      else sm100::mbar_arrive(bar);
    }
    __syncwarp();
    if (lane < rg && bytes > 0) {
      uint8_t* dst = ring + (uint32_t)pc.slot * a.slot_bytes + (uint32_t)lane * row_stride;
      const uint8_t* src = rr.w + (size_t)rr.n * (size_t)hegemv::row_bytes_dev(rr.qt, K);
      if (rr.qt == HE_Q4_K) bulk_g2s(dst, src + (uint32_t)blk0 * 144, bytes, bar);
      else if (rr.qt == HE_Q6_K) bulk_g2s(dst, src + (uint32_t)blk0 * 224, bytes, bar);
      else {
        bulk_g2s(dst, src + (uint32_t)blk0 * 256, (uint32_t)nblk * 256, bar);
        bulk_g2s(dst + nblk * 256, src + K + (uint32_t)blk0 * 16, (uint32_t)nblk * 16, bar);
      }
    }
    advance(pc);
  };

  // Programmatic dependent launch: let the next kernel of the stream start its own weight prefetch while this
  // grid drains, start ours before the producer of the activations has finished, and only then wait for it.
  asm volatile("griddepcontrol.launch_dependents;");
  for (int i = 0; i < a.n_slots - 1; ++i) issue();
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const bool push = COMM && (a.comm.mode & 1) != 0;
  uint32_t push_seq = 0;
  size_t push_off = 0;                 // float offset of slot (parity, my rank) inside a receive region
  if (push) {
    push_seq = *reinterpret_cast<volatile uint32_t*>(a.comm.state);
    push_off = ((size_t)(push_seq & 1u) * a.comm.world + a.comm.rank) * a.comm.slot_floats;
  }
  auto push_store = [&](int r, int n, float v) {
    const size_t off = push_off + (size_t)r * a.comm.width + n;
    for (int q = 0; q < a.comm.world; ++q) ll_store(a.comm.recv[q] + off, v, push_seq + 1u);
  };

  if (R >= 2 && a.x_image != nullptr) {   // single-row launches keep the in-CTA prologue (he_gemv refuses an image)
    // rows already normalised and quantised by he_gemv_prequant (complete: griddepcontrol.wait above): copy the image
    const uint32_t img16 = ((uint32_t)R * s.xq_row + (uint32_t)R * s.sc_row * 8 + 64) >> 4;
    const uint4* src = reinterpret_cast<const uint4*>(a.x_image);
    uint4* dst = reinterpret_cast<uint4*>(smem);
    for (uint32_t i = threadIdx.x; i < img16; i += blockDim.x) {
      uint4 v;
      asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i));
      dst[i] = v;
    }
    __syncthreads();
  } else {
    prologue<R, COMM>(a, s, red);
  }

  if constexpr (P2) {
    // lane = (row pair tp, block bq2 of the unit, half hsel of the block); rows tp and tp + rg/2 of the item: for a
    // gate/up pair segment these are gate row n and up row n, so the activation epilogue needs no shuffle
    const int hsel = lane & 1, bq2 = (lane >> 1) & (BQ - 1), tp = lane >> (bq_shift + 1), hp = rg >> 1;
    float accA[R], accB[R];
    Cursor cc{gw, 0, 0, 0u, my_units};
    ItemLoc L = pL;
    RowRef rA, rB;
    while (cc.left > 0) {
      issue();
      if (cc.uk == 0) {
        L = locate(a, cc.item, rg_shift);
        rA = row_of(a, L, tp, rg);
        rB = row_of(a, L, tp + hp, rg);
#pragma unroll
        for (int r = 0; r < R; ++r) accA[r] = accB[r] = 0.f;
        const HeGemvSeg& fsg = a.seg[L.si];
        if (fsg.qtype != HE_Q4_K && fsg.qtype != HE_Q6_K && fsg.qtype != HE_Q8_0 && fsg.epi < 3) {
          // float-weight rows: the whole warp walks each row with coalesced loads (nothing was staged for them)
          for (int t = 0; t < rg; ++t) {
            const RowRef fr = row_of(a, L, t, rg);
            if (!fr.valid) break;
            float fa[R];
#pragma unroll
            for (int r = 0; r < R; ++r) fa[r] = 0.f;
            hegemv::row_float_coop<R>(fr.w + (size_t)fr.n * (size_t)hegemv::row_bytes_dev(fr.qt, K), fr.qt, K, a.x,
                                      a.x_dtype, a.x_stride, a.norm_w, s, lane, fa);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              const float v = warp_sum(fa[r]);
              if (lane == 0) {
                const size_t off = (size_t)r * fsg.out_stride + fr.n;
                if (fsg.epi == 0) reinterpret_cast<float*>(fsg.out)[off] = v;
                else if (fsg.epi == 1) reinterpret_cast<__nv_bfloat16*>(fsg.out)[off] = f32_to_bf16(v);
                else reinterpret_cast<float*>(fsg.out)[off] += v;
              }
            }
          }
        }
      }
      const bool quant_item = rA.qt == HE_Q4_K || rA.qt == HE_Q6_K || rA.qt == HE_Q8_0;
      if (!sm100::mbar_wait(&bars[warp][cc.slot], cc.parity, &abort_flag, a.status, 201)) break;
      const int blk0 = cc.uk << bq_shift, nblk = min(BQ, nb - blk0);
      if (bq2 < nblk && quant_item) {
        const int b = blk0 + bq2;
        const uint8_t* slot = ring + (uint32_t)cc.slot * a.slot_bytes;
        const uint8_t* pa = slot + (uint32_t)tp * row_stride;
        const uint8_t* pb = slot + (uint32_t)(tp + hp) * row_stride;
        if (rA.qt == HE_Q4_K) hegemv::half_q4k_x2<R>(pa + bq2 * 144, pb + bq2 * 144, b, hsel, s, accA, accB);
        else if (rA.qt == HE_Q6_K) hegemv::half_q6k_x2<R>(pa + bq2 * 224, pb + bq2 * 224, b, hsel, s, accA, accB);
        else
          hegemv::half_q80_x2<R>(pa + bq2 * 256, pa + nblk * 256 + bq2 * 16, pb + bq2 * 256,
                                 pb + nblk * 256 + bq2 * 16, b, hsel, s, accA, accB);
      }
      __syncwarp();   // every lane is done reading the slot before it may be refilled in the next iteration
      if (cc.uk == upi - 1 && quant_item) {
        const HeGemvSeg& sg = a.seg[L.si];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float va = accA[r], vb = accB[r];
          for (int o = 1; o < 2 * BQ; o <<= 1) {
            va += __shfl_xor_sync(0xffffffffu, va, o);
            vb += __shfl_xor_sync(0xffffffffu, vb, o);
          }
          accA[r] = va;
          accB[r] = vb;
        }
        if ((lane & (2 * BQ - 1)) == 0) {
          if (sg.epi >= 3) {
            if (rA.valid) {
#pragma unroll
              for (int r = 0; r < R; ++r)
                reinterpret_cast<__nv_bfloat16*>(sg.out)[(size_t)r * sg.out_stride + rA.n] =
                    f32_to_bf16(apply_act(accA[r], sg.epi) * accB[r]);
            }
          } else {
#pragma unroll
            for (int r = 0; r < R; ++r) {
              if (rA.valid) {
                const size_t off = (size_t)r * sg.out_stride + rA.n;
                if (sg.epi == 0) reinterpret_cast<float*>(sg.out)[off] = accA[r];
                else if (sg.epi == 1) reinterpret_cast<__nv_bfloat16*>(sg.out)[off] = f32_to_bf16(accA[r]);
                else reinterpret_cast<float*>(sg.out)[off] += accA[r];
              }
              if (rB.valid) {
                const size_t off = (size_t)r * sg.out_stride + rB.n;
                if (sg.epi == 0) reinterpret_cast<float*>(sg.out)[off] = accB[r];
                else if (sg.epi == 1) reinterpret_cast<__nv_bfloat16*>(sg.out)[off] = f32_to_bf16(accB[r]);
                else reinterpret_cast<float*>(sg.out)[off] += accB[r];
              }
            }
          }
        }
      }
      advance(cc);
    }
  } else {
    const int t_row = lane >> bq_shift, bq = lane & (BQ - 1);
    float acc[R];
    Cursor cc{gw, 0, 0, 0u, my_units};
    ItemLoc L = pL;
    RowRef rr;
    while (cc.left > 0) {
      issue();
      if (cc.uk == 0) {
        L = locate(a, cc.item, rg_shift);
        rr = row_of(a, L, t_row, rg);
  #pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        const HeGemvSeg& fsg = a.seg[L.si];
        if (fsg.qtype != HE_Q4_K && fsg.qtype != HE_Q6_K && fsg.qtype != HE_Q8_0 && fsg.epi < 3) {
          // float-weight rows: the whole warp walks each row with coalesced loads (nothing was staged for them)
          for (int t = 0; t < rg; ++t) {
            const RowRef fr = row_of(a, L, t, rg);
            if (!fr.valid) break;
            float fa[R];
  #pragma unroll
            for (int r = 0; r < R; ++r) fa[r] = 0.f;
            hegemv::row_float_coop<R>(fr.w + (size_t)fr.n * (size_t)hegemv::row_bytes_dev(fr.qt, K), fr.qt, K, a.x,
                                      a.x_dtype, a.x_stride, a.norm_w, s, lane, fa);
  #pragma unroll
            for (int r = 0; r < R; ++r) {
              const float v = warp_sum(fa[r]);
              if (lane == 0) {
                const size_t off = (size_t)r * fsg.out_stride + fr.n;
                if (push) push_store(r, fr.n, v);
                else if (fsg.epi == 0) reinterpret_cast<float*>(fsg.out)[off] = v;
                else if (fsg.epi == 1) reinterpret_cast<__nv_bfloat16*>(fsg.out)[off] = f32_to_bf16(v);
                else reinterpret_cast<float*>(fsg.out)[off] += v;
              }
            }
          }
        }
      }
      const bool float_item = !(rr.qt == HE_Q4_K || rr.qt == HE_Q6_K || rr.qt == HE_Q8_0) && a.seg[L.si].epi < 3;
      if (!sm100::mbar_wait(&bars[warp][cc.slot], cc.parity, &abort_flag, a.status, 201)) break;
      const int blk0 = cc.uk << bq_shift, nblk = min(BQ, nb - blk0);
      if (bq < nblk && !float_item) {
        const int b = blk0 + bq;
        const uint8_t* rowp = ring + (uint32_t)cc.slot * a.slot_bytes + (uint32_t)t_row * row_stride;
        if (rr.qt == HE_Q4_K) hegemv::block_q4k<R>(rowp + bq * 144, b, s, acc);
        else if (rr.qt == HE_Q6_K) hegemv::block_q6k<R>(rowp + bq * 224, b, s, acc);
        else if (rr.qt == HE_Q8_0) hegemv::block_q80<R>(rowp + bq * 256, rowp + nblk * 256 + bq * 16, b, s, acc);
        else {
          const uint32_t es = rr.qt == HE_F32 ? 4 : 2;
          hegemv::block_float<R>(rr.w + (size_t)rr.n * (size_t)hegemv::row_bytes_dev(rr.qt, K) + (size_t)b * 256 * es,
                                 rr.qt, b, a.x, a.x_dtype, a.x_stride, a.norm_w, s, acc);
        }
      }
      __syncwarp();   // every lane is done reading the slot before it may be refilled in the next iteration
      if (cc.uk == upi - 1 && !float_item) {
        const HeGemvSeg& sg = a.seg[L.si];
  #pragma unroll
        for (int r = 0; r < R; ++r) {
          float v = acc[r];
          for (int o = 1; o < BQ; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          acc[r] = v;
        }
        if (sg.epi >= 3) {
          const int hp = rg >> 1;
  #pragma unroll
          for (int r = 0; r < R; ++r) {
            const float up = __shfl_sync(0xffffffffu, acc[r], (lane + hp * BQ) & 31);
            if (bq == 0 && t_row < hp && rr.valid)
              reinterpret_cast<__nv_bfloat16*>(sg.out)[(size_t)r * sg.out_stride + rr.n] =
                  f32_to_bf16(apply_act(acc[r], sg.epi) * up);
          }
        } else if (bq == 0 && rr.valid) {
  #pragma unroll
          for (int r = 0; r < R; ++r) {
            const size_t off = (size_t)r * sg.out_stride + rr.n;
            if (push) push_store(r, rr.n, acc[r]);
            else if (sg.epi == 0) reinterpret_cast<float*>(sg.out)[off] = acc[r];
            else if (sg.epi == 1) reinterpret_cast<__nv_bfloat16*>(sg.out)[off] = f32_to_bf16(acc[r]);
            else reinterpret_cast<float*>(sg.out)[off] += acc[r];
          }
        }
      }
      advance(cc);
    }
  }
  if (push) {
    // the words carry their own tag, so nothing has to be published: the last CTA of the grid only advances the
    // local sequence number for the launches that follow in this stream
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(a.comm.state + 1, 1u);
      if (prev == gridDim.x - 1) {
        a.comm.state[1] = 0;
        *reinterpret_cast<volatile uint32_t*>(a.comm.state) = push_seq + 1u;
      }
    }
  }
}

template <int R, int NW, bool COMM, bool P2>
int launch_nw_c(const HeGemvArgs& a, size_t smem, long long items, int num_sms, cudaStream_t stream) {
  static size_t configured[64] = {};   // per device: the attribute belongs to the (function, device) pair
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (smem > configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<R, NW, COMM, P2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = smem;
  }
  // one CTA per SM as soon as there is an item for each: with fewer items than warps the busy warps are spread over
  // all SMs (the kernel deals items out CTA-first) instead of filling a few CTAs and leaving the other SMs idle
  long long grid = items;
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) grid = 1;
  static const bool pdl = []() {
    const char* e = getenv("HE_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(NW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_kernel<R, NW, COMM, P2>, a);
  if (e != cudaSuccess) return (int)e;
  return 0;
}

template <int R, int NW>
int launch_nw(const HeGemvArgs& a, size_t smem, long long items, int num_sms, cudaStream_t stream, bool p2) {
  if (a.comm.mode != 0) return launch_nw_c<R, NW, true, false>(a, smem, items, num_sms, stream);
  if constexpr (R >= 2) {
    if (p2) return launch_nw_c<R, NW, false, true>(a, smem, items, num_sms, stream);
  }
  return launch_nw_c<R, NW, false, false>(a, smem, items, num_sms, stream);
}

template <int R>
int launch_gemv(HeGemvArgs a, int num_sms, cudaStream_t stream) {
  const int K = a.K, nb = K >> 8;
  long long rows = 0;
  int per_block = 144;
  for (int i = 0; i < a.n_seg; ++i) {
    const HeGemvSeg& sg = a.seg[i];
    rows += (long long)sg.n_rows * (sg.epi >= 3 ? 2 : 1);
    const int types[2] = {sg.qtype, sg.epi >= 3 ? sg.qtype2 : sg.qtype};
    for (int t = 0; t < 2; ++t) {
      const int pb = types[t] == HE_Q6_K ? 224 : (types[t] == HE_Q8_0 ? 272 : 144);
      if (pb > per_block) per_block = pb;
    }
  }
  a.slot_bytes = 32 * per_block;
  const size_t x_bytes = ((size_t)R * nb * hegemv::XQ_STRIDE + (size_t)R * nb * 8 * 8 + 64 + 127) & ~(size_t)127;
  const size_t budget = 224 * 1024;
  // 16 warps per CTA when two ring slots each still fit beside the activations, else 12, else 8
  int nw = 16;
  if (x_bytes + (size_t)2 * 16 * a.slot_bytes > budget) nw = 12;   // Q6_K / Q8_0 slots: 12 warps x 2 slots still fit
  if (x_bytes + (size_t)2 * nw * a.slot_bytes > budget) nw = 8;
  static const int nw_env = []() { const char* e = getenv("HE_GEMV_NW"); return e ? atoi(e) : 0; }();
  if (nw_env == 8 || (nw_env == 12 && nw == 16)) nw = nw_env;
  int n_slots = MAX_SLOTS;
  while (n_slots > 2 && x_bytes + (size_t)n_slots * nw * a.slot_bytes > budget) --n_slots;
  if (x_bytes + (size_t)n_slots * nw * a.slot_bytes > budget) return -HE_ERR_BAD_ARG;
  a.n_slots = n_slots;
  // rows per item: as many as keeps every warp of the grid busy for at least two items
  const long long warps = (long long)num_sms * nw;
  int rg = 8;
  if (nb >= 20) {
    // K >= 5120, any block type (measured on B200 for Q4_K, Q6_K and Q8_0; narrower models measured faster with the
    // plain rule below): what matters is (a) lanes not idling in the last unit of a row --
    // a unit is 32/rg blocks wide, so K = 5120 (20 blocks) wants rg = 8, K = 6144 (24 blocks) rg = 4 -- and
    // (b) at least about half as many work items as warps; pick the rg with the best product of the two
    double best = -1.0;
    for (int cand = 8; cand >= 2; cand >>= 1) {
      const int bq = 32 / cand;
      const double eff = (double)nb / (double)(((nb + bq - 1) / bq) * bq);
      const double fill = (double)(rows / cand) / (0.5 * (double)warps);
      const double score = eff * (fill < 1.0 ? fill : 1.0);
      if (score > best + 1e-9) { best = score; rg = cand; }
    }
  } else {
    while (rg > 2 && rows / rg < 2 * warps) rg >>= 1;
  }
  static const int rg_env = []() { const char* e = getenv("HE_GEMV_RG"); return e ? atoi(e) : 0; }();
  if (rg_env == 2 || rg_env == 4 || rg_env == 8) rg = rg_env;
  a.rg = rg;
  long long items = 0;
  for (int i = 0; i < a.n_seg; ++i) {
    const int per = a.seg[i].epi >= 3 ? rg / 2 : rg;
    items += (a.seg[i].n_rows + per - 1) / per;
  }
  const size_t smem = x_bytes + (size_t)n_slots * nw * a.slot_bytes;
  // two weight rows per lane for batches of 2+ rows (HE_GEMV_PAIR=0: one block of one row per lane as for one row);
  // a gate/up pair segment qualifies when both weights have the same block type, float rows take the warp-wide path
  static const bool pair_env = []() { const char* e = getenv("HE_GEMV_PAIR"); return !(e != nullptr && e[0] == '0'); }();
  bool p2 = R >= 2 && pair_env && a.comm.mode == 0;
  for (int i = 0; i < a.n_seg && p2; ++i) {
    const HeGemvSeg& sg = a.seg[i];
    const bool quant = sg.qtype == HE_Q4_K || sg.qtype == HE_Q6_K || sg.qtype == HE_Q8_0;
    if (sg.epi >= 3 && (!quant || sg.qtype2 != sg.qtype)) p2 = false;
  }
  if (nw == 16) return launch_nw<R, 16>(a, smem, items, num_sms, stream, p2);
  if (nw == 12) return launch_nw<R, 12>(a, smem, items, num_sms, stream, p2);
  return launch_nw<R, 8>(a, smem, items, num_sms, stream, p2);
}

}  // namespace

// Launch the fused GEMV.  `args` is a host pointer to HeGemvArgs (copied by value into the launch).
// K must be a multiple of 256.  Returns -HE_ERR_BAD_ARG when the activation rows plus the staging rings do
// not fit shared memory (callers then split the activation rows over two launches).
// Bytes of the activation image of R rows of K columns (what he_gemv_prequant writes and he_gemv copies).
HE_API long long he_gemv_image_bytes(int R, int K) {
  const long long nb = K >> 8;
  return (((long long)R * nb * hegemv::XQ_STRIDE + (long long)R * nb * 8 * 8 + 64 + 127) / 128) * 128;
}

// image <- (optional RMSNorm with norm_w) + per-32 int8 quantisation of the R rows x[r][0..K).  K % 256 == 0.
HE_API int he_gemv_prequant(const void* x, int x_dtype, long long x_stride, const float* norm_w, float eps, int K,
                            int R, void* image, cudaStream_t stream) {
  if (K % 256 != 0 || R < 1 || R > 8 || x == nullptr || image == nullptr) return -HE_ERR_BAD_ARG;
  cudaError_t le = launch_pdl(gemv_prequant_kernel, dim3(R), dim3(512), 0, stream, x, x_dtype, x_stride, norm_w, eps,
                              K, R, (uint8_t*)image);
  if (le != cudaSuccess) return (int)le;
  return 0;
}

HE_API int he_gemv(const HeGemvArgs* args, int num_sms, cudaStream_t stream) {
  const HeGemvArgs& a = *args;
  if (a.K % 256 != 0 || a.n_seg < 1 || a.n_seg > 4 || a.R < 1 || a.R > 8) return -HE_ERR_BAD_ARG;
  // the reduce prologue computes its rows itself; one row is cheaper to quantise in the CTA than to copy
  if (a.x_image != nullptr && (a.comm.mode != 0 || a.R < 2)) return -HE_ERR_BAD_ARG;
  if (a.comm.mode != 0) {
    const HeGemvComm& c = a.comm;
    if (c.world < 2 || c.world > GEMV_MAX_WORLD || c.rank < 0 || c.rank >= c.world || c.state == nullptr ||
        (long long)a.R * c.width > c.slot_floats)
      return -HE_ERR_BAD_ARG;
    for (int q = 0; q < c.world; ++q)
      if (c.recv[q] == nullptr || c.flags[q] == nullptr) return -HE_ERR_BAD_ARG;
    // push: one fp32-store segment as wide as the reduced tensor
    if ((c.mode & 1) && (a.n_seg != 1 || a.seg[0].epi != 0 || a.seg[0].n_rows != c.width)) return -HE_ERR_BAD_ARG;
    // reduce: fp32 residual rows of that width through the one-pass norm prologue (at most 8192 columns), and every
    // segment quantised (float-typed weights read the activation rows from global memory, not the reduced values)
    if (c.mode & 2) {
      if (a.x_dtype != 0 || a.norm_w == nullptr || a.K != c.width || a.K > 8192 || c.width % 8 != 0)
        return -HE_ERR_BAD_ARG;
      for (int i = 0; i < a.n_seg; ++i) {
        const int t[2] = {a.seg[i].qtype, a.seg[i].epi >= 3 ? a.seg[i].qtype2 : a.seg[i].qtype};
        for (int j = 0; j < 2; ++j)
          if (t[j] != HE_Q4_K && t[j] != HE_Q6_K && t[j] != HE_Q8_0) return -HE_ERR_BAD_ARG;
      }
    }
  }
  switch (a.R) {
    case 1: return launch_gemv<1>(a, num_sms, stream);
    case 2: return launch_gemv<2>(a, num_sms, stream);
    case 3: return launch_gemv<3>(a, num_sms, stream);
    case 4: return launch_gemv<4>(a, num_sms, stream);
    case 5: return launch_gemv<5>(a, num_sms, stream);
    case 6: return launch_gemv<6>(a, num_sms, stream);
    case 7: return launch_gemv<7>(a, num_sms, stream);
    default: return launch_gemv<8>(a, num_sms, stream);
  }
}

HE_API int he_gemv_args_size() { return (int)sizeof(HeGemvArgs); }
