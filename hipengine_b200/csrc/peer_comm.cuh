// Peer-memory plumbing shared by the decode GEMV (push epilogue / reduce prologue) and the small collective kernels
// of comm.cu.  The reference engine is single-device: no counterpart there.
#pragma once

#include "common.cuh"

// Tensor-parallel decode: the all-reduce of a row-parallel projection is folded into the two GEMVs around it.
//   push   (mode bit 0): this launch is the row-parallel projection.  Its epilogue stores every partial output
//          straight into slot (parity, my rank) of EVERY rank's receive region (plain stores over NVLink for peers).
//          Each element travels as one 8-byte word {fp32 value, sequence tag}: an aligned 8-byte store lands as a
//          whole, so a reader that sees the tag of the current push holds valid data -- no fence, no separate flag,
//          one link crossing of latency.  The last CTA to finish advances the local sequence number.
//   reduce (mode bit 1): this launch is the first consumer of the residual afterwards.  Its prologue reads the
//          words of all ranks, re-reading (bounded) those whose tag is not yet the current one, forms
//          h + sum over ranks (rank order, so replicas stay bit-identical) in registers, feeds that to the norm /
//          quantisation, and the last CTA through the prologue writes the new residual back in place.
// Receive region of a rank: [2 parities][world][max_rows * width] words, then [2][world] u32 stamps (used by the
// (max, id) merge of the greedy head).  `state` is local: [0] sequence number of the last completed push, [1] CTAs
// that finished the current push, [2..9] CTAs that have read residual row r in the current reduce.  Two parities
// suffice: a rank needs every peer's words to finish a reduce, so it is never more than one push ahead of the
// slowest rank, and a slot is overwritten only two pushes later.
constexpr int GEMV_MAX_WORLD = 8;
struct HeGemvComm {
  uint2* recv[GEMV_MAX_WORLD];
  uint32_t* flags[GEMV_MAX_WORLD];
  uint32_t* state;
  int world, rank;
  int slot_floats;      // max_rows * width (words per slot)
  int width;            // row length of the reduced tensor (the hidden size)
  int mode;             // bit 0: push from the epilogue, bit 1: reduce into the prologue
  unsigned wait_limit;  // re-reads before a wait gives up
};

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}

// Eight consecutive tagged words -> eight floats, re-reading until every tag equals `tag` (bounded: after `limit`
// re-reads the status word gets HE_ERR_WAIT_TIMEOUT and whatever is there is returned).
__device__ __forceinline__ void ll_load8(const uint2* p, uint32_t tag, unsigned limit, int* status, float (&out)[8]) {
  uint4 w[4];
  unsigned tries = 0;
  for (;;) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(w[i].x), "=r"(w[i].y), "=r"(w[i].z), "=r"(w[i].w)
                   : "l"(reinterpret_cast<const uint4*>(p) + i));
    bool ok = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) ok = ok && w[i].y == tag && w[i].w == tag;
    if (ok) break;
    if (++tries > limit) {
      if (status != nullptr) atomicCAS(status, 0, HE_ERR_WAIT_TIMEOUT);
      break;
    }
    __nanosleep(20);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i].x);
    out[2 * i + 1] = __uint_as_float(w[i].z);
  }
}

__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
