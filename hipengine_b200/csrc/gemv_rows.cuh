// Consumers of the quantized GEMV: one lane owns one 256-element block of one weight row (staged in shared
// memory by a bulk copy) and dots it against the int8-quantised activation rows, also in shared memory.
// Owning a whole block amortises the scale decode over 256 weights and lets the integer dot of a 32-wide
// sub-block finish before a single int->float conversion.
//
// Device weight layouts (every row is contiguous and 16-byte aligned so one cp.async.bulk moves a row chunk):
//   Q4_K : 144-byte GGUF blocks as stored (d, dmin, 12 scale bytes, 128 nibble bytes)
//   Q6_K : 224-byte blocks = [ql 128][qh 64][scales 16][d fp16][14 pad]
//   Q8_0 : per row [K int8][K/32 fp16 scales][pad to 16]
//   F32 / F16 / BF16 : plain rows
// Activation layout in shared memory: per row, block b at xq + b*XQ_STRIDE (256 int8 + 16 pad so that lanes
// working on different blocks hit different banks), scales dx[b*8 + sub], block sums sx[b*8 + sub].
#pragma once

#include "common.cuh"

namespace hegemv {

using namespace he;

constexpr int XQ_STRIDE = 272;

struct SmemView {
  int8_t* xq;      // [R][nb * XQ_STRIDE]
  float* dx;       // [R][K/32]
  float* sx;       // [R][K/32]   dx * sum(q) per 32-block
  float* inv_rms;  // [R]
  int xq_row;      // bytes per activation row in xq
  int sc_row;      // floats per activation row in dx / sx
};

__host__ __device__ __forceinline__ long long row_bytes_dev(int qtype, int K) {
  switch (qtype) {
    case HE_Q4_K: return (long long)(K >> 8) * 144;
    case HE_Q6_K: return (long long)(K >> 8) * 224;
    case HE_Q8_0: return (long long)K + (((K >> 4) + 15) / 16) * 16;
    case HE_F32: return (long long)K * 4;
    default: return (long long)K * 2;
  }
}

__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// ---------------------------------------------------------------- Q4_K: one 144-byte block
template <int R>
__device__ __forceinline__ void block_q4k(const uint8_t* blk, int b, const SmemView& s, float (&acc)[R]) {
  const uint4 meta = *reinterpret_cast<const uint4*>(blk);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&meta.x));
  // 6-bit scales / mins of the 8 sub-blocks (bytes of sc_lo, sc_hi, mn_lo, mn_hi)
  const uint32_t sc_lo = meta.y & 0x3F3F3F3Fu, mn_lo = meta.z & 0x3F3F3F3Fu;
  const uint32_t sc_hi = (meta.w & 0x0F0F0F0Fu) | ((meta.y >> 2) & 0x30303030u);
  const uint32_t mn_hi = ((meta.w >> 4) & 0x0F0F0F0Fu) | ((meta.z >> 2) & 0x30303030u);
  float part[R];
#pragma unroll
  for (int r = 0; r < R; ++r) part[r] = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {   // 64 weights: sub-block 2j in the low nibbles, 2j+1 in the high nibbles
    const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + j * 32);
    const uint4 q1 = *reinterpret_cast<const uint4*>(blk + 32 + j * 32);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const uint32_t scw = (j < 2 ? sc_lo : sc_hi) >> (16 * (j & 1));
    const uint32_t mnw = (j < 2 ? mn_lo : mn_hi) >> (16 * (j & 1));
    const float ds0 = dd.x * (float)(scw & 0xFFu), ds1 = dd.x * 0.0625f * (float)((scw >> 8) & 0xFFu);
    const float dm0 = dd.y * (float)(mnw & 0xFFu), dm1 = dd.y * (float)((mnw >> 8) & 0xFFu);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + 64 * j;
      const int4 xa = *reinterpret_cast<const int4*>(xb);
      const int4 xb1 = *reinterpret_cast<const int4*>(xb + 16);
      const int4 xc = *reinterpret_cast<const int4*>(xb + 32);
      const int4 xd = *reinterpret_cast<const int4*>(xb + 48);
      const int xl[8] = {xa.x, xa.y, xa.z, xa.w, xb1.x, xb1.y, xb1.z, xb1.w};
      const int xh[8] = {xc.x, xc.y, xc.z, xc.w, xd.x, xd.y, xd.z, xd.w};
      int dl = 0, dh = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dl = __dp4a((int)(qw[i] & 0x0F0F0F0Fu), xl[i], dl);
        dh = dp4a_us(qw[i] & 0xF0F0F0F0u, xh[i], dh);     // 16 * q, folded into ds1
      }
      const float2 dx = *reinterpret_cast<const float2*>(s.dx + (size_t)r * s.sc_row + b * 8 + 2 * j);
      const float2 sx = *reinterpret_cast<const float2*>(s.sx + (size_t)r * s.sc_row + b * 8 + 2 * j);
      part[r] += ds0 * dx.x * (float)dl + ds1 * dx.y * (float)dh - dm0 * sx.x - dm1 * sx.y;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] += part[r];
}

// ---------------------------------------------------------------- Q6_K: one 224-byte block
template <int R>
__device__ __forceinline__ void block_q6k(const uint8_t* blk, int b, const SmemView& s, float (&acc)[R]) {
  const uint4 scv = *reinterpret_cast<const uint4*>(blk + 192);
  const float d = __half2float(*reinterpret_cast<const __half*>(blk + 208));
#pragma unroll
  for (int half = 0; half < 2; ++half) {
#pragma unroll
    for (int l16 = 0; l16 < 2; ++l16) {   // positions l = 16*l16 .. +15 of this half
      const uint4 la = *reinterpret_cast<const uint4*>(blk + half * 64 + l16 * 16);
      const uint4 lb = *reinterpret_cast<const uint4*>(blk + half * 64 + 32 + l16 * 16);
      const uint4 hh = *reinterpret_cast<const uint4*>(blk + 128 + half * 32 + l16 * 16);
      const uint32_t lav[4] = {la.x, la.y, la.z, la.w}, lbv[4] = {lb.x, lb.y, lb.z, lb.w};
      const uint32_t hv[4] = {hh.x, hh.y, hh.z, hh.w};
      uint32_t q[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        q[0][u] = __vsub4((lav[u] & 0x0F0F0F0Fu) | ((hv[u] & 0x03030303u) << 4), 0x20202020u);
        q[1][u] = __vsub4((lbv[u] & 0x0F0F0F0Fu) | (((hv[u] >> 2) & 0x03030303u) << 4), 0x20202020u);
        q[2][u] = __vsub4(((lav[u] >> 4) & 0x0F0F0F0Fu) | (((hv[u] >> 4) & 0x03030303u) << 4), 0x20202020u);
        q[3][u] = __vsub4(((lbv[u] >> 4) & 0x0F0F0F0Fu) | (((hv[u] >> 6) & 0x03030303u) << 4), 0x20202020u);
      }
      float dsc[4];
#pragma unroll
      for (int qt = 0; qt < 4; ++qt) dsc[qt] = d * (float)byte_of(scv, half * 8 + 2 * qt + l16);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + half * 128 + l16 * 16;
        const float4 dxq = *reinterpret_cast<const float4*>(s.dx + (size_t)r * s.sc_row + b * 8 + half * 4);
        const float dxa[4] = {dxq.x, dxq.y, dxq.z, dxq.w};
        float t = 0.f;
#pragma unroll
        for (int qt = 0; qt < 4; ++qt) {
          const int4 xv = *reinterpret_cast<const int4*>(xb + 32 * qt);
          int ds = __dp4a((int)q[qt][0], xv.x, 0);
          ds = __dp4a((int)q[qt][1], xv.y, ds);
          ds = __dp4a((int)q[qt][2], xv.z, ds);
          ds = __dp4a((int)q[qt][3], xv.w, ds);
          t += dsc[qt] * dxa[qt] * (float)ds;
        }
        acc[r] += t;
      }
    }
  }
}

// ---------------------------------------------------------------- Q8_0: 256 int8 at `qs`, 8 fp16 scales at `sc`
template <int R>
__device__ __forceinline__ void block_q80(const uint8_t* qs, const uint8_t* sc, int b, const SmemView& s,
                                          float (&acc)[R]) {
  const uint4 scv = *reinterpret_cast<const uint4*>(sc);
  const __half2* sh = reinterpret_cast<const __half2*>(&scv);
#pragma unroll
  for (int sb = 0; sb < 8; ++sb) {
    const uint4 w0 = *reinterpret_cast<const uint4*>(qs + sb * 32);
    const uint4 w1 = *reinterpret_cast<const uint4*>(qs + sb * 32 + 16);
    const float2 dpair = __half22float2(sh[sb >> 1]);
    const float d = (sb & 1) ? dpair.y : dpair.x;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + sb * 32;
      const int4 x0 = *reinterpret_cast<const int4*>(xb);
      const int4 x1 = *reinterpret_cast<const int4*>(xb + 16);
      int ds = __dp4a((int)w0.x, x0.x, 0);
      ds = __dp4a((int)w0.y, x0.y, ds); ds = __dp4a((int)w0.z, x0.z, ds); ds = __dp4a((int)w0.w, x0.w, ds);
      ds = __dp4a((int)w1.x, x1.x, ds); ds = __dp4a((int)w1.y, x1.y, ds);
      ds = __dp4a((int)w1.z, x1.z, ds); ds = __dp4a((int)w1.w, x1.w, ds);
      acc[r] += d * s.dx[(size_t)r * s.sc_row + b * 8 + sb] * (float)ds;
    }
  }
}

// ---------------------------------------------------------------- two weight rows x half a block (multi-row batches)
// With several activation rows the loop above is bound by shared-memory loads of the activations: a 128-bit load by 32
// lanes costs four wavefronts whatever its addresses, and every lane reloads R x 256 activation bytes for its one
// weight block (measured on 17408 x 5120 Q4_K with 4 rows: shared pipe 51 % busy, top stalls short scoreboard and
// MIO throttle, issue slots 43 %).  Here a lane owns HALF a block (128 elements, half `h`) of TWO weight rows (the
// same block index of both): each activation word is loaded once and used for both rows, which halves the
// activation traffic per weight while the staged unit (rows x blocks in a ring slot) stays as it is.

struct Q4KHalfScales {
  float2 dd;        // d, dmin
  uint32_t sc, mn;  // 6-bit scales / mins of the half's four sub-blocks, one per byte
};

__device__ __forceinline__ Q4KHalfScales q4k_half_scales(const uint8_t* blk, int h) {
  const uint4 meta = *reinterpret_cast<const uint4*>(blk);
  Q4KHalfScales o;
  o.dd = __half22float2(*reinterpret_cast<const __half2*>(&meta.x));
  const uint32_t sc_lo = meta.y & 0x3F3F3F3Fu, mn_lo = meta.z & 0x3F3F3F3Fu;
  const uint32_t sc_hi = (meta.w & 0x0F0F0F0Fu) | ((meta.y >> 2) & 0x30303030u);
  const uint32_t mn_hi = ((meta.w >> 4) & 0x0F0F0F0Fu) | ((meta.z >> 2) & 0x30303030u);
  o.sc = h ? sc_hi : sc_lo;
  o.mn = h ? mn_hi : mn_lo;
  return o;
}

template <int R>
__device__ __forceinline__ void half_q4k_x2(const uint8_t* blkA, const uint8_t* blkB, int b, int h, const SmemView& s,
                                            float (&accA)[R], float (&accB)[R]) {
  const Q4KHalfScales mA = q4k_half_scales(blkA, h), mB = q4k_half_scales(blkB, h);
  float pA[R], pB[R];
#pragma unroll
  for (int r = 0; r < R; ++r) pA[r] = pB[r] = 0.f;
#pragma unroll
  for (int jj = 0; jj < 2; ++jj) {   // 64 weights: sub-block 2j in the low nibbles, 2j+1 in the high nibbles
    const int j = 2 * h + jj;
    const uint4 a0 = *reinterpret_cast<const uint4*>(blkA + 16 + j * 32);
    const uint4 a1 = *reinterpret_cast<const uint4*>(blkA + 32 + j * 32);
    const uint4 b0 = *reinterpret_cast<const uint4*>(blkB + 16 + j * 32);
    const uint4 b1 = *reinterpret_cast<const uint4*>(blkB + 32 + j * 32);
    const uint32_t qa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t qb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    const uint32_t scA = mA.sc >> (16 * jj), mnA = mA.mn >> (16 * jj);
    const uint32_t scB = mB.sc >> (16 * jj), mnB = mB.mn >> (16 * jj);
    const float ds0A = mA.dd.x * (float)(scA & 0xFFu), ds1A = mA.dd.x * 0.0625f * (float)((scA >> 8) & 0xFFu);
    const float dm0A = mA.dd.y * (float)(mnA & 0xFFu), dm1A = mA.dd.y * (float)((mnA >> 8) & 0xFFu);
    const float ds0B = mB.dd.x * (float)(scB & 0xFFu), ds1B = mB.dd.x * 0.0625f * (float)((scB >> 8) & 0xFFu);
    const float dm0B = mB.dd.y * (float)(mnB & 0xFFu), dm1B = mB.dd.y * (float)((mnB >> 8) & 0xFFu);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + 64 * j;
      const int4 xa = *reinterpret_cast<const int4*>(xb);
      const int4 xb1 = *reinterpret_cast<const int4*>(xb + 16);
      const int4 xc = *reinterpret_cast<const int4*>(xb + 32);
      const int4 xd = *reinterpret_cast<const int4*>(xb + 48);
      const int xl[8] = {xa.x, xa.y, xa.z, xa.w, xb1.x, xb1.y, xb1.z, xb1.w};
      const int xh[8] = {xc.x, xc.y, xc.z, xc.w, xd.x, xd.y, xd.z, xd.w};
      int dlA = 0, dhA = 0, dlB = 0, dhB = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dlA = __dp4a((int)(qa[i] & 0x0F0F0F0Fu), xl[i], dlA);
        dhA = dp4a_us(qa[i] & 0xF0F0F0F0u, xh[i], dhA);     // 16 * q, folded into ds1
        dlB = __dp4a((int)(qb[i] & 0x0F0F0F0Fu), xl[i], dlB);
        dhB = dp4a_us(qb[i] & 0xF0F0F0F0u, xh[i], dhB);
      }
      const float2 dx = *reinterpret_cast<const float2*>(s.dx + (size_t)r * s.sc_row + b * 8 + 2 * j);
      const float2 sx = *reinterpret_cast<const float2*>(s.sx + (size_t)r * s.sc_row + b * 8 + 2 * j);
      pA[r] += ds0A * dx.x * (float)dlA + ds1A * dx.y * (float)dhA - dm0A * sx.x - dm1A * sx.y;
      pB[r] += ds0B * dx.x * (float)dlB + ds1B * dx.y * (float)dhB - dm0B * sx.x - dm1B * sx.y;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    accA[r] += pA[r];
    accB[r] += pB[r];
  }
}

// The 16 six-bit values of positions l = 16*l16 .. +15 of quarter qt (0..3) of half `half`, minus 32, as int8 words.
__device__ __forceinline__ void q6k_unpack16(const uint8_t* blk, int half, int l16, uint32_t (&q)[4][4]) {
  const uint4 la = *reinterpret_cast<const uint4*>(blk + half * 64 + l16 * 16);
  const uint4 lb = *reinterpret_cast<const uint4*>(blk + half * 64 + 32 + l16 * 16);
  const uint4 hh = *reinterpret_cast<const uint4*>(blk + 128 + half * 32 + l16 * 16);
  const uint32_t lav[4] = {la.x, la.y, la.z, la.w}, lbv[4] = {lb.x, lb.y, lb.z, lb.w};
  const uint32_t hv[4] = {hh.x, hh.y, hh.z, hh.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    q[0][u] = __vsub4((lav[u] & 0x0F0F0F0Fu) | ((hv[u] & 0x03030303u) << 4), 0x20202020u);
    q[1][u] = __vsub4((lbv[u] & 0x0F0F0F0Fu) | (((hv[u] >> 2) & 0x03030303u) << 4), 0x20202020u);
    q[2][u] = __vsub4(((lav[u] >> 4) & 0x0F0F0F0Fu) | (((hv[u] >> 4) & 0x03030303u) << 4), 0x20202020u);
    q[3][u] = __vsub4(((lbv[u] >> 4) & 0x0F0F0F0Fu) | (((hv[u] >> 6) & 0x03030303u) << 4), 0x20202020u);
  }
}

template <int R>
__device__ __forceinline__ void half_q6k_x2(const uint8_t* blkA, const uint8_t* blkB, int b, int h, const SmemView& s,
                                            float (&accA)[R], float (&accB)[R]) {
  const uint4 scvA = *reinterpret_cast<const uint4*>(blkA + 192);
  const uint4 scvB = *reinterpret_cast<const uint4*>(blkB + 192);
  const float dA = __half2float(*reinterpret_cast<const __half*>(blkA + 208));
  const float dB = __half2float(*reinterpret_cast<const __half*>(blkB + 208));
#pragma unroll
  for (int l16 = 0; l16 < 2; ++l16) {
    uint32_t qA[4][4], qB[4][4];
    q6k_unpack16(blkA, h, l16, qA);
    q6k_unpack16(blkB, h, l16, qB);
    float dscA[4], dscB[4];
#pragma unroll
    for (int qt = 0; qt < 4; ++qt) {
      dscA[qt] = dA * (float)byte_of(scvA, h * 8 + 2 * qt + l16);
      dscB[qt] = dB * (float)byte_of(scvB, h * 8 + 2 * qt + l16);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + h * 128 + l16 * 16;
      const float4 dxq = *reinterpret_cast<const float4*>(s.dx + (size_t)r * s.sc_row + b * 8 + h * 4);
      const float dxa[4] = {dxq.x, dxq.y, dxq.z, dxq.w};
      float tA = 0.f, tB = 0.f;
#pragma unroll
      for (int qt = 0; qt < 4; ++qt) {
        const int4 xv = *reinterpret_cast<const int4*>(xb + 32 * qt);
        int da = __dp4a((int)qA[qt][0], xv.x, 0);
        da = __dp4a((int)qA[qt][1], xv.y, da);
        da = __dp4a((int)qA[qt][2], xv.z, da);
        da = __dp4a((int)qA[qt][3], xv.w, da);
        int db = __dp4a((int)qB[qt][0], xv.x, 0);
        db = __dp4a((int)qB[qt][1], xv.y, db);
        db = __dp4a((int)qB[qt][2], xv.z, db);
        db = __dp4a((int)qB[qt][3], xv.w, db);
        tA += dscA[qt] * dxa[qt] * (float)da;
        tB += dscB[qt] * dxa[qt] * (float)db;
      }
      accA[r] += tA;
      accB[r] += tB;
    }
  }
}

template <int R>
__device__ __forceinline__ void half_q80_x2(const uint8_t* qsA, const uint8_t* scA, const uint8_t* qsB,
                                            const uint8_t* scB, int b, int h, const SmemView& s, float (&accA)[R],
                                            float (&accB)[R]) {
  const uint2 svA = *reinterpret_cast<const uint2*>(scA + h * 8);   // the half's four fp16 scales
  const uint2 svB = *reinterpret_cast<const uint2*>(scB + h * 8);
  const __half2* shA = reinterpret_cast<const __half2*>(&svA);
  const __half2* shB = reinterpret_cast<const __half2*>(&svB);
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int sb = h * 4 + u;
    const uint4 a0 = *reinterpret_cast<const uint4*>(qsA + sb * 32);
    const uint4 a1 = *reinterpret_cast<const uint4*>(qsA + sb * 32 + 16);
    const uint4 b0 = *reinterpret_cast<const uint4*>(qsB + sb * 32);
    const uint4 b1 = *reinterpret_cast<const uint4*>(qsB + sb * 32 + 16);
    const float2 pa = __half22float2(shA[u >> 1]), pb = __half22float2(shB[u >> 1]);
    const float dA = (u & 1) ? pa.y : pa.x, dB = (u & 1) ? pb.y : pb.x;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xb = s.xq + (size_t)r * s.xq_row + (size_t)b * XQ_STRIDE + sb * 32;
      const int4 x0 = *reinterpret_cast<const int4*>(xb);
      const int4 x1 = *reinterpret_cast<const int4*>(xb + 16);
      int da = __dp4a((int)a0.x, x0.x, 0);
      da = __dp4a((int)a0.y, x0.y, da); da = __dp4a((int)a0.z, x0.z, da); da = __dp4a((int)a0.w, x0.w, da);
      da = __dp4a((int)a1.x, x1.x, da); da = __dp4a((int)a1.y, x1.y, da);
      da = __dp4a((int)a1.z, x1.z, da); da = __dp4a((int)a1.w, x1.w, da);
      int db = __dp4a((int)b0.x, x0.x, 0);
      db = __dp4a((int)b0.y, x0.y, db); db = __dp4a((int)b0.z, x0.z, db); db = __dp4a((int)b0.w, x0.w, db);
      db = __dp4a((int)b1.x, x1.x, db); db = __dp4a((int)b1.y, x1.y, db);
      db = __dp4a((int)b1.z, x1.z, db); db = __dp4a((int)b1.w, x1.w, db);
      const float dxv = s.dx[(size_t)r * s.sc_row + b * 8 + sb];
      accA[r] += dA * dxv * (float)da;
      accB[r] += dB * dxv * (float)db;
    }
  }
}

// ---------------------------------------------------------------- float weights: 256 elements at `w`
// Activations are re-read in fp32 from global memory (L1/L2 resident) with the RMSNorm applied on the fly, so
// the few F32 projections (router, ssm_alpha/beta) do not pay int8 activation rounding.
template <int R>
__device__ __forceinline__ void block_float(const uint8_t* w, int qtype, int b, const void* x, int x_dtype,
                                            long long x_stride, const float* norm_w, const SmemView& s,
                                            float (&acc)[R]) {
  for (int e = 0; e < 256; e += 4) {
    float wv[4];
    if (qtype == HE_F32) {
      const float4 f = *reinterpret_cast<const float4*>(w + (size_t)e * 4);
      wv[0] = f.x; wv[1] = f.y; wv[2] = f.z; wv[3] = f.w;
    } else {
      const uint2 u = *reinterpret_cast<const uint2*>(w + (size_t)e * 2);
      if (qtype == HE_BF16) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        wv[0] = a.x; wv[1] = a.y; wv[2] = c.x; wv[3] = c.y;
      } else {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        wv[0] = a.x; wv[1] = a.y; wv[2] = c.x; wv[3] = c.y;
      }
    }
    const int k = b * 256 + e;
    float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
    if (norm_w != nullptr) nw = __ldg(reinterpret_cast<const float4*>(norm_w + k));
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float xv[4];
      const size_t off = (size_t)r * x_stride + k;
      if (x_dtype == 0) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off));
        xv[0] = f.x; xv[1] = f.y; xv[2] = f.z; xv[3] = f.w;
      } else {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + off));
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        xv[0] = a.x; xv[1] = a.y; xv[2] = c.x; xv[3] = c.y;
      }
      const float ir = s.inv_rms[r];
      acc[r] += wv[0] * (xv[0] * ir * nw.x) + wv[1] * (xv[1] * ir * nw.y) + wv[2] * (xv[2] * ir * nw.z) +
                wv[3] * (xv[3] * ir * nw.w);
    }
  }
}

// Whole-warp dot product of one float-weight row (coalesced loads), partial sums left in acc[] of every lane.
template <int R>
__device__ __forceinline__ void row_float_coop(const uint8_t* w, int qtype, int K, const void* x, int x_dtype,
                                               long long x_stride, const float* norm_w, const SmemView& s, int lane,
                                               float (&acc)[R]) {
  for (int k = lane * 4; k < K; k += 128) {
    float wv[4];
    if (qtype == HE_F32) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(w + (size_t)k * 4));
      wv[0] = f.x; wv[1] = f.y; wv[2] = f.z; wv[3] = f.w;
    } else {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(w + (size_t)k * 2));
      if (qtype == HE_BF16) {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        wv[0] = a.x; wv[1] = a.y; wv[2] = c.x; wv[3] = c.y;
      } else {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        wv[0] = a.x; wv[1] = a.y; wv[2] = c.x; wv[3] = c.y;
      }
    }
    float4 nw = make_float4(1.f, 1.f, 1.f, 1.f);
    if (norm_w != nullptr) nw = __ldg(reinterpret_cast<const float4*>(norm_w + k));
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float xv[4];
      const size_t off = (size_t)r * x_stride + k;
      if (x_dtype == 0) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off));
        xv[0] = f.x; xv[1] = f.y; xv[2] = f.z; xv[3] = f.w;
      } else {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(x) + off));
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        xv[0] = a.x; xv[1] = a.y; xv[2] = c.x; xv[3] = c.y;
      }
      const float ir = s.inv_rms[r];
      acc[r] += wv[0] * (xv[0] * ir * nw.x) + wv[1] * (xv[1] * ir * nw.y) + wv[2] * (xv[2] * ir * nw.z) +
                wv[3] * (xv[3] * ir * nw.w);
    }
  }
}

}  // namespace hegemv
