// Quantized GEMV for decode (1..8 activation rows): Q4_K / Q6_K / Q8_0 / F32 / F16 / BF16 weights.
//
// One launch = [prologue] + [row loop] + [epilogue]:
//   prologue : every CTA loads the activation rows, optionally applies RMSNorm (fp32 statistics, weight
//              used directly), and quantizes them to int8 per 32 elements (scale d = amax/127 and the
//              block sum d*sum(q)) into shared memory.  Doing this per CTA removes two launches per
//              projection from the decode graph; the rows are tiny and L2-resident.
//   row loop : one warp per output row; 128-bit streaming loads of the weight bytes, nibble unpack in
//              registers, dp4a against the int8 activations, per-sub-block fp32 scaling.
//   epilogue : fp32/bf16 store, fp32 residual add in place, or act(gate)*up for gate/up pairs.
// Up to four weight segments (e.g. attn_qkv + attn_gate + ssm_alpha + ssm_beta) share one launch.
//
// Behavioural reference: the decode GEMV family in hipengine/kernels/hip_gfx1100/quant/gguf_q4_k_gemv.hip
// (Q8_1 activation quantize + integer dot) and the oracle hipengine/kernels/cpu_reference/ops.py:466-537.
//
// Device weight layouts ("repack"):
//   Q4_K : the 144-byte GGUF block is already 16-byte aligned -> used as stored.
//   Q6_K : planar  [ql: rows*nb*128][qh: rows*nb*64][sc: rows*nb*16][d: rows*nb*2]   (nb = K/256)
//   Q8_0 : planar  [qs: rows*K int8][d: rows*(K/32) fp16]
#include "common.cuh"

using namespace he;

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
  int need_xf;
};

namespace {

struct SmemView {
  int8_t* xq;
  float* dx;
  float* sx;
  float* xf;
};

__device__ __forceinline__ SmemView carve(uint8_t* smem, int R, int K, int need_xf) {
  SmemView v;
  v.xq = reinterpret_cast<int8_t*>(smem);
  v.dx = reinterpret_cast<float*>(smem + (size_t)R * K);
  v.sx = v.dx + (size_t)R * (K / 32);
  v.xf = need_xf ? v.sx + (size_t)R * (K / 32) : nullptr;
  return v;
}

__device__ __forceinline__ void load8(const void* x, int dtype, size_t off, float (&v)[8]) {
  if (dtype == 0) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + off);
    float4 a = p[0], b = p[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + off);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
}

// Activation prologue: (optional RMSNorm) + per-32 int8 quantisation into shared memory.
template <int R>
__device__ void prologue(const HeGemvArgs& a, const SmemView& s, float* red) {
  const int K = a.K;
  const int n_groups = K / 8;
  for (int r = 0; r < R; ++r) {
    float inv_rms = 1.f;
    const size_t base = (size_t)r * a.x_stride;
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
    for (int g0 = 0; g0 < n_groups; g0 += blockDim.x) {
      const int g = g0 + threadIdx.x;
      const bool valid = g < n_groups;
      float v[8];
      if (valid) {
        load8(a.x, a.x_dtype, base + (size_t)g * 8, v);
        if (a.norm_w != nullptr) {
          const float4* wp = reinterpret_cast<const float4*>(a.norm_w + (size_t)g * 8);
          float4 w0 = wp[0], w1 = wp[1];
          v[0] *= inv_rms * w0.x; v[1] *= inv_rms * w0.y; v[2] *= inv_rms * w0.z; v[3] *= inv_rms * w0.w;
          v[4] *= inv_rms * w1.x; v[5] *= inv_rms * w1.y; v[6] *= inv_rms * w1.z; v[7] *= inv_rms * w1.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
      }
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
        uint32_t p0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
        uint32_t p1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
        *reinterpret_cast<uint2*>(s.xq + (size_t)r * K + (size_t)g * 8) = make_uint2(p0, p1);
        if ((g & 3) == 0) {
          s.dx[(size_t)r * (K / 32) + (g >> 2)] = d;
          s.sx[(size_t)r * (K / 32) + (g >> 2)] = d * (float)qsum;
        }
        if (s.xf != nullptr) {
          float4* xp = reinterpret_cast<float4*>(s.xf + (size_t)r * K + (size_t)g * 8);
          xp[0] = make_float4(v[0], v[1], v[2], v[3]);
          xp[1] = make_float4(v[4], v[5], v[6], v[7]);
        }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ int dot16(const uint32_t (&w)[4], const int4& x) {
  int s = __dp4a((int)w[0], x.x, 0);
  s = __dp4a((int)w[1], x.y, s);
  s = __dp4a((int)w[2], x.z, s);
  s = __dp4a((int)w[3], x.w, s);
  return s;
}

// ---- per-row dot products (one warp per row; all lanes return partial sums in acc[])

template <int R>
__device__ __forceinline__ void row_q4k(const uint8_t* w, long long n, int K, const SmemView& s, int lane, float (&acc)[R]) {
  const int nb = K >> 8;
  const uint8_t* wrow = w + (size_t)n * nb * 144;
  const int c = lane & 7, j = c >> 1, h = c & 1;
  for (int b = lane >> 3; b < nb; b += 4) {
    const uint8_t* blk = wrow + (size_t)b * 144;
    const uint4 meta = ldg128_stream(blk);
    const uint4 qv = ldg128_stream(blk + 16 + c * 16);
    const float d = half_bits_to_f32((uint16_t)(meta.x & 0xffff));
    const float dmin = half_bits_to_f32((uint16_t)(meta.x >> 16));
    int sc0, m0, sc1, m1;
    k4_scale_min_w(meta.y, meta.z, meta.w, 2 * j, sc0, m0);
    k4_scale_min_w(meta.y, meta.z, meta.w, 2 * j + 1, sc1, m1);
    const uint32_t lo[4] = {qv.x & 0x0F0F0F0Fu, qv.y & 0x0F0F0F0Fu, qv.z & 0x0F0F0F0Fu, qv.w & 0x0F0F0F0Fu};
    const uint32_t hi[4] = {(qv.x >> 4) & 0x0F0F0F0Fu, (qv.y >> 4) & 0x0F0F0F0Fu, (qv.z >> 4) & 0x0F0F0F0Fu,
                            (qv.w >> 4) & 0x0F0F0F0Fu};
    const float ds0 = d * (float)sc0, ds1 = d * (float)sc1;
    const float dm0 = 0.5f * dmin * (float)m0, dm1 = 0.5f * dmin * (float)m1;
    const int e0 = b * 256 + 64 * j + 16 * h;
    const int sb = b * 8 + 2 * j;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xr = s.xq + (size_t)r * K;
      const int4 xl = *reinterpret_cast<const int4*>(xr + e0);
      const int4 xh = *reinterpret_cast<const int4*>(xr + e0 + 32);
      const float* dxr = s.dx + (size_t)r * (K >> 5);
      const float* sxr = s.sx + (size_t)r * (K >> 5);
      const int dl = dot16(lo, xl), dh = dot16(hi, xh);
      acc[r] += ds0 * dxr[sb] * (float)dl + ds1 * dxr[sb + 1] * (float)dh - dm0 * sxr[sb] - dm1 * sxr[sb + 1];
    }
  }
}

template <int R>
__device__ __forceinline__ void row_q6k(const uint8_t* w, long long n, long long n_total, int K, const SmemView& s,
                                        int lane, float (&acc)[R]) {
  const int nb = K >> 8;
  const size_t nblk = (size_t)n_total * nb;
  const uint8_t* ql = w;
  const uint8_t* qh = w + nblk * 128;
  const uint8_t* scp = w + nblk * 192;
  const uint16_t* dp = reinterpret_cast<const uint16_t*>(w + nblk * 208);
  const int l0 = (lane & 3) * 8, half = (lane >> 2) & 1;
  for (int b = lane >> 3; b < nb; b += 4) {
    const size_t gb = (size_t)n * nb + b;
    const uint2 la = ldg64_stream(ql + gb * 128 + half * 64 + l0);
    const uint2 lb = ldg64_stream(ql + gb * 128 + half * 64 + 32 + l0);
    const uint2 hh = ldg64_stream(qh + gb * 64 + half * 32 + l0);
    const uint4 scv = ldg128(scp + gb * 16);
    const float d = half_bits_to_f32(__ldg(dp + gb));
    uint32_t q[4][2];
    const uint32_t lav[2] = {la.x, la.y}, lbv[2] = {lb.x, lb.y}, hv[2] = {hh.x, hh.y};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      q[0][t] = __vsub4((lav[t] & 0x0F0F0F0Fu) | ((hv[t] & 0x03030303u) << 4), 0x20202020u);
      q[1][t] = __vsub4((lbv[t] & 0x0F0F0F0Fu) | (((hv[t] >> 2) & 0x03030303u) << 4), 0x20202020u);
      q[2][t] = __vsub4(((lav[t] >> 4) & 0x0F0F0F0Fu) | (((hv[t] >> 4) & 0x03030303u) << 4), 0x20202020u);
      q[3][t] = __vsub4(((lbv[t] >> 4) & 0x0F0F0F0Fu) | (((hv[t] >> 6) & 0x03030303u) << 4), 0x20202020u);
    }
    const int sidx = half * 8 + (l0 >> 4);
    float dsc[4];
#pragma unroll
    for (int qt = 0; qt < 4; ++qt) dsc[qt] = d * (float)byte_of(scv, sidx + 2 * qt);
    const int e0 = b * 256 + half * 128 + l0;
    const int sb = b * 8 + half * 4;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int8_t* xr = s.xq + (size_t)r * K + e0;
      const float* dxr = s.dx + (size_t)r * (K >> 5) + sb;
      float t = 0.f;
#pragma unroll
      for (int qt = 0; qt < 4; ++qt) {
        const int2 xv = *reinterpret_cast<const int2*>(xr + 32 * qt);
        int dsum = __dp4a((int)q[qt][0], xv.x, 0);
        dsum = __dp4a((int)q[qt][1], xv.y, dsum);
        t += dsc[qt] * dxr[qt] * (float)dsum;
      }
      acc[r] += t;
    }
  }
}

template <int R>
__device__ __forceinline__ void row_q80(const uint8_t* w, long long n, long long n_total, int K, const SmemView& s,
                                        int lane, float (&acc)[R]) {
  const int8_t* qs = reinterpret_cast<const int8_t*>(w) + (size_t)n * K;
  const uint16_t* dp = reinterpret_cast<const uint16_t*>(w + (size_t)n_total * K) + (size_t)n * (K >> 5);
  for (int e0 = lane * 16; e0 < K; e0 += 512) {
    const uint4 qv = ldg128_stream(qs + e0);
    const float d = half_bits_to_f32(__ldg(dp + (e0 >> 5)));
    const uint32_t wv[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int4 xv = *reinterpret_cast<const int4*>(s.xq + (size_t)r * K + e0);
      acc[r] += d * s.dx[(size_t)r * (K >> 5) + (e0 >> 5)] * (float)dot16(wv, xv);
    }
  }
}

template <int R>
__device__ __forceinline__ void row_float(const void* w, int qtype, long long n, int K, const SmemView& s, int lane,
                                          float (&acc)[R]) {
  if (qtype == HE_F32) {
    const float* wr = reinterpret_cast<const float*>(w) + (size_t)n * K;
    for (int e0 = lane * 4; e0 < K; e0 += 128) {
      const float4 wv = __ldg(reinterpret_cast<const float4*>(wr + e0));
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float4 xv = *reinterpret_cast<const float4*>(s.xf + (size_t)r * K + e0);
        acc[r] += wv.x * xv.x + wv.y * xv.y + wv.z * xv.z + wv.w * xv.w;
      }
    }
  } else {
    const uint16_t* wr = reinterpret_cast<const uint16_t*>(w) + (size_t)n * K;
    for (int e0 = lane * 8; e0 < K; e0 += 256) {
      const uint4 u = ldg128_stream(wr + e0);
      float wv[8];
      if (qtype == HE_BF16) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); wv[2 * i] = f.x; wv[2 * i + 1] = f.y; }
      } else {
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); wv[2 * i] = f.x; wv[2 * i + 1] = f.y; }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const float* xv = s.xf + (size_t)r * K + e0;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r] += wv[i] * xv[i];
      }
    }
  }
}

template <int R>
__device__ __forceinline__ void row_dot(const void* w, int qtype, long long n, long long n_total, int K,
                                        const SmemView& s, int lane, float (&acc)[R]) {
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.f;
  switch (qtype) {
    case HE_Q4_K: row_q4k<R>(reinterpret_cast<const uint8_t*>(w), n, K, s, lane, acc); break;
    case HE_Q6_K: row_q6k<R>(reinterpret_cast<const uint8_t*>(w), n, n_total, K, s, lane, acc); break;
    case HE_Q8_0: row_q80<R>(reinterpret_cast<const uint8_t*>(w), n, n_total, K, s, lane, acc); break;
    default: row_float<R>(w, qtype, n, K, s, lane, acc); break;
  }
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = warp_sum(acc[r]);
}

template <int R>
__global__ void __launch_bounds__(256) gemv_kernel(const __grid_constant__ HeGemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float red[33];
  const SmemView s = carve(smem, R, a.K, a.need_xf);
  prologue<R>(a, s, red);

  const int lane = threadIdx.x & 31;
  const int warps_per_cta = blockDim.x >> 5;
  const long long total_warps = (long long)gridDim.x * warps_per_cta;
  long long total_rows = 0;
  for (int i = 0; i < a.n_seg; ++i) total_rows += a.seg[i].n_rows;

  for (long long g = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); g < total_rows; g += total_warps) {
    long long n = g;
    int si = 0;
    while (si < a.n_seg - 1 && n >= a.seg[si].n_rows) { n -= a.seg[si].n_rows; ++si; }
    const HeGemvSeg& sg = a.seg[si];
    float acc[R];
    row_dot<R>(sg.w, sg.qtype, n, sg.n_rows, a.K, s, lane, acc);
    if (sg.epi >= 3) {
      float acc2[R];
      row_dot<R>(sg.w2, sg.qtype2, n, sg.n_rows, a.K, s, lane, acc2);
      if (lane == 0) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(sg.out);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float gte = sg.epi == 3 ? silu_f(acc[r]) : gelu_tanh_f(acc[r]);
          o[(size_t)r * sg.out_stride + n] = f32_to_bf16(gte * acc2[r]);
        }
      }
    } else if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const size_t off = (size_t)r * sg.out_stride + n;
        if (sg.epi == 0) reinterpret_cast<float*>(sg.out)[off] = acc[r];
        else if (sg.epi == 1) reinterpret_cast<__nv_bfloat16*>(sg.out)[off] = f32_to_bf16(acc[r]);
        else reinterpret_cast<float*>(sg.out)[off] += acc[r];
      }
    }
  }
}

template <int R>
int launch_gemv(const HeGemvArgs& a, int num_sms, cudaStream_t stream) {
  size_t smem = (size_t)R * a.K + (size_t)R * (a.K / 32) * 8 + (a.need_xf ? (size_t)R * a.K * 4 : 0);
  long long total_rows = 0;
  for (int i = 0; i < a.n_seg; ++i) total_rows += a.seg[i].n_rows;
  static int configured_smem[9] = {0};
  if ((int)smem > configured_smem[R]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured_smem[R] = (int)smem;
  }
  int ctas_per_sm = (int)((200 * 1024) / (smem + 1024));
  if (ctas_per_sm > 8) ctas_per_sm = 8;
  if (ctas_per_sm < 1) ctas_per_sm = 1;
  long long want = (total_rows + 7) / 8;
  long long grid = (long long)num_sms * ctas_per_sm;
  if (grid > want) grid = want;
  if (grid < 1) grid = 1;
  gemv_kernel<R><<<(unsigned)grid, 256, smem, stream>>>(a);
  HE_LAUNCH_CHECK();
  return 0;
}

}  // namespace

// Launch the fused GEMV.  `args` is a host pointer to HeGemvArgs (copied by value into the launch).
HE_API int he_gemv(const HeGemvArgs* args, int num_sms, cudaStream_t stream) {
  const HeGemvArgs& a = *args;
  if (a.K % 32 != 0 || a.n_seg < 1 || a.n_seg > 4 || a.R < 1 || a.R > 8) return -HE_ERR_BAD_ARG;
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

// ------------------------------------------------------------------------------------------------
// Repack kernels: GGUF row-major blocks -> planar device layouts (and nothing for Q4_K).

__global__ void repack_q6k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, long long nblk) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (block, 2-byte unit)
  const long long b = i / 105;
  const int u = (int)(i % 105);
  if (b >= nblk) return;
  const uint8_t* src = raw + b * 210 + u * 2;
  const int off = u * 2;
  uint8_t* dst;
  if (off < 128) dst = out + b * 128 + off;
  else if (off < 192) dst = out + nblk * 128 + b * 64 + (off - 128);
  else if (off < 208) dst = out + nblk * 192 + b * 16 + (off - 192);
  else dst = out + nblk * 208 + b * 2;
  dst[0] = src[0];
  dst[1] = src[1];
}

__global__ void repack_q80_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, long long nblk) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (block, 2-byte unit)
  const long long b = i / 17;
  const int u = (int)(i % 17);
  if (b >= nblk) return;
  const uint8_t* src = raw + b * 34 + u * 2;
  uint8_t* dst = (u == 0) ? out + nblk * 32 + b * 2 : out + b * 32 + (u - 1) * 2;
  dst[0] = src[0];
  dst[1] = src[1];
}

HE_API int he_repack(const void* raw, void* out, int qtype, long long rows, long long K, cudaStream_t stream) {
  if (qtype == HE_Q6_K) {
    const long long nblk = rows * (K / 256), n = nblk * 105;
    repack_q6k_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nblk);
  } else if (qtype == HE_Q8_0) {
    const long long nblk = rows * (K / 32), n = nblk * 17;
    repack_q80_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)raw, (uint8_t*)out, nblk);
  } else {
    return -HE_ERR_BAD_ARG;
  }
  HE_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Dequantize device-layout weights to bf16 [rows][K] (B operand of the tensor-core GEMM) and
// embedding-row gather (token ids -> fp32 hidden rows).

__device__ __forceinline__ float dequant_elem(const uint8_t* w, int qtype, long long n, long long n_total, int K,
                                              int e) {
  if (qtype == HE_Q4_K) {
    const uint8_t* blk = w + ((size_t)n * (K >> 8) + (e >> 8)) * 144;
    const int ib = e & 255, sb = ib >> 5, l = ib & 31;
    int sc, m;
    k4_scale_min(blk + 4, sb, sc, m);
    const float d = half_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
    const float dmin = half_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2));
    const uint8_t byte = blk[16 + (sb >> 1) * 32 + l];
    const int q = (sb & 1) ? (byte >> 4) : (byte & 15);
    return (d * (float)sc) * (float)q - dmin * (float)m;
  } else if (qtype == HE_Q6_K) {
    const int nb = K >> 8;
    const size_t nblk = (size_t)n_total * nb, gb = (size_t)n * nb + (e >> 8);
    const int ib = e & 255, half = ib >> 7, qt = (ib & 127) >> 5, l = ib & 31;
    const uint8_t lq = w[gb * 128 + half * 64 + (qt & 1) * 32 + l];
    const uint8_t hq = w[nblk * 128 + gb * 64 + half * 32 + l];
    const int lo = (qt >= 2) ? (lq >> 4) : (lq & 15);
    const int hi = (hq >> (2 * qt)) & 3;
    const int q = (lo | (hi << 4)) - 32;
    const int8_t sc = reinterpret_cast<const int8_t*>(w + nblk * 192)[gb * 16 + half * 8 + 2 * qt + (l >> 4)];
    const float d = half_bits_to_f32(reinterpret_cast<const uint16_t*>(w + nblk * 208)[gb]);
    return (d * (float)sc) * (float)q;
  } else if (qtype == HE_Q8_0) {
    const int8_t q = reinterpret_cast<const int8_t*>(w)[(size_t)n * K + e];
    const float d = half_bits_to_f32(
        reinterpret_cast<const uint16_t*>(w + (size_t)n_total * K)[(size_t)n * (K >> 5) + (e >> 5)]);
    return d * (float)q;
  } else if (qtype == HE_F32) {
    return reinterpret_cast<const float*>(w)[(size_t)n * K + e];
  } else if (qtype == HE_BF16) {
    return bf16_to_f32(reinterpret_cast<const __nv_bfloat16*>(w)[(size_t)n * K + e]);
  } else {
    return __half2float(reinterpret_cast<const __half*>(w)[(size_t)n * K + e]);
  }
}

__global__ void dequant_bf16_kernel(const uint8_t* __restrict__ w, __nv_bfloat16* __restrict__ out, int qtype,
                                    long long row0, long long rows, long long n_total, int K) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= rows * K) return;
  const long long n = i / K;
  const int e = (int)(i % K);
  __align__(16) __nv_bfloat16 v[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) v[t] = f32_to_bf16(dequant_elem(w, qtype, row0 + n, n_total, K, e + t));
  *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(v);
}

// Dequantize rows [row0, row0+rows) of a device-layout weight with `n_total` rows into bf16 [rows][K].
HE_API int he_dequant_bf16(const void* w, void* out, int qtype, long long row0, long long rows, long long n_total,
                           int K, cudaStream_t stream) {
  if (K % 8 != 0) return -HE_ERR_BAD_ARG;
  const long long n = rows * K / 8;
  dequant_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)w, (__nv_bfloat16*)out, qtype,
                                                                        row0, rows, n_total, K);
  HE_LAUNCH_CHECK();
  return 0;
}

__global__ void embed_kernel(const uint8_t* __restrict__ w, int qtype, long long vocab, int K,
                             const int64_t* __restrict__ ids, float* __restrict__ out, float scale, int n_tok) {
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  long long id = ids[t];
  if (id < 0 || id >= vocab) id = 0;
  for (int e = threadIdx.x; e < K; e += blockDim.x)
    out[(size_t)t * K + e] = dequant_elem(w, qtype, id, vocab, K, e) * scale;
}

// out[t][:] = dequant(table[ids[t]]) * scale   (fp32 residual stream rows)
HE_API int he_embed(const void* w, int qtype, long long vocab, int K, const void* ids, void* out, float scale,
                    int n_tok, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  embed_kernel<<<n_tok, 256, 0, stream>>>((const uint8_t*)w, qtype, vocab, K, (const int64_t*)ids, (float*)out, scale,
                                          n_tok);
  HE_LAUNCH_CHECK();
  return 0;
}
