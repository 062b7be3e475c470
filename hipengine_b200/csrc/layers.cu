// Row-wise layer glue: RMSNorm, activation*mul, fused split-Q|gate + QK-RMSNorm + partial RoPE + paged
// KV write, causal conv1d + SiLU with rolling state, embedding-free bookkeeping kernels.
//
// Behavioural references: hipengine/kernels/hip_gfx1100/fused/gguf_ops.hip (GGUF F32-weight RMSNorm,
// fused split-qgate + head RMSNorm + partial rotary), attention/paged_kv_write.hip (append K/V through
// the live-span block table), linear_attn/conv.hip (depthwise causal conv, kernel 4, rolling state),
// runtime/state.hip (device-side position bookkeeping so a decode step can live in one graph).
#include "common.cuh"

using namespace he;

namespace {

// ---------------------------------------------------------------- RMSNorm rows: fp32 [T][H] -> bf16/f32 [T][H]
template <typename OutT>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           OutT* __restrict__ out, int H, float eps,
                                                           long long x_stride, long long out_stride) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  __shared__ float red[33];
  const float* xr = x + (size_t)blockIdx.x * x_stride;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  OutT* orow = out + (size_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
    if (w != nullptr) g = *reinterpret_cast<const float4*>(w + i);
    const float o0 = v.x * inv * g.x, o1 = v.y * inv * g.y, o2 = v.z * inv * g.z, o3 = v.w * inv * g.w;
    if constexpr (sizeof(OutT) == 2) {
      __nv_bfloat162 a = __floats2bfloat162_rn(o0, o1), b = __floats2bfloat162_rn(o2, o3);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&a);
      pk.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(orow + i) = pk;
    } else {
      *reinterpret_cast<float4*>(orow + i) = make_float4(o0, o1, o2, o3);
    }
  }
}

// ---------------------------------------------------------------- act(gate) * up over packed [T][2F] bf16 -> [T][F] bf16
__global__ void act_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T,
                               int F, int act) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= T * F) return;
  const long long t = i / F;
  const int f = (int)(i % F);
  const uint4 gv = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + f);
  const uint4 uv = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + F + f);
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
  __align__(16) __nv_bfloat162 o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 g = __bfloat1622float2(g2[k]), u = __bfloat1622float2(u2[k]);
    const float a0 = act == 0 ? silu_f(g.x) : gelu_tanh_f(g.x);
    const float a1 = act == 0 ? silu_f(g.y) : gelu_tanh_f(g.y);
    o[k] = __floats2bfloat162_rn(a0 * u.x, a1 * u.y);
  }
  *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(o);
}

// same with the packed gate | up rows in fp32 (split-K accumulators of small batches)
__global__ void act_mul_f32_kernel(const float* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long T, int F,
                                   int act) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= T * F) return;
  const long long t = i / F;
  const int f = (int)(i % F);
  const float4 g = *reinterpret_cast<const float4*>(gu + (size_t)t * 2 * F + f);
  const float4 u = *reinterpret_cast<const float4*>(gu + (size_t)t * 2 * F + F + f);
  const float gx[4] = {g.x, g.y, g.z, g.w}, ux[4] = {u.x, u.y, u.z, u.w};
  __align__(8) __nv_bfloat162 o[2];
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const float a0 = act == 0 ? silu_f(gx[2 * k]) : gelu_tanh_f(gx[2 * k]);
    const float a1 = act == 0 ? silu_f(gx[2 * k + 1]) : gelu_tanh_f(gx[2 * k + 1]);
    o[k] = __floats2bfloat162_rn(a0 * ux[2 * k], a1 * ux[2 * k + 1]);
  }
  *reinterpret_cast<uint2*>(out + i) = *reinterpret_cast<const uint2*>(o);
}

// ---------------------------------------------------------------- residual add: h (fp32) += y (bf16)
__global__ void resid_add_bf16_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ y, long long n) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 hv = *reinterpret_cast<float4*>(h + i);
  const uint2 yv = *reinterpret_cast<const uint2*>(y + i);
  const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&yv);
  const float2 a = __bfloat1622float2(y2[0]), b = __bfloat1622float2(y2[1]);
  hv.x += a.x; hv.y += a.y; hv.z += b.x; hv.w += b.y;
  *reinterpret_cast<float4*>(h + i) = hv;
}

// ---------------------------------------------------------------- fused QK-norm + partial RoPE + KV write
struct QkvArgs {
  const void* q;      // [T][q_stride]: per head [Q(D) | gate(D)] when gated, else [Q(D)]
  const void* k;      // [T][k_stride]
  const void* v;      // [T][v_stride]
  int in_dtype;       // 0 f32, 1 bf16
  long long q_stride, k_stride, v_stride;
  const float* q_norm;   // [D] or null
  const float* k_norm;   // [D] or null
  int v_norm;            // 1: weightless RMSNorm on V (Gemma)
  __nv_bfloat16* q_out;    // [T][H][D]
  __nv_bfloat16* gate_out; // [T][H][D] or null
  __nv_bfloat16* kv_cache; // [n_pages][2][Hkv][PAGE][D]
  const int* block_table;  // [n_slots][max_pages]
  const int* slot;         // [T] row of block_table per token
  const int* pos;          // [T] absolute position
  int max_pages;
  int H, Hkv, D, page;
  int gated;
  int rope_dim;
  float theta;
  float eps;
  float q_scale;           // multiplied into Q after norm/rope (1 = none)
  int rope_denom;          // frequency spacing: inv_freq_i = theta^(-2i / rope_denom); 0 -> rope_dim
};

__device__ __forceinline__ float load_in(const void* p, int dtype, size_t i) {
  return dtype == 0 ? reinterpret_cast<const float*>(p)[i] : bf16_to_f32(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// grid (T, H + 2*Hkv); block D threads (D <= 512, multiple of 32)
__global__ void qkv_post_kernel(const QkvArgs a) {
  extern __shared__ float sh[];  // [D]
  __shared__ float red[33];
  const int t = blockIdx.x, hh = blockIdx.y, d = threadIdx.x;
  const int D = a.D;
  pdl_wait();
  pdl_launch();
  int kind, h;  // 0 q, 1 k, 2 v
  if (hh < a.H) { kind = 0; h = hh; }
  else if (hh < a.H + a.Hkv) { kind = 1; h = hh - a.H; }
  else { kind = 2; h = hh - a.H - a.Hkv; }
  float x;
  if (kind == 0) x = load_in(a.q, a.in_dtype, (size_t)t * a.q_stride + (size_t)h * D * (a.gated ? 2 : 1) + d);
  else if (kind == 1) x = load_in(a.k, a.in_dtype, (size_t)t * a.k_stride + (size_t)h * D + d);
  else x = load_in(a.v, a.in_dtype, (size_t)t * a.v_stride + (size_t)h * D + d);

  const float* nw = kind == 0 ? a.q_norm : (kind == 1 ? a.k_norm : nullptr);
  const bool do_norm = (kind < 2 && nw != nullptr) || (kind == 2 && a.v_norm);
  if (do_norm) {
    const float ss = block_sum(x * x, red);
    x = x * rsqrtf(ss / (float)D + a.eps);
    if (nw != nullptr) x *= nw[d];
  }
  const int p = a.pos[t];
  if (kind < 2 && a.rope_dim > 0) {
    sh[d] = x;
    __syncthreads();
    const int half = a.rope_dim >> 1;
    if (d < a.rope_dim) {
      const int i = d < half ? d : d - half;
      const float inv_freq = powf(a.theta, -2.0f * (float)i / (float)(a.rope_denom > 0 ? a.rope_denom : a.rope_dim));
      float sn, cs;
      sincosf((float)p * inv_freq, &sn, &cs);
      const float other = sh[d < half ? d + half : d - half];
      x = d < half ? x * cs - other * sn : x * cs + other * sn;
    }
  }
  if (kind == 0) {
    a.q_out[((size_t)t * a.H + h) * D + d] = f32_to_bf16(x * a.q_scale);
    if (a.gated && a.gate_out != nullptr) {
      const float g = load_in(a.q, a.in_dtype, (size_t)t * a.q_stride + (size_t)h * D * 2 + D + d);
      a.gate_out[((size_t)t * a.H + h) * D + d] = f32_to_bf16(g);
    }
  } else {
    const int s = a.slot[t];
    if (!HE_INDEX_OK(p / a.page, a.max_pages, HE_SITE_KV_WRITE_PAGE)) return;
    const int page_id = a.block_table[(size_t)s * a.max_pages + p / a.page];
    const size_t off = ((((size_t)page_id * 2 + (kind - 1)) * a.Hkv + h) * a.page + (p % a.page)) * D + d;
    a.kv_cache[off] = f32_to_bf16(x);
  }
}

// ---------------------------------------------------------------- causal conv1d (k<=4) + SiLU with rolling state
struct ConvArgs {
  const void* x;        // [T][x_stride] (first C columns used)
  int in_dtype;
  long long x_stride;
  const float* w;       // [C][KW]
  float* state;         // [n_slots][C][KW-1]  (oldest first)
  const int* seg_start; // [n_seg+1] cumulative token offsets
  const int* seg_slot;  // [n_seg]
  const int* tok_seg;   // [T] segment of each token
  float* out;           // [T][C] fp32
  float* journal;       // optional [T][C][KW-1]: state after each token (verify chains), else null
  int C, KW, T, n_seg;
};

// one thread per (8 channels, CONV_TOK consecutive tokens); the 8 x KW filter taps are loaded once per thread
// and reused for all its tokens (they used to dominate the load traffic at one token per thread).
constexpr int CONV_TOK = 8;
template <int KWT>
__global__ void __launch_bounds__(256) conv_fwd_kernel(const ConvArgs a) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const int C8 = a.C >> 3;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int n_tchunks = (a.T + CONV_TOK - 1) / CONV_TOK;
  if (i >= (long long)n_tchunks * C8) return;
  const int t_first = (int)(i / C8) * CONV_TOK, c = (int)(i % C8) * 8;
  constexpr int KW = KWT;
  float wreg[8][KW];
  if constexpr (KW == 4) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float4 w4 = __ldg(reinterpret_cast<const float4*>(a.w + (size_t)(c + e) * 4));
      wreg[e][0] = w4.x; wreg[e][1] = w4.y; wreg[e][2] = w4.z; wreg[e][3] = w4.w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
#pragma unroll
      for (int k = 0; k < KW; ++k) wreg[e][k] = __ldg(a.w + (size_t)(c + e) * KW + k);
  }
  const int t_last = min(a.T, t_first + CONV_TOK);
  for (int t = t_first; t < t_last; ++t) {
    const int sg = a.tok_seg[t];
    const int s0 = a.seg_start[sg];
    const int local = t - s0;
    const float* st = a.state + ((size_t)a.seg_slot[sg] * a.C + c) * (KW - 1);
    float acc[8], win[KW][8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < KW; ++k) {
      const int idx = local + k;  // index into [state(KW-1) ++ x_seg]
      if (idx < KW - 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[k][e] = st[(size_t)e * (KW - 1) + idx];
      } else {
        const size_t off = (size_t)(s0 + idx - (KW - 1)) * a.x_stride + c;
        if (a.in_dtype == 0) {
          const float4 v0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + off);
          const float4 v1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.x) + off + 4);
          win[k][0] = v0.x; win[k][1] = v0.y; win[k][2] = v0.z; win[k][3] = v0.w;
          win[k][4] = v1.x; win[k][5] = v1.y; win[k][6] = v1.z; win[k][7] = v1.w;
        } else {
          const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.x) + off);
          const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h2[e]);
            win[k][2 * e] = f.x; win[k][2 * e + 1] = f.y;
          }
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += win[k][e] * wreg[e][k];
    }
    float* o = a.out + (size_t)t * a.C + c;
    *reinterpret_cast<float4*>(o) = make_float4(silu_f(acc[0]), silu_f(acc[1]), silu_f(acc[2]), silu_f(acc[3]));
    *reinterpret_cast<float4*>(o + 4) = make_float4(silu_f(acc[4]), silu_f(acc[5]), silu_f(acc[6]), silu_f(acc[7]));
    if (a.journal != nullptr) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float* j = a.journal + ((size_t)t * a.C + c + e) * (KW - 1);
#pragma unroll
        for (int k = 1; k < KW; ++k) j[k - 1] = win[k][e];
      }
    }
  }
}

// one thread per (segment, channel): new state = last KW-1 entries of [state ++ x_seg]
__global__ void conv_state_kernel(const ConvArgs a) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)a.n_seg * a.C) return;
  const int sg = (int)(i / a.C), c = (int)(i % a.C);
  const int s0 = a.seg_start[sg], n = a.seg_start[sg + 1] - s0;
  const int KW = a.KW;
  float* st = a.state + ((size_t)a.seg_slot[sg] * a.C + c) * (KW - 1);
  float nv[3];
  for (int j = 0; j < KW - 1; ++j) {
    const int idx = n + j;
    nv[j] = idx < KW - 1 ? st[idx] : load_in(a.x, a.in_dtype, (size_t)(s0 + idx - (KW - 1)) * a.x_stride + c);
  }
  for (int j = 0; j < KW - 1; ++j) st[j] = nv[j];
}

// ---------------------------------------------------------------- bookkeeping
__global__ void advance_positions_kernel(int* pos, int* ctx_len, const int* active, int n, int delta) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  if (active == nullptr || active[i]) {
    pos[i] += delta;
    if (ctx_len != nullptr) ctx_len[i] += delta;
  }
}

}  // namespace

HE_API int he_rmsnorm_rows(const void* x, const void* w, void* out, int out_bf16, int T, int H, float eps,
                           long long x_stride, long long out_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 4 != 0) return -HE_ERR_BAD_ARG;
  if (out_bf16)
    (void)launch_pdl(rmsnorm_rows_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, (const float*)x, (const float*)w, (__nv_bfloat16*)out, H,
                                                              eps, x_stride, out_stride);
  else
    (void)launch_pdl(rmsnorm_rows_kernel<float>, dim3(T), dim3(256), 0, stream, (const float*)x, (const float*)w, (float*)out, H, eps, x_stride,
                                                      out_stride);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_act_mul(const void* gu, void* out, long long T, int F, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F % 8 != 0) return -HE_ERR_BAD_ARG;
  const long long n = T * F / 8;
  (void)launch_pdl(act_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F,
                                                                   act);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_act_mul_f32(const void* gu, void* out, long long T, int F, int act, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F % 4 != 0) return -HE_ERR_BAD_ARG;
  const long long n = T * F / 4;
  (void)launch_pdl(act_mul_f32_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, (const float*)gu, (__nv_bfloat16*)out, T, F, act);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_resid_add_bf16(void* h, const void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0) return -HE_ERR_BAD_ARG;
  (void)launch_pdl(resid_add_bf16_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, (float*)h, (const __nv_bfloat16*)y, n);
  HE_LAUNCH_CHECK();
  return 0;
}

__global__ void resid_add_f32_kernel(float* __restrict__ h, const float* __restrict__ y, long long n) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 a = *reinterpret_cast<float4*>(h + i);
  const float4 b = *reinterpret_cast<const float4*>(y + i);
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  *reinterpret_cast<float4*>(h + i) = a;
}

// h[i] += y[i] (fp32, contiguous, n % 4 == 0): residual add after a reduced row-parallel projection
HE_API int he_resid_add_f32(void* h, const void* y, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 != 0) return -HE_ERR_BAD_ARG;
  (void)launch_pdl(resid_add_f32_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, stream, (float*)h, (const float*)y, n);
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------- sandwich-norm residual updates (Gemma)
// h[t] += RMSNorm(y[t]) * w        (y fp32 or bf16; one CTA per row)
__global__ void __launch_bounds__(256) norm_add_kernel(float* __restrict__ h, long long ldh, const void* __restrict__ y,
                                                       int y_dtype, long long ldy, const float* __restrict__ w, int H,
                                                       float eps) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  __shared__ float red[33];
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float v = load_in(y, y_dtype, (size_t)t * ldy + i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += 256)
    h[(size_t)t * ldh + i] += load_in(y, y_dtype, (size_t)t * ldy + i) * inv * w[i];
}

// h[t] = (h[t] + RMSNorm(RMSNorm(d[t])*w1 + RMSNorm(e[t])*w2) * w3) * scalar[0]
// d: dense-branch output, e: expert-branch output (either fp32 or bf16).
__global__ void __launch_bounds__(256) ffn_combine_kernel(float* __restrict__ h, long long ldh,
                                                          const void* __restrict__ d, int d_dtype, long long ldd,
                                                          const void* __restrict__ e, int e_dtype, long long lde,
                                                          const float* __restrict__ w1, const float* __restrict__ w2,
                                                          const float* __restrict__ w3,
                                                          const float* __restrict__ scalar, int H, float eps) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  extern __shared__ float buf[];   // [H]
  __shared__ float red[33];
  const int t = blockIdx.x;
  float sd = 0.f, se = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float a = load_in(d, d_dtype, (size_t)t * ldd + i), b = load_in(e, e_dtype, (size_t)t * lde + i);
    sd += a * a; se += b * b;
  }
  sd = block_sum(sd, red);
  se = block_sum(se, red);
  const float id = rsqrtf(sd / (float)H + eps), ie = rsqrtf(se / (float)H + eps);
  float sc = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    const float c = load_in(d, d_dtype, (size_t)t * ldd + i) * id * w1[i] +
                    load_in(e, e_dtype, (size_t)t * lde + i) * ie * w2[i];
    buf[i] = c;
    sc += c * c;
  }
  sc = block_sum(sc, red);
  const float ic = rsqrtf(sc / (float)H + eps);
  const float s = scalar != nullptr ? scalar[0] : 1.f;
  for (int i = threadIdx.x; i < H; i += 256)
    h[(size_t)t * ldh + i] = (h[(size_t)t * ldh + i] + buf[i] * ic * w3[i]) * s;
}

HE_API int he_norm_add(void* h, long long ldh, const void* y, int y_dtype, long long ldy, const void* w, int T, int H,
                       float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  (void)launch_pdl(norm_add_kernel, dim3(T), dim3(256), 0, stream, (float*)h, ldh, y, y_dtype, ldy, (const float*)w, H, eps);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_ffn_combine(void* h, long long ldh, const void* d, int d_dtype, long long ldd, const void* e, int e_dtype,
                          long long lde, const void* w1, const void* w2, const void* w3, const void* scalar, int T,
                          int H, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((size_t)H * sizeof(float) > 48 * 1024) return -HE_ERR_BAD_ARG;
  (void)launch_pdl(ffn_combine_kernel, dim3(T), dim3(256), (size_t)H * sizeof(float), stream, (float*)h, ldh, d, d_dtype, ldd, e, e_dtype, lde,
                                                                    (const float*)w1, (const float*)w2,
                                                                    (const float*)w3, (const float*)scalar, H, eps);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_qkv_post(const QkvArgs* args, int T, cudaStream_t stream) {
  const QkvArgs& a = *args;
  if (T <= 0) return 0;
  if (a.D % 32 != 0 || a.D > 512) return -HE_ERR_BAD_ARG;
  dim3 grid(T, a.H + 2 * a.Hkv);
  cudaError_t le = launch_pdl(qkv_post_kernel, grid, dim3(a.D), a.D * sizeof(float), stream, a);
  if (le != cudaSuccess) return (int)le;
  return 0;
}
HE_API int he_qkv_args_size() { return (int)sizeof(QkvArgs); }

HE_API int he_conv1d(const ConvArgs* args, int update_state, cudaStream_t stream) {
  const ConvArgs& a = *args;
  if (a.T <= 0) return 0;
  if (a.KW < 2 || a.KW > 4) return -HE_ERR_BAD_ARG;
  if (a.C % 8 != 0) return -HE_ERR_BAD_ARG;
  const long long n = (long long)((a.T + CONV_TOK - 1) / CONV_TOK) * (a.C / 8);
  const unsigned nblk = (unsigned)((n + 255) / 256);
  if (a.KW == 4) (void)launch_pdl(conv_fwd_kernel<4>, dim3(nblk), dim3(256), 0, stream, a);
  else if (a.KW == 3) (void)launch_pdl(conv_fwd_kernel<3>, dim3(nblk), dim3(256), 0, stream, a);
  else (void)launch_pdl(conv_fwd_kernel<2>, dim3(nblk), dim3(256), 0, stream, a);
  HE_LAUNCH_CHECK();
  if (update_state) {
    const long long m = (long long)a.n_seg * a.C;
    (void)launch_pdl(conv_state_kernel, dim3((unsigned)((m + 255) / 256)), dim3(256), 0, stream, a);
    HE_LAUNCH_CHECK();
  }
  return 0;
}
HE_API int he_conv_args_size() { return (int)sizeof(ConvArgs); }

HE_API int he_advance_positions(void* pos, void* ctx_len, const void* active, int n, int delta, cudaStream_t stream) {
  if (n <= 0) return 0;
  (void)launch_pdl(advance_positions_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, (int*)pos, (int*)ctx_len, (const int*)active, n, delta);
  HE_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------- skinny fp32 GEMM: out[T][N] = x[T][K] * W[N][K]^T
// For the few projections whose weights stay F32 in GGUF files (router, ssm_alpha/beta) at prefill row counts.
namespace {
constexpr int SG_TM = 64, SG_TN = 64, SG_TK = 16;
__global__ void __launch_bounds__(256) small_gemm_f32_kernel(const void* __restrict__ x, int x_dtype,
                                                             long long x_stride, const float* __restrict__ w,
                                                             float* __restrict__ out, long long out_stride, int T,
                                                             int N, int K) {
  __shared__ float xs[SG_TK][SG_TM + 1];
  __shared__ float ws[SG_TK][SG_TN + 1];
  const int t0 = blockIdx.y * SG_TM, n0 = blockIdx.x * SG_TN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4x4 outputs each
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += SG_TK) {
    for (int i = threadIdx.x; i < SG_TM * SG_TK; i += 256) {
      const int r = i / SG_TK, kk = i % SG_TK;
      const int t = t0 + r, k = k0 + kk;
      xs[kk][r] = (t < T && k < K) ? load_in(x, x_dtype, (size_t)t * x_stride + k) : 0.f;
    }
    for (int i = threadIdx.x; i < SG_TN * SG_TK; i += 256) {
      const int r = i / SG_TK, kk = i % SG_TK;
      const int n = n0 + r, k = k0 + kk;
      ws[kk][r] = (n < N && k < K) ? w[(size_t)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SG_TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[kk][ty * 4 + i]; b[i] = ws[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (t < T && n < N) out[(size_t)t * out_stride + n] = acc[i][j];
    }
}
}  // namespace

HE_API int he_small_gemm_f32(const void* x, int x_dtype, long long x_stride, const void* w, void* out,
                             long long out_stride, int T, int N, int K, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  dim3 grid((N + SG_TN - 1) / SG_TN, (T + SG_TM - 1) / SG_TM);
  small_gemm_f32_kernel<<<grid, 256, 0, stream>>>(x, x_dtype, x_stride, (const float*)w, (float*)out, out_stride, T, N,
                                                  K);
  HE_LAUNCH_CHECK();
  return 0;
}
