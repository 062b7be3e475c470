// Gated DeltaNet (linear attention): prepare (L2-norm q,k + gates), the recurrent scan over packed
// segments (decode rows, verify chains and prefill share one kernel), and the gated output RMSNorm.
//
// Per V head the state S is [Dk x Dv] fp32 and each step is
//     S <- decay*S ;  kv = k^T S ;  delta = beta*(v - kv) ;  S <- S + k (x) delta ;  o = q^T S
// (hipengine/kernels/hip_gfx1100/linear_attn/gdn.hip:126-330; oracle hipengine/kernels/cpu_reference/ops.py:1967-2012).
// Columns of S are independent, so a head is split into Dv/32 column slices, one CTA each: with 48 heads x 4
// slices a single request already fills the 148 SMs.  Inside a CTA a column is owned by 4 lanes of one warp
// (rows r = lane%4 + 4*i), so the two reductions per token are two xor-shuffles and no block barrier.
// GGUF head order: V head h reads K head h % num_k_heads (gdn.hip:106-118).
#include "common.cuh"

using namespace he;

namespace {

struct GdnPrepArgs {
  float* qkv;            // [T][C] conv output, q and k normalised in place
  const float* a;        // [T][a_stride]
  const float* b;        // [T][b_stride]
  long long a_stride, b_stride;
  const float* ssm_a;    // [Hv]  (negative coefficient)
  const float* dt_bias;  // [Hv]
  float* decay;          // [T][Hv]
  float* beta;           // [T][Hv]
  int C, G, Hv, S, T;
};

// grid T, block 256
__global__ void __launch_bounds__(256) gdn_prepare_kernel(const GdnPrepArgs p) {
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  float* row = p.qkv + (size_t)t * p.C;
  const float qscale = rsqrtf((float)p.S);
  for (int h = warp; h < 2 * p.G; h += nwarp) {
    float* v = row + (size_t)h * p.S;
    float ss = 0.f;
    for (int i = lane; i < p.S; i += 32) ss += v[i] * v[i];
    ss = warp_sum(ss);
    float inv = 1.f / fmaxf(sqrtf(ss), 1e-6f);
    if (h < p.G) inv *= qscale;
    for (int i = lane; i < p.S; i += 32) v[i] *= inv;
  }
  for (int h = threadIdx.x; h < p.Hv; h += blockDim.x) {
    const float av = p.a[(size_t)t * p.a_stride + h], bv = p.b[(size_t)t * p.b_stride + h];
    p.beta[(size_t)t * p.Hv + h] = sigmoid_f(bv);
    p.decay[(size_t)t * p.Hv + h] = __expf(p.ssm_a[h] * softplus20_f(av + p.dt_bias[h]));
  }
}

struct GdnScanArgs {
  const float* qkv;       // [T][C]  prepared conv output: q | k | v
  const float* decay;     // [T][Hv]
  const float* beta;      // [T][Hv]
  float* state;           // [n_slots][Hv][Dk][Dv]
  const int* seg_start;   // [n_seg+1]
  const int* seg_slot;    // [n_seg]
  float* out;             // [T][Hv][Dv]
  float* journal;         // optional [T][Hv][Dk][Dv] state after each token
  int C, G, Hv, T, n_seg;
  int write_state;        // 1: store the final state back to `state`
};

constexpr int DK = 128;       // state rows (key dim)
constexpr int DV = 128;       // state cols (value dim)
constexpr int SLICE = 32;     // columns per CTA
constexpr int TCH = 16;       // tokens staged per shared-memory chunk

constexpr int KPAD = DK + DK / 8;   // 4 pad floats per 32 so the 4 row groups of a column land in different banks

// grid (n_seg, Hv, DV/SLICE), block 32*LPC.  A column of S is owned by LPC lanes of one warp; lane ks owns rows
// ks*RPL .. ks*RPL+RPL-1 (RPL = 128/LPC).  LPC = 4 keeps more of the state per thread (fewer shuffles per token);
// LPC = 8 doubles the warps when only a few (segment, head) pairs exist, which is what hides the issue latency of
// this strictly sequential recurrence during a single-request prefill.
template <int LPC>
__global__ void __launch_bounds__(32 * LPC) gdn_scan_kernel(const GdnScanArgs p) {
  constexpr int RPL = DK / LPC;            // rows per lane: 32 or 16
  constexpr int NT = 32 * LPC;             // threads
  constexpr int CPW = 32 / LPC;            // columns per warp
  __shared__ __align__(16) float sq[TCH][KPAD];
  __shared__ __align__(16) float sk[TCH][KPAD];
  __shared__ float sv[TCH][SLICE];
  __shared__ float sdec[TCH], sbeta[TCH];
  const int sg = blockIdx.x, h = blockIdx.y, sl = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cw = warp * CPW + lane / LPC;               // column inside the slice
  const int col = sl * SLICE + cw;                      // column of S owned (with LPC-1 other lanes)
  const int ks = lane % LPC;
  const int kh = h % p.G;
  const int s0 = p.seg_start[sg], s1 = p.seg_start[sg + 1];
  float* Sg = p.state + (((size_t)p.seg_slot[sg] * p.Hv + h) * DK) * DV;
  float S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) S[i] = Sg[(size_t)(ks * RPL + i) * DV + col];
  const int koff = ks * RPL + ((ks * RPL) >> 5) * 4;    // padded offset of this lane's rows in sq / sk

  const size_t q_off = (size_t)kh * DK, k_off = (size_t)p.G * DK + (size_t)kh * DK;
  const size_t v_off = (size_t)2 * p.G * DK + (size_t)h * DV + sl * SLICE;

  for (int c0 = s0; c0 < s1; c0 += TCH) {
    const int n = min(TCH, s1 - c0);
    __syncthreads();
    for (int i = tid; i < n * (DK / 4); i += NT) {
      const int tt = i / (DK / 4), d4 = (i % (DK / 4)) * 4;
      const float* row = p.qkv + (size_t)(c0 + tt) * p.C;
      const int dst = d4 + (d4 >> 5) * 4;
      *reinterpret_cast<float4*>(&sq[tt][dst]) = *reinterpret_cast<const float4*>(row + q_off + d4);
      *reinterpret_cast<float4*>(&sk[tt][dst]) = *reinterpret_cast<const float4*>(row + k_off + d4);
    }
    for (int i = tid; i < n * SLICE; i += NT) {
      const int tt = i / SLICE, d = i % SLICE;
      sv[tt][d] = p.qkv[(size_t)(c0 + tt) * p.C + v_off + d];
    }
    if (tid < n) {
      sdec[tid] = p.decay[(size_t)(c0 + tid) * p.Hv + h];
      sbeta[tid] = p.beta[(size_t)(c0 + tid) * p.Hv + h];
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float dec = sdec[tt], bet = sbeta[tt];
      float kr[RPL];
#pragma unroll
      for (int i4 = 0; i4 < RPL / 4; ++i4) {
        const float4 kv4 = *reinterpret_cast<const float4*>(&sk[tt][koff + i4 * 4]);
        kr[i4 * 4] = kv4.x; kr[i4 * 4 + 1] = kv4.y; kr[i4 * 4 + 2] = kv4.z; kr[i4 * 4 + 3] = kv4.w;
      }
      // four independent partial sums per reduction keep the FMA pipe busy (the chains are otherwise serial)
      float kv4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        S[i] *= dec;
        kv4[i & 3] += kr[i] * S[i];
      }
      float kv = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
#pragma unroll
      for (int o = 1; o < LPC; o <<= 1) kv += __shfl_xor_sync(0xffffffffu, kv, o);
      const float delta = (sv[tt][cw] - kv) * bet;
      float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i4 = 0; i4 < RPL / 4; ++i4) {
        const float4 q4 = *reinterpret_cast<const float4*>(&sq[tt][koff + i4 * 4]);
        S[i4 * 4] += kr[i4 * 4] * delta;         o4[0] += q4.x * S[i4 * 4];
        S[i4 * 4 + 1] += kr[i4 * 4 + 1] * delta; o4[1] += q4.y * S[i4 * 4 + 1];
        S[i4 * 4 + 2] += kr[i4 * 4 + 2] * delta; o4[2] += q4.z * S[i4 * 4 + 2];
        S[i4 * 4 + 3] += kr[i4 * 4 + 3] * delta; o4[3] += q4.w * S[i4 * 4 + 3];
      }
      float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
#pragma unroll
      for (int of = 1; of < LPC; of <<= 1) o += __shfl_xor_sync(0xffffffffu, o, of);
      if (ks == 0) p.out[((size_t)(c0 + tt) * p.Hv + h) * DV + col] = o;
      if (p.journal != nullptr) {
        float* J = p.journal + (((size_t)(c0 + tt) * p.Hv + h) * DK) * DV;
#pragma unroll
        for (int i = 0; i < RPL; ++i) J[(size_t)(ks * RPL + i) * DV + col] = S[i];
      }
    }
  }
  if (p.write_state) {
#pragma unroll
    for (int i = 0; i < RPL; ++i) Sg[(size_t)(ks * RPL + i) * DV + col] = S[i];
  }
}

// out[t][h][:] = RMSNorm(o[t][h][:]) * w * SiLU(z[t][h][:])  -> bf16.  One warp per (t, h).
__global__ void gdn_gated_norm_kernel(const float* __restrict__ o, const void* __restrict__ z, int z_dtype,
                                      long long z_stride, const float* __restrict__ w,
                                      __nv_bfloat16* __restrict__ out, long long out_stride, int T, int Hv, int Dv,
                                      float eps) {
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= (long long)T * Hv) return;
  const int t = (int)(gw / Hv), h = (int)(gw % Hv);
  const float* orow = o + ((size_t)t * Hv + h) * Dv;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) ss += orow[i] * orow[i];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)Dv + eps);
  for (int i = lane; i < Dv; i += 32) {
    const size_t zi = (size_t)t * z_stride + (size_t)h * Dv + i;
    const float zv = z_dtype == 0 ? reinterpret_cast<const float*>(z)[zi]
                                  : bf16_to_f32(reinterpret_cast<const __nv_bfloat16*>(z)[zi]);
    out[(size_t)t * out_stride + (size_t)h * Dv + i] = f32_to_bf16(orow[i] * inv * w[i] * silu_f(zv));
  }
}

// Copy one journalled state row into the canonical slot (speculative commit): dst[slot] = journal[row].
__global__ void gdn_commit_kernel(float* __restrict__ state, const float* __restrict__ journal,
                                  const int* __restrict__ seg_slot, const int* __restrict__ commit_row,
                                  long long per_slot) {
  const int sg = blockIdx.y;
  const int row = commit_row[sg];
  if (row < 0) return;
  const float4* src = reinterpret_cast<const float4*>(journal + (size_t)row * per_slot);
  float4* dst = reinterpret_cast<float4*>(state + (size_t)seg_slot[sg] * per_slot);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_slot / 4;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------------- decode fast path
// For single-token segments (plain decode) the five kernels conv -> conv state -> prepare -> scan -> gated norm
// collapse into two launches; a decode step is bound by launch latency, not by this arithmetic.
struct GdnDecodeArgs {
  const float* x;         // [R][x_stride] pre-conv projections q | k | v (fp32)
  long long x_stride;
  const float* conv_w;    // [C][4]
  float* conv_state;      // [n_slots][C][3]
  const float* a;         // [R][a_stride]
  const float* b;         // [R][b_stride]
  long long a_stride, b_stride;
  const float* ssm_a;     // [Hv]
  const float* dt_bias;   // [Hv]
  const int* slot;        // [R]
  float* qkv;             // [R][C] conv output (q, k normalised)
  float* decay;           // [R][Hv]
  float* beta;            // [R][Hv]
  float* state;           // [n_slots][Hv][128][128]
  const void* z;          // [R][z_stride] gate input
  int z_dtype;
  long long z_stride;
  const float* norm_w;    // [128]
  __nv_bfloat16* out;     // [R][out_stride]
  long long out_stride;
  float eps;
  int C, G, Hv, R;
};

// grid (C/128, R), block 128: one channel per thread.  conv(k=4)+SiLU, rolling state shift, L2 norm of q/k heads,
// and (block 0) the decay / beta gates of the row.
__global__ void __launch_bounds__(128) gdn_decode_pre_kernel(const GdnDecodeArgs p) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.y, blk = blockIdx.x, c = blk * 128 + threadIdx.x;
  float* st = p.conv_state + ((size_t)p.slot[r] * p.C + c) * 3;
  const float4 w = __ldg(reinterpret_cast<const float4*>(p.conv_w + (size_t)c * 4));
  const float xv = p.x[(size_t)r * p.x_stride + c];
  const float s0 = st[0], s1 = st[1], s2 = st[2];
  float y = silu_f(w.x * s0 + w.y * s1 + w.z * s2 + w.w * xv);
  st[0] = s1; st[1] = s2; st[2] = xv;
  if (blk < 2 * p.G) {
    const float ss = block_sum(y * y, red);
    float inv = 1.f / fmaxf(sqrtf(ss), 1e-6f);
    if (blk < p.G) inv *= rsqrtf(128.f);
    y *= inv;
  }
  p.qkv[(size_t)r * p.C + c] = y;
  if (blk == 0) {
    for (int h = threadIdx.x; h < p.Hv; h += 128) {
      const float av = p.a[(size_t)r * p.a_stride + h], bv = p.b[(size_t)r * p.b_stride + h];
      p.beta[(size_t)r * p.Hv + h] = sigmoid_f(bv);
      p.decay[(size_t)r * p.Hv + h] = __expf(p.ssm_a[h] * softplus20_f(av + p.dt_bias[h]));
    }
  }
}

// grid (Hv, R), block 512: thread (col = tid/4, ks = tid%4) owns rows ks*32..+31 of one column of S.
// One recurrent step, then RMSNorm over the head's 128 outputs * w * SiLU(z) -> bf16.
__global__ void __launch_bounds__(512) gdn_decode_step_kernel(const GdnDecodeArgs p) {
  __shared__ __align__(16) float sq[KPAD];
  __shared__ __align__(16) float sk[KPAD];
  __shared__ float red[32];
  const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x;
  const int col = tid >> 2, ks = tid & 3;
  const int kh = h % p.G;
  const float* row = p.qkv + (size_t)r * p.C;
  pdl_wait();
  pdl_launch();
  if (tid < 128) {
    const int dst = tid + (tid >> 5) * 4;
    sq[dst] = row[(size_t)kh * DK + tid];
    sk[dst] = row[(size_t)p.G * DK + (size_t)kh * DK + tid];
  }
  float* Sg = p.state + (((size_t)p.slot[r] * p.Hv + h) * DK) * DV;
  float S[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) S[i] = Sg[(size_t)(ks * 32 + i) * DV + col];
  const float v = row[(size_t)2 * p.G * DK + (size_t)h * DV + col];
  const float dec = p.decay[(size_t)r * p.Hv + h], bet = p.beta[(size_t)r * p.Hv + h];
  __syncthreads();
  float kr[32];
#pragma unroll
  for (int i4 = 0; i4 < 8; ++i4) {
    const float4 k4 = *reinterpret_cast<const float4*>(&sk[ks * 36 + i4 * 4]);
    kr[i4 * 4] = k4.x; kr[i4 * 4 + 1] = k4.y; kr[i4 * 4 + 2] = k4.z; kr[i4 * 4 + 3] = k4.w;
  }
  float kv4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    S[i] *= dec;
    kv4[i & 3] += kr[i] * S[i];
  }
  float kv = (kv4[0] + kv4[1]) + (kv4[2] + kv4[3]);
  kv += __shfl_xor_sync(0xffffffffu, kv, 1);
  kv += __shfl_xor_sync(0xffffffffu, kv, 2);
  const float delta = (v - kv) * bet;
  float o4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i4 = 0; i4 < 8; ++i4) {
    const float4 q4 = *reinterpret_cast<const float4*>(&sq[ks * 36 + i4 * 4]);
    S[i4 * 4] += kr[i4 * 4] * delta;         o4[0] += q4.x * S[i4 * 4];
    S[i4 * 4 + 1] += kr[i4 * 4 + 1] * delta; o4[1] += q4.y * S[i4 * 4 + 1];
    S[i4 * 4 + 2] += kr[i4 * 4 + 2] * delta; o4[2] += q4.z * S[i4 * 4 + 2];
    S[i4 * 4 + 3] += kr[i4 * 4 + 3] * delta; o4[3] += q4.w * S[i4 * 4 + 3];
  }
  float o = (o4[0] + o4[1]) + (o4[2] + o4[3]);
  o += __shfl_xor_sync(0xffffffffu, o, 1);
  o += __shfl_xor_sync(0xffffffffu, o, 2);
#pragma unroll
  for (int i = 0; i < 32; ++i) Sg[(size_t)(ks * 32 + i) * DV + col] = S[i];
  const float ss = block_sum(ks == 0 ? o * o : 0.f, red);
  if (ks == 0) {
    const float inv = rsqrtf(ss / (float)DV + p.eps);
    const size_t zi = (size_t)r * p.z_stride + (size_t)h * DV + col;
    const float zv = p.z_dtype == 0 ? reinterpret_cast<const float*>(p.z)[zi]
                                    : bf16_to_f32(reinterpret_cast<const __nv_bfloat16*>(p.z)[zi]);
    p.out[(size_t)r * p.out_stride + (size_t)h * DV + col] = f32_to_bf16(o * inv * p.norm_w[col] * silu_f(zv));
  }
}

}  // namespace

HE_API int he_gdn_prepare(const GdnPrepArgs* args, cudaStream_t stream) {
  if (args->T <= 0) return 0;
  gdn_prepare_kernel<<<args->T, 256, 0, stream>>>(*args);
  HE_LAUNCH_CHECK();
  return 0;
}
HE_API int he_gdn_prep_args_size() { return (int)sizeof(GdnPrepArgs); }

HE_API int he_gdn_scan(const GdnScanArgs* args, cudaStream_t stream) {
  if (args->T <= 0 || args->n_seg <= 0) return 0;
  dim3 grid(args->n_seg, args->Hv, DV / SLICE);
  // few (segment, head) pairs and long segments: spread every column over 8 lanes to double the resident warps
  const bool wide = (long long)args->n_seg * args->Hv * (DV / SLICE) <= 1024 && args->T >= 64 * args->n_seg;
  if (wide) gdn_scan_kernel<8><<<grid, 256, 0, stream>>>(*args);
  else gdn_scan_kernel<4><<<grid, 128, 0, stream>>>(*args);
  HE_LAUNCH_CHECK();
  return 0;
}
HE_API int he_gdn_scan_args_size() { return (int)sizeof(GdnScanArgs); }

HE_API int he_gdn_gated_norm(const void* o, const void* z, int z_dtype, long long z_stride, const void* w, void* out,
                             long long out_stride, int T, int Hv, int Dv, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long warps = (long long)T * Hv;
  gdn_gated_norm_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, stream>>>(
      (const float*)o, z, z_dtype, z_stride, (const float*)w, (__nv_bfloat16*)out, out_stride, T, Hv, Dv, eps);
  HE_LAUNCH_CHECK();
  return 0;
}

// state[seg_slot[s]] = journal[commit_row[s]] for each segment s with commit_row[s] >= 0.
// per_slot = floats per slot (Hv*Dk*Dv for GDN state, C*(KW-1) for conv state); must be a multiple of 4.
HE_API int he_state_commit(void* state, const void* journal, const void* seg_slot, const void* commit_row, int n_seg,
                           long long per_slot, cudaStream_t stream) {
  if (n_seg <= 0) return 0;
  if (per_slot % 4 != 0) return -HE_ERR_BAD_ARG;
  dim3 grid(64, n_seg);
  gdn_commit_kernel<<<grid, 256, 0, stream>>>((float*)state, (const float*)journal, (const int*)seg_slot,
                                              (const int*)commit_row, per_slot);
  HE_LAUNCH_CHECK();
  return 0;
}

// Decode fast path (every row is a single-token segment, no journal): conv + gates + one scan step + gated norm
// in two launches.  Requires state size 128, conv kernel 4, C % 128 == 0.
HE_API int he_gdn_decode(const GdnDecodeArgs* args, cudaStream_t stream) {
  const GdnDecodeArgs& a = *args;
  if (a.R <= 0) return 0;
  if (a.C % 128 != 0 || a.C != 2 * a.G * 128 + a.Hv * 128 || a.Hv % a.G != 0) return -HE_ERR_BAD_ARG;
  cudaError_t e = launch_pdl(gdn_decode_pre_kernel, dim3(a.C / 128, a.R), dim3(128), 0, stream, a);
  if (e != cudaSuccess) return (int)e;
  e = launch_pdl(gdn_decode_step_kernel, dim3(a.Hv, a.R), dim3(512), 0, stream, a);
  if (e != cudaSuccess) return (int)e;
  return 0;
}
HE_API int he_gdn_decode_args_size() { return (int)sizeof(GdnDecodeArgs); }
