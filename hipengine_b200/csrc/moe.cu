// Mixture-of-experts kernels: router select, expert grouping for the tensor-core path, selected-expert GEMV
// for decode, combine with the shared expert.
//
//   decode (<= 8 rows)  : route -> gate/up GEMV over the selected (token, expert) pairs with act(g)*u fused
//                         -> down GEMV that sums the k experts of a token in a fixed order and adds the
//                         result to the fp32 residual stream.  Expert ids never leave the device.
//   prefill / verify    : route -> group (histogram, 128-row padded prefix, scatter) -> gather rows ->
//                         grouped tcgen05 GEMM (gemm_sm100.cu) -> act*up -> grouped GEMM -> combine.
//
// Behavioural references: hipengine/kernels/hip_gfx1100/moe/router.hip (softmax over all experts -> top-k ->
// renormalise by max(sum, 6.1e-5)), moe/group_scatter.hip (count / prefix / scatter), fused/paro_combine.hip
// (weighted sum + sigmoid shared-expert gate + residual) and the oracle cpu_reference/ops.py:575-700.
#include "common.cuh"
#include "gemv_rows.cuh"

using namespace he;
using hegemv::SmemView;
using hegemv::XQ_STRIDE;

namespace {

// ------------------------------------------------------------------------------------------ router select
// One warp per token.  mode 0: softmax over all experts, top-k, renormalise (Qwen).  mode 1: top-k on the
// logits, softmax over the selected k only (Gemma), times per-expert scale if given.
template <int MAXPL>
__global__ void moe_route_kernel(const float* __restrict__ logits, long long ld, int T, int E, int k, int mode,
                                 const float* __restrict__ expert_scale, int* __restrict__ ids,
                                 float* __restrict__ wts) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  float v[MAXPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < E ? logits[(size_t)t * ld + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float den = 0.f;
#pragma unroll
  for (int i = 0; i < MAXPL; ++i) den += (i * 32 + lane < E) ? __expf(v[i] - mx) : 0.f;
  den = warp_sum(den);
  float sel_sum = 0.f;
  float my_w = 0.f;   // lane j keeps the j-th selected weight (k <= 32)
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int e = i * 32 + lane;
      if (v[i] > bv) { bv = v[i]; bi = e; }   // ascending e within a lane: the lower id wins ties
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int i = 0; i < MAXPL; ++i)
        if (i == (bi >> 5)) v[i] = -INFINITY;
    }
    const float p = mode == 0 ? __expf(bv - mx) / den : bv;
    if (lane == j) { my_w = p; my_id = bi; }
    sel_sum += (mode == 0) ? p : 0.f;
  }
  if (mode == 0) {
    my_w = my_w / fmaxf(sel_sum, 6.1e-5f);
  } else {
    float m2 = warp_max(lane < k ? my_w : -INFINITY);
    const float ex = lane < k ? __expf(my_w - m2) : 0.f;
    const float s2 = warp_sum(ex);
    my_w = ex / s2;
    if (expert_scale != nullptr && lane < k) my_w *= expert_scale[my_id];
  }
  if (lane < k) {
    ids[(size_t)t * k + lane] = my_id;
    wts[(size_t)t * k + lane] = my_w;
  }
}

// ------------------------------------------------------------------------------------------ grouping
// Single CTA: histogram of expert ids over the P = T*k pairs, prefix over experts with every expert's rows
// padded to a multiple of 128, scatter.  pos[pair] = row in the sorted matrix, tile_group[tile] = expert of
// that 128-row tile or -1.  meta[0] = padded row count in use.
// Expert parallelism: only experts [e_lo, e_lo + E) are local; pairs routed elsewhere get pos = -1 and are skipped by
// the gather and the combine (their owners add them in through the cross-rank reduction of the partial outputs).
__global__ void __launch_bounds__(1024) moe_group_kernel(const int* __restrict__ ids, int P, int E, int e_lo,
                                                         int* __restrict__ pos, int* __restrict__ tile_group,
                                                         int max_tiles, int* __restrict__ meta) {
  extern __shared__ int sm[];
  int* cnt = sm;            // [E]
  int* off = sm + E;        // [E + 1]
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p] - e_lo;
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = run;
      run += (cnt[e] + 127) & ~127;
    }
    off[E] = run;
    meta[0] = run;
  }
  __syncthreads();
  for (int tl = threadIdx.x; tl < max_tiles; tl += blockDim.x) tile_group[tl] = -1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    for (int r = off[e]; r < off[e + 1]; r += 128) tile_group[r >> 7] = e;
    cnt[e] = 0;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = ids[p] - e_lo;
    pos[p] = (e >= 0 && e < E) ? off[e] + atomicAdd(&cnt[e], 1) : -1;
  }
}

// sorted[pos[p]][:] = x[p / k][:]   (bf16 rows of K elements, K % 8 == 0)
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const int* __restrict__ pos,
                                  int P, int k, int K, __nv_bfloat16* __restrict__ sorted, long long lds) {
  const int p = blockIdx.x;
  if (p >= P || pos[p] < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(p / k) * ldx);
  uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)pos[p] * lds);
  for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// h[t][:] += sum_j wts[t][j] * y[pos[t*k+j]][:] + sigmoid(sg[t]) * ysh[t][:]
__global__ void moe_combine_kernel(float* __restrict__ h, long long ldh, const __nv_bfloat16* __restrict__ y,
                                   long long ldy, const int* __restrict__ pos, const float* __restrict__ wts,
                                   int k, const __nv_bfloat16* __restrict__ ysh, long long ldsh,
                                   const float* __restrict__ sg, long long ldsg, int N) {
  const int t = blockIdx.x;
  for (int n = threadIdx.x * 2; n < N; n += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
    for (int j = 0; j < k; ++j) {
      const int pj = pos[(size_t)t * k + j];
      if (pj < 0) continue;     // expert lives on another rank
      const float w = wts[(size_t)t * k + j];
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y + (size_t)pj * ldy + n));
      a0 += w * f.x; a1 += w * f.y;
    }
    if (ysh != nullptr) {
      const float g = sg != nullptr ? sigmoid_f(sg[(size_t)t * ldsg]) : 1.f;
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(ysh + (size_t)t * ldsh + n));
      a0 += g * f.x; a1 += g * f.y;
    }
    float2* hp = reinterpret_cast<float2*>(h + (size_t)t * ldh + n);
    float2 hv = *hp;
    hv.x += a0; hv.y += a1;
    *hp = hv;
  }
}

// act[t][:] *= sigmoid(sg[t])   (bf16 rows; folds the shared-expert gate into its activation: the down
// projection is linear, so scaling its input scales its output)
__global__ void moe_scale_rows_kernel(__nv_bfloat16* __restrict__ act, long long ld, int N,
                                      const float* __restrict__ sg, long long ldsg) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const int t = blockIdx.x;
  const float g = sigmoid_f(sg[(size_t)t * ldsg]);
  for (int n = threadIdx.x; n < N; n += blockDim.x)
    act[(size_t)t * ld + n] = f32_to_bf16(bf16_to_f32(act[(size_t)t * ld + n]) * g);
}

// ------------------------------------------------------------------------------------------ selected GEMV
// Quantise 8 consecutive values (4 neighbouring lanes form a 32-wide block) into the shared activation row.
__device__ __forceinline__ void quant8(const SmemView& s, int r, int g, bool valid, const float (&v)[8]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float d = amax / 127.f;
  const float inv = d > 0.f ? 1.f / d : 0.f;
  int q[8], qsum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) { q[i] = __float2int_rn(v[i] * inv); qsum += q[i]; }
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
  qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
  if (valid) {
    const uint32_t p0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t p1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2*>(s.xq + (size_t)r * s.xq_row + (size_t)(g >> 5) * XQ_STRIDE + (g & 31) * 8) =
        make_uint2(p0, p1);
    if ((g & 3) == 0) {
      s.dx[(size_t)r * s.sc_row + (g >> 2)] = d;
      s.sx[(size_t)r * s.sc_row + (g >> 2)] = d * (float)qsum;
    }
  }
}

__device__ __forceinline__ SmemView carve(uint8_t* base, int rows, int K) {
  SmemView s;
  const int nb = K >> 8;
  s.xq_row = nb * XQ_STRIDE;
  s.sc_row = K >> 5;
  s.xq = reinterpret_cast<int8_t*>(base);
  s.dx = reinterpret_cast<float*>(base + (size_t)rows * s.xq_row);
  s.sx = s.dx + (size_t)rows * s.sc_row;
  s.inv_rms = s.sx + (size_t)rows * s.sc_row;
  return s;
}
__host__ __device__ inline size_t carve_bytes(int rows, int K) {
  return (size_t)rows * (K >> 8) * XQ_STRIDE + (size_t)rows * (K >> 5) * 8 + 64;
}

// dot of block b of one quantised weight row with activation row `r` of the view
__device__ __forceinline__ float dot_block(const uint8_t* row, int qtype, int K, int b, const SmemView& s, int r) {
  SmemView v = s;
  v.xq += (size_t)r * s.xq_row;
  v.dx += (size_t)r * s.sc_row;
  v.sx += (size_t)r * s.sc_row;
  float acc[1] = {0.f};
  if (qtype == HE_Q4_K) hegemv::block_q4k<1>(row + (size_t)b * 144, b, v, acc);
  else if (qtype == HE_Q6_K) hegemv::block_q6k<1>(row + (size_t)b * 224, b, v, acc);
  else hegemv::block_q80<1>(row + (size_t)b * 256, row + K + (size_t)b * 16, b, v, acc);
  return acc[0];
}

struct MoeSelArgs {
  const void* x;            // gate/up: fp32 residual rows [T][ldx]; down: bf16 activations [T*k][ldx]
  long long ldx;
  const float* norm_w;      // gate/up only
  float eps;
  const int* ids;           // [T][k]
  const float* wts;         // [T][k]
  const uint8_t* w1;        // gate experts (or down experts)
  const uint8_t* w2;        // up experts
  int qtype1, qtype2;
  int T, k, K, N;           // K = input width, N = rows per expert
  int act;                  // 0 silu, 1 gelu_tanh
  void* out;                // gate/up: bf16 [T*k][ldo]; down: fp32 residual [T][ldo], accumulated in place
  long long ldo;
  int rows_per_cta;
  int expert_rows;          // rows between consecutive experts in w1 / w2 (0 -> N); 2N for a fused gate|up tensor
  int expert_lo, expert_n;  // local expert range [lo, lo + n) (expert parallelism); n <= 0 -> all experts local
};

// grid (ceil(N / rows_per_cta), T*k), 256 threads
__global__ void __launch_bounds__(256) moe_gateup_sel_kernel(const MoeSelArgs a) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  // no early pdl_launch(): the grid spans several waves, and a successor made resident early would only
  // hold SM resources that the later waves of this grid need
  extern __shared__ __align__(16) uint8_t smem_moe[];
  __shared__ float red[32];
  const SmemView s = carve(smem_moe, 1, a.K);
  const int pair = blockIdx.y, t = pair / a.k;
  const int e = a.ids[pair] - a.expert_lo;
  if (a.expert_n > 0 && (e < 0 || e >= a.expert_n)) return;     // not a local expert (uniform for the CTA)
  const float* xr = reinterpret_cast<const float*>(a.x) + (size_t)t * a.ldx;
  // RMSNorm + int8 quantisation of the token's row
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < a.K; i += 1024) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(xr + i));
    ss += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
  }
  ss = block_sum(ss, red);
  const float inv_rms = a.norm_w != nullptr ? rsqrtf(ss / (float)a.K + a.eps) : 1.f;
  const int n_groups = a.K / 8;
  for (int g0 = 0; g0 < n_groups; g0 += 256) {
    const int g = g0 + threadIdx.x;
    const bool valid = g < n_groups;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (valid) {
      const float4 f0 = __ldg(reinterpret_cast<const float4*>(xr + g * 8));
      const float4 f1 = __ldg(reinterpret_cast<const float4*>(xr + g * 8 + 4));
      float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
      if (a.norm_w != nullptr) {
        w0 = __ldg(reinterpret_cast<const float4*>(a.norm_w + g * 8));
        w1 = __ldg(reinterpret_cast<const float4*>(a.norm_w + g * 8 + 4));
      }
      v[0] = f0.x * inv_rms * w0.x; v[1] = f0.y * inv_rms * w0.y; v[2] = f0.z * inv_rms * w0.z; v[3] = f0.w * inv_rms * w0.w;
      v[4] = f1.x * inv_rms * w1.x; v[5] = f1.y * inv_rms * w1.y; v[6] = f1.z * inv_rms * w1.z; v[7] = f1.w * inv_rms * w1.w;
    }
    quant8(s, 0, g, valid, v);
  }
  __syncthreads();
  const int nblk = a.K >> 8;
  int lpr = 1;
  while (lpr < nblk && lpr < 32) lpr <<= 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % lpr, rin = lane / lpr, rpp = 32 / lpr;
  const long long rb1 = hegemv::row_bytes_dev(a.qtype1, a.K), rb2 = hegemv::row_bytes_dev(a.qtype2, a.K);
  const int erows = a.expert_rows > 0 ? a.expert_rows : a.N;
  const uint8_t* w1e = a.w1 + (size_t)e * erows * rb1;
  const uint8_t* w2e = a.w2 + (size_t)e * erows * rb2;
  const int row_end = min(a.N, (int)(blockIdx.x + 1) * a.rows_per_cta);
  for (int n0 = blockIdx.x * a.rows_per_cta + warp * rpp; n0 < row_end; n0 += 8 * rpp) {
    const int n = n0 + rin;
    float g = 0.f, u = 0.f;
    if (n < row_end) {
      for (int b = sub; b < nblk; b += lpr) {
        g += dot_block(w1e + (size_t)n * rb1, a.qtype1, a.K, b, s, 0);
        u += dot_block(w2e + (size_t)n * rb2, a.qtype2, a.K, b, s, 0);
      }
    }
    for (int off = 1; off < lpr; off <<= 1) {
      g += __shfl_xor_sync(0xffffffffu, g, off);
      u += __shfl_xor_sync(0xffffffffu, u, off);
    }
    if (sub == 0 && n < row_end) {
      const float av = a.act == 0 ? silu_f(g) : gelu_tanh_f(g);
      reinterpret_cast<__nv_bfloat16*>(a.out)[(size_t)pair * a.ldo + n] = f32_to_bf16(av * u);
    }
  }
}

// grid (ceil(N / rows_per_cta), T), 256 threads.  K = expert FFN width; activations of the token's k experts
// are quantised into k shared rows; an output row is owned by lpr lanes covering all (expert, block) items.
__global__ void __launch_bounds__(256) moe_down_sel_kernel(const MoeSelArgs a) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  // no early pdl_launch(): the grid spans several waves, and a successor made resident early would only
  // hold SM resources that the later waves of this grid need
  extern __shared__ __align__(16) uint8_t smem_moe[];
  __shared__ int e_s[32];
  __shared__ float w_s[32];
  const SmemView s = carve(smem_moe, a.k, a.K);
  const int t = blockIdx.y;
  if (threadIdx.x < a.k) {
    const int e = a.ids[(size_t)t * a.k + threadIdx.x] - a.expert_lo;
    const bool local = a.expert_n <= 0 || (e >= 0 && e < a.expert_n);
    e_s[threadIdx.x] = local ? e : -1;                                        // -1: expert lives on another rank
    w_s[threadIdx.x] = local ? a.wts[(size_t)t * a.k + threadIdx.x] : 0.f;
  }
  const int gpr = a.K / 8;   // 8-element groups per row
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(a.x) + (size_t)t * a.k * a.ldx;
  for (int i0 = 0; i0 < a.k * gpr; i0 += 256) {
    const int i = i0 + threadIdx.x;
    const bool valid = i < a.k * gpr;
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = 0.f;
    const int j = valid ? i / gpr : 0, g = valid ? i % gpr : 0;
    if (valid) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(xb + (size_t)j * a.ldx + g * 8));
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(h2[q]);
        v[2 * q] = f.x; v[2 * q + 1] = f.y;
      }
    }
    quant8(s, j, g, valid, v);   // gpr % 4 == 0, so the 4 lanes of a 32-block share j
  }
  __syncthreads();
  const int nblk = a.K >> 8, items = a.k * nblk;
  int lpr = 1;
  while (lpr < items && lpr < 32) lpr <<= 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % lpr, rin = lane / lpr, rpp = 32 / lpr;
  const long long rb = hegemv::row_bytes_dev(a.qtype1, a.K);
  const int row_end = min(a.N, (int)(blockIdx.x + 1) * a.rows_per_cta);
  float* out = reinterpret_cast<float*>(a.out) + (size_t)t * a.ldo;
  for (int n0 = blockIdx.x * a.rows_per_cta + warp * rpp; n0 < row_end; n0 += 8 * rpp) {
    const int n = n0 + rin;
    float acc = 0.f;
    if (n < row_end) {
      for (int it = sub; it < items; it += lpr) {
        const int j = it / nblk, b = it % nblk;
        if (e_s[j] < 0) continue;      // its activation row was never written on this rank
        const uint8_t* row = a.w1 + ((size_t)e_s[j] * (a.expert_rows > 0 ? a.expert_rows : a.N) + n) * rb;
        acc += w_s[j] * dot_block(row, a.qtype1, a.K, b, s, j);
      }
    }
    for (int off = 1; off < lpr; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == 0 && n < row_end) out[n] += acc;
  }
}

template <typename F>
int set_smem(F fn, size_t bytes) {
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace

HE_API int he_moe_route(const float* logits, long long ld, int T, int E, int k, int mode, const float* expert_scale,
                        int* ids, float* wts, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (k > 32 || k <= 0 || E > 512 || E < k) return -HE_ERR_BAD_ARG;
  const int wpb = 4;
  const dim3 grid((T + wpb - 1) / wpb);
  if (E <= 128) (void)launch_pdl(moe_route_kernel<4>, dim3(grid), dim3(wpb * 32), 0, stream, logits, ld, T, E, k, mode, expert_scale, ids, wts);
  else if (E <= 256) (void)launch_pdl(moe_route_kernel<8>, dim3(grid), dim3(wpb * 32), 0, stream, logits, ld, T, E, k, mode, expert_scale, ids, wts);
  else (void)launch_pdl(moe_route_kernel<16>, dim3(grid), dim3(wpb * 32), 0, stream, logits, ld, T, E, k, mode, expert_scale, ids, wts);
  HE_LAUNCH_CHECK();
  return 0;
}

// Upper bound of sorted rows for P pairs over E experts (every expert padded to 128 rows).
HE_API long long he_moe_sorted_rows_bound(long long P, int E) {
  const long long tiles = (P + 127) / 128 + E;
  return tiles * 128;
}

HE_API int he_moe_group(const int* ids, int P, int E, int e_lo, int* pos, int* tile_group, int max_tiles, int* meta,
                        cudaStream_t stream) {
  if (P <= 0) return 0;
  moe_group_kernel<<<1, 1024, (2 * E + 1) * sizeof(int), stream>>>(ids, P, E, e_lo, pos, tile_group, max_tiles, meta);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_moe_gather(const void* x, long long ldx, const int* pos, int P, int k, int K, void* sorted,
                         long long lds, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (K % 8 != 0) return -HE_ERR_BAD_ARG;
  moe_gather_kernel<<<P, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, pos, P, k, K,
                                           reinterpret_cast<__nv_bfloat16*>(sorted), lds);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_moe_combine(float* h, long long ldh, const void* y, long long ldy, const int* pos, const float* wts,
                          int T, int k, const void* ysh, long long ldsh, const float* sg, long long ldsg, int N,
                          cudaStream_t stream) {
  if (T <= 0) return 0;
  if (N % 2 != 0) return -HE_ERR_BAD_ARG;
  moe_combine_kernel<<<T, 256, 0, stream>>>(h, ldh, reinterpret_cast<const __nv_bfloat16*>(y), ldy, pos, wts, k,
                                            reinterpret_cast<const __nv_bfloat16*>(ysh), ldsh, sg, ldsg, N);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_moe_scale_rows(void* act, long long ld, int T, int N, const float* sg, long long ldsg,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  (void)launch_pdl(moe_scale_rows_kernel, dim3(T), dim3(256), 0, stream, reinterpret_cast<__nv_bfloat16*>(act), ld, N, sg, ldsg);
  HE_LAUNCH_CHECK();
  return 0;
}

static int check_sel(const MoeSelArgs& a) {
  if (a.K % 256 != 0 || a.k <= 0 || a.k > 32 || a.N <= 0) return -HE_ERR_BAD_ARG;
  const int ok1 = a.qtype1 == HE_Q4_K || a.qtype1 == HE_Q6_K || a.qtype1 == HE_Q8_0;
  return ok1 ? 0 : -HE_ERR_BAD_ARG;
}

HE_API int he_moe_gateup_sel(const MoeSelArgs* args, cudaStream_t stream) {
  MoeSelArgs a = *args;
  if (a.T <= 0) return 0;
  int rc = check_sel(a);
  if (rc != 0) return rc;
  if (!(a.qtype2 == HE_Q4_K || a.qtype2 == HE_Q6_K || a.qtype2 == HE_Q8_0)) return -HE_ERR_BAD_ARG;
  a.rows_per_cta = a.T * a.k >= 32 ? 64 : 32;
  const size_t smem = carve_bytes(1, a.K);
  rc = set_smem(moe_gateup_sel_kernel, smem);
  if (rc != 0) return rc;
  const dim3 grid((a.N + a.rows_per_cta - 1) / a.rows_per_cta, a.T * a.k);
  (void)launch_pdl(moe_gateup_sel_kernel, dim3(grid), dim3(256), smem, stream, a);
  HE_LAUNCH_CHECK();
  return 0;
}

HE_API int he_moe_down_sel(const MoeSelArgs* args, cudaStream_t stream) {
  MoeSelArgs a = *args;
  if (a.T <= 0) return 0;
  int rc = check_sel(a);
  if (rc != 0) return rc;
  a.rows_per_cta = a.T >= 4 ? 64 : 32;
  const size_t smem = carve_bytes(a.k, a.K);
  rc = set_smem(moe_down_sel_kernel, smem);
  if (rc != 0) return rc;
  const dim3 grid((a.N + a.rows_per_cta - 1) / a.rows_per_cta, a.T);
  (void)launch_pdl(moe_down_sel_kernel, dim3(grid), dim3(256), smem, stream, a);
  HE_LAUNCH_CHECK();
  return 0;
}
HE_API int he_moe_sel_args_size() { return (int)sizeof(MoeSelArgs); }
