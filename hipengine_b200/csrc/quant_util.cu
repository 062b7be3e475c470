// GGUF -> device layout repack, element dequantization, bf16 widening and embedding-row gather.
//
// Device layouts (rows contiguous and 16-byte aligned, see gemv_rows.cuh):
//   Q4_K : 144-byte GGUF blocks unchanged
//   Q6_K : 224-byte blocks  [ql 128][qh 64][scales 16][d fp16][14 zero pad]   (GGUF block is 210 bytes)
//   Q8_0 : per row [K int8][K/32 fp16 scales][pad to 16]                      (GGUF block is 34 bytes)
// The repack is lossless; he_unpack restores the exact GGUF bytes (round-trip tested).
// Row dequantization mirrors the reference's embedding / dequant kernels
// (hipengine/kernels/hip_gfx1100/quant/gguf_q6_k_embedding.hip) and its NumPy oracle (hipengine/quant/gguf.py:604-665).
#include "common.cuh"
#include "gemv_rows.cuh"

using namespace he;

namespace {

__global__ void repack_q6k_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, long long nblk,
                                  int inverse) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (block, 2-byte unit of 224)
  const long long b = i / 112;
  const int u = (int)(i % 112) * 2;
  if (b >= nblk) return;
  if (!inverse) {
    uint8_t* dst = out + b * 224 + u;
    if (u < 210) {
      const uint8_t* src = raw + b * 210 + u;
      dst[0] = src[0];
      dst[1] = src[1];
    } else {
      dst[0] = 0;
      dst[1] = 0;
    }
  } else if (u < 210) {
    const uint8_t* src = raw + b * 224 + u;
    uint8_t* dst = out + b * 210 + u;
    dst[0] = src[0];
    dst[1] = src[1];
  }
}

__global__ void repack_q80_kernel(const uint8_t* __restrict__ raw, uint8_t* __restrict__ out, long long rows, int K,
                                  long long row_bytes, int inverse) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // one thread per (row, block, 2-byte unit)
  const int nb = K >> 5;
  const long long per_row = (long long)nb * 17;
  const long long r = i / per_row;
  if (r >= rows) return;
  const int rem = (int)(i % per_row);
  const int b = rem / 17, u = rem % 17;
  const size_t g = (size_t)r * nb * 34 + (size_t)b * 34 + u * 2;                    // GGUF offset
  const size_t d = (size_t)r * row_bytes + (u == 0 ? (size_t)K + b * 2 : (size_t)b * 32 + (u - 1) * 2);
  if (!inverse) {
    out[d] = raw[g];
    out[d + 1] = raw[g + 1];
  } else {
    out[g] = raw[d];
    out[g + 1] = raw[d + 1];
  }
}

}  // namespace

// Device bytes needed for `rows` rows of K columns of GGML type `qtype`.
HE_API long long he_device_row_bytes(int qtype, int K) { return hegemv::row_bytes_dev(qtype, K); }

// inverse = 0: GGUF bytes -> device layout; inverse = 1: device layout -> GGUF bytes.
HE_API int he_repack(const void* src, void* dst, int qtype, long long rows, long long K, int inverse,
                     cudaStream_t stream) {
  if (qtype == HE_Q6_K) {
    const long long nblk = rows * (K / 256), n = nblk * 112;
    repack_q6k_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)src, (uint8_t*)dst, nblk,
                                                                        inverse);
  } else if (qtype == HE_Q8_0) {
    const long long n = rows * (K / 32) * 17;
    const long long rb = hegemv::row_bytes_dev(HE_Q8_0, (int)K);
    if (!inverse) cudaMemsetAsync(dst, 0, (size_t)(rows * rb), stream);
    repack_q80_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)src, (uint8_t*)dst, rows, (int)K,
                                                                        rb, inverse);
  } else {
    return -HE_ERR_BAD_ARG;
  }
  HE_LAUNCH_CHECK();
  return 0;
}

namespace {

// Exact fp32 value of element e of row n (same operation order as the GGUF reference dequantizers).
__device__ __forceinline__ float dequant_elem(const uint8_t* w, int qtype, long long n, int K, int e) {
  const uint8_t* row = w + (size_t)n * hegemv::row_bytes_dev(qtype, K);
  if (qtype == HE_Q4_K) {
    const uint8_t* blk = row + (size_t)(e >> 8) * 144;
    const int ib = e & 255, sb = ib >> 5, l = ib & 31;
    int sc, m;
    k4_scale_min(blk + 4, sb, sc, m);
    const float d = half_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk));
    const float dmin = half_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 2));
    const uint8_t byte = blk[16 + (sb >> 1) * 32 + l];
    const int q = (sb & 1) ? (byte >> 4) : (byte & 15);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)m));
  } else if (qtype == HE_Q6_K) {
    const uint8_t* blk = row + (size_t)(e >> 8) * 224;
    const int ib = e & 255, half = ib >> 7, qt = (ib & 127) >> 5, l = ib & 31;
    const uint8_t lq = blk[half * 64 + (qt & 1) * 32 + l];
    const uint8_t hq = blk[128 + half * 32 + l];
    const int lo = (qt >= 2) ? (lq >> 4) : (lq & 15);
    const int hi = (hq >> (2 * qt)) & 3;
    const int q = (lo | (hi << 4)) - 32;
    const int8_t sc = reinterpret_cast<const int8_t*>(blk + 192)[half * 8 + 2 * qt + (l >> 4)];
    const float d = half_bits_to_f32(*reinterpret_cast<const uint16_t*>(blk + 208));
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
  } else if (qtype == HE_Q8_0) {
    const int8_t q = reinterpret_cast<const int8_t*>(row)[e];
    const float d = half_bits_to_f32(reinterpret_cast<const uint16_t*>(row + K)[e >> 5]);
    return __fmul_rn(d, (float)q);
  } else if (qtype == HE_F32) {
    return reinterpret_cast<const float*>(row)[e];
  } else if (qtype == HE_BF16) {
    return bf16_to_f32(reinterpret_cast<const __nv_bfloat16*>(row)[e]);
  } else {
    return __half2float(reinterpret_cast<const __half*>(row)[e]);
  }
}

__global__ void dequant_bf16_kernel(const uint8_t* __restrict__ w, __nv_bfloat16* __restrict__ out, int qtype,
                                    long long row0, long long rows, int K) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= rows * K) return;
  const long long n = i / K;
  const int e = (int)(i % K);
  __align__(16) __nv_bfloat16 v[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) v[t] = f32_to_bf16(dequant_elem(w, qtype, row0 + n, K, e + t));
  *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(v);
}

__global__ void embed_kernel(const uint8_t* __restrict__ w, int qtype, long long vocab, int K,
                             const int64_t* __restrict__ ids, float* __restrict__ out, float scale, int n_tok) {
  pdl_wait();      // launched with programmatic stream serialization: order after all earlier kernels
  pdl_launch();
  const int t = blockIdx.x;
  if (t >= n_tok) return;
  long long id = ids[t];
  if (!HE_INDEX_OK(id, vocab, HE_SITE_EMBED_TOKEN) || id < 0 || id >= vocab) id = 0;
  for (int e = threadIdx.x; e < K; e += blockDim.x)
    out[(size_t)t * K + e] = dequant_elem(w, qtype, id, K, e) * scale;
}

}  // namespace

// Dequantize rows [row0, row0+rows) of a device-layout weight into bf16 [rows][K] (exact value, RNE to bf16).
HE_API int he_dequant_bf16(const void* w, void* out, int qtype, long long row0, long long rows, long long n_total,
                           int K, cudaStream_t stream) {
  (void)n_total;
  if (K % 8 != 0) return -HE_ERR_BAD_ARG;
  const long long n = rows * K / 8;
  dequant_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const uint8_t*)w, (__nv_bfloat16*)out, qtype,
                                                                        row0, rows, K);
  HE_LAUNCH_CHECK();
  return 0;
}

// out[t][:] = dequant(table[ids[t]]) * scale   (fp32 residual stream rows)
HE_API int he_embed(const void* w, int qtype, long long vocab, int K, const void* ids, void* out, float scale,
                    int n_tok, cudaStream_t stream) {
  if (n_tok <= 0) return 0;
  (void)launch_pdl(embed_kernel, dim3(n_tok), dim3(256), 0, stream, (const uint8_t*)w, qtype, vocab, K, (const int64_t*)ids, (float*)out, scale,
                                          n_tok);
  HE_LAUNCH_CHECK();
  return 0;
}
