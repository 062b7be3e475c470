// Shared device/host helpers for the sm_100a kernel library.
//
// Every launcher in this library is an `extern "C"` function that takes raw
// device pointers plus a stream and returns 0 on success or a CUDA error code.
// Nothing here allocates; callers (PyTorch tensors) own all memory.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define HE_API extern "C" __attribute__((visibility("default")))

// GGML type codes used across the C ABI (same numbering as the GGUF file format).
enum HeQType : int {
  HE_F32 = 0,
  HE_F16 = 1,
  HE_Q8_0 = 8,
  HE_Q4_K = 12,
  HE_Q6_K = 14,
  HE_BF16 = 30,
};

// Status-word codes written by kernels whose bounded waits or checks gave up.
enum HeStatus : int {
  HE_OK = 0,
  HE_ERR_WAIT_TIMEOUT = 1,
  HE_ERR_BOUNDS = 2,
  HE_ERR_BAD_ARG = 3,
};

#define HE_LAUNCH_CHECK()                                   \
  do {                                                      \
    cudaError_t _e = cudaGetLastError();                    \
    if (_e != cudaSuccess) return (int)_e;                  \
  } while (0)

// ---------------------------------------------------------------- range checks of the "checked" library variant
// Built with -DHE_BOUNDS_CHECK=1 (library variant "checked"), every index that a kernel takes from device data
// (token ids, block-table pages, expert ids, row selectors) is tested against its limit before it is used; a violation
// records {HE_ERR_BOUNDS, site, index, limit} in a per-translation-unit device word and the access is skipped or the
// index clamped -- never performed out of range.  he_bounds_status() collects the words.  In the product build
// HE_INDEX_OK() is the constant true and none of this exists.  (The role compute-sanitizer's memcheck would play;
// the reference plans the same status-word build for its bounds checks.)
enum HeBoundsSite : int {
  HE_SITE_EMBED_TOKEN = 1,
  HE_SITE_KV_WRITE_PAGE = 2,
  HE_SITE_ATTN_DECODE_PAGE = 3,
  HE_SITE_MOE_EXPERT_ID = 4,
  HE_SITE_GATHER_ROW = 5,
  HE_SITE_STATE_SLOT = 6,
};

#if defined(HE_BOUNDS_CHECK) && defined(__CUDACC__)
typedef int (*HeBoundsReader)(int* out4, int reset);
extern "C" void he_bounds_register_reader(HeBoundsReader fn);   // runtime.cpp
namespace he {
static __device__ int g_bounds_word[4];
__device__ __forceinline__ bool bounds_ok(long long idx, long long lim, int site) {
  if (idx >= 0 && idx < lim) return true;
  if (atomicCAS(&g_bounds_word[0], 0, (int)HE_ERR_BOUNDS) == 0) {
    g_bounds_word[1] = site;
    g_bounds_word[2] = (int)idx;
    g_bounds_word[3] = (int)lim;
  }
  return false;
}
static int bounds_read_tu(int* out4, int reset) {
  int w[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(w, g_bounds_word, sizeof(w)) != cudaSuccess) return -1;
  if (reset && w[0] != 0) {
    const int z[4] = {0, 0, 0, 0};
    cudaMemcpyToSymbol(g_bounds_word, z, sizeof(z));
  }
  for (int i = 0; i < 4; ++i) out4[i] = w[i];
  return w[0];
}
struct BoundsRegistration {
  BoundsRegistration() { he_bounds_register_reader(&bounds_read_tu); }
};
static BoundsRegistration g_bounds_registration;   // internal linkage: one per translation unit
}  // namespace he
#define HE_INDEX_OK(idx, lim, site) (he::bounds_ok((long long)(idx), (long long)(lim), (site)))
#else
#define HE_INDEX_OK(idx, lim, site) (true)
#endif

namespace he {

__device__ __forceinline__ float bf16_to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f32_to_bf16(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the total.  `red` must hold >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float softplus20_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg64(const void* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }

// Streaming 128-bit load that does not allocate in L1 (weights are read once per step).
__device__ __forceinline__ uint4 ldg128_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg64_stream(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ float half_bits_to_f32(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}

// Unpack the 6-bit (scale, min) pair of sub-block j (0..7) from the 12 packed bytes of a Q4_K/Q5_K block.
__device__ __forceinline__ void k4_scale_min(const uint8_t* q, int j, int& sc, int& m) {
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Same unpack from the three little-endian words holding the 12 scale bytes (no local-memory indexing).
__device__ __forceinline__ void k4_scale_min_w(uint32_t w0, uint32_t w1, uint32_t w2, int j, int& sc, int& m) {
  if (j < 4) {
    sc = (w0 >> (8 * j)) & 63;
    m = (w1 >> (8 * j)) & 63;
  } else {
    const int t = j - 4;
    sc = ((w2 >> (8 * t)) & 0xF) | (((w0 >> (8 * t + 6)) & 3) << 4);
    m = ((w2 >> (8 * t + 4)) & 0xF) | (((w1 >> (8 * t + 6)) & 3) << 4);
  }
}

// Signed byte i (0..15) of a 128-bit register quad.
__device__ __forceinline__ int byte_of(const uint4& v, int i) {
  const uint32_t w = i < 8 ? (i < 4 ? v.x : v.y) : (i < 12 ? v.z : v.w);
  return (int)(int8_t)(w >> ((i & 3) * 8));
}

}  // namespace he

// ---------------------------------------------------------------- programmatic dependent launch
// Kernels on the decode path are launched with the "programmatic stream serialization" attribute: the grid may be
// scheduled while its predecessor in the stream is still draining, which hides the launch latency between the
// many short kernels of a decode step.  Such a kernel must call pdl_wait() before it reads anything the predecessor
// wrote (or writes anything the predecessor reads); pdl_launch() lets its own successor start being scheduled.
// HE_PDL=0 in the environment turns the attribute off (plain stream order).
#include <cstdlib>
namespace he {
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;"); }

inline bool pdl_enabled() {
  static const bool on = []() {
    const char* e = getenv("HE_PDL");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
}  // namespace he
