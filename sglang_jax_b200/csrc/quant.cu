// Dynamic per-token FP8 (e4m3) activation quantisation feeding the fp8 tensor-core GEMMs:
//   q[t, :] = round_e4m3(x[t, :] / s[t]),  s[t] = max|x[t, :]| / 448.
// One CTA per row, two passes over the row (the second one hits L1/L2), 16-byte loads and
// 8-byte stores.  The gated variant reads `[T, 2K]` (gate | up), applies silu(gate) * up on
// the fly and quantises the product, so the bf16 intermediate of the expert FFN is never
// written (reference semantics: python/sgl_jax/srt/utils/quantization/quantization_utils.py
// `quantize_tensor`, python/sgl_jax/srt/layers/moe.py activation quantisation before each expert GEMM).
#include <cuda_fp8.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr float kE4m3Max = 448.f;

__device__ __forceinline__ void unpack8q(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <bool GATED>
__device__ __forceinline__ void load_row_vec(const uint4* row, int v, int nvec, float* f) {
  unpack8q(row[v], f);
  if constexpr (GATED) {
    float u[8];
    unpack8q(row[nvec + v], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = f[e] / (1.f + __expf(-f[e])) * u[e];
  }
}

template <bool GATED>
__global__ void quant_fp8_rows_kernel(uint8_t* __restrict__ q, float* __restrict__ scale,
                                      const __nv_bfloat16* __restrict__ x, int K, const int* __restrict__ valid_rows) {
  const size_t t = blockIdx.x;
  if (valid_rows != nullptr && static_cast<int>(t) >= *valid_rows) return;
  const int nvec = K >> 3;
  const uint4* row = reinterpret_cast<const uint4*>(x + t * static_cast<size_t>(GATED ? 2 * K : K));
  __shared__ float red[32];
  float m = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load_row_vec<GATED>(row, v, nvec, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(f[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = m;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  m = 0.f;
  for (int i = 0; i < nw; ++i) m = fmaxf(m, red[i]);
  // NaN / inf inputs keep the row finite on the quantised side: the scale saturates
  const float s = fmaxf(fminf(m, 3.0e38f) / kE4m3Max, 1e-12f);
  if (threadIdx.x == 0) scale[t] = s;
  const float inv = 1.f / s;
  uint2* dst = reinterpret_cast<uint2*>(q + t * static_cast<size_t>(K));
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load_row_vec<GATED>(row, v, nvec, f);
    uint32_t pk[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t word = 0;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const float2 pr = make_float2(f[4 * h + 2 * p] * inv, f[4 * h + 2 * p + 1] * inv);
        const uint32_t two = __nv_cvt_float2_to_fp8x2(pr, __NV_SATFINITE, __NV_E4M3);
        word |= two << (16 * p);
      }
      pk[h] = word;
    }
    dst[v] = make_uint2(pk[0], pk[1]);
  }
}

// Short rows (K <= 4096): one warp per row, eight rows per CTA, shuffle-only reduction.
template <bool GATED>
__global__ void quant_fp8_rows_warp_kernel(uint8_t* __restrict__ q, float* __restrict__ scale,
                                           const __nv_bfloat16* __restrict__ x, long long T, int K,
                                           const int* __restrict__ valid_rows) {
  const long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long limit = valid_rows != nullptr ? min(static_cast<long long>(*valid_rows), T) : T;
  if (t >= limit) return;
  const int lane = threadIdx.x & 31;
  const int nvec = K >> 3;
  const uint4* row = reinterpret_cast<const uint4*>(x + t * static_cast<size_t>(GATED ? 2 * K : K));
  float m = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float f[8];
    load_row_vec<GATED>(row, v, nvec, f);
#pragma unroll
    for (int e = 0; e < 8; ++e) m = fmaxf(m, fabsf(f[e]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float s = fmaxf(fminf(m, 3.0e38f) / kE4m3Max, 1e-12f);
  if (lane == 0) scale[t] = s;
  const float inv = 1.f / s;
  uint2* dst = reinterpret_cast<uint2*>(q + t * static_cast<size_t>(K));
  for (int v = lane; v < nvec; v += 32) {
    float f[8];
    load_row_vec<GATED>(row, v, nvec, f);
    uint32_t pk[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t word = 0;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const float2 pr = make_float2(f[4 * h + 2 * p] * inv, f[4 * h + 2 * p + 1] * inv);
        word |= static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(pr, __NV_SATFINITE, __NV_E4M3)) << (16 * p);
      }
      pk[h] = word;
    }
    dst[v] = make_uint2(pk[0], pk[1]);
  }
}

}  // namespace
}  // namespace sglb

// `x [T, K]` bf16 (`gated`: `[T, 2K]`, quantises silu(x[:, :K]) * x[:, K:]) -> `q [T, K]` e4m3 and `scale [T]`.
// `valid_rows` (device int, may be null): rows at or past it are left untouched.
extern "C" int sglb_quant_fp8_rows(void* q, float* scale, const void* x, long long T, int K, int gated,
                                   const int* valid_rows, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (K % 8 || K <= 0) return -kBadArgument;
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* qq = static_cast<uint8_t*>(q);
  if (K <= 4096) {
    const unsigned blocks = static_cast<unsigned>((T + 7) / 8);
    if (gated) quant_fp8_rows_warp_kernel<true><<<blocks, 256, 0, s>>>(qq, scale, xx, T, K, valid_rows);
    else quant_fp8_rows_warp_kernel<false><<<blocks, 256, 0, s>>>(qq, scale, xx, T, K, valid_rows);
    return static_cast<int>(cudaGetLastError());
  }
  const int nvec = K / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 512) threads = 512;
  if (gated) quant_fp8_rows_kernel<true><<<static_cast<unsigned>(T), threads, 0, s>>>(qq, scale, xx, K, valid_rows);
  else quant_fp8_rows_kernel<false><<<static_cast<unsigned>(T), threads, 0, s>>>(qq, scale, xx, K, valid_rows);
  return static_cast<int>(cudaGetLastError());
}
