// LoRA batched gather matrix-vector kernels (multi-adapter serving).
//
// Every token t carries an adapter slot s(t) (-1 = none).  Two launches per projection:
//   shrink:  h[t, :]  = A[s(t)] x[t]                 A: [slots, R, K]  (R = stack * r_max)
//   expand:  y[t, o] += scale[s(t)] * B_j[s(t)][o, :] . h[t, j*r : (j+1)*r]
// Counterpart of the reference's `lora/backend/bgmv_backend.py` einsum.  The op is bound by
// the adapter weights it streams (ranks are 8..64), so plain vectorised loads are enough:
// the shrink gives one warp per (token, output row) and reduces over K with 16-byte loads;
// the expand gives one thread per (token, 2 output columns).
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace sglb {

__global__ void lora_shrink_kernel(float* __restrict__ h, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ a, const int* __restrict__ slots, int T, int R,
                                   int K) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= static_cast<long long>(T) * R) return;
  const int t = static_cast<int>(warp / R), r = static_cast<int>(warp % R);
  const int s = slots[t];
  if (s < 0) {
    if (lane == 0) h[warp] = 0.f;
    return;
  }
  const __nv_bfloat16* xr = x + static_cast<size_t>(t) * K;
  const __nv_bfloat16* ar = a + (static_cast<size_t>(s) * R + r) * K;
  float acc = 0.f;
  const int nvec = K / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(xr);
  const uint4* av = reinterpret_cast<const uint4*>(ar);
  for (int i = lane; i < nvec; i += 32) {
    const uint4 p = __ldg(xv + i), q = __ldg(av + i);
    const uint32_t pw[4] = {p.x, p.y, p.z, p.w}, qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc += __uint_as_float(pw[e] << 16) * __uint_as_float(qw[e] << 16);
      acc += __uint_as_float(pw[e] & 0xffff0000u) * __uint_as_float(qw[e] & 0xffff0000u);
    }
  }
  for (int i = nvec * 8 + lane; i < K; i += 32) acc += __bfloat162float(xr[i]) * __bfloat162float(ar[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) h[warp] = acc;
}

// y: [T, ldy] bf16 (columns y_off .. y_off + N updated), b: [slots, N, r], h: [T, R] (columns h_off .. h_off + r)
__global__ void lora_expand_kernel(__nv_bfloat16* __restrict__ y, const float* __restrict__ h,
                                   const __nv_bfloat16* __restrict__ b, const int* __restrict__ slots,
                                   const float* __restrict__ scale, int T, int N, int r, int R, int h_off, int ldy,
                                   int y_off) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int half_n = (N + 1) / 2;
  if (idx >= static_cast<long long>(T) * half_n) return;
  const int t = static_cast<int>(idx / half_n);
  const int o = static_cast<int>(idx % half_n) * 2;
  const int s = slots[t];
  if (s < 0) return;
  const float sc = scale[s];
  const float* hr = h + static_cast<size_t>(t) * R + h_off;
  const __nv_bfloat16* b0 = b + (static_cast<size_t>(s) * N + o) * r;
  float acc0 = 0.f, acc1 = 0.f;
  const bool two = o + 1 < N;
  for (int i = 0; i < r; ++i) {
    const float hv = hr[i];
    acc0 += hv * __bfloat162float(b0[i]);
    if (two) acc1 += hv * __bfloat162float(b0[r + i]);
  }
  __nv_bfloat16* yr = y + static_cast<size_t>(t) * ldy + y_off + o;
  yr[0] = __float2bfloat16(__bfloat162float(yr[0]) + sc * acc0);
  if (two) yr[1] = __float2bfloat16(__bfloat162float(yr[1]) + sc * acc1);
}

}  // namespace sglb

extern "C" {

int sglb_lora_shrink(float* h, const void* x, const void* a, const int* slots, int T, int R, int K, cudaStream_t s) {
  if (T <= 0 || R <= 0) return 0;
  if (K % 8) return -sglb::kBadArgument;
  const long long threads = static_cast<long long>(T) * R * 32;
  const int block = 256;
  sglb::lora_shrink_kernel<<<static_cast<unsigned>((threads + block - 1) / block), block, 0, s>>>(
      h, static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(a), slots, T, R, K);
  return static_cast<int>(cudaGetLastError());
}

int sglb_lora_expand(void* y, const float* h, const void* b, const int* slots, const float* scale, int T, int N, int r,
                     int R, int h_off, int ldy, int y_off, cudaStream_t s) {
  if (T <= 0 || N <= 0) return 0;
  const long long threads = static_cast<long long>(T) * ((N + 1) / 2);
  const int block = 256;
  sglb::lora_expand_kernel<<<static_cast<unsigned>((threads + block - 1) / block), block, 0, s>>>(
      static_cast<__nv_bfloat16*>(y), h, static_cast<const __nv_bfloat16*>(b), slots, scale, T, N, r, R, h_off, ldy,
      y_off);
  return static_cast<int>(cudaGetLastError());
}
}
