// Decode-step kernels of the linear-attention token mixers (Gated DeltaNet of Qwen3-Next / Qwen3.5,
// Kimi Delta Attention): the per-request recurrent state lives in a slot pool and is updated in place.
//
//   delta_rule_step   S <- diag-or-scalar decay * S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q
//                     one CTA per (request, value head); thread j owns column j of the [Dk, Dv] state and
//                     walks it twice (the second walk hits L1 / L2), so DRAM sees the state once in each
//                     direction: the step is bound by those 2 * Dk * Dv * 4 bytes.
//   conv1d_update     short causal convolution over the last K inputs of every channel + SiLU, shifting
//                     the per-request window in place.
//
// Reference math: python/sgl_jax/srt/kernels/gdn/gated_delta.py (recurrent form),
// python/sgl_jax/srt/kernels/kda/kda.py, python/sgl_jax/srt/layers/attention/linear/short_convolution.py.
#include <math.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int kMaxDk = 256;

__global__ void delta_rule_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                       const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                                       const float* __restrict__ beta, float* __restrict__ state,
                                       const long long* __restrict__ slots, __nv_bfloat16* __restrict__ out, int H,
                                       int Hqk, int DK, int Dv, int gate_per_channel, int l2norm) {
  const int b = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int hq = h / (H / Hqk);                       // q / k heads may be shared by several value heads
  __shared__ float qs[kMaxDk], ks[kMaxDk], decay[kMaxDk];
  __shared__ float red[3][8];
  const __nv_bfloat16* qp = q + (static_cast<size_t>(b) * Hqk + hq) * DK;
  const __nv_bfloat16* kp = k + (static_cast<size_t>(b) * Hqk + hq) * DK;
  float qv = 0.f, kv = 0.f, kq = 0.f;
  for (int i = j; i < DK; i += blockDim.x) {
    const float qi = __bfloat162float(qp[i]), ki = __bfloat162float(kp[i]);
    qs[i] = qi;
    ks[i] = ki;
    qv += qi * qi;
    kv += ki * ki;
    kq += ki * qi;
    decay[i] = __expf(gate_per_channel ? g[(static_cast<size_t>(b) * H + h) * DK + i] : g[static_cast<size_t>(b) * H + h]);
  }
  // block-wide sums: |q|^2, |k|^2 for the L2 normalisation, k.q for the closed form of the output
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    qv += __shfl_xor_sync(0xffffffffu, qv, o);
    kv += __shfl_xor_sync(0xffffffffu, kv, o);
    kq += __shfl_xor_sync(0xffffffffu, kq, o);
  }
  if ((j & 31) == 0) {
    red[0][j >> 5] = qv;
    red[1][j >> 5] = kv;
    red[2][j >> 5] = kq;
  }
  __syncthreads();
  float qn = 0.f, kn = 0.f, kqs = 0.f;
  for (int w = 0; w < (blockDim.x + 31) / 32; ++w) {
    qn += red[0][w];
    kn += red[1][w];
    kqs += red[2][w];
  }
  const float qscale = (l2norm ? rsqrtf(qn + 1e-6f) : 1.f) * rsqrtf(static_cast<float>(DK));
  const float kscale = l2norm ? rsqrtf(kn + 1e-6f) : 1.f;
  if (j >= Dv) return;
  float* S = state + (static_cast<size_t>(slots[b]) * H + h) * DK * Dv + j;
  // pass 1: with s_i = decay_i S_i:  kvm = sum_i s_i k_i,  oq = sum_i s_i q_i
  float kvm = 0.f, oq = 0.f;
#pragma unroll 8
  for (int i = 0; i < DK; ++i) {
    const float si = S[static_cast<size_t>(i) * Dv] * decay[i];
    kvm += si * ks[i];
    oq += si * qs[i];
  }
  const size_t bh = static_cast<size_t>(b) * H + h;
  const float d = (__bfloat162float(v[bh * Dv + j]) - kvm * kscale) * beta[bh] * kscale;
  // pass 2 (the column is still in L1 / L2): S_i <- s_i + k_i d
#pragma unroll 8
  for (int i = 0; i < DK; ++i) {
    float* p = S + static_cast<size_t>(i) * Dv;
    *p = *p * decay[i] + ks[i] * d;
  }
  // o = sum_i (s_i + k_i d) q_i = oq + d (k . q)
  out[bh * Dv + j] = __float2bfloat16((oq + d * kqs) * qscale);
}

template <typename T>
__global__ void conv1d_update_kernel(const __nv_bfloat16* __restrict__ x, T* __restrict__ state,
                                     const __nv_bfloat16* __restrict__ weight, const long long* __restrict__ slots,
                                     __nv_bfloat16* __restrict__ y, int C, int K, int silu) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  T* st = state + (static_cast<size_t>(slots[b]) * C + c) * (K - 1);
  const __nv_bfloat16* w = weight + static_cast<size_t>(c) * K;
  const float xv = __bfloat162float(x[static_cast<size_t>(b) * C + c]);
  float acc = xv * __bfloat162float(w[K - 1]);
  for (int t = 0; t < K - 1; ++t) {
    const float sv = static_cast<float>(st[t]);
    acc += sv * __bfloat162float(w[t]);
    if (t > 0) st[t - 1] = static_cast<T>(sv);
  }
  st[K - 2] = static_cast<T>(xv);
  if (silu) acc = acc / (1.f + __expf(-acc));
  y[static_cast<size_t>(b) * C + c] = __float2bfloat16(acc);
}

}  // namespace
}  // namespace sglb

extern "C" {

// q, k [B, Hqk, Dk] bf16; v [B, H, Dv] bf16; g [B, H] (or [B, H, Dk] with gate_per_channel) fp32 log-decay;
// beta [B, H] fp32; state pool [slots, H, Dk, Dv] fp32, updated in place at `slots[b]`; out [B, H, Dv] bf16.
int sglb_delta_rule_step(const void* q, const void* k, const void* v, const float* g, const float* beta, float* state,
                         const long long* slots, void* out, int B, int H, int Hqk, int Dk, int Dv,
                         int gate_per_channel, int l2norm, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (Dv > 256 || Dv % 32 != 0 || H % Hqk != 0 || Dk > kMaxDk || Dk < 1) return -kBadArgument;
  dim3 grid(B, H);
  const int threads = Dv < 64 ? 64 : Dv;
  delta_rule_step_kernel<<<grid, threads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      g, beta, state, slots, static_cast<__nv_bfloat16*>(out), H, Hqk, Dk, Dv, gate_per_channel, l2norm);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// x [B, C] bf16; state pool [slots, C, K-1] (bf16 if state_is_bf16 else fp32), shifted in place; weight [C, K] bf16.
int sglb_conv1d_update(const void* x, void* state, const void* weight, const long long* slots, void* y, int B, int C,
                       int K, int silu, int state_is_bf16, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (K < 2 || K > 8) return -kBadArgument;
  dim3 grid((C + 127) / 128, B);
  if (state_is_bf16)
    conv1d_update_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(state),
        static_cast<const __nv_bfloat16*>(weight), slots, static_cast<__nv_bfloat16*>(y), C, K, silu);
  else
    conv1d_update_kernel<float><<<grid, 128, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<float*>(state), static_cast<const __nv_bfloat16*>(weight),
        slots, static_cast<__nv_bfloat16*>(y), C, K, silu);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // extern "C"
