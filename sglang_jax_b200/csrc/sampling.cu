// Sort-free filtered sampling: temperature, top-k, top-p and min-p filtering followed by hashed
// Gumbel-max sampling, one CTA per row of the logits, no scratch in global memory.
//
// The three filters each keep a prefix of the row sorted by probability, so their intersection is
// `{ i : e_i >= tau }` for one threshold tau, where e_i = exp(x_i / T - max) (so e_max = 1):
//   top-k   keeps i while  count(e > e_i)            <  k
//   top-p   keeps i while  sum(e_j : e_j > e_i)      <  top_p * sum(e)
//   min-p   keeps i while  e_i                       >= min_p
// tau is found exactly by a three-level radix select on the bit pattern of e (12 + 10 + 10 bits,
// positive floats order like their bit patterns): each level histograms counts and masses of one
// digit in shared memory, a block-wide suffix scan finds the lowest digit whose largest member still
// passes, and the next level refines inside it.  Masses are accumulated in 2^-40 fixed point, which
// makes the result independent of the order of the atomics.  Ties at tau are all kept.
//
// The draw reproduces the seeded sampler of the reference (python/sgl_jax/srt/layers/sampler.py:250-293):
//   step_seed = seed * 19349663 ^ position * 73856093,  hash = step_seed * 805306457 ^ col * 479001599   (int32 wrap)
//   u = (hash mod 2^24) / 2^24,  token = argmax_i log(p_i + 1e-9) - log(-log(u_i + 1e-9) + 1e-9)
// with p the filtered, renormalised probabilities.  That hash is kept bit for bit for requests that carry
// a seed (`hash_mode` 0); its uniforms are correlated across neighbouring columns, so draws without a
// request seed (`hash_mode` 1) pass (step_seed, col) through a 32-bit avalanche mix instead.
// Rows with top_k <= 1 return the first maximal index.
#include <float.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int kSampleThreads = 1024;
constexpr int kBins = 1024;
constexpr float kFix = 1099511627776.f;       // 2^40
constexpr float kInvFix = 1.f / 1099511627776.f;

template <typename T>
__device__ __forceinline__ float ldf(const T* p, int i) {
  if constexpr (sizeof(T) == 2) return __bfloat162float(p[i]);
  else return p[i];
}

// exp(x / T - max) in [0, 1]; NaN counts as 0.  The product is rounded on its own (no fused multiply-add
// with the subtraction), exactly as in the pass that took the maximum, so the largest entry gives exp(0) = 1
// and nothing exceeds it.
template <typename T>
__device__ __forceinline__ float expo(const T* x, int i, float inv_t, float m) {
  const float e = __expf(__fmul_rn(ldf(x, i), inv_t) - m);
  return e <= 1.f ? e : (e > 1.f ? 1.f : 0.f);
}

struct Smem {
  int cnt[kBins];
  unsigned long long mass[kBins];
  unsigned long long red_u[32];
  float red_f[32];
  int red_i[32];
  int sel;
  int sel_c;
  unsigned long long sel_s;
};

__device__ __forceinline__ float block_max(float v, Smem& sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm.red_f[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sm.red_f[0];
#pragma unroll
  for (int i = 1; i < kSampleThreads / 32; ++i) r = fmaxf(r, sm.red_f[i]);
  return r;
}

__device__ __forceinline__ unsigned long long block_sum_u64(unsigned long long v, Smem& sm) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm.red_u[threadIdx.x >> 5] = v;
  __syncthreads();
  unsigned long long r = 0;
#pragma unroll
  for (int i = 0; i < kSampleThreads / 32; ++i) r += sm.red_u[i];
  return r;
}

// Lowest digit whose largest member passes top-k / top-p given the count and mass above the current
// prefix (`carry_*`).  Thread t owns digit kBins - 1 - t, so a prefix scan over threads is a suffix
// scan over digits.  Updates the carries to the count and mass strictly above the chosen digit.
__device__ __forceinline__ int select_digit(Smem& sm, int k, unsigned long long p_mass, int& carry_c,
                                            unsigned long long& carry_s) {
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int d = kBins - 1 - tid;
  const int c = sm.cnt[d];
  const unsigned long long s = sm.mass[d];
  int ic = c;
  unsigned long long is = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int tc = __shfl_up_sync(0xffffffffu, ic, o);
    const unsigned long long ts = __shfl_up_sync(0xffffffffu, is, o);
    if (lane >= o) {
      ic += tc;
      is += ts;
    }
  }
  __syncthreads();
  if (lane == 31) {
    sm.red_i[w] = ic;
    sm.red_u[w] = is;
  }
  if (tid == 0) sm.sel = -1;
  __syncthreads();
  int oc = 0;
  unsigned long long os = 0;
  for (int i = 0; i < w; ++i) {
    oc += sm.red_i[i];
    os += sm.red_u[i];
  }
  const int above_c = carry_c + oc + ic - c;
  const unsigned long long above_s = carry_s + os + is - s;
  const bool ok = c > 0 && ((above_c < k && above_s < p_mass) || above_c == 0);
  if (ok) atomicMax(&sm.sel, tid);
  __syncthreads();
  if (tid == sm.sel) {
    sm.sel_c = above_c;
    sm.sel_s = above_s;
  }
  __syncthreads();
  carry_c = sm.sel_c;
  carry_s = sm.sel_s;
  return kBins - 1 - sm.sel;
}

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(int* __restrict__ out, float* __restrict__ probs_out, const T* __restrict__ logits, long long row_stride,
              int V, const float* __restrict__ temps, const int* __restrict__ top_ks, const float* __restrict__ top_ps,
              const float* __restrict__ min_ps, const int* __restrict__ seeds, const int* __restrict__ positions,
              int hash_mode) {
  __shared__ Smem sm;
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + row * row_stride;
  int k = top_ks[row];
  if (k > V) k = V;

  if (k <= 1) {                                            // greedy row: first maximal index
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = tid; i < V; i += kSampleThreads) {
      const float v = ldf(x, i);
      if (v > best) {
        best = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if ((tid & 31) == 0) {
      sm.red_f[tid >> 5] = best;
      sm.red_i[tid >> 5] = bi;
    }
    __syncthreads();
    if (tid == 0) {
      for (int i = 1; i < kSampleThreads / 32; ++i)
        if (sm.red_f[i] > best || (sm.red_f[i] == best && sm.red_i[i] < bi)) {
          best = sm.red_f[i];
          bi = sm.red_i[i];
        }
      out[row] = bi == 0x7fffffff ? 0 : bi;
    }
    if (probs_out != nullptr)
      for (int i = tid; i < V; i += kSampleThreads) probs_out[static_cast<size_t>(row) * V + i] = 0.f;
    return;
  }

  const float inv_t = 1.f / fmaxf(temps[row], 1e-6f);
  const float top_p = top_ps[row];
  const float min_p = min_ps[row];
  const bool need_kp = k < V || top_p < 1.f;

  float m = -FLT_MAX;
  for (int i = tid; i < V; i += kSampleThreads) m = fmaxf(m, __fmul_rn(ldf(x, i), inv_t));
  m = block_max(m, sm);

  // level 1: digit = bits >> 20 (e <= 1 -> at most 0x3F8), plus the total mass
  for (int i = tid; i < kBins; i += kSampleThreads) {
    sm.cnt[i] = 0;
    sm.mass[i] = 0;
  }
  __syncthreads();
  unsigned long long local = 0;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float e = expo(x, i, inv_t, m);
    const unsigned long long q = static_cast<unsigned long long>(e * kFix);
    local += q;
    if (need_kp) {
      const unsigned d = __float_as_uint(e) >> 20;
      atomicAdd(&sm.cnt[d], 1);
      atomicAdd(&sm.mass[d], q);
    }
  }
  const unsigned long long total = block_sum_u64(local, sm);
  unsigned tau = 0;
  unsigned long long kept_mass = total;
  if (need_kp) {
    const unsigned long long p_mass = top_p >= 1.f ? ~0ull
                                                   : static_cast<unsigned long long>(static_cast<double>(fmaxf(top_p, 0.f)) *
                                                                                     static_cast<double>(total));
    int carry_c = 0;
    unsigned long long carry_s = 0;
    const unsigned d1 = select_digit(sm, k, p_mass, carry_c, carry_s);
    // level 2: digit = (bits >> 10) & 1023 among members of d1
    for (int i = tid; i < kBins; i += kSampleThreads) {
      sm.cnt[i] = 0;
      sm.mass[i] = 0;
    }
    __syncthreads();
    for (int i = tid; i < V; i += kSampleThreads) {
      const float e = expo(x, i, inv_t, m);
      const unsigned b = __float_as_uint(e);
      if ((b >> 20) == d1) {
        atomicAdd(&sm.cnt[(b >> 10) & 1023], 1);
        atomicAdd(&sm.mass[(b >> 10) & 1023], static_cast<unsigned long long>(e * kFix));
      }
    }
    __syncthreads();
    const unsigned d2 = select_digit(sm, k, p_mass, carry_c, carry_s);
    // level 3: digit = bits & 1023 among members of (d1, d2)
    for (int i = tid; i < kBins; i += kSampleThreads) {
      sm.cnt[i] = 0;
      sm.mass[i] = 0;
    }
    __syncthreads();
    const unsigned hi = (d1 << 10) | d2;
    for (int i = tid; i < V; i += kSampleThreads) {
      const float e = expo(x, i, inv_t, m);
      const unsigned b = __float_as_uint(e);
      if ((b >> 10) == hi) {
        atomicAdd(&sm.cnt[b & 1023], 1);
        atomicAdd(&sm.mass[b & 1023], static_cast<unsigned long long>(e * kFix));
      }
    }
    __syncthreads();
    const unsigned d3 = select_digit(sm, k, p_mass, carry_c, carry_s);
    tau = (hi << 10) | d3;
    kept_mass = carry_s + sm.mass[d3];
  }
  const unsigned t_min = min_p > 0.f ? __float_as_uint(fminf(min_p, 1.f)) : 0u;
  if (t_min > tau) {                                       // min-p cuts deeper: its mass needs one more pass
    tau = t_min;
    unsigned long long lm = 0;
    for (int i = tid; i < V; i += kSampleThreads) {
      const float e = expo(x, i, inv_t, m);
      if (__float_as_uint(e) >= tau) lm += static_cast<unsigned long long>(e * kFix);
    }
    kept_mass = block_sum_u64(lm, sm);
  }
  const float inv_z = 1.f / fmaxf(static_cast<float>(kept_mass) * kInvFix, 1e-30f);

  const unsigned step_seed = (static_cast<unsigned>(seeds[row]) * 19349663u) ^ (static_cast<unsigned>(positions[row]) * 73856093u);
  const unsigned mixed = step_seed * 805306457u;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float e = expo(x, i, inv_t, m);
    const float p = __float_as_uint(e) >= tau ? e * inv_z : 0.f;
    if (probs_out != nullptr) probs_out[static_cast<size_t>(row) * V + i] = p;
    unsigned h = mixed ^ (static_cast<unsigned>(i) * 479001599u);
    if (hash_mode != 0) {
      h = (mixed + static_cast<unsigned>(i) * 0x9E3779B9u) ^ step_seed;
      h ^= h >> 16;
      h *= 0x85ebca6bu;
      h ^= h >> 13;
      h *= 0xc2b2ae35u;
      h ^= h >> 16;
      h >>= 8;
    }
    const float u = static_cast<float>(h & 0xffffffu) * (1.f / 16777216.f);
    const float score = logf(p + 1e-9f) - logf(-logf(u + 1e-9f) + 1e-9f);
    if (score > best) {
      best = score;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  __syncthreads();
  if ((tid & 31) == 0) {
    sm.red_f[tid >> 5] = best;
    sm.red_i[tid >> 5] = bi;
  }
  __syncthreads();
  if (tid == 0) {
    for (int i = 1; i < kSampleThreads / 32; ++i)
      if (sm.red_f[i] > best || (sm.red_f[i] == best && sm.red_i[i] < bi)) {
        best = sm.red_f[i];
        bi = sm.red_i[i];
      }
    out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace
}  // namespace sglb

// `logits [B, V]` (fp32: dtype_bytes 4, bf16: 2; rows `row_stride` elements apart) -> `out [B]` sampled ids.
// `probs_out` (nullable, fp32 `[B, V]` contiguous) receives the filtered, renormalised probabilities.
extern "C" int sglb_sample_filtered(int* out, float* probs_out, const void* logits, int B, int V, long long row_stride,
                                    int dtype_bytes, const float* temperatures, const int* top_ks, const float* top_ps,
                                    const float* min_ps, const int* seeds, const int* positions, int hash_mode,
                                    cudaStream_t s) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (V <= 0 || (dtype_bytes != 2 && dtype_bytes != 4)) return -kBadArgument;
  if (dtype_bytes == 4)
    sample_kernel<float><<<B, kSampleThreads, 0, s>>>(out, probs_out, static_cast<const float*>(logits), row_stride, V,
                                                      temperatures, top_ks, top_ps, min_ps, seeds, positions, hash_mode);
  else
    sample_kernel<__nv_bfloat16><<<B, kSampleThreads, 0, s>>>(out, probs_out, static_cast<const __nv_bfloat16*>(logits),
                                                              row_stride, V, temperatures, top_ks, top_ps, min_ps, seeds,
                                                              positions, hash_mode);
  return static_cast<int>(cudaGetLastError());
}
