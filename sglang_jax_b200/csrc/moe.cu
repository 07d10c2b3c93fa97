// Mixture-of-experts routing and token (un)permutation.
//
//   topk_route     scores = softmax | sigmoid | tanh (fp32) of router logits; optional selection bias
//                  (choose by score + bias, weigh by the unbiased score); optional group-limited
//                  routing (group score = max, or sum of the top 2 when biased; keep `topk_group`
//                  groups); top-k by repeated argmax (ties -> lowest index); optional renormalise;
//                  times `routed_scaling_factor`.
//                  Semantics: python/sgl_jax/srt/layers/gate.py:59-333 and
//                  python/sgl_jax/srt/kernels/{biased_topk,grouped_topk}/v1/kernel.py.
//   moe_align      counts the (token, k) pairs routed to this rank's experts, builds the expert
//                  row offsets, the pair -> sorted-row map and the 128-row tile list the grouped
//                  GEMM walks.
//   moe_gather     x_sorted[row] = x[token of row]
//   moe_combine    out[t] = sum_j weight[t, j] * y_sorted[row(t, j)]   (fixed j order: deterministic)
//                  = the unpermute + weighted sum of python/sgl_jax/srt/layers/moe.py:684-760.
#include <float.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int kMaxExperts = 512;
constexpr int kMaxTopK = 16;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// one warp per token; scores live in shared memory (E floats per warp)
template <typename T>
__global__ void topk_route_kernel(const T* __restrict__ logits, const float* __restrict__ bias,
                                  float* __restrict__ out_w, int* __restrict__ out_ids, int Tn, int E, int k,
                                  int scoring, int renorm, int num_groups, int topk_group, float scale) {
  extern __shared__ float smem[];
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * warps + wid;
  if (t >= Tn) return;
  float* sc = smem + wid * 2 * E;     // unbiased scores
  float* ch = sc + E;                 // selection scores (biased / group-masked)
  const T* row = logits + static_cast<size_t>(t) * E;
  // ---- scores
  float mx = -FLT_MAX;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, to_f(row[e]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float x = to_f(row[e]);
    float s;
    if (scoring == 0) s = __expf(x - mx);
    else if (scoring == 1) s = 1.f / (1.f + __expf(-x));
    else s = tanhf(x);
    sc[e] = s;
    sum += s;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncwarp();
  for (int e = lane; e < E; e += 32) {
    if (scoring == 0) sc[e] = sc[e] / sum;
    ch[e] = sc[e] + (bias != nullptr ? bias[e] : 0.f);
  }
  __syncwarp();
  // ---- group-limited routing
  if (num_groups > 1) {
    const int gs = E / num_groups;
    float gscore = -FLT_MAX;
    if (lane < num_groups) {
      float m1 = -FLT_MAX, m2 = -FLT_MAX;
      for (int i = 0; i < gs; ++i) {
        const float v = ch[lane * gs + i];
        if (v > m1) {
          m2 = m1;
          m1 = v;
        } else if (v > m2) {
          m2 = v;
        }
      }
      gscore = bias != nullptr ? m1 + m2 : m1;
    }
    // keep the topk_group best groups: a group survives if fewer than topk_group groups beat it
    int beaten = 0;
    for (int g = 0; g < num_groups; ++g) {
      const float og = __shfl_sync(0xffffffffu, gscore, g);
      if (og > gscore || (og == gscore && g < lane)) ++beaten;
    }
    const bool keep = lane < num_groups && beaten < topk_group;
    const unsigned keep_mask = __ballot_sync(0xffffffffu, keep);
    for (int e = lane; e < E; e += 32)
      if (!((keep_mask >> (e / gs)) & 1u)) ch[e] = -FLT_MAX;
    __syncwarp();
  }
  // ---- top-k by repeated argmax
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < k; ++j) {
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = ch[e];
      if (v > best || (v == best && e < bi)) {
        best = v;
        bi = e;
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
    if (bi == 0x7fffffff) bi = 0;
    const float w = sc[bi];
    wsum += w;
    if (lane == j) {
      my_w = w;
      my_id = bi;
    }
    __syncwarp();
    if (lane == 0) ch[bi] = -FLT_MAX;
    __syncwarp();
  }
  if (lane < k) {
    float w = my_w;
    if (renorm) w = w / fmaxf(wsum, 1e-20f);
    out_w[static_cast<size_t>(t) * k + lane] = w * scale;
    out_ids[static_cast<size_t>(t) * k + lane] = my_id;
  }
}

// Single CTA.  pairs = T * k.  Experts [e0, e0 + E_local) are local.
//   offsets[E_local + 1], pair_row[pairs] (sorted row or -1), row_token[rows_cap] (token of each
//   sorted row), tile lists for the prefill-shaped grouped GEMM, counts[0] = number of local rows,
//   counts[1] = number of token tiles.
__global__ void moe_align_kernel(const int* __restrict__ topk_ids, int pairs, int k, int e0, int E_local,
                                 int* __restrict__ offsets, int* __restrict__ pair_row, int* __restrict__ row_token,
                                 int* __restrict__ tile_group, int* __restrict__ tile_row0, int* __restrict__ counts,
                                 int* __restrict__ expert_hist /* [E_local] optional, accumulates */) {
  __shared__ int cnt[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  __shared__ int fill[kMaxExperts];
  for (int e = threadIdx.x; e < E_local; e += blockDim.x) {
    cnt[e] = 0;
    fill[e] = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - e0;
    if (e >= 0 && e < E_local) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0, tiles = 0;
    for (int e = 0; e < E_local; ++e) {
      off[e] = acc;
      for (int r = 0; r < cnt[e]; r += 128) {
        tile_group[tiles] = e;
        tile_row0[tiles] = acc + r;
        ++tiles;
      }
      acc += cnt[e];
    }
    off[E_local] = acc;
    counts[0] = acc;
    counts[1] = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E_local; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < E_local && expert_hist != nullptr) expert_hist[e] += cnt[e];
  }
  __syncthreads();
  // Row order inside an expert is whatever the atomics produce; every sorted row is computed
  // independently of its neighbours and the combine step sums in (token, j) order, so results do
  // not depend on it.
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i] - e0;
    if (e >= 0 && e < E_local) {
      const int row = off[e] + atomicAdd(&fill[e], 1);
      pair_row[i] = row;
      row_token[row] = i / k;
    } else {
      pair_row[i] = -1;
    }
  }
}

__global__ void moe_gather_kernel(__nv_bfloat16* __restrict__ x_sorted, const __nv_bfloat16* __restrict__ x,
                                  const int* __restrict__ row_token, const int* __restrict__ counts, int H) {
  const int row = blockIdx.x;
  if (row >= counts[0]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row_token[row]) * H);
  uint4* dst = reinterpret_cast<uint4*>(x_sorted + static_cast<size_t>(row) * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = src[i];
}

// out[t] (+)= sum_j w[t, j] * y[pair_row[t*k + j]]; pairs routed elsewhere contribute nothing.
__global__ void moe_combine_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ y,
                                   const float* __restrict__ w, const int* __restrict__ pair_row, int k, int H,
                                   const __nv_bfloat16* __restrict__ add /* optional [T, H] (shared expert) */) {
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (add != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(add + t * H)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int j = 0; j < k; ++j) {
      const int row = pair_row[t * k + j];
      if (row < 0) continue;
      const float wj = w[t * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(y + static_cast<size_t>(row) * H)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += wj * f.x;
        acc[2 * e + 1] += wj * f.y;
      }
    }
    reinterpret_cast<uint4*>(out + t * H)[i] =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

}  // namespace
}  // namespace sglb

extern "C" {

// scoring: 0 softmax, 1 sigmoid, 2 tanh.  logits fp32 (dtype_bytes 4) or bf16 (2).  bias fp32 or null.
int sglb_topk_route(const void* logits, int dtype_bytes, const float* bias, float* out_w, int* out_ids, int T, int E,
                    int k, int scoring, int renorm, int num_groups, int topk_group, float scale, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (E > kMaxExperts || k > kMaxTopK || k > 32 || k > E || (num_groups > 1 && (E % num_groups || num_groups > 32)))
    return -kBadArgument;
  const int warps = 4;
  const int blocks = (T + warps - 1) / warps;
  const size_t smem = warps * 2 * E * sizeof(float);
  if (dtype_bytes == 4)
    topk_route_kernel<float><<<blocks, warps * 32, smem, s>>>(static_cast<const float*>(logits), bias, out_w, out_ids, T,
                                                             E, k, scoring, renorm, num_groups, topk_group, scale);
  else
    topk_route_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, s>>>(static_cast<const __nv_bfloat16*>(logits), bias,
                                                                      out_w, out_ids, T, E, k, scoring, renorm,
                                                                      num_groups, topk_group, scale);
  return static_cast<int>(cudaGetLastError());
}

int sglb_moe_align(const int* topk_ids, int pairs, int k, int e0, int E_local, int* offsets, int* pair_row,
                   int* row_token, int* tile_group, int* tile_row0, int* counts, int* expert_hist, cudaStream_t s) {
  using namespace sglb;
  if (E_local > kMaxExperts) return -kBadArgument;
  moe_align_kernel<<<1, 1024, 0, s>>>(topk_ids, pairs, k, e0, E_local, offsets, pair_row, row_token, tile_group,
                                      tile_row0, counts, expert_hist);
  return static_cast<int>(cudaGetLastError());
}

int sglb_moe_gather(void* x_sorted, const void* x, const int* row_token, const int* counts, int max_rows, int H,
                    cudaStream_t s) {
  using namespace sglb;
  if (max_rows <= 0) return 0;
  if (H % 8) return -kBadArgument;
  moe_gather_kernel<<<max_rows, 128, 0, s>>>(static_cast<__nv_bfloat16*>(x_sorted),
                                             static_cast<const __nv_bfloat16*>(x), row_token, counts, H);
  return static_cast<int>(cudaGetLastError());
}

int sglb_moe_combine(void* out, const void* y, const float* w, const int* pair_row, int T, int k, int H,
                     const void* add, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (H % 8) return -kBadArgument;
  moe_combine_kernel<<<T, 128, 0, s>>>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(y), w,
                                       pair_row, k, H, static_cast<const __nv_bfloat16*>(add));
  return static_cast<int>(cudaGetLastError());
}
}
