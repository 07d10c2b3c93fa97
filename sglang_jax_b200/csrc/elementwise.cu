// Bandwidth-bound ops of the decoder layer: RMSNorm (+ fused residual add), SiLU-gate,
// embedding gather, greedy argmax, and the fused per-head q/k RMSNorm + RoPE + paged KV write.
// All are single-pass, 16-byte vectorised and keep their statistics in fp32
// (reference semantics: python/sgl_jax/srt/layers/layernorm.py:30-253,
//  python/sgl_jax/srt/layers/embeddings.py:539-601, python/sgl_jax/srt/kernels/update_kv_cache/).
#include <float.h>

#include "common.cuh"

namespace sglb {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  const float r = red[0];
  __syncthreads();
  return r;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}

// One CTA per row.  H % 8 == 0.  With ADD: residual <- x + residual (bf16), y <- norm(residual).
// Row data is kept in registers between the two passes (H <= 8 * 8 * blockDim).
template <bool ADD, int VPT>
__global__ void rmsnorm_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x,
                               __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ w, int H,
                               float eps, int gemma) {
  __shared__ float red[32];
  pdl_wait();
  const size_t row = blockIdx.x;
  const uint4* xv = reinterpret_cast<const uint4*>(x + row * H);
  uint4* rv = ADD ? reinterpret_cast<uint4*>(residual + row * H) : nullptr;
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* yv = reinterpret_cast<uint4*>(y + row * H);
  const int nvec = H >> 3;
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      unpack8(xv[idx], vals[i]);
      if (ADD) {
        float r[8];
        unpack8(rv[idx], r);
#pragma unroll
        for (int e = 0; e < 8; ++e) vals[i][e] += r[e];
        const uint4 packed = pack8(vals[i]);
        rv[idx] = packed;
        unpack8(packed, vals[i]);   // normalise the rounded sum, as the unfused sequence would
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
    }
  }
  const float tot = block_sum(ss, red);
  const float inv = rsqrtf(tot / H + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float wf[8], o[8];
      unpack8(wv[idx], wf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = vals[i][e] * inv * (gemma ? wf[e] + 1.f : wf[e]);
      yv[idx] = pack8(o);
    }
  }
}

// out[t, i] = silu(x[t, i]) * x[t, I + i]
__global__ void silu_mul_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x, long long T,
                                int I) {
  pdl_wait();
  const int nvec = I >> 3;
  const long long total = T * nvec;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = idx / nvec;
    const int v = static_cast<int>(idx - t * nvec);
    const uint4* row = reinterpret_cast<const uint4*>(x + t * 2 * I);
    float a[8], b[8], o[8];
    unpack8(row[v], a);
    unpack8(row[nvec + v], b);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = a[e] / (1.f + __expf(-a[e])) * b[e];
    reinterpret_cast<uint4*>(out + t * I)[v] = pack8(o);
  }
}

// out[t] = table[ids[t] - vocab_start] (zeros when outside this shard and `masked`)
__global__ void embedding_kernel(__nv_bfloat16* __restrict__ out, const int* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ table, int H, int rows, int vocab_start,
                                 int masked) {
  pdl_wait();
  const size_t t = blockIdx.x;
  int id = ids[t] - vocab_start;
  const bool ok = id >= 0 && id < rows;
  if (!ok) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * H);
  uint4* dst = reinterpret_cast<uint4*>(out + t * H);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = (ok || !masked) ? src[i] : z;
}

// first maximal index per row
template <typename T>
__global__ void argmax_kernel(int* __restrict__ out, const T* __restrict__ logits, int V, long long row_stride) {
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + blockIdx.x * row_stride;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  int scalar_from = 0;
  if constexpr (sizeof(T) == 2) {
    // 16-byte loads, four in flight per thread, when the row starts on a 16-byte boundary
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int nvec = V / 8;
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      constexpr int U = 4;
      for (int base = threadIdx.x; base < nvec; base += blockDim.x * U) {
        uint4 q[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int idx = base + u * blockDim.x;
          q[u] = idx < nvec ? __ldg(rv + idx) : make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int idx = base + u * blockDim.x;
          const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float v = __uint_as_float((e & 1) ? (w[e >> 1] & 0xffff0000u) : (w[e >> 1] << 16));
            const int i = idx * 8 + e;
            if (v > best || (v == best && i < bi)) {
              best = v;
              bi = i;
            }
          }
        }
      }
      scalar_from = nvec * 8;
    }
  }
  for (int i = scalar_from + threadIdx.x; i < V; i += blockDim.x) {
    float v;
    if constexpr (sizeof(T) == 2) v = __bfloat162float(row[i]);
    else v = row[i];
    if (v > best || (v == best && i < bi)) {
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
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -FLT_MAX;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (l == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// One warp per (token, head) of the fused qkv row:
//   q heads: optional RMSNorm over the head, RoPE, -> q_out[t, h, :]
//   k heads: optional RMSNorm, RoPE, -> cache[page, 0, h, off, :]
//   v heads: -> cache[page, 1, h, off, :]
// Lane l holds elements l, l+32, l+64, ... of the head, so the neox partner i + rd/2 of an element
// lives in the same lane (rd/2 is a multiple of 32).
#ifdef SGLB_BOUNDS_CHECK
// Checked build only: the extent of the KV buffers and where to report, set by sglb_debug_set_kv_pages().
__device__ int g_dbg_kv_pages = 0;
__device__ Status* g_dbg_status = nullptr;
#endif

template <int D>
__global__ void rope_qknorm_kvwrite_kernel(__nv_bfloat16* __restrict__ q_out, const __nv_bfloat16* __restrict__ qkv,
                                           const int* __restrict__ positions, const float* __restrict__ cos_sin,
                                           const __nv_bfloat16* __restrict__ q_w, const __nv_bfloat16* __restrict__ k_w,
                                           float eps, long long T, int Hq, int Hkv, int rd,
                                           __nv_bfloat16* __restrict__ kv, const int* __restrict__ loc, int page_size,
                                           int is_neox) {
  pdl_wait();
  constexpr int E = D / 32;
  const int heads = Hq + 2 * Hkv;
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  if (wid >= T * heads) return;
  const int lane = threadIdx.x & 31;
  const long long t = wid / heads;
  const int h = static_cast<int>(wid - t * heads);
  const __nv_bfloat16* src = qkv + (t * heads + h) * D;
  float v[E];
#pragma unroll
  for (int j = 0; j < E; ++j) v[j] = __bfloat162float(src[lane + 32 * j]);
  const bool is_q = h < Hq;
  const bool is_k = !is_q && h < Hq + Hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? q_w : k_w;
    if (nw != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < E; ++j) ss += v[j] * v[j];
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / D + eps);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        // round to bf16 like the unfused norm would before the rotation
        v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * __bfloat162float(nw[lane + 32 * j])));
      }
    }
    if (cos_sin != nullptr) {
      const float* cs = cos_sin + static_cast<long long>(positions[t]) * rd;
      const int half = rd >> 1;
      if (is_neox) {
        constexpr int kMaxPairs = E / 2 > 0 ? E / 2 : 1;
        const int pj = half / 32;            // register distance between partners
#pragma unroll
        for (int j = 0; j < kMaxPairs; ++j) {
          if (j < pj) {
            const int i = lane + 32 * j;     // index in the first half
            const float c = cs[i], s = cs[half + i];
            const float a = v[j], b = v[j + pj];
            v[j] = a * c - b * s;
            v[j + pj] = b * c + a * s;
          }
        }
      } else {
        // interleaved pairs (2p, 2p+1): partner sits in the neighbouring lane
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const int i = lane + 32 * j;
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          if (i < rd) {
            const int pidx = i >> 1;
            const float c = cs[pidx], s = cs[half + pidx];
            v[j] = (i & 1) ? (v[j] * c + other * s) : (v[j] * c - other * s);
          }
        }
      }
    }
  }
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (t * Hq + h) * D;
  } else {
    if (kv == nullptr) return;
    const int slot = loc[t];
    const int page = slot / page_size, off = slot - page * page_size;
#ifdef SGLB_BOUNDS_CHECK
    if (g_dbg_kv_pages > 0 && (slot < 0 || page >= g_dbg_kv_pages)) {
      if (lane == 0) report(g_dbg_status, kOutOfBounds, static_cast<int>(t), slot);
      return;
    }
#endif
    const int kvsel = is_k ? 0 : 1;
    const int hh = is_k ? h - Hq : h - Hq - Hkv;
    dst = kv + ((((static_cast<long long>(page) * 2 + kvsel) * Hkv + hh) * page_size) + off) * D;
  }
#pragma unroll
  for (int j = 0; j < E; ++j) dst[lane + 32 * j] = __float2bfloat16(v[j]);
}

// page_table[rows[i], pos[i]] = ids[i]
__global__ void page_table_scatter_kernel(int* __restrict__ table, int max_pages, const int* __restrict__ rows,
                                          const int* __restrict__ pos, const int* __restrict__ ids, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) table[static_cast<long long>(rows[i]) * max_pages + pos[i]] = ids[i];
}

// ids < 0 are placeholders -slot: replace from the future-token map (overlap scheduling)
__global__ void resolve_future_kernel(int* __restrict__ ids, const int* __restrict__ future_map, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int v = ids[i];
    if (v < 0) ids[i] = future_map[-v];
  }
}

}  // namespace
}  // namespace sglb

extern "C" {

int sglb_rmsnorm(void* y, const void* x, const void* w, long long T, int H, float eps, int gemma, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (H % 8 || H > 8 * 8 * 1024) return -kBadArgument;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  int vpt = 1;
  while (vpt * threads < nvec) vpt *= 2;
  auto* yy = static_cast<__nv_bfloat16*>(y);
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* ww = static_cast<const __nv_bfloat16*>(w);
  switch (vpt) {
    case 1: launch_pdl(rmsnorm_kernel<false, 1>, dim3(T), dim3(threads), 0, s, yy, xx, nullptr, ww, H, eps, gemma); break;
    case 2: launch_pdl(rmsnorm_kernel<false, 2>, dim3(T), dim3(threads), 0, s, yy, xx, nullptr, ww, H, eps, gemma); break;
    case 4: launch_pdl(rmsnorm_kernel<false, 4>, dim3(T), dim3(threads), 0, s, yy, xx, nullptr, ww, H, eps, gemma); break;
    default: launch_pdl(rmsnorm_kernel<false, 8>, dim3(T), dim3(threads), 0, s, yy, xx, nullptr, ww, H, eps, gemma); break;
  }
  return static_cast<int>(cudaGetLastError());
}

int sglb_fused_add_rmsnorm(void* y, const void* x, void* residual, const void* w, long long T, int H, float eps,
                           int gemma, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (H % 8 || H > 8 * 8 * 1024) return -kBadArgument;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  int vpt = 1;
  while (vpt * threads < nvec) vpt *= 2;
  auto* yy = static_cast<__nv_bfloat16*>(y);
  auto* xx = static_cast<const __nv_bfloat16*>(x);
  auto* rr = static_cast<__nv_bfloat16*>(residual);
  auto* ww = static_cast<const __nv_bfloat16*>(w);
  switch (vpt) {
    case 1: launch_pdl(rmsnorm_kernel<true, 1>, dim3(T), dim3(threads), 0, s, yy, xx, rr, ww, H, eps, gemma); break;
    case 2: launch_pdl(rmsnorm_kernel<true, 2>, dim3(T), dim3(threads), 0, s, yy, xx, rr, ww, H, eps, gemma); break;
    case 4: launch_pdl(rmsnorm_kernel<true, 4>, dim3(T), dim3(threads), 0, s, yy, xx, rr, ww, H, eps, gemma); break;
    default: launch_pdl(rmsnorm_kernel<true, 8>, dim3(T), dim3(threads), 0, s, yy, xx, rr, ww, H, eps, gemma); break;
  }
  return static_cast<int>(cudaGetLastError());
}

int sglb_silu_and_mul(void* out, const void* x, long long T, int I, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (I % 8) return -kBadArgument;
  const long long total = T * (I / 8);
  const int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  launch_pdl(silu_mul_kernel, dim3(static_cast<int>(blocks)), dim3(threads), 0, s, static_cast<__nv_bfloat16*>(out),
                                                               static_cast<const __nv_bfloat16*>(x), T, I);
  return static_cast<int>(cudaGetLastError());
}

int sglb_embedding(void* out, const int* ids, const void* table, long long T, int H, int rows, int vocab_start,
                   int masked, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (H % 8) return -kBadArgument;
  int threads = H / 8 < 256 ? ((H / 8 + 31) / 32) * 32 : 256;
  launch_pdl(embedding_kernel, dim3(T), dim3(threads), 0, s, static_cast<__nv_bfloat16*>(out), ids,
                                         static_cast<const __nv_bfloat16*>(table), H, rows, vocab_start, masked);
  return static_cast<int>(cudaGetLastError());
}

// dtype_bytes: 4 = fp32 logits, 2 = bf16 logits
int sglb_argmax(int* out, const void* logits, int B, int V, long long row_stride, int dtype_bytes, cudaStream_t s) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (dtype_bytes == 4) launch_pdl(argmax_kernel<float>, dim3(B), dim3(1024), 0, s, out, static_cast<const float*>(logits), V, row_stride);
  else launch_pdl(argmax_kernel<__nv_bfloat16>, dim3(B), dim3(1024), 0, s, out, static_cast<const __nv_bfloat16*>(logits), V, row_stride);
  return static_cast<int>(cudaGetLastError());
}

// Checked build (-DSGLB_BOUNDS_CHECK): tell the KV-write kernel how many pages the KV buffers have; a slot outside
// them is then reported through the status word (code kOutOfBounds, aux = token row, slot) and its store skipped.
// Returns 1 when the library was built with the checks, 0 otherwise (the call is then a no-op).
int sglb_debug_set_kv_pages(int pages) {
#ifdef SGLB_BOUNDS_CHECK
  sglb::Status* st = sglb::device_status();
  if (cudaMemcpyToSymbol(sglb::g_dbg_kv_pages, &pages, sizeof(int)) != cudaSuccess) return -sglb::kBadArgument;
  if (cudaMemcpyToSymbol(sglb::g_dbg_status, &st, sizeof(st)) != cudaSuccess) return -sglb::kBadArgument;
  return 1;
#else
  (void)pages;
  return 0;
#endif
}

int sglb_rope_qknorm_kvwrite(void* q_out, const void* qkv, const int* positions, const float* cos_sin, const void* q_w,
                             const void* k_w, float eps, long long T, int Hq, int Hkv, int D, int rotary_dim,
                             void* kv_buffer, const int* loc, int page_size, int is_neox, cudaStream_t s) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (is_neox && cos_sin != nullptr && ((rotary_dim / 2) % 32 != 0 || rotary_dim > D)) return -kBadArgument;
  const long long warps = T * (Hq + 2 * Hkv);
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  auto* qo = static_cast<__nv_bfloat16*>(q_out);
  auto* in = static_cast<const __nv_bfloat16*>(qkv);
  auto* qw = static_cast<const __nv_bfloat16*>(q_w);
  auto* kw = static_cast<const __nv_bfloat16*>(k_w);
  auto* kv = static_cast<__nv_bfloat16*>(kv_buffer);
  switch (D) {
    case 64:
      launch_pdl(rope_qknorm_kvwrite_kernel<64>, dim3(blocks), dim3(threads), 0, s, qo, in, positions, cos_sin, qw, kw, eps, T, Hq, Hkv,
                                                                rotary_dim, kv, loc, page_size, is_neox);
      break;
    case 128:
      launch_pdl(rope_qknorm_kvwrite_kernel<128>, dim3(blocks), dim3(threads), 0, s, qo, in, positions, cos_sin, qw, kw, eps, T, Hq, Hkv,
                                                                 rotary_dim, kv, loc, page_size, is_neox);
      break;
    case 256:
      launch_pdl(rope_qknorm_kvwrite_kernel<256>, dim3(blocks), dim3(threads), 0, s, qo, in, positions, cos_sin, qw, kw, eps, T, Hq, Hkv,
                                                                 rotary_dim, kv, loc, page_size, is_neox);
      break;
    default:
      return -kBadArgument;
  }
  return static_cast<int>(cudaGetLastError());
}

int sglb_page_table_scatter(int* table, int max_pages, const int* rows, const int* pos, const int* ids, int n,
                            cudaStream_t s) {
  if (n <= 0) return 0;
  sglb::page_table_scatter_kernel<<<(n + 255) / 256, 256, 0, s>>>(table, max_pages, rows, pos, ids, n);
  return static_cast<int>(cudaGetLastError());
}

int sglb_resolve_future(int* ids, const int* future_map, int n, cudaStream_t s) {
  if (n <= 0) return 0;
  sglb::resolve_future_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, future_map, n);
  return static_cast<int>(cudaGetLastError());
}
}
