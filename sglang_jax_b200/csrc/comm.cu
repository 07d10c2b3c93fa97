// Tensor-parallel collectives fused with the ops around them, over NVLink peer memory.
//
// Buffers are symmetric allocations (same size on every rank, every rank holds device pointers
// to all peers' copies).  Kernels use plain peer loads / stores (no TMA, no multicast) and
// epoch-valued flags in symmetric memory for cross-GPU ordering; every flag wait is bounded and
// reports kTimeoutPeerFlag through the status word instead of hanging.
//
//   ar_residual_rmsnorm   all-reduce of the row-parallel GEMM partials, fused with the residual
//                         add and the RMSNorm that follow it in a decoder layer.  Two-shot over
//                         token rows: rank r sums rows [r*R, (r+1)*R) of all peers' partials
//                         (reduce-scatter), adds its slice of the residual stream, normalises,
//                         and stores the normalised rows into every peer's activation buffer
//                         (all-gather).  The residual stream therefore stays token-sharded.
//   argmax_gather         vocab-parallel greedy pick: local (max, index) per row is pushed to
//                         all peers, every rank reduces the `world` candidates (ties -> lowest
//                         global index), so the full logits never cross NVLink.
//
// The reference reaches the same dataflow through GSPMD-inserted collectives after o_proj /
// down_proj and around the vocab-parallel head (python/sgl_jax/srt/layers/linear.py:102,
// python/sgl_jax/srt/layers/logits_processor.py:523).
#include <float.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxBlocks = 64;

struct Peers {
  void* p[kMaxWorld];
};

// Block-level barrier across ranks: block b of every rank meets block b of all peers.
// flags layout on every rank: [kMaxBlocks][kMaxWorld] u32; `epochs` is rank-local [kMaxBlocks].
// Returns false if a peer did not show up within the limit.
__device__ __forceinline__ bool rank_barrier(const Peers& flags, uint32_t* epochs, int rank, int world,
                                             Status* st, int phase_tag) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    s_epoch = epochs[blockIdx.x] + 1;
    epochs[blockIdx.x] = s_epoch;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t e = s_epoch;
  if (threadIdx.x < world) {
    __threadfence_system();
    uint32_t* remote = static_cast<uint32_t*>(flags.p[threadIdx.x]) + blockIdx.x * kMaxWorld + rank;
    st_release_sys(remote, e);
    const uint32_t* mine = static_cast<const uint32_t*>(flags.p[rank]) + blockIdx.x * kMaxWorld + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    // epochs only grow; a peer that is already one barrier ahead also satisfies the wait
    while (static_cast<int32_t>(ld_acquire_sys(mine) - e) < 0) {
      if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > kWaitLimitNs) {
        report(st, kTimeoutPeerFlag, threadIdx.x, phase_tag);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
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

template <int VPT>
__global__ void __launch_bounds__(1024, 1)
ar_residual_rmsnorm_kernel(const Peers ypart, const Peers gathered, const Peers flags, uint32_t* epochs,
                           __nv_bfloat16* residual, const __nv_bfloat16* w, int T, int H, int rank, int world,
                           float eps, int gemma, int has_residual, int rs_mode, Status* st) {
  __shared__ float red[32];
  const int rows_per = (T + world - 1) / world;
  const int r0 = rank * rows_per;
  const int r1 = min(T, r0 + rows_per);
  const int nvec = H >> 3;
  // every rank's GEMM has finished writing its partials
  const bool ok = rank_barrier(flags, epochs, rank, world, st, 1);
  if (ok) {
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int row = r0 + blockIdx.x; row < r1; row += gridDim.x) {
      const size_t base = static_cast<size_t>(row) * nvec;
      float vals[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
          uint4 part[kMaxWorld];
#pragma unroll
          for (int p = 0; p < kMaxWorld; ++p) {
            if (p < world) {
              // rs_mode: the GEMM epilogues already pushed every rank's slice into this rank's
              // buffer as [src rank][local row][H]; otherwise pull the slice from each peer.
              const uint4* src = rs_mode
                  ? reinterpret_cast<const uint4*>(ypart.p[rank]) + (static_cast<size_t>(p) * rows_per + (row - r0)) * nvec + idx
                  : reinterpret_cast<const uint4*>(ypart.p[p]) + base + idx;
              part[p] = __ldcg(src);
            }
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) vals[i][e] = 0.f;
#pragma unroll
          for (int p = 0; p < kMaxWorld; ++p) {
            if (p < world) {
              float f[8];
              unpack8(part[p], f);
#pragma unroll
              for (int e = 0; e < 8; ++e) vals[i][e] += f[e];
            }
          }
          if (has_residual) {
            uint4* rv = reinterpret_cast<uint4*>(residual) + base + idx;
            float r[8];
            unpack8(*rv, r);
#pragma unroll
            for (int e = 0; e < 8; ++e) vals[i][e] += r[e];
            const uint4 packed = pack8(vals[i]);
            *rv = packed;
            unpack8(packed, vals[i]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
        }
      }
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < ((blockDim.x + 31) >> 5) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) red[0] = t;
      }
      __syncthreads();
      const float inv = rsqrtf(red[0] / H + eps);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
          float wf[8], o[8];
          unpack8(wv[idx], wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = vals[i][e] * inv * (gemma ? wf[e] + 1.f : wf[e]);
          const uint4 out = pack8(o);
#pragma unroll
          for (int p = 0; p < kMaxWorld; ++p)
            if (p < world) reinterpret_cast<uint4*>(gathered.p[p])[base + idx] = out;
        }
      }
    }
  }
  // every rank's normalised rows have landed everywhere
  rank_barrier(flags, epochs, rank, world, st, 2);
}

// cand layout on every rank: [world][B] of (float value, int index)
struct Cand {
  float v;
  int i;
};

template <typename T>
__global__ void __launch_bounds__(1024, 1)
argmax_gather_kernel(int* __restrict__ out, const T* __restrict__ logits, int V, long long row_stride, int vocab_start,
                     int vocab_limit, const Peers cand, const Peers flags, uint32_t* epochs, int B, int rank,
                     int world, Status* st) {
  __shared__ float sv[32];
  __shared__ int si[32];
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const T* lr = logits + row * row_stride;
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      if (vocab_start + i >= vocab_limit) break;      // padding columns of the last shard
      float v;
      if constexpr (sizeof(T) == 2) v = __bfloat162float(lr[i]);
      else v = lr[i];
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
    const int wdx = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) {
      sv[wdx] = best;
      si[wdx] = bi;
    }
    __syncthreads();
    if (wdx == 0) {
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
      if (l < world) {
        const int gi = bi == 0x7fffffff ? 0x7fffffff : bi + vocab_start;
        const long long packed = (static_cast<long long>(gi) << 32) |
                                 static_cast<long long>(static_cast<unsigned int>(__float_as_int(best)));
        reinterpret_cast<long long*>(static_cast<Cand*>(cand.p[l]))[rank * B + row] = packed;
      }
    }
    __syncthreads();
  }
  const bool ok = rank_barrier(flags, epochs, rank, world, st, 3);
  if (ok) {
    const Cand* mine = static_cast<const Cand*>(cand.p[rank]);
    for (int row = blockIdx.x * blockDim.x + threadIdx.x; row < B; row += gridDim.x * blockDim.x) {
      float best = -FLT_MAX;
      int bi = 0x7fffffff;
      for (int p = 0; p < world; ++p) {
        // 8-byte L1-bypassing load: (value, index) written by rank p
        const long long raw = __ldcg(reinterpret_cast<const long long*>(mine + p * B + row));
        const float v = __int_as_float(static_cast<int>(raw & 0xffffffffll));
        const int i = static_cast<int>(raw >> 32);
        if (v > best || (v == best && i < bi)) {
          best = v;
          bi = i;
        }
      }
      out[row] = bi == 0x7fffffff ? 0 : bi;
    }
  }
  // nobody overwrites the candidate buffers of a rank that is still reading them
  rank_barrier(flags, epochs, rank, world, st, 4);
}

// Vocabulary-parallel logits gather by peer stores: rank r's shard `[B, Vp]` lands in columns
// [r * Vp, (r + 1) * Vp) of every rank's `[B, world * Vp]` symmetric buffer.  The first barrier holds the
// pushes back until every rank has consumed the previous contents (its sampling kernels precede this launch
// on its stream), the second returns once every peer's pushes into this rank's buffer are visible.
template <typename T>
__global__ void __launch_bounds__(1024, 1)
logits_gather_kernel(const T* __restrict__ logits, int Vp, long long row_stride, const Peers out, const Peers flags,
                     uint32_t* epochs, int B, int rank, int world, Status* st) {
  if (!rank_barrier(flags, epochs, rank, world, st, 5)) return;
  const long long full = static_cast<long long>(world) * Vp;
  const bool vec = (Vp * sizeof(T)) % 16 == 0 && (row_stride * sizeof(T)) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  for (int row = blockIdx.x; row < B; row += gridDim.x) {
    const T* src = logits + row * row_stride;
    const long long dst_off = row * full + static_cast<long long>(rank) * Vp;
    if (vec) {
      const int nvec = static_cast<int>(Vp * sizeof(T) / 16);
      const uint4* sv = reinterpret_cast<const uint4*>(src);
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        const uint4 v = sv[i];
        for (int p = 0; p < world; ++p) reinterpret_cast<uint4*>(static_cast<T*>(out.p[p]) + dst_off)[i] = v;
      }
    } else {
      for (int i = threadIdx.x; i < Vp; i += blockDim.x) {
        const T v = src[i];
        for (int p = 0; p < world; ++p) (static_cast<T*>(out.p[p]) + dst_off)[i] = v;
      }
    }
  }
  rank_barrier(flags, epochs, rank, world, st, 6);
}


// ---------------------------------------------------------------------------------------------
// Expert-parallel token all-to-all (dispatch / combine) over NVLink peer stores.
//
// Tokens are sharded over the ranks (rank r routes only the rows of its slice).  Dispatch: every
// (token, expert) pair is stored into the receive region this rank owns on the expert's rank
// (`recv_x[dst][src * cap + slot]`, slot handed out by an atomic counter, with the pair's global expert
// id, routing weight and return address); the last CTA publishes the per-destination counts.  The
// receiver runs its local experts on what arrived (a batch of rows with top-1 "routing" to the expert
// named in the metadata) and `moe_combine_send` stores each weighted expert output back into slot
// (token, j) of the sender's `ret` buffer; the sender then sums its `k` slots per token together with
// the residual add and RMSNorm (`ep_reduce_residual_rmsnorm_kernel`) and all-gathers the normalised rows.
// Cross-rank ordering is by the epoch barriers at the head of the receiving kernels (bounded waits).
// Counterpart of the reference's in-kernel remote-DMA scatter / gather
// (python/sgl_jax/srt/kernels/fused_moe/v1/kernel.py:1019-1135, :1189-1222).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, const float* __restrict__ w,
                    int pairs, int k, int H, int experts_per_rank, int world, int rank, int cap, const Peers recv_x,
                    const Peers recv_meta, int* send_count, int* done_ctr, const Peers recv_count) {
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int p = blockIdx.x * warps + wid; p < pairs; p += gridDim.x * warps) {
    const int e = ids[p];
    int d = e / experts_per_rank;
    if (e < 0 || d >= world) continue;            // padding pair
    int slot = 0;
    if (lane == 0) slot = atomicAdd(&send_count[d], 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= cap) continue;                    // cannot happen with cap >= pairs
    const size_t row = static_cast<size_t>(rank) * cap + slot;
    const uint4* src = reinterpret_cast<const uint4*>(x) + static_cast<size_t>(p / k) * nvec;
    uint4* dst = reinterpret_cast<uint4*>(recv_x.p[d]) + row * nvec;
    for (int i = lane; i < nvec; i += 32) dst[i] = src[i];
    if (lane == 0) {
      // meta: (global expert id, return slot on the source = pair index, weight bits, unused)
      reinterpret_cast<int4*>(recv_meta.p[d])[row] = make_int4(e, p, __float_as_int(w[p]), 0);
    }
  }
  // the CTA that finishes last tells every destination how many rows this rank sent it
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(done_ctr, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      __threadfence_system();
      for (int d = 0; d < world; ++d) {
        static_cast<int*>(recv_count.p[d])[rank] = send_count[d];
        send_count[d] = 0;
      }
      *done_ctr = 0;
      __threadfence_system();
    }
  }
}

// After every rank's dispatch has landed (barrier): mark the unused slots of each source region as
// "no expert" (-1) in the flat id / weight arrays the expert pipeline reads, and publish the row total.
__global__ void __launch_bounds__(1024, 1)
moe_recv_prepare_kernel(const Peers flags, uint32_t* epochs, int rank, int world, int cap, const int4* __restrict__ meta,
                        const int* __restrict__ recv_count, int* __restrict__ out_ids, float* __restrict__ out_w,
                        int* __restrict__ total, Status* st) {
  if (!rank_barrier(flags, epochs, rank, world, st, 7)) return;
  const int n = world * cap;
  for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < n; q += gridDim.x * blockDim.x) {
    const int s = q / cap, slot = q - s * cap;
    const int cnt = __ldcg(recv_count + s);
    if (slot < cnt) {
      const int4 m = __ldcg(meta + q);
      out_ids[q] = m.x;
      out_w[q] = __int_as_float(m.z);
    } else {
      out_ids[q] = -1;
      out_w[q] = 0.f;
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int t = 0;
    for (int s = 0; s < world; ++s) t += __ldcg(recv_count + s);
    *total = t;
  }
}

// y_sorted[r] (expert output of the received row that sorted position r holds) times its routing
// weight goes back to the rank and slot it came from.
__global__ void __launch_bounds__(256)
moe_combine_send_kernel(const __nv_bfloat16* __restrict__ y_sorted, const int* __restrict__ row_token,
                        const int* __restrict__ n_valid, const int4* __restrict__ meta, int H, int cap, int world,
                        const Peers ret) {
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  const int rows = *n_valid;
  for (int r = blockIdx.x * warps + wid; r < rows; r += gridDim.x * warps) {
    const int q = row_token[r];
    const int s = q / cap;
    if (q < 0 || s >= world) continue;
    const int4 m = meta[q];
    const float wgt = __int_as_float(m.z);
    const uint4* src = reinterpret_cast<const uint4*>(y_sorted) + static_cast<size_t>(r) * nvec;
    uint4* dst = reinterpret_cast<uint4*>(ret.p[s]) + static_cast<size_t>(m.y) * nvec;
    for (int i = lane; i < nvec; i += 32) {
      float f[8];
      unpack8(src[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= wgt;
      dst[i] = pack8(f);
    }
  }
}

// Token owner: out = sum over the k return slots of each owned token (+ residual) -> RMSNorm -> all-gather.
// Same shape as ar_residual_rmsnorm_kernel with the `world` slices replaced by `k` slots of `ret`.
template <int VPT>
__global__ void __launch_bounds__(1024, 1)
ep_reduce_residual_rmsnorm_kernel(const __nv_bfloat16* __restrict__ ret, const Peers gathered, const Peers flags,
                                  uint32_t* epochs, __nv_bfloat16* residual, const __nv_bfloat16* w, int T, int H, int k,
                                  int rows_per, int rank, int world, float eps, int gemma, int has_residual,
                                  Status* st) {
  __shared__ float red[32];
  const int r0 = rank * rows_per;
  const int r1 = min(T, r0 + rows_per);
  const int nvec = H >> 3;
  // every rank's combine stores have landed
  const bool ok = rank_barrier(flags, epochs, rank, world, st, 8);
  if (ok) {
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int row = r0 + blockIdx.x; row < r1; row += gridDim.x) {
      const size_t base = static_cast<size_t>(row) * nvec;
      const uint4* slots = reinterpret_cast<const uint4*>(ret) + static_cast<size_t>(row - r0) * k * nvec;
      float vals[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
#pragma unroll
          for (int e = 0; e < 8; ++e) vals[i][e] = 0.f;
          for (int j = 0; j < k; ++j) {
            float f[8];
            unpack8(__ldcg(slots + static_cast<size_t>(j) * nvec + idx), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) vals[i][e] += f[e];
          }
          if (has_residual) {
            uint4* rv = reinterpret_cast<uint4*>(residual) + base + idx;
            float r[8];
            unpack8(*rv, r);
#pragma unroll
            for (int e = 0; e < 8; ++e) vals[i][e] += r[e];
            const uint4 packed = pack8(vals[i]);
            *rv = packed;
            unpack8(packed, vals[i]);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
        }
      }
      ss = warp_sum(ss);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = threadIdx.x < ((blockDim.x + 31) >> 5) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) red[0] = t;
      }
      __syncthreads();
      const float inv = rsqrtf(red[0] / H + eps);
      __syncthreads();
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * blockDim.x;
        if (idx < nvec) {
          float wf[8], o[8];
          unpack8(wv[idx], wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = vals[i][e] * inv * (gemma ? wf[e] + 1.f : wf[e]);
          const uint4 out = pack8(o);
#pragma unroll
          for (int p = 0; p < kMaxWorld; ++p)
            if (p < world) reinterpret_cast<uint4*>(gathered.p[p])[base + idx] = out;
        }
      }
    }
  }
  rank_barrier(flags, epochs, rank, world, st, 9);
}

__global__ void barrier_only_kernel(const Peers flags, uint32_t* epochs, int rank, int world, Status* st) {
  rank_barrier(flags, epochs, rank, world, st, 9);
}

Peers make_peers(void* const* ptrs, int world) {
  Peers p{};
  for (int i = 0; i < world && i < kMaxWorld; ++i) p.p[i] = ptrs[i];
  return p;
}

}  // namespace
}  // namespace sglb

extern "C" {

int sglb_comm_max_blocks() { return sglb::kMaxBlocks; }
int sglb_comm_flag_bytes() { return sglb::kMaxBlocks * sglb::kMaxWorld * 4; }

// ypart_ptrs / gathered_ptrs / flag_ptrs: host arrays of `world` device pointers (peer views of the
// symmetric buffers; entry `rank` is the local one).  `residual` may be null (no residual add).
int sglb_ar_residual_rmsnorm(void* const* ypart_ptrs, void* const* gathered_ptrs, void* const* flag_ptrs,
                             void* epochs, void* residual, const void* w, int T, int H, int rank, int world, float eps,
                             int gemma, int rs_mode, cudaStream_t stream) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (world < 1 || world > kMaxWorld || H % 8 || H > 8 * 1024 * 4) return -kBadArgument;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  int vpt = 1;
  while (vpt * threads < nvec) vpt *= 2;
  const int rows_per = (T + world - 1) / world;
  const int blocks = rows_per < kMaxBlocks ? rows_per : kMaxBlocks;
  Peers yp = make_peers(ypart_ptrs, world), gp = make_peers(gathered_ptrs, world), fp = make_peers(flag_ptrs, world);
  auto* res = static_cast<__nv_bfloat16*>(residual);
  auto* ww = static_cast<const __nv_bfloat16*>(w);
  auto* ep = static_cast<uint32_t*>(epochs);
  Status* st = device_status();
  const int hr = residual != nullptr;
  switch (vpt) {
    case 1: ar_residual_rmsnorm_kernel<1><<<blocks, threads, 0, stream>>>(yp, gp, fp, ep, res, ww, T, H, rank, world, eps, gemma, hr, rs_mode, st); break;
    case 2: ar_residual_rmsnorm_kernel<2><<<blocks, threads, 0, stream>>>(yp, gp, fp, ep, res, ww, T, H, rank, world, eps, gemma, hr, rs_mode, st); break;
    default: ar_residual_rmsnorm_kernel<4><<<blocks, threads, 0, stream>>>(yp, gp, fp, ep, res, ww, T, H, rank, world, eps, gemma, hr, rs_mode, st); break;
  }
  return static_cast<int>(cudaGetLastError());
}

// logits: this rank's shard [B, V] (dtype_bytes 4 = fp32, 2 = bf16); columns at or beyond
// `vocab_limit - vocab_start` are padding.  cand buffers hold world*B (float,int) pairs.
int sglb_argmax_gather(int* out, const void* logits, int B, int V, long long row_stride, int dtype_bytes,
                       int vocab_start, int vocab_limit, void* const* cand_ptrs, void* const* flag_ptrs, void* epochs,
                       int rank, int world, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (world < 1 || world > kMaxWorld) return -kBadArgument;
  Peers cp = make_peers(cand_ptrs, world), fp = make_peers(flag_ptrs, world);
  const int blocks = B < kMaxBlocks ? B : kMaxBlocks;
  auto* ep = static_cast<uint32_t*>(epochs);
  Status* st = device_status();
  if (dtype_bytes == 4)
    argmax_gather_kernel<float><<<blocks, 1024, 0, stream>>>(out, static_cast<const float*>(logits), V, row_stride,
                                                              vocab_start, vocab_limit, cp, fp, ep, B, rank, world, st);
  else
    argmax_gather_kernel<__nv_bfloat16><<<blocks, 1024, 0, stream>>>(out, static_cast<const __nv_bfloat16*>(logits), V,
                                                                      row_stride, vocab_start, vocab_limit, cp, fp, ep,
                                                                      B, rank, world, st);
  return static_cast<int>(cudaGetLastError());
}

// logits: this rank's shard [B, Vp] (dtype_bytes 4 = fp32, 2 = bf16); out_ptrs: every rank's [B, world * Vp]
// symmetric buffer of the same dtype.
int sglb_logits_gather(const void* logits, int B, int Vp, long long row_stride, int dtype_bytes, void* const* out_ptrs,
                       void* const* flag_ptrs, void* epochs, int rank, int world, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (world < 1 || world > kMaxWorld || Vp <= 0 || (dtype_bytes != 2 && dtype_bytes != 4)) return -kBadArgument;
  Peers op = make_peers(out_ptrs, world), fp = make_peers(flag_ptrs, world);
  const int blocks = B < kMaxBlocks ? B : kMaxBlocks;
  auto* ep = static_cast<uint32_t*>(epochs);
  Status* st = device_status();
  if (dtype_bytes == 4)
    logits_gather_kernel<float><<<blocks, 1024, 0, stream>>>(static_cast<const float*>(logits), Vp, row_stride, op, fp,
                                                              ep, B, rank, world, st);
  else
    logits_gather_kernel<__nv_bfloat16><<<blocks, 1024, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), Vp,
                                                                      row_stride, op, fp, ep, B, rank, world, st);
  return static_cast<int>(cudaGetLastError());
}

// ---- expert-parallel all-to-all (see the kernels above) -------------------------------------------------------
// x: this rank's token rows [pairs / k, H] bf16; ids / w: [pairs] global expert ids (negative = padding) and routing
// weights.  recv_x_ptrs / recv_meta_ptrs / recv_count_ptrs: every rank's receive buffers ([world * cap, H] bf16,
// [world * cap] int4, [world] int; symmetric memory).  send_count ([world] ints) and done_ctr (1 int) are local,
// zero when idle.
int sglb_moe_dispatch(const void* x, const int* ids, const float* w, int pairs, int k, int H, int experts_per_rank,
                      int world, int rank, int cap, void* const* recv_x_ptrs, void* const* recv_meta_ptrs,
                      void* send_count, void* done_ctr, void* const* recv_count_ptrs, cudaStream_t stream) {
  using namespace sglb;
  if (pairs <= 0) pairs = 0;
  if (world < 1 || world > kMaxWorld || H % 8 || k < 1 || experts_per_rank < 1 || pairs > cap) return -kBadArgument;
  Peers rx = make_peers(recv_x_ptrs, world), rm = make_peers(recv_meta_ptrs, world), rc = make_peers(recv_count_ptrs, world);
  int blocks = (pairs + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 592) blocks = 592;
  moe_dispatch_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ids, w, pairs, k, H,
                                                  experts_per_rank, world, rank, cap, rx, rm,
                                                  static_cast<int*>(send_count), static_cast<int*>(done_ctr), rc);
  return static_cast<int>(cudaGetLastError());
}

int sglb_moe_recv_prepare(void* const* flag_ptrs, void* epochs, int rank, int world, int cap, const void* meta,
                          const int* recv_count, int* out_ids, float* out_w, int* total, cudaStream_t stream) {
  using namespace sglb;
  if (world < 1 || world > kMaxWorld) return -kBadArgument;
  Peers fp = make_peers(flag_ptrs, world);
  moe_recv_prepare_kernel<<<16, 1024, 0, stream>>>(fp, static_cast<uint32_t*>(epochs), rank, world, cap,
                                                   static_cast<const int4*>(meta), recv_count, out_ids, out_w, total,
                                                   device_status());
  return static_cast<int>(cudaGetLastError());
}

int sglb_moe_combine_send(const void* y_sorted, const int* row_token, const int* n_valid, const void* meta, int max_rows,
                          int H, int cap, int world, void* const* ret_ptrs, cudaStream_t stream) {
  using namespace sglb;
  if (world < 1 || world > kMaxWorld || H % 8) return -kBadArgument;
  Peers rp = make_peers(ret_ptrs, world);
  int blocks = (max_rows + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 592) blocks = 592;
  moe_combine_send_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y_sorted), row_token, n_valid,
                                                      static_cast<const int4*>(meta), H, cap, world, rp);
  return static_cast<int>(cudaGetLastError());
}

// ret: this rank's [rows_per * k, H] return slots; the rest as sglb_ar_residual_rmsnorm.
int sglb_ep_reduce_residual_rmsnorm(const void* ret, void* const* gathered_ptrs, void* const* flag_ptrs, void* epochs,
                                    void* residual, const void* w, int T, int H, int k, int rows_per, int rank, int world,
                                    float eps, int gemma, cudaStream_t stream) {
  using namespace sglb;
  if (T <= 0) return 0;
  if (world < 1 || world > kMaxWorld || H % 8 || H > 8 * 1024 * 4 || k < 1) return -kBadArgument;
  const int nvec = H / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  int vpt = 1;
  while (vpt * threads < nvec) vpt *= 2;
  int blocks = rows_per < kMaxBlocks ? rows_per : kMaxBlocks;
  if (blocks < 1) blocks = 1;
  Peers gp = make_peers(gathered_ptrs, world), fp = make_peers(flag_ptrs, world);
  auto* rt = static_cast<const __nv_bfloat16*>(ret);
  auto* res = static_cast<__nv_bfloat16*>(residual);
  auto* ww = static_cast<const __nv_bfloat16*>(w);
  auto* ep = static_cast<uint32_t*>(epochs);
  Status* st = device_status();
  const int hr = residual != nullptr;
  switch (vpt) {
    case 1: ep_reduce_residual_rmsnorm_kernel<1><<<blocks, threads, 0, stream>>>(rt, gp, fp, ep, res, ww, T, H, k, rows_per, rank, world, eps, gemma, hr, st); break;
    case 2: ep_reduce_residual_rmsnorm_kernel<2><<<blocks, threads, 0, stream>>>(rt, gp, fp, ep, res, ww, T, H, k, rows_per, rank, world, eps, gemma, hr, st); break;
    default: ep_reduce_residual_rmsnorm_kernel<4><<<blocks, threads, 0, stream>>>(rt, gp, fp, ep, res, ww, T, H, k, rows_per, rank, world, eps, gemma, hr, st); break;
  }
  return static_cast<int>(cudaGetLastError());
}

// One cross-rank barrier with `blocks` CTAs (tests: a rank that never launches makes the others'
// bounded waits expire and report through the status word).
int sglb_comm_barrier(void* const* flag_ptrs, void* epochs, int rank, int world, int blocks, cudaStream_t stream) {
  using namespace sglb;
  if (world < 1 || world > kMaxWorld || blocks < 1 || blocks > kMaxBlocks) return -kBadArgument;
  Peers fp = make_peers(flag_ptrs, world);
  barrier_only_kernel<<<blocks, 32, 0, stream>>>(fp, static_cast<uint32_t*>(epochs), rank, world, device_status());
  return static_cast<int>(cudaGetLastError());
}
}
