// Ragged paged attention over the paged KV cache  [pages, 2, Hkv, P, D]  (bf16).
//
//   paged_decode   one query token per sequence, GQA heads of one KV head packed into the MMA
//                  M dimension, KV split over CTAs (flash-decoding) + a small combine kernel.
//   paged_extend   prefill / mixed: a 64-row query tile of one sequence and one query head per
//                  CTA, causal over `prefix_len + i`, online softmax (flash attention).
//
// Both stream K/V tiles of 64 tokens through a multi-stage shared-memory ring filled by TMA
// tensor copies straight out of the page pool ("page gathers": one copy per page-run, the
// page id comes from the device-resident page table), 128-byte swizzled so that ldmatrix is
// bank-conflict free.  No multicast is used anywhere.  All barrier waits are bounded.
//
// Semantics follow the reference kernel's contract
// (python/sgl_jax/srt/kernels/ragged_paged_attention/ragged_paged_attention_v3.py:1667 and its
// jnp oracle `ref_ragged_paged_attention` :94): causal GQA attention over a ragged batch with
// optional sliding window and logit soft-cap; the KV write itself happens in the fused
// RoPE kernel that precedes this one on the stream.
#include <cstdlib>
#include <math.h>

#include <unordered_map>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int TN = 64;            // KV tokens per tile
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr float kLog2e = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16* q;       // [T, Hq, D]
  __nv_bfloat16* out;           // [T, Hq, D]
  float* part_o;                // decode splits: [B, Hq, S, D]
  float* part_lse;              // decode splits: [B, Hq, S]
  const int* page_table;        // [rows, max_pages]
  const int* req_pool_indices;  // [B]
  const int* seq_lens;          // [B]
  const int* prefix_lens;       // [B]   (extend)
  const int* cu_q_lens;         // [B+1] (extend)
  Status* status;
  int B, Hq, Hkv, max_pages, page_size, num_splits;
  int kv_evict_first;           // decode: KV tiles carry an L2 evict-first hint
  int window;                   // 0 = none
  float scale, soft_cap;
  // extend only: visibility inside the last `tail_len` keys, [B, mask_rows, tail_len] bytes (null = causal)
  const uint8_t* tail_mask;
  int tail_len, mask_rows;
  int bidirectional;            // extend only: every query row sees every key of its sequence (encoders)
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of (row, 16-byte chunk) inside a [rows][64 bf16] half tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

// One stage: K halves then V halves, each half tile TN x 64 bf16 = 8 KB.
template <int D>
struct Stage {
  static constexpr int kHalves = D / 64;
  static constexpr int kHalfBytes = TN * 128;
  static constexpr int kBytes = 2 * kHalves * kHalfBytes;
};

// Issue the TMA copies of KV tile `tile` (tokens tile*64 ..) of one sequence / KV head.
template <int D>
__device__ __forceinline__ void issue_tile(const CUtensorMap* tmap, uint32_t smem_stage, uint32_t bar,
                                           const int* pt_row, int max_pages, int page_size, int Hkv, int kvh,
                                           int tile, uint64_t policy = 0) {
  using S = Stage<D>;
  mbar_expect_tx(bar, S::kBytes);
  const int tok0 = tile * TN;
  const int run = page_size < TN ? page_size : TN;          // tokens per copy
  const int n_runs = TN / run;
  for (int r = 0; r < n_runs; ++r) {
    const int tok = tok0 + r * run;
    int pg = tok / page_size;
    if (pg >= max_pages) pg = max_pages - 1;
    const int page = pt_row[pg];
    const int off = tok - (tok / page_size) * page_size;
#pragma unroll
    for (int kv = 0; kv < 2; ++kv) {
      const int row = ((page * 2 + kv) * Hkv + kvh) * page_size + off;
#pragma unroll
      for (int h = 0; h < S::kHalves; ++h) {
        const uint32_t dst = smem_stage + (kv * S::kHalves + h) * S::kHalfBytes + r * run * 128;
        if (policy != 0) tma_load_2d_hint(dst, tmap, bar, h * 64, row, policy);
        else tma_load_2d(dst, tmap, bar, h * 64, row);
      }
    }
  }
}

// Per-warp flash-attention state for a 16-row query fragment.
template <int D>
struct WarpState {
  float o[D / 8][4];
  float m[2];   // running max (scaled, log2 domain) for rows g and g+8
  float l[2];   // running sum
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m[0] = m[1] = -INFINITY;
    l[0] = l[1] = 0.f;
  }
};

// Process NT (16 or 64) KV tokens starting at tile-local row `r0` against the warp's 16 query rows.
// `kmax[i]` (i = 0 for row g, 1 for row g+8) is the last visible KV index (inclusive) and `kmin[i]`
// the first, in absolute token positions; `tok_base` is the absolute index of tile row 0.
// With MASK, keys at absolute index >= `tail_start` are visible to row i only where
// `mask_row[i][key - tail_start]` is non-zero (speculative token trees, bidirectional blocks).
template <int D, int NT, bool MASK = false>
__device__ __forceinline__ void attend(WarpState<D>& st, const uint32_t (&qf)[D / 16][4], uint32_t k_smem,
                                       uint32_t v_smem, int r0, int tok_base, const int (&kmin)[2],
                                       const int (&kmax)[2], float scale_log2, float soft_cap, float scale,
                                       const uint8_t* const* mask_row = nullptr, int tail_start = 0) {
  constexpr int NJ = NT / 8;
  const int lane = threadIdx.x & 31;
  const int t4 = lane & 3;
  float s[NJ][4];
#pragma unroll
  for (int j = 0; j < NJ; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
  // S = Q K^T
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int half = kk / 4;             // which 64-wide half of D
    const int c0 = (kk % 4) * 2;         // 16-byte chunk of the k-step inside the half
#pragma unroll
    for (int jp = 0; jp < NJ / 2; ++jp) {
      // x4: matrices (tokens 16jp..+7, chunk c0), (same, c0+1), (tokens 16jp+8.., c0), (same, c0+1)
      const int row = r0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = c0 + ((lane >> 3) & 1);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(k_smem + half * Stage<D>::kHalfBytes + sw_off(row, chunk), b0, b1, b2, b3);
      mma16816(s[2 * jp], qf[kk], b0, b1);
      mma16816(s[2 * jp + 1], qf[kk], b2, b3);
    }
  }
  // scale / soft-cap / mask, tile max
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const int tok = tok_base + r0 + j * 8 + t4 * 2 + (e & 1);
      float v = s[j][e];
      if (soft_cap > 0.f) v = soft_cap * tanhf(v * scale / soft_cap) * kLog2e;
      else v *= scale_log2;
      bool ok = tok <= kmax[i] && tok >= kmin[i];
      if (MASK) {
        if (ok && tok >= tail_start) ok = mask_row[i] != nullptr && mask_row[i][tok - tail_start] != 0;
      }
      v = ok ? v : -INFINITY;
      s[j][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
  }
  float corr[2], mnew[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mnew[i] = fmaxf(st.m[i], mx[i]);
    const float mref = mnew[i] == -INFINITY ? 0.f : mnew[i];
    corr[i] = exp2f(st.m[i] - mref);          // st.m = -inf -> 0
    st.m[i] = mnew[i];
    mnew[i] = mref;
  }
  float rs[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(s[j][e] - mnew[e >> 1]);
      s[j][e] = pv;
      rs[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) st.l[i] = st.l[i] * corr[i] + rs[i];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) {
    st.o[n][0] *= corr[0];
    st.o[n][1] *= corr[0];
    st.o[n][2] *= corr[1];
    st.o[n][3] *= corr[1];
  }
  // O += P V
#pragma unroll
  for (int kk = 0; kk < NT / 16; ++kk) {
    uint32_t pa[4];
    pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      // x4.trans: (tokens 16kk..+7, d 16np..+7), (tokens +8.., same d), (tokens 16kk.., d 16np+8..), (tokens +8.., d +8..)
      const int row = r0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int dcol = np * 16 + ((lane >> 4) << 3);
      const int half = dcol / 64;
      const int chunk = (dcol % 64) / 8;
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(v_smem + half * Stage<D>::kHalfBytes + sw_off(row, chunk), b0, b1, b2, b3);
      mma16816(st.o[2 * np], pa, b0, b1);
      mma16816(st.o[2 * np + 1], pa, b2, b3);
    }
  }
}

// ------------------------------------------------------------------------------------------- decode
template <int D>
__global__ void __launch_bounds__(kThreads, 1)
paged_decode_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p, int stages) {
  using S = Stage<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + stages * S::kBytes);
  uint64_t* empty_bar = full_bar + stages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + stages);
  float* merge = reinterpret_cast<float*>(smem);   // reused after the main loop

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  pdl_wait();
  const int seq = p.seq_lens[b];
  const int* pt_row = p.page_table + static_cast<size_t>(p.req_pool_indices[b]) * p.max_pages;

  int first_tok = 0;
  if (p.window > 0 && seq > p.window) first_tok = seq - p.window;
  const int tile_lo = first_tok / TN;
  const int tile_hi = (seq + TN - 1) / TN;
  const int n_tiles = tile_hi - tile_lo;
  const int per = (n_tiles + p.num_splits - 1) / p.num_splits;
  const int t0 = tile_lo + split * per;
  const int t1 = min(t0 + per, tile_hi);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  WarpState<D> st;
  st.init();
  if (warp == kConsumerWarps) {
    if (lane == 0) {
      prefetch_tmap(&tmap);
      int stage = 0;
      uint32_t phase = 0;
      // a decode step reads every KV tile exactly once: do not let it displace the rest of L2
      const uint64_t pol = p.kv_evict_first ? l2_policy_evict_first() : 0;
      for (int t = t0; t < t1 && !*abort_flag; ++t) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
          report(p.status, kTimeoutEmptyBarrier, b, t);
          *abort_flag = 1;
          break;
        }
        issue_tile<D>(&tmap, smem_u32(smem + stage * S::kBytes), smem_u32(&full_bar[stage]), pt_row, p.max_pages,
                      p.page_size, p.Hkv, kvh, t, pol);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // Q fragments: rows = query heads of this KV group (zero beyond G)
    uint32_t qf[D / 16][4];
    const int g = lane >> 2, t4 = lane & 3;
    const __nv_bfloat16* qrow = p.q + (static_cast<size_t>(b) * p.Hq + kvh * G + g) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      qf[kk][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + t4 * 2) : 0u;
      qf[kk][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + kk * 16 + 8 + t4 * 2) : 0u;
      qf[kk][1] = (g + 8) < G ? *reinterpret_cast<const uint32_t*>(qrow + 8 * D + kk * 16 + t4 * 2) : 0u;
      qf[kk][3] = (g + 8) < G ? *reinterpret_cast<const uint32_t*>(qrow + 8 * D + kk * 16 + 8 + t4 * 2) : 0u;
    }
    const int kmin[2] = {first_tok, first_tok};
    const int kmax[2] = {seq - 1, seq - 1};
    const float scale_log2 = p.scale * kLog2e;
    int stage = 0;
    uint32_t phase = 0;
    for (int t = t0; t < t1 && !*abort_flag; ++t) {
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
        report(p.status, kTimeoutFullBarrier, b, t);
        *abort_flag = 1;
        break;
      }
      const uint32_t ks = smem_u32(smem + stage * S::kBytes);
      const uint32_t vs = ks + S::kHalves * S::kHalfBytes;
      // each consumer warp owns 16 of the tile's 64 tokens
      if (t * TN + warp * 16 < seq)
        attend<D, 16>(st, qf, ks, vs, warp * 16, t * TN, kmin, kmax, scale_log2, p.soft_cap, p.scale);
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
  }
  __syncthreads();   // ring is idle now: reuse it for the cross-warp merge

  // merge the four warps' (m, l, O) states; rows 0..7 only unless G > 8
  float* m_s = merge;                         // [4][16]
  float* l_s = merge + 64;                    // [4][16]
  float* o_s = merge + 128;                   // [4][16][D]
  if (warp < kConsumerWarps) {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float l = st.l[i];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (t4 == 0) {
        m_s[warp * 16 + g + 8 * i] = st.m[i];
        l_s[warp * 16 + g + 8 * i] = l;
      }
    }
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
      float* r0p = o_s + (warp * 16 + g) * D + n * 8 + t4 * 2;
      r0p[0] = st.o[n][0];
      r0p[1] = st.o[n][1];
      float* r1p = r0p + 8 * D;
      r1p[0] = st.o[n][2];
      r1p[1] = st.o[n][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += kThreads) {
    const int r = idx / D, d = idx - r * D;
    float mmax = -INFINITY;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) mmax = fmaxf(mmax, m_s[w * 16 + r]);
    float lsum = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const float mw = m_s[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mmax);
      lsum += l_s[w * 16 + r] * f;
      acc += o_s[(w * 16 + r) * D + d] * f;
    }
    const int hq = kvh * G + r;
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    if (p.num_splits == 1) {
      p.out[(static_cast<size_t>(b) * p.Hq + hq) * D + d] = __float2bfloat16(acc * inv);
    } else {
      const size_t base = (static_cast<size_t>(b) * p.Hq + hq) * p.num_splits + split;
      p.part_o[base * D + d] = acc * inv;
      if (d == 0) p.part_lse[base] = lsum > 0.f ? mmax + log2f(lsum) : -INFINITY;
    }
  }
}

template <int D>
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                      __nv_bfloat16* __restrict__ out, int num_splits) {
  pdl_wait();
  const int row = blockIdx.x;   // b * Hq + h
  const float* lse = part_lse + static_cast<size_t>(row) * num_splits;
  float mmax = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mmax = fmaxf(mmax, lse[s]);
  float wsum = 0.f;
  for (int s = 0; s < num_splits; ++s) wsum += (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mmax);
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mmax);
      acc += w * part_o[(static_cast<size_t>(row) * num_splits + s) * D + d];
    }
    out[static_cast<size_t>(row) * D + d] = __float2bfloat16(acc * inv);
  }
}

// ------------------------------------------------------------------------------------------- extend
constexpr int BQ = 64;   // query rows per CTA (16 per consumer warp)

template <int D>
__global__ void __launch_bounds__(kThreads, 2)
paged_extend_kernel(const __grid_constant__ CUtensorMap tmap, const AttnParams p, int stages) {
  using S = Stage<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + stages * S::kBytes);
  uint64_t* empty_bar = full_bar + stages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + stages);

  // locate (sequence, query tile) of this CTA: tiles are numbered sequence by sequence
  int b = 0, tile_in_seq = 0;
  {
    int acc = 0;
    const int want = blockIdx.x;
    bool found = false;
    for (int i = 0; i < p.B; ++i) {
      const int n = p.cu_q_lens[i + 1] - p.cu_q_lens[i];
      const int nt = (n + BQ - 1) / BQ;
      if (want < acc + nt) {
        b = i;
        tile_in_seq = want - acc;
        found = true;
        break;
      }
      acc += nt;
    }
    if (!found) return;   // uniform for the whole CTA
  }
  const int hq = blockIdx.y;
  const int G = p.Hq / p.Hkv;
  const int kvh = hq / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = p.cu_q_lens[b];
  const int q_len = p.cu_q_lens[b + 1] - q_begin;
  const int prefix = p.prefix_lens[b];
  const int seq = p.seq_lens[b];
  const int q0 = tile_in_seq * BQ;                         // first query row (within the sequence's new tokens)
  const int q_hi = min(q0 + BQ, q_len);
  const bool masked = p.tail_mask != nullptr || p.bidirectional != 0;
  const int kv_end = masked ? seq : min(seq, prefix + q_hi);   // causal upper bound for this tile
  int first_tok = 0;
  if (p.window > 0) first_tok = max(0, prefix + q0 - p.window + 1);
  const int t0 = first_tok / TN;
  const int t1 = (kv_end + TN - 1) / TN;
  const int* pt_row = p.page_table + static_cast<size_t>(p.req_pool_indices[b]) * p.max_pages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    if (lane == 0) {
      prefetch_tmap(&tmap);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = t0; t < t1 && !*abort_flag; ++t) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
          report(p.status, kTimeoutEmptyBarrier, b, t);
          *abort_flag = 1;
          break;
        }
        issue_tile<D>(&tmap, smem_u32(smem + stage * S::kBytes), smem_u32(&full_bar[stage]), pt_row, p.max_pages,
                      p.page_size, p.Hkv, kvh, t);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    return;
  }

  WarpState<D> st;
  st.init();
  const int g = lane >> 2, t4 = lane & 3;
  const int r_lo = q0 + warp * 16 + g;        // this thread's two query rows (within the sequence)
  const int r_hi = r_lo + 8;
  uint32_t qf[D / 16][4];
  {
    const __nv_bfloat16* qa = p.q + (static_cast<size_t>(q_begin + r_lo) * p.Hq + hq) * D;
    const __nv_bfloat16* qb = p.q + (static_cast<size_t>(q_begin + r_hi) * p.Hq + hq) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      qf[kk][0] = r_lo < q_len ? *reinterpret_cast<const uint32_t*>(qa + kk * 16 + t4 * 2) : 0u;
      qf[kk][2] = r_lo < q_len ? *reinterpret_cast<const uint32_t*>(qa + kk * 16 + 8 + t4 * 2) : 0u;
      qf[kk][1] = r_hi < q_len ? *reinterpret_cast<const uint32_t*>(qb + kk * 16 + t4 * 2) : 0u;
      qf[kk][3] = r_hi < q_len ? *reinterpret_cast<const uint32_t*>(qb + kk * 16 + 8 + t4 * 2) : 0u;
    }
  }
  const int kmax[2] = {masked ? seq - 1 : min(prefix + r_lo, seq - 1), masked ? seq - 1 : min(prefix + r_hi, seq - 1)};
  const uint8_t* mask_row[2] = {nullptr, nullptr};
  if (p.tail_mask != nullptr) {
    const uint8_t* mb = p.tail_mask + static_cast<size_t>(b) * p.mask_rows * p.tail_len;
    if (r_lo < q_len && r_lo < p.mask_rows) mask_row[0] = mb + static_cast<size_t>(r_lo) * p.tail_len;
    if (r_hi < q_len && r_hi < p.mask_rows) mask_row[1] = mb + static_cast<size_t>(r_hi) * p.tail_len;
  }
  const int tail_start = seq - p.tail_len;
  int kmin[2] = {0, 0};
  if (p.window > 0) {
    kmin[0] = max(0, prefix + r_lo - p.window + 1);
    kmin[1] = max(0, prefix + r_hi - p.window + 1);
  }
  // rows of this warp see KV up to prefix + q0 + warp*16 + 15: later tiles are fully masked for it
  const int warp_kv_end = masked ? seq : min(seq, prefix + min(q0 + warp * 16 + 16, q_len));
  const float scale_log2 = p.scale * kLog2e;
  int stage = 0;
  uint32_t phase = 0;
  for (int t = t0; t < t1 && !*abort_flag; ++t) {
    if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
      report(p.status, kTimeoutFullBarrier, b, t);
      *abort_flag = 1;
      break;
    }
    const uint32_t ks = smem_u32(smem + stage * S::kBytes);
    const uint32_t vs = ks + S::kHalves * S::kHalfBytes;
    if (t * TN < warp_kv_end && q0 + warp * 16 < q_len) {
      if (masked && (t + 1) * TN > tail_start)
        attend<D, TN, true>(st, qf, ks, vs, 0, t * TN, kmin, kmax, scale_log2, p.soft_cap, p.scale, mask_row,
                            tail_start);
      else
        attend<D, TN>(st, qf, ks, vs, 0, t * TN, kmin, kmax, scale_log2, p.soft_cap, p.scale);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
  }
  // finalize
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float l = st.l[i];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    st.l[i] = l > 0.f ? 1.f / l : 0.f;
  }
  if (r_lo < q_len) {
    __nv_bfloat16* o = p.out + (static_cast<size_t>(q_begin + r_lo) * p.Hq + hq) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(o + n * 8 + t4 * 2) = pack_bf16(st.o[n][0] * st.l[0], st.o[n][1] * st.l[0]);
  }
  if (r_hi < q_len) {
    __nv_bfloat16* o = p.out + (static_cast<size_t>(q_begin + r_hi) * p.Hq + hq) * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(o + n * 8 + t4 * 2) = pack_bf16(st.o[n][2] * st.l[1], st.o[n][3] * st.l[1]);
  }
}


// ---------------------------------------------------------------------------------------------
// Prefill attention on the 5th-generation tensor cores (head_dim 128, causal, bf16).
//
// One CTA per (128-row query tile of one sequence, query head).  Warp 0 drives TMA (Q tile once, then
// 128-token K/V tiles gathered page by page into a two-stage ring), warp 1 issues tcgen05.mma, warps 2..5
// (one thread per query row) do the softmax:
//
//   S_j = Q K_j^T            128 x 128 x 128, accumulator in tensor memory (two S buffers, so S_{j+1}
//                            is computed while the softmax of S_j runs)
//   P_j = exp2(S_j - m)      read with tcgen05.ld, written as bf16 into a 128-byte-swizzled smem tile
//   O  += P_j V_j            128 x 128 x 128, accumulator stays in tensor memory for the whole row of tiles
//
// The running maximum is only raised when it grows by more than 2^8: then the softmax threads wait for
// the P V product in flight, multiply O (tcgen05.ld / tcgen05.st) and the row sums by the correction
// factor, and carry on; between such events O is never touched by the CUDA cores.  K is the K-major B
// operand of the first product; V, laid out [token][dim] by the same TMA gathers, is the MN-major B
// operand of the second.  All waits are bounded; a timeout unwinds through the normal teardown.
// Reference contract: python/sgl_jax/srt/kernels/ragged_paged_attention/ragged_paged_attention_v3.py:1667.
// ---------------------------------------------------------------------------------------------
namespace tc {
// Two CTAs share an SM (113 KB of shared memory and 256 columns of tensor memory each): while one CTA's four
// softmax warps work through their exponentials, the other CTA's products keep the tensor pipe busy.
constexpr int BQ2 = 128, BKV = 64, HD = 128;
constexpr int kBlk = 128 * 128;                    // bytes of one [128 rows][64 bf16] swizzled block (Q halves, P)
constexpr int kBlkKV = BKV * 128;                  // bytes of one [64 keys][64 bf16] swizzled block
constexpr int kQBytes = 2 * kBlk;
constexpr int kKVStage = 4 * kBlkKV;               // K (2 blocks by dim half) + V (2 blocks by dim half)
constexpr int kStagesKV = 2;
constexpr int kPBytes = kBlk;
constexpr int kSmem = kQBytes + kStagesKV * kKVStage + kPBytes + 256 + 768;   // 113 KB: two CTAs per SM
constexpr int kTmemCols = 256;                     // S (2 x 64 columns) + O (128 columns)
constexpr int kThreadsTc = 192;
constexpr float kRescale = 8.f;                    // raise the running max only past 2^8

struct Bars {
  // p_ready[i] / pv_done[i] serve the tiles with (tile & 1) == i: each completes once per two tiles, so a waiter is
  // never more than one phase behind the barrier it waits on
  // K and V of a stage have barriers of their own: the K half is free again as soon as Q K^T of its tile is done,
  // one whole tile before the V half, so the loads of the next keys start that much earlier
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_free[2], p_ready[2], pv_done[2];
  uint32_t tmem_slot;
  int abort_flag;
};
}  // namespace tc

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(tc::kThreadsTc, 2)
paged_extend_tc_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_q,
                       const AttnParams p) {
  using namespace tc;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + kQBytes;
  uint8_t* p_s = kv_s + kStagesKV * kKVStage;
  Bars* bars = reinterpret_cast<Bars*>(p_s + kPBytes);
  volatile int* abort_flag = &bars->abort_flag;
  if (reinterpret_cast<uint8_t*>(bars) + sizeof(Bars) > smem_raw + kSmem) {
    // the dynamic window started less aligned than the carve-up allows for: refuse, uniformly, before any barrier
    if (threadIdx.x == 0) report(p.status, kBadArgument, blockIdx.x, 9000);
    return;
  }

  // (sequence, 128-row query tile) of this CTA
  int b = 0, tile_in_seq = 0;
  {
    int acc = 0;
    const int want = blockIdx.x;
    bool found = false;
    for (int i = 0; i < p.B; ++i) {
      const int n = p.cu_q_lens[i + 1] - p.cu_q_lens[i];
      const int nt = (n + BQ2 - 1) / BQ2;
      if (want < acc + nt) {
        b = i;
        tile_in_seq = want - acc;
        found = true;
        break;
      }
      acc += nt;
    }
    if (!found) return;
  }
  const int hq = blockIdx.y;
  const int kvh = hq / (p.Hq / p.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = p.cu_q_lens[b];
  const int q_len = p.cu_q_lens[b + 1] - q_begin;
  const int prefix = p.prefix_lens[b];
  const int seq = p.seq_lens[b];
  const int q0 = tile_in_seq * BQ2;
  const int q_hi = min(q0 + BQ2, q_len);
  const int kv_end = p.bidirectional ? seq : min(seq, prefix + q_hi);
  const int n_tiles = (kv_end + BKV - 1) / BKV;
  const int* pt_row = p.page_table + static_cast<size_t>(p.req_pool_indices[b]) * p.max_pages;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_kv);
    prefetch_tmap(&tmap_q);
    mbar_init(smem_u32(&bars->q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->k_full[i]), 1);
      mbar_init(smem_u32(&bars->k_empty[i]), 1);
      mbar_init(smem_u32(&bars->v_full[i]), 1);
      mbar_init(smem_u32(&bars->v_empty[i]), 1);
      mbar_init(smem_u32(&bars->s_full[i]), 1);
      mbar_init(smem_u32(&bars->s_free[i]), 4);       // one arrival per softmax warp
      mbar_init(smem_u32(&bars->p_ready[i]), 4);
      mbar_init(smem_u32(&bars->pv_done[i]), 1);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_slot;
  const uint32_t tmem_o = tmem_base + 2 * BKV;      // S buffers at columns 0 and 64, O at 128

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t qb = smem_u32(&bars->q_full);
      mbar_expect_tx(qb, kQBytes);
      tma_load_2d(smem_u32(q_s), &tmap_q, qb, hq * HD, q_begin + q0);
      tma_load_2d(smem_u32(q_s + kBlk), &tmap_q, qb, hq * HD + 64, q_begin + q0);
      const int run = p.page_size < 64 ? p.page_size : 64;       // tokens per TMA box
      const int n_runs = BKV / run;
      // one half (kv = 0: keys, 1: values) of tile j into its stage; false when the wait for the slot ran out
      auto load_half = [&](int j, int kv) -> bool {
        const int st = j & 1;
        uint64_t* empty = kv == 0 ? &bars->k_empty[st] : &bars->v_empty[st];
        uint64_t* full = kv == 0 ? &bars->k_full[st] : &bars->v_full[st];
        if (!mbar_wait(smem_u32(empty), ((j >> 1) & 1) ^ 1)) {
          report(p.status, kTimeoutEmptyBarrier, b, j);
          *abort_flag = 1;
          return false;
        }
        const uint32_t fb = smem_u32(full);
        mbar_expect_tx(fb, 2 * kBlkKV);
        const uint32_t base = smem_u32(kv_s + st * kKVStage) + kv * 2 * kBlkKV;
        for (int r = 0; r < n_runs; ++r) {
          const int tok = j * BKV + r * run;
          int pg = tok / p.page_size;
          if (pg >= p.max_pages) pg = p.max_pages - 1;
          const int page = pt_row[pg];
          const int off = tok - (tok / p.page_size) * p.page_size;
          const int row = ((page * 2 + kv) * p.Hkv + kvh) * p.page_size + off;
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tma_load_2d(base + h * kBlkKV + r * run * 128, &tmap_kv, fb, h * 64, row);
        }
        return true;
      };
      // order of slot availability: K(j + 1) frees after Q K^T (j - 1), V(j) after P V (j - 2), which comes later
      bool fed = load_half(0, 0);
      for (int j = 0; fed && j < n_tiles && !*abort_flag; ++j) {
        if (j + 1 < n_tiles) fed = load_half(j + 1, 0);
        if (fed) fed = load_half(j, 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc(BQ2, BKV, 1, 1);                  // Q (K-major) x K (K-major)
      constexpr uint32_t idesc_pv = make_idesc(BQ2, HD, 1, 1) | (1u << 16);     // P (K-major) x V (MN-major)
      bool ok = mbar_wait(smem_u32(&bars->q_full), 0);
      if (!ok) {
        report(p.status, kTimeoutFullBarrier, b, -1);
        *abort_flag = 1;
      }
      tc_fence_after_sync();
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_pv = [&](int i) -> bool {
        // P_i is in shared memory (and O has been rescaled if that was due)
        if (!mbar_wait(smem_u32(&bars->p_ready[i & 1]), (i >> 1) & 1)) {
          report(p.status, kTimeoutTmemFull, b, 1000 + i);
          return false;
        }
        if (!mbar_wait(smem_u32(&bars->v_full[i & 1]), (i >> 1) & 1)) {
          report(p.status, kTimeoutFullBarrier, b, 5000 + i);
          return false;
        }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(kv_s + (i & 1) * kKVStage) + 2 * kBlkKV;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(p_addr) + 2 * kk;
          const uint64_t db = make_smem_desc_sw128_mn(v_addr + kk * 16 * 128, kBlkKV);
          umma_bf16(tmem_o, da, db, idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars->v_empty[i & 1]));
        umma_commit(smem_u32(&bars->pv_done[i & 1]));
        return true;
      };
      for (int j = 0; ok && j < n_tiles && !*abort_flag; ++j) {
        const int st = j & 1;
        if (!mbar_wait(smem_u32(&bars->k_full[st]), (j >> 1) & 1) ||
            !mbar_wait(smem_u32(&bars->s_free[st]), ((j >> 1) & 1) ^ 1)) {
          report(p.status, kTimeoutFullBarrier, b, j);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(kv_s + st * kKVStage);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t da = make_smem_desc_sw128(q_addr + (kk >> 2) * kBlk) + 2 * (kk & 3);
          const uint64_t db = make_smem_desc_sw128(k_addr + (kk >> 2) * kBlkKV) + 2 * (kk & 3);
          umma_bf16(tmem_base + st * BKV, da, db, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars->k_empty[st]));
        umma_commit(smem_u32(&bars->s_full[st]));
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok && !*abort_flag) ok = issue_pv(n_tiles - 1);
      if (!ok) *abort_flag = 1;
    }
  } else if (n_tiles > 0) {
    // ------------------------------------------------------------------ softmax (warps 2..5, one thread per row)
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(qd * 32) << 16;
    const int r_seq = q0 + row;                                     // row within the sequence's new tokens
    const int kmax = (p.bidirectional || r_seq >= q_len) ? seq - 1 : min(prefix + r_seq, seq - 1);
    const float scale_log2 = p.scale * kLog2e;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      // (votes keep the warp's control flow uniform: one lane per warp arrives on the barriers below)
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->s_full[st]), (j >> 1) & 1))) {
        report(p.status, kTimeoutTmemFull, b, j);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after_sync();
      uint32_t v0[32], v1[32];
      const uint32_t s_addr = tmem_base + lane_base + st * BKV;
      tmem_ld32(s_addr, v0);
      tmem_ld32(s_addr + 32, v1);
      tmem_ld_wait();
      // S_j is in registers: the MMA warp may overwrite this S buffer with tile j + 2
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->s_free[st]));
      const int kv0 = j * BKV;
      const int nvalid = kmax - kv0 + 1;                            // keys [kv0, kv0 + nvalid) are visible
      float mx = -INFINITY;
      if (nvalid >= BKV) {
#pragma unroll
        for (int e = 0; e < 32; ++e) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[e]), __uint_as_float(v1[e])));
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          if (e < nvalid) mx = fmaxf(mx, __uint_as_float(v0[e]));
          if (e + 32 < nvalid) mx = fmaxf(mx, __uint_as_float(v1[e]));
        }
      }
      mx *= scale_log2;
      // the previous P V product must be done before P is overwritten (and before O may be rescaled)
      if (j >= 1 && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&bars->pv_done[(j - 1) & 1]), ((j - 1) >> 1) & 1))) {
        report(p.status, kTimeoutTmemFull, b, 2000 + j);
        *abort_flag = 1;
        ok = false;
        break;
      }
      // Raising the maximum is a warp-wide step (tcgen05.ld / .st are warp-collective): rows that do not need it
      // take part with a factor of one.
      const bool raise = j > 0 && mx > m_used + kRescale;
      if (j == 0) {
        m_used = mx;
      } else if (__any_sync(0xffffffffu, raise)) {
        // rare: bring O and the row sum to the new maximum
        tc_fence_after_sync();
        const float f = raise ? exp2f(m_used - mx) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_base + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
          tmem_st32(tmem_o + lane_base + c0, o);
        }
        tmem_st_wait();
        if (raise) m_used = mx;
      }
      // P = exp2(S * scale - m), bf16, into the swizzled P tile: chunk c (8 keys) of this row
      float sum = 0.f;
      uint8_t* prow = p_s + row * 128;
      const int sw = row & 7;
      const bool full = nvalid >= BKV;                  // no key of this tile is masked for this row
      auto emit = [&](const uint32_t (&v)[32], int cbase) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float e8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float pv = ex2_approx(fmaf(__uint_as_float(v[c * 8 + e]), scale_log2, -m_used));
            if (!full && cbase * 8 + c * 8 + e >= nvalid) pv = 0.f;
            e8[e] = pv;
          }
          sum += ((e8[0] + e8[1]) + (e8[2] + e8[3])) + ((e8[4] + e8[5]) + (e8[6] + e8[7]));
          const int chunk = cbase + c;                  // 0..7 over the 64 keys
          const uint4 packed = make_uint4(pack_bf16(e8[0], e8[1]), pack_bf16(e8[2], e8[3]), pack_bf16(e8[4], e8[5]),
                                          pack_bf16(e8[6], e8[7]));
          *reinterpret_cast<uint4*>(prow + ((chunk ^ sw) << 4)) = packed;
        }
      };
      emit(v0, 0);
      emit(v1, 4);
      l += sum;
      // make the generic-proxy writes visible to the tensor core's async proxy, then hand P over
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars->p_ready[st]));
    }
    // epilogue: O / l
    if (ok && mbar_wait(smem_u32(&bars->pv_done[(n_tiles - 1) & 1]), ((n_tiles - 1) >> 1) & 1)) {
      tc_fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(q_begin + r_seq) * p.Hq + hq) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_base + c0, o);
        tmem_ld_wait();
        if (r_seq < q_len) {
#pragma unroll
          for (int e = 0; e < 32; e += 8)
            *reinterpret_cast<uint4*>(orow + c0 + e) =
                make_uint4(pack_bf16(__uint_as_float(o[e]) * inv, __uint_as_float(o[e + 1]) * inv),
                           pack_bf16(__uint_as_float(o[e + 2]) * inv, __uint_as_float(o[e + 3]) * inv),
                           pack_bf16(__uint_as_float(o[e + 4]) * inv, __uint_as_float(o[e + 5]) * inv),
                           pack_bf16(__uint_as_float(o[e + 6]) * inv, __uint_as_float(o[e + 7]) * inv));
        }
      }
    } else if (ok) {
      report(p.status, kTimeoutTmemFull, b, 3000);
      *abort_flag = 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// tensor map over the whole page pool viewed as [num_pages*2*Hkv*P, D]; box = 64 x min(P, 64)
struct TmapKey {
  const void* ptr;
  long long rows;
  int D, box_rows;
  bool operator==(const TmapKey& o) const { return ptr == o.ptr && rows == o.rows && D == o.D && box_rows == o.box_rows; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    return std::hash<const void*>()(k.ptr) ^ (std::hash<long long>()(k.rows) * 31) ^ (k.D * 131) ^ (k.box_rows * 7);
  }
};
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;

bool get_kv_tmap(const void* kv, long long rows, int D, int page_size, CUtensorMap* out) {
  const int box_rows = page_size < TN ? page_size : TN;
  TmapKey key{kv, rows, D, box_rows};
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out = it->second;
    return true;
  }
  CUtensorMap m;
  if (!encode_tmap_2d(&m, kv, D, rows, static_cast<uint64_t>(D) * 2, 64, box_rows, 2)) return false;
  if (g_tmaps.size() > 4096) g_tmaps.clear();
  g_tmaps.emplace(key, m);
  *out = m;
  return true;
}

template <int D>
int smem_bytes(int stages) { return stages * Stage<D>::kBytes + stages * 16 + 64 + 1024; }

}  // namespace
}  // namespace sglb

extern "C" {

// Suggested number of KV splits for a decode launch (fixed per CUDA graph).
int sglb_decode_num_splits(int B, int Hkv, int max_seq_len) {
  const int sms = sglb::sm_count();
  const int ctas = B * Hkv;
  int splits = (2 * sms + ctas - 1) / ctas;
  const int tiles = (max_seq_len + sglb::TN - 1) / sglb::TN;
  splits = splits < 1 ? 1 : splits;
  if (splits > tiles / 2) splits = tiles / 2 > 0 ? tiles / 2 : 1;
  if (splits > 32) splits = 32;
  return splits;
}

int sglb_paged_decode(const void* q, void* out, const void* kv_buffer, long long num_pages, const int* page_table,
                      int max_pages, const int* req_pool_indices, const int* seq_lens, int B, int Hq, int Hkv, int D,
                      int page_size, float scale, int window, float soft_cap, int num_splits, float* part_o,
                      float* part_lse, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv != 0 || Hq / Hkv > 16) return -kBadArgument;
  if (page_size < TN ? (TN % page_size != 0) : (page_size % TN != 0)) return -kBadArgument;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return -kBadArgument;
  CUtensorMap tm;
  if (!get_kv_tmap(kv_buffer, num_pages * 2 * Hkv * page_size, D, page_size, &tm)) return -100;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o;
  p.part_lse = part_lse;
  p.page_table = page_table;
  p.req_pool_indices = req_pool_indices;
  p.seq_lens = seq_lens;
  p.status = device_status();
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.max_pages = max_pages; p.page_size = page_size;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  p.window = window; p.scale = scale; p.soft_cap = soft_cap;
  // measured 135 -> 131 us at B=128, 8 KV heads, 1400 tokens (110 -> 101 us at B=32, 4096 tokens)
  static const int evf = [] { const char* e = getenv("SGLB_DECODE_KV_EVICT_FIRST"); return e ? atoi(e) : 1; }();
  p.kv_evict_first = evf;
  // 3 stages of 32 KB leave room for two CTAs per SM (registers allow two): measured 134 us vs 150 us with
  // 4 stages / one CTA per SM at B=128, 8 KV heads, 1400 tokens
  const int stages = 3;
  dim3 grid(B, Hkv, p.num_splits);
  cudaError_t e;
  if (D == 128) {
    static bool cfg = false;
    const int sm = smem_bytes<128>(stages);
    if (!cfg) { cudaFuncSetAttribute(paged_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm); cfg = true; }
    launch_pdl(paged_decode_kernel<128>, grid, dim3(kThreads), sm, stream, tm, p, stages);
    e = cudaGetLastError();
    if (e == cudaSuccess && p.num_splits > 1) {
      launch_pdl(decode_combine_kernel<128>, dim3(B * Hq), dim3(128), 0, stream, part_o, part_lse, p.out, p.num_splits);
      e = cudaGetLastError();
    }
  } else {
    static bool cfg = false;
    const int sm = smem_bytes<64>(stages);
    if (!cfg) { cudaFuncSetAttribute(paged_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm); cfg = true; }
    launch_pdl(paged_decode_kernel<64>, grid, dim3(kThreads), sm, stream, tm, p, stages);
    e = cudaGetLastError();
    if (e == cudaSuccess && p.num_splits > 1) {
      launch_pdl(decode_combine_kernel<64>, dim3(B * Hq), dim3(64), 0, stream, part_o, part_lse, p.out, p.num_splits);
      e = cudaGetLastError();
    }
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// Causal (or bidirectional: `bidirectional` != 0) prefill attention for head_dim 128 on tcgen05 (see
// paged_extend_tc_kernel).  `total_q` = rows of q; `num_q_tiles_bound` >= sum_b ceil(q_len_b / 128).
int sglb_paged_extend_tc(const void* q, void* out, const void* kv_buffer, long long num_pages, const int* page_table,
                         int max_pages, const int* req_pool_indices, const int* seq_lens, const int* prefix_lens,
                         const int* cu_q_lens, int B, int num_q_tiles_bound, int total_q, int Hq, int Hkv, int D,
                         int page_size, float scale, int bidirectional, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0 || num_q_tiles_bound <= 0 || total_q <= 0) return 0;
  if (D != 128 || Hq % Hkv != 0) return -kBadArgument;
  if (page_size < TN ? (TN % page_size != 0) : (page_size % TN != 0)) return -kBadArgument;
  CUtensorMap tm, tq;
  if (!get_kv_tmap(kv_buffer, num_pages * 2 * Hkv * page_size, D, page_size, &tm)) return -100;
  // q viewed as [total_q, Hq * D]: one box = 128 rows x 64 columns (half a head)
  if (!encode_tmap_2d(&tq, q, static_cast<uint64_t>(Hq) * D, total_q, static_cast<uint64_t>(Hq) * D * 2, 64, 128, 2))
    return -101;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table;
  p.req_pool_indices = req_pool_indices;
  p.seq_lens = seq_lens;
  p.prefix_lens = prefix_lens;
  p.cu_q_lens = cu_q_lens;
  p.status = device_status();
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.max_pages = max_pages; p.page_size = page_size;
  p.num_splits = 1; p.scale = scale;
  p.bidirectional = bidirectional;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(paged_extend_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tc::kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    // two CTAs per SM need the whole shared-memory carve-out
    cudaFuncSetAttribute(paged_extend_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cfg = true;
  }
  dim3 grid(num_q_tiles_bound, Hq, 1);
  paged_extend_tc_kernel<<<grid, tc::kThreadsTc, tc::kSmem, stream>>>(tm, tq, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

// `num_q_tiles_bound` >= sum_b ceil(q_len_b / 64); T/64 + B always is.
// `tail_mask` (optional, [B, mask_rows, tail_len] bytes): visibility of the last `tail_len` keys of
// every sequence per query row; earlier keys are visible to all rows and the causal rule is dropped.
int sglb_paged_extend_masked(const void* q, void* out, const void* kv_buffer, long long num_pages,
                             const int* page_table, int max_pages, const int* req_pool_indices, const int* seq_lens,
                             const int* prefix_lens, const int* cu_q_lens, int B, int num_q_tiles_bound, int Hq,
                             int Hkv, int D, int page_size, float scale, int window, float soft_cap,
                             const void* tail_mask, int tail_len, int mask_rows, cudaStream_t stream);

int sglb_paged_extend(const void* q, void* out, const void* kv_buffer, long long num_pages, const int* page_table,
                      int max_pages, const int* req_pool_indices, const int* seq_lens, const int* prefix_lens,
                      const int* cu_q_lens, int B, int num_q_tiles_bound, int Hq, int Hkv, int D, int page_size,
                      float scale, int window, float soft_cap, cudaStream_t stream) {
  return sglb_paged_extend_masked(q, out, kv_buffer, num_pages, page_table, max_pages, req_pool_indices, seq_lens,
                                  prefix_lens, cu_q_lens, B, num_q_tiles_bound, Hq, Hkv, D, page_size, scale, window,
                                  soft_cap, nullptr, 0, 0, stream);
}

int sglb_paged_extend_masked(const void* q, void* out, const void* kv_buffer, long long num_pages,
                             const int* page_table, int max_pages, const int* req_pool_indices, const int* seq_lens,
                             const int* prefix_lens, const int* cu_q_lens, int B, int num_q_tiles_bound, int Hq,
                             int Hkv, int D, int page_size, float scale, int window, float soft_cap,
                             const void* tail_mask, int tail_len, int mask_rows, cudaStream_t stream) {
  using namespace sglb;
  if (tail_mask != nullptr && (tail_len <= 0 || mask_rows <= 0)) return -kBadArgument;
  if (B <= 0 || num_q_tiles_bound <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv != 0) return -kBadArgument;
  if (page_size < TN ? (TN % page_size != 0) : (page_size % TN != 0)) return -kBadArgument;
  CUtensorMap tm;
  if (!get_kv_tmap(kv_buffer, num_pages * 2 * Hkv * page_size, D, page_size, &tm)) return -100;
  AttnParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.page_table = page_table;
  p.req_pool_indices = req_pool_indices;
  p.seq_lens = seq_lens;
  p.prefix_lens = prefix_lens;
  p.cu_q_lens = cu_q_lens;
  p.status = device_status();
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.max_pages = max_pages; p.page_size = page_size;
  p.num_splits = 1; p.window = window; p.scale = scale; p.soft_cap = soft_cap;
  p.tail_mask = static_cast<const uint8_t*>(tail_mask);
  p.tail_len = tail_mask ? tail_len : 0;
  p.mask_rows = mask_rows;
  p.bidirectional = (tail_mask == nullptr && mask_rows < 0) ? 1 : 0;   // mask_rows -1 without a mask: no causal rule
  const int stages = 3;
  dim3 grid(num_q_tiles_bound, Hq, 1);
  cudaError_t e;
  if (D == 128) {
    static bool cfg = false;
    const int sm = smem_bytes<128>(stages);
    if (!cfg) { cudaFuncSetAttribute(paged_extend_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm); cfg = true; }
    paged_extend_kernel<128><<<grid, kThreads, sm, stream>>>(tm, p, stages);
    e = cudaGetLastError();
  } else {
    static bool cfg = false;
    const int sm = smem_bytes<64>(stages);
    if (!cfg) { cudaFuncSetAttribute(paged_extend_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, sm); cfg = true; }
    paged_extend_kernel<64><<<grid, kThreads, sm, stream>>>(tm, p, stages);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
}
