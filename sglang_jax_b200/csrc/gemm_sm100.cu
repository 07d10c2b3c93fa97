// bf16 GEMM  out[M, N] = x[M, K] . w[N, K]^T (+ bias)  on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel:
//   warp 0      TMA producer: 128-byte-swizzled operand tiles into a multi-stage smem ring
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) per 16-wide K slice,
//               tcgen05.commit releases smem stages / publishes finished accumulators
//   warps 2..5  epilogue: tcgen05.ld the fp32 accumulator out of tensor memory, convert, store
// The accumulator is double buffered in tensor memory (2 x BN columns) so the epilogue of tile
// i overlaps the main loop of tile i+1.
//
// Two operand assignments share the kernel:
//   MODE 0 ("tokens on M")   A = x tile (128 tokens), B = w tile (BN outputs).  Prefill.
//   MODE 1 ("weights on M")  A = w tile (128 outputs), B = x (all tokens, BN >= M).  Decode:
//          the 128-row MMA dimension is filled with weight rows, so a batch of 1..256 tokens
//          wastes no tensor-core rows, weights are streamed exactly once, and K is split over
//          CTAs so that all SMs pull HBM bandwidth.  Split partials go through an fp32
//          workspace; the CTA that arrives last for a tile sums them in split order
//          (deterministic) and writes the bf16 result.
//
// The reference project has no counterpart kernel: its dense projections are
// `lax.dot_general` calls lowered by XLA (python/sgl_jax/srt/layers/linear.py:102).
#include <cstdlib>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "common.cuh"
#include "gemm_noalloc.h"

namespace sglb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int kNumThreads = 192;
constexpr int kEpiThreads = 128;
constexpr int kDoneCounterOffset = 2048;   // second counter bank (stream-K clean-up)

template <int BN>
struct Cfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : 2 * BN;      // power of two for BN in {16..256}
  static constexpr int kStagingBytes = 4 * 32 * 32 * 2;             // per-epilogue-warp 32x32 bf16 transpose tile
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarBytes + 1024;  // +1024 alignment slack
  static constexpr int CW = BN >= 32 ? 32 : 16;                      // columns per tcgen05.ld
};

struct Params {
  __nv_bfloat16* out;            // [M, N] row-major
  const __nv_bfloat16* bias;     // [N] or null
  float* workspace;              // split-K partials: [tile][split][BN][128] fp32
  int* counters;                 // one per output tile, zero when idle
  Status* status;
  int M, N, K;
  int tiles_a, tiles_b;          // tiles along the A-operand rows / B-operand rows
  int splits;                    // K splits (interleaved policy); workspace slots per tile
  int kb_total;                  // K blocks (ceil(K / 64))
  int units_per_cta;             // > 0: stream-K policy, each CTA owns this many consecutive K-block units
  int total_units;               // tiles * kb_total
  // grouped GEMM (MoE experts): rows of x are sorted by group, w is [groups * N, K]
  const int* group_offsets;      // [groups + 1] row offsets into x / out, device memory; null = dense
  const int* tile_group;         // MODE 0: group of each 128-row token tile
  const int* tile_row0;          // MODE 0: first row of each token tile
  const int* num_token_tiles;    // MODE 0: number of valid entries in the two lists (device scalar)
  int groups;
  // fused reduce-scatter epilogue (tensor parallel row-parallel GEMM): token row t of the partial
  // product is stored straight into the receive buffer of the rank that owns the row,
  //   rs_peer[t / rs_rows_per] + ((rs_rank * rs_rows_per + t % rs_rows_per) * N + n),
  // over NVLink peer mappings, tile by tile while the remaining tiles are still being computed.
  __nv_bfloat16* rs_peer[8];
  int rs_world, rs_rank, rs_rows_per;
  unsigned long long* debug_stamps;   // optional [16] globaltimer stamps of CTA 0 (profiling aid)
  int l2_hints;                       // decode mode: stream weights evict-first, keep the token tile evict-last
  const float* scale_x;               // fp8: per-token activation scale [M]
  const float* scale_w;               // fp8: per-output-channel weight scale [N]
  // ---- FUSE == 1: the same kernel also reduces the received slices, adds the residual, applies RMSNorm and
  // all-gathers the normalised rows (see "fused tail" below).  Row ownership: rank o owns token rows
  // [o * rs_rows_per, (o + 1) * rs_rows_per), cut into chunks of kChunkRows rows.
  __nv_bfloat16* ag_peer[8];          // every rank's [M, N] buffer of normalised activations
  __nv_bfloat16* ag_mc;               // NVSwitch multicast address of that buffer (multimem.st) or null
  uint32_t* flag_peer[8];             // every rank's flag block (kFlagWords u32, symmetric memory)
  __nv_bfloat16* residual;            // [M, N] local residual stream (rows of this rank's slice are updated) or null
  const __nv_bfloat16* norm_w;        // [N]
  uint32_t* seq;                      // device-resident call counter of the fused context (local memory)
  int* tail_ctrs;                     // local counters (kTailCtrInts ints), zero when idle
  float eps;
  int gemma, defer, per_tile, nchunks;
  // ---- FUSE == 2: the token operand is the all-gather buffer written by a FUSE == 1 launch that did not
  // wait for its peers: the TMA producer waits for the arrival flag of a chunk before its first load of it.
  const uint32_t* ag_flags;           // this rank's flag block
  const uint32_t* ag_seq;
  int ag_world, ag_rows_per, ag_nchunks;
};

// Flag block layout (u32, epoch valued, symmetric memory):
//   [kRsFlag + chunk * 8 + src]      on the owner: src's partial rows of that chunk have all been pushed
//   [kAgFlag + owner * kMaxChunks + chunk]  on every rank: the owner's normalised rows of that chunk have landed
constexpr int kChunkRows = 128;
constexpr int kMaxChunks = 160;
constexpr int kRsFlag = 0;
constexpr int kAgFlag = kMaxChunks * 8;
constexpr int kFlagWords = kAgFlag + 8 * kMaxChunks;
// local counters: [0] CTAs done with their GEMM work, [1] CTAs that left the tail, then per chunk: next row to
// hand out, rows finished, and (per 128-row token tile) weight tiles finished
constexpr int kCtrDone = 0, kCtrExit = 1, kCtrNextRow = 8, kCtrRowsDone = kCtrNextRow + kMaxChunks,
              kCtrTile = kCtrRowsDone + kMaxChunks, kTailCtrInts = kCtrTile + kMaxChunks;

// Ownership layout shared by the producer, the consumer and the host: large batches (at least four 128-row
// tiles per rank) are cut into slices that are multiples of 128 rows: a token tile never straddles two
// owners, so arrival can be signalled per tile, at the price of slices that differ by up to one tile.
// Smaller batches are split evenly to the row and signalled once per rank.
__host__ __device__ inline void fused_layout(int M, int world, int* rows_per, int* nchunks, int* per_tile) {
  if (M >= 4 * kChunkRows * world && M > 256) {
    const int r = (M + world - 1) / world;
    *rows_per = (r + kChunkRows - 1) / kChunkRows * kChunkRows;
    *nchunks = *rows_per / kChunkRows;
    *per_tile = 1;
  } else {
    *rows_per = (M + world - 1) / world;
    *nchunks = (*rows_per + kChunkRows - 1) / kChunkRows;
    *per_tile = 0;
  }
}

__device__ __forceinline__ __nv_bfloat16* out_ptr(const Params& p, int tok, int gn) {
  if (p.rs_world == 0) return p.out + static_cast<size_t>(tok) * p.N + gn;
  const int owner = tok / p.rs_rows_per;
  const int local = tok - owner * p.rs_rows_per;
  return p.rs_peer[owner] + (static_cast<size_t>(p.rs_rank) * p.rs_rows_per + local) * p.N + gn;
}

// One piece of work: K blocks [kb0, kb1) of output tile (ta, tb).  `n_contrib` CTAs contribute to
// the tile; this one writes workspace slot `slot` (n_contrib == 1: the tile is stored directly).
struct Seg {
  int ta, tb, kb0, kb1, tile_id, slot, n_contrib;
  int a_row, b_row;     // TMA row coordinates of the A / B operand tiles
  int m0, m_limit;      // first output token row of the tile, exclusive bound of valid token rows
  int n0;               // first output column of the tile
  int w_off;            // offset of this tile's weight rows in `scale_w` (grouped: group * N)
};

// Two decompositions share the kernel:
//  * interleaved (units_per_cta == 0): work item w = blockIdx.x + i * gridDim.x is a whole tile or one
//    of `splits` equal K ranges of it.  Consecutive CTAs take consecutive A tiles of the same B
//    tile, so the B tile is fetched from HBM once and then hit in L2 (prefill).
//  * stream-K (units_per_cta > 0): the tiles' K blocks form one long list that is cut into equal
//    consecutive ranges, one per CTA, so every SM streams the same number of weight bytes whatever
//    the tile count is (decode).  A range may end / start in the middle of a tile: those tiles get
//    their partial sums through the workspace.
template <int BN, int MODE>
struct SegIter {
  int it, u, u_end;
  __device__ explicit SegIter(const Params& p) : it(0), u(0), u_end(0) {
    if (p.units_per_cta > 0) {
      u = blockIdx.x * p.units_per_cta;
      u_end = min(p.total_units, u + p.units_per_cta);
    }
  }
  __device__ __forceinline__ void dense_coords(const Params& p, Seg& s) const {
    s.a_row = s.ta * BM;
    s.b_row = s.tb * BN;
    if (MODE == 0) {
      s.m0 = s.ta * BM;
      s.n0 = s.tb * BN;
    } else {
      s.m0 = s.tb * BN;
      s.n0 = s.ta * BM;
    }
    s.m_limit = p.M;
    s.w_off = 0;
  }
  __device__ bool next(const Params& p, Seg& s) {
    if (p.group_offsets != nullptr) return MODE == 0 ? next_grouped_tokens_on_m(p, s) : next_grouped_weights_on_m(p, s);
    if (p.units_per_cta > 0) {
      if (u >= u_end) return false;
      const int tile = u / p.kb_total;
      s.kb0 = u - tile * p.kb_total;
      s.kb1 = min(p.kb_total, s.kb0 + (u_end - u));
      u += s.kb1 - s.kb0;
      s.tile_id = tile;
      s.tb = tile / p.tiles_a;
      s.ta = tile - s.tb * p.tiles_a;
      const int first_cta = (tile * p.kb_total) / p.units_per_cta;
      const int last_cta = ((tile + 1) * p.kb_total - 1) / p.units_per_cta;
      s.slot = blockIdx.x - first_cta;
      s.n_contrib = last_cta - first_cta + 1;
      dense_coords(p, s);
      return true;
    }
    const int num_tiles = p.tiles_a * p.tiles_b;
    const int w = blockIdx.x + it * gridDim.x;
    if (w >= num_tiles * p.splits) return false;
    ++it;
    const int sp = w / num_tiles;
    const int t = w - sp * num_tiles;
    const int kb_per_split = (p.kb_total + p.splits - 1) / p.splits;
    s.tb = t / p.tiles_a;
    s.ta = t - s.tb * p.tiles_a;
    s.kb0 = sp * kb_per_split;
    s.kb1 = min(s.kb0 + kb_per_split, p.kb_total);
    s.tile_id = t;
    s.slot = sp;
    s.n_contrib = p.splits;
    dense_coords(p, s);
    return true;
  }
  // Grouped, decode shape: stream-K over (group, weight tile, K block); the group's tokens are the
  // B operand (at most BN of them).  Groups without tokens are skipped.
  __device__ bool next_grouped_weights_on_m(const Params& p, Seg& s) {
    while (u < u_end) {
      const int tile = u / p.kb_total;                 // = group * tiles_a + ta
      const int g = tile / p.tiles_a;
      const int row_lo = p.group_offsets[g], row_hi = p.group_offsets[g + 1];
      const int kb0 = u - tile * p.kb_total;
      const int kb1 = min(p.kb_total, kb0 + (u_end - u));
      u += kb1 - kb0;
      if (row_hi <= row_lo) continue;
      s.kb0 = kb0;
      s.kb1 = kb1;
      s.tile_id = tile;
      s.ta = tile - g * p.tiles_a;
      s.tb = 0;
      const int first_cta = (tile * p.kb_total) / p.units_per_cta;
      const int last_cta = ((tile + 1) * p.kb_total - 1) / p.units_per_cta;
      s.slot = blockIdx.x - first_cta;
      s.n_contrib = last_cta - first_cta + 1;
      s.a_row = g * p.N + s.ta * BM;
      s.w_off = g * p.N;
      s.b_row = row_lo;
      s.m0 = row_lo;
      s.m_limit = min(row_hi, row_lo + BN);
      s.n0 = s.ta * BM;
      return true;
    }
    return false;
  }
  // Grouped, prefill shape: whole (token tile, weight tile) pairs from the device-side tile list.
  __device__ bool next_grouped_tokens_on_m(const Params& p, Seg& s) {
    const int n_tok_tiles = *p.num_token_tiles;
    const int w = blockIdx.x + it * gridDim.x;
    if (w >= n_tok_tiles * p.tiles_b) return false;
    ++it;
    s.tb = w / n_tok_tiles;
    s.ta = w - s.tb * n_tok_tiles;
    const int g = p.tile_group[s.ta];
    const int row0 = p.tile_row0[s.ta];
    s.kb0 = 0;
    s.kb1 = p.kb_total;
    s.tile_id = w;
    s.slot = 0;
    s.n_contrib = 1;
    s.a_row = row0;
    s.b_row = g * p.N + s.tb * BN;
    s.w_off = g * p.N;
    s.m0 = row0;
    s.m_limit = min(p.group_offsets[g + 1], row0 + BM);
    s.n0 = s.tb * BN;
    return true;
  }
};

// FP8: both operands are e4m3 bytes (128 per swizzle row instead of 64 bf16, so the byte layout of a
// stage is unchanged), `tcgen05.mma.kind::f8f6f4` accumulates in fp32 and the epilogue multiplies by
// `scale_x[token] * scale_w[channel]` (per-token activation scale, per-channel weight scale).
template <int BN, int MODE, bool FP8 = false, int FUSE = 0>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const Params p) {
  using C = Cfg<BN>;
  constexpr int kBKE = FP8 ? 2 * BK : BK;       // elements per K block (128 bytes either way)
  extern __shared__ uint8_t smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + C::kStagingBytes);
  uint64_t* full_bar = bars;                         // [kStages]
  uint64_t* empty_bar = bars + C::kStages;           // [kStages]
  uint64_t* tmem_full_bar = bars + 2 * C::kStages;   // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  auto stamp = [&](int i) {
    if (p.debug_stamps != nullptr && blockIdx.x == 0) p.debug_stamps[i] = global_timer_ns();
  };
  if (threadIdx.x == 0) stamp(0);

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tmem_full_bar[a]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[a]), kEpiThreads);
    }
    *abort_flag = 0;
    *last_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // everything above is CTA-local; operands, counters and the tile lists may come from the previous kernel
  pdl_wait();
  if (threadIdx.x == 0) stamp(1);
  // fused tail: every launch of the fused context is one epoch; the last CTA to leave publishes it
  [[maybe_unused]] uint32_t epoch = 0;
  if constexpr (FUSE == 1) epoch = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      SegIter<BN, MODE> iter(p);
      Seg sg;
      // decode mode: operand A is the weight matrix, read exactly once by the whole grid; operand B is
      // the token tile every CTA re-reads for each k-block
      const uint64_t pol_a = l2_policy_evict_first(), pol_b = l2_policy_evict_last();
      [[maybe_unused]] uint32_t ag_epoch = 0;
      [[maybe_unused]] unsigned long long ag_seen[(8 * kMaxChunks + 63) / 64] = {};
      if constexpr (FUSE == 2) ag_epoch = *reinterpret_cast<const volatile uint32_t*>(p.ag_seq);
      // rows [r_lo, r_hi) of the gathered buffer are about to be read: wait for their chunks' arrival flags
      auto ag_wait_rows = [&](int r_lo, int r_hi) -> bool {
        if constexpr (FUSE == 2) {
          r_hi = min(r_hi, p.M);
          for (int r = r_lo; r < r_hi;) {
            const int o = r / p.ag_rows_per;
            const int j = (r - o * p.ag_rows_per) / kChunkRows;
            const int id = o * kMaxChunks + j;
            if (!((ag_seen[id >> 6] >> (id & 63)) & 1ull)) {
              if (!wait_flag_ge(p.ag_flags + kAgFlag + id, ag_epoch)) {
                report(p.status, kTimeoutPeerFlag, o, 20 + j);
                return false;
              }
              ag_seen[id >> 6] |= 1ull << (id & 63);
            }
            r = min(o * p.ag_rows_per + (j + 1) * kChunkRows, (o + 1) * p.ag_rows_per);   // first row of the next chunk
          }
        }
        return true;
      };
      while (!*abort_flag && iter.next(p, sg)) {
        if constexpr (FUSE == 2) {
          const bool got = MODE == 0 ? ag_wait_rows(sg.a_row, sg.a_row + BM) : ag_wait_rows(0, p.M);
          if (!got) {
            *abort_flag = 1;
            break;
          }
        }
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
            report(p.status, kTimeoutEmptyBarrier, sg.tile_id, kb);
            *abort_flag = 1;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, C::kStageBytes);
          uint8_t* sa = stage_base + stage * C::kStageBytes;
          if (MODE == 1 && p.l2_hints) {
            tma_load_2d_hint(smem_u32(sa), &tmap_a, fb, kb * kBKE, sg.a_row, pol_a);
            tma_load_2d_hint(smem_u32(sa + C::kStageBytesA), &tmap_b, fb, kb * kBKE, sg.b_row, pol_b);
          } else {
            tma_load_2d(smem_u32(sa), &tmap_a, fb, kb * kBKE, sg.a_row);
            tma_load_2d(smem_u32(sa + C::kStageBytesA), &tmap_b, fb, kb * kBKE, sg.b_row);
          }
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      stamp(2);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = FP8 ? make_idesc(BM, BN, 0, 0) : make_idesc(BM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      SegIter<BN, MODE> iter(p);
      Seg sg;
      while (!*abort_flag && iter.next(p, sg)) {
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[acc]), acc_phase ^ 1)) {
          report(p.status, kTimeoutTmemEmpty, sg.tile_id, acc);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
            report(p.status, kTimeoutFullBarrier, sg.tile_id, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stage_base + stage * C::kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + C::kStageBytesA);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advance 16 bf16 = 32 bytes along K inside the swizzle row: +2 in 16-byte units
            if constexpr (FP8) umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            else umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));
          if (++stage == C::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&tmem_full_bar[acc]));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      stamp(3);
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                 // TMEM lane quadrant this warp may access
    const int row = q * 32 + lane;          // accumulator row (0..127) of this thread
    const int epi_tid = threadIdx.x - 64;   // 0..127
    uint8_t* my_stage = staging + q * (32 * 32 * 2);
    int acc = 0;
    uint32_t acc_phase = 0;
    Seg pending[2];
    int n_pending = 0;
    SegIter<BN, MODE> iter(p);
    Seg sg;
    auto store_chunk = [&](const Seg& sg, const float* f, int c0) {
      // f[0..CW): accumulator row `row`, columns c0..c0+CW of this tile
      if constexpr (MODE == 0) {
        // rows are tokens, columns are outputs: transpose through smem so that global stores
        // are 16-byte vectors covering whole 64-byte row segments
        const int gm0 = sg.m0 + q * 32;
        const int gn0 = sg.n0 + c0;
        float sx = 1.f;
        if constexpr (FP8) sx = (gm0 + lane) < sg.m_limit ? p.scale_x[gm0 + lane] : 0.f;
#pragma unroll
        for (int j = 0; j < C::CW / 8; ++j) {
          float g[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            g[e] = f[j * 8 + e];
            if constexpr (FP8) {
              const int gn = gn0 + j * 8 + e;
              g[e] *= sx * (gn < p.N ? p.scale_w[sg.w_off + gn] : 0.f);
            }
            if (p.bias != nullptr) {
              const int gn = gn0 + j * 8 + e;
              if (gn < p.N) g[e] += __bfloat162float(p.bias[gn]);
            }
          }
          uint4 v = make_uint4(pack_bf16(g[0], g[1]), pack_bf16(g[2], g[3]), pack_bf16(g[4], g[5]),
                               pack_bf16(g[6], g[7]));
          const int pj = j ^ ((lane >> 1) & (C::CW / 8 - 1));
          *reinterpret_cast<uint4*>(my_stage + lane * (C::CW * 2) + pj * 16) = v;
        }
        __syncwarp();
        constexpr int kChunksPerRow = C::CW / 8;            // 16-byte chunks per staged row
        constexpr int kRowsPerIt = 32 / kChunksPerRow;
#pragma unroll
        for (int it = 0; it < 32 / kRowsPerIt; ++it) {
          const int r = it * kRowsPerIt + lane / kChunksPerRow;
          const int jj = lane % kChunksPerRow;
          const int pj = jj ^ ((r >> 1) & (kChunksPerRow - 1));
          const uint4 v = *reinterpret_cast<const uint4*>(my_stage + r * (C::CW * 2) + pj * 16);
          const int gm = gm0 + r;
          const int gn = gn0 + jj * 8;
          if (gm < sg.m_limit && gn < p.N) {
            *reinterpret_cast<uint4*>(out_ptr(p, gm, gn)) = v;
          }
        }
        __syncwarp();
      } else {
        // rows are outputs (weight rows), columns are tokens: out[token][n].  Transpose the
        // [128 n] x [CW tokens] chunk through shared memory so that every token's 128 outputs
        // leave as 16-byte vectors (256 contiguous bytes per token).
        __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(staging);
        const int gn_row = sg.n0 + row;
        const float b = (p.bias != nullptr && gn_row < p.N) ? __bfloat162float(p.bias[gn_row]) : 0.f;
        if constexpr (FP8) {
          const float sw = gn_row < p.N ? p.scale_w[sg.w_off + gn_row] : 0.f;
#pragma unroll
          for (int e = 0; e < C::CW; ++e) {
            const int tok = sg.m0 + c0 + e;
            st[e * BM + row] = __float2bfloat16(f[e] * sw * (tok < sg.m_limit ? p.scale_x[tok] : 0.f) + b);
          }
        } else {
#pragma unroll
          for (int e = 0; e < C::CW; ++e) st[e * BM + row] = __float2bfloat16(f[e] + b);
        }
        named_bar_sync(2, kEpiThreads);
#pragma unroll
        for (int v = 0; v < C::CW * (BM / 8) / kEpiThreads; ++v) {
          const int vid = v * kEpiThreads + epi_tid;
          const int e = vid / (BM / 8);
          const int part = vid - e * (BM / 8);
          const int tok = sg.m0 + c0 + e;
          const int gn = sg.n0 + part * 8;
          if (tok < sg.m_limit && gn < p.N)
            *reinterpret_cast<uint4*>(out_ptr(p, tok, gn)) = *reinterpret_cast<const uint4*>(st + e * BM + part * 8);
        }
        named_bar_sync(2, kEpiThreads);
      }
    };
    while (!*abort_flag && iter.next(p, sg)) {
      if (!mbar_wait(smem_u32(&tmem_full_bar[acc]), acc_phase)) {
        report(p.status, kTimeoutTmemFull, sg.tile_id, acc);
        *abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      if (epi_tid == 0) stamp(4);
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int tile_id = sg.tile_id;
      const bool direct = (sg.n_contrib == 1);
      float* ws_tile = direct ? nullptr
                              : p.workspace + (static_cast<size_t>(tile_id) * p.splits + sg.slot) * (BM * BN);


#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += C::CW) {
        uint32_t v[32];
        if constexpr (C::CW == 32) tmem_ld32(t_addr + c0, v);
        else tmem_ld16(t_addr + c0, v);
        tmem_ld_wait();
        if (direct) {
          float f[C::CW];
#pragma unroll
          for (int e = 0; e < C::CW; ++e) f[e] = __uint_as_float(v[e]);
          store_chunk(sg, f, c0);
        } else {
          // layout [col / 4][row][4]: the 32 rows of a warp write 512 contiguous bytes
          uint4* dst = reinterpret_cast<uint4*>(ws_tile) + (c0 / 4) * BM + row;
#pragma unroll
          for (int e = 0; e < C::CW / 4; ++e) dst[e * BM] = make_uint4(v[4 * e], v[4 * e + 1], v[4 * e + 2], v[4 * e + 3]);
        }
      }
      // accumulator drained: hand the TMEM buffer back to the MMA warp
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&tmem_empty_bar[acc]));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;

      if constexpr (FUSE == 1 && MODE == 0) {
        if (p.per_tile && direct) {
          // this rank's partial rows of token tile `ta`: once all weight tiles of the token tile have been
          // pushed, tell the owner of those rows (release at system scope orders the peer stores before it)
          named_bar_sync(1, kEpiThreads);
          if (epi_tid == 0) {
            fence_acq_rel_sys();
            const int old = atomicAdd(&p.tail_ctrs[kCtrTile + sg.ta], 1);
            if (old == p.tiles_b - 1) {
              fence_acq_rel_sys();
              const int owner = sg.m0 / p.rs_rows_per;
              const int j = (sg.m0 - owner * p.rs_rows_per) / kChunkRows;
              st_release_sys(p.flag_peer[owner] + kRsFlag + j * 8 + p.rs_rank, epoch);
            }
          }
        }
      }

      if (!direct) {
        __threadfence();
        named_bar_sync(1, kEpiThreads);
        if (epi_tid == 0) stamp(8);
        if (p.units_per_cta > 0) {
          // stream-K: publish the partial now, reduce later (after all of this CTA's partials are
          // out, so that no CTA ever waits for a CTA that is itself waiting)
          if (epi_tid == 0) atomicAdd(&p.counters[tile_id], 1);
          if (n_pending < 2) pending[n_pending++] = sg;
        } else {
          if (epi_tid == 0) {
            const int old = atomicAdd(&p.counters[tile_id], 1);
            const int last = (old == sg.n_contrib - 1) ? 1 : 0;
            if (last) p.counters[tile_id] = 0;    // leave the counter clean for the next launch
            *last_flag = last;
          }
          named_bar_sync(1, kEpiThreads);
          const bool is_last = *last_flag != 0;
          named_bar_sync(1, kEpiThreads);
          if (is_last) {
            __threadfence();
            const float* ws0 = p.workspace + static_cast<size_t>(tile_id) * p.splits * (BM * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += C::CW) {
              float f[C::CW];
#pragma unroll
              for (int e = 0; e < C::CW; ++e) f[e] = 0.f;
              for (int sp = 0; sp < sg.n_contrib; ++sp) {
                const uint4* src = reinterpret_cast<const uint4*>(ws0 + static_cast<size_t>(sp) * (BM * BN)) + (c0 / 4) * BM + row;
#pragma unroll
                for (int e = 0; e < C::CW / 4; ++e) {
                  const uint4 q4 = __ldcg(src + e * BM);
                  f[4 * e] += __uint_as_float(q4.x);
                  f[4 * e + 1] += __uint_as_float(q4.y);
                  f[4 * e + 2] += __uint_as_float(q4.z);
                  f[4 * e + 3] += __uint_as_float(q4.w);
                }
              }
              store_chunk(sg, f, c0);
            }
          }
        }
      }
    }

    // ---- stream-K: cooperative reduction of the tiles this CTA shares with its neighbours.  Every
    // contributor of a tile sums a different subset of the tile's column chunks over all partials
    // (in slot order: deterministic), so the fix-up work per CTA is one tile's worth of reads no
    // matter how many CTAs share the tile.
    for (int pi = 0; pi < n_pending && !*abort_flag; ++pi) {
      const Seg ps = pending[pi];
      if (epi_tid == 0) {
        const uint64_t t0 = global_timer_ns();
        uint32_t spins = 0;
        int ok = 1;
        while (*reinterpret_cast<volatile int*>(&p.counters[ps.tile_id]) < ps.n_contrib) {
          if ((++spins & 0xff) == 0 && global_timer_ns() - t0 > kWaitLimitNs) {
            report(p.status, kTimeoutTmemFull, ps.tile_id, 100 + ps.slot);
            *abort_flag = 1;
            ok = 0;
            break;
          }
        }
        *last_flag = ok;
        __threadfence();
      }
      named_bar_sync(1, kEpiThreads);
      const bool ok = *last_flag != 0;
      named_bar_sync(1, kEpiThreads);
      if (epi_tid == 0) stamp(9 + 2 * pi);
      if (ok) {
        const float* ws0 = p.workspace + static_cast<size_t>(ps.tile_id) * p.splits * (BM * BN);
#pragma unroll 1
        for (int c0 = ps.slot * C::CW; c0 < BN; c0 += ps.n_contrib * C::CW) {
          float f[C::CW];
#pragma unroll
          for (int e = 0; e < C::CW; ++e) f[e] = 0.f;
          int sp = 0;
          for (; sp + 1 < ps.n_contrib; sp += 2) {      // two partials in flight per thread
            const uint4* s0 = reinterpret_cast<const uint4*>(ws0 + static_cast<size_t>(sp) * (BM * BN)) + (c0 / 4) * BM + row;
            const uint4* s1 = s0 + (BM * BN) / 4;
            uint4 a4[C::CW / 4], b4[C::CW / 4];
#pragma unroll
            for (int e = 0; e < C::CW / 4; ++e) {
              a4[e] = __ldcg(s0 + e * BM);
              b4[e] = __ldcg(s1 + e * BM);
            }
#pragma unroll
            for (int e = 0; e < C::CW / 4; ++e) {
              f[4 * e] += __uint_as_float(a4[e].x);
              f[4 * e + 1] += __uint_as_float(a4[e].y);
              f[4 * e + 2] += __uint_as_float(a4[e].z);
              f[4 * e + 3] += __uint_as_float(a4[e].w);
              f[4 * e] += __uint_as_float(b4[e].x);
              f[4 * e + 1] += __uint_as_float(b4[e].y);
              f[4 * e + 2] += __uint_as_float(b4[e].z);
              f[4 * e + 3] += __uint_as_float(b4[e].w);
            }
          }
          if (sp < ps.n_contrib) {
            const uint4* s0 = reinterpret_cast<const uint4*>(ws0 + static_cast<size_t>(sp) * (BM * BN)) + (c0 / 4) * BM + row;
#pragma unroll
            for (int e = 0; e < C::CW / 4; ++e) {
              const uint4 q4 = __ldcg(s0 + e * BM);
              f[4 * e] += __uint_as_float(q4.x);
              f[4 * e + 1] += __uint_as_float(q4.y);
              f[4 * e + 2] += __uint_as_float(q4.z);
              f[4 * e + 3] += __uint_as_float(q4.w);
            }
          }
          store_chunk(ps, f, c0);
        }
      }
      // the contributor that finishes last leaves both counters clean for the next launch
      named_bar_sync(1, kEpiThreads);
      if (epi_tid == 0) stamp(10 + 2 * pi);
      if (epi_tid == 0) {
        const int old = atomicAdd(&p.counters[kDoneCounterOffset + ps.tile_id], 1);
        if (old == ps.n_contrib - 1) {
          p.counters[kDoneCounterOffset + ps.tile_id] = 0;
          p.counters[ps.tile_id] = 0;
        }
      }
    }
  }

  // ------------------------------------------------------------------ fused tail
  // Reduce-scatter arrival -> sum of the `world` partial slices + residual -> RMSNorm -> all-gather by peer
  // stores, done by the warps of this same launch as their CTA runs out of GEMM work.  One warp owns one row
  // at a time (rows are handed out by an atomic counter per chunk): pass 1 sums the slices and the residual,
  // keeps the row in the now idle operand ring of shared memory and accumulates the sum of squares; pass 2
  // normalises and pushes.  Nothing in here is a CTA-wide barrier, so the six warps of a CTA work on six rows
  // independently.  Cross-GPU ordering is by epoch-valued flags (bounded waits); no wait depends on a CTA of
  // this GPU that could itself be waiting.
  if constexpr (FUSE == 1) {
    const int tid = threadIdx.x;
    __syncthreads();                 // the epilogue's peer stores are issued, every role is done with the operand ring
    if (tid == 0 && !p.per_tile) {
      // small batches: the CTA that finishes last tells every owner that all of this rank's rows are out
      fence_acq_rel_sys();
      const int old = atomicAdd(&p.tail_ctrs[kCtrDone], 1);
      if (old == static_cast<int>(gridDim.x) - 1) {
        fence_acq_rel_sys();
        for (int o = 0; o < p.rs_world; ++o)
          for (int j = 0; j < p.nchunks; ++j) st_release_sys(p.flag_peer[o] + kRsFlag + j * 8 + p.rs_rank, epoch);
      }
    }
    const int nvec = p.N >> 3;
    const uint4* wv = reinterpret_cast<const uint4*>(p.norm_w);
    const uint4* ybase = reinterpret_cast<const uint4*>(p.rs_peer[p.rs_rank]);
    const uint32_t* my_flags = p.flag_peer[p.rs_rank];
    const int slice0 = p.rs_rank * p.rs_rows_per;
    const int slice_rows = max(0, min(p.M, slice0 + p.rs_rows_per) - slice0);
    // sum of the `world` slices (+ residual, which is updated in place) of 8 consecutive values of one row
    auto reduce8 = [&](const uint4 (&part)[8], int local, size_t gbase, int idx, float (&v)[8]) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
#pragma unroll
      for (int sl = 0; sl < 8; ++sl) {
        if (sl < p.rs_world) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&part[sl]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t = __bfloat1622float2(h[e]);
            v[2 * e] += t.x;
            v[2 * e + 1] += t.y;
          }
        }
      }
      if (p.residual != nullptr) {
        uint4* rv = reinterpret_cast<uint4*>(p.residual) + gbase + idx;
        const uint4 r4 = *rv;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r4);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(h[e]);
          v[2 * e] += t.x;
          v[2 * e + 1] += t.y;
        }
        // the residual stream is bf16: normalise what the next layer will read back
        const uint4 packed = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]),
                                        pack_bf16(v[6], v[7]));
        *rv = packed;
        const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 t = __bfloat1622float2(hp[e]);
          v[2 * e] = t.x;
          v[2 * e + 1] = t.y;
        }
      }
    };
    auto load_parts = [&](uint4 (&part)[8], int local, int idx) {
#pragma unroll
      for (int sl = 0; sl < 8; ++sl)
        if (sl < p.rs_world) part[sl] = __ldcg(ybase + (static_cast<size_t>(sl) * p.rs_rows_per + local) * nvec + idx);
    };
    auto push8 = [&](const float (&v)[8], float inv, size_t gbase, int idx) {
      const uint4 w4 = wv[idx];
      const __nv_bfloat162* hw = reinterpret_cast<const __nv_bfloat162*>(&w4);
      const float g = p.gemma ? 1.f : 0.f;
      float o8[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = __bfloat1622float2(hw[e]);
        o8[2 * e] = v[2 * e] * inv * (t.x + g);
        o8[2 * e + 1] = v[2 * e + 1] * inv * (t.y + g);
      }
      const uint4 out4 = make_uint4(pack_bf16(o8[0], o8[1]), pack_bf16(o8[2], o8[3]), pack_bf16(o8[4], o8[5]),
                                    pack_bf16(o8[6], o8[7]));
      if (p.ag_mc != nullptr) {
        multimem_st_v4(reinterpret_cast<uint4*>(p.ag_mc) + gbase + idx, out4);
      } else {
#pragma unroll
        for (int d = 0; d < 8; ++d)
          if (d < p.rs_world) reinterpret_cast<uint4*>(p.ag_peer[d])[gbase + idx] = out4;
      }
    };
    // a row of chunk j has been pushed everywhere: count it; the last row of the chunk tells every rank
    auto row_done = [&](int j, int nrows) {
      fence_acq_rel_sys();
      const int old = atomicAdd(&p.tail_ctrs[kCtrRowsDone + j], 1);
      if (old == nrows - 1) {
        fence_acq_rel_sys();
        for (int d = 0; d < p.rs_world; ++d) st_release_sys(p.flag_peer[d] + kAgFlag + p.rs_rank * kMaxChunks + j, epoch);
      }
    };

    if (slice_rows <= 2 * static_cast<int>(gridDim.x) && nvec <= 4 * kNumThreads) {
      // ---- small slices: one CTA per row (two at most), every load of the row in flight at once
      __shared__ float s_red[2][kNumThreads / 32];
      __shared__ int s_ok;
      for (int lr_all = blockIdx.x, pass = 0; lr_all < slice_rows && !*abort_flag; lr_all += gridDim.x, ++pass) {
        const int j = lr_all / kChunkRows;
        const int row = slice0 + lr_all;
        const int c0 = slice0 + j * kChunkRows;
        const int nrows = min(min(c0 + kChunkRows, slice0 + p.rs_rows_per), p.M) - c0;
        if (tid == 0) s_ok = 1;
        __syncthreads();
        if (tid < p.rs_world && !wait_flag_ge(my_flags + kRsFlag + j * 8 + tid, epoch)) {
          report(p.status, kTimeoutPeerFlag, tid, 10);
          s_ok = 0;
        }
        __syncthreads();
        if (s_ok) {
          const size_t gbase = static_cast<size_t>(row) * nvec;
          float vals[4][8];
          float ss = 0.f;
          {
            uint4 part[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (tid + i * kNumThreads < nvec) load_parts(part[i], lr_all, tid + i * kNumThreads);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int idx = tid + i * kNumThreads;
              if (idx < nvec) {
                reduce8(part[i], lr_all, gbase, idx, vals[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += vals[i][e] * vals[i][e];
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (lane == 0) s_red[pass & 1][warp] = ss;
          __syncthreads();
          float tot = 0.f;
#pragma unroll
          for (int wdx = 0; wdx < kNumThreads / 32; ++wdx) tot += s_red[pass & 1][wdx];
          const float inv = rsqrtf(tot / p.N + p.eps);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * kNumThreads;
            if (idx < nvec) push8(vals[i], inv, gbase, idx);
          }
          __syncthreads();
          if (tid == 0) row_done(j, nrows);
        } else {
          *abort_flag = 1;
        }
      }
    } else {
      // ---- prefill-sized slices: one warp per row (rows handed out by an atomic counter per chunk), the row
      // kept in the now idle operand ring between the two passes; no CTA-wide barrier, so the warps of a CTA
      // work on different rows independently
      constexpr int kRingBytes = C::kStages * C::kStageBytes;
      const int tail_warps = min(kNumThreads / 32, kRingBytes / (p.N * 4));
      float* stash = reinterpret_cast<float*>(stage_base) + static_cast<size_t>(warp) * p.N;
      if (warp < tail_warps) {
        for (int j = 0; j < p.nchunks && !*abort_flag; ++j) {
          const int c0 = slice0 + j * kChunkRows;
          const int nrows = min(min(c0 + kChunkRows, slice0 + p.rs_rows_per), p.M) - c0;
          if (nrows <= 0) break;
          bool waited = false;
          for (;;) {
            int lr = 0;
            if (lane == 0) lr = atomicAdd(&p.tail_ctrs[kCtrNextRow + j], 1);
            lr = __shfl_sync(0xffffffffu, lr, 0);
            if (lr >= nrows) break;
            if (!waited) {
              int good = 1;
              if (lane < p.rs_world && !wait_flag_ge(my_flags + kRsFlag + j * 8 + lane, epoch)) {
                report(p.status, kTimeoutPeerFlag, lane, 10);
                good = 0;
              }
              good = __all_sync(0xffffffffu, good);
              waited = true;
              if (!good) {
                *abort_flag = 1;
                break;
              }
            }
            const int row = c0 + lr;
            const int local = row - slice0;
            const size_t gbase = static_cast<size_t>(row) * nvec;
            float ss = 0.f;
            // two vectors per lane and step: their loads are all issued before the first use
            for (int idx = lane; idx < nvec; idx += 64) {
              uint4 pa[8], pb[8];
              const bool two = idx + 32 < nvec;
              load_parts(pa, local, idx);
              if (two) load_parts(pb, local, idx + 32);
              float v[8];
              reduce8(pa, local, gbase, idx, v);
#pragma unroll
              for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
              reinterpret_cast<float4*>(stash)[2 * idx] = make_float4(v[0], v[1], v[2], v[3]);
              reinterpret_cast<float4*>(stash)[2 * idx + 1] = make_float4(v[4], v[5], v[6], v[7]);
              if (two) {
                reduce8(pb, local, gbase, idx + 32, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
                reinterpret_cast<float4*>(stash)[2 * (idx + 32)] = make_float4(v[0], v[1], v[2], v[3]);
                reinterpret_cast<float4*>(stash)[2 * (idx + 32) + 1] = make_float4(v[4], v[5], v[6], v[7]);
              }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = rsqrtf(ss / p.N + p.eps);
            for (int idx = lane; idx < nvec; idx += 32) {
              const float4 a4 = reinterpret_cast<const float4*>(stash)[2 * idx];
              const float4 b4 = reinterpret_cast<const float4*>(stash)[2 * idx + 1];
              const float v[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
              push8(v, inv, gbase, idx);
            }
            __syncwarp();
            if (lane == 0) row_done(j, nrows);
          }
        }
      }
    }
    // without a flag-aware consumer the launch only ends once every rank's rows have landed here
    if (!p.defer && blockIdx.x == 0 && !*abort_flag) {
      for (int id = tid; id < p.rs_world * p.nchunks; id += kNumThreads) {
        const int o = id / p.nchunks, j = id - o * p.nchunks;
        if (o * p.rs_rows_per + j * kChunkRows < p.M) {
          if (!wait_flag_ge(my_flags + kAgFlag + o * kMaxChunks + j, epoch)) report(p.status, kTimeoutPeerFlag, o, 30);
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      *last_flag = 0;
      const int old = atomicAdd(&p.tail_ctrs[kCtrExit], 1);
      if (old == static_cast<int>(gridDim.x) - 1) {
        *last_flag = 1;
      }
    }
    __syncthreads();
    if (*last_flag) {
      // last CTA out: leave the counters clean and publish the epoch for the next launch / the consumer
      for (int i = tid; i < kTailCtrInts; i += kNumThreads) p.tail_ctrs[i] = 0;
      __threadfence();
      __syncthreads();
      if (tid == 0) *reinterpret_cast<volatile uint32_t*>(p.seq) = epoch;
    }
  }

  // ------------------------------------------------------------------ teardown
  if (threadIdx.x == 64) stamp(5);
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) stamp(6);
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA's smem is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
    if (lane == 0) stamp(7);
  }
}

template <int BN, int MODE, bool FP8 = false, int FUSE = 0>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const Params& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN>;
  auto* kern = gemm_bf16_kernel<BN, MODE, FP8, FUSE>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  return launch_pdl(kern, dim3(grid), dim3(kNumThreads), C::kSmemBytes, stream, ta, tb, p);
}

inline int pick_bn_tokens(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

}  // namespace
}  // namespace sglb

extern "C" {

// Bytes of fp32 workspace / number of int counters the launcher may use for given shapes.
// (Upper bounds; callers allocate once for their largest decode shape.)
size_t sglb_gemm_workspace_bytes(int M, int N, int K) {
  if (M > 256) return 0;
  const int bn = sglb::pick_bn_tokens(M);
  const size_t tiles = (N + 127) / 128;
  return tiles * 16 /*max splits*/ * 128 * bn * sizeof(float);
}

int sglb_gemm_max_counters(int N) { return (N + 127) / 128 + 8; }

// out[M,N] = x[M,K] . w[N,K]^T + bias.  All bf16, row-major, K and N multiples of 8,
// pointers 16-byte aligned.  `workspace`/`counters` are only touched when M <= 256 and the
// launcher decides to split K; `counters` must be zero on entry (the kernel restores zeros).
// force_mode: -1 auto, 0 tokens-on-M, 1 weights-on-M.  force_splits: 0 auto.
struct SglbFusedHost {
  int kind;                    // 1: GEMM -> reduce-scatter -> residual + RMSNorm -> all-gather; 2: all-gather -> GEMM
  void* const* gathered;       // [world] every rank's buffer of normalised activations
  void* gathered_mc;           // multicast address of that buffer or null
  void* const* flags;          // [world] every rank's flag block
  void* seq;                   // device u32: call counter of the fused context
  void* ctrs;                  // device ints: local tail counters
  void* residual;
  const void* norm_w;
  float eps;
  int gemma, defer, world, rank;
};
int sglb_gemm_bf16_impl(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, int* counters, int force_mode, int force_splits,
                        void* const* rs_peers, int rs_world, int rs_rank, cudaStream_t stream,
                        const float* scale_x = nullptr, const float* scale_w = nullptr,
                        const SglbFusedHost* fused = nullptr);

// out[M,N] (bf16) = (x_q[M,K] . w_q[N,K]^T) * scale_x[M] * scale_w[N] + bias with e4m3 operands
// (per-token activation scales, per-output-channel weight scales; K a multiple of 16).
int sglb_gemm_fp8(const void* x_q, const void* w_q, const float* scale_x, const float* scale_w, const void* bias,
                  void* out, int M, int N, int K, void* workspace, size_t workspace_bytes, int* counters,
                  cudaStream_t stream) {
  if (scale_x == nullptr || scale_w == nullptr || K % 16 != 0) return -sglb::kBadArgument;
  return sglb_gemm_bf16_impl(x_q, w_q, bias, out, M, N, K, workspace, workspace_bytes, counters, -1, 0, nullptr, 0, 0,
                             stream, scale_x, scale_w);
}

int sglb_gemm_bf16(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, void* workspace,
                   size_t workspace_bytes, int* counters, int force_mode, int force_splits, cudaStream_t stream) {
  return sglb_gemm_bf16_impl(x, w, bias, out, M, N, K, workspace, workspace_bytes, counters, force_mode, force_splits,
                             nullptr, 0, 0, stream);
}

// Row-parallel GEMM whose epilogue performs the reduce-scatter sends: `rs_peers[r]` is rank r's
// receive buffer ([world][ceil(M / world)][N] bf16, symmetric memory).  A cross-rank barrier must
// separate this launch from the kernel that reduces the received slices (sglb_ar_residual_rmsnorm
// with rs_mode = 1 starts with one).
int sglb_gemm_bf16_rs(const void* x, const void* w, int M, int N, int K, void* workspace, size_t workspace_bytes,
                      int* counters, void* const* rs_peers, int rs_world, int rs_rank, cudaStream_t stream) {
  if (rs_world < 1 || rs_world > 8 || rs_peers == nullptr) return -sglb::kBadArgument;
  return sglb_gemm_bf16_impl(x, w, nullptr, nullptr, M, N, K, workspace, workspace_bytes, counters, -1, 0, rs_peers,
                             rs_world, rs_rank, stream);
}

static unsigned long long* g_debug_stamps = nullptr;

// Decode-mode loads carry L2 eviction hints (weights evict-first, token tile evict-last): measured
// 278 -> 248 us for the four GEMMs of a Qwen3-32B layer at 128 tokens.  SGLB_GEMM_L2_HINTS=0 turns them off.
static int gemm_l2_hints() {
  static const int v = [] { const char* e = getenv("SGLB_GEMM_L2_HINTS"); return e ? atoi(e) : 1; }();
  return v;
}
// Profiling aid: when set, CTA 0 of every dense GEMM launch writes globaltimer stamps (kernel start,
// after set-up barrier, producer done, MMA issue done, first accumulator ready, epilogue done,
// teardown barrier, TMEM freed) into this device buffer of 16 u64.
void sglb_gemm_set_debug_stamps(void* dev_ptr) { g_debug_stamps = static_cast<unsigned long long*>(dev_ptr); }

int sglb_gemm_bf16_impl(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                        void* workspace, size_t workspace_bytes, int* counters, int force_mode, int force_splits,
                        void* const* rs_peers, int rs_world, int rs_rank, cudaStream_t stream,
                        const float* scale_x, const float* scale_w, const SglbFusedHost* fused) {
  using namespace sglb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (N % 8)) return -kBadArgument;
  const bool fp8 = scale_x != nullptr;
  const int eb = fp8 ? 1 : 2;                          // operand element bytes
  const int bke = fp8 ? 2 * BK : BK;                   // elements per 128-byte K block
  const int kb_total = (K + bke - 1) / bke;
  const int sms = sm_count();
  // Decode-sized batches: both operand assignments stream the weights once; they differ in how many
  // activation bytes each K block re-reads from L2 per weight byte (tokens-on-M with 256 weight rows
  // per tile: M*128 B per 32 KiB of weights; weights-on-M: BN*128 B per 16 KiB).
  static const int decode_mode = [] {
    const char* e = getenv("SGLB_DECODE_GEMM_MODE");
    return e ? atoi(e) : 1;
  }();
  int mode = force_mode >= 0 ? force_mode : (M <= 256 ? decode_mode : 0);
  if (mode == 1 && M > 256) mode = 0;

  Params p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.workspace = static_cast<float*>(workspace);
  p.counters = counters;
  p.status = device_status();
  p.M = M;
  p.N = N;
  p.K = K;
  p.kb_total = kb_total;
  p.splits = 1;
  p.debug_stamps = g_debug_stamps;
  p.l2_hints = gemm_l2_hints();
  p.scale_x = scale_x;
  p.scale_w = scale_w;
  if (rs_world > 0) {
    p.rs_world = rs_world;
    p.rs_rank = rs_rank;
    p.rs_rows_per = (M + rs_world - 1) / rs_world;
    for (int r = 0; r < rs_world; ++r) p.rs_peer[r] = static_cast<__nv_bfloat16*>(rs_peers[r]);
  }
  const int fuse = fused != nullptr ? fused->kind : 0;
  if (fuse != 0) {
    if (fp8 || fused->world < 1 || fused->world > 8 || M > kMaxChunks * kChunkRows) return -kBadArgument;
    int rows_per = 0, nchunks = 0, per_tile = 0;
    fused_layout(M, fused->world, &rows_per, &nchunks, &per_tile);
    if (fuse == 1) {
      if (rs_world != fused->world || N > 6 * kNumThreads * 8) return -kBadArgument;
      p.rs_rows_per = rows_per;
      p.nchunks = nchunks;
      p.per_tile = per_tile;
      for (int r = 0; r < fused->world; ++r) {
        p.ag_peer[r] = static_cast<__nv_bfloat16*>(fused->gathered[r]);
        p.flag_peer[r] = static_cast<uint32_t*>(fused->flags[r]);
      }
      p.ag_mc = static_cast<__nv_bfloat16*>(fused->gathered_mc);
      p.residual = static_cast<__nv_bfloat16*>(fused->residual);
      p.norm_w = static_cast<const __nv_bfloat16*>(fused->norm_w);
      p.seq = static_cast<uint32_t*>(fused->seq);
      p.tail_ctrs = static_cast<int*>(fused->ctrs);
      p.eps = fused->eps;
      p.gemma = fused->gemma;
      p.defer = fused->defer;
    } else {
      p.ag_flags = static_cast<const uint32_t*>(fused->flags[fused->rank]);
      p.ag_seq = static_cast<const uint32_t*>(fused->seq);
      p.ag_world = fused->world;
      p.ag_rows_per = rows_per;
      p.ag_nchunks = nchunks;
    }
  }

  CUtensorMap ta, tb;
  cudaError_t err;
  if (mode == 0) {
    const int bn = (N >= 256 && (static_cast<long long>((M + 127) / 128) * ((N + 255) / 256) >= sms || N % 256 == 0))
                       ? 256 : 128;
    p.tiles_a = (M + BM - 1) / BM;
    p.tiles_b = (N + bn - 1) / bn;
    if (!encode_tmap_2d(&ta, x, K, M, static_cast<uint64_t>(K) * eb, bke, BM, eb)) return -100;
    if (!encode_tmap_2d(&tb, w, K, N, static_cast<uint64_t>(K) * eb, bke, bn, eb)) return -101;
    int grid = min(p.tiles_a * p.tiles_b, sms);
    if (M <= 256 && force_splits <= 0 && workspace != nullptr && counters != nullptr) {
      // decode-sized: stream-K so that every SM streams the same number of weight bytes
      const int tiles = p.tiles_a * p.tiles_b;
      const int total = tiles * kb_total;
      int upc = (total + sms - 1) / sms;
      if (upc < 8) upc = min(8, kb_total);
      const int max_contrib = (kb_total + upc - 1) / upc + 1;
      const size_t need = static_cast<size_t>(tiles) * max_contrib * BM * bn * sizeof(float);
      if (need <= workspace_bytes && tiles <= kDoneCounterOffset) {
        p.units_per_cta = upc;
        p.total_units = total;
        p.splits = max_contrib;
        grid = (total + upc - 1) / upc;
      }
    }
    if (fp8) err = bn == 256 ? launch<256, 0, true>(ta, tb, p, grid, stream) : launch<128, 0, true>(ta, tb, p, grid, stream);
    else if (fuse == 1) err = bn == 256 ? launch<256, 0, false, 1>(ta, tb, p, grid, stream) : launch<128, 0, false, 1>(ta, tb, p, grid, stream);
    else if (fuse == 2) err = bn == 256 ? launch<256, 0, false, 2>(ta, tb, p, grid, stream) : launch<128, 0, false, 2>(ta, tb, p, grid, stream);
    else err = bn == 256 ? launch<256, 0>(ta, tb, p, grid, stream) : launch<128, 0>(ta, tb, p, grid, stream);
  } else {
    const int bn = pick_bn_tokens(M);
    p.tiles_a = (N + BM - 1) / BM;
    p.tiles_b = 1;
    int splits = force_splits > 0 ? force_splits : 1;
    int grid = 0;
    if (force_splits <= 0 && workspace != nullptr && counters != nullptr) {
      // stream-K: equal consecutive K-block ranges per CTA.  A range is kept long enough that the
      // fp32 fix-up traffic of a shared tile (2 * 128 * bn * 4 bytes per contributor) stays small
      // next to the weight bytes the contributor streams (16 KiB per K block).
      const int total = p.tiles_a * kb_total;
      const int min_upc = bn >= 128 ? 16 : (bn >= 64 ? 12 : 8);
      int upc = (total + sms - 1) / sms;
      if (upc < min_upc) upc = min(min_upc, kb_total);   // never force several tiles onto one CTA
      const int max_contrib = (kb_total + upc - 1) / upc + 1;
      const size_t need = static_cast<size_t>(p.tiles_a) * max_contrib * BM * bn * sizeof(float);
      if (need <= workspace_bytes && p.tiles_a <= kDoneCounterOffset) {
        p.units_per_cta = upc;
        p.total_units = total;
        splits = max_contrib;               // workspace slots per tile
        grid = (total + upc - 1) / upc;
      }
    }
    if (p.units_per_cta == 0) {
      if (splits > 1) {
        const size_t need = static_cast<size_t>(p.tiles_a) * splits * BM * bn * sizeof(float);
        if (workspace == nullptr || counters == nullptr || need > workspace_bytes) splits = 1;
      }
      // every split must own at least one K block
      while (splits > 1 && (kb_total + splits - 1) / splits * (splits - 1) >= kb_total) --splits;
      grid = min(p.tiles_a * splits, sms);
    }
    p.splits = splits;
    if (!encode_tmap_2d(&ta, w, K, N, static_cast<uint64_t>(K) * eb, bke, BM, eb)) return -100;
    if (!encode_tmap_2d(&tb, x, K, M, static_cast<uint64_t>(K) * eb, bke, bn, eb)) return -101;
    if (fp8) {
      switch (bn) {
        case 16: err = launch<16, 1, true>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1, true>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1, true>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1, true>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1, true>(ta, tb, p, grid, stream); break;
      }
    } else if (fuse == 1) {
      switch (bn) {
        case 16: err = launch<16, 1, false, 1>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1, false, 1>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1, false, 1>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1, false, 1>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1, false, 1>(ta, tb, p, grid, stream); break;
      }
    } else if (fuse == 2) {
      switch (bn) {
        case 16: err = launch<16, 1, false, 2>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1, false, 2>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1, false, 2>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1, false, 2>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1, false, 2>(ta, tb, p, grid, stream); break;
      }
    } else {
      switch (bn) {
        case 16: err = launch<16, 1>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1>(ta, tb, p, grid, stream); break;
      }
    }
  }
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}

// Sizes of the fused context's flag block (u32 words, symmetric memory) and local counter block (ints).
int sglb_fused_flag_words() { return sglb::kFlagWords; }
int sglb_fused_ctr_ints() { return sglb::kTailCtrInts; }
int sglb_fused_max_tokens() { return sglb::kMaxChunks * sglb::kChunkRows; }
// rows_per / nchunks / per_tile of the ownership layout for M tokens over `world` ranks
void sglb_fused_layout(int M, int world, int* out3) { sglb::fused_layout(M, world, out3, out3 + 1, out3 + 2); }

// One launch for the row-parallel half of a decoder layer under tensor parallelism:
//   partial = x[M, K] . w[N, K]^T  (this rank's K shard)
//   -> reduce-scatter over token rows (the epilogue stores each row into its owner's receive buffer
//      `ypart_ptrs[owner]`, laid out [src rank][rows_per][N], over NVLink peer mappings)
//   -> owner: sum of the `world` slices + residual (updated in place for the owned rows) -> RMSNorm
//   -> all-gather: normalised rows stored into every rank's `gathered_ptrs[r]` ([M, N]; `gathered_mc` non-null
//      selects one multimem.st through the NVSwitch multicast mapping instead of `world` peer stores).
// `defer` = 1 returns without waiting for the peers' rows: the consumer must be sglb_gemm_bf16_ag (which waits
// per chunk) on the same stream.  `seq` (one u32) and `ctrs` (sglb_fused_ctr_ints ints) are device memory owned
// by the fused context, zero at creation; `flag_ptrs` are the ranks' flag blocks (sglb_fused_flag_words u32,
// zero at creation, symmetric memory).  Every rank must issue the same sequence of fused launches.
int sglb_gemm_rs_norm_ag(const void* x, const void* w, int M, int N, int K, void* workspace, size_t workspace_bytes,
                         int* counters, void* const* ypart_ptrs, void* const* gathered_ptrs, void* gathered_mc,
                         void* const* flag_ptrs, void* seq, void* ctrs, void* residual, const void* norm_w, float eps,
                         int gemma, int defer, int world, int rank, cudaStream_t stream) {
  if (world < 1 || world > 8 || ypart_ptrs == nullptr || gathered_ptrs == nullptr || flag_ptrs == nullptr ||
      seq == nullptr || ctrs == nullptr || norm_w == nullptr)
    return -sglb::kBadArgument;
  SglbFusedHost f{1, gathered_ptrs, gathered_mc, flag_ptrs, seq, ctrs, residual, norm_w, eps, gemma, defer, world, rank};
  return sglb_gemm_bf16_impl(x, w, nullptr, nullptr, M, N, K, workspace, workspace_bytes, counters, -1, 0, ypart_ptrs,
                             world, rank, stream, nullptr, nullptr, &f);
}

// Column-parallel GEMM whose token operand `x` is this rank's all-gather buffer of a deferred
// sglb_gemm_rs_norm_ag launch with the same M and world: the TMA producer waits for each chunk's arrival flag
// before its first load of it (plain loads of this GPU's own memory; the peers wrote it with stores).
int sglb_gemm_bf16_ag(const void* x, const void* w, const void* bias, void* out, int M, int N, int K, void* workspace,
                      size_t workspace_bytes, int* counters, void* const* flag_ptrs, void* seq, int world, int rank,
                      cudaStream_t stream) {
  if (world < 1 || world > 8 || flag_ptrs == nullptr || seq == nullptr) return -sglb::kBadArgument;
  SglbFusedHost f{2, nullptr, nullptr, flag_ptrs, seq, nullptr, nullptr, nullptr, 0.f, 0, 0, world, rank};
  return sglb_gemm_bf16_impl(x, w, bias, out, M, N, K, workspace, workspace_bytes, counters, -1, 0, nullptr, 0, 0, stream,
                             nullptr, nullptr, &f);
}
}

namespace sglb {
namespace {
__global__ void fused_wait_gather_kernel(const uint32_t* flags, const uint32_t* seq, int M, int world, int rows_per,
                                         int nchunks, Status* st) {
  const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(seq);
  for (int id = threadIdx.x; id < world * nchunks; id += blockDim.x) {
    const int o = id / nchunks, j = id - o * nchunks;
    if (o * rows_per + j * kChunkRows < M && !wait_flag_ge(flags + kAgFlag + o * kMaxChunks + j, epoch))
      report(st, kTimeoutPeerFlag, o, 40);
  }
}
}  // namespace
}  // namespace sglb

// Blocks the stream until every rank's rows of the last deferred sglb_gemm_rs_norm_ag launch (M tokens) have
// landed in this rank's all-gather buffer: for consumers that are not sglb_gemm_bf16_ag.
extern "C" int sglb_fused_wait_gather(const void* flags_local, const void* seq, int M, int world, cudaStream_t stream) {
  using namespace sglb;
  if (world < 1 || world > 8 || M <= 0 || M > kMaxChunks * kChunkRows) return -kBadArgument;
  int rows_per = 0, nchunks = 0, per_tile = 0;
  fused_layout(M, world, &rows_per, &nchunks, &per_tile);
  fused_wait_gather_kernel<<<1, 128, 0, stream>>>(static_cast<const uint32_t*>(flags_local),
                                                  static_cast<const uint32_t*>(seq), M, world, rows_per, nchunks,
                                                  device_status());
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry point (declared in gemm_noalloc.h).
//
// Same decode-shaped GEMM (weights on the MMA M dimension, K split over CTAs), but every byte of
// scratch it needs — split-K partial tiles, tile counters and its status word — lives in the
// file-scope device array below, so the call performs no cudaMalloc / cudaFree and calls no
// allocating library routine.  The array is part of the library image: each GPU that loads the
// library carries kNoAllocScratchBytes of it until the process exits.
// ---------------------------------------------------------------------------------------------
namespace sglb {
namespace {

constexpr size_t kNoAllocHeaderBytes = 8192;                       // status word + tile counters
constexpr size_t kNoAllocCounterOffset = 256;                      // counters start here
constexpr int kNoAllocMaxCounters = (kNoAllocHeaderBytes - kNoAllocCounterOffset) / sizeof(int);
constexpr size_t kNoAllocWorkspaceBytes = size_t(8) << 20;         // 8 MiB of fp32 partial tiles
constexpr size_t kNoAllocScratchBytes = kNoAllocHeaderBytes + kNoAllocWorkspaceBytes;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Host code may not use `g_noalloc_scratch` as a pointer: on the host that name is only a handle
// for the runtime.  The device address is looked up once per device, with that device current.
unsigned char* g_noalloc_dev_ptr[16] = {};
std::mutex g_noalloc_mu;
thread_local char g_noalloc_error[256] = "";

unsigned char* noalloc_scratch_ptr(int* rc) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 16) {
    *rc = e != cudaSuccess ? static_cast<int>(e) : -kBadArgument;
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_dev_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *rc = e != cudaSuccess ? static_cast<int>(e) : -kBadArgument;
      return nullptr;
    }
    g_noalloc_dev_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *rc = 0;
  return g_noalloc_dev_ptr[dev];
}

}  // namespace
}  // namespace sglb

extern "C" {

size_t sglb_gemm_bf16_noalloc_scratch_bytes() { return sglb::kNoAllocScratchBytes; }

const char* sglb_gemm_bf16_noalloc_last_error() { return sglb::g_noalloc_error; }

int sglb_gemm_bf16_noalloc(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                           int splits, cudaStream_t stream) {
  using namespace sglb;
  auto fail = [&](int code, const char* fmt, long long a = 0, long long b = 0) {
    snprintf(g_noalloc_error, sizeof(g_noalloc_error), fmt, a, b);
    return code;
  };
  g_noalloc_error[0] = 0;
  if (M <= 0 || N <= 0 || K <= 0) return fail(-kBadArgument, "M, N and K must be positive");
  if (M > 256) return fail(-kBadArgument, "M = %lld exceeds the 256-token limit of the allocation-free GEMM", M);
  if ((K % 8) || (N % 8)) return fail(-kBadArgument, "N and K must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(-kBadArgument, "x, w and out must be 16-byte aligned");
  const int kb_total = (K + BK - 1) / BK;
  const int bn = pick_bn_tokens(M);
  const int tiles = (N + BM - 1) / BM;
  const int sms = sm_count();
  if (splits <= 0) {
    splits = (sms + tiles - 1) / tiles;
    splits = min(splits, max(1, kb_total / 8));
    splits = min(splits, 16);
    // auto mode never asks for more scratch than the static array holds
    while (splits > 1 && static_cast<size_t>(tiles) * splits * BM * bn * sizeof(float) > kNoAllocWorkspaceBytes) --splits;
  }
  while (splits > 1 && (kb_total + splits - 1) / splits * (splits - 1) >= kb_total) --splits;
  const size_t need = splits > 1 ? static_cast<size_t>(tiles) * splits * BM * bn * sizeof(float) : 0;
  if (need > kNoAllocWorkspaceBytes)
    return fail(-kBadArgument, "split-K partials need %lld bytes but the static scratch holds %lld; lower `splits`",
                static_cast<long long>(need), static_cast<long long>(kNoAllocWorkspaceBytes));
  if (splits > 1 && tiles > kNoAllocMaxCounters)
    return fail(-kBadArgument, "N needs %lld tile counters but the static scratch holds %lld", tiles,
                kNoAllocMaxCounters);
  int rc = 0;
  unsigned char* scratch = noalloc_scratch_ptr(&rc);
  if (scratch == nullptr) return fail(rc, "cudaGetSymbolAddress failed for the static scratch (code %lld)", rc);
  // The array keeps whatever the previous call left: status word and counters must start at zero.
  cudaError_t e = cudaMemsetAsync(scratch, 0, kNoAllocHeaderBytes, stream);
  if (e != cudaSuccess) return fail(static_cast<int>(e), "cudaMemsetAsync failed (code %lld)", e);

  Params p{};
  p.l2_hints = gemm_l2_hints();
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = reinterpret_cast<Status*>(scratch);
  p.counters = reinterpret_cast<int*>(scratch + kNoAllocCounterOffset);
  p.workspace = reinterpret_cast<float*>(scratch + kNoAllocHeaderBytes);
  p.M = M;
  p.N = N;
  p.K = K;
  p.kb_total = kb_total;
  p.splits = splits;
  p.tiles_a = tiles;
  p.tiles_b = 1;
  CUtensorMap ta, tb;
  if (!encode_tmap_2d(&ta, w, K, N, static_cast<uint64_t>(K) * 2, BK, BM, 2)) return fail(-100, "tensor map (w) failed");
  if (!encode_tmap_2d(&tb, x, K, M, static_cast<uint64_t>(K) * 2, BK, bn, 2)) return fail(-101, "tensor map (x) failed");
  const int grid = min(tiles * splits, sms);
  switch (bn) {
    case 16: e = launch<16, 1>(ta, tb, p, grid, stream); break;
    case 32: e = launch<32, 1>(ta, tb, p, grid, stream); break;
    case 64: e = launch<64, 1>(ta, tb, p, grid, stream); break;
    case 128: e = launch<128, 1>(ta, tb, p, grid, stream); break;
    default: e = launch<256, 1>(ta, tb, p, grid, stream); break;
  }
  if (e != cudaSuccess) return fail(static_cast<int>(e), "kernel launch failed (code %lld)", e);
  return 0;
}

// Copies the entry point's status word (code, block, aux0, aux1) to the host with a blocking copy; the caller
// synchronises the stream it launched on first (see gemm_noalloc.h).
int sglb_gemm_bf16_noalloc_status(int* out4) {
  using namespace sglb;
  int rc = 0;
  unsigned char* scratch = noalloc_scratch_ptr(&rc);
  if (scratch == nullptr) return rc;
  Status h;
  cudaError_t e = cudaMemcpy(&h, scratch, sizeof(h), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (out4) {
    out4[0] = h.code;
    out4[1] = h.block;
    out4[2] = h.aux0;
    out4[3] = h.aux1;
  }
  return h.code;
}
}

// ---------------------------------------------------------------------------------------------
// Grouped GEMM for MoE experts: out[r, :] = x[r, :] . w[g(r)]^T for rows r sorted by group g.
//   x    [rows, K]  (rows = routed (token, expert) pairs, sorted by expert)
//   w    [groups, N, K]
//   out  [rows, N]
//   group_offsets [groups + 1] (device)
// rows <= 256: decode shape, weights on the MMA M dimension, stream-K over (group, weight tile, K);
// every group must then hold at most BN >= rows tokens, which `rows <= BN` guarantees.
// rows  > 256: prefill shape, (token tile, weight tile) pairs from the device-side tile list built
// by sglb_moe_align (tile_group / tile_row0 / num_token_tiles, at most rows/128 + groups tiles).
// The reference's counterpart is the Megablox grouped matmul
// (python/sgl_jax/srt/kernels/gmm/megablox_gmm_kernel/gmm.py:311).
// ---------------------------------------------------------------------------------------------
static int grouped_gemm_impl(const void* x, const void* w, void* out, const int* group_offsets, const int* tile_group,
                             const int* tile_row0, const int* num_token_tiles, int rows, int N, int K, int groups,
                             void* workspace, size_t workspace_bytes, int* counters, cudaStream_t stream,
                             const float* scale_x, const float* scale_w) {
  using namespace sglb;
  if (rows <= 0 || groups <= 0) return 0;
  if ((K % 8) || (N % 8)) return -kBadArgument;
  const bool fp8 = scale_x != nullptr;
  const int eb = fp8 ? 1 : 2;
  const int bke = fp8 ? 2 * BK : BK;
  if (fp8 && K % 16) return -kBadArgument;
  const int kb_total = (K + bke - 1) / bke;
  const int sms = sm_count();
  Params p{};
  p.l2_hints = gemm_l2_hints();
  p.scale_x = scale_x;
  p.scale_w = scale_w;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.workspace = static_cast<float*>(workspace);
  p.counters = counters;
  p.status = device_status();
  p.M = rows;
  p.N = N;
  p.K = K;
  p.kb_total = kb_total;
  p.splits = 1;
  p.group_offsets = group_offsets;
  p.groups = groups;
  CUtensorMap ta, tb;
  cudaError_t err;
  if (rows <= 256) {
    const int bn = pick_bn_tokens(rows);
    p.tiles_a = (N + BM - 1) / BM;        // weight tiles per group
    p.tiles_b = 1;
    const int total = groups * p.tiles_a * kb_total;
    const int min_upc = bn >= 128 ? 16 : (bn >= 64 ? 12 : 8);
    int upc = (total + sms - 1) / sms;
    if (upc < min_upc) upc = min(min_upc, kb_total > 0 ? kb_total : 1);
    int max_contrib = (kb_total + upc - 1) / upc + 1;
    size_t need = static_cast<size_t>(groups) * p.tiles_a * max_contrib * BM * bn * sizeof(float);
    if (need > workspace_bytes || groups * p.tiles_a > kDoneCounterOffset || workspace == nullptr || counters == nullptr) {
      // no room for shared tiles: whole tiles per CTA
      upc = kb_total * ((total / kb_total + sms - 1) / sms);
      max_contrib = 1;
    }
    p.units_per_cta = upc;
    p.total_units = total;
    p.splits = max_contrib;
    const int grid = (total + upc - 1) / upc;
    // weights [groups*N, K] on the A operand; when N is not a multiple of 128 the last tile of a
    // group reads rows of the next group, which are masked at the store (gn < N).
    if (!encode_tmap_2d(&ta, w, K, static_cast<uint64_t>(groups) * N, static_cast<uint64_t>(K) * eb, bke, BM, eb)) return -100;
    if (!encode_tmap_2d(&tb, x, K, rows, static_cast<uint64_t>(K) * eb, bke, bn, eb)) return -101;
    if (fp8) {
      switch (bn) {
        case 16: err = launch<16, 1, true>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1, true>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1, true>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1, true>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1, true>(ta, tb, p, grid, stream); break;
      }
    } else {
      switch (bn) {
        case 16: err = launch<16, 1>(ta, tb, p, grid, stream); break;
        case 32: err = launch<32, 1>(ta, tb, p, grid, stream); break;
        case 64: err = launch<64, 1>(ta, tb, p, grid, stream); break;
        case 128: err = launch<128, 1>(ta, tb, p, grid, stream); break;
        default: err = launch<256, 1>(ta, tb, p, grid, stream); break;
      }
    }
  } else {
    if (tile_group == nullptr || tile_row0 == nullptr || num_token_tiles == nullptr) return -kBadArgument;
    const int bn = (N % 256 == 0) ? 256 : 128;
    p.tile_group = tile_group;
    p.tile_row0 = tile_row0;
    p.num_token_tiles = num_token_tiles;
    p.tiles_a = rows / BM + groups;       // upper bound of token tiles
    p.tiles_b = (N + bn - 1) / bn;
    if (!encode_tmap_2d(&ta, x, K, rows, static_cast<uint64_t>(K) * eb, bke, BM, eb)) return -100;
    if (!encode_tmap_2d(&tb, w, K, static_cast<uint64_t>(groups) * N, static_cast<uint64_t>(K) * eb, bke, bn, eb)) return -101;
    const int grid = min(p.tiles_a * p.tiles_b, sms);
    if (fp8) err = bn == 256 ? launch<256, 0, true>(ta, tb, p, grid, stream) : launch<128, 0, true>(ta, tb, p, grid, stream);
    else err = bn == 256 ? launch<256, 0>(ta, tb, p, grid, stream) : launch<128, 0>(ta, tb, p, grid, stream);
  }
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}

extern "C" int sglb_grouped_gemm_bf16(const void* x, const void* w, void* out, const int* group_offsets,
                                       const int* tile_group, const int* tile_row0, const int* num_token_tiles,
                                       int rows, int N, int K, int groups, void* workspace, size_t workspace_bytes,
                                       int* counters, cudaStream_t stream) {
  return grouped_gemm_impl(x, w, out, group_offsets, tile_group, tile_row0, num_token_tiles, rows, N, K, groups,
                           workspace, workspace_bytes, counters, stream, nullptr, nullptr);
}

// e4m3 operands: `x_q [rows, K]` with per-row scales `scale_x [rows]`, `w_q [groups * N, K]` with per-row
// (= per expert output channel) scales `scale_w [groups * N]`; bf16 output.
extern "C" int sglb_grouped_gemm_fp8(const void* x_q, const void* w_q, const float* scale_x, const float* scale_w,
                                      void* out, const int* group_offsets, const int* tile_group, const int* tile_row0,
                                      const int* num_token_tiles, int rows, int N, int K, int groups, void* workspace,
                                      size_t workspace_bytes, int* counters, cudaStream_t stream) {
  if (scale_x == nullptr || scale_w == nullptr) return -sglb::kBadArgument;
  return grouped_gemm_impl(x_q, w_q, out, group_offsets, tile_group, tile_row0, num_token_tiles, rows, N, K, groups,
                           workspace, workspace_bytes, counters, stream, scale_x, scale_w);
}
