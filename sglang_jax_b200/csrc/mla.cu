// Absorbed multi-head latent attention, decode step (DeepSeek-V2/V3, Kimi-K2, GLM-5).
//
// Every head attends over the same latent cache rows  [pages, P, R + 64]  (R = kv_lora_rank = 512,
// 64 rotary lanes): logits = q_latent . c + q_pe . k_pe, output = softmax . c  (the caller applies
// W_UV).  This is multi-query attention with a 576-wide key and a 512-wide value that alias the same
// bytes, so one tile of 64 tokens (72 KB) streamed by TMA serves both products.
//
// One CTA handles 16 heads of one sequence and one KV split.  Its four consumer warps split the work
// along different axes in the two products: for S = Q K^T each warp owns 16 of the tile's 64 tokens
// (Q fragments come from shared memory, 36 k-steps); the scaled logits go through a double-buffered
// shared tile so that every warp sees the whole 16 x 64 row block, computes the (identical) online
// softmax statistics, and then accumulates its own 128 of the 512 output lanes of O += P V.  No
// cross-warp merge is needed at the end.  A fifth warp issues the TMA copies (page gathers through
// the device page table).  All barrier waits are bounded; no multicast is used.
//
// Reference contract: python/sgl_jax/srt/kernels/mla/v2/kernel.py:1338 (oracle mla/v1/ref.py).
#include <cstdlib>
#include <math.h>

#include <unordered_map>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int TN = 64;                 // tokens per tile
constexpr int R = 512;                 // latent width (value width)
constexpr int DK = 576;                // key width = R + rotary lanes
constexpr int kChunks = DK / 64;       // 9 column blocks of 64 bf16 (128-byte swizzle rows)
constexpr int kChunkBytes = TN * 128;  // 8 KB
constexpr int kStageBytes = kChunks * kChunkBytes;   // 72 KB
constexpr int kStages = 2;
constexpr int kQBytes = kChunks * 16 * 128;          // 16 heads x 576 bf16, swizzled per 64-lane block
constexpr int kSBytes = 2 * 16 * TN * 4;             // double-buffered logits tile
constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kSmemBytes = kStages * kStageBytes + kQBytes + kSBytes + 128 + 1024;
constexpr float kLog2e = 1.4426950408889634f;

struct MlaParams {
  const __nv_bfloat16* q_lat;   // [B, H, 512]
  const __nv_bfloat16* q_pe;    // [B, H, 64]
  __nv_bfloat16* out;           // [B, H, 512]
  float* part_o;                // [B, H, splits, 512]
  float* part_lse;              // [B, H, splits]
  const int* page_table;        // [rows, max_pages]
  const int* req_pool_indices;  // [B]
  const int* seq_lens;          // [B]
  Status* status;
  int B, H, max_pages, page_size, num_splits;
  float scale;
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
// byte offset of (row, 16-byte chunk) inside a [rows][64 bf16] block with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__global__ void __launch_bounds__(kThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_sm = smem + kStages * kStageBytes;
  float* s_sm = reinterpret_cast<float*>(q_sm + kQBytes);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(s_sm) + kSBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kStages);

  const int b = blockIdx.x, hg = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = p.seq_lens[b];
  const int* pt_row = p.page_table + static_cast<size_t>(p.req_pool_indices[b]) * p.max_pages;
  const int n_tiles = (seq + TN - 1) / TN;
  const int per = (n_tiles + p.num_splits - 1) / p.num_splits;
  const int t0 = split * per;
  const int t1 = min(t0 + per, n_tiles);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kConsumerWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap);
      const uint64_t pol = l2_policy_evict_first();      // every latent row is read once per head group
      int stage = 0;
      uint32_t phase = 0;
      const int run = p.page_size < TN ? p.page_size : TN;
      const int n_runs = TN / run;
      for (int t = t0; t < t1 && !*abort_flag; ++t) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
          report(p.status, kTimeoutEmptyBarrier, b, t);
          *abort_flag = 1;
          break;
        }
        const uint32_t bar = smem_u32(&full_bar[stage]);
        const uint32_t dst0 = smem_u32(smem + stage * kStageBytes);
        mbar_expect_tx(bar, kStageBytes);
        for (int r = 0; r < n_runs; ++r) {
          const int tok = t * TN + r * run;
          int pg = tok / p.page_size;
          if (pg >= p.max_pages) pg = p.max_pages - 1;
          const int row = pt_row[pg] * p.page_size + (tok - pg * p.page_size);
#pragma unroll
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d_hint(dst0 + c * kChunkBytes + r * run * 128, &tmap, bar, c * 64, row, pol);
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int g = lane >> 2, t4 = lane & 3;
    const int ctid = threadIdx.x;                       // 0..127
    // stage the 16 query rows (zero rows beyond H) into swizzled shared memory
    for (int v = ctid; v < 16 * (DK / 8); v += kConsumerWarps * 32) {
      const int r = v / (DK / 8), c8 = v - r * (DK / 8);          // row, 16-byte chunk along the 576 lanes
      const int h = hg * 16 + r;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (h < p.H) {
        const size_t bh = static_cast<size_t>(b) * p.H + h;
        val = c8 < R / 8 ? *reinterpret_cast<const uint4*>(p.q_lat + bh * R + c8 * 8)
                         : *reinterpret_cast<const uint4*>(p.q_pe + bh * 64 + (c8 - R / 8) * 8);
      }
      const int blk = c8 / 8, ch = c8 % 8;
      *reinterpret_cast<uint4*>(q_sm + blk * (16 * 128) + sw_off(r, ch)) = val;
    }
    named_bar_sync(1, kConsumerWarps * 32);

    float o[16][4];                                      // this warp's 128 output lanes of rows g, g+8
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale_log2 = p.scale * kLog2e;
    const uint32_t q_base = smem_u32(q_sm);
    int stage = 0;
    uint32_t phase = 0;
    int sbuf = 0;
    for (int t = t0; t < t1 && !*abort_flag; ++t) {
      if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
        report(p.status, kTimeoutFullBarrier, b, t);
        *abort_flag = 1;
        break;
      }
      const uint32_t kv = smem_u32(smem + stage * kStageBytes);
      // ---- S[:, 16w .. 16w+15] = Q K^T over the 576 key lanes
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < DK / 16; ++kk) {
        const int blk = kk >> 2, c0 = (kk & 3) * 2;
        uint32_t a[4];
        ldsm_x4(q_base + blk * (16 * 128) + sw_off((lane & 7) + (((lane >> 3) & 1) << 3), c0 + (lane >> 4)),
                a[0], a[1], a[2], a[3]);
        const int row = warp * 16 + (lane & 7) + ((lane >> 4) << 3);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kv + blk * kChunkBytes + sw_off(row, c0 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma16816(s[0], a, b0, b1);
        mma16816(s[1], a, b2, b3);
      }
      float* sb = s_sm + sbuf * (16 * TN);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = warp * 16 + j * 8 + t4 * 2 + (e & 1);
          const int tok = t * TN + col;
          sb[(g + 8 * (e >> 1)) * TN + col] = tok < seq ? s[j][e] * scale_log2 : -INFINITY;
        }
      }
      named_bar_sync(1, kConsumerWarps * 32);
      // ---- online softmax over the whole 16 x 64 block (every warp computes the same statistics)
      float pr[8][4];                                    // [j][e]: cols 8j + 2*t4 + (e&1), row g + 8*(e>>1)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 lo = *reinterpret_cast<const float2*>(sb + g * TN + j * 8 + t4 * 2);
        const float2 hi = *reinterpret_cast<const float2*>(sb + (g + 8) * TN + j * 8 + t4 * 2);
        pr[j][0] = lo.x; pr[j][1] = lo.y; pr[j][2] = hi.x; pr[j][3] = hi.y;
        mx[0] = fmaxf(mx[0], fmaxf(lo.x, lo.y));
        mx[1] = fmaxf(mx[1], fmaxf(hi.x, hi.y));
      }
      float corr[2], mref[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
        mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        const float mnew = fmaxf(m_run[i], mx[i]);
        mref[i] = mnew == -INFINITY ? 0.f : mnew;
        corr[i] = exp2f(m_run[i] - mref[i]);
        m_run[i] = mnew;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(pr[j][e] - mref[e >> 1]);
          pr[j][e] = pv;
          rs[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 1);
        rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 2);
        l_run[i] = l_run[i] * corr[i] + rs[i];
      }
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0];
        o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
      // ---- O[:, 128w .. 128w+127] += P V   (V = the first 512 lanes of the same rows)
#pragma unroll
      for (int kk = 0; kk < TN / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = pack_bf16(pr[2 * kk][0], pr[2 * kk][1]);
        pa[1] = pack_bf16(pr[2 * kk][2], pr[2 * kk][3]);
        pa[2] = pack_bf16(pr[2 * kk + 1][0], pr[2 * kk + 1][1]);
        pa[3] = pack_bf16(pr[2 * kk + 1][2], pr[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int dcol = warp * 128 + np * 16 + ((lane >> 4) << 3);
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(kv + (dcol >> 6) * kChunkBytes + sw_off(row, (dcol & 63) >> 3), b0, b1, b2, b3);
          mma16816(o[2 * np], pa, b0, b1);
          mma16816(o[2 * np + 1], pa, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
      if (++stage == kStages) {
        stage = 0;
        phase ^= 1;
      }
      sbuf ^= 1;
    }
    // ---- write out (rows g and g+8 of this head group, this warp's 128 lanes)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int h = hg * 16 + g + 8 * i;
      if (h >= p.H) continue;
      const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
      const size_t bh = static_cast<size_t>(b) * p.H + h;
      if (p.num_splits == 1) {
        __nv_bfloat16* dst = p.out + bh * R + warp * 128 + t4 * 2;
#pragma unroll
        for (int n = 0; n < 16; ++n)
          *reinterpret_cast<uint32_t*>(dst + n * 8) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
      } else {
        float* dst = p.part_o + (bh * p.num_splits + split) * R + warp * 128 + t4 * 2;
#pragma unroll
        for (int n = 0; n < 16; ++n)
          *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
        if (warp == 0 && t4 == 0)
          p.part_lse[bh * p.num_splits + split] = l_run[i] > 0.f ? m_run[i] + log2f(l_run[i]) : -INFINITY;
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the CTA's shared memory is released
    const uint64_t ts = global_timer_ns();
    while (global_timer_ns() - ts < 200000ull) __nanosleep(1000);
  }
}

__global__ void mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                   __nv_bfloat16* __restrict__ out, int num_splits) {
  const int row = blockIdx.x;   // b * H + h
  const float* lse = part_lse + static_cast<size_t>(row) * num_splits;
  float mmax = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mmax = fmaxf(mmax, lse[s]);
  float wsum = 0.f;
  for (int s = 0; s < num_splits; ++s) wsum += (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mmax);
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  for (int d = threadIdx.x; d < R; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float w = (lse[s] == -INFINITY) ? 0.f : exp2f(lse[s] - mmax);
      acc += w * part_o[(static_cast<size_t>(row) * num_splits + s) * R + d];
    }
    out[static_cast<size_t>(row) * R + d] = __float2bfloat16(acc * inv);
  }
}

struct Key {
  const void* p; long long rows; int box;
  bool operator==(const Key& o) const { return p == o.p && rows == o.rows && box == o.box; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    return std::hash<const void*>()(k.p) ^ (std::hash<long long>()(k.rows) * 1315423911u) ^ (k.box * 2654435761u);
  }
};
std::unordered_map<Key, CUtensorMap, KeyHash> g_maps;

bool get_map(const void* kv, long long rows, int page_size, CUtensorMap* out) {
  const int box_rows = page_size < TN ? page_size : TN;
  Key key{kv, rows, box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) {
    *out = it->second;
    return true;
  }
  CUtensorMap m;
  if (!encode_tmap_2d(&m, kv, DK, rows, static_cast<uint64_t>(DK) * 2, 64, box_rows, 2)) return false;
  if (g_maps.size() > 1024) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace
}  // namespace sglb

extern "C" {

// Absorbed-MLA decode.  `kv_buffer` is the latent cache [num_pages, page_size, 576] (bf16); `q_lat`
// [B, H, 512], `q_pe` [B, H, 64]; `out` [B, H, 512].  With `num_splits > 1` the partial buffers
// `part_o [B, H, splits, 512]` and `part_lse [B, H, splits]` (fp32) are required.
int sglb_mla_decode(const void* q_lat, const void* q_pe, void* out, const void* kv_buffer, long long num_pages,
                    const int* page_table, int max_pages, const int* req_pool_indices, const int* seq_lens, int B,
                    int H, int kv_lora_rank, int rope_dim, int page_size, float scale, int num_splits, float* part_o,
                    float* part_lse, cudaStream_t stream) {
  using namespace sglb;
  if (B <= 0) return 0;
  if (kv_lora_rank != R || rope_dim != DK - R) return -kBadArgument;
  if (page_size < TN ? (TN % page_size != 0) : (page_size % TN != 0)) return -kBadArgument;
  if (num_splits > 1 && (part_o == nullptr || part_lse == nullptr)) return -kBadArgument;
  CUtensorMap tm;
  if (!get_map(kv_buffer, num_pages * page_size, page_size, &tm)) return -100;
  MlaParams p{};
  p.q_lat = static_cast<const __nv_bfloat16*>(q_lat);
  p.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.part_o = part_o;
  p.part_lse = part_lse;
  p.page_table = page_table;
  p.req_pool_indices = req_pool_indices;
  p.seq_lens = seq_lens;
  p.status = device_status();
  p.B = B; p.H = H; p.max_pages = max_pages; p.page_size = page_size;
  p.num_splits = num_splits < 1 ? 1 : num_splits;
  p.scale = scale;
  static bool cfg = false;
  if (!cfg) {
    cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    cfg = true;
  }
  dim3 grid(B, (H + 15) / 16, p.num_splits);
  mla_decode_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tm, p);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess && p.num_splits > 1) {
    mla_combine_kernel<<<B * H, 128, 0, stream>>>(part_o, part_lse, p.out, p.num_splits);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}

}  // extern "C"
