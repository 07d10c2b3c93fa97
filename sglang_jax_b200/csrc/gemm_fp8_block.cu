// Block-scaled FP8 GEMM (the DeepSeek-V3 weight format) on the 5th-generation tensor cores.
//
//   out[m, n] = sum_kb  sx[kb, m] * sw[n / 128, kb] * sum_{k in block kb} xq[m, k] * wq[n, k]
//
// xq [M, K] e4m3 with one fp32 scale per token and 128-wide K group (`sx`, stored [K/128, M] so that the
// 128 token rows of a tile read consecutive floats), wq [N, K] e4m3 with one fp32 scale per 128 x 128 block
// (`sw [N/128, K/128]`, the checkpoint's `weight_scale_inv`), bf16 output, fp32 accumulation.
//
// The tensor core cannot apply a scale that changes along K, so every 128-wide K block is multiplied on its
// own into tensor memory (tcgen05.mma kind::f8f6f4, 128 x 128 x 32 per instruction, accumulate reset per
// block) and "promoted": eight warps (two per lane quarter of tensor memory, each owning 64 of the 128
// columns) read the block's partial product out of tensor memory (tcgen05.ld, both loads in flight before
// one wait), hand the buffer back, multiply by the two scales and add to fp32 accumulators in registers,
// while the MMA warp already fills the other half of tensor memory with the next block.  One K block is exactly one
// 128-byte swizzle row, i.e. one stage of the TMA ring.
//
// Dense and grouped (MoE experts: rows sorted by expert, 128-row token tiles from the list `moe_align`
// builds) share the kernel.  Reference counterpart: the block-wise quantised matmul
// python/sgl_jax/srt/kernels/quantized_matmul/quantized_matmul_kernels/blockwise_kernel.py:200.
#include <cuda_fp8.h>

#include "common.cuh"

namespace sglb {
namespace {

constexpr int BM = 128, BN = 128, BKB = 128;      // tile, and bytes (= fp8 elements) of one K block
constexpr int kStages = 6;
constexpr int kStageBytes = (BM + BN) * BKB;
constexpr int kEpi = 256;                        // promotion / epilogue threads: warps 2..9
constexpr int kThreads = 64 + kEpi;
constexpr int kCols = BN / 2;                     // accumulator columns per promotion thread
constexpr int kAccBufs = 4;                       // K-block products in flight in tensor memory (4 x 128 columns)
constexpr int kSmem = kStages * kStageBytes + (2 * kStages + 2 * kAccBufs) * 8 + 16 + 1024;

struct BParams {
  __nv_bfloat16* out;        // [M, N]
  const float* sx;           // [KB, sx_stride]
  const float* sw;           // [groups][NB][KB]
  const __nv_bfloat16* bias; // [N] or null (dense only)
  Status* status;
  int M, N, K, KB, NB, sx_stride;
  int tiles_m, tiles_n;
  // grouped
  const int* group_offsets;  // [groups + 1] or null
  const int* tile_group;
  const int* tile_row0;
  const int* num_token_tiles;
};

struct BTile {
  int a_row, b_row, m0, m_limit, n0, sw_off;
};

__device__ __forceinline__ bool next_tile(const BParams& p, int& it, BTile& t) {
  const int w = blockIdx.x + it * gridDim.x;
  if (p.group_offsets == nullptr) {
    if (w >= p.tiles_m * p.tiles_n) return false;
    ++it;
    const int tn = w / p.tiles_m, tm = w - tn * p.tiles_m;
    t.a_row = tm * BM;
    t.b_row = tn * BN;
    t.m0 = tm * BM;
    t.m_limit = p.M;
    t.n0 = tn * BN;
    t.sw_off = tn * p.KB;
    return true;
  }
  const int ntt = *p.num_token_tiles;
  if (w >= ntt * p.tiles_n) return false;
  ++it;
  const int tn = w / ntt, tm = w - tn * ntt;
  const int g = p.tile_group[tm];
  const int row0 = p.tile_row0[tm];
  t.a_row = row0;
  t.b_row = g * p.N + tn * BN;
  t.m0 = row0;
  t.m_limit = min(p.group_offsets[g + 1], row0 + BM);
  t.n0 = tn * BN;
  t.sw_off = (g * p.NB + tn) * p.KB;
  return true;
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const BParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  // The hand-over of one K block (commit -> promotion warps wake -> tcgen05.ld -> arrive -> MMA warp wakes) is a
  // round trip of about a microsecond, several times the block's MMA time: four buffers keep that many in flight.
  uint64_t* acc_full = bars + 2 * kStages;       // [kAccBufs] one K block's product is in tensor memory
  uint64_t* acc_empty = acc_full + kAccBufs;     // [kAccBufs] ... and has been read out again
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + kAccBufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
      mbar_init(smem_u32(&acc_full[a]), 1);
      mbar_init(smem_u32(&acc_empty[a]), kEpi / 32);   // one arrival per promotion warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kAccBufs * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0, it = 0;
      uint32_t phase = 0;
      BTile t;
      while (!*abort_flag && next_tile(p, it, t)) {
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
            report(p.status, kTimeoutEmptyBarrier, t.m0, kb);
            *abort_flag = 1;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, kStageBytes);
          uint8_t* sa = smem + stage * kStageBytes;
          tma_load_2d(smem_u32(sa), &tmap_a, fb, kb * BKB, t.a_row);
          tma_load_2d(smem_u32(sa + BM * BKB), &tmap_b, fb, kb * BKB, t.b_row);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 0, 0);
      int stage = 0, it = 0, buf = 0;
      uint32_t phase = 0, buf_phase = 0;
      BTile t;
      bool ok = true;
      while (ok && !*abort_flag && next_tile(p, it, t)) {
        for (int kb = 0; kb < p.KB; ++kb) {
          if (!mbar_wait(smem_u32(&acc_empty[buf]), buf_phase ^ 1)) {
            report(p.status, kTimeoutTmemEmpty, t.m0, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
            report(p.status, kTimeoutFullBarrier, t.m0, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + BM * BKB);
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(d_tmem, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
          umma_commit(smem_u32(&empty_bar[stage]));
          umma_commit(smem_u32(&acc_full[buf]));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
          if (++buf == kAccBufs) {
            buf = 0;
            buf_phase ^= 1;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ promotion + epilogue (warps 2..9)
    const int q = warp & 3;                        // lane quarter of tensor memory this warp may read
    const int col0 = ((warp - 2) >> 2) * kCols;    // its half of the tile's columns
    const int row = q * 32 + lane;
    int it = 0, buf = 0;
    uint32_t buf_phase = 0;
    BTile t;
    bool ok = true;
    while (ok && !*abort_flag && next_tile(p, it, t)) {
      float acc[kCols];
#pragma unroll
      for (int c = 0; c < kCols; ++c) acc[c] = 0.f;
      const int m = t.m0 + row;
      const bool live = m < t.m_limit;
      // The scale of a K block comes from global memory (an L2 round trip): a register ring keeps the loads four
      // blocks ahead of their use, so that latency stays off the per-block critical path.
      auto load_scale = [&](int kb) -> float {
        if (kb >= p.KB) return 0.f;
        return (live ? __ldg(p.sx + static_cast<size_t>(kb) * p.sx_stride + m) : 0.f) * __ldg(p.sw + t.sw_off + kb);
      };
      float ring[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ring[i] = load_scale(i);
      for (int kb0 = 0; ok && kb0 < p.KB; kb0 += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int kb = kb0 + i;
          if (kb >= p.KB) break;
          const float s = ring[i];
          ring[i] = load_scale(kb + 4);
          if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&acc_full[buf]), buf_phase))) {
            report(p.status, kTimeoutTmemFull, t.m0, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + col0;
          uint32_t v0[32], v1[32];
          tmem_ld32(taddr, v0);
          tmem_ld32(taddr + 32, v1);
          tmem_ld_wait();
          // the block's product is in registers: the MMA warp may reuse this part of tensor memory
          // (one elected lane per warp arrives: hundreds of arrivals on one barrier word would serialise)
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            acc[e] = fmaf(s, __uint_as_float(v0[e]), acc[e]);
            acc[32 + e] = fmaf(s, __uint_as_float(v1[e]), acc[32 + e]);
          }
          if (++buf == kAccBufs) {
            buf = 0;
            buf_phase ^= 1;
          }
        }
      }
      if (!ok) break;
      if (live) {
        __nv_bfloat16* orow = p.out + static_cast<size_t>(m) * p.N + t.n0 + col0;
#pragma unroll
        for (int c = 0; c < kCols; c += 8) {
          if (t.n0 + col0 + c < p.N) {
            float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (p.bias != nullptr) {
#pragma unroll
              for (int e = 0; e < 8; ++e) b[e] = __bfloat162float(p.bias[t.n0 + col0 + c + e]);
            }
            *reinterpret_cast<uint4*>(orow + c) =
                make_uint4(pack_bf16(acc[c] + b[0], acc[c + 1] + b[1]), pack_bf16(acc[c + 2] + b[2], acc[c + 3] + b[3]),
                           pack_bf16(acc[c + 4] + b[4], acc[c + 5] + b[5]), pack_bf16(acc[c + 6] + b[6], acc[c + 7] + b[7]));
          }
        }
      }
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
    tmem_dealloc(tmem_base, kAccBufs * BN);
  }
}

// x [rows, K] bf16 -> e4m3 with one scale per row and 128-wide group; scales stored [K/128, stride].
// One warp per (row, 4 groups): 16 lanes per group of 128 (8 elements per lane).
__global__ void quant_fp8_group128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                          float* __restrict__ sx, int rows, int K, int stride, const int* valid_rows) {
  const int n = valid_rows != nullptr ? min(rows, *valid_rows) : rows;
  const int groups = K >> 7;
  const int warps = blockDim.x >> 5;
  const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4, l16 = lane & 15;
  const long long pairs = static_cast<long long>(n) * ((groups + 1) / 2);
  for (long long w = static_cast<long long>(blockIdx.x) * warps + wid; w < pairs; w += static_cast<long long>(gridDim.x) * warps) {
    const int r = static_cast<int>(w / ((groups + 1) / 2));
    const int g = static_cast<int>(w - static_cast<long long>(r) * ((groups + 1) / 2)) * 2 + half;
    float f[8];
    float amax = 0.f;
    const bool live = g < groups;
    if (live) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * K + g * 128 + l16 * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 t = __bfloat1622float2(h[e]);
        f[2 * e] = t.x;
        f[2 * e + 1] = t.y;
        amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (live) {
      const float scale = fmaxf(amax / 448.f, 1e-12f);
      const float inv = 1.f / scale;
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_fp8_storage_t b0 = __nv_cvt_float_to_fp8(f[e] * inv, __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8_storage_t b1 = __nv_cvt_float_to_fp8(f[4 + e] * inv, __NV_SATFINITE, __NV_E4M3);
        lo |= static_cast<uint32_t>(b0) << (8 * e);
        hi |= static_cast<uint32_t>(b1) << (8 * e);
      }
      *reinterpret_cast<uint2*>(q + static_cast<size_t>(r) * K + g * 128 + l16 * 8) = make_uint2(lo, hi);
      if (l16 == 0) sx[static_cast<size_t>(g) * stride + r] = scale;
    }
  }
}

}  // namespace
}  // namespace sglb


extern "C" {

// x [rows, K] bf16 (K a multiple of 128) -> q [rows, K] e4m3, sx [K/128, stride] fp32 (stride >= rows).
// `valid_rows` (device int, may be null) bounds the rows actually quantised.
int sglb_quant_fp8_group128(const void* x, void* q, float* sx, int rows, int K, int stride, const int* valid_rows,
                            cudaStream_t stream) {
  using namespace sglb;
  if (rows <= 0) return 0;
  if (K % 128 || stride < rows) return -kBadArgument;
  const long long pairs = static_cast<long long>(rows) * ((K / 128 + 1) / 2);
  long long blocks = (pairs + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  quant_fp8_group128_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), sx, rows, K, stride, valid_rows);
  return static_cast<int>(cudaGetLastError());
}

static int fp8_block_launch(const void* xq, const void* wq, const float* sx, int sx_stride, const float* sw,
                            const void* bias, void* out, int M, int N, int K, int groups, const int* group_offsets,
                            const int* tile_group, const int* tile_row0, const int* num_token_tiles,
                            cudaStream_t stream) {
  using namespace sglb;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (K % 128 || N % 8) return -kBadArgument;
  BParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.sx = sx;
  p.sw = sw;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = device_status();
  p.M = M;
  p.N = N;
  p.K = K;
  p.KB = K / 128;
  p.NB = (N + 127) / 128;
  p.sx_stride = sx_stride;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_offsets = group_offsets;
  p.tile_group = tile_group;
  p.tile_row0 = tile_row0;
  p.num_token_tiles = num_token_tiles;
  p.tiles_m = group_offsets != nullptr ? M / BM + groups : (M + BM - 1) / BM;
  CUtensorMap ta, tb;
  if (!encode_tmap_2d(&ta, xq, K, M, static_cast<uint64_t>(K), BKB, BM, 1)) return -100;
  if (!encode_tmap_2d(&tb, wq, K, static_cast<uint64_t>(groups > 0 ? groups : 1) * N, static_cast<uint64_t>(K), BKB, BN, 1))
    return -101;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int grid = p.tiles_m * p.tiles_n;
  const int sms = sm_count();
  if (grid > sms) grid = sms;
  cudaError_t err = launch_pdl(gemm_fp8_block_kernel, dim3(grid), dim3(kThreads), kSmem, stream, ta, tb, p);
  return err == cudaSuccess ? 0 : static_cast<int>(err);
}

// out[M, N] (bf16) = block-scaled product of xq [M, K] e4m3 (scales sx [K/128, sx_stride]) and wq [N, K] e4m3
// (scales sw [ceil(N/128), K/128]) (+ bias).  K a multiple of 128, N of 8.
int sglb_gemm_fp8_block(const void* xq, const void* wq, const float* sx, int sx_stride, const float* sw, const void* bias,
                        void* out, int M, int N, int K, cudaStream_t stream) {
  return fp8_block_launch(xq, wq, sx, sx_stride, sw, bias, out, M, N, K, 0, nullptr, nullptr, nullptr, nullptr, stream);
}

// Grouped form for routed experts: rows of xq sorted by expert, wq [groups * N, K], sw [groups][N/128][K/128];
// tile lists as built by sglb_moe_align.  N must be a multiple of 128.
int sglb_grouped_gemm_fp8_block(const void* xq, const void* wq, const float* sx, int sx_stride, const float* sw,
                                void* out, const int* group_offsets, const int* tile_group, const int* tile_row0,
                                const int* num_token_tiles, int rows, int N, int K, int groups, cudaStream_t stream) {
  if (N % 128 || group_offsets == nullptr || tile_group == nullptr || tile_row0 == nullptr || num_token_tiles == nullptr)
    return -sglb::kBadArgument;
  return fp8_block_launch(xq, wq, sx, sx_stride, sw, nullptr, out, rows, N, K, groups, group_offsets, tile_group,
                          tile_row0, num_token_tiles, stream);
}
}
