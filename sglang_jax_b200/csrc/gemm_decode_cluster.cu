// Decode-sized GEMM with split-K inside a thread-block cluster.
//
//   out[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]),   x [M, K] bf16 (M <= 128 tokens), w [N, K] bf16, out [M, N] bf16
//
// With a handful of tokens the product is a stream of the weight matrix: the work that can be spread over the 148 SMs
// is K, not M x N.  The persistent kernel in gemm_sm100.cu splits K stream-K style and repairs the shared tiles
// through global memory (partials dumped as fp32, counters, fences, a second pass).  Here the `csize` CTAs of one
// cluster share one 128-row weight tile instead: CTA r multiplies K blocks [r, r + 1) * K / csize into its own
// tensor-memory accumulator (weight rows on the MMA M dimension, tokens on N), and the partial sums meet in
// distributed shared memory: accumulator row i goes to the CTA that owns rows [o * 128 / csize, (o + 1) * 128 /
// csize), as fp32 `st.shared::cluster` stores, one cluster barrier later every CTA sums the csize partials of its
// rows and writes them out.  No global scratch, no atomics, no memory fences, one launch.
//
// Every CTA issues its own TMA loads (plain per-CTA `cp.async.bulk.tensor`, nothing is broadcast across the cluster);
// waits on mbarriers are bounded; an aborting CTA still arrives at the cluster barrier, so its peers never wait for it.
#include "common.cuh"

namespace sglb {
namespace {

constexpr int CBM = 128;                 // weight rows per tile (MMA M)
constexpr int CBK = 64;                  // bf16 elements per K block: one 128-byte swizzle row
// (the ring holds 144 - 192 KB in flight per SM: weight bytes come from HBM with a latency of a couple of microseconds)
constexpr int kCThreads = 192;           // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

struct CParams {
  __nv_bfloat16* out;
  const __nv_bfloat16* bias;
  Status* status;
  int M, N, K, kb_total, csize;
};

template <int BN>
struct CCfg {
  static constexpr int kStageA = CBM * CBK * 2;                 // 16 KB of weights
  static constexpr int kStageB = BN * CBK * 2;                  // tokens
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = BN >= 128 ? 6 : 8;
  static constexpr int kRing = kStages * kStage;
  static constexpr int kReduce = CBM * BN * 4;                  // csize partials of 128 / csize rows x BN fp32
  // the reduce buffer reuses the front of the ring once every CTA of the cluster is done with its operands
  static_assert(kReduce <= kRing, "reduce buffer must fit into the operand ring");
  static constexpr int kSmem = kRing + 256 + 1024;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// address of this CTA's shared-memory location `addr` inside CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kCThreads, 1)
gemm_decode_cluster_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                           const CParams p) {
  using C = CCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  float* red = reinterpret_cast<float*>(smem);                          // [src rank][BN / 4][rows_per][4], aliases the ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kRing);
  constexpr int kCStages = C::kStages;
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kCStages;
  uint64_t* acc_bar = bars + 2 * kCStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int csize = p.csize;
  const int rank = static_cast<int>(cluster_ctarank());
  const int tile = blockIdx.x / csize;
  const int n0 = tile * CBM;
  const int m0 = blockIdx.y * BN;
  const int kb0 = static_cast<int>(static_cast<long long>(p.kb_total) * rank / csize);
  const int kb1 = static_cast<int>(static_cast<long long>(p.kb_total) * (rank + 1) / csize);
  const int rows_per = CBM / csize;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_w);
    prefetch_tmap(&tmap_x);
    for (int s = 0; s < kCStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(acc_bar), 1);
    *abort_flag = 0;
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
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1 && !*abort_flag; ++kb) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1)) {
          report(p.status, kTimeoutEmptyBarrier, tile, kb);
          *abort_flag = 1;
          break;
        }
        const uint32_t fb = smem_u32(&full_bar[stage]);
        mbar_expect_tx(fb, C::kStage);
        uint8_t* sa = ring + stage * C::kStage;
        tma_load_2d(smem_u32(sa), &tmap_w, fb, kb * CBK, n0);
        tma_load_2d(smem_u32(sa + C::kStageA), &tmap_x, fb, kb * CBK, m0);
        if (++stage == kCStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(CBM, BN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && !*abort_flag; ++kb) {
        if (!mbar_wait(smem_u32(&full_bar[stage]), phase)) {
          report(p.status, kTimeoutFullBarrier, tile, kb);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(ring + stage * C::kStage);
        const uint64_t da = make_smem_desc_sw128(sa);
        const uint64_t db = make_smem_desc_sw128(sa + C::kStageA);
#pragma unroll
        for (int k = 0; k < CBK / 16; ++k) umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(smem_u32(&empty_bar[stage]));
        if (++stage == kCStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(smem_u32(acc_bar));
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps: scatter the partial rows
    const int q = warp & 3;
    const int row = q * 32 + lane;                       // accumulator row = weight row of the tile
    bool have = kb1 > kb0;
    if (have && !__all_sync(0xffffffffu, mbar_wait(smem_u32(acc_bar), 0))) {
      if (lane == 0) report(p.status, kTimeoutTmemFull, tile, rank);
      *abort_flag = 1;
      have = false;
    }
    tc_fence_after_sync();
    // every MMA of this CTA has read its operands.  Once all CTAs of the cluster are here, their rings are free to
    // receive partial rows (the producer / MMA warps arrive at the same barrier from their own code path below)
    __syncwarp();
    cluster_arrive();
    cluster_wait();
    const int owner = row / rows_per;
    const int lrow = row - owner * rows_per;
    // destination inside the owner's reduce buffer: [this rank][col / 4][lrow][4] floats
    const uint32_t dst0 = map_to_cta(smem_u32(red), static_cast<uint32_t>(owner)) +
                          static_cast<uint32_t>(((rank * (BN / 4)) * rows_per + lrow) * 16);
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    constexpr int CW = BN < 32 ? 16 : 32;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += CW) {
      uint32_t v[32];
      if (have) {
        if constexpr (CW == 32) tmem_ld32(taddr + c0, v);
        else tmem_ld16(taddr + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < CW; ++e) v[e] = 0u;          // a rank without K blocks (or an aborted one) adds zeros
      }
#pragma unroll
      for (int e = 0; e < CW / 4; ++e)
        st_cluster_v4(dst0 + static_cast<uint32_t>(((c0 / 4 + e) * rows_per) * 16), v[4 * e], v[4 * e + 1], v[4 * e + 2],
                      v[4 * e + 3]);
    }
    tc_fence_before_sync();
  }

  if (warp < 2) {
    // first cluster barrier (rings free), from the producer / MMA warps: their lanes rejoin first, the barrier
    // instructions are warp-aligned
    __syncwarp();
    cluster_arrive();
    cluster_wait();
  }
  // second barrier, every thread of every CTA: the partial rows are in their owners' shared memory after this
  __syncwarp();
  cluster_arrive();
  cluster_wait();

  if (warp >= 2 && !*abort_flag) {
    // ------------------------------------------------------------------ owner: sum the csize partials of my rows
    const int t = threadIdx.x - 64;                      // 0..127
    const int items = (BN / 4) * rows_per;               // (column group of 4 tokens, row) pairs
    const float4* rv = reinterpret_cast<const float4*>(red);
    for (int it = t; it < items; it += 128) {
      const int c4 = it / rows_per;
      const int lrow = it - c4 * rows_per;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int src = 0; src < csize; ++src) {
        const float4 a = rv[(src * (BN / 4) + c4) * rows_per + lrow];
        s.x += a.x;
        s.y += a.y;
        s.z += a.z;
        s.w += a.w;
      }
      const int n = n0 + rank * rows_per + lrow;
      if (n < p.N) {
        const float b = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
        const int tok = m0 + c4 * 4;
        const float o[4] = {s.x + b, s.y + b, s.z + b, s.w + b};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (tok + e < p.M) p.out[static_cast<size_t>(tok + e) * p.N + n] = __float2bfloat16(o[e]);
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
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN>
cudaError_t launch_cluster(const CUtensorMap& tw, const CUtensorMap& tx, const CParams& p, dim3 grid, cudaStream_t stream) {
  auto* kern = gemm_decode_cluster_kernel<BN>;
  static bool cfg_done = false;
  if (!cfg_done) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CCfg<BN>::kSmem);
    if (e != cudaSuccess) return e;
    cfg_done = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kCThreads);
  cfg.dynamicSmemBytes = CCfg<BN>::kSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, p);
}

}  // namespace
}  // namespace sglb

extern "C" {

// Cluster size this launcher would use for the shape (0: the shape is outside its range).
int sglb_gemm_decode_cluster_size(int M, int N, int K) {
  if (M < 1 || M > 128 || N < 8 || K < 64 || (K % 64) != 0 || (N % 8) != 0) return 0;
  const int tiles = (N + 127) / 128;
  const int kb = K / 64;
  int cs = 1;
  // as many CTAs as SMs without a second wave, at least two K blocks per CTA
  while (cs < 8 && tiles * (cs * 2) <= sglb::sm_count() && kb / (cs * 2) >= 2) cs *= 2;
  return cs;
}

// out = x . w^T (+ bias) for M <= 128 tokens with split-K inside thread-block clusters (see the top of this file).
// Needs K a multiple of 64 and N a multiple of 8; 16-byte aligned operands.  Returns 0, a negative argument code,
// or a positive CUDA error.
int sglb_gemm_decode_cluster(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                             cudaStream_t stream) {
  using namespace sglb;
  const int cs = sglb_gemm_decode_cluster_size(M, N, K);
  if (cs == 0) return -kBadArgument;
  int bn = 16;
  while (bn < M) bn *= 2;                                 // 16, 32, 64, 128
  CUtensorMap tw, tx;
  if (!encode_tmap_2d(&tw, w, K, N, static_cast<uint64_t>(K) * 2, CBK, CBM, 2)) return -100;
  if (!encode_tmap_2d(&tx, x, K, M, static_cast<uint64_t>(K) * 2, CBK, bn, 2)) return -101;
  CParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.status = device_status();
  p.M = M;
  p.N = N;
  p.K = K;
  p.kb_total = K / CBK;
  p.csize = cs;
  const dim3 grid(((N + 127) / 128) * cs, 1, 1);
  cudaError_t e;
  switch (bn) {
    case 16: e = launch_cluster<16>(tw, tx, p, grid, stream); break;
    case 32: e = launch_cluster<32>(tw, tx, p, grid, stream); break;
    case 64: e = launch_cluster<64>(tw, tx, p, grid, stream); break;
    default: e = launch_cluster<128>(tw, tx, p, grid, stream); break;
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
}
