// Speculative-decoding helpers: greedy tree verification and tree-mask construction.
//
// Counterparts of the reference's `kernels/speculative/verify_tree_greedy_kernel.py` and
// `build_eagle_tree_structure_kernel.py`.  The trees are tiny (<= 64 nodes), so one warp
// handles one request.
#include <cstdint>
#include <cuda_runtime.h>

#include "common.cuh"

namespace sglb {

// tokens / parent / target: [B, n] int64.  parent[i] is the tree index of node i's parent (-1 root).
// Walks from the root: the child whose token equals the target's choice at the current node is accepted.
__global__ void verify_tree_greedy_kernel(const long long* __restrict__ tokens, const long long* __restrict__ parent,
                                          const long long* __restrict__ target, long long* __restrict__ accept,
                                          long long* __restrict__ path, long long* __restrict__ bonus, int n,
                                          int max_depth) {
  const int b = blockIdx.x;
  const int lane = threadIdx.x;
  const long long* tok = tokens + static_cast<size_t>(b) * n;
  const long long* par = parent + static_cast<size_t>(b) * n;
  const long long* tgt = target + static_cast<size_t>(b) * n;
  long long* pth = path + static_cast<size_t>(b) * (max_depth + 1);
  int cur = 0, acc = 0;
  if (lane == 0) pth[0] = 0;
  for (int d = 1; d <= max_depth; ++d) {
    const long long want = tgt[cur];
    int found = 0x7fffffff;
    for (int i = 1 + lane; i < n; i += 32)
      if (par[i] == cur && tok[i] == want && i < found) found = i;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) found = min(found, __shfl_xor_sync(0xffffffffu, found, o));
    if (found == 0x7fffffff) {
      for (int k = d + lane; k <= max_depth; k += 32) pth[k] = -1;
      break;
    }
    cur = found;
    ++acc;
    if (lane == 0) pth[d] = cur;
  }
  if (lane == 0) {
    accept[b] = acc;
    bonus[b] = tgt[cur];
  }
}

// mask[b, i, j] = 1 when j is i or an ancestor of i; depth[b, i] = number of ancestors.
__global__ void tree_mask_kernel(const long long* __restrict__ parent, uint8_t* __restrict__ mask,
                                 long long* __restrict__ depth, int n) {
  const int b = blockIdx.x;
  const long long* par = parent + static_cast<size_t>(b) * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    uint8_t* row = mask + (static_cast<size_t>(b) * n + i) * n;
    for (int j = 0; j < n; ++j) row[j] = 0;
    row[i] = 1;
    int d = 0;
    long long c = par[i];
    // a parent index is always smaller than its child's, so the walk ends within n steps
    for (int step = 0; step < n && c >= 0 && c < n; ++step) {
      row[c] = 1;
      ++d;
      c = par[c];
    }
    depth[static_cast<size_t>(b) * n + i] = d;
  }
}

}  // namespace sglb

extern "C" {

int sglb_verify_tree_greedy(const long long* tokens, const long long* parent, const long long* target,
                            long long* accept, long long* path, long long* bonus, int B, int n, int max_depth,
                            cudaStream_t s) {
  if (B <= 0) return 0;
  if (n <= 0 || max_depth < 0) return -sglb::kBadArgument;
  sglb::verify_tree_greedy_kernel<<<B, 32, 0, s>>>(tokens, parent, target, accept, path, bonus, n, max_depth);
  return static_cast<int>(cudaGetLastError());
}

int sglb_tree_mask(const long long* parent, void* mask, long long* depth, int B, int n, cudaStream_t s) {
  if (B <= 0) return 0;
  if (n <= 0) return -sglb::kBadArgument;
  sglb::tree_mask_kernel<<<B, 64, 0, s>>>(parent, static_cast<uint8_t*>(mask), depth, n);
  return static_cast<int>(cudaGetLastError());
}
}
