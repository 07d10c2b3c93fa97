// Page-granular KV movement between pools: device <-> pinned host (hierarchical cache tier)
// and device <-> device / peer (prefill -> decode hand-over).
//
// One launch moves `n` pages of one layer: page i goes from `src + src_pages[i] * src_stride`
// to `dst + dst_pages[i] * dst_stride`.  Either side may be pinned host memory (reachable
// from the device under unified addressing) or a peer GPU's buffer, so the same kernel
// backs the D2H write-back, the H2D load-back and the P2P push.  Counterpart of the
// reference's page gather/scatter jits (`mem_cache/host_kv_pool.py`, `disaggregation/prefill.py:86-101`).
#include <cstdint>
#include <cuda_runtime.h>

#include "common.cuh"

namespace sglb {

__global__ void kv_page_copy_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src,
                                    const long long* __restrict__ dst_pages, const long long* __restrict__ src_pages,
                                    int n, long long page_bytes, long long dst_stride, long long src_stride) {
  // blockIdx.y = page, blockIdx.x strides over the page's 16-byte words
  const int pg = blockIdx.y;
  if (pg >= n) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + src_pages[pg] * src_stride);
  uint4* d = reinterpret_cast<uint4*>(dst + dst_pages[pg] * dst_stride);
  const long long words = page_bytes >> 4;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < words;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    d[i] = s[i];
}

}  // namespace sglb

extern "C" {

// All sizes in bytes; bases, strides and page_bytes must be multiples of 16.
int sglb_kv_page_copy(void* dst, const void* src, const long long* dst_pages, const long long* src_pages, int n,
                      long long page_bytes, long long dst_stride, long long src_stride, cudaStream_t s) {
  if (n <= 0) return 0;
  if ((page_bytes | dst_stride | src_stride) & 15) return -sglb::kBadArgument;
  if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) return -sglb::kBadArgument;
  const long long words = page_bytes >> 4;
  int bx = static_cast<int>((words + 255) / 256);
  if (bx > 32) bx = 32;
  if (bx < 1) bx = 1;
  int done = 0;
  while (done < n) {
    const int chunk = n - done > 65535 ? 65535 : n - done;
    dim3 grid(bx, chunk);
    sglb::kv_page_copy_kernel<<<grid, 256, 0, s>>>(static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src),
                                                   dst_pages + done, src_pages + done, chunk, page_bytes, dst_stride,
                                                   src_stride);
    done += chunk;
  }
  return static_cast<int>(cudaGetLastError());
}

// Lets kernels running on `device` dereference memory of `peer` (needed before a page copy reads a peer's pool
// through a CUDA IPC mapping).  Returns 0 when access is on (now or already), a negative code when the two
// devices cannot reach each other, a positive CUDA error otherwise.  The current device is left unchanged.
int sglb_enable_peer_access(int device, int peer) {
  if (device == peer) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, device, peer);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (!can) return -sglb::kBadArgument;
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  e = cudaDeviceEnablePeerAccess(peer, 0);
  cudaSetDevice(prev);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();      // clear the sticky-less error state this call leaves behind
    return 0;
  }
  return static_cast<int>(e);
}
}
