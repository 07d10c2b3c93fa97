// Host-side runtime pieces shared by the kernels: per-device status word, TMA tensor-map
// encoding through the driver entry point (no link-time dependency on libcuda), SM count.
#include <mutex>

#include "common.cuh"

namespace sglb {

namespace {
constexpr int kMaxDevices = 16;
Status* g_status[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_mu;

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;

EncodeFn get_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<EncodeFn>(fn);
  return g_encode;
}
}  // namespace

Status* device_status() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    Status* p = nullptr;
    if (cudaMalloc(&p, sizeof(Status)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(Status));
    g_status[dev] = p;
  }
  return g_status[dev];
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("SGLB_PDL");
    return e == nullptr || atoi(e) != 0;
  }();
  return on;
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return 148;
  if (!g_sm_count[dev]) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

// 2-D row-major tensor [rows, inner_elems] with a 128-byte swizzle; the box is
// box_inner x box_rows elements.  The box's inner extent must be 128 bytes.
bool encode_tmap_2d(CUtensorMap* out, const void* base, uint64_t inner_elems, uint64_t rows,
                    uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows, int elem_bytes) {
  EncodeFn enc = get_encode();
  if (!enc) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15)) return false;
  cuuint64_t dims[2] = {inner_elems, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace sglb

extern "C" {

// Copies the status word to the host and clears it.  Returns the status code (0 = ok).
int sglb_read_status(int* out4) {
  sglb::Status* d = sglb::device_status();
  if (!d) return -1;
  sglb::Status h;
  if (cudaMemcpy(&h, d, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  if (out4) {
    out4[0] = h.code;
    out4[1] = h.block;
    out4[2] = h.aux0;
    out4[3] = h.aux1;
  }
  if (h.code != 0) cudaMemset(d, 0, sizeof(h));
  return h.code;
}

int sglb_sm_count() { return sglb::sm_count(); }

const char* sglb_version() { return "sglb200-sm100a-0.1"; }
}
