// Host-side runtime shared by every kernel translation unit: the per-device status word for
// bounded waits, TMA descriptor encoding (driver entry point resolved at run time), device
// properties, and a tiny probe kernel.
#include "common.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace tsb {

namespace {
constexpr int kMaxDevices = 64;
int* g_status[kMaxDevices] = {nullptr};
int g_sm_count[kMaxDevices] = {0};
std::mutex g_mu;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
int g_last_encode_result = 0;

EncodeTiledFn resolve_encode() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || fn == nullptr) {
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

int* device_status_word() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

int read_and_clear_status(cudaStream_t stream) {
  int* p = device_status_word();
  if (!p) return -1;
  int h = 0;
  if (cudaMemcpyAsync(&h, p, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  if (h != 0) cudaMemsetAsync(p, 0, sizeof(int), stream);
  return h;
}

int sm_count() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sm_count[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    g_sm_count[dev] = n > 0 ? n : 148;
  }
  return g_sm_count[dev];
}

bool pdl_all_enabled() {
  static const bool on = [] {
    const char* e = getenv("TESSERACT_PDL_ALL");
    return e == nullptr || atoi(e) != 0;
  }();
  return on;
}

bool make_tmap_nd(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                  const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  EncodeTiledFn enc = resolve_encode();
  if (!enc) return false;
  // The driver call needs a current context. A thread that has only ever been handed work by another
  // runtime instance (e.g. an autograd worker) may not have bound one yet; a runtime call binds it.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  CUtensorMapDataType dt;
  switch (elem_bytes) {
    case 1: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case 2: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case 4: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return false;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstride[4];
  cuuint32_t bdim[5];
  cuuint32_t estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) gstride[i - 1] = strides_bytes[i];
  }
  g_last_encode_result = 0;
  CUresult r = enc(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstride, bdim, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_encode_result = static_cast<int>(r);
    if (getenv("TESSERACT_DEBUG")) {
      fprintf(stderr, "[tesseract_b200] cuTensorMapEncodeTiled failed: result=%d base=%p elem=%d rank=%d", (int)r,
              base, elem_bytes, rank);
      for (int i = 0; i < rank; ++i)
        fprintf(stderr, " dim%d=%llu box%d=%u stride%d=%llu", i, (unsigned long long)dims[i], i, box[i], i,
                (unsigned long long)(i ? strides_bytes[i] : (uint64_t)elem_bytes));
      fprintf(stderr, "\n");
    }
  }
  return r == CUDA_SUCCESS;
}

bool make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                  uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[2] = {static_cast<uint64_t>(elem_bytes), row_stride_bytes};
  uint32_t box[2] = {box_cols, box_rows};
  return make_tmap_nd(out, base, elem_bytes, 2, dims, strides, box, swizzle128);
}

__global__ void probe_kernel(int* out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *out = 100;
}

}  // namespace tsb

// Returns the first non-zero code recorded by a bounded wait on the current device since the last
// call (0 = none), synchronising `stream`. -1 if the status word could not be read.
TSB_EXPORT int tsb_read_status(void* stream) {
  return tsb::read_and_clear_status(static_cast<cudaStream_t>(stream));
}

// CUresult of the most recent failed tensor-map encoding (0 if the last one succeeded).
TSB_EXPORT int tsb_last_tmap_error() { return tsb::g_last_encode_result; }

TSB_EXPORT int tsb_sm_count() { return tsb::sm_count(); }

// Launches a one-thread kernel that writes 100 into *out (int32, device memory): proves that
// sm_100a device code in this library loads and runs. Returns the cudaError_t of the launch.
TSB_EXPORT int tsb_probe(int* out, void* stream) {
  tsb::probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(out);
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT const char* tsb_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }
