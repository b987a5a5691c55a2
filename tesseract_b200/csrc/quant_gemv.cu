// Weight-only quantised GEMV for decode-shaped calls (M <= 16 rows of activations):
//   y[m, n] = sum_k x[m, k] * dequant(W[n, k])   with INT8 per-row scales or INT4 per-group scales.
// One warp per output row n, 128-bit weight loads (16 int8 or 32 int4 per lane per step), fp32
// accumulation, one shuffle reduction per (m, n). The reference kernel uses one CTA per output ELEMENT
// (grid (N, M), src/cuda/DequantMatMul.cu:95-127,216-258); here every weight byte is read exactly once
// for all M rows. Packing follows include/tesseract/quant/Pack.hpp:40-103: INT8 in [-127, 127] with
// scale[n]; INT4 two's-complement nibbles in [-7, 7], low nibble = even k, scale[n, k / group].
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kGemvWarps = 8;
constexpr int kMaxM = 16;

template <typename T>
__device__ __forceinline__ void load_x16(const T* p, float (&f)[16]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      f[i] = to_f32<T>(pa[i]);
      f[8 + i] = to_f32<T>(pb[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; i += 4) {
      const float4 a = *reinterpret_cast<const float4*>(p + i);
      f[i] = a.x; f[i + 1] = a.y; f[i + 2] = a.z; f[i + 3] = a.w;
    }
  }
}

template <typename T, int MT>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_w8_kernel(const T* __restrict__ x, const int8_t* __restrict__ w, const float* __restrict__ scale,
               const T* __restrict__ bias, T* __restrict__ y, int M, int N, int K) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kGemvWarps + warp;
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  const int8_t* wrow = w + static_cast<long long>(n) * K;
  for (int k = lane * 16; k < K; k += 32 * 16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(wrow + k);
    const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
    float wf[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) wf[i] = static_cast<float>(q[i]);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < M) {
        float xf[16];
        load_x16<T>(x + static_cast<long long>(m) * K + k, xf);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[m] = fmaf(xf[i], wf[i], acc[m]);
      }
    }
  }
  const float s = scale[n];
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < M) {
      float out = v * s;
      if (bias) out += to_f32<T>(bias[n]);
      y[static_cast<long long>(m) * N + n] = from_f32<T>(out);
    }
  }
}

// INT4 group-quantised: each lane handles 32 consecutive k (16 packed bytes) per step; a group never
// straddles a lane's 32 elements because group % 32 == 0.
template <typename T, int MT>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_w4g_kernel(const T* __restrict__ x, const uint8_t* __restrict__ w, const float* __restrict__ scale,
                const T* __restrict__ bias, T* __restrict__ y, int M, int N, int K, int group) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kGemvWarps + warp;
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  const uint8_t* wrow = w + static_cast<long long>(n) * (K / 2);
  const float* srow = scale + static_cast<long long>(n) * (K / group);
  for (int k = lane * 32; k < K; k += 32 * 32) {
    const uint4 raw = *reinterpret_cast<const uint4*>(wrow + k / 2);
    const uint8_t* q = reinterpret_cast<const uint8_t*>(&raw);
    const float gs = srow[k / group];
    float wf[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      int lo = q[i] & 0xF, hi = q[i] >> 4;
      lo = lo > 7 ? lo - 16 : lo;
      hi = hi > 7 ? hi - 16 : hi;
      wf[2 * i] = static_cast<float>(lo) * gs;
      wf[2 * i + 1] = static_cast<float>(hi) * gs;
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < M) {
        float xf[16];
        load_x16<T>(x + static_cast<long long>(m) * K + k, xf);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[m] = fmaf(xf[i], wf[i], acc[m]);
        load_x16<T>(x + static_cast<long long>(m) * K + k + 16, xf);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[m] = fmaf(xf[i], wf[16 + i], acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    const float v = warp_sum(acc[m]);
    if (lane == 0 && m < M) {
      float out = v;
      if (bias) out += to_f32<T>(bias[n]);
      y[static_cast<long long>(m) * N + n] = from_f32<T>(out);
    }
  }
}

// Batches above kMaxM rows: the packed weights are widened to bf16 once per call and the product runs on the tcgen05
// GEMM (the reference dequantises into its library GEMM the same way, src/cuda/DequantMatMul.cu:216-258). One thread
// per 16 packed bytes: 16 INT8 values of one row, or 32 INT4 values of one scale group.
__global__ void __launch_bounds__(256)
dequant_w8_bf16_kernel(const int8_t* __restrict__ w, const float* __restrict__ scale, __nv_bfloat16* __restrict__ out,
                       long long nvec, int K) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
    const long long e0 = i * 16;
    const float s = scale[e0 / K];
    const uint4 raw = *reinterpret_cast<const uint4*>(w + e0);
    const int8_t* q = reinterpret_cast<const int8_t*>(&raw);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = pack_bf16x2(static_cast<float>(q[2 * j]) * s, static_cast<float>(q[2 * j + 1]) * s);
    *reinterpret_cast<uint4*>(out + e0) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(out + e0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

__global__ void __launch_bounds__(256)
dequant_w4g_bf16_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale, __nv_bfloat16* __restrict__ out,
                        long long nvec, int K, int group) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
    const long long e0 = i * 32;                       // 32 values = 16 packed bytes, inside one group (group % 32 == 0)
    const long long row = e0 / K;
    const int k = static_cast<int>(e0 - row * K);
    const float gs = scale[row * (K / group) + k / group];
    const uint4 raw = *reinterpret_cast<const uint4*>(w + e0 / 2);
    const uint8_t* q = reinterpret_cast<const uint8_t*>(&raw);
    uint32_t o[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      int lo = q[j] & 0xF, hi = q[j] >> 4;             // low nibble = even k; two's complement nibbles
      lo = lo > 7 ? lo - 16 : lo;
      hi = hi > 7 ? hi - 16 : hi;
      o[j] = pack_bf16x2(static_cast<float>(lo) * gs, static_cast<float>(hi) * gs);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<uint4*>(out + e0 + 8 * j) = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
  }
}

template <typename T>
int launch_w8(const void* x, const void* w, const float* scale, const void* bias, void* y, int M, int N, int K,
              cudaStream_t s) {
  const int grid = (N + kGemvWarps - 1) / kGemvWarps;
#define TSB_W8(MT)                                                                                                    \
  gemv_w8_kernel<T, MT><<<grid, kGemvWarps * 32, 0, s>>>(static_cast<const T*>(x), static_cast<const int8_t*>(w), scale, \
                                                         static_cast<const T*>(bias), static_cast<T*>(y), M, N, K)
  if (M <= 1) TSB_W8(1);
  else if (M <= 2) TSB_W8(2);
  else if (M <= 4) TSB_W8(4);
  else if (M <= 8) TSB_W8(8);
  else TSB_W8(16);
#undef TSB_W8
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int launch_w4(const void* x, const void* w, const float* scale, const void* bias, void* y, int M, int N, int K,
              int group, cudaStream_t s) {
  const int grid = (N + kGemvWarps - 1) / kGemvWarps;
#define TSB_W4(MT)                                                                                          \
  gemv_w4g_kernel<T, MT><<<grid, kGemvWarps * 32, 0, s>>>(static_cast<const T*>(x), static_cast<const uint8_t*>(w), \
                                                          scale, static_cast<const T*>(bias), static_cast<T*>(y), M, \
                                                          N, K, group)
  if (M <= 1) TSB_W4(1);
  else if (M <= 2) TSB_W4(2);
  else if (M <= 4) TSB_W4(4);
  else if (M <= 8) TSB_W4(8);
  else TSB_W4(16);
#undef TSB_W4
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace tsb

// y [M, N] = x [M, K] @ (q_weight [N, K] int8 * scale [N])^T (+ bias). M <= 16, K % 16 == 0.
// dtype of x / bias / y: 0 = fp32, 1 = bf16, 2 = fp16.
TSB_EXPORT int tsb_gemv_w8(const void* x, const void* q_weight, const float* scale, const void* bias, void* y, int M,
                           int N, int K, int dtype, void* stream) {
  using namespace tsb;
  if (M <= 0 || M > kMaxM || N <= 0 || K <= 0 || K % 16) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0: return launch_w8<float>(x, q_weight, scale, bias, y, M, N, K, s);
    case 1: return launch_w8<__nv_bfloat16>(x, q_weight, scale, bias, y, M, N, K, s);
    case 2: return launch_w8<__half>(x, q_weight, scale, bias, y, M, N, K, s);
    default: return -2;
  }
}

// INT4 group variant: q_weight uint8 [N, K / 2], scale fp32 [N, K / group]; K % 32 == 0, group % 32 == 0.
TSB_EXPORT int tsb_gemv_w4g(const void* x, const void* q_weight, const float* scale, const void* bias, void* y, int M,
                            int N, int K, int group, int dtype, void* stream) {
  using namespace tsb;
  if (M <= 0 || M > kMaxM || N <= 0 || K <= 0 || K % 32 || group <= 0 || group % 32 || K % group) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0: return launch_w4<float>(x, q_weight, scale, bias, y, M, N, K, group, s);
    case 1: return launch_w4<__nv_bfloat16>(x, q_weight, scale, bias, y, M, N, K, group, s);
    case 2: return launch_w4<__half>(x, q_weight, scale, bias, y, M, N, K, group, s);
    default: return -2;
  }
}

// out [N, K] bf16 = q_weight [N, K] int8 * scale[n]. K % 16 == 0; q_weight and out 16-byte aligned.
TSB_EXPORT int tsb_dequant_w8_bf16(const void* q_weight, const float* scale, void* out, long long N, int K, void* stream) {
  using namespace tsb;
  if (N <= 0 || K <= 0 || K % 16 || !q_weight || !scale || !out) return -2;
  if ((reinterpret_cast<uintptr_t>(q_weight) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  const long long nvec = N * K / 16;
  long long blocks = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  dequant_w8_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int8_t*>(q_weight), scale, static_cast<__nv_bfloat16*>(out), nvec, K);
  return static_cast<int>(cudaGetLastError());
}

// out [N, K] bf16 = INT4 nibbles [N, K / 2] * scale[n, k / group]. K % 32 == 0, group % 32 == 0, K % group == 0.
TSB_EXPORT int tsb_dequant_w4g_bf16(const void* q_weight, const float* scale, void* out, long long N, int K, int group,
                                    void* stream) {
  using namespace tsb;
  if (N <= 0 || K <= 0 || K % 32 || group <= 0 || group % 32 || K % group || !q_weight || !scale || !out) return -2;
  if ((reinterpret_cast<uintptr_t>(q_weight) | reinterpret_cast<uintptr_t>(out)) & 15) return -2;
  const long long nvec = N * K / 32;
  long long blocks = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  dequant_w4g_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q_weight), scale, static_cast<__nv_bfloat16*>(out), nvec, K, group);
  return static_cast<int>(cudaGetLastError());
}
