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
