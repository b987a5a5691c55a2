// Block-scaled FP8 (E4M3) GEMM on tcgen05 and its quantisers.
//
//   C[M, N] (bf16) = sum over 128-wide K blocks kb of  sa[kb, m] * sb[n / 128, kb] * (A8[m, kb] . B8[n, kb])
//
// A8 [M, K] and B8 [N, K] are E4M3 bytes, K-major. Activation scales are per row and 128-wide K block ("1 x 128"),
// stored K-block-major (sa [K / 128][M]) so that a warp reads 32 consecutive floats; weight scales are per
// 128 x 128 block (sb [N / 128][K / 128]).
//
// Kernel: persistent, one CTA per SM, 320 threads. Warp 0 streams 128 x 128-byte operand tiles with TMA into a
// 128-byte-swizzled ring (one stage = one K block = one scale block), warp 1 issues four
// tcgen05.mma.kind::f8f6f4 (128 x 128 x 32) per stage into one of four TMEM buffers and commits, warps 2..9 read the
// finished block product with tcgen05.ld, multiply by the block's scale and add it into fp32 registers (64 per
// thread: a thread owns half an output row of the tile; warps 2..5 take columns 0..63, warps 6..9 columns 64..127)
// while the tensor core already works on the next K blocks.
// After the last K block the row is converted to bf16 and stored. All waits are bounded (mbar_wait).
// Replaces the reference's per-tensor-scale cuBLASLt FP8 path (src/cuda/Fp8MatMul.cu:93-157) and its
// f32 -> e4m3 conversion kernel (src/cuda/Fp8MatMul.cu:34-41).
#include "common.cuh"

#include <cuda_fp8.h>

namespace tsb {
namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BKB = 128;  // bytes (= fp8 elements) of K per stage: one scale block
constexpr int kStages = 6;
constexpr int kStageBytes = (BM + BN) * BKB;  // 32 KB
constexpr int kSmemBytes = kStages * kStageBytes + 1024;
constexpr int kThreads = 320;   // TMA warp, MMA warp, eight promotion / epilogue warps
constexpr int kAccBufs = 4;     // block products in flight in TMEM
constexpr int kTmemCols = kAccBufs * BN;
constexpr float kE4M3Max = 448.f;

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                __nv_bfloat16* __restrict__ C, const float* __restrict__ sa, const float* __restrict__ sb, int M, int N,
                int K, long long ldc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[kAccBufs];
  __shared__ __align__(8) uint64_t tmem_empty_bar[kAccBufs];
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = K / BKB;  // host guarantees K % 128 == 0

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  auto tile_mn = [&](int t, int& m0, int& n0) {  // 16 row blocks per group, n fastest inside a group's columns
    constexpr int GM = 16;
    const int group_size = GM * num_n;
    const int gid = t / group_size;
    const int first_m = gid * GM;
    const int gm = min(num_m - first_m, GM);
    const int r = t - gid * group_size;
    m0 = (first_m + r % gm) * BM;
    n0 = (r / gm) * BN;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int m0, n0;
        tile_mn(t, m0, n0);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * kStageBytes;
          uint8_t* sB = sA + BM * BKB;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BKB, m0);
          tma_load_2d(sB, &tmB, &full_bar[stage], kb * BKB, n0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 0, 0, 0, 0);  // e4m3 x e4m3, both K-major, fp32 accumulate
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
          const uint32_t a_base = smem_u32(smem + stage * kStageBytes);
          const uint32_t b_base = a_base + BM * BKB;
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f8(d_tmem, adesc, bdesc, idesc, k != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);      // the stage may be refilled once these MMAs have read it
          umma_commit(&tmem_full_bar[acc]);    // the block product is complete
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++acc == kAccBufs) {
            acc = 0;
            acc_phase ^= 1u;
          }
        }
      }
    }
  } else {
    constexpr int HN = BN / 2;          // columns per promotion warp
    const int q = warp & 3;             // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;   // 0: columns [0, 64), 1: columns [64, 128) of the tile
    const int row_in_tile = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0;
      tile_mn(t, m0, n0);
      const int row = m0 + row_in_tile;
      const int srow = min(row, M - 1);
      float accum[HN];
#pragma unroll
      for (int j = 0; j < HN; ++j) accum[j] = 0.f;
      for (int kb = 0; kb < num_kb; ++kb) {
        const float scale = __ldg(sa + static_cast<long long>(kb) * M + srow) * __ldg(sb + static_cast<long long>(n0 / 128) * num_kb + kb);
        ok = mbar_wait(&tmem_full_bar[acc], acc_phase, &cta_abort, status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        {
          uint32_t r0[32], r1[32];  // both loads in flight before the single wait
          const uint32_t t0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN + half * HN);
          tmem_ld_32x32(t0, r0);
          tmem_ld_32x32(t0 + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) accum[j] = fmaf(scale, __uint_as_float(r0[j]), accum[j]);
#pragma unroll
          for (int j = 0; j < 32; ++j) accum[32 + j] = fmaf(scale, __uint_as_float(r1[j]), accum[32 + j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) break;
      if (row < M) {
        __nv_bfloat16* crow = C + static_cast<long long>(row) * ldc + n0 + half * HN;
        const bool vec = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll
        for (int v = 0; v < HN / 8; ++v) {
          const int col = n0 + half * HN + v * 8;
          if (vec && col + 8 <= N) {
            uint4 o;
            o.x = pack_bf16x2(accum[v * 8 + 0], accum[v * 8 + 1]);
            o.y = pack_bf16x2(accum[v * 8 + 2], accum[v * 8 + 3]);
            o.z = pack_bf16x2(accum[v * 8 + 4], accum[v * 8 + 5]);
            o.w = pack_bf16x2(accum[v * 8 + 6], accum[v * 8 + 7]);
            reinterpret_cast<uint4*>(crow)[v] = o;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col + j < N) crow[v * 8 + j] = __float2bfloat16(accum[v * 8 + j]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Per-tensor-scaled variant: C = (sa * sb) * A8 * B8^T with ONE scale per operand (the reference's FP8 contract,
// src/cuda/Fp8MatMul.cu:93-157). The whole K range accumulates in TMEM, so the kernel has the shape of the bf16
// GEMM -- 128 x 256 tiles, accumulator double-buffered across tiles, epilogue once per tile -- with 128 K bytes per
// stage and kind::f8f6f4 instructions: half the operand bytes per FLOP of the bf16 kernel.
// The tile width PBN is 256 for problems that fill the GPU and 128 / 64 for small ones (a 1024^3 product has only 32
// tiles of 128 x 256 for 148 SMs).
constexpr int kPStages = 4;
constexpr int kPThreads = 192;
template <int PBN>
struct PtCfg {
  static constexpr int kStageBytes = (BM + PBN) * BKB;  // 48 KB at PBN = 256
  static constexpr int kSmemBytes = kPStages * kStageBytes + 1024;
};

template <int PBN>
__global__ void __launch_bounds__(kPThreads, 1)
gemm_fp8_pt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   __nv_bfloat16* __restrict__ C, const float* __restrict__ scale_a, const float* __restrict__ scale_b,
                   int M, int N, int K, long long ldc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kPStages];
  __shared__ __align__(8) uint64_t empty_bar[kPStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + PBN - 1) / PBN;
  const int num_tiles = num_m * num_n;
  const int num_kb = K / BKB;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full_bar[a], 1);
      mbar_init(&tmem_empty_bar[a], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, 2 * PBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  auto tile_mn = [&](int t, int& m0, int& n0) {
    constexpr int GM = 16;
    const int group_size = GM * num_n;
    const int gid = t / group_size;
    const int first_m = gid * GM;
    const int gm = min(num_m - first_m, GM);
    const int r = t - gid * group_size;
    m0 = (first_m + r % gm) * BM;
    n0 = (r / gm) * PBN;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int m0, n0;
        tile_mn(t, m0, n0);
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * PtCfg<PBN>::kStageBytes;
          uint8_t* sB = sA + BM * BKB;
          mbar_expect_tx(&full_bar[stage], PtCfg<PBN>::kStageBytes);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BKB, m0);
          tma_load_2d(sB, &tmB, &full_bar[stage], kb * BKB, n0);
          if (++stage == kPStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, PBN, 0, 0, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        bool ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, &cta_abort, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * PBN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * PtCfg<PBN>::kStageBytes);
          const uint32_t b_base = a_base + BM * BKB;
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k)
            umma_f8(d_tmem, umma_smem_desc_sw128(a_base + k * 32, 16, 1024), umma_smem_desc_sw128(b_base + k * 32, 16, 1024),
                    idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kPStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tmem_full_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const float scale = __ldg(scale_a) * __ldg(scale_b);
    const bool vec = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int m0, n0;
      tile_mn(t, m0, n0);
      const bool ok = mbar_wait(&tmem_full_bar[acc], acc_phase, &cta_abort, status);
      if (!__all_sync(0xffffffffu, ok ? 1 : 0)) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      __nv_bfloat16* crow = C + static_cast<long long>(row) * ldc;
#pragma unroll 1
      for (int c = 0; c < PBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * PBN + c * 32), r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (vec && col0 + v * 8 + 8 <= N) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]) * scale, __uint_as_float(r[v * 8 + 1]) * scale);
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]) * scale, __uint_as_float(r[v * 8 + 3]) * scale);
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]) * scale, __uint_as_float(r[v * 8 + 5]) * scale);
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]) * scale, __uint_as_float(r[v * 8 + 7]) * scale);
              *reinterpret_cast<uint4*>(crow + col0 + v * 8) = o;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col0 + v * 8 + j < N) crow[col0 + v * 8 + j] = __float2bfloat16(__uint_as_float(r[v * 8 + j]) * scale);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * PBN);
  }
}

// One CTA per 1024 elements: q = e4m3(x / scale) with a given per-tensor scale.
template <typename T>
__global__ void __launch_bounds__(256)
quant_tensor_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, const float* __restrict__ scale, long long n);

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

template <typename T>
__global__ void __launch_bounds__(256)
quant_tensor_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, const float* __restrict__ scale, long long n) {
  const float inv = 1.f / __ldg(scale);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    q[i] = to_e4m3(to_f32<T>(x[i]) * inv);
}

// One warp per (row, 128-wide K block): absmax -> scale = absmax / 448 (1 if the block is zero) -> e4m3 bytes.
template <typename T>
__global__ void __launch_bounds__(256)
quant_act_1x128_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales, int M, int K,
                       long long ldx) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int nkb = K / 128;
  if (w >= static_cast<long long>(M) * nkb) return;
  const int row = static_cast<int>(w / nkb), kb = static_cast<int>(w % nkb);
  const T* src = x + static_cast<long long>(row) * ldx + kb * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = to_f32<T>(src[j]);
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / kE4M3Max : 1.f;
  const float inv = 1.f / scale;
  uchar4 o;
  o.x = to_e4m3(v[0] * inv);
  o.y = to_e4m3(v[1] * inv);
  o.z = to_e4m3(v[2] * inv);
  o.w = to_e4m3(v[3] * inv);
  reinterpret_cast<uchar4*>(q + static_cast<long long>(row) * K + kb * 128)[lane] = o;
  if (lane == 0) scales[static_cast<long long>(kb) * M + row] = scale;
}

// One CTA (256 threads) per 128 x 128 weight block.
template <typename T>
__global__ void __launch_bounds__(256)
quant_weight_128x128_kernel(const T* __restrict__ w, uint8_t* __restrict__ q, float* __restrict__ scales, int N, int K,
                            long long ldw) {
  __shared__ float red[8];
  const int nb = blockIdx.y, kb = blockIdx.x;
  const int nkb = K / 128;
  float amax = 0.f;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = nb * 128 + i / 128, c = kb * 128 + i % 128;
    if (r < N) amax = fmaxf(amax, fabsf(to_f32<T>(w[static_cast<long long>(r) * ldw + c])));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax > 0.f ? amax / kE4M3Max : 1.f;
  const float inv = 1.f / scale;
  for (int i = threadIdx.x; i < 128 * 128; i += 256) {
    const int r = nb * 128 + i / 128, c = kb * 128 + i % 128;
    if (r < N) q[static_cast<long long>(r) * K + c] = to_e4m3(to_f32<T>(w[static_cast<long long>(r) * ldw + c]) * inv);
  }
  if (threadIdx.x == 0) scales[static_cast<long long>(nb) * nkb + kb] = scale;
}

}  // namespace
}  // namespace tsb

// C [M, N] bf16 (row stride ldc) = block-scaled A8 [M, K] x B8 [N, K]^T; sa fp32 [K / 128][M], sb fp32 [ceil(N / 128)][K / 128].
// K % 128 == 0; A8 and B8 contiguous rows of K bytes, 16-byte aligned. Returns 0, a cudaError_t, -2 or -3.
TSB_EXPORT int tsb_gemm_fp8_blockscaled(const void* A8, const void* B8, void* C, const float* sa, const float* sb, int M,
                                        int N, int K, long long ldc, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || K % 128 || !sa || !sb) return -2;
  if ((reinterpret_cast<uintptr_t>(A8) & 15) || (reinterpret_cast<uintptr_t>(B8) & 15)) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A8, 1, M, K, static_cast<uint64_t>(K), BM, BKB, true)) return -3;
  if (!make_tmap_2d(&tb, B8, 1, N, K, static_cast<uint64_t>(K), BN, BKB, true)) return -3;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  gemm_fp8_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(
      ta, tb, static_cast<__nv_bfloat16*>(C), sa, sb, M, N, K, ldc, device_status_word());
  return static_cast<int>(cudaGetLastError());
}

// x [M, K] (fp32 / bf16 / fp16, row stride ldx) -> q e4m3 [M, K], scales fp32 [K / 128][M]. K % 128 == 0.
TSB_EXPORT int tsb_quant_act_1x128(const void* x, void* q, float* scales, int M, int K, long long ldx, int dtype,
                                   void* stream) {
  using namespace tsb;
  if (M <= 0 || K <= 0 || K % 128) return -2;
  const long long warps = static_cast<long long>(M) * (K / 128);
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* qo = static_cast<uint8_t*>(q);
  switch (dtype) {
    case 0: quant_act_1x128_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), qo, scales, M, K, ldx); break;
    case 1: quant_act_1x128_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), qo, scales, M, K, ldx); break;
    case 2: quant_act_1x128_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(x), qo, scales, M, K, ldx); break;
    default: return -2;
  }
  return static_cast<int>(cudaGetLastError());
}

// w [N, K] (row stride ldw) -> q e4m3 [N, K], scales fp32 [ceil(N / 128)][K / 128]. K % 128 == 0.
TSB_EXPORT int tsb_quant_weight_128x128(const void* w, void* q, float* scales, int N, int K, long long ldw, int dtype,
                                        void* stream) {
  using namespace tsb;
  if (N <= 0 || K <= 0 || K % 128) return -2;
  const dim3 grid(K / 128, (N + 127) / 128);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* qo = static_cast<uint8_t*>(q);
  switch (dtype) {
    case 0: quant_weight_128x128_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(w), qo, scales, N, K, ldw); break;
    case 1: quant_weight_128x128_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(w), qo, scales, N, K, ldw); break;
    case 2: quant_weight_128x128_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(w), qo, scales, N, K, ldw); break;
    default: return -2;
  }
  return static_cast<int>(cudaGetLastError());
}

// C [M, N] bf16 = (scale_a * scale_b) * A8 [M, K] * B8 [N, K]^T with one fp32 scale per operand (device scalars).
// K % 128 == 0; operands contiguous rows of K bytes, 16-byte aligned.
TSB_EXPORT int tsb_gemm_fp8_pertensor(const void* A8, const void* B8, void* C, const float* scale_a, const float* scale_b,
                                      int M, int N, int K, long long ldc, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || K % 128 || !scale_a || !scale_b) return -2;
  if ((reinterpret_cast<uintptr_t>(A8) & 15) || (reinterpret_cast<uintptr_t>(B8) & 15)) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A8, 1, M, K, static_cast<uint64_t>(K), BM, BKB, true)) return -3;
  const int num_m = (M + BM - 1) / BM;
  auto tiles_at = [&](int bn) { return num_m * ((N + bn - 1) / bn); };
  const int sms = sm_count();
  // the widest tile that still gives at least half the SMs a tile each
  const int bn = 2 * tiles_at(256) >= sms ? 256 : (2 * tiles_at(128) >= sms ? 128 : 64);
  if (!make_tmap_2d(&tb, B8, 1, N, K, static_cast<uint64_t>(K), bn, BKB, true)) return -3;
  auto launch = [&](auto kernel, int smem_bytes, PerDeviceFlag& attr) -> int {
    if (attr.unset()) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
      if (e != cudaSuccess) return static_cast<int>(e);
      attr.set();
    }
    int grid = tiles_at(bn) < sms ? tiles_at(bn) : sms;
    kernel<<<grid, kPThreads, smem_bytes, static_cast<cudaStream_t>(stream)>>>(
        ta, tb, static_cast<__nv_bfloat16*>(C), scale_a, scale_b, M, N, K, ldc, device_status_word());
    return static_cast<int>(cudaGetLastError());
  };
  static PerDeviceFlag attr256, attr128, attr64;
  if (bn == 256) return launch(gemm_fp8_pt_kernel<256>, PtCfg<256>::kSmemBytes, attr256);
  if (bn == 128) return launch(gemm_fp8_pt_kernel<128>, PtCfg<128>::kSmemBytes, attr128);
  return launch(gemm_fp8_pt_kernel<64>, PtCfg<64>::kSmemBytes, attr64);
}

// q [n] e4m3 = x [n] / *scale (device scalar), saturating. dtype: 0 fp32, 1 bf16, 2 fp16.
TSB_EXPORT int tsb_quant_tensor_e4m3(const void* x, void* q, const float* scale, long long n, int dtype, void* stream) {
  using namespace tsb;
  if (n <= 0 || !scale) return -2;
  long long blocks = (n + 1023) / 1024;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* qo = static_cast<uint8_t*>(q);
  switch (dtype) {
    case 0: quant_tensor_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const float*>(x), qo, scale, n); break;
    case 1: quant_tensor_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), qo, scale, n); break;
    case 2: quant_tensor_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, s>>>(static_cast<const __half*>(x), qo, scale, n); break;
    default: return -2;
  }
  return static_cast<int>(cudaGetLastError());
}
