// Split-K GEMM for decode-shaped calls, reduced inside a thread-block cluster through distributed shared memory.
//
//   C[M, N] (bf16) = A[M, K] * B[N, K]^T,   few rows (one or two 128-row blocks), a weight matrix that is streamed once.
//
// A plain tiling of such a problem has fewer tiles than SMs, and a split-K that adds fp32 partial sums into global
// memory pays a zero fill, S atomic passes and a cast over the [M, N] output -- at 256 rows that traffic is as large
// as the weight matrix itself. Here the S CTAs that share an output tile form one cluster: every CTA multiplies
// its K slice (TMA -> 128-byte-swizzled ring -> tcgen05.mma, accumulator in TMEM), parks the fp32 partial tile in its
// own shared memory (the operand ring is idle by then), the cluster synchronises, and CTA r sums the r-th column
// slice of all S partial tiles with ld.shared::cluster and writes bf16 -- nothing but the final output touches
// global memory. No TMA multicast is used; clusters serve only the reduction.
// One tile per CTA (not persistent): grid = tiles * S, cluster = (S, 1, 1), S in {1, 2, 4, 8}.
#include "common.cuh"

namespace tsb {
namespace {

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kStages = 6;
constexpr int kStageBytes = (BM + BN) * BK * 2;             // 32 KB
constexpr int kPartRow = BN * 4 + 16;                       // fp32 partial row, padded against bank conflicts
constexpr int kPartBytes = BM * kPartRow;                   // 67.6 KB, aliases the operand ring
constexpr int kSmemBytes = kStages * kStageBytes + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

template <int S>
__global__ void __launch_bounds__(kThreads, 1)
gemm_cluster_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           __nv_bfloat16* __restrict__ C, int M, int N, int K, long long ldc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = static_cast<int>(cluster_ctarank());   // == blockIdx.x % S
  const int tile = static_cast<int>(blockIdx.x) / S;
  const int num_n = (N + BN - 1) / BN;
  const int m0 = (tile / num_n) * BM;
  const int n0 = (tile % num_n) * BN;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_per = (total_kb + S - 1) / S;
  const int kb0 = slice * kb_per;
  const int kb1 = min(total_kb, kb0 + kb_per);
  const bool have_work = kb1 > kb0;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status)) break;
        uint8_t* sA = smem + stage * kStageBytes;
        uint8_t* sB = sA + BM * BK * 2;
        mbar_expect_tx(&full_bar[stage], kStageBytes);
        tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
        tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(smem + stage * kStageBytes);
        const uint32_t b_base = a_base + BM * BK * 2;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_f16(tmem_base, umma_smem_desc_sw128(a_base + k * 32, 16, 1024), umma_smem_desc_sw128(b_base + k * 32, 16, 1024),
                   idesc, (kb > kb0 || k != 0) ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      umma_commit(&acc_bar);  // arrives when every MMA above has finished (at once if there were none)
    }
  } else {
    // epilogue warps, part 1: TMEM -> fp32 partial tile in this CTA's shared memory (the ring is idle now)
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = mbar_wait(&acc_bar, 0, &cta_abort, status);
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    tc_fence_after();
    uint8_t* prow = smem + row * kPartRow;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      if (warp_ok && have_work) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c * 32), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<uint4*>(prow + (c * 32 + i) * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    }
    tc_fence_before();
  }

  // every thread of every CTA of the cluster: the partial tiles are complete and visible cluster-wide
  __syncthreads();
  cluster_sync_all();

  if (warp >= 2) {
    // part 2: this CTA owns the columns [slice * BN / S, (slice + 1) * BN / S) of the tile
    constexpr int kCols = BN / S;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int grow = m0 + row;
    const uint32_t local = smem_u32(smem + row * kPartRow + slice * kCols * 4);
    float acc[kCols];
#pragma unroll
    for (int i = 0; i < kCols; ++i) acc[i] = 0.f;
#pragma unroll
    for (int r = 0; r < S; ++r) {
      const uint32_t remote = map_to_cta(local, static_cast<uint32_t>(r));
#pragma unroll
      for (int i = 0; i < kCols; i += 4) {
        const float4 v = ld_cluster_f4(remote + i * 4);
        acc[i] += v.x;
        acc[i + 1] += v.y;
        acc[i + 2] += v.z;
        acc[i + 3] += v.w;
      }
    }
    if (grow < M) {
      __nv_bfloat16* crow = C + static_cast<long long>(grow) * ldc;
      const int col0 = n0 + slice * kCols;
      const bool vec = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll
      for (int i = 0; i < kCols; i += 8) {
        if (vec && col0 + i + 8 <= N) {
          uint4 o;
          o.x = pack_bf16x2(acc[i], acc[i + 1]);
          o.y = pack_bf16x2(acc[i + 2], acc[i + 3]);
          o.z = pack_bf16x2(acc[i + 4], acc[i + 5]);
          o.w = pack_bf16x2(acc[i + 6], acc[i + 7]);
          *reinterpret_cast<uint4*>(crow + col0 + i) = o;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (col0 + i + j < N) crow[col0 + i + j] = __float2bfloat16(acc[i + j]);
        }
      }
    }
  }

  // nobody leaves (and frees its shared memory) before every CTA of the cluster has finished reading
  cluster_sync_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, BN);
  }
}

template <int S>
int launch_ck(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, cudaStream_t s) {
  auto kern = gemm_cluster_splitk_kernel<S>;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * S), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, tb, static_cast<__nv_bfloat16*>(C), M, N, K, ldc,
                                             device_status_word()));
}

}  // namespace
}  // namespace tsb

// C [M, N] bf16 (row stride ldc) = A [M, K] (lda) * B [N, K]^T (ldb), K cut into `split` slices (1, 2, 4 or 8) that
// are reduced through the shared memory of a thread-block cluster. Rows 16-byte aligned, lda / ldb multiples of 8.
TSB_EXPORT int tsb_gemm_cluster_splitk(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                                       long long ldb, long long ldc, int split, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8)) return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, A, 2, M, K, lda * 2, BM, BK, true)) return -3;
  if (!make_tmap_2d(&tb, B, 2, N, K, ldb * 2, BN, BK, true)) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (split) {
    case 1: return launch_ck<1>(ta, tb, C, M, N, K, ldc, s);
    case 2: return launch_ck<2>(ta, tb, C, M, N, K, ldc, s);
    case 4: return launch_ck<4>(ta, tb, C, M, N, K, ldc, s);
    case 8: return launch_ck<8>(ta, tb, C, M, N, K, ldc, s);
    default: return -2;
  }
}
