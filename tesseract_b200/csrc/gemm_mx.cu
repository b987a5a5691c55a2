// Block-scaled fp8 GEMM for prompt- and training-sized M on the tensor core's own block scaling:
//   C[M, N] (bf16) = Aq[M, K] (E4M3, one power-of-two scale per row and 32 columns) * W[N, K]^T (E4M3, one
//   power-of-two scale per 128 x 128 block),  tcgen05.mma kind::mxf8f6f4.block_scale, fp32 accumulators in TMEM.
//
// The sibling kernel gemm_fp8.cu keeps exact fp32 scales and therefore has to pull every 128-deep partial product out
// of tensor memory, scale it in registers and add it up there; that caps it below the bf16 GEMM. With power-of-two
// scales the multiply-accumulate over the whole K range stays in TMEM and the kernel is the bf16 pipeline on half the
// operand bytes with twice the MMA rate.
//
// Persistent, warp-specialised, one CTA per SM, 192 threads:
//   warp 0      TMA producer: per stage a 128 x 128-byte tile of Aq, a 192 x 128-byte tile of W and the stage's scale
//               bytes (one 512-byte atom for the 128 activation rows, two for the 256 weight rows around the tile) into
//               a 5-stage ring
//   warp 1      allocates TMEM; one thread copies the stage's scales from shared to tensor memory (tcgen05.cp
//               32x128b.warpx4: 32 rows of 16 bytes become 4 columns, replicated in the four lane quadrants) and issues
//               four K = 32 MMAs; copies and MMAs execute in issue order, so one set of scale columns serves every stage
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (double-buffered, 2 x 192 columns), bf16, store
// Scale atoms (global and shared memory): 128 rows x 4 K blocks as 512 bytes, byte r % 32 * 16 + r / 32 * 4 + j for row
// r and K block j -- the layout tcgen05.cp turns into "lane r % 32, column r / 32, byte j". A tile of 192 columns
// starts on a multiple of 64 rows of W: the two atoms from the 128-row boundary below it are loaded and the MMA reads
// its B scales from column offset 0 or 2. All waits are bounded (common.cuh).
//
// A first version wrote the scales into tensor memory from four extra warps with tcgen05.st behind the stage barriers;
// it was correct and ran at 1100 TFLOP/s (8192^3), below the bf16 GEMM: every stage paid a cross-warp round trip.
//
// The reference's fp8 GEMM is one scale per tensor through cuBLASLt (src/cuda/Fp8MatMul.cu:93-157).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;           // bytes = E4M3 elements per stage
constexpr int BN = 192;
constexpr int kStages = 5;
constexpr int kThreads = 192;
constexpr int kAtom = 512;        // bytes of one scale atom (128 rows x 4 K blocks)

constexpr int kStageA = BM * BK;                 // 16 KB
constexpr int kStageB = BN * BK;                 // 24 KB
constexpr int kStageSf = 3 * kAtom;              // activation atom, two weight atoms
constexpr int kStage = kStageA + kStageB + 2048; // scale bytes in their own 2 KB: the operand tiles stay 1024-aligned
constexpr int kSmem = kStages * kStage + 1024;
constexpr int kTmemCols = 512;
constexpr int kSfaCol = 2 * BN;                  // 4 columns: scales of the 128 activation rows
constexpr int kSfbCol = 2 * BN + 4;              // 8 columns: scales of the 256 weight rows around the tile

struct Tile {
  int m_blk, n_blk;
};
__device__ __forceinline__ Tile tile_of(int t, int num_m, int num_n) {
  constexpr int GM = 16;          // 16 row blocks per group: the tiles in flight stay compact in (m, n) for L2 reuse
  const int group_size = GM * num_n;
  const int group_id = t / group_size;
  const int first_m = group_id * GM;
  const int gm = min(num_m - first_m, GM);
  const int r = t - group_id * group_size;
  return {first_m + r % gm, r / gm};
}

__device__ __forceinline__ uint32_t mx_idesc(uint32_t n, uint32_t sf_id) {
  return (sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf_id << 29);
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// Shared-memory descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, K-major, no swizzle; 8-row core
// matrices are 128 bytes apart (stride byte offset); the leading byte offset is not used by a 16-byte-wide source.
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
  return d;
}
__device__ __forceinline__ void tmem_cp_32x128b_x4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, __nv_bfloat16* __restrict__ C, int M,
               int N, int K, long long ldc, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ __align__(8) uint64_t tmem_full_bar[2], tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int nkb = K / BK;
  const int n_atoms = (N + 127) / 128;            // weight scale atoms per K block

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kStages; ++s) {
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
    tmem_alloc(&tmem_base_smem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tc = tile_of(t, num_m, num_n);
        const int m0 = tc.m_blk * BM, n0 = tc.n_blk * BN;
        const int atom0 = n0 >> 7;                               // weight atom that holds the tile's first row
        const int atom1 = min(atom0 + 1, n_atoms - 1);
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * kStage;
          uint8_t* sB = sA + kStageA;
          uint8_t* sS = sB + kStageB;
          mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(kStageA + kStageB + kStageSf));
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);
          bulk_load(sS, sfa + (static_cast<long long>(tc.m_blk) * nkb + kb) * kAtom, kAtom, &full_bar[stage]);
          bulk_load(sS + kAtom, sfb + (static_cast<long long>(atom0) * nkb + kb) * kAtom, kAtom, &full_bar[stage]);
          bulk_load(sS + 2 * kAtom, sfb + (static_cast<long long>(atom1) * nkb + kb) * kAtom, kAtom, &full_bar[stage]);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tc = tile_of(t, num_m, num_n);
        const int n0 = tc.n_blk * BN;
        ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, &cta_abort, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        const uint32_t sfa_t = tmem_base + kSfaCol;
        const uint32_t sfb_t = tmem_base + kSfbCol;
        const uint32_t sfb_read = sfb_t + static_cast<uint32_t>((n0 & 127) >> 5);   // 0 or 2: the tile starts 0 / 64 rows in
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * kStage);
          const uint32_t b_base = a_base + kStageA;
          const uint32_t s_base = b_base + kStageB;
          tmem_cp_32x128b_x4(sfa_t, sf_smem_desc(s_base));
          tmem_cp_32x128b_x4(sfb_t, sf_smem_desc(s_base + kAtom));
          tmem_cp_32x128b_x4(sfb_t + 4, sf_smem_desc(s_base + 2 * kAtom));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8(d_tmem, umma_smem_desc_sw128(a_base + k * 32, 16, 1024),
                      umma_smem_desc_sw128(b_base + k * 32, 16, 1024), mx_idesc(BN, k), sfa_t, sfb_read,
                      (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == kStages) {
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
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const bool vec_ok = (ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const Tile tc = tile_of(t, num_m, num_n);
      const int m0 = tc.m_blk * BM, n0 = tc.n_blk * BN;
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, &cta_abort, status)) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      __nv_bfloat16* crow = C + static_cast<long long>(row) * ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN + c * 32), r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < M && col0 < N) {
          if (vec_ok && col0 + 32 <= N) {
            uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              dst[v] = o;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < N) crow[col0 + j] = __float2bfloat16(__uint_as_float(r[j]));
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

  // ------------------------------------------------------------ tear-down
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

// Weight scales fp32 [rows][cols] (powers of two) -> atoms [rows][cols][128] words: every word of atom (r, c) is the
// exponent byte of scale (r, c) four times (all 128 rows and 4 K blocks of a 128 x 128 weight block share one scale).
__global__ void weight_scale_atoms_kernel(const float* __restrict__ w_scale, uint32_t* __restrict__ atoms, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n * 128) return;
  atoms[i] = ((__float_as_uint(w_scale[i >> 7]) >> 23) & 0xffu) * 0x01010101u;
}

}  // namespace
}  // namespace tsb

// atoms: uint32 [ceil(N / 128)][K / 128][128] from w_scale fp32 [ceil(N / 128)][K / 128] (powers of two).
TSB_EXPORT int tsb_mx_weight_scale_atoms(const float* w_scale, void* atoms, int scale_rows, int scale_cols, void* stream) {
  if (!w_scale || !atoms || scale_rows <= 0 || scale_cols <= 0) return -2;
  const long long n = static_cast<long long>(scale_rows) * scale_cols;
  const unsigned blocks = static_cast<unsigned>((n * 128 + 255) / 256);
  tsb::weight_scale_atoms_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w_scale, static_cast<uint32_t*>(atoms), n);
  return static_cast<int>(cudaGetLastError());
}

// C [M, N] bf16 (row stride ldc) = dequant(Aq, sfa) * dequant(W, sfb)^T for any M (meant for M > 256; below that
// tsb_gemm_decode_mx streams the weights once).
//   Aq: E4M3 bytes [M, K], dense rows; sfa: scale atoms [ceil(M / 128)][K / 128][512 bytes] as tsb_quant_act_mx writes
//       them with atoms = 1 (byte r % 32 * 16 + r % 128 / 32 * 4 + j of atom (r / 128, k / 128) = UE8M0 exponent of
//       Aq[r, 128 (k / 128) + 32 j .. + 31]).
//   W: E4M3 bytes [N, K] (row stride ldw bytes, a multiple of 16); sfb: tsb_mx_weight_scale_atoms of its block scales.
//   K % 128 == 0.
TSB_EXPORT int tsb_gemm_mx(const void* Aq, const void* sfa, const void* W, const void* sfb, void* C, int M, int N, int K,
                           long long ldw, long long ldc, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || K % BK || !Aq || !sfa || !W || !sfb || !C) return -2;
  if ((reinterpret_cast<uintptr_t>(Aq) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldw % 16) ||
      (reinterpret_cast<uintptr_t>(sfa) & 15) || (reinterpret_cast<uintptr_t>(sfb) & 15))
    return -2;
  CUtensorMap ta, tb;
  if (!make_tmap_2d(&ta, Aq, 1, M, K, K, BM, BK, true)) return -3;
  if (!make_tmap_2d(&tb, W, 1, N, K, ldw, BN, BK, true)) return -3;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  gemm_mx_kernel<<<grid, kThreads, kSmem, static_cast<cudaStream_t>(stream)>>>(
      ta, tb, static_cast<const uint8_t*>(sfa), static_cast<const uint8_t*>(sfb), static_cast<__nv_bfloat16*>(C), M, N, K,
      ldc, device_status_word());
  return static_cast<int>(cudaGetLastError());
}
