// bf16 GEMM on the 5th-generation tensor cores: C[M,N] (+)= op(A) * op(B), fp32 accumulation in TMEM.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A and B into a 128-byte-swizzled smem ring
//   warp 1      allocates TMEM; one thread issues tcgen05.mma (128 x BN x 16) and tcgen05.commit
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (double-buffered in TMEM), convert, store
// Operands may be K-major (row-major [rows, K]) or M/N-major (row-major [K, rows]); the second form is
// what the backward GEMMs of a Linear layer need (dX = dY * W, dW = dY^T * X) without any transposes.
//
// Replaces the cuBLASLt bridge of the reference (src/cuda/MatMul.cpp:422-490) for every dense
// Linear forward/backward.
#include "common.cuh"

#include <mutex>
#include <type_traits>
#include <unordered_map>

namespace tsb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int kGemmThreads = 192;

template <int BN>
struct GemmCfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : (BN >= 64 ? 8 : 10));
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = (2 * BN < 32) ? 32 : 2 * BN;
};

struct TileCoord {
  int m_blk, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(int t, int num_m, int num_n) {
  constexpr int GM = 16;
  const int group_size = GM * num_n;
  const int group_id = t / group_size;
  const int first_m = group_id * GM;
  const int gm = min(num_m - first_m, GM);
  const int r = t - group_id * group_size;
  return {first_m + r % gm, r / gm};
}

// Grouped GEMMs (MoE experts) run through the same kernel. `offsets` (device, int32 [groups + 1], every entry a
// multiple of 128, so no 128-row block and no 64-row reduction step straddles two groups) is read by the kernel,
// never by the host:
//   mode 1  rows grouped (expert forward / input gradient): row block m belongs to the group g with
//           offsets[g] <= 128 m < offsets[g + 1]; the B tensor map stacks the groups' matrices and its row
//           coordinate advances by b_group_rows per group; row blocks at or beyond offsets[groups] are skipped.
//   mode 2  reduction grouped (expert weight gradient, A and B both MN-major): work item (g, m_blk, n_blk) reduces
//           over rows [offsets[g], offsets[g + 1]) and writes C + g * c_group_stride; an empty group adds nothing.
//   mode 1 with `row_tags` (expert-parallel return path): the result rows do not go to C but straight to the rank
//           each row came from -- row r with tag t >= 0 is stored at peer_out[t >> 24] + (t & 0xFFFFFF) * ldc (peer-mapped
//           memory of that rank, over NVLink), rows with a negative tag (padding) are dropped. The all-to-all that
//           returns expert results is the epilogue of the down projection; nothing is written locally.
struct GroupArgs {
  const int* offsets;
  int groups;
  int mode;
  long long b_group_rows;
  long long c_group_stride;
  const int* row_tags = nullptr;
  long long peer_rows = 0;
  void* peer_out[8] = {};
};

__device__ __forceinline__ int group_of_row(const GroupArgs& g, int row) {
  int e = 0;
  while (e + 1 < g.groups && __ldg(g.offsets + e + 1) <= row) ++e;
  return e;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool ACCUM>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* __restrict__ C,
                 int M, int N, int K, long long ldc, int* status, int split_k, GroupArgs grp) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  // split_k > 1: work item t covers K slice (t % split_k) of output tile (t / split_k); slices are summed with
  // fp32 atomics by the epilogue (ATOMIC_OUT instantiation, C zero-initialised by the caller)
  const int gmode = grp.offsets ? grp.mode : 0;
  const int num_tiles = num_m * num_n * (gmode == 2 ? grp.groups : split_k);
  const int total_kb = (K + BK - 1) / BK;
  const int kb_per = (total_kb + split_k - 1) / split_k;
  const int m_limit = (gmode == 1) ? __ldg(grp.offsets + grp.groups) : M;  // mode 1: rows in use
  const int tiles_per_group = num_m * num_n;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
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
    tmem_alloc(&tmem_base_smem, Cfg::kTmemCols);
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
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const TileCoord tc = (gmode == 2) ? tile_coord(t % tiles_per_group, num_m, num_n) : tile_coord(t / split_k, num_m, num_n);
        const int m0 = tc.m_blk * BM;
        const int n0 = tc.n_blk * BN;
        int kb0 = (t % split_k) * kb_per;
        int kb1 = min(total_kb, kb0 + kb_per);
        int b_row_off = 0;  // rows of the stacked B tensor map before this tile's group
        if (gmode == 1) {
          if (m0 >= m_limit) continue;
          b_row_off = static_cast<int>(group_of_row(grp, m0) * grp.b_group_rows);
        } else if (gmode == 2) {
          const int g = t / tiles_per_group;
          kb0 = __ldg(grp.offsets + g) / BK;
          kb1 = __ldg(grp.offsets + g + 1) / BK;
        }
        bool ok = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + Cfg::kStageBytesA;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sA + i * 8192, &tmA, &full_bar[stage], m0 + i * 64, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0 + b_row_off);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sB + i * 8192, &tmB, &full_bar[stage], n0 + i * 64, kb * BK + b_row_off);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int kb0 = (t % split_k) * kb_per;
        int kb1 = min(total_kb, kb0 + kb_per);
        if (gmode == 1) {
          if (tile_coord(t, num_m, num_n).m_blk * BM >= m_limit) continue;
        } else if (gmode == 2) {
          const int g = t / tiles_per_group;
          kb0 = __ldg(grp.offsets + g) / BK;
          kb1 = __ldg(grp.offsets + g + 1) / BK;
        }
        bool ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, &cta_abort, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_base = a_base + Cfg::kStageBytesA;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc_sw128(a_base + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb > kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tmem_full_bar[acc]);  // accumulator complete
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int row_in_tile = q * 32 + lane;
    const bool vec_ok = (ldc % (16 / sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileCoord tc = (gmode == 2) ? tile_coord(t % tiles_per_group, num_m, num_n) : tile_coord(t / split_k, num_m, num_n);
      const int m0 = tc.m_blk * BM;
      const int n0 = tc.n_blk * BN;
      bool empty_slice = (t % split_k) * kb_per >= total_kb;
      OutT* Cg = C;
      if (gmode == 1) {
        if (m0 >= m_limit) continue;
      } else if (gmode == 2) {
        const int g = t / tiles_per_group;
        empty_slice = __ldg(grp.offsets + g) >= __ldg(grp.offsets + g + 1);
        Cg = C + static_cast<long long>(g) * grp.c_group_stride;
      }
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, &cta_abort, status)) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      OutT* crow = Cg + static_cast<long long>(row) * ldc;
      bool row_ok = row < M;
      if (gmode == 1 && grp.row_tags) {
        const int tag = row_ok ? __ldg(grp.row_tags + row) : -1;
        const long long slot = tag & 0xFFFFFF;
        row_ok = tag >= 0 && slot < grp.peer_rows;
        if (row_ok) {
          const int owner = (tag >> 24) & 7;
          void* base = grp.peer_out[0];      // selected by comparison: a dynamic index would move the array to local memory
#pragma unroll
          for (int r = 1; r < 8; ++r)
            if (owner == r) base = grp.peer_out[r];
          crow = static_cast<OutT*>(base) + slot * ldc;
        }
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN + c * 32), r);
        tmem_ld_wait();
        if (gmode == 2 && empty_slice) {  // a group without rows: nothing was accumulated
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        const int col0 = n0 + c * 32;
        if (row_ok && col0 < N) {
          if (vec_ok && col0 + 32 <= N) {
            if constexpr (sizeof(OutT) == 2) {
              uint4* dst = reinterpret_cast<uint4*>(crow + col0);
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                if constexpr (ACCUM) {
                  const uint4 old = dst[v];
                  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const float2 of = __bfloat1622float2(o2[j]);
                    f[2 * j] += of.x;
                    f[2 * j + 1] += of.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[0], f[1]);
                o.y = pack_bf16x2(f[2], f[3]);
                o.z = pack_bf16x2(f[4], f[5]);
                o.w = pack_bf16x2(f[6], f[7]);
                dst[v] = o;
              }
            } else {
              float4* dst = reinterpret_cast<float4*>(crow + col0);
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                                       __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
                if (split_k > 1) {
                  if (!empty_slice) atomicAdd(&dst[v], o);
                  continue;
                }
                if constexpr (ACCUM) {
                  const float4 old = dst[v];
                  o.x += old.x;
                  o.y += old.y;
                  o.z += old.z;
                  o.w += old.w;
                }
                dst[v] = o;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (col0 + j < N) {
                float v = __uint_as_float(r[j]);
                if constexpr (sizeof(OutT) == 4) {
                  if (split_k > 1) {
                    if (!empty_slice) atomicAdd(reinterpret_cast<float*>(crow) + col0 + j, v);
                    continue;
                  }
                }
                if constexpr (ACCUM) v += to_f32<OutT>(crow[col0 + j]);
                crow[col0 + j] = from_f32<OutT>(v);
              }
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

  // ------------------------------------------------------------ tear-down
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      // Give copies and MMAs that are still in flight a bounded moment to land before TMEM goes away.
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------- tensor-map cache
struct TmapKey {
  const void* p;
  uint64_t rows, cols, stride;
  uint32_t br, bc;
  bool operator==(const TmapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && stride == o.stride && br == o.br && bc == o.bc;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.p) * 0x9E3779B97F4A7C15ull;
    h ^= k.rows * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= k.cols * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    h ^= k.stride + (h << 6) + (h >> 2);
    h ^= (static_cast<size_t>(k.br) << 32 | k.bc) + (h << 6) + (h >> 2);
    return h;
  }
};
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmaps;
std::mutex g_tmap_mu;

bool cached_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t stride_bytes,
                    uint32_t box_rows, uint32_t box_cols) {
  TmapKey key{base, rows, cols, stride_bytes, box_rows, box_cols};
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  auto it = g_tmaps.find(key);
  if (it != g_tmaps.end()) {
    *out = it->second;
    return true;
  }
  if (!make_tmap_2d(out, base, 2, rows, cols, stride_bytes, box_rows, box_cols, true)) return false;
  if (g_tmaps.size() > 8192) g_tmaps.clear();
  g_tmaps.emplace(key, *out);
  return true;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool ACCUM>
int launch_cfg(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int max_ctas,
               cudaStream_t stream, int split_k = 1, GroupArgs grp = GroupArgs{nullptr, 0, 0, 0, 0}) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT, ACCUM>;
  static PerDeviceFlag attr_set;
  if (attr_set.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set.set();
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * ((grp.offsets && grp.mode == 2) ? grp.groups : split_k);
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  if (tiles < grid) grid = tiles;
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(ta, tb, static_cast<OutT*>(C), M, N, K, ldc,
                                                        device_status_word(), split_k, grp);
  return static_cast<int>(cudaGetLastError());
}

template <int BN, bool A_MN, bool B_MN>
int launch_out(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int out_f32,
               int accumulate, int max_ctas, cudaStream_t s) {
  if (out_f32) {
    return accumulate ? launch_cfg<BN, A_MN, B_MN, float, true>(ta, tb, C, M, N, K, ldc, max_ctas, s)
                      : launch_cfg<BN, A_MN, B_MN, float, false>(ta, tb, C, M, N, K, ldc, max_ctas, s);
  }
  return accumulate ? launch_cfg<BN, A_MN, B_MN, __nv_bfloat16, true>(ta, tb, C, M, N, K, ldc, max_ctas, s)
                    : launch_cfg<BN, A_MN, B_MN, __nv_bfloat16, false>(ta, tb, C, M, N, K, ldc, max_ctas, s);
}

template <int BN>
int launch_major(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc, int a_mn,
                 int b_mn, int out_f32, int accumulate, int max_ctas, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_out<BN, false, false>(ta, tb, C, M, N, K, ldc, out_f32, accumulate, max_ctas, s);
  if (!a_mn && b_mn) return launch_out<BN, false, true>(ta, tb, C, M, N, K, ldc, out_f32, accumulate, max_ctas, s);
  if (a_mn && !b_mn) return launch_out<BN, true, false>(ta, tb, C, M, N, K, ldc, out_f32, accumulate, max_ctas, s);
  return launch_out<BN, true, true>(ta, tb, C, M, N, K, ldc, out_f32, accumulate, max_ctas, s);
}

}  // namespace
}  // namespace tsb

// C[M,N] (+)= op(A) * op(B) with bf16 inputs and fp32 accumulation.
//   a_mn == 0: A is row-major [M, K] (row stride lda elements);  a_mn == 1: A is row-major [K, M].
//   b_mn == 0: B is row-major [N, K] (row stride ldb elements);  b_mn == 1: B is row-major [K, N].
//   C is row-major [M, N] with row stride ldc; bf16, or fp32 when out_f32 != 0; accumulate != 0 adds
//   into the existing contents of C.
// Requirements: A and B 16-byte aligned with row strides that are multiples of 8 elements.
// block_n: 0 = choose, else 32 / 64 / 128 / 256. max_ctas: 0 = one CTA per SM, else a cap (used when some SMs are
// reserved for a concurrent communication kernel).
// Returns 0, a cudaError_t, or -2 (bad argument) / -3 (tensor map encoding failed).
TSB_EXPORT int tsb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int out_f32, int accumulate,
                             int block_n, int max_ctas, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8))
    return -2;
  int bn = block_n;
  if (bn == 0) {
    const int sms = sm_count();
    const long long mt = (M + BM - 1) / BM;
    auto tiles = [&](int b) { return mt * ((N + b - 1) / b); };
    // largest tile that still gives every SM work; decode-shaped calls (few rows) stream the weight matrix
    // and want as many CTAs pulling on HBM as possible, so they go down to 32-column tiles
    if (N >= 256 && tiles(256) >= sms) bn = 256;
    else if (N >= 128 && tiles(128) >= sms) bn = 128;
    else if (N >= 64 && tiles(64) >= sms) bn = 64;
    else if (N >= 128 && tiles(128) * 2 >= sms && mt > 2) bn = 128;
    else bn = (N >= 64 && tiles(32) > 2 * sms) ? 64 : 32;
  }
  if (bn == 32 && b_mn) bn = 64;  // an N-major B tile is built from 64-column (128-byte) boxes
  if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return -2;
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn) ok = cached_tmap_2d(&ta, A, M, K, lda * 2, BM, BK);
  else ok = cached_tmap_2d(&ta, A, K, M, lda * 2, BK, 64);
  if (!ok) return -3;
  if (!b_mn) ok = cached_tmap_2d(&tb, B, N, K, ldb * 2, bn, BK);
  else ok = cached_tmap_2d(&tb, B, K, N, ldb * 2, BK, 64);
  if (!ok) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (bn) {
    case 256: return launch_major<256>(ta, tb, C, M, N, K, ldc, a_mn, b_mn, out_f32, accumulate, max_ctas, s);
    case 128: return launch_major<128>(ta, tb, C, M, N, K, ldc, a_mn, b_mn, out_f32, accumulate, max_ctas, s);
    case 64: return launch_major<64>(ta, tb, C, M, N, K, ldc, a_mn, b_mn, out_f32, accumulate, max_ctas, s);
    default: return launch_major<32>(ta, tb, C, M, N, K, ldc, a_mn, b_mn, out_f32, accumulate, max_ctas, s);
  }
}

// Grouped GEMM for mixture-of-experts layers; `offsets` (int32 [groups + 1], multiples of 128) stays on the device.
//   mode 1 (rows grouped):  C[r, :] = A[r, :] * op(B[g(r)])  for the row blocks below offsets[groups].
//       A [rows_cap, K] bf16 (lda), C [rows_cap, N] bf16 (ldc); rows_cap >= offsets[groups] is the allocated height.
//       b_mn = 0: B[g] is [N, K];  b_mn = 1: B[g] is [K, N]  (row stride ldb); B[g] starts b_group_stride elements
//       after B[g - 1] (a multiple of ldb: the groups need not be packed, e.g. expert weights in a flat arena).
//   mode 2 (reduction grouped, expert weight gradient):  C[g] (+)= A[rows of g, :]^T * B[rows of g, :]
//       A [rows_cap, M] bf16 (lda), B [rows_cap, N] bf16 (ldb), C[g] [M, N] fp32 or bf16 (ldc), C[g] starting
//       c_group_stride elements after C[g - 1].
// Returns 0, a cudaError_t, -2 (bad argument) or -3 (tensor map encoding failed).
TSB_EXPORT int tsb_gemm_grouped(const void* A, const void* B, void* C, const int* offsets, int groups, int mode,
                                int rows_cap, int M, int N, int K, long long lda, long long ldb, long long ldc, int b_mn,
                                long long b_group_stride, long long c_group_stride, int out_f32, int accumulate,
                                void* stream) {
  using namespace tsb;
  if (!offsets || groups < 1 || groups > 1024 || rows_cap <= 0 || rows_cap % BM || N <= 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8)) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap ta, tb;
  if (mode == 1) {
    if (K <= 0 || K % 8 || out_f32 || accumulate) return -2;
    if (b_mn && (K % BK)) return -2;  // the stacked [groups * K, N] map must not read across a group boundary
    const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
    if (!cached_tmap_2d(&ta, A, rows_cap, K, lda * 2, BM, BK)) return -3;
    if (b_group_stride <= 0 || b_group_stride % ldb) return -2;
    const long long grows = b_group_stride / ldb;  // rows of the stacked map per group
    if (grows < (b_mn ? K : N)) return -2;
    const uint64_t map_rows = static_cast<uint64_t>(groups - 1) * grows + (b_mn ? K : N);
    const bool ok = b_mn ? cached_tmap_2d(&tb, B, map_rows, N, ldb * 2, BK, 64)
                         : cached_tmap_2d(&tb, B, map_rows, K, ldb * 2, bn, BK);
    if (!ok) return -3;
    GroupArgs g{offsets, groups, 1, grows, 0};
    auto go = [&](auto bn_tag, auto bmn_tag) {
      return launch_cfg<decltype(bn_tag)::value, false, decltype(bmn_tag)::value, __nv_bfloat16, false>(
          ta, tb, C, rows_cap, N, K, ldc, 0, s, 1, g);
    };
    using T = std::true_type;
    using F = std::false_type;
    if (bn == 256) return b_mn ? go(std::integral_constant<int, 256>{}, T{}) : go(std::integral_constant<int, 256>{}, F{});
    if (bn == 128) return b_mn ? go(std::integral_constant<int, 128>{}, T{}) : go(std::integral_constant<int, 128>{}, F{});
    return b_mn ? go(std::integral_constant<int, 64>{}, T{}) : go(std::integral_constant<int, 64>{}, F{});
  }
  if (mode == 2) {
    if (M <= 0 || M % 8 || N % 8) return -2;
    const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
    if (!cached_tmap_2d(&ta, A, rows_cap, M, lda * 2, BK, 64)) return -3;
    if (!cached_tmap_2d(&tb, B, rows_cap, N, ldb * 2, BK, 64)) return -3;
    if (c_group_stride < static_cast<long long>(M - 1) * ldc + N) return -2;
    GroupArgs g{offsets, groups, 2, 0, c_group_stride};
    auto go = [&](auto bn_tag) {
      constexpr int kBn = decltype(bn_tag)::value;
      if (out_f32)
        return accumulate ? launch_cfg<kBn, true, true, float, true>(ta, tb, C, M, N, rows_cap, ldc, 0, s, 1, g)
                          : launch_cfg<kBn, true, true, float, false>(ta, tb, C, M, N, rows_cap, ldc, 0, s, 1, g);
      return accumulate ? launch_cfg<kBn, true, true, __nv_bfloat16, true>(ta, tb, C, M, N, rows_cap, ldc, 0, s, 1, g)
                        : launch_cfg<kBn, true, true, __nv_bfloat16, false>(ta, tb, C, M, N, rows_cap, ldc, 0, s, 1, g);
    };
    if (bn == 256) return go(std::integral_constant<int, 256>{});
    if (bn == 128) return go(std::integral_constant<int, 128>{});
    return go(std::integral_constant<int, 64>{});
  }
  return -2;
}

// Row-grouped GEMM (mode 1 above) whose result rows are scattered to peer-mapped buffers instead of a local C:
// row r goes to peer_out[tags[r] >> 24] + (tags[r] & 0xFFFFFF) * ld_out when tags[r] >= 0 (and the slot is below
// peer_rows), nowhere otherwise. peer_out: `world` (<= 8) device pointers as mapped in this process, 16-byte aligned,
// ld_out % 8 == 0. Plain stores: the caller orders them with its own barrier (e.g. tsb_symm_barrier).
TSB_EXPORT int tsb_gemm_grouped_scatter(const void* A, const void* B, const int* offsets, int groups, int rows_cap, int N,
                                        int K, long long lda, long long ldb, int b_mn, long long b_group_stride,
                                        const int* tags, void* const* peer_out, int world, long long peer_rows,
                                        long long ld_out, void* stream) {
  using namespace tsb;
  if (!offsets || !tags || !peer_out || world < 1 || world > 8 || groups < 1 || groups > 1024 || rows_cap <= 0 ||
      rows_cap % BM || N <= 0 || K <= 0 || K % 8 || ld_out % 8 || peer_rows <= 0 || peer_rows > 0xFFFFFF)
    return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8)) return -2;
  if (b_mn && (K % BK)) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CUtensorMap ta, tb;
  const int bn = (N >= 256) ? 256 : (N >= 128 ? 128 : 64);
  if (!cached_tmap_2d(&ta, A, rows_cap, K, lda * 2, BM, BK)) return -3;
  if (b_group_stride <= 0 || b_group_stride % ldb) return -2;
  const long long grows = b_group_stride / ldb;
  if (grows < (b_mn ? K : N)) return -2;
  const uint64_t map_rows = static_cast<uint64_t>(groups - 1) * grows + (b_mn ? K : N);
  const bool ok = b_mn ? cached_tmap_2d(&tb, B, map_rows, N, ldb * 2, BK, 64)
                       : cached_tmap_2d(&tb, B, map_rows, K, ldb * 2, bn, BK);
  if (!ok) return -3;
  GroupArgs g{offsets, groups, 1, grows, 0};
  g.row_tags = tags;
  g.peer_rows = peer_rows;
  for (int r = 0; r < world; ++r) {
    if (!peer_out[r] || (reinterpret_cast<uintptr_t>(peer_out[r]) & 15)) return -2;
    g.peer_out[r] = peer_out[r];
  }
  void* C = peer_out[0];   // only its alignment is looked at
  auto go = [&](auto bn_tag, auto bmn_tag) {
    return launch_cfg<decltype(bn_tag)::value, false, decltype(bmn_tag)::value, __nv_bfloat16, false>(
        ta, tb, C, rows_cap, N, K, ld_out, 0, s, 1, g);
  };
  using T = std::true_type;
  using F = std::false_type;
  if (bn == 256) return b_mn ? go(std::integral_constant<int, 256>{}, T{}) : go(std::integral_constant<int, 256>{}, F{});
  if (bn == 128) return b_mn ? go(std::integral_constant<int, 128>{}, T{}) : go(std::integral_constant<int, 128>{}, F{});
  return b_mn ? go(std::integral_constant<int, 64>{}, T{}) : go(std::integral_constant<int, 64>{}, F{});
}

// Split-K variant for decode-shaped calls (few rows, the weight matrix is streamed once): the K range is cut into
// `split_k` slices that run as independent work items, so that all SMs pull on HBM, and their fp32 partial sums are
// added into C32 with vector atomics. C32 (fp32 [M, N], row stride ldc) must be zero on entry. A is [M, K] row-major,
// B is [N, K] (b_mn = 0) or [K, N] (b_mn = 1). block_n: 64 or 128.
TSB_EXPORT int tsb_gemm_bf16_splitk(const void* A, const void* B, float* C32, int M, int N, int K, long long lda,
                                    long long ldb, long long ldc, int b_mn, int split_k, int block_n, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || split_k < 1 || split_k > 64) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8) || (ldc % 4))
    return -2;
  const int bn = block_n == 64 ? 64 : 128;
  CUtensorMap ta, tb;
  if (!cached_tmap_2d(&ta, A, M, K, lda * 2, BM, BK)) return -3;
  if (!(b_mn ? cached_tmap_2d(&tb, B, K, N, ldb * 2, BK, 64) : cached_tmap_2d(&tb, B, N, K, ldb * 2, bn, BK))) return -3;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 128)
    return b_mn ? launch_cfg<128, false, true, float, false>(ta, tb, C32, M, N, K, ldc, 0, s, split_k)
                : launch_cfg<128, false, false, float, false>(ta, tb, C32, M, N, K, ldc, 0, s, split_k);
  return b_mn ? launch_cfg<64, false, true, float, false>(ta, tb, C32, M, N, K, ldc, 0, s, split_k)
              : launch_cfg<64, false, false, float, false>(ta, tb, C32, M, N, K, ldc, 0, s, split_k);
}
