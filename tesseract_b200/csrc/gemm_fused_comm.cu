// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one kernel each):
//
//   MODE_SCATTER  row-parallel GEMM -> reduce-scatter:  C_partial = A * op(B) is never written locally; the
//                 epilogue of every 128-row tile stores it straight into the OWNING rank's staging slot
//                 [source rank][local row][N] through that rank's peer mapping, tile by tile while the tensor
//                 cores work on the next tile. Tiles owned by other ranks are computed first (rotated by rank,
//                 so at any moment the ranks write to different peers), the local ones last. A small second
//                 kernel sums the `world` slots after a cross-rank barrier.
//   MODE_GATHER   all-gather -> column-parallel GEMM:    a few CTAs of the same persistent kernel PUSH this rank's
//                 token shard into every rank's landing buffer (local bulk loads into shared memory, 16-byte
//                 stores to the peer, one destination per time slot so the ranks never write to the same peer)
//                 and bump a per-128-row counter on the receiver with a system-scope release; the TMA producer of
//                 every GEMM CTA waits (bounded) for the counter of the row block it is about to load. The local
//                 shard is consumed first, the others in arrival order. Remote data crosses NVLink exactly once,
//                 as writes, and the GEMM reads only local memory (no TMA multicast, no remote operand reads).
//                 When the caller keeps the gathered rows, the copy CTAs also move them from the landing buffer
//                 to the caller's tensor as they arrive.
//
// The GEMM pipeline itself is the one of gemm_tcgen05.cu (TMA -> 128B-swizzled smem ring -> tcgen05.mma with
// TMEM double buffering -> tcgen05.ld epilogue); here the epilogue goes through a per-warp shared-memory
// transpose so that each store instruction writes 128 contiguous bytes of four rows -- full NVLink packets.
// Replaces cuBLASLt + ncclAllReduce / ncclAllGather of the reference's TP path
// (src/distributed/NcclCommBackend.cpp:134-164, benchmarks/bench_cuda_nccl_tp.cpp:88-222).
#include "common.cuh"

#include <cstring>

namespace tsb {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kMaxWorld = 8;
constexpr int MODE_SCATTER = 1;
constexpr int MODE_GATHER = 2;
constexpr int kPiece = 32768;   // bytes per bulk copy
constexpr int kCopyBufs = 6;

template <int BN>
struct Cfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = (BN >= 256) ? 4 : 6;
  static constexpr int kEpiBytes = 4 * 4096;  // one [32 x 64] bf16 staging tile per epilogue warp
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;
  static constexpr int kTmemCols = 2 * BN;
};

struct TpArgs {
  __nv_bfloat16* peer_out[kMaxWorld];   // SCATTER: staging base of every rank ([world][rows_per_rank][N])
  __nv_bfloat16* peer_land[kMaxWorld];  // GATHER: landing buffer [M][K] of every rank (peer_land[rank] is local)
  int* peer_flags[kMaxWorld];           // GATHER: per-128-row-block arrival counters of every rank
  const __nv_bfloat16* x_local;         // GATHER: this rank's token shard [rows_per_rank][K], contiguous, local
  __nv_bfloat16* x_full;                // GATHER: optional local [M][K] copy of the gathered rows (may be null)
  int* chunk_flags;                     // GATHER: == peer_flags[rank]
  int flag_target;                      // GATHER: counter value meaning "the whole block has landed"
  int comm_ctas;                        // GATHER: CTAs [0, comm_ctas) copy, the rest multiply
  int parts;                            // GATHER: slices (= counter increments) per block and call
  int phase_mask;                       // GATHER: bit 0 push the shard, bit 1 multiply (+ keep a copy)
  int rows_per_rank, rank, world;
};

struct TileCoord {
  int m_blk, n_blk;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int num_m, int num_n, int m_rot) {
  constexpr int GM = 16;
  const int group_size = GM * num_n;
  const int group_id = t / group_size;
  const int first_m = group_id * GM;
  const int gm = min(num_m - first_m, GM);
  const int r = t - group_id * group_size;
  int m = first_m + r % gm + m_rot;
  if (m >= num_m) m -= num_m;
  return {m, r / gm};
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Copy CTA of MODE_GATHER, phase 1 (all threads): PUSH this rank's token shard into the landing buffer of every
// rank. Time slot s sends the whole shard to rank (rank - s) mod world, so in every slot the ranks write to
// distinct peers and each receiver gets the shards in the order its GEMM consumes them. A work item is one
// 1 / parts slice of a 128-row block for one destination; items are dealt round-robin to the copy CTAs. The bytes
// come through shared memory: one thread prefetches 32 KB pieces of the LOCAL shard with bulk copies (six in
// flight), all threads store them to the peer with 16-byte stores, and after the last piece of an item one thread
// issues a system-scope release increment of the receiver's counter for that block.
__device__ bool gather_push_cta(uint8_t* smem, uint64_t* bars, const TpArgs& a, int K, volatile int* cta_abort,
                                int* status, int* pieces_done) {
  const int tid = threadIdx.x;
  const long long chunk_bytes = static_cast<long long>(BM) * K * 2;
  const int bpr = a.rows_per_rank / BM;
  const long long slice = chunk_bytes / a.parts;
  const int ppi = static_cast<int>((slice + kPiece - 1) / kPiece);
  const int items_per_slot = bpr * a.parts;
  const int n_items = a.world * items_per_slot;
  const int cta = static_cast<int>(blockIdx.x);
  const int my_items = cta < n_items ? (n_items - cta + a.comm_ctas - 1) / a.comm_ctas : 0;
  const int n_pieces = my_items * ppi;
  const uint8_t* shard = reinterpret_cast<const uint8_t*>(a.x_local);
  const long long shard_off = static_cast<long long>(a.rank) * bpr * chunk_bytes;  // this shard inside [M][K]

  auto decode = [&](int i, int& slot, int& blk, long long& off, uint32_t& bytes, bool& last) {
    const int j = i / ppi, pi = i - j * ppi;
    const int it = cta + j * a.comm_ctas;
    slot = it / items_per_slot;
    const int r = it - slot * items_per_slot;
    blk = r / a.parts;
    off = static_cast<long long>(blk) * chunk_bytes + static_cast<long long>(r - blk * a.parts) * slice +
          static_cast<long long>(pi) * kPiece;
    bytes = static_cast<uint32_t>(min(static_cast<long long>(kPiece), slice - static_cast<long long>(pi) * kPiece));
    last = (pi == ppi - 1);
  };
  auto issue_load = [&](int i) {
    int slot, blk;
    long long off;
    uint32_t bytes;
    bool last;
    decode(i, slot, blk, off, bytes, last);
    const int s = i % kCopyBufs;
    mbar_expect_tx(&bars[s], bytes);
    bulk_g2s(smem + s * kPiece, shard + off, bytes, &bars[s]);
  };

  if (tid == 0)
    for (int i = 0; i < n_pieces && i < kCopyBufs; ++i) issue_load(i);
  bool good = true;
  for (int i = 0; i < n_pieces; ++i) {
    const int s = i % kCopyBufs;
    const bool ok = mbar_wait(&bars[s], (i / kCopyBufs) & 1, cta_abort, status);
    if (__syncthreads_or(ok ? 0 : 1)) {
      good = false;
      break;
    }
    int slot, blk;
    long long off;
    uint32_t bytes;
    bool last;
    decode(i, slot, blk, off, bytes, last);
    int dst_rank = a.rank - slot;
    if (dst_rank < 0) dst_rank += a.world;
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.peer_land[dst_rank]) + shard_off + off;
    uint8_t* dst2 = (slot == 0 && a.x_full) ? reinterpret_cast<uint8_t*>(a.x_full) + shard_off + off : nullptr;
    const uint8_t* src = smem + s * kPiece;
    for (uint32_t o = tid * 16; o < bytes; o += kThreads * 16) {
      const uint4 v = *reinterpret_cast<const uint4*>(src + o);
      *reinterpret_cast<uint4*>(dst + o) = v;
      if (dst2) *reinterpret_cast<uint4*>(dst2 + o) = v;
    }
    __syncthreads();  // every thread has read the buffer and issued its stores
    if (tid == 0) {
      if (i + kCopyBufs < n_pieces) issue_load(i + kCopyBufs);
      if (last) {
        __threadfence_system();
        red_release_sys_add(a.peer_flags[dst_rank] + a.rank * bpr + blk, 1);
      }
    }
  }
  *pieces_done = good ? n_pieces : 0;
  return good;
}

// Copy CTA of MODE_GATHER, phase 2 (one thread): copies the remote shards from the landing buffer into x_full (the
// tensor the caller keeps for the weight gradient) as they arrive, local memory to local memory through the same
// ring of shared-memory buffers. `g0` pieces have already gone through the ring in this launch.
__device__ void gather_keep_cta(uint8_t* smem, uint64_t* bars, const TpArgs& a, int num_m, int K, int g0,
                                volatile int* cta_abort, int* status) {
  const long long chunk_bytes = static_cast<long long>(BM) * K * 2;
  const long long slice = chunk_bytes / a.comm_ctas;  // host guarantees divisibility and 16-byte multiples
  const int ppc = static_cast<int>((slice + kPiece - 1) / kPiece);
  const int bpr = a.rows_per_rank / BM;
  const int n_blocks = num_m - bpr;  // remote blocks, in consumption order
  const int n_pieces = ppc * n_blocks;
  const long long cta_off = static_cast<long long>(blockIdx.x) * slice;
  const uint8_t* land = reinterpret_cast<const uint8_t*>(a.peer_land[a.rank]);
  uint8_t* keep = reinterpret_cast<uint8_t*>(a.x_full);
  int waited_blocks = 0;
  bool good = true;

  auto piece_off = [&](int i, int& ci, uint32_t& bytes) -> long long {
    ci = i / ppc;
    const int pi = i - ci * ppc;
    int mb = (a.rank + 1) * bpr + ci;
    if (mb >= num_m) mb -= num_m;
    bytes = static_cast<uint32_t>(min(static_cast<long long>(kPiece), slice - static_cast<long long>(pi) * kPiece));
    return static_cast<long long>(mb) * chunk_bytes + cta_off + static_cast<long long>(pi) * kPiece;
  };
  auto issue_load = [&](int i) -> bool {
    int ci;
    uint32_t bytes;
    const long long off = piece_off(i, ci, bytes);
    while (waited_blocks <= ci) {  // the block's pushes must have landed
      int mb = (a.rank + 1) * bpr + waited_blocks;
      if (mb >= num_m) mb -= num_m;
      const long long t0 = clock64();
      while (ld_acquire_sys(&a.chunk_flags[mb]) < a.flag_target) {
        if (*cta_abort || clock64() - t0 > kWaitCycleLimit) {
          if (!*cta_abort && status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
          *cta_abort = 1;
          return false;
        }
        __nanosleep(200);
      }
      fence_proxy_async_all();
      ++waited_blocks;
    }
    const int s = (g0 + i) % kCopyBufs;
    mbar_expect_tx(&bars[s], bytes);
    bulk_g2s(smem + s * kPiece, land + off, bytes, &bars[s]);
    return true;
  };

  int issued = 0;
  for (; issued < n_pieces && issued < kCopyBufs && good; ++issued) good = issue_load(issued);
  for (int i = 0; i < n_pieces && good; ++i) {
    const int s = (g0 + i) % kCopyBufs;
    if (!mbar_wait(&bars[s], ((g0 + i) / kCopyBufs) & 1, cta_abort, status)) break;
    int ci;
    uint32_t bytes;
    const long long off = piece_off(i, ci, bytes);
    bulk_s2g(keep + off, smem + s * kPiece, bytes);
    tma_store_commit();
    // the buffer of the previous piece is free once its store has read shared memory
    tma_store_wait_read<1>();
    if (i >= 1 && i - 1 + kCopyBufs < n_pieces) good = issue_load(i - 1 + kCopyBufs);
  }
  tma_store_wait_all<0>();
}

template <int BN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               __nv_bfloat16* __restrict__ C, int M, int N, int K, long long ldc, TpArgs args, int* status) {
  using C_ = Cfg<BN>;
  constexpr int STAGES = C_::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + STAGES * C_::kStageBytes;

  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t tmem_full_bar[2];
  __shared__ __align__(8) uint64_t tmem_empty_bar[2];
  __shared__ __align__(8) uint64_t copy_bar[kCopyBufs];
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (K + BK - 1) / BK;
  const int bpr = args.rows_per_rank / BM;
  // SCATTER: blocks owned by rank+1 first, own blocks last. GATHER: own blocks first.
  const int m_rot = (MODE == MODE_SCATTER) ? ((args.rank + 1) % args.world) * bpr : args.rank * bpr;
  const int comm_ctas = (MODE == MODE_GATHER) ? args.comm_ctas : 0;
  const bool is_copy_cta = (MODE == MODE_GATHER) && static_cast<int>(blockIdx.x) < comm_ctas;
  const int gemm_cta = static_cast<int>(blockIdx.x) - comm_ctas;
  const int gemm_ctas = static_cast<int>(gridDim.x) - comm_ctas;

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
    for (int s = 0; s < kCopyBufs; ++s) mbar_init(&copy_bar[s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (is_copy_cta) {
    __syncthreads();
    int g0 = 0;
    bool good = true;
    if (args.phase_mask & 1) good = gather_push_cta(smem, copy_bar, args, K, &cta_abort, status, &g0);
    if (good && (args.phase_mask & 2) && args.x_full != nullptr && threadIdx.x == 0)
      gather_keep_cta(smem, copy_bar, args, num_m, K, g0, &cta_abort, status);
    return;  // copy CTAs hold no TMEM
  }
  if (MODE == MODE_GATHER && !(args.phase_mask & 2)) return;  // push-only launch (rank emulation on one GPU)
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, C_::kTmemCols);
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
      int ready_blk = -1;
      for (int t = gemm_cta; t < num_tiles; t += gemm_ctas) {
        const TileCoord tc = tile_coord(t, num_m, num_n, m_rot);
        const int m0 = tc.m_blk * BM;
        const int n0 = tc.n_blk * BN;
        bool ok = true;
        if (MODE == MODE_GATHER && ready_blk != tc.m_blk) {
          // wait until the copy CTAs have landed this row block in local memory
          const long long t0 = clock64();
          while (ld_acquire_sys(&args.chunk_flags[tc.m_blk]) < args.flag_target) {
            if (cta_abort) { ok = false; break; }
            if (clock64() - t0 > kWaitCycleLimit) {
              cta_abort = 1;
              if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
          if (!ok) break;
          fence_proxy_async_all();  // generic-proxy acquire -> async-proxy (TMA) reads
          ready_blk = tc.m_blk;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * C_::kStageBytes;
          uint8_t* sB = sA + C_::kStageBytesA;
          mbar_expect_tx(&full_bar[stage], C_::kStageBytes);
          tma_load_2d(sA, &tmA, &full_bar[stage], kb * BK, m0);
          if (!B_MN) {
            tma_load_2d(sB, &tmB, &full_bar[stage], kb * BK, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sB + i * 8192, &tmB, &full_bar[stage], n0 + i * 64, kb * BK);
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
      constexpr uint32_t idesc = umma_idesc(BM, BN, 1, 1, 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = gemm_cta; t < num_tiles; t += gemm_ctas) {
        bool ok = mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1u, &cta_abort, status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &cta_abort, status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_base = smem_u32(smem + stage * C_::kStageBytes);
          const uint32_t b_base = a_base + C_::kStageBytesA;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = umma_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc_sw128(b_base + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
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
    uint8_t* st = epi_smem + q * 4096;  // [32 rows][128 B], 16-byte chunks XOR-swizzled by row
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = gemm_cta; t < num_tiles; t += gemm_ctas) {
      const TileCoord tc = tile_coord(t, num_m, num_n, m_rot);
      const int m0 = tc.m_blk * BM;
      const int n0 = tc.n_blk * BN;
      if (!mbar_wait(&tmem_full_bar[acc], acc_phase, &cta_abort, status)) break;
      tc_fence_after();
      // destination of row r of this warp's 32-row band
      const int band0 = m0 + q * 32;
      __nv_bfloat16* band_dst;
      long long row_stride;
      if (MODE == MODE_SCATTER) {
        const int owner = m0 / args.rows_per_rank;
        const long long lr = band0 - static_cast<long long>(owner) * args.rows_per_rank;
        band_dst = args.peer_out[owner] + (static_cast<long long>(args.rank) * args.rows_per_rank + lr) * N;
        row_stride = N;
      } else {
        band_dst = C + static_cast<long long>(band0) * ldc;
        row_stride = ldc;
      }
#pragma unroll 1
      for (int cg = 0; cg < BN / 64; ++cg) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                            static_cast<uint32_t>(acc * BN + cg * 64 + half * 32), r);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[k * 8 + 0]), __uint_as_float(r[k * 8 + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[k * 8 + 2]), __uint_as_float(r[k * 8 + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[k * 8 + 4]), __uint_as_float(r[k * 8 + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[k * 8 + 6]), __uint_as_float(r[k * 8 + 7]));
            const int j = half * 4 + k;
            *reinterpret_cast<uint4*>(st + lane * 128 + ((j ^ (lane & 7)) * 16)) = v;
          }
        }
        __syncwarp();
        const int col = n0 + cg * 64 + (lane & 7) * 8;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + (lane >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(st + rr * 128 + (((lane & 7) ^ (rr & 7)) * 16));
          if (band0 + rr < M && col < N)
            *reinterpret_cast<uint4*>(band_dst + static_cast<long long>(rr) * row_stride + col) = v;
        }
        __syncwarp();
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
    tmem_dealloc(tmem_base, C_::kTmemCols);
  }
}

// out[i] = sum_s staging[s][i]  (bf16 in, fp32 sum, bf16 out); n elements per slot, n % 8 == 0.
__global__ void __launch_bounds__(256)
reduce_slots_kernel(const __nv_bfloat16* __restrict__ staging, __nv_bfloat16* __restrict__ out, int slots, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < slots; ++s) {
      const uint4 raw = *reinterpret_cast<const uint4*>(staging + s * n + i * 8);
      const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(e[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}

// Cross-rank barrier over flag pads in peer-mapped memory: rank r writes `epoch` into slot r of every rank's
// pad (release, system scope) and waits until every slot of its own pad has reached `epoch` (acquire). Waits are
// bounded; on timeout the status word is set and the kernel returns.
struct BarrierArgs {
  int* pads[kMaxWorld];
};
__global__ void symm_barrier_kernel(BarrierArgs pads, int rank, int world, int epoch, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(pads.pads[r] + rank), "r"(epoch) : "memory");
  const int* mine = pads.pads[rank] + r;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= epoch) break;
    if (clock64() - t0 > kWaitCycleLimit) {
      if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
      break;
    }
    __nanosleep(100);
  }
}

bool tmap2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t stride_bytes, uint32_t br,
            uint32_t bc) {
  return make_tmap_2d(out, base, 2, rows, cols, stride_bytes, br, bc, true);
}

template <int BN, bool B_MN, int MODE>
int launch_tp(const CUtensorMap& ta, const CUtensorMap& tb, void* C, int M, int N, int K, long long ldc,
              const TpArgs& args, int grid, cudaStream_t s) {
  auto kern = gemm_tp_kernel<BN, B_MN, MODE>;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr = true;
  }
  kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, s>>>(ta, tb, static_cast<__nv_bfloat16*>(C), M, N, K, ldc, args,
                                                   device_status_word());
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace tsb

// ------------------------------------------------------------------ peer memory (CUDA IPC)
TSB_EXPORT int tsb_symm_alloc(long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*out, 0, static_cast<size_t>(bytes)));
}
TSB_EXPORT int tsb_symm_free(void* p) { return static_cast<int>(cudaFree(p)); }
// handle: 64 bytes (cudaIpcMemHandle_t)
TSB_EXPORT int tsb_ipc_export(void* p, void* handle64) {
  return static_cast<int>(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), p));
}
TSB_EXPORT int tsb_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
TSB_EXPORT int tsb_ipc_close(void* p) { return static_cast<int>(cudaIpcCloseMemHandle(p)); }

// pads[r] = address (in this process) of rank r's flag pad (world int32 slots each).
TSB_EXPORT int tsb_symm_barrier(void* const* pads, int rank, int world, int epoch, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld) return -2;
  BarrierArgs a;
  for (int i = 0; i < kMaxWorld; ++i) a.pads[i] = i < world ? static_cast<int*>(pads[i]) : nullptr;
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, rank, world, epoch, device_status_word());
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_reduce_slots(const void* staging, void* out, int slots, long long n, void* stream) {
  using namespace tsb;
  if (slots < 1 || n <= 0 || n % 8) return -2;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  reduce_slots_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(staging), static_cast<__nv_bfloat16*>(out), slots, n);
  return static_cast<int>(cudaGetLastError());
}

// Row-parallel GEMM fused with the scatter half of a reduce-scatter.
//   A [M, K] bf16 row-major (lda); B [N, K] (b_mn = 0) or [K, N] (b_mn = 1) (ldb); no local C.
//   peer_out[r]: rank r's staging buffer [world][rows_per_rank][N] bf16, mapped into this process.
//   Tile (row block owned by rank o) is written to peer_out[o][rank][...]. M = world * rows_per_rank,
//   rows_per_rank % 128 == 0, N % 8 == 0. Follow with tsb_symm_barrier + tsb_reduce_slots on every rank.
TSB_EXPORT int tsb_gemm_rs(const void* A, const void* B, void* const* peer_out, int M, int N, int K, long long lda,
                           long long ldb, int b_mn, int rows_per_rank, int rank, int world, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rows_per_rank % BM || M != rows_per_rank * world || N % 8 || N < 128) return -2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda % 8) || (ldb % 8)) return -2;
  CUtensorMap ta, tb;
  const int bn = (N >= 256) ? 256 : 128;
  if (!tmap2d(&ta, A, M, K, lda * 2, BM, BK)) return -3;
  if (!(b_mn ? tmap2d(&tb, B, K, N, ldb * 2, BK, 64) : tmap2d(&tb, B, N, K, ldb * 2, bn, BK))) return -3;
  TpArgs args{};
  for (int i = 0; i < world; ++i) args.peer_out[i] = static_cast<__nv_bfloat16*>(peer_out[i]);
  args.rows_per_rank = rows_per_rank;
  args.rank = rank;
  args.world = world;
  const int tiles = (M / BM) * ((N + bn - 1) / bn);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256)
    return b_mn ? launch_tp<256, true, MODE_SCATTER>(ta, tb, nullptr, M, N, K, N, args, grid, s)
                : launch_tp<256, false, MODE_SCATTER>(ta, tb, nullptr, M, N, K, N, args, grid, s);
  return b_mn ? launch_tp<128, true, MODE_SCATTER>(ta, tb, nullptr, M, N, K, N, args, grid, s)
              : launch_tp<128, false, MODE_SCATTER>(ta, tb, nullptr, M, N, K, N, args, grid, s);
}

// All-gather fused with the column-parallel GEMM: C [M, N] = gather(x_local)[M, K] * op(B).
//   x_local [rows_per_rank][K] bf16 contiguous: this rank's token shard (any local memory).
//   peer_land[r]: rank r's landing buffer [M][K] bf16 (peer mapping; peer_land[rank] is local and feeds the GEMM).
//   peer_flags[r]: rank r's int32 [M / 128] arrival counters (peer mapping), zero at allocation;
//   flag_target = (#calls so far on these counters, this one included) * parts.
//   x_full: optional local [M][K] tensor that also receives the gathered rows (for the weight gradient); null to
//   leave them in the landing buffer only. comm_ctas must divide 128 * K * 2 / 16; parts in {1, 2, 4, 8}.
//   phase_mask: 3 in production; 1 = push only and 2 = multiply only let one GPU emulate the ranks in two passes.
//   Every rank must have passed a barrier after its previous use of the landing buffer before any rank calls this.
TSB_EXPORT int tsb_gemm_ag(const void* x_local, void* const* peer_land, void* const* peer_flags, void* x_full,
                           const void* B, void* C, int flag_target, int comm_ctas, int parts, int phase_mask, int M,
                           int N, int K, long long ldb, long long ldc, int b_mn, int rows_per_rank, int rank, int world,
                           void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rows_per_rank % BM || M != rows_per_rank * world || N % 8 || N < 128 || K % 8)
    return -2;
  if (comm_ctas < 1 || (static_cast<long long>(BM) * K * 2) % (16LL * comm_ctas)) return -2;
  if (parts != 1 && parts != 2 && parts != 4 && parts != 8) return -2;
  if (rank < 0 || rank >= world || (phase_mask & 3) == 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x_full) & 15) || (reinterpret_cast<uintptr_t>(x_local) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (ldb % 8) || (ldc % 8))
    return -2;
  for (int i = 0; i < world; ++i)
    if (!peer_land[i] || !peer_flags[i] || (reinterpret_cast<uintptr_t>(peer_land[i]) & 15)) return -2;
  CUtensorMap ta, tb;
  const int bn = (N >= 256) ? 256 : 128;
  if (!tmap2d(&ta, peer_land[rank], M, K, static_cast<uint64_t>(K) * 2, BM, BK)) return -3;
  if (!(b_mn ? tmap2d(&tb, B, K, N, ldb * 2, BK, 64) : tmap2d(&tb, B, N, K, ldb * 2, bn, BK))) return -3;
  TpArgs args{};
  for (int i = 0; i < world; ++i) {
    args.peer_land[i] = static_cast<__nv_bfloat16*>(peer_land[i]);
    args.peer_flags[i] = static_cast<int*>(peer_flags[i]);
  }
  args.x_local = static_cast<const __nv_bfloat16*>(x_local);
  args.x_full = static_cast<__nv_bfloat16*>(x_full);
  args.chunk_flags = args.peer_flags[rank];
  args.flag_target = flag_target;
  args.comm_ctas = comm_ctas;
  args.parts = parts;
  args.phase_mask = phase_mask;
  args.rows_per_rank = rows_per_rank;
  args.rank = rank;
  args.world = world;
  const int grid = sm_count();  // every CTA must be resident: GEMM CTAs wait for data other CTAs and ranks deliver
  if (comm_ctas >= grid) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256)
    return b_mn ? launch_tp<256, true, MODE_GATHER>(ta, tb, C, M, N, K, ldc, args, grid, s)
                : launch_tp<256, false, MODE_GATHER>(ta, tb, C, M, N, K, ldc, args, grid, s);
  return b_mn ? launch_tp<128, true, MODE_GATHER>(ta, tb, C, M, N, K, ldc, args, grid, s)
              : launch_tp<128, false, MODE_GATHER>(ta, tb, C, M, N, K, ldc, args, grid, s);
}
