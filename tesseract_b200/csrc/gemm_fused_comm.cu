// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one kernel each):
//
//   MODE_SCATTER  row-parallel GEMM -> reduce-scatter:  C_partial = A * op(B) is never written locally; the
//                 epilogue of every 128-row tile stores it straight into the OWNING rank's staging slot
//                 [source rank][local row][N] through that rank's peer mapping, tile by tile while the tensor
//                 cores work on the next tile. Tiles owned by other ranks are computed first (rotated by rank,
//                 so at any moment the ranks write to different peers), the local ones last. A small second
//                 kernel sums the `world` slots after a cross-rank barrier.
//   MODE_GATHER   all-gather -> column-parallel GEMM:    four extra warps in every CTA of the same persistent kernel
//                 PUSH this rank's token shard into every rank's landing buffer (16-byte loads from local memory,
//                 stores to the peer, one destination per time slot so the ranks never write to the same peer)
//                 and bump a per-128-row counter on the receiver with a system-scope release; the TMA producer of
//                 every CTA waits (bounded) for the counter of the row block it is about to load. The local
//                 shard is consumed first, the others in arrival order. Remote data crosses NVLink exactly once,
//                 as writes, and the GEMM reads only local memory (no TMA multicast, no remote operand reads).
//                 When the caller keeps the gathered rows, the push warps also move them from the landing buffer
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
constexpr int kGemmThreads = 192;  // TMA producer, MMA issuer, four epilogue warps
constexpr int kPushWarps = 4;
constexpr int kThreads = kGemmThreads + 32 * kPushWarps;  // + warps that move activations between ranks in MODE_GATHER
constexpr int kMaxWorld = 8;
constexpr int MODE_SCATTER = 1;
constexpr int MODE_GATHER = 2;

template <int BN>
struct Cfg {
  static constexpr int kStageBytesA = BM * BK * 2;
  static constexpr int kStageBytesB = BN * BK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = (BN >= 256) ? 4 : 6;
  static constexpr int kEpiBytes = 4 * 2 * 4096;  // two [32 x 64] bf16 staging tiles per epilogue warp
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024;
  static constexpr int kTmemCols = 2 * BN;
};

struct TpArgs {
  __nv_bfloat16* peer_out[kMaxWorld];   // SCATTER: staging base of every rank ([world][rows_per_rank][N])
  __nv_bfloat16* peer_land[kMaxWorld];  // GATHER: landing buffer [M][K] of every rank (peer_land[rank] is local)
  int* peer_flags[kMaxWorld];           // GATHER: arrival counters [world][nsub] of every rank
  const __nv_bfloat16* x_local;         // GATHER: this rank's token shard [rows_per_rank][K], contiguous, local
  __nv_bfloat16* x_full;                // GATHER: optional local [M][K] copy of the gathered rows (may be null)
  int* chunk_flags;                     // GATHER: == peer_flags[rank]
  int flag_target;                      // GATHER: counter value meaning "the sub-chunk has landed"
  int nsub;                             // GATHER: sub-chunks (of whole 128-row blocks) per shard
  int phase_mask;                       // GATHER: bit 0 push the shard, bit 1 multiply (+ keep a copy)
  long long* trace;                     // GATHER: optional [gridDim.x][8] globaltimer stamps (null = off)
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

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Arrival counters and barrier epochs only ever grow, modulo 2^32: "has the counter reached the target" is decided
// on the wrapped difference, which stays correct across the wrap as long as the two are less than 2^31 apart.
__device__ __forceinline__ bool counter_behind(int value, int target) {
  return static_cast<int>(static_cast<unsigned>(value) - static_cast<unsigned>(target)) < 0;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Push warps of MODE_GATHER. Every CTA of the kernel carries kPushWarps (four) extra warps that take no part in the
// GEMM: together they PUSH this rank's token shard into the landing buffer of every rank with plain 16-byte loads
// (local) and stores (peer). Spreading the copy over all SMs matters: one SM sustains only a few tens of GB/s
// towards a peer, 148 of them saturate the links without taking an SM away from the tensor cores. Time slot s sends
// the shard to rank (rank - s) mod world, so at any moment the ranks write to distinct peers and each receiver gets
// the shards in the order its GEMM consumes them (its own shard the GEMM reads in place). A shard is sent as `nsub`
// sub-chunks of whole 128-row blocks; every push warp of the grid streams one contiguous slice of a sub-chunk,
// and when the four warps of a CTA have issued their part, ONE thread of the CTA makes it visible with a
// system-scope fence and increments the receiver's counter for (source rank, sub-chunk). A counter that has risen
// by gridDim.x means the sub-chunk has landed. Fences are kept this rare on purpose: a system-scope fence stalls
// the SM's stores for about two microseconds, and one per 16 KB slice halved the push bandwidth.
constexpr int kPushUnroll = 8;

__device__ __forceinline__ long long global_ns() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// trace slots per CTA: 0 kernel start, 1 remote pushes fenced, 2 all pushes done, 3 first wait for a remote block
// begins, 4 it ends, 5 last TMA load issued, 6 epilogue of the last tile done, 7 kept copy done
__device__ __forceinline__ void trace_stamp(const TpArgs& a, int slot) {
  if (a.trace) a.trace[static_cast<long long>(blockIdx.x) * 8 + slot] = global_ns();
}

__device__ __forceinline__ void push_warps_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kPushWarps) : "memory"); }

// Copies bytes [0, bytes) from src to dst (and dst2 if not null); warp g of G takes one contiguous slice (a
// multiple of 512 bytes) and streams it in passes of 4 KB, the loads of the next pass in flight during the stores.
__device__ __forceinline__ void sliced_copy16(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                              uint8_t* __restrict__ dst2, long long bytes, int g, int G, int lane) {
  constexpr long long kPass = 512LL * kPushUnroll;
  const long long slice = ((bytes + G - 1) / G + 511) / 512 * 512;
  const long long lo = static_cast<long long>(g) * slice;
  const long long hi = min(bytes, lo + slice);
  if (lo >= hi) return;
  uint4 cur[kPushUnroll], nxt[kPushUnroll];
  auto load = [&](uint4* v, long long o0) {
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const long long o = o0 + (u * 32 + lane) * 16LL;
      if (o < hi) v[u] = *reinterpret_cast<const uint4*>(src + o);
    }
  };
  load(cur, lo);
  for (long long o0 = lo; o0 < hi; o0 += kPass) {
    if (o0 + kPass < hi) load(nxt, o0 + kPass);
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) {
      const long long o = o0 + (u * 32 + lane) * 16LL;
      if (o < hi) {
        *reinterpret_cast<uint4*>(dst + o) = cur[u];
        if (dst2) *reinterpret_cast<uint4*>(dst2 + o) = cur[u];
      }
    }
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) cur[u] = nxt[u];
  }
}

__device__ void gather_push_warps(const TpArgs& a, int K, int pw, int lane) {
  const long long shard_bytes = static_cast<long long>(a.rows_per_rank) * K * 2;
  const long long sub_bytes = shard_bytes / a.nsub;  // host: nsub divides the blocks of a shard
  const int G = static_cast<int>(gridDim.x) * kPushWarps;
  const int g = static_cast<int>(blockIdx.x) * kPushWarps + pw;
  const uint8_t* shard = reinterpret_cast<const uint8_t*>(a.x_local);
  const long long shard_off = static_cast<long long>(a.rank) * shard_bytes;  // this shard inside [M][K]
  // remote destinations first (slots 1 .. world-1); the local copy, which no GEMM warp waits for, goes last
  for (int s = 1; s <= a.world; ++s) {
    const int slot = (s == a.world) ? 0 : s;
    int dst_rank = a.rank - slot;
    if (dst_rank < 0) dst_rank += a.world;
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.peer_land[dst_rank]) + shard_off;
    uint8_t* dst2 = (slot == 0 && a.x_full) ? reinterpret_cast<uint8_t*>(a.x_full) + shard_off : nullptr;
    for (int j = 0; j < a.nsub; ++j) {
      const long long base = static_cast<long long>(j) * sub_bytes;
      sliced_copy16(shard + base, dst + base, dst2 ? dst2 + base : nullptr, sub_bytes, g, G, lane);
      push_warps_sync();  // the four push warps of this CTA have issued their stores of the sub-chunk
      if (pw == 0 && lane == 0) {
        __threadfence_system();
        red_release_sys_add(a.peer_flags[dst_rank] + a.rank * a.nsub + j, 1);
        if (j == a.nsub - 1 && (s == a.world - 1 || s == a.world)) trace_stamp(a, s == a.world ? 2 : 1);
      }
    }
  }
}

// After the push: copy the remote shards from the landing buffer into x_full (the tensor the caller keeps for the
// weight gradient) as they arrive, in consumption order. Local memory to local memory; waits are bounded.
__device__ void gather_keep_warps(const TpArgs& a, int K, int pw, int lane, int* status) {
  const long long shard_bytes = static_cast<long long>(a.rows_per_rank) * K * 2;
  const long long sub_bytes = shard_bytes / a.nsub;
  const int G = static_cast<int>(gridDim.x) * kPushWarps;
  const int g = static_cast<int>(blockIdx.x) * kPushWarps + pw;
  const uint8_t* land = reinterpret_cast<const uint8_t*>(a.peer_land[a.rank]);
  uint8_t* keep = reinterpret_cast<uint8_t*>(a.x_full);
  for (int s = 1; s < a.world; ++s) {
    int src_rank = a.rank + s;
    if (src_rank >= a.world) src_rank -= a.world;
    for (int j = 0; j < a.nsub; ++j) {
      const long long t0 = clock64();
      bool ok = true;
      while (counter_behind(ld_acquire_sys(&a.chunk_flags[src_rank * a.nsub + j]), a.flag_target)) {
        if (clock64() - t0 > kWaitCycleLimit) {
          ok = false;
          break;
        }
        __nanosleep(500);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0 && status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
        return;
      }
      const long long off = static_cast<long long>(src_rank) * shard_bytes + static_cast<long long>(j) * sub_bytes;
      sliced_copy16(land + off, keep + off, nullptr, sub_bytes, g, G, lane);
    }
  }
}

template <int BN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmAL,
               const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
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
  const int gemm_cta = static_cast<int>(blockIdx.x);
  const int gemm_ctas = static_cast<int>(gridDim.x);
  const bool do_gemm = (MODE != MODE_GATHER) || (args.phase_mask & 2);

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
    tma_prefetch_desc(&tmAL);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1 && do_gemm) {
    tmem_alloc(&tmem_base_smem, C_::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp >= kGemmThreads / 32) {
    // ------------------------------------------------------------ push warps (MODE_GATHER only)
    if (MODE == MODE_GATHER) {
      const int pw = warp - kGemmThreads / 32;
      if (pw == 0 && lane == 0) trace_stamp(args, 0);
      if (args.phase_mask & 1) gather_push_warps(args, K, pw, lane);
      if ((args.phase_mask & 2) && args.x_full != nullptr) {
        gather_keep_warps(args, K, pw, lane, status);
        if (pw == 0 && lane == 0) trace_stamp(args, 7);
      }
    }
  } else if (!do_gemm) {
    // push-only launch (rank emulation on one GPU): the GEMM warps have nothing to do
  } else if (warp == 0) {
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
        // MODE_GATHER reads the rows of this rank's own shard in place (tmAL), the others from the landing buffer
        const bool own = (MODE == MODE_GATHER) && tc.m_blk >= m_rot && tc.m_blk < m_rot + bpr;
        const CUtensorMap* mapA = own ? &tmAL : &tmA;
        const int m0a = own ? m0 - m_rot * BM : m0;
        if (MODE == MODE_GATHER && !own && ready_blk != tc.m_blk) {
          // wait until the owner's push warps have landed the sub-chunk of this row block in local memory
          const int owner = tc.m_blk / bpr;
          const int* flag = &args.chunk_flags[owner * args.nsub + (tc.m_blk - owner * bpr) / (bpr / args.nsub)];
          const long long t0 = clock64();
          const bool first_wait = (ready_blk < 0);
          if (first_wait) trace_stamp(args, 3);
          while (counter_behind(ld_acquire_sys(flag), args.flag_target)) {
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
          if (first_wait) trace_stamp(args, 4);
          ready_blk = tc.m_blk;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &cta_abort, status);
          if (!ok) break;
          uint8_t* sA = smem + stage * C_::kStageBytes;
          uint8_t* sB = sA + C_::kStageBytesA;
          mbar_expect_tx(&full_bar[stage], C_::kStageBytes);
          tma_load_2d(sA, mapA, &full_bar[stage], kb * BK, m0a);
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
      if (MODE == MODE_GATHER) trace_stamp(args, 5);
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
    uint8_t* st_base = epi_smem + q * 8192;  // 2 x [32 rows][128 B], 16-byte chunks XOR-swizzled by row
    uint32_t st_sel = 0;
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
        uint8_t* st = st_base + (st_sel & 1u) * 4096;
        if (MODE == MODE_GATHER) {
          // the bulk store issued from this buffer two column groups ago must have read it
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
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
        if (MODE == MODE_GATHER) {
          // local output: one bulk tensor store per [32 x 64] tile (the staging layout is the 128-byte swizzle).
          // It leaves through the TMA unit, not through the load/store queue that the push warps fill with
          // stores waiting for NVLink, so the epilogue never queues behind them.
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && band0 < M && n0 + cg * 64 < N) {
            tma_store_2d(&tmC, st, n0 + cg * 64, band0);
            tma_store_commit();
          }
          ++st_sel;
        } else {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (MODE == MODE_GATHER && lane == 0) tma_store_wait_all<0>();
    if (MODE == MODE_GATHER && warp == 2 && lane == 0) trace_stamp(args, 6);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1 && do_gemm) {
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
__global__ void symm_barrier_kernel(BarrierArgs pads, int rank, int world, int epoch, long long limit_cycles,
                                    int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(pads.pads[r] + rank), "r"(epoch) : "memory");
  const int* mine = pads.pads[rank] + r;
  const long long t0 = clock64();
  while (true) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (!counter_behind(v, epoch)) break;
    if (clock64() - t0 > limit_cycles) {
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
int launch_tp(const CUtensorMap& ta, const CUtensorMap& tal, const CUtensorMap& tb, const CUtensorMap& tc, void* C, int M, int N, int K, long long ldc,
              const TpArgs& args, int grid, cudaStream_t s) {
  auto kern = gemm_tp_kernel<BN, B_MN, MODE>;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, s>>>(ta, tal, tb, tc, static_cast<__nv_bfloat16*>(C), M, N, K, ldc, args,
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
// limit_cycles: how long (SM clock cycles) a rank waits for its peers before it gives up, records
// kStatusFlagTimeout in the status word and returns; <= 0 selects the library default of about one second.
TSB_EXPORT int tsb_symm_barrier_limit(void* const* pads, int rank, int world, int epoch, long long limit_cycles,
                                      void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld) return -2;
  BarrierArgs a;
  for (int i = 0; i < kMaxWorld; ++i) a.pads[i] = i < world ? static_cast<int*>(pads[i]) : nullptr;
  symm_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      a, rank, world, epoch, limit_cycles > 0 ? limit_cycles : kWaitCycleLimit, device_status_word());
  return static_cast<int>(cudaGetLastError());
}
TSB_EXPORT int tsb_symm_barrier(void* const* pads, int rank, int world, int epoch, void* stream) {
  return tsb_symm_barrier_limit(pads, rank, world, epoch, 0, stream);
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
    return b_mn ? launch_tp<256, true, MODE_SCATTER>(ta, ta, tb, ta, nullptr, M, N, K, N, args, grid, s)
                : launch_tp<256, false, MODE_SCATTER>(ta, ta, tb, ta, nullptr, M, N, K, N, args, grid, s);
  return b_mn ? launch_tp<128, true, MODE_SCATTER>(ta, ta, tb, ta, nullptr, M, N, K, N, args, grid, s)
              : launch_tp<128, false, MODE_SCATTER>(ta, ta, tb, ta, nullptr, M, N, K, N, args, grid, s);
}

// All-gather fused with the column-parallel GEMM: C [M, N] = gather(x_local)[M, K] * op(B).
//   x_local [rows_per_rank][K] bf16 contiguous: this rank's token shard (any local memory).
//   peer_land[r]: rank r's landing buffer [M][K] bf16 (peer mapping; peer_land[rank] is local and feeds the GEMM).
//   peer_flags[r]: rank r's int32 [world * nsub] arrival counters (peer mapping), zero at allocation;
//   calls = number of calls so far on these counters, this one included, modulo 2^32 (every call adds the grid
//   size to each counter; counters and target wrap together).
//   x_full: optional local [M][K] tensor that also receives the gathered rows (for the weight gradient); null to
//   leave them in the landing buffer only. nsub: sub-chunks per shard, a divisor of rows_per_rank / 128.
//   trace: null, or int64 [SM count][8] that receives globaltimer stamps of the phases of every CTA (diagnostics).
//   phase_mask: 3 in production; 1 = push only and 2 = multiply only let one GPU emulate the ranks in two passes.
//   Every rank must have passed a barrier after its previous use of the landing buffer before any rank calls this.
TSB_EXPORT int tsb_gemm_ag(const void* x_local, void* const* peer_land, void* const* peer_flags, void* x_full,
                           const void* B, void* C, int calls, int nsub, int phase_mask, int M,
                           int N, int K, long long ldb, long long ldc, int b_mn, int rows_per_rank, int rank, int world,
                           void* trace, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rows_per_rank % BM || M != rows_per_rank * world || N % 8 || N < 128 || K % 8)
    return -2;
  if (nsub < 1 || (rows_per_rank / BM) % nsub) return -2;
  if (rank < 0 || rank >= world || (phase_mask & 3) == 0) return -2;
  if ((reinterpret_cast<uintptr_t>(x_full) & 15) || (reinterpret_cast<uintptr_t>(x_local) & 15) ||
      (reinterpret_cast<uintptr_t>(B) & 15) || (ldb % 8) || (ldc % 8))
    return -2;
  for (int i = 0; i < world; ++i)
    if (!peer_land[i] || !peer_flags[i] || (reinterpret_cast<uintptr_t>(peer_land[i]) & 15)) return -2;
  CUtensorMap ta, tb;
  const int bn = (N >= 256) ? 256 : 128;
  CUtensorMap tal;
  if (!tmap2d(&ta, peer_land[rank], M, K, static_cast<uint64_t>(K) * 2, BM, BK)) return -3;
  if (!tmap2d(&tal, x_local, rows_per_rank, K, static_cast<uint64_t>(K) * 2, BM, BK)) return -3;
  CUtensorMap tcm;  // output, stored in [32 x 64] tiles
  if ((reinterpret_cast<uintptr_t>(C) & 15) || !tmap2d(&tcm, C, M, N, static_cast<uint64_t>(ldc) * 2, 32, 64)) return -3;
  if (!(b_mn ? tmap2d(&tb, B, K, N, ldb * 2, BK, 64) : tmap2d(&tb, B, N, K, ldb * 2, bn, BK))) return -3;
  TpArgs args{};
  for (int i = 0; i < world; ++i) {
    args.peer_land[i] = static_cast<__nv_bfloat16*>(peer_land[i]);
    args.peer_flags[i] = static_cast<int*>(peer_flags[i]);
  }
  args.x_local = static_cast<const __nv_bfloat16*>(x_local);
  args.x_full = static_cast<__nv_bfloat16*>(x_full);
  args.chunk_flags = args.peer_flags[rank];
  args.nsub = nsub;
  args.trace = static_cast<long long*>(trace);
  args.phase_mask = phase_mask;
  args.rows_per_rank = rows_per_rank;
  args.rank = rank;
  args.world = world;
  const int grid = sm_count();  // one resident CTA per SM: its GEMM warps wait for data that push warps deliver
  args.flag_target = static_cast<int>(static_cast<unsigned>(calls) * static_cast<unsigned>(grid));  // modulo 2^32
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 256)
    return b_mn ? launch_tp<256, true, MODE_GATHER>(ta, tal, tb, tcm, C, M, N, K, ldc, args, grid, s)
                : launch_tp<256, false, MODE_GATHER>(ta, tal, tb, tcm, C, M, N, K, ldc, args, grid, s);
  return b_mn ? launch_tp<128, true, MODE_GATHER>(ta, tal, tb, tcm, C, M, N, K, ldc, args, grid, s)
              : launch_tp<128, false, MODE_GATHER>(ta, tal, tb, tcm, C, M, N, K, ldc, args, grid, s);
}
