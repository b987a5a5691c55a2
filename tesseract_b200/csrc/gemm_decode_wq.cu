// Weight-streaming GEMM for decode-sized batches:  Y[M, N] (bf16) = X[M, K] (bf16) * W[N, K]^T,  M <= 128 per CTA row
// block, W either bf16 or block-scaled fp8 (E4M3 payload, one fp32 scale per 128 x 128 block of W -- the weight
// half of the "1 x 128 activation / 128 x 128 weight" scheme; activations stay bf16, so nothing is quantised at
// run time and the only error is the weight rounding).
//
// A decode step multiplies a handful of rows with every weight matrix of the model once: the kernel is a copy of W
// through the tensor cores, and what matters is bytes in flight, not FLOPs.
//   * One CTA owns BN weight rows (16 .. 256, chosen by the host so that tiles x split fill the SMs) and one of S
//     K slices; the S CTAs of a tile form a cluster and reduce their fp32 partial tiles through distributed shared
//     memory (each CTA sums 128 / S batch rows from all S partials and writes bf16), so only Y touches HBM.
//   * fp8 weights: TMA brings raw E4M3 tiles (BN x 64 bytes) into a deep ring; four conversion warps turn each into the
//     128-byte-swizzled bf16 operand tile the MMA reads, applying the block scale on the way. The E4M3 byte is
//     re-based into a bf16 bit pattern with two logic operations ((b & 0x7f) << 4 | sign << 8 is the value times
//     2^-120, subnormals included) and one packed bf16 multiply by (scale * 2^120) restores it. The conversion
//     warps work in four pairs, each owning one converted-tile slot, so that four stages are in conversion at once.
//     Weights packed tile-major ([tile][k step][BN][64] bytes) arrive by one bulk copy per stage.
//   * bf16 weights: TMA writes the operand tiles directly (the conversion warps idle).
//   * Programmatic dependent launch: the kernel may be launched while its predecessor in the stream is still
//     running. Barrier set-up, TMEM allocation and the first ring of WEIGHT loads (which do not depend on the
//     predecessor) happen before griddepcontrol.wait; only the activation loads come after it. In a decode step,
//     where a GEMM lasts 5 to 40 microseconds, this hides the launch ramp behind the previous kernel's tail.
// Accumulation: tcgen05.mma kind::f16, 128 x BN x 16, fp32 in TMEM. All waits are bounded (common.cuh).
//
// Replaces the reference's cuBLASLt call for M <= 16 .. 256 (src/cuda/MatMul.cpp:422-490) and its dequantising
// CUDA-core kernels for quantised weights at batch sizes above a GEMV (src/cuda/DequantMatMul.cu:95-127).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int BM = 128;           // batch rows per CTA (MMA M)
constexpr int BK = 64;            // K elements per pipeline step
constexpr int kMaxStages = 8;     // upper bound of every ring (barrier arrays)
constexpr int kConvWarps = 8;
constexpr int kConvGroups = 4;    // conversion warps work in pairs; a pair owns one converted-tile slot
constexpr int kSmemBudget = 220 * 1024;   // dynamic shared memory the kernel asks for, always (static smem comes on top)
constexpr int kMaxScaleSteps = 512;       // 128-wide K blocks of one CTA's K slice whose scales are staged in smem
constexpr int kThreads = 192 + 32 * kConvWarps;   // producer, MMA, 4 epilogue warps, 8 conversion warps
constexpr int kMaxBN = 256;

// Shared-memory plan of one launch (sizes depend on the batch rows and the tile width, so the rings are as deep as
// the 226 KB allow: what bounds the kernel is bytes in flight per SM).
struct Layout {
  int x_rows;       // rows of the activation box (batch rows rounded up to 8, at most 128)
  int x_pitch;      // bytes between activation stages
  int x_stages;     // activation ring depth: 8 while a stage is at most 8 KB (up to 64 rows), else 4
  int c_pitch;      // bytes between operand tiles of W ([BN][128 B], 1024-aligned)
  int r_pitch;      // bytes between raw fp8 tiles ([BN][64 B]); 0 on the bf16 path
  int c_stages;     // operand-tile ring (bf16: filled by TMA; fp8: filled by the conversion warps)
  int r_stages;     // raw ring (fp8 path)
};

// rb: 128-row blocks of the batch that one CTA multiplies with the weight tile it streams (1, or 2 for 129 .. 256 rows:
// the tile is then loaded -- and, for fp8, widened -- once for both blocks, into two accumulators).
inline Layout make_layout(int M, int bn, bool fp8, int rb) {
  Layout L{};
  const int rows = (M >= BM || rb > 1) ? BM : ((M + 7) / 8) * 8;
  L.x_rows = rows;
  L.x_pitch = rb * (((rows * BK * 2 + 1023) / 1024) * 1024);
  L.c_pitch = ((bn * BK * 2 + 1023) / 1024) * 1024;
  // the MMA reads 128 activation rows from a stage whatever x_rows is; the bytes past the box belong to later
  // buffers (their content only reaches accumulator rows that are never stored), but must lie inside the allocation
  L.x_stages = L.x_pitch <= 8192 ? 8 : ((rb > 1 && fp8) ? 3 : 4);
  const int x_ring = L.x_stages * L.x_pitch;
  const int x_overread = rb * BM * BK * 2 - L.x_pitch;     // > 0 when x_rows < 128
  int avail = kSmemBudget - 1024 - x_ring;
  if (!fp8) {
    L.r_pitch = 0;
    L.r_stages = 0;
    L.c_stages = avail / L.c_pitch;
    if (L.c_stages > kMaxStages) L.c_stages = kMaxStages;
  } else {
    // converted tiles: as many as fit next to a raw ring of at least six stages, at most four (the conversion warps
    // and the tensor core hand tiles back and forth; with two slots each hand-over is on the critical path)
    L.r_pitch = ((bn * BK + 1023) / 1024) * 1024;
    L.c_stages = kConvGroups;      // one converted-tile slot per pair of conversion warps
    avail -= L.c_stages * L.c_pitch;
    L.r_stages = avail / L.r_pitch;
    if (L.r_stages > kMaxStages) L.r_stages = kMaxStages;
    // The conversion pairs run up to kConvGroups stages ahead of the multiply. A pair that waits for the second fill
    // of a raw slot must find the first fill landed (an mbarrier wait tells phases apart by parity only), which the
    // in-order multiply guarantees as long as the raw ring is at least kConvGroups deep.
    if (L.r_stages < kConvGroups) L.r_stages = 0;
  }
  (void)x_overread;   // always covered: the W rings that follow the activation ring are larger than 16 KB in total
  return L;
}

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
// One contiguous run of global memory -> shared memory through the bulk-copy engine (no tensor map, no per-row work).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Two E4M3 bytes, already spread to bits [7:0] and [23:16] of `y` -> packed bf16x2 holding value * 2^-120 each:
// exponent and mantissa move up by four bits, the sign by eight. (Both MMA operands must have the same 16-bit format:
// bf16 activations against fp16 weights is not a legal tcgen05.mma kind::f16 instruction, so the weights are widened
// to bf16 and the one-instruction E4M3 -> f16x2 hardware conversion cannot be used here.)
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_rebased(uint32_t y) {
  return ((y & 0x007f007fu) << 4) | ((y & 0x00800080u) << 8);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int S, bool FP8, int RB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_decode_wq_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                      const uint8_t* __restrict__ w_packed, const float* __restrict__ w_scale,
                      __nv_bfloat16* __restrict__ Y, int M, int N, int K,
                      long long ldy, int BN, int scale_cols, int scale_rows, const Layout L, int flags, int* status) {
  const int CST = L.c_stages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sC = sX + L.x_stages * L.x_pitch;         // operand tiles of W: [BN rows][128 B], swizzled
  uint8_t* sR = sC + CST * L.c_pitch;                // raw fp8 tiles: [BN rows][64 B], linear (fp8 path only)
  __shared__ __align__(8) uint64_t full_x[kMaxStages], empty_x[kMaxStages];
  __shared__ __align__(8) uint64_t full_c[kMaxStages], empty_c[kMaxStages];
  __shared__ __align__(8) uint64_t full_r[kMaxStages], empty_r[kMaxStages];
  __shared__ uint32_t s_scale[FP8 ? 3 * kMaxScaleSteps : 1];   // bf16x2 (scale * 2^120) per (row block, K block)
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = static_cast<int>(cluster_ctarank());
  const int tile = static_cast<int>(blockIdx.x) / S;
  const int n0 = tile * BN;
  const int m0 = static_cast<int>(blockIdx.y) * BM * RB;
  constexpr int kXBlock = BM * BK * 2;             // one 128-row activation tile inside a stage
  const int total_kb = (K + BK - 1) / BK;
  const int kb_per = (total_kb + S - 1) / S;
  const int kb0 = slice * kb_per;
  const int kb1 = min(total_kb, kb0 + kb_per);
  const int nk = max(0, kb1 - kb0);
  const uint32_t w_stage_bytes = static_cast<uint32_t>(BN) * BK * (FP8 ? 1 : 2);

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full_x[s], 1);
      mbar_init(&empty_x[s], 1);
      mbar_init(&full_c[s], FP8 ? kConvWarps / kConvGroups : 1);
      mbar_init(&empty_c[s], 1);
      mbar_init(&full_r[s], 1);
      mbar_init(&empty_r[s], kConvWarps / kConvGroups);
    }
    mbar_init(&acc_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
    pdl_trigger();     // whatever follows in the stream may start its own prologue
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, RB * kMaxBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int WST = FP8 ? L.r_stages : L.c_stages;
      const bool packed = (flags & 2) != 0;
      const uint32_t x_bytes = static_cast<uint32_t>(RB * L.x_rows) * BK * 2;
      uint64_t* w_full = FP8 ? full_r : full_c;
      uint64_t* w_empty = FP8 ? empty_r : empty_c;
      uint8_t* w_base = FP8 ? sR : sC;
      const uint32_t w_pitch = static_cast<uint32_t>(FP8 ? L.r_pitch : L.c_pitch);
      int w_issued = 0, ws = 0, x_issued = 0, xs = 0;
      uint32_t wphase = 0, xphase = 0;
      auto issue_w = [&]() {
        mbar_expect_tx(&w_full[ws], w_stage_bytes);
        if (packed)   // tile-major weights: tile (n tile, k step) is one contiguous run of BN * 64 bytes
          bulk_load(w_base + ws * w_pitch,
                    w_packed + (static_cast<long long>(tile) * total_kb + kb0 + w_issued) * w_stage_bytes, w_stage_bytes,
                    &w_full[ws]);
        else
          tma_load_2d(w_base + ws * w_pitch, &tmW, &w_full[ws], (kb0 + w_issued) * BK, n0);
        ++w_issued;
        if (++ws == WST) {
          ws = 0;
          wphase ^= 1u;
        }
      };
      // weights do not depend on the kernel before this one: fill the ring before waiting for it
      while (w_issued < nk && w_issued < WST) issue_w();
      pdl_wait();
      // The two rings advance independently: whichever has a free slot gets its next load, so the (small)
      // activation loads never queue behind a weight slot that is still being multiplied.
      long long t0 = clock64();
      uint32_t spins = 0;
      while (x_issued < nk || w_issued < nk) {
        bool progress = false;
        if (w_issued < nk && mbar_test_wait(&w_empty[ws], wphase ^ 1u)) {
          issue_w();
          progress = true;
        }
        if (x_issued < nk && mbar_test_wait(&empty_x[xs], xphase ^ 1u)) {
          mbar_expect_tx(&full_x[xs], x_bytes);
#pragma unroll
          for (int rb = 0; rb < RB; ++rb)
            tma_load_2d(sX + xs * L.x_pitch + rb * kXBlock, &tmX, &full_x[xs], (kb0 + x_issued) * BK, m0 + rb * BM);
          ++x_issued;
          if (++xs == L.x_stages) {
            xs = 0;
            xphase ^= 1u;
          }
          progress = true;
        }
        if (progress) {
          t0 = clock64();
          spins = 0;
        } else if ((++spins & 255u) == 0u) {
          if (cta_abort) break;
          if (clock64() - t0 > kWaitCycleLimit) {
            cta_abort = 1;
            if (status) atomicCAS(status, kStatusOk, kStatusMbarTimeout);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, static_cast<uint32_t>(BN), 1, 1, 0, 0);   // bf16 x bf16 -> fp32
      int xs = 0, cs = 0;
      uint32_t xphase = 0, cphase = 0;
      for (int i = 0; i < nk; ++i) {
        if (!mbar_wait(&full_x[xs], xphase, &cta_abort, status)) break;
        if (!mbar_wait(&full_c[cs], cphase, &cta_abort, status)) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(sX + xs * L.x_pitch);
        const uint32_t b_base = smem_u32(sC + cs * L.c_pitch);
        if (flags & 1) {        // measurement aid: consume the stages without multiplying
          mbar_arrive(&empty_x[xs]);
          mbar_arrive(&empty_c[cs]);
        } else {
#pragma unroll
          for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_f16(tmem_base + static_cast<uint32_t>(rb * kMaxBN),
                       umma_smem_desc_sw128(a_base + rb * kXBlock + k * 32, 16, 1024),
                       umma_smem_desc_sw128(b_base + k * 32, 16, 1024), idesc, (i | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_x[xs]);
          umma_commit(&empty_c[cs]);
        }
        if (++xs == L.x_stages) {
          xs = 0;
          xphase ^= 1u;
        }
        if (++cs == CST) {
          cs = 0;
          cphase ^= 1u;
        }
      }
      umma_commit(&acc_bar);
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------ fp8 -> bf16 conversion warps
    if (FP8) {
      // Four groups of two warps; group g converts the stages i = g, g + 4, ... into converted-tile slot g, which it
      // owns. Several stages are therefore in conversion at once and the per-stage hand-over costs (barrier waits,
      // the proxy fence, the arrivals) are paid once per 16 .. 32 chunks of a thread instead of once per 4 .. 7.
      const int cw = warp - 6;
      const int grp = cw >> 1;                     // 0 .. kConvGroups - 1
      const int t = (cw & 1) * 32 + lane;          // 0 .. 63 within the group
      const int tall = cw * 32 + lane;             // 0 .. 255 over all conversion warps
      // thread t converts the 16-byte output chunk c = t & 7 of rows (t >> 3) + 8 j: eight fp8 bytes in, eight bf16 out
      const int c = t & 7;
      const int r0 = t >> 3;
      const int rblk0 = n0 >> 7;
      // the block scales of this CTA's rows and K slice, times 2^120, as packed bf16 pairs: once, into shared memory
      const int kblk_first = (kb0 * BK) >> 7;
      const int n_kblk = nk > 0 ? ((((kb0 + nk) * BK + 127) >> 7) - kblk_first) : 0;
      for (int e = tall; e < 3 * n_kblk && e < 3 * kMaxScaleSteps; e += 32 * kConvWarps) {
        const int b3 = e / n_kblk, kk = e - b3 * n_kblk;
        const float sc = __ldg(w_scale + static_cast<long long>(min(rblk0 + b3, scale_rows - 1)) * scale_cols +
                               min(kblk_first + kk, scale_cols - 1)) * 1.329227995784916e36f;   // 2^120
        const __nv_bfloat162 s2 = __float2bfloat162_rn(sc);
        s_scale[b3 * kMaxScaleSteps + kk] = *reinterpret_cast<const uint32_t*>(&s2);
      }
      asm volatile("bar.sync 2, %0;" ::"n"(32 * kConvWarps) : "memory");   // conversion warps only
      uint8_t* out = sC + grp * L.c_pitch;
      uint32_t cphase = 0;
      for (int i = grp; i < nk; i += kConvGroups) {
        const int rs = i % L.r_stages;
        const uint32_t rphase = static_cast<uint32_t>(i / L.r_stages) & 1u;
        bool ok = mbar_wait(&full_r[rs], rphase, &cta_abort, status);
        ok = ok && mbar_wait(&empty_c[grp], cphase ^ 1u, &cta_abort, status);
        if (!__all_sync(0xffffffffu, ok ? 1 : 0)) break;
        const uint8_t* raw = sR + rs * L.r_pitch;
        const int kk = min((((kb0 + i) * BK) >> 7) - kblk_first, kMaxScaleSteps - 1);
        const uint32_t sb[3] = {s_scale[kk], s_scale[kMaxScaleSteps + kk], s_scale[2 * kMaxScaleSteps + kk]};
#pragma unroll 4
        for (int r = r0; r < BN; r += 8) {
          const int rb = ((n0 + r) >> 7) - rblk0;
          const uint32_t sbits = rb == 0 ? sb[0] : (rb == 1 ? sb[1] : sb[2]);
          const uint2 b = *reinterpret_cast<const uint2*>(raw + r * BK + c * 8);
          uint4 o;
          o.x = mul_bf16x2(e4m3x2_to_bf16x2_rebased(__byte_perm(b.x, 0u, 0x4140u)), sbits);
          o.y = mul_bf16x2(e4m3x2_to_bf16x2_rebased(__byte_perm(b.x, 0u, 0x4342u)), sbits);
          o.z = mul_bf16x2(e4m3x2_to_bf16x2_rebased(__byte_perm(b.y, 0u, 0x4140u)), sbits);
          o.w = mul_bf16x2(e4m3x2_to_bf16x2_rebased(__byte_perm(b.y, 0u, 0x4342u)), sbits);
          *reinterpret_cast<uint4*>(out + r * 128 + ((c ^ (r & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();                // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&full_c[grp]);
          mbar_arrive(&empty_r[rs]);
        }
        cphase ^= 1u;
      }
    }
  }

  // ---------------------------------------------------------------- epilogue (warps 2..5)
  // Only the batch rows that exist are moved: a 16-row batch occupies one warp's lanes, the other three have nothing
  // to do. Without a K split the bf16 result goes from the accumulator registers straight to global memory; with one,
  // every CTA parks its fp32 partial rows in shared memory (over the idle rings) and sums an equal share of the rows
  // from all S partials through distributed shared memory, several vectors in flight per thread.
  const int part_pitch = BN * 4 + 16;            // fp32 partial row, padded against bank conflicts
  const int m_valid = min(M - m0, RB * BM);      // batch rows of this CTA that exist
  if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = mbar_wait(&acc_bar, 0, &cta_abort, status);
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    tc_fence_after();
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
      const int rows_here = m_valid - rb * BM;
      if (q * 32 >= rows_here) continue;         // warp-uniform
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(rb * kMaxBN);
      if (S == 1) {
        const int grow = m0 + rb * BM + row;
        __nv_bfloat16* yrow = Y + static_cast<long long>(grow) * ldy + n0;
        const bool vec_ok = (ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          if (warp_ok && nk > 0) {
            tmem_ld_32x16(t_row + static_cast<uint32_t>(c), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
          if (row < rows_here) {
            if (vec_ok && n0 + c + 16 <= N) {
              uint4 o0, o1;
              o0.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
              o0.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
              o0.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
              o0.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
              o1.x = pack_bf16x2(__uint_as_float(r[8]), __uint_as_float(r[9]));
              o1.y = pack_bf16x2(__uint_as_float(r[10]), __uint_as_float(r[11]));
              o1.z = pack_bf16x2(__uint_as_float(r[12]), __uint_as_float(r[13]));
              o1.w = pack_bf16x2(__uint_as_float(r[14]), __uint_as_float(r[15]));
              *reinterpret_cast<uint4*>(yrow + c) = o0;
              *reinterpret_cast<uint4*>(yrow + c + 8) = o1;
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n0 + c + i < N) yrow[c + i] = __float2bfloat16(__uint_as_float(r[i]));
            }
          }
        }
      } else {
        uint8_t* prow = smem + (rb * BM + row) * part_pitch;
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          if (warp_ok && nk > 0) {
            tmem_ld_32x16(t_row + static_cast<uint32_t>(c), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(prow + (c + i) * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (S > 1) {
    cluster_sync_all();
    if (warp >= 2 && warp < 6) {
      // CTA `slice` sums an equal share of the existing batch rows from all S partial tiles
      const int rows_per = (m_valid + S - 1) / S;
      const int row_lo = slice * rows_per;
      const int row_hi = min(m_valid, row_lo + rows_per);
      const int t = (warp - 2) * 32 + lane;        // 0 .. 127
      const int vec_per_row = BN / 4;
      const int total = max(0, row_hi - row_lo) * vec_per_row;
      const bool vec_ok = (ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 7) == 0);
      constexpr int U = S >= 8 ? 2 : 4;            // vectors per thread and pass: U * S remote loads in flight
      for (int it0 = t; it0 < total; it0 += 128 * U) {
        float4 v[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int it = it0 + u * 128;
          if (it < total) {
            const int rr = it / vec_per_row;
            const uint32_t local = smem_u32(smem + (row_lo + rr) * part_pitch + (it - rr * vec_per_row) * 16);
#pragma unroll
            for (int r = 0; r < S; ++r) v[u][r] = ld_cluster_f4(map_to_cta(local, static_cast<uint32_t>(r)));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int it = it0 + u * 128;
          if (it >= total) break;
          const int rr = it / vec_per_row;
          const int cv = it - rr * vec_per_row;
          float4 acc = v[u][0];
#pragma unroll
          for (int r = 1; r < S; ++r) {
            acc.x += v[u][r].x;
            acc.y += v[u][r].y;
            acc.z += v[u][r].z;
            acc.w += v[u][r].w;
          }
          const int col = n0 + cv * 4;
          __nv_bfloat16* dst = Y + static_cast<long long>(m0 + row_lo + rr) * ldy + col;
          if (vec_ok && col + 4 <= N) {
            uint2 o;
            o.x = pack_bf16x2(acc.x, acc.y);
            o.y = pack_bf16x2(acc.z, acc.w);
            *reinterpret_cast<uint2*>(dst) = o;
          } else {
            const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int j = 0; j < 4; ++j)
              if (col + j < N) dst[j] = __float2bfloat16(a4[j]);
          }
        }
      }
    }
    // nobody leaves (and frees its shared memory) before every CTA of the cluster has finished reading
    cluster_sync_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, RB * kMaxBN);
  }
}

template <int S, bool FP8, int RB>
cudaError_t config_wq(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* at, int grid_x, int grid_y, int pdl, cudaStream_t s) {
  auto kern = gemm_decode_wq_kernel<S, FP8, RB>;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    attr.set();
  }
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(static_cast<unsigned>(grid_x), static_cast<unsigned>(grid_y), 1);
  cfg->blockDim = dim3(kThreads, 1, 1);
  cfg->dynamicSmemBytes = kSmemBudget;
  cfg->stream = s;
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  int n_attr = 1;
  if (pdl) {
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    n_attr = 2;
  }
  cfg->attrs = at;
  cfg->numAttrs = n_attr;
  return cudaSuccess;
}

template <int S, bool FP8, int RB>
int launch_wq(const CUtensorMap& tx, const CUtensorMap& tw, const void* w_packed, const float* w_scale, void* Y, int M,
              int N, int K,
              long long ldy, int BN, int scale_cols, int scale_rows, const Layout& L, int pdl, int flags,
              cudaStream_t s) {
  flags |= (pdl >> 4) & 1;    // pdl bit 4: measurement aid (stages consumed without multiplying)
  pdl &= 1;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  const int tiles = (N + BN - 1) / BN;
  cudaError_t e = config_wq<S, FP8, RB>(&cfg, at, tiles * S, (M + RB * BM - 1) / (RB * BM), pdl, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_decode_wq_kernel<S, FP8, RB>, tx, tw,
                                             static_cast<const uint8_t*>(w_packed), w_scale,
                                             static_cast<__nv_bfloat16*>(Y), M, N, K, ldy, BN, scale_cols, scale_rows, L,
                                             flags, device_status_word()));
}

// CTAs of this kernel that can be resident at once when launched as clusters of S: a GPC takes whole clusters only,
// so the number is below the SM count for S > 1. Asked from the runtime once per (device, S, weight format).
template <int S, bool FP8>
int resident_ctas() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count();
  if (cached[dev] == 0) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    int clusters = 0;
    if (config_wq<S, FP8, 1>(&cfg, at, S * 64, 1, 0, nullptr) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&clusters, gemm_decode_wq_kernel<S, FP8, 1>, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sm_count() / S * 3 / 4;
    }
    cached[dev] = clusters * S;
  }
  return cached[dev];
}

int resident_ctas_for(int split, bool fp8) {
  switch (split) {
    case 1: return fp8 ? resident_ctas<1, true>() : resident_ctas<1, false>();
    case 2: return fp8 ? resident_ctas<2, true>() : resident_ctas<2, false>();
    case 4: return fp8 ? resident_ctas<4, true>() : resident_ctas<4, false>();
    default: return fp8 ? resident_ctas<8, true>() : resident_ctas<8, false>();
  }
}

// Tile width and K split for N weight rows and `kb` K steps. The kernel is not persistent, and a second wave of
// CTAs costs about as much as the first, so only plans whose CTAs are all resident at once are considered; among
// them the one that keeps the most SMs streaming wins (K slices of fewer than 16 steps and very narrow tiles are
// marked down: their fixed costs show). Measured on B200 at 16 .. 256 rows: 138 CTAs of 208 rows for N = 28672,
// 32 x 4 CTAs of 128 rows for N = 4096.
bool layout_ok(const Layout& L, bool fp8, int bn, int rb) {
  return (fp8 ? L.r_stages : L.c_stages) >= (fp8 ? kConvGroups : 3) && rb * BM * (bn * 4 + 16) <= kSmemBudget - 1024;
}

// One candidate family: tile widths and K splits for a given number of row blocks per CTA. Returns the score of the
// best single-wave plan (< 0 if there is none).
double plan_family(int M, int N, int kb, bool fp8, int fixed_bn, int rb, int* bn_out, int* split_out) {
  const int row_ctas = (M + rb * BM - 1) / (rb * BM);
  double best = -1.0;
  for (int s : {1, 2, 4, 8}) {
    if (s > 1 && kb / s < 8) break;
    int cap = resident_ctas_for(s, fp8);
    const int sms = sm_count();
    const int safe = s == 1 ? sms : (s == 2 ? sms - sms % 16 : (s == 4 ? (sms / 18) * 16 : (sms / 18) * 16 - 16));
    if (cap <= 0 || cap > sms) cap = safe;
    for (int bn = 256; bn >= 32; bn -= 16) {
      if (fixed_bn > 0 && bn != fixed_bn) continue;
      const Layout L = make_layout(M, bn, fp8, rb);
      if (!layout_ok(L, fp8, bn, rb)) continue;
      const int tiles = (N + bn - 1) / bn;
      const int ctas = tiles * s * row_ctas;
      if (ctas > cap) continue;
      const double useful = static_cast<double>(N) / (static_cast<double>(tiles) * bn);
      // at equal CTA counts the plan with fewer K steps per CTA wins (a step costs about the same whatever its width)
      double score = static_cast<double>(ctas) * useful - 0.02 * ((kb + s - 1) / s);
      if (kb / s < 16) score *= 0.85;
      if (s == 8) score *= 0.9;
      if (bn < 64) score *= 0.85;
      if (score > best + 1e-9) {
        best = score;
        *bn_out = bn;
        *split_out = s;
      }
    }
  }
  return best;
}

// Tile width, K split and row blocks per CTA for M batch rows, N weight rows and `kb` K steps. The kernel is not
// persistent, and a second wave of CTAs costs about as much as the first, so only plans whose CTAs are all resident
// at once are considered; among them the one that keeps the most SMs streaming wins (K slices of fewer than 16 steps
// and very narrow tiles are marked down: their fixed costs show). 129 .. 256 rows: one CTA takes both 128-row blocks
// when the rings still fit, so the weights are streamed once. Measured on B200 at 16 .. 128 rows: 138 CTAs of 208
// rows for N = 28672, 32 x 4 CTAs of 128 rows for N = 4096.
void plan_tiles(int M, int N, int kb, bool fp8, int fixed_bn, int* bn_out, int* split_out, int* rb_out) {
  int bn = 128, s = 1, rb = 1;
  double best = -1.0;
  if (M > BM && M <= 2 * BM) {
    int b2 = 0, s2 = 0;
    const double sc2 = plan_family(M, N, kb, fp8, fixed_bn, 2, &b2, &s2);
    if (sc2 > 0.0) {
      best = sc2;
      bn = b2;
      s = s2;
      rb = 2;
    }
  }
  if (best < 0.0) {
    int b1 = 0, s1 = 0;
    const double sc1 = plan_family(M, N, kb, fp8, fixed_bn, 1, &b1, &s1);
    if (sc1 > 0.0) {
      best = sc1;
      bn = b1;
      s = s1;
      rb = 1;
    }
  }
  if (best < 0.0) {   // more tiles than resident CTAs at every width: several waves of the widest tile that has room
    rb = (M > BM && M <= 2 * BM && !fp8) ? 2 : 1;
    bn = fixed_bn > 0 ? fixed_bn : 32;
    s = 1;
    for (int b = 256; b >= 32 && fixed_bn <= 0; b -= 16) {
      if (layout_ok(make_layout(M, b, fp8, rb), fp8, b, rb)) {
        bn = b;
        break;
      }
    }
  }
  *bn_out = bn;
  *split_out = s;
  *rb_out = rb;
}

}  // namespace
}  // namespace tsb

// Y [M, N] bf16 (row stride ldy) = X [M, K] bf16 (row stride ldx) * W [N, K]^T.
//   w_fp8 = 0: W is bf16 [N, K] (row stride ldw elements);  w_scale ignored.
//   w_fp8 = 1: W is E4M3 bytes [N, K] (row stride ldw bytes), w_scale is fp32 [ceil(N/128), ceil(K/128)] row-major:
//              W_real[n, k] = e4m3(W[n, k]) * w_scale[n / 128, k / 128]; scales below 2^7 in magnitude.
//   w_fp8 = 2: the same E4M3 weights pre-packed tile-major for this kernel: [ceil(N / bn)][K / 64][bn][64] bytes
//              (rows past N zero), so that every tile a CTA streams is one contiguous run of bn * 64 bytes in HBM
//              instead of bn 64-byte pieces a row apart; `bn` must be the width the weights were packed with.
//   K % 64 == 0 for fp8 (16 for bf16), rows 16-byte aligned. bn / split: 0 = chosen here; otherwise bn a multiple of
//   16 in [32, 256], split in {1, 2, 4, 8}. pdl != 0: launch with programmatic stream serialisation (the kernel
//   may start while the previous kernel in the stream is still running; it waits for it before reading X).
TSB_EXPORT int tsb_gemm_decode_wq(const void* X, const void* W, const float* w_scale, void* Y, int M, int N, int K,
                                  long long ldx, long long ldw, long long ldy, int w_fp8, int bn, int split, int pdl,
                                  void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || !X || !W || !Y || w_fp8 < 0 || w_fp8 > 2) return -2;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldx % 8)) return -2;
  const bool fp8 = w_fp8 != 0, packed = w_fp8 == 2;
  if (packed ? (K % 64 || !w_scale || bn <= 0) : (fp8 ? (ldw % 16 || K % 64 || !w_scale) : (ldw % 8 || K % 16))) return -2;
  const int kb = (K + BK - 1) / BK;
  int rb = 1;
  {
    int pbn = 0, ps = 0, prb = 1;
    plan_tiles(M, N, kb, fp8, bn > 0 ? bn : 0, &pbn, &ps, &prb);
    if (bn <= 0) bn = pbn;
    if (split <= 0) split = ps;
    rb = prb;
  }
  if (bn < 32 || bn > kMaxBN || bn % 16 || (split != 1 && split != 2 && split != 4 && split != 8)) return -2;
  Layout L = make_layout(M, bn, fp8, rb);
  if (!layout_ok(L, fp8, bn, rb) && rb == 2) {   // a caller-given width that has no room for two row blocks
    rb = 1;
    L = make_layout(M, bn, fp8, rb);
  }
  if ((fp8 ? L.r_stages : L.c_stages) < (fp8 ? kConvGroups : 2) || rb * BM * (bn * 4 + 16) > kSmemBudget - 1024)
    return -2;   // no room for the rings at this width
  if (fp8 && (kb + split - 1) / split * BK / 128 + 2 > kMaxScaleSteps) return -2;
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, X, 2, M, K, ldx * 2, L.x_rows, BK, true)) return -3;
  bool ok;
  if (packed) {
    ok = make_tmap_2d(&tw, X, 2, M, K, ldx * 2, L.x_rows, BK, true);   // unused by the kernel: tiles come by bulk copy
  } else if (fp8) {
    ok = make_tmap_2d(&tw, W, 1, N, K, ldw, bn, BK, false);
  } else {
    ok = make_tmap_2d(&tw, W, 2, N, K, ldw * 2, bn, BK, true);
  }
  if (!ok) return -3;
  const int scale_cols = (K + 127) / 128, scale_rows = (N + 127) / 128;
  const int flags = packed ? 2 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TSB_WQ_ARGS tx, tw, W, w_scale, Y, M, N, K, ldy, bn, scale_cols, scale_rows, L, pdl, flags, s
#define TSB_WQ(S_)                                                                            \
  return fp8 ? (rb == 2 ? launch_wq<S_, true, 2>(TSB_WQ_ARGS) : launch_wq<S_, true, 1>(TSB_WQ_ARGS))  \
             : (rb == 2 ? launch_wq<S_, false, 2>(TSB_WQ_ARGS) : launch_wq<S_, false, 1>(TSB_WQ_ARGS))
  switch (split) {
    case 1: TSB_WQ(1);
    case 2: TSB_WQ(2);
    case 4: TSB_WQ(4);
    default: TSB_WQ(8);
  }
#undef TSB_WQ
#undef TSB_WQ_ARGS
}

// The plan the call above makes for a problem (host only): *bn (pass a positive value to fix the tile width, as for
// packed weights), *split, and the ring depth it leads to.
TSB_EXPORT int tsb_gemm_decode_wq_plan(int M, int N, int K, int w_fp8, int* bn, int* split, int* w_stages,
                                       int* resident) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || !bn || !split) return -2;
  const int fixed = *bn > 0 ? *bn : 0;
  int rb = 1;
  plan_tiles(M, N, (K + BK - 1) / BK, w_fp8 != 0, fixed, bn, split, &rb);
  const Layout L = make_layout(M, *bn, w_fp8 != 0, rb);
  if (w_stages) *w_stages = (w_fp8 ? L.r_stages : L.c_stages) * (rb == 2 ? -1 : 1);   // negative: two row blocks per CTA
  if (resident) *resident = resident_ctas_for(*split, w_fp8 != 0);   // what the runtime reports for that cluster size
  return 0;
}
