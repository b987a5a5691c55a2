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
//     2^-120, subnormals included) and one packed bf16 multiply by (scale * 2^120) restores it -- about 1.5
//     instructions per element, which keeps the conversion well under the HBM rate of one SM.
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
constexpr int kXStages = 4;       // activation ring [128 x 64] bf16, 16 KB each
constexpr int kCStagesF8 = 2;     // converted-weight ring (fp8 path), up to 32 KB each
constexpr int kRStages = 6;       // raw fp8 ring, up to 16 KB each
constexpr int kCStagesBf = 4;     // weight ring (bf16 path), up to 32 KB each
constexpr int kConvWarps = 4;
constexpr int kThreads = 192 + 32 * kConvWarps;   // producer, MMA, 4 epilogue warps, 4 conversion warps
constexpr int kXBytes = BM * BK * 2;
constexpr int kMaxBN = 256;

__host__ __device__ constexpr int smem_bytes_for(bool fp8) {
  return kXStages * kXBytes + (fp8 ? kCStagesF8 * kMaxBN * BK * 2 + kRStages * kMaxBN * BK : kCStagesBf * kMaxBN * BK * 2) +
         1024;
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
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Two E4M3 bytes (low 16 bits of `b2`) -> packed bf16x2 holding value * 2^-120 each.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_rebased(uint32_t b2) {
  const uint32_t lo = b2 & 0xffu, hi = (b2 >> 8) & 0xffu;
  const uint32_t l = ((lo & 0x7fu) << 4) | ((lo & 0x80u) << 8);
  const uint32_t h = ((hi & 0x7fu) << 4) | ((hi & 0x80u) << 8);
  return l | (h << 16);
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int S, bool FP8>
__global__ void __launch_bounds__(kThreads, 1)
gemm_decode_wq_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                      const float* __restrict__ w_scale, __nv_bfloat16* __restrict__ Y, int M, int N, int K,
                      long long ldy, int BN, int scale_cols, int scale_rows, int* status) {
  constexpr int CST = FP8 ? kCStagesF8 : kCStagesBf;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sC = sX + kXStages * kXBytes;             // operand tiles of W: [BN rows][128 B], swizzled
  uint8_t* sR = sC + CST * kMaxBN * BK * 2;          // raw fp8 tiles: [BN rows][64 B], linear (fp8 path only)
  __shared__ __align__(8) uint64_t full_x[kXStages], empty_x[kXStages];
  __shared__ __align__(8) uint64_t full_c[kCStagesBf], empty_c[kCStagesBf];
  __shared__ __align__(8) uint64_t full_r[kRStages], empty_r[kRStages];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = static_cast<int>(cluster_ctarank());
  const int tile = static_cast<int>(blockIdx.x) / S;
  const int n0 = tile * BN;
  const int m0 = static_cast<int>(blockIdx.y) * BM;
  const int total_kb = (K + BK - 1) / BK;
  const int kb_per = (total_kb + S - 1) / S;
  const int kb0 = slice * kb_per;
  const int kb1 = min(total_kb, kb0 + kb_per);
  const int nk = max(0, kb1 - kb0);
  const uint32_t w_stage_bytes = static_cast<uint32_t>(BN) * BK * (FP8 ? 1 : 2);

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kXStages; ++s) {
      mbar_init(&full_x[s], 1);
      mbar_init(&empty_x[s], 1);
    }
    for (int s = 0; s < kCStagesBf; ++s) {
      mbar_init(&full_c[s], FP8 ? kConvWarps : 1);
      mbar_init(&empty_c[s], 1);
    }
    for (int s = 0; s < kRStages; ++s) {
      mbar_init(&full_r[s], 1);
      mbar_init(&empty_r[s], kConvWarps);
    }
    mbar_init(&acc_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
    pdl_launch_dependents();     // whatever follows in the stream may start its own prologue
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, kMaxBN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      constexpr int WST = FP8 ? kRStages : kCStagesBf;
      uint64_t* w_full = FP8 ? full_r : full_c;
      uint64_t* w_empty = FP8 ? empty_r : empty_c;
      uint8_t* w_base = FP8 ? sR : sC;
      const uint32_t w_pitch = FP8 ? kMaxBN * BK : kMaxBN * BK * 2;
      int w_issued = 0, ws = 0;
      uint32_t wphase = 0;
      bool ok = true;
      auto issue_w = [&]() {
        ok = mbar_wait(&w_empty[ws], wphase ^ 1u, &cta_abort, status);
        if (!ok) return;
        mbar_expect_tx(&w_full[ws], w_stage_bytes);
        tma_load_2d(w_base + ws * w_pitch, &tmW, &w_full[ws], (kb0 + w_issued) * BK, n0);
        ++w_issued;
        if (++ws == WST) {
          ws = 0;
          wphase ^= 1u;
        }
      };
      // weights do not depend on the kernel before this one: fill the ring before waiting for it
      while (ok && w_issued < nk && w_issued < WST) issue_w();
      pdl_wait();
      int xs = 0;
      uint32_t xphase = 0;
      for (int i = 0; i < nk && ok; ++i) {
        ok = mbar_wait(&empty_x[xs], xphase ^ 1u, &cta_abort, status);
        if (!ok) break;
        mbar_expect_tx(&full_x[xs], kXBytes);
        tma_load_2d(sX + xs * kXBytes, &tmX, &full_x[xs], (kb0 + i) * BK, m0);
        if (++xs == kXStages) {
          xs = 0;
          xphase ^= 1u;
        }
        if (w_issued < nk) issue_w();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(BM, static_cast<uint32_t>(BN), 1, 1, 0, 0);
      int xs = 0, cs = 0;
      uint32_t xphase = 0, cphase = 0;
      for (int i = 0; i < nk; ++i) {
        if (!mbar_wait(&full_x[xs], xphase, &cta_abort, status)) break;
        if (!mbar_wait(&full_c[cs], cphase, &cta_abort, status)) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(sX + xs * kXBytes);
        const uint32_t b_base = smem_u32(sC + cs * (kMaxBN * BK * 2));
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_f16(tmem_base, umma_smem_desc_sw128(a_base + k * 32, 16, 1024),
                   umma_smem_desc_sw128(b_base + k * 32, 16, 1024), idesc, (i | k) != 0 ? 1u : 0u);
        umma_commit(&empty_x[xs]);
        umma_commit(&empty_c[cs]);
        if (++xs == kXStages) {
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
      const int cw = warp - 6;
      const int t = cw * 32 + lane;              // 0 .. 127
      int rs = 0, cs = 0;
      uint32_t rphase = 0, cphase = 0;
      const int items = BN * 8;                  // 16-byte output chunks per stage
      for (int i = 0; i < nk; ++i) {
        bool ok = mbar_wait(&full_r[rs], rphase, &cta_abort, status);
        ok = ok && mbar_wait(&empty_c[cs], cphase ^ 1u, &cta_abort, status);
        if (!__all_sync(0xffffffffu, ok ? 1 : 0)) break;
        const uint8_t* raw = sR + rs * (kMaxBN * BK);
        uint8_t* out = sC + cs * (kMaxBN * BK * 2);
        const int kblk = min(((kb0 + i) * BK) >> 7, scale_cols - 1);
        for (int it = t; it < items; it += 32 * kConvWarps) {
          const int r = it >> 3, c = it & 7;
          const int rblk = min((n0 + r) >> 7, scale_rows - 1);
          const float sc = __ldg(w_scale + static_cast<long long>(rblk) * scale_cols + kblk) * 1.329227995784916e36f;  // 2^120
          const __nv_bfloat162 s2 = __float2bfloat162_rn(sc);
          const uint32_t sbits = *reinterpret_cast<const uint32_t*>(&s2);
          const uint2 b = *reinterpret_cast<const uint2*>(raw + r * BK + c * 8);
          uint4 o;
          o.x = mul_bf16x2(e4m3x2_to_bf16x2_rebased(b.x), sbits);
          o.y = mul_bf16x2(e4m3x2_to_bf16x2_rebased(b.x >> 16), sbits);
          o.z = mul_bf16x2(e4m3x2_to_bf16x2_rebased(b.y), sbits);
          o.w = mul_bf16x2(e4m3x2_to_bf16x2_rebased(b.y >> 16), sbits);
          *reinterpret_cast<uint4*>(out + r * 128 + ((c ^ (r & 7)) << 4)) = o;
        }
        fence_proxy_async_smem();                // generic-proxy stores -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&full_c[cs]);
          mbar_arrive(&empty_r[rs]);
        }
        if (++rs == kRStages) {
          rs = 0;
          rphase ^= 1u;
        }
        if (++cs == CST) {
          cs = 0;
          cphase ^= 1u;
        }
      }
    }
  }

  // ---------------------------------------------------------------- epilogue (warps 2..5)
  const int part_pitch = BN * 4 + 16;            // fp32 partial row, padded against bank conflicts
  if (warp >= 2 && warp < 6) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = mbar_wait(&acc_bar, 0, &cta_abort, status);
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    tc_fence_after();
    // the rings are idle now: park this CTA's partial tile over them
    uint8_t* prow = smem + row * part_pitch;
    for (int c = 0; c < BN; c += 32) {
      uint32_t r[32];
      if (warp_ok && nk > 0) {
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(c), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
#pragma unroll
      for (int i = 0; i < 32; i += 4)
        if (c + i < BN) *reinterpret_cast<uint4*>(prow + (c + i) * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    }
    tc_fence_before();
  }
  __syncthreads();
  cluster_sync_all();

  if (warp >= 2 && warp < 6) {
    // CTA `slice` sums batch rows [slice * 128 / S, (slice + 1) * 128 / S) of all S partial tiles
    constexpr int kRows = BM / S;
    const int t = (warp - 2) * 32 + lane;        // 0 .. 127
    const int vec_per_row = BN / 4;
    const int total = kRows * vec_per_row;
    const bool vec_ok = (ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 7) == 0);
    for (int it = t; it < total; it += 128) {
      const int rr = it / vec_per_row;
      const int cv = it - rr * vec_per_row;
      const int row = slice * kRows + rr;
      const int grow = m0 + row;
      if (grow >= M) break;                      // rows are visited in increasing order
      const uint32_t local = smem_u32(smem + row * part_pitch + cv * 16);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < S; ++r) {
        const float4 v = ld_cluster_f4(map_to_cta(local, static_cast<uint32_t>(r)));
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      const int col = n0 + cv * 4;
      __nv_bfloat16* dst = Y + static_cast<long long>(grow) * ldy + col;
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

  // nobody leaves (and frees its shared memory) before every CTA of the cluster has finished reading
  cluster_sync_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kMaxBN);
  }
}

template <int S, bool FP8>
int launch_wq(const CUtensorMap& tx, const CUtensorMap& tw, const float* w_scale, void* Y, int M, int N, int K,
              long long ldy, int BN, int scale_cols, int scale_rows, int pdl, cudaStream_t s) {
  auto kern = gemm_decode_wq_kernel<S, FP8>;
  static PerDeviceFlag attr;
  constexpr int smem = smem_bytes_for(FP8);
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  const int tiles = (N + BN - 1) / BN;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tiles * S), static_cast<unsigned>((M + BM - 1) / BM), 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[2];
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
  cfg.attrs = at;
  cfg.numAttrs = n_attr;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, tx, tw, w_scale, static_cast<__nv_bfloat16*>(Y), M, N, K, ldy,
                                             BN, scale_cols, scale_rows, device_status_word()));
}

// Tile width and K split for N weight rows and `kb` K steps: fill the SMs with one wave of CTAs when possible.
void plan_tiles(int N, int kb, int row_blocks, int sms, int* bn_out, int* split_out) {
  int best_bn = 128, best_s = 1;
  double best = -1.0;
  for (int s : {1, 2, 4, 8}) {
    if (s > kb) break;
    for (int bn = 256; bn >= 32; bn -= 16) {
      if ((bn * 4 + 16) * BM > smem_bytes_for(true) - 1024) continue;
      const int ctas = ((N + bn - 1) / bn) * s * row_blocks;
      const int waves = (ctas + sms - 1) / sms;
      // streamed weight rows per wave-slot, discounted by the padding of the last tile and by short K slices
      const double useful = static_cast<double>(N) / (static_cast<double>((N + bn - 1) / bn) * bn);
      const double eff = static_cast<double>(ctas) / (static_cast<double>(waves) * sms) * useful *
                         (kb / s >= 8 ? 1.0 : 0.6 + 0.05 * (kb / s)) * (bn >= 64 ? 1.0 : 0.8);
      if (eff > best + 1e-9) {
        best = eff;
        best_bn = bn;
        best_s = s;
      }
    }
  }
  *bn_out = best_bn;
  *split_out = best_s;
}

}  // namespace
}  // namespace tsb

// Y [M, N] bf16 (row stride ldy) = X [M, K] bf16 (row stride ldx) * W [N, K]^T.
//   w_fp8 = 0: W is bf16 [N, K] (row stride ldw elements);  w_scale ignored.
//   w_fp8 = 1: W is E4M3 bytes [N, K] (row stride ldw bytes), w_scale is fp32 [ceil(N/128), ceil(K/128)] row-major:
//              W_real[n, k] = e4m3(W[n, k]) * w_scale[n / 128, k / 128]; scales below 2^7 in magnitude.
//   K % 64 == 0 for fp8 (16 for bf16), rows 16-byte aligned. bn / split: 0 = chosen here; otherwise bn a multiple of
//   16 in [32, 256], split in {1, 2, 4, 8}. pdl != 0: launch with programmatic stream serialisation (the kernel
//   may start while the previous kernel in the stream is still running; it waits for it before reading X).
TSB_EXPORT int tsb_gemm_decode_wq(const void* X, const void* W, const float* w_scale, void* Y, int M, int N, int K,
                                  long long ldx, long long ldw, long long ldy, int w_fp8, int bn, int split, int pdl,
                                  void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || !X || !W || !Y) return -2;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldx % 8)) return -2;
  if (w_fp8 ? (ldw % 16 || K % 64 || !w_scale) : (ldw % 8 || K % 16)) return -2;
  const int kb = (K + BK - 1) / BK;
  const int row_blocks = (M + BM - 1) / BM;
  if (bn <= 0 || split <= 0) plan_tiles(N, kb, row_blocks, sm_count(), &bn, &split);
  if (bn < 32 || bn > kMaxBN || bn % 16 || (split != 1 && split != 2 && split != 4 && split != 8)) return -2;
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, X, 2, M, K, ldx * 2, BM, BK, true)) return -3;
  if (w_fp8 ? !make_tmap_2d(&tw, W, 1, N, K, ldw, bn, BK, false) : !make_tmap_2d(&tw, W, 2, N, K, ldw * 2, bn, BK, true))
    return -3;
  const int scale_cols = (K + 127) / 128, scale_rows = (N + 127) / 128;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TSB_WQ(S_)                                                                                                    \
  return w_fp8 ? launch_wq<S_, true>(tx, tw, w_scale, Y, M, N, K, ldy, bn, scale_cols, scale_rows, pdl, s)         \
               : launch_wq<S_, false>(tx, tw, w_scale, Y, M, N, K, ldy, bn, scale_cols, scale_rows, pdl, s)
  switch (split) {
    case 1: TSB_WQ(1);
    case 2: TSB_WQ(2);
    case 4: TSB_WQ(4);
    default: TSB_WQ(8);
  }
#undef TSB_WQ
}
