// FlashAttention backward on tcgen05 tensor cores (bf16, head_dim 64 or 128, causal or full, GQA).
//
// The reference has no attention backward kernel: it differentiates the matmul -> softmax -> matmul
// composite and keeps the [B, H, S, S] probabilities (src/ops/cpu/Attention.cpp:232-242,272-303). This
// kernel recomputes P from the saved log-sum-exp and never materialises an S x S tensor.
//
// One CTA per (128-key tile, KV head, batch). It keeps K_j and V_j in shared memory and the dK_j / dV_j
// accumulators in TMEM (fp32) while it walks over every query tile that can see the key tile, for each of
// the H / Hkv query heads that share the KV head (so the GQA reduction costs nothing). Per step:
//   S  = Q_i K_j^T              (tensor core -> TMEM)         dP = dO_i V_j^T        (tensor core -> TMEM)
//   P  = exp2(S * c - lse_i)    (threads, one query row each) dS = P * (dP - delta_i) * scale
//   dV_j += P^T dO_i            dK_j += dS^T Q_i              dQ_i  = dS K_j         (tensor core)
// P and dS are written once to 128-byte-swizzled shared memory and read by the tensor core both K-major
// (for dQ) and M-major (for dV, dK) through different descriptors. dQ_i tiles are added into an fp32
// scratch tensor with vector atomics and converted to bf16 by a small second kernel.
// delta_i = rowsum(dO_i * O_i) comes from a small pre-pass.
#include "common.cuh"

namespace tsb {

bool make_bshd_tmap(CUtensorMap* out, const void* base, int B, int S, int Hn, int D, long long sb, long long ss,
                    long long sh, int box_rows);

namespace {

constexpr int kBwdThreads = 192;
constexpr int BT = 128;  // tile edge (queries and keys)

template <int D>
struct BwdCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kPBytes = BT * BT * 2;
  static constexpr int kSmemBytes = 4 * kTileBytes + 2 * kPBytes + 1024;
  static constexpr int kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;
};

struct BwdParams {
  const float* lse;    // [B, H, Sq]
  const float* delta;  // [B, H, Sq]
  float* dq_acc;       // [B, Sq, H, D] fp32, zero-initialised
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int B, Sq, Sk, H, Hkv;
  long long dk_sb, dk_ss, dk_sh, dv_sb, dv_ss, dv_sh;
  float scale, scale_log2;
  int causal;
  int* status;
};

template <int ROWS>
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int ks) {
  const int half = ks >> 2;
  return umma_smem_desc_sw128(base + half * (ROWS * 128) + (ks & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int ks, uint32_t half_stride) {
  return umma_smem_desc_sw128(base + ks * 2048, half_stride, 1024);
}

// Store 32 consecutive bf16 (as 16 packed words) of `row` starting at column c*32 into a [128 x 128] tile
// kept as two 64-column halves with the 128-byte swizzle.
__device__ __forceinline__ void store_row_chunk_sw128(uint8_t* tile, int row, int c, const uint32_t (&packed)[16]) {
  uint8_t* prow = tile + (c >> 1) * 16384 + row * 128;
#pragma unroll
  for (int q4 = 0; q4 < 4; ++q4) {
    const int chunk = (c & 1) * 4 + q4;
    const int sw = chunk ^ (row & 7);
    *reinterpret_cast<uint4*>(prow + sw * 16) =
        make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
  }
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, BwdParams p) {
  using Cfg = BwdCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::kTileBytes;
  uint8_t* sQ = sV + Cfg::kTileBytes;
  uint8_t* sDO = sQ + Cfg::kTileBytes;
  uint8_t* sP = sDO + Cfg::kTileBytes;
  uint8_t* sDS = sP + Cfg::kPBytes;

  __shared__ __align__(8) uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_full, dq_full, dq_read;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.x;  // key tile
  const int hk = blockIdx.y;
  const int b = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int c0 = j * BT;
  const int offset = p.Sk - p.Sq;
  const int n_q = (p.Sq + BT - 1) / BT;
  int i_min = 0;
  if (p.causal) {
    const int first = c0 - offset;  // first query row that can see key c0
    i_min = first <= 0 ? 0 : first / BT;
  }
  const int per_head = n_q > i_min ? n_q - i_min : 0;
  const int n_iter = per_head * G;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    mbar_init(&kv_full, 1);
    mbar_init(&qdo_full, 1);
    mbar_init(&qdo_empty, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&pds_full, 128);
    mbar_init(&dq_full, 1);
    mbar_init(&dq_read, 128);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 5) {
    tmem_alloc(&tmem_base_smem, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(&kv_full, 2 * Cfg::kTileBytes);
#pragma unroll
      for (int hf = 0; hf < Cfg::kHalves; ++hf) {
        tma_load_4d(sK + hf * 16384, &tmK, &kv_full, hf * 64, c0, hk, b);
        tma_load_4d(sV + hf * 16384, &tmV, &kv_full, hf * 64, c0, hk, b);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int g = t / per_head;
        const int i = i_min + (t - g * per_head);
        const int h = hk * G + g;
        if (!mbar_wait(&qdo_empty, (t & 1) ^ 1u, &cta_abort, p.status)) break;
        mbar_expect_tx(&qdo_full, 2 * Cfg::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < Cfg::kHalves; ++hf) {
          tma_load_4d(sQ + hf * 16384, &tmQ, &qdo_full, hf * 64, i * BT, h, b);
          tma_load_4d(sDO + hf * 16384, &tmDO, &qdo_full, hf * 64, i * BT, h, b);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = umma_idesc(BT, BT, 1, 1, 0, 0);   // S, dP: both operands K-major
      constexpr uint32_t idesc_kv = umma_idesc(BT, D, 1, 1, 1, 1);   // dV, dK: both operands M/N-major
      constexpr uint32_t idesc_q = umma_idesc(BT, D, 1, 1, 0, 1);    // dQ: dS K-major, K N-major
      const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV), q_base = smem_u32(sQ), do_base = smem_u32(sDO);
      const uint32_t p_base = smem_u32(sP), ds_base = smem_u32(sDS);
      bool ok = mbar_wait(&kv_full, 0, &cta_abort, p.status);
      for (int t = 0; ok && t < n_iter; ++t) {
        const uint32_t ph = t & 1;
        if (!mbar_wait(&qdo_full, ph, &cta_abort, p.status)) break;
        if (!mbar_wait(&dq_read, ph ^ 1u, &cta_abort, p.status)) break;  // dQ columns alias dP
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16(tmem_base + Cfg::kColS, kmajor_desc<128>(q_base, ks), kmajor_desc<128>(k_base, ks), idesc_s, ks != 0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16(tmem_base + Cfg::kColDP, kmajor_desc<128>(do_base, ks), kmajor_desc<128>(v_base, ks), idesc_s,
                   ks != 0);
        umma_commit(&sdp_full);
        if (!mbar_wait(&pds_full, ph, &cta_abort, p.status)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)   // dV += P^T dO   (K = query rows)
          umma_f16(tmem_base + Cfg::kColDV, mnmajor_desc(p_base, ks, 16384), mnmajor_desc(do_base, ks, 16384), idesc_kv,
                   (t | ks) != 0);
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)   // dK += dS^T Q
          umma_f16(tmem_base + Cfg::kColDK, mnmajor_desc(ds_base, ks, 16384), mnmajor_desc(q_base, ks, 16384), idesc_kv,
                   (t | ks) != 0);
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks)   // dQ = dS K       (K = key rows)
          umma_f16(tmem_base + Cfg::kColDP, kmajor_desc<128>(ds_base, ks), mnmajor_desc(k_base, ks, 16384), idesc_q,
                   ks != 0);
        umma_commit(&qdo_empty);
        umma_commit(&dq_full);
      }
    }
  } else {
    // ---------------------------------------------------------------- compute warps 0..3
    const int row = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    bool ok = true;
    const float log2e = 1.4426950408889634f;
    for (int t = 0; t < n_iter; ++t) {
      const int g = t / per_head;
      const int i = i_min + (t - g * per_head);
      const int h = hk * G + g;
      const int qi = i * BT + row;
      const uint32_t ph = t & 1;
      float lse_l2 = 0.f, delta = 0.f;
      int vis = 0;
      if (qi < p.Sq) {
        const long long idx = (static_cast<long long>(b) * p.H + h) * p.Sq + qi;
        const float lse = p.lse[idx];
        delta = p.delta[idx];
        int lim = p.Sk - c0;
        if (p.causal) lim = min(lim, qi + offset - c0 + 1);
        vis = max(0, min(BT, lim));
        if (lse == -INFINITY) vis = 0;
        lse_l2 = lse * log2e;
      }
      const bool all_full = __all_sync(0xffffffffu, vis == BT) != 0;
      if (!mbar_wait(&sdp_full, ph, &cta_abort, p.status)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BT / 32; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColS + c * 32, rs);
        tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColDP + c * 32, rp);
        tmem_ld_wait();
        uint32_t pk[16], dsk[16];
        if (all_full) {  // interior tile: no per-element visibility test
          const float nd = -delta;
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(rs[e]), p.scale_log2, -lse_l2));
            const float p1 = exp2f(fmaf(__uint_as_float(rs[e + 1]), p.scale_log2, -lse_l2));
            const float d0 = p0 * ((__uint_as_float(rp[e]) + nd) * p.scale);
            const float d1 = p1 * ((__uint_as_float(rp[e + 1]) + nd) * p.scale);
            pk[e >> 1] = pack_bf16x2(p0, p1);
            dsk[e >> 1] = pack_bf16x2(d0, d1);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float p0 = 0.f, p1 = 0.f;
            if (c * 32 + e < vis) p0 = exp2f(__uint_as_float(rs[e]) * p.scale_log2 - lse_l2);
            if (c * 32 + e + 1 < vis) p1 = exp2f(__uint_as_float(rs[e + 1]) * p.scale_log2 - lse_l2);
            const float d0 = p0 * (__uint_as_float(rp[e]) - delta) * p.scale;
            const float d1 = p1 * (__uint_as_float(rp[e + 1]) - delta) * p.scale;
            pk[e >> 1] = pack_bf16x2(p0, p1);
            dsk[e >> 1] = pack_bf16x2(d0, d1);
          }
        }
        store_row_chunk_sw128(sP, row, c, pk);
        store_row_chunk_sw128(sDS, row, c, dsk);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&pds_full);
      // dQ tile -> fp32 scratch
      if (!mbar_wait(&dq_full, ph, &cta_abort, p.status)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = p.dq_acc + ((static_cast<long long>(b) * p.Sq + qi) * p.H + h) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColDP + c * 32, r);
        tmem_ld_wait();
        if (qi < p.Sq) {
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            atomicAdd(reinterpret_cast<float4*>(dq_row + c * 32 + e),
                      make_float4(__uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]),
                                  __uint_as_float(r[e + 3])));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&dq_read);
    }
    // ---------------------------------------------------------------- dK, dV out
    // tcgen05.ld is warp-collective (.sync.aligned): every lane of the warp issues it, and only the global
    // stores are predicated on the row being inside the sequence.
    const int kr = c0 + row;
    const bool in_range = kr < p.Sk;
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    __nv_bfloat16* dk_row = p.dk + b * p.dk_sb + static_cast<long long>(in_range ? kr : 0) * p.dk_ss + hk * p.dk_sh;
    __nv_bfloat16* dv_row = p.dv + b * p.dv_sb + static_cast<long long>(in_range ? kr : 0) * p.dv_ss + hk * p.dv_sh;
    if (warp_ok && n_iter > 0) {
      // the last dq_full wait above covered every MMA issued before it, including the dK / dV updates
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColDK + c * 32, r);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
            *reinterpret_cast<uint4*>(dk_row + c * 32 + e) = v;
          }
        }
        tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColDV + c * 32, r);
        tmem_ld_wait();
        if (in_range) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
            *reinterpret_cast<uint4*>(dv_row + c * 32 + e) = v;
          }
        }
      }
    } else if (warp_ok && in_range) {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        *reinterpret_cast<uint4*>(dk_row + c * 8) = z;
        *reinterpret_cast<uint4*>(dv_row + c * 8) = z;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row.
template <int D>
__global__ void __launch_bounds__(256)
flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                       float* __restrict__ delta, int B, int Sq, int H, long long do_sb, long long do_ss,
                       long long do_sh, long long o_sb, long long o_ss, long long o_sh) {
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * Sq * H;
  if (wid >= total) return;
  const int h = static_cast<int>(wid % H);
  const long long bs = wid / H;
  const int s = static_cast<int>(bs % Sq);
  const int b = static_cast<int>(bs / Sq);
  const __nv_bfloat16* a = dO + b * do_sb + static_cast<long long>(s) * do_ss + h * do_sh;
  const __nv_bfloat16* c = O + b * o_sb + static_cast<long long>(s) * o_ss + h * o_sh;
  float acc = 0.f;
  constexpr int PER = D / 32;  // 2 or 4 elements per lane
  if constexpr (PER == 4) {
    const uint2 x = *reinterpret_cast<const uint2*>(a + lane * 4);
    const uint2 y = *reinterpret_cast<const uint2*>(c + lane * 4);
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    const float2 y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&y.x));
    const float2 y1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&y.y));
    acc = x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y;
  } else {
    const uint32_t x = *reinterpret_cast<const uint32_t*>(a + lane * 2);
    const uint32_t y = *reinterpret_cast<const uint32_t*>(c + lane * 2);
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x));
    const float2 y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&y));
    acc = x0.x * y0.x + x0.y * y0.y;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[(static_cast<long long>(b) * H + h) * Sq + s] = acc;
}

// dq[b, s, h, :] (bf16, strided) = dq_acc[b, s, h, :] (fp32, contiguous)
__global__ void __launch_bounds__(256)
flash_bwd_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows, int H, int D,
                            int Sq, long long sb, long long ss, long long sh) {
  const int vpr = D / 8;
  const long long n = rows * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vpr;  // (b, s, h) flattened
    const int c = static_cast<int>(i - r * vpr) * 8;
    const int h = static_cast<int>(r % H);
    const long long bs = r / H;
    const int s = static_cast<int>(bs % Sq);
    const long long b = bs / Sq;
    const float4 x = *reinterpret_cast<const float4*>(acc + r * D + c);
    const float4 y = *reinterpret_cast<const float4*>(acc + r * D + c + 4);
    uint4 v;
    v.x = pack_bf16x2(x.x, x.y);
    v.y = pack_bf16x2(x.z, x.w);
    v.z = pack_bf16x2(y.x, y.y);
    v.w = pack_bf16x2(y.z, y.w);
    *reinterpret_cast<uint4*>(dq + b * sb + static_cast<long long>(s) * ss + h * sh + c) = v;
  }
}

}  // namespace
}  // namespace tsb

// Bytes of fp32 scratch tsb_flash_bwd needs: the dQ accumulator [B, Sq, H, D] followed by delta [B, H, Sq].
TSB_EXPORT long long tsb_flash_bwd_scratch_bytes(int B, int Sq, int H, int D) {
  return (static_cast<long long>(B) * Sq * H * D + static_cast<long long>(B) * H * Sq) * 4;
}

// Gradients of tsb_flash_fwd. dO and O are [B, Sq, H, D] with the strides of q's gradient layout given
// separately (do_* / o is contiguous BSHD). dq / dk / dv are bf16 views; dq, dk, dv share the stride triple
// (g_sb, g_ss, g_sh) -- they are usually slices of one packed [B, S, H + 2 Hkv, D] buffer -- when
// dkv_strides == NULL, else dk / dv use dkv_strides[0..2].
// scratch: tsb_flash_bwd_scratch_bytes() bytes of device memory (contents are overwritten).
TSB_EXPORT int tsb_flash_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o,
                             const float* lse, void* dq, void* dk, void* dv, void* scratch, int B, int Sq, int Sk,
                             int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                             long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                             long long g_sb, long long g_ss, long long g_sh, float scale, int causal, void* stream) {
  using namespace tsb;
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128)) return -2;
  if (!scratch) return -2;
  const long long strides[] = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, g_sb, g_ss, g_sh};
  for (long long s : strides)
    if (s % 8) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // dO and O are contiguous [B, Sq, H, D]
  const long long c_sh = D, c_ss = static_cast<long long>(H) * D, c_sb = c_ss * Sq;
  float* dq_acc = static_cast<float*>(scratch);
  float* delta = dq_acc + static_cast<long long>(B) * Sq * H * D;
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(B) * Sq * H * D * 4, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const long long rows = static_cast<long long>(B) * Sq * H;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    if (D == 128)
      flash_bwd_delta_kernel<128><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dO),
                                                          static_cast<const __nv_bfloat16*>(o), delta, B, Sq, H, c_sb,
                                                          c_ss, c_sh, c_sb, c_ss, c_sh);
    else
      flash_bwd_delta_kernel<64><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dO),
                                                         static_cast<const __nv_bfloat16*>(o), delta, B, Sq, H, c_sb,
                                                         c_ss, c_sh, c_sb, c_ss, c_sh);
  }
  CUtensorMap tq, tk, tv, tdo;
  if (!make_bshd_tmap(&tq, q, B, Sq, H, D, q_sb, q_ss, q_sh, 128)) return -3;
  if (!make_bshd_tmap(&tk, k, B, Sk, Hkv, D, k_sb, k_ss, k_sh, 128)) return -3;
  if (!make_bshd_tmap(&tv, v, B, Sk, Hkv, D, v_sb, v_ss, v_sh, 128)) return -3;
  if (!make_bshd_tmap(&tdo, dO, B, Sq, H, D, c_sb, c_ss, c_sh, 128)) return -3;
  BwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq_acc = dq_acc;
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv;
  p.dk_sb = g_sb; p.dk_ss = g_ss; p.dk_sh = g_sh;
  p.dv_sb = g_sb; p.dv_ss = g_ss; p.dv_sh = g_sh;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = device_status_word();
  dim3 grid((Sk + BT - 1) / BT, Hkv, B);
  if (D == 128) {
    static PerDeviceFlag attr;
    if (attr.unset()) {
      e = cudaFuncSetAttribute(flash_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               BwdCfg<128>::kSmemBytes);
      if (e != cudaSuccess) return static_cast<int>(e);
      attr.set();
    }
    flash_bwd_kernel<128><<<grid, kBwdThreads, BwdCfg<128>::kSmemBytes, s>>>(tq, tk, tv, tdo, p);
  } else {
    static PerDeviceFlag attr;
    if (attr.unset()) {
      e = cudaFuncSetAttribute(flash_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               BwdCfg<64>::kSmemBytes);
      if (e != cudaSuccess) return static_cast<int>(e);
      attr.set();
    }
    flash_bwd_kernel<64><<<grid, kBwdThreads, BwdCfg<64>::kSmemBytes, s>>>(tq, tk, tv, tdo, p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long rows = static_cast<long long>(B) * Sq * H;
  long long blocks = (rows * (D / 8) + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  flash_bwd_dq_convert_kernel<<<static_cast<unsigned>(blocks), 256, 0, s>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), rows, H,
                                                                            D, Sq, g_sb, g_ss, g_sh);
  return static_cast<int>(cudaGetLastError());
}
