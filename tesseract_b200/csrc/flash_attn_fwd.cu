// FlashAttention forward on tcgen05 tensor cores (bf16, head_dim 64 or 128, causal or full, GQA).
//
// One CTA per (128-query tile, head, batch); 6 warps:
//   warps 0-3  softmax: each thread owns one query row. S = Q K^T is read from TMEM (tcgen05.ld), the
//              online-softmax statistics live in registers, P is written to shared memory as bf16 in the
//              128-byte-swizzled K-major layout the tensor core reads, and the running output is kept in
//              fp32 registers (O = O * alpha + P V, with P V read back from TMEM every tile).
//   warp 4     TMA producer: Q once, then K and V tiles through a two-stage ring (4-D tensor maps over
//              [batch, seq, head, dim] views with arbitrary batch/seq/head strides, so a packed QKV
//              projection output is consumed in place).
//   warp 5     allocates TMEM and issues the MMAs: S_{j+1} = Q K_{j+1}^T is in flight while the softmax
//              warps work on tile j; P_j V_j follows as soon as P_j is in shared memory.
// Causal masking follows the reference: key j is visible to query i iff j <= i + (Sk - Sq); a fully masked
// row produces zeros; softmax statistics are fp32; scale is folded into the exponent
// (src/cuda/FusedAttention.cu:69-80,318-331,368-567 is the WMMA kernel this replaces).
// Also writes the per-row log-sum-exp needed by the backward kernel.
#include "common.cuh"

#include <algorithm>

#include <cstdlib>
#include <cstring>

namespace tsb {
namespace {

constexpr int kFaThreads = 192;
constexpr int BQ = 128;
constexpr int BKV = 128;

template <int D>
struct FaCfg {
  static constexpr int kHalves = D / 64;                 // 64-wide (128-byte) column blocks per tile
  static constexpr int kTileBytes = 128 * D * 2;         // Q, K, V tiles: 128 rows x D bf16
  static constexpr int kPBytes = BQ * BKV * 2;           // P tile: 128 x 128 bf16
  static constexpr int kSmemBytes = kTileBytes * 5 + kPBytes + 1024;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS0 = 0, kColS1 = 128, kColO = 256;
};

struct FaParams {
  __nv_bfloat16* o;
  float* lse;
  int B, Sq, Sk, H, Hkv;
  long long o_sb, o_ss, o_sh;
  const int* cu_seqlens;  // varlen: int32 [B + 1] row offsets of the sequences in the packed token axis, else null
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  int causal;
  int* status;
};

// Descriptor for k-step `ks` (16 elements along K) of a K-major [rows x D] tile made of 64-column halves.
template <int ROWS>
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int ks) {
  const int half = ks >> 2;
  return umma_smem_desc_sw128(base + half * (ROWS * 128) + (ks & 3) * 32, 16, 1024);
}
// Descriptor for k-step `ks` (16 rows) of an MN-major tile: [k rows][N contiguous], 64-wide N halves
// `half_stride` bytes apart.
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int ks, uint32_t half_stride) {
  return umma_smem_desc_sw128(base + ks * 2048, half_stride, 1024);
}

// LAZY = true: the output accumulates in TMEM over all key tiles (the P V product adds to it) and is rescaled only
// when a row's maximum has grown by more than 2^8 since the reference maximum of its exponents was set; the score
// row is read from TMEM once per tile and kept in registers for both the maximum and the exponentials.
// LAZY = false: the output is folded into fp32 registers after every tile (two reads of the score row per tile).
template <int D, bool LAZY>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FaParams p_in) {
  using Cfg = FaCfg<D>;
  // Variable-length batches: the sequences sit one after another on ONE token axis (tensor maps with batch 1);
  // block z handles sequence z, whose rows start at cu_seqlens[z]. Tiles that reach past its end read rows of the
  // next sequence (or the zero fill) and the length mask below discards them.
  FaParams p = p_in;
  int row0 = 0;
  int bb = blockIdx.z;
  if (p_in.cu_seqlens) {
    row0 = p_in.cu_seqlens[blockIdx.z];
    p.Sq = p.Sk = p_in.cu_seqlens[blockIdx.z + 1] - row0;
    bb = 0;
    if (static_cast<int>(gridDim.x - 1 - blockIdx.x) * BQ >= p.Sq) return;  // no query rows: the whole CTA leaves
  }
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::kTileBytes;      // 2 stages
  uint8_t* sV = sK + 2 * Cfg::kTileBytes;  // 2 stages
  uint8_t* sP = sV + 2 * Cfg::kTileBytes;

  __shared__ __align__(8) uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2];
  __shared__ __align__(8) uint64_t s_full[2], s_free[2], p_full, o_full;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) query tiles first under causal masking
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qt * BQ;
  const int offset = p.Sk - p.Sq;

  int n_tiles = (p.Sk + BKV - 1) / BKV;
  if (p.causal) {
    const int last_col = q0 + BQ - 1 + offset;
    const int lim = last_col < 0 ? 0 : last_col / BKV + 1;
    n_tiles = min(n_tiles, lim);
  }

  if (threadIdx.x == 0) {
    cta_abort = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
    }
    mbar_init(&p_full, 128);
    mbar_init(&o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(&tmem_base_smem, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(&q_full, Cfg::kTileBytes);
#pragma unroll
      for (int hf = 0; hf < Cfg::kHalves; ++hf) tma_load_4d(sQ + hf * 16384, &tmQ, &q_full, hf * 64, q0 + row0, h, bb);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1u;
        if (!mbar_wait(&k_empty[st], par, &cta_abort, p.status)) break;
        mbar_expect_tx(&k_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < Cfg::kHalves; ++hf)
          tma_load_4d(sK + st * Cfg::kTileBytes + hf * 16384, &tmK, &k_full[st], hf * 64, j * BKV + row0, hk, bb);
        if (!mbar_wait(&v_empty[st], par, &cta_abort, p.status)) break;
        mbar_expect_tx(&v_full[st], Cfg::kTileBytes);
#pragma unroll
        for (int hf = 0; hf < Cfg::kHalves; ++hf)
          tma_load_4d(sV + st * Cfg::kTileBytes + hf * 16384, &tmV, &v_full[st], hf * 64, j * BKV + row0, hk, bb);
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = umma_idesc(BQ, BKV, 1, 1, 0, 0);  // S = Q K^T, both K-major
      constexpr uint32_t idesc_o = umma_idesc(BQ, D, 1, 1, 0, 1);    // O = P V, V is N-major
      const uint32_t q_base = smem_u32(sQ);
      const uint32_t p_base = smem_u32(sP);
      bool ok = mbar_wait(&q_full, 0, &cta_abort, p.status);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, &cta_abort, p.status)) return false;
        if (!mbar_wait(&s_free[st], ((j >> 1) & 1) ^ 1u, &cta_abort, p.status)) return false;
        tc_fence_after();
        const uint32_t k_base = smem_u32(sK + st * Cfg::kTileBytes);
        const uint32_t d = tmem_base + (st ? Cfg::kColS1 : Cfg::kColS0);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
          umma_f16(d, kmajor_desc<128>(q_base, ks), kmajor_desc<128>(k_base, ks), idesc_s, ks != 0);
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        if (!mbar_wait(&p_full, j & 1, &cta_abort, p.status)) break;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, &cta_abort, p.status)) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(sV + st * Cfg::kTileBytes);
        const uint32_t d = tmem_base + Cfg::kColO;
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          umma_f16(d, kmajor_desc<128>(p_base, ks), mnmajor_desc(v_base, ks, 16384), idesc_o,
                   LAZY ? ((j | ks) != 0) : (ks != 0));
        umma_commit(&o_full);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + output (warps 0..3)
    const int row = warp * 32 + lane;        // row within the tile == TMEM lane
    const int qi = q0 + row;                 // query index
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const int row_limit = qi + offset;  // last visible key under causal masking
    if constexpr (LAZY) {
      float m_ref = -INFINITY, l_run = 0.f;  // m_ref: the maximum the exponents of this row currently refer to
      bool ok = true;
      const float kGrow = 8.f;                // rescale when the maximum has grown by more than 2^8
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        // a failed (timed-out) wait leaves the loop warp-uniformly: the TMEM accesses below are warp-collective
        if (!__all_sync(0xffffffffu, mbar_wait(&s_full[st], (j >> 1) & 1, &cta_abort, p.status) ? 1 : 0)) { ok = false; break; }
        tc_fence_after();
        const uint32_t s_addr = tmem_base + lane_addr + (st ? Cfg::kColS1 : Cfg::kColS0);
        uint32_t sr[BKV];
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) tmem_ld_32x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_free[st]);              // the scores live in registers now: the MMA warp may refill the buffer
        const int c0 = j * BKV;
        const bool need_mask = (p.causal && c0 + BKV - 1 > q0 + offset) || (c0 + BKV > p.Sk);
        int vis = BKV;
        if (need_mask) {
          int lim = p.Sk - c0;
          if (p.causal) lim = min(lim, row_limit - c0 + 1);
          vis = max(0, min(BKV, lim));
        }
        float m_tile = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < BKV; ++i)
            if (i < vis) m_tile = fmaxf(m_tile, __uint_as_float(sr[i]));
        } else {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < BKV; i += 4) {
            m0 = fmaxf(m0, __uint_as_float(sr[i]));
            m1 = fmaxf(m1, __uint_as_float(sr[i + 1]));
            m2 = fmaxf(m2, __uint_as_float(sr[i + 2]));
            m3 = fmaxf(m3, __uint_as_float(sr[i + 3]));
          }
          m_tile = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
        // the previous P V product must be finished: it reads sP, and a rescale below rewrites its result
        if (j > 0) {
          if (!__all_sync(0xffffffffu, mbar_wait(&o_full, (j - 1) & 1, &cta_abort, p.status) ? 1 : 0)) { ok = false; break; }
          tc_fence_after();
        }
        float factor = 1.f;
        bool grow = false;
        if (m_tile != -INFINITY) {
          if (m_ref == -INFINITY) {
            m_ref = m_tile;                    // first visible scores of this row: nothing accumulated yet
            grow = (j > 0);                    // (earlier tiles were fully masked for this row: O and l are zero)
            factor = 1.f;
          } else if ((m_tile - m_ref) * p.scale_log2 > kGrow) {
            factor = exp2f((m_ref - m_tile) * p.scale_log2);
            m_ref = m_tile;
            grow = true;
          }
        }
        if (j > 0 && __any_sync(0xffffffffu, grow && factor != 1.f)) {
          // warp-collective: every lane rescales its own TMEM lane (factor 1 where nothing changed)
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColO + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st_32x32(tmem_base + lane_addr + Cfg::kColO + c * 32, r);
          }
          tmem_st_wait();
        }
        l_run *= factor;
        const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
        const float mneg = -m_use * p.scale_log2;
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = exp2f(fmaf(__uint_as_float(sr[c * 32 + i]), p.scale_log2, mneg));
            float p1 = exp2f(fmaf(__uint_as_float(sr[c * 32 + i + 1]), p.scale_log2, mneg));
            if (need_mask) {
              if (c * 32 + i >= vis) p0 = 0.f;
              if (c * 32 + i + 1 >= vis) p1 = 0.f;
            }
            // the denominator sums what the tensor core will actually multiply (bf16-rounded P)
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            const float2 pf = __bfloat1622float2(pb);
            l0 += pf.x;
            l1 += pf.y;
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
          }
          const int half = c >> 1;
          uint8_t* prow = sP + half * 16384 + row * 128;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int chunk = (c & 1) * 4 + q4;
            const int sw = chunk ^ (row & 7);
            *reinterpret_cast<uint4*>(prow + sw * 16) =
                make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
          }
        }
        l_run += l0 + l1;
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(&p_full);
      }
      // every lane of the warp takes part in the TMEM reads; only the global stores depend on the row
      const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
      bool have_o = false;
      if (warp_ok && n_tiles > 0) have_o = mbar_wait(&o_full, (n_tiles - 1) & 1, &cta_abort, p.status);
      have_o = __all_sync(0xffffffffu, have_o ? 1 : 0) != 0;
      if (have_o) tc_fence_after();
      if (warp_ok && (have_o || n_tiles == 0)) {
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow = p.o + bb * p.o_sb + static_cast<long long>(row0 + (qi < p.Sq ? qi : 0)) * p.o_ss + h * p.o_sh;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          if (have_o) {
            tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColO + c * 32, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (qi < p.Sq) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[e]) * inv_l, __uint_as_float(r[e + 1]) * inv_l);
              v.y = pack_bf16x2(__uint_as_float(r[e + 2]) * inv_l, __uint_as_float(r[e + 3]) * inv_l);
              v.z = pack_bf16x2(__uint_as_float(r[e + 4]) * inv_l, __uint_as_float(r[e + 5]) * inv_l);
              v.w = pack_bf16x2(__uint_as_float(r[e + 6]) * inv_l, __uint_as_float(r[e + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + c * 32 + e) = v;
            }
          }
        }
        if (qi < p.Sq && p.lse) {
          const float lse = l_run > 0.f ? (m_ref * p.scale + __logf(l_run)) : -INFINITY;
          p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + qi] = lse;
        }
      }
    } else {
    float o_acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 1.f;
    bool ok = true;
    const int row_limit = qi + offset;  // last visible key under causal masking

    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&s_full[st], (j >> 1) & 1, &cta_abort, p.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + lane_addr + (st ? Cfg::kColS1 : Cfg::kColS0);
      const int c0 = j * BKV;
      const bool need_mask = (p.causal && c0 + BKV - 1 > q0 + offset) || (c0 + BKV > p.Sk);
      int vis = BKV;  // number of visible columns of this tile for this row
      if (need_mask) {
        int lim = p.Sk - c0;
        if (p.causal) lim = min(lim, row_limit - c0 + 1);
        vis = max(0, min(BKV, lim));
      }
      // pass 1: row maximum (tiles that need no masking skip the per-element visibility test)
      float m_tile = -INFINITY;
      if (need_mask) {
#pragma unroll 1
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < vis) m_tile = fmaxf(m_tile, __uint_as_float(r[i]));
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(s_addr + c * 32, r);
          tmem_ld_wait();
          float m0 = fmaxf(__uint_as_float(r[0]), __uint_as_float(r[1]));
          float m1 = fmaxf(__uint_as_float(r[2]), __uint_as_float(r[3]));
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            m0 = fmaxf(m0, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
            m1 = fmaxf(m1, fmaxf(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])));
          }
          m_tile = fmaxf(m_tile, fmaxf(m0, m1));
        }
      }
      const float m_new = fmaxf(m_run, m_tile);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_use) * p.scale_log2);
      // fold the previous tile's P V into the running output (this also means sP is free again)
      if (j > 0) {
        if (!mbar_wait(&o_full, (j - 1) & 1, &cta_abort, p.status)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColO + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha_prev + __uint_as_float(r[i]);
        }
      }
      // pass 2: P = exp2((S - m) * scale) as bf16 into swizzled shared memory
      float l_tile = 0.f;
#pragma unroll 1
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
        const float mneg = -m_use * p.scale_log2;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float p0 = (c * 32 + i < vis) ? exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, mneg)) : 0.f;
            float p1 = (c * 32 + i + 1 < vis) ? exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, mneg)) : 0.f;
            // the denominator sums what the tensor core will actually multiply (bf16-rounded P)
            const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
            const float2 pf = __bfloat1622float2(pb);
            l_tile += pf.x + pf.y;
            packed[i >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
          }
        } else {
          // interior tiles: the denominator sums the fp32 probabilities (the bf16 rounding of P is unbiased, so
          // the two agree to well below the output precision) -- two instructions fewer per pair
          float l0 = 0.f, l1 = 0.f;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(r[i]), p.scale_log2, mneg));
            const float p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, mneg));
            l0 += p0;
            l1 += p1;
            packed[i >> 1] = pack_bf16x2(p0, p1);
          }
          l_tile += l0 + l1;
        }
        // columns [c*32, c*32+32) = four 16-byte chunks of row `row` in half (c >> 1)
        const int half = c >> 1;
        uint8_t* prow = sP + half * 16384 + row * 128;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int chunk = (c & 1) * 4 + q4;
          const int sw = chunk ^ (row & 7);
          *reinterpret_cast<uint4*>(prow + sw * 16) =
              make_uint4(packed[q4 * 4], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
        }
      }
      tc_fence_before();
      mbar_arrive(&s_free[st]);
      fence_proxy_async_smem();
      mbar_arrive(&p_full);
      l_run = l_run * alpha + l_tile;
      m_run = m_new;
      alpha_prev = alpha;
      // alpha_prev rescales the output accumulated BEFORE tile j when tile j's P V is folded in
    }
    if (ok && n_tiles > 0) {
      if (mbar_wait(&o_full, (n_tiles - 1) & 1, &cta_abort, p.status)) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + lane_addr + Cfg::kColO + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = o_acc[c * 32 + i] * alpha_prev + __uint_as_float(r[i]);
        }
      } else {
        ok = false;
      }
    }
    if (ok && qi < p.Sq) {
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.o + bb * p.o_sb + static_cast<long long>(row0 + qi) * p.o_ss + h * p.o_sh;
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        uint4 v;
        v.x = pack_bf16x2(o_acc[c * 8 + 0] * inv_l, o_acc[c * 8 + 1] * inv_l);
        v.y = pack_bf16x2(o_acc[c * 8 + 2] * inv_l, o_acc[c * 8 + 3] * inv_l);
        v.z = pack_bf16x2(o_acc[c * 8 + 4] * inv_l, o_acc[c * 8 + 5] * inv_l);
        v.w = pack_bf16x2(o_acc[c * 8 + 6] * inv_l, o_acc[c * 8 + 7] * inv_l);
        *reinterpret_cast<uint4*>(orow + c * 8) = v;
      }
      if (p.lse) {
        const float lse = l_run > 0.f ? (m_run * p.scale + __logf(l_run)) : -INFINITY;
        p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + qi] = lse;
      }
    }
    }  // eager variant
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace

// 4-D map over a [batch, seq, head, dim] bf16 view; box = 64 dims x 128 rows of one (head, batch).
bool make_bshd_tmap(CUtensorMap* out, const void* base, int B, int S, int Hn, int D, long long sb, long long ss,
                    long long sh, int box_rows) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(S), static_cast<uint64_t>(Hn),
                      static_cast<uint64_t>(B)};
  uint64_t strides[4] = {2, static_cast<uint64_t>(ss) * 2, static_cast<uint64_t>(sh) * 2,
                         static_cast<uint64_t>(sb) * 2};
  uint32_t box[4] = {64, static_cast<uint32_t>(box_rows), 1, 1};
  return make_tmap_nd(out, base, 2, 4, dims, strides, box, true);
}

}  // namespace tsb

// o[b, s, h, :] = softmax(scale * q k^T [+ causal mask]) v for bf16 BSHD views.
//   q: [B, Sq, H, D], k / v: [B, Sk, Hkv, D]; strides (batch, seq, head) in elements, unit stride in D;
//   every base pointer 16-byte aligned and every stride a multiple of 8 elements. D is 64 or 128.
//   lse (fp32 [B, H, Sq], may be NULL) receives log-sum-exp of the scaled scores per row.
TSB_EXPORT int tsb_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                             int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                             long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                             long long o_sb, long long o_ss, long long o_sh, float scale, int causal, void* stream) {
  using namespace tsb;
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128)) return -2;
  const long long strides[] = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh, o_sb, o_ss, o_sh};
  for (long long s : strides)
    if (s % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -2;
  CUtensorMap tq, tk, tv;
  if (!make_bshd_tmap(&tq, q, B, Sq, H, D, q_sb, q_ss, q_sh, 128)) return -3;
  if (!make_bshd_tmap(&tk, k, B, Sk, Hkv, D, k_sb, k_ss, k_sh, 128)) return -3;
  if (!make_bshd_tmap(&tv, v, B, Sk, Hkv, D, v_sb, v_ss, v_sh, 128)) return -3;
  FaParams p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.cu_seqlens = nullptr;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv;
  p.o_sb = o_sb; p.o_ss = o_ss; p.o_sh = o_sh;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal;
  p.status = device_status_word();
  dim3 grid((Sq + BQ - 1) / BQ, H, B);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // TESSERACT_FLASH_FWD=lazy selects the variant that keeps the output in TMEM and rescales it only when a row
  // maximum has grown by more than 2^8; measured at 417 TFLOP/s against 436 for the default on the S = 4096 case
  static const bool lazy = [] {
    const char* e = getenv("TESSERACT_FLASH_FWD");
    return e && strcmp(e, "lazy") == 0;
  }();
  auto launch = [&](auto kern, int smem_bytes) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    kern<<<grid, kFaThreads, smem_bytes, s>>>(tq, tk, tv, p);
    return 0;
  };
  int rc;
  if (D == 128)
    rc = lazy ? launch(flash_fwd_kernel<128, true>, FaCfg<128>::kSmemBytes) : launch(flash_fwd_kernel<128, false>, FaCfg<128>::kSmemBytes);
  else
    rc = lazy ? launch(flash_fwd_kernel<64, true>, FaCfg<64>::kSmemBytes) : launch(flash_fwd_kernel<64, false>, FaCfg<64>::kSmemBytes);
  if (rc) return rc;
  return static_cast<int>(cudaGetLastError());
}

// Variable-length causal self-attention over sequences packed on one token axis (batched prefill of prompts of
// different lengths in ONE launch): q [T, H, D], k / v [T, Hkv, D], o [T, H, D] bf16 with token / head strides in
// elements (unit stride in D, multiples of 8, 16-byte aligned bases); cu_seqlens int32 [n_seqs + 1] on the device,
// cu_seqlens[0] = 0, cu_seqlens[n_seqs] = T; max_len >= the longest sequence. D is 64 or 128.
TSB_EXPORT int tsb_flash_fwd_varlen(const void* q, const void* k, const void* v, void* o, const int* cu_seqlens,
                                    int n_seqs, int max_len, int T, int H, int Hkv, int D, long long q_ss, long long q_sh,
                                    long long k_ss, long long k_sh, long long v_ss, long long v_sh, long long o_ss,
                                    long long o_sh, float scale, void* stream) {
  using namespace tsb;
  if (n_seqs <= 0 || max_len <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128) || !cu_seqlens)
    return -2;
  const long long strides[] = {q_ss, q_sh, k_ss, k_sh, v_ss, v_sh, o_ss, o_sh};
  for (long long st : strides)
    if (st % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -2;
  CUtensorMap tq, tk, tv;
  const long long big = static_cast<long long>(T) * std::max({q_ss, k_ss, v_ss});  // batch stride of the single batch
  if (!make_bshd_tmap(&tq, q, 1, T, H, D, big, q_ss, q_sh, 128)) return -3;
  if (!make_bshd_tmap(&tk, k, 1, T, Hkv, D, big, k_ss, k_sh, 128)) return -3;
  if (!make_bshd_tmap(&tv, v, 1, T, Hkv, D, big, v_ss, v_sh, 128)) return -3;
  FaParams p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = nullptr;
  p.cu_seqlens = cu_seqlens;
  p.B = n_seqs; p.Sq = max_len; p.Sk = max_len; p.H = H; p.Hkv = Hkv;
  p.o_sb = 0; p.o_ss = o_ss; p.o_sh = o_sh;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = 1;
  p.status = device_status_word();
  dim3 grid((max_len + BQ - 1) / BQ, H, n_seqs);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto launch = [&](auto kern, int smem_bytes) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    kern<<<grid, kFaThreads, smem_bytes, s>>>(tq, tk, tv, p);
    return 0;
  };
  const int rc = (D == 128) ? launch(flash_fwd_kernel<128, false>, FaCfg<128>::kSmemBytes)
                            : launch(flash_fwd_kernel<64, false>, FaCfg<64>::kSmemBytes);
  if (rc) return rc;
  return static_cast<int>(cudaGetLastError());
}
