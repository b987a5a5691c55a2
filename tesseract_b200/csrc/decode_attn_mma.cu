// Split-K paged decode attention on tensor cores (warp-level mma.sync), bf16 / fp16 or INT8 KV.
//
// Decode attention is a stream over the KV cache: 512 bytes of K and V per (token, KV head) against a handful of
// FMAs per byte. On CUDA cores those FMAs, the bf16 -> fp32 conversions and the shuffle reductions cost ~75 warp
// instructions per token and cap the kernel near 2 TB/s; here the two products run on the tensor cores
// (m16n8k16, the G <= 8 query heads of a GQA group padded to the 16-row M dimension) and K / V go global ->
// shared with 16-byte cp.async in a three-stage per-warp ring, so the kernel is bound by HBM, not by issue slots.
//
// One CTA per (key split, KV head, request); its 4 warps take 16-token tiles round-robin. Per tile and warp:
//   S[head, token]  = Q[head, :] . K[token, :]      ldmatrix (K row-major)       -> 2 x D/16 mma
//   P               = exp2(S * c - m) with online (m, l) per head, kept in the accumulator layout,
//                     which IS the A-operand layout of the next product (no shuffles, no shared memory)
//   O[head, :]     += P[head, token] . V[token, :]   ldmatrix.trans (V row-major) -> D/8 mma
// The warps' (m, l, O) are merged through shared memory and written as the split's partial (or the final output
// when there is one split); the merge of splits is decode_merge_kernel of decode_attn.cu.
// Same inputs, pool layout and clamping rules as tsb_paged_decode (src/cuda/PagedAttention.cu:88-171 is the
// reference's one-CTA-per-(request, head) CUDA-core kernel).
#include "common.cuh"

#include <type_traits>

namespace tsb {
namespace {

constexpr int kWarps = 4;
constexpr int kTile = 16;     // tokens per warp tile
constexpr int kStagesD = 3;   // cp.async ring depth per warp

template <typename T>
struct MmaT;
template <>
struct MmaT<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) { return pack_bf16x2(lo, hi); }
};
template <>
struct MmaT<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// S += Q K^T on the int8 tensor-core path: A = int8 queries (16 rows x 32), B = int8 keys (32 x 8 tokens), int32 sums.
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte async copy; src_bytes = 0 zero-fills the destination (rows past the end of the sequence).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct MmaDecParams {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const float* k_scale;  // INT8 pools: per-(token, head) scales, else null
  const float* v_scale;
  const int* tables;
  const int* lens;
  void* out;
  float* part_o;
  float* part_ml;
  int A, H, Hkv, bs, nb, max_logical, splits, gh;  // gh = query heads per CTA (<= 8)
  float scale_log2;
  int* status;           // device status word: a block-table entry outside the pool is reported there
};

// INT8 pools: the raw int8 rows (and their scales) travel through the cp.async ring. S = Q K^T runs on the int8
// tensor-core path straight from the raw key rows: the queries are quantised once per CTA (one scale per head,
// |q| / 127), the sums are exact int32, and query scale x key scale multiply S afterwards. The values are widened to
// fp16 in a per-warp conversion buffer (int8 is exact in fp16) for P V, with the V scales riding on P.
template <typename T, int D, bool INT8>
__global__ void __launch_bounds__(kWarps * 32)
paged_decode_mma_kernel(MmaDecParams p) {
  pdl_trigger();
  pdl_grid_wait();
  // INT8 pools run their products in fp16 whatever the model type: int8 -> fp16 is one byte-permute and half a
  // subtract per element (1024 + u is exact in fp16), and |k|, |v| <= 128 with fp32 accumulation loses nothing.
  using MT = typename std::conditional<INT8, __half, T>::type;
  constexpr int kRowBytes = D * 2 + 16;           // padded row: consecutive rows fall into different 16-byte bank groups
  constexpr int kTileBytes = kTile * kRowBytes;   // one K (or V) tile as the tensor core reads it
  constexpr int kRawRow = INT8 ? D : D * 2;       // bytes per pool row
  constexpr int kRawTile = kTile * kRawRow;
  constexpr int kRawKRow = D + 16;                // INT8: raw key rows are padded in the ring (ldmatrix reads them)
  constexpr int kRawKTile = kTile * kRawKRow;
  constexpr int kStageBytes = INT8 ? (kRawKTile + kRawTile + 2 * kTile * 4) : 2 * kTileBytes;  // ring stage
  constexpr int kConvBytes = INT8 ? kTileBytes : 0;                                            // widened V
  constexpr int kWarpBytes = kStagesD * kStageBytes + kConvBytes;
  constexpr int kChunks = kRawRow / 16;           // 16-byte pieces per pool row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));

  const int split = blockIdx.x;
  const int hgrp = blockIdx.y;
  const int a = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int sub = G / p.gh;
  const int hk = hgrp / sub;
  const int h0 = hk * G + (hgrp % sub) * p.gh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int len = p.lens[a];
  const int chunk = ((len + p.splits - 1) / p.splits + 15) & ~15;
  const int t_begin = split * chunk;
  const int t_end = min(len, t_begin + chunk);
  const int n_tiles = t_end > t_begin ? (t_end - t_begin + kTile - 1) / kTile : 0;

  uint8_t* wsmem = smem + warp * kWarpBytes;
  const uint32_t wsmem_u32 = smem_u32(wsmem);
  const int* table = p.tables + static_cast<long long>(a) * p.max_logical;

  // Q as the A operand (rows = heads, padded to 16 with zeros). 16-bit pools: per k-step of 16, a0 = (head g,
  // d 2t..2t+1), a2 = (+8). INT8 pools: the row is quantised to int8 with one scale (|q|max / 127) and a k-step covers
  // 32 columns: a0 = (head g, d 4t..4t+3), a2 = (+16).
  uint32_t qa[INT8 ? D / 32 : D / 16][2];
  float q_scale = 1.f;
  {
    const T* qrow = static_cast<const T*>(p.q) + (static_cast<long long>(a) * p.H + h0 + g) * D;
    if constexpr (INT8) {
      float qv[D / 32][8];
      float amax = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 32; ++ks)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          qv[ks][e] = g < p.gh ? to_f32<T>(qrow[ks * 32 + (e >> 2) * 16 + 4 * t4 + (e & 3)]) : 0.f;
          amax = fmaxf(amax, fabsf(qv[ks][e]));
        }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      q_scale = amax > 0.f ? amax / 127.f : 1.f;
      const float inv = 1.f / q_scale;
#pragma unroll
      for (int ks = 0; ks < D / 32; ++ks)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t w = 0u;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int qi = max(-127, min(127, __float2int_rn(qv[ks][hh * 4 + e] * inv)));
            w |= (static_cast<uint32_t>(qi) & 0xffu) << (8 * e);
          }
          qa[ks][hh] = w;
        }
    } else {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        if (g < p.gh) {
          if constexpr (std::is_same<MT, T>::value) {
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t4 + 8);
          } else {
            const T* q0 = qrow + ks * 16 + 2 * t4;
            qa[ks][0] = MmaT<MT>::pack(to_f32<T>(q0[0]), to_f32<T>(q0[1]));
            qa[ks][1] = MmaT<MT>::pack(to_f32<T>(q0[8]), to_f32<T>(q0[9]));
          }
        } else {
          qa[ks][0] = qa[ks][1] = 0u;
        }
      }
    }
  }
  float o[D / 8][2];  // O[head g][d = nb*8 + 2t, +1]
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = 0.f;
  float m_run = -INFINITY, l_part = 0.f;  // l_part: this lane's share of the row sum (reduced at the end)

  // tiles of this warp: warp, warp + 4, ... ; `issue(j)` starts the copies of this warp's j-th tile
  const int my_tiles = n_tiles > warp ? (n_tiles - warp + kWarps - 1) / kWarps : 0;
  // Pool row of token t for this KV head (block-table lookup, clamped): computed once per tile by lanes 0..15,
  // one row each, and handed to the copying lanes with shuffles -- the copy loop itself is then two cp.async and
  // one shuffle per 16-byte piece, no divisions and no table reads.
  auto row_of = [&](int t, bool valid) -> long long {
    int blk = valid ? table[t / p.bs] : 0;
    if (blk < 0 || blk >= p.nb) {       // never read outside the pool: block 0 instead, and the host hears of it
      if (p.status) atomicCAS(p.status, kStatusOk, kStatusBadIndex);
      blk = 0;
    }
    return (static_cast<long long>(blk) * p.Hkv + hk) * p.bs + (valid ? t % p.bs : 0);
  };
  auto issue = [&](int j) {
    const int tile = warp + j * kWarps;
    const int tok0 = t_begin + tile * kTile;
    const uint32_t dstK = wsmem_u32 + (j % kStagesD) * kStageBytes;
    const uint32_t dstV = dstK + (INT8 ? kRawKTile : kTileBytes);
    const int my_t = tok0 + (lane & 15);
    const bool my_valid = my_t < t_end;
    const long long my_row = row_of(my_t, my_valid);           // lanes 16..31 duplicate lanes 0..15
    constexpr int kRowsPerIter = 32 / kChunks;
    const int piece = lane % kChunks;
#pragma unroll
    for (int i = 0; i < kTile / kRowsPerIter; ++i) {
      const int r = i * kRowsPerIter + lane / kChunks;
      const long long row = __shfl_sync(0xffffffffu, my_row, r);
      const int valid = __shfl_sync(0xffffffffu, static_cast<int>(my_valid), r);
      const size_t off = static_cast<size_t>(row) * kRawRow + piece * 16;
      const uint32_t dk = r * (INT8 ? kRawKRow : kRowBytes) + piece * 16;
      const uint32_t dv = r * (INT8 ? kRawRow : kRowBytes) + piece * 16;
      cp_async16(dstK + dk, static_cast<const char*>(p.k_pool) + off, valid ? 16 : 0);
      cp_async16(dstV + dv, static_cast<const char*>(p.v_pool) + off, valid ? 16 : 0);
    }
    if constexpr (INT8) {
      // scales: 16 K + 16 V floats per tile, 4 bytes each -> one 4-byte async copy per lane
      const float* src = (lane < 16 ? p.k_scale : p.v_scale) + my_row;
      const uint32_t dst = dstK + kRawKTile + kRawTile + lane * 4;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(my_valid ? 4 : 0) : "memory");
    }
  };
#pragma unroll
  for (int j = 0; j < kStagesD - 1; ++j) {
    if (j < my_tiles) issue(j);
    cp_async_commit();
  }

  for (int j = 0; j < my_tiles; ++j) {
    if (j + kStagesD - 1 < my_tiles) issue(j + kStagesD - 1);
    cp_async_commit();
    cp_async_wait<kStagesD - 1>();
    __syncwarp();
    const uint32_t stage_u32 = wsmem_u32 + (j % kStagesD) * kStageBytes;
    uint32_t sK = stage_u32, sV = stage_u32 + kTileBytes;
    const float* sc = nullptr;
    if constexpr (INT8) {
      const uint8_t* raw = wsmem + (j % kStagesD) * kStageBytes;
      uint8_t* conv = wsmem + kStagesD * kStageBytes;
      sc = reinterpret_cast<const float*>(raw + kRawKTile + kRawTile);
      // widen the kTile value rows of D int8 to fp16: each lane converts 16-byte pieces (the keys stay int8)
#pragma unroll
      for (int i = 0; i < (kTile * kChunks + 31) / 32; ++i) {
        const int c = lane + 32 * i;
        if (c >= kTile * kChunks) break;
        const int r = c / kChunks, piece = c % kChunks;
        const uint4 v = *reinterpret_cast<const uint4*>(raw + kRawKTile + r * kRawRow + piece * 16);
        const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
        uint32_t w[8];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          // bytes x (int8) -> u = x + 128 -> fp16 bit patterns 0x6400 | u = 1024 + u -> minus 1152 = x, exactly
          const uint32_t u = vw[q4] ^ 0x80808080u;
          const uint32_t lo = __byte_perm(u, 0x64646464u, 0x4140);  // (1024 + u0, 1024 + u1)
          const uint32_t hi = __byte_perm(u, 0x64646464u, 0x4342);  // (1024 + u2, 1024 + u3)
          const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
          const __half2 a = __hsub2(*reinterpret_cast<const __half2*>(&lo), bias);
          const __half2 b = __hsub2(*reinterpret_cast<const __half2*>(&hi), bias);
          w[2 * q4] = *reinterpret_cast<const uint32_t*>(&a);
          w[2 * q4 + 1] = *reinterpret_cast<const uint32_t*>(&b);
        }
        uint8_t* dst = conv + r * kRowBytes + piece * 32;
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
      }
      __syncwarp();
      sV = smem_u32(conv);
    }
    const int tok0 = t_begin + (warp + j * kWarps) * kTile;

    // ---- S = Q K^T : two 8-token column blocks
    float s[2][4];
    if constexpr (INT8) {
      int si[2][4];
#pragma unroll
      for (int b = 0; b < 2; ++b) si[b][0] = si[b][1] = si[b][2] = si[b][3] = 0;
#pragma unroll
      for (int ks = 0; ks < D / 32; ++ks) {
        // 8 x 16-byte matrices: (tokens 0-7, d 0-15), (tokens 0-7, d 16-31), (tokens 8-15, d 0-15), (tokens 8-15, d 16-31)
        uint32_t kb[4];
        const int mat = lane >> 3;
        const int r = (mat >> 1) * 8 + (lane & 7);
        ldsm_x4(kb, sK + r * kRawKRow + ks * 32 + (mat & 1) * 16);
        const uint32_t afrag[4] = {qa[ks][0], 0u, qa[ks][1], 0u};
        mma_s8(si[0], afrag, kb[0], kb[1]);
        mma_s8(si[1], afrag, kb[2], kb[3]);
      }
#pragma unroll
      for (int b = 0; b < 2; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[b][e] = static_cast<float>(si[b][e]) * q_scale;
    } else {
#pragma unroll
      for (int b = 0; b < 2; ++b) s[b][0] = s[b][1] = s[b][2] = s[b][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        // matrices: (tokens 0-7, d 0-7), (tokens 0-7, d 8-15), (tokens 8-15, d 0-7), (tokens 8-15, d 8-15)
        uint32_t kb[4];
        const int mat = lane >> 3;
        const int r = (mat >> 1) * 8 + (lane & 7);
        ldsm_x4(kb, sK + r * kRowBytes + ks * 32 + (mat & 1) * 16);
        const uint32_t afrag[4] = {qa[ks][0], 0u, qa[ks][1], 0u};
        MmaT<MT>::mma(s[0], afrag, kb[0], kb[1]);
        MmaT<MT>::mma(s[1], afrag, kb[2], kb[3]);
      }
    }
    // ---- online softmax for head row g (rows g + 8 are padding); this lane holds tokens b*8 + 2t, +1
    float mx = -INFINITY;
#pragma unroll
    for (int b = 0; b < 2; ++b) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = tok0 + b * 8 + 2 * t4 + e;
        float sv = s[b][e] * p.scale_log2;
        if constexpr (INT8) sv *= sc[b * 8 + 2 * t4 + e];
        s[b][e] = t < t_end ? sv : -INFINITY;
        mx = fmaxf(mx, s[b][e]);
      }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float corr = m_run == -INFINITY ? 0.f : exp2f(m_run - m_use);
    uint32_t pa[4];
    {
      const float p00 = exp2f(s[0][0] - m_use), p01 = exp2f(s[0][1] - m_use);
      const float p10 = exp2f(s[1][0] - m_use), p11 = exp2f(s[1][1] - m_use);
      l_part = l_part * corr + (p00 + p01 + p10 + p11);
      float w00 = p00, w01 = p01, w10 = p10, w11 = p11;
      if constexpr (INT8) {  // V scales ride on P
        w00 *= sc[16 + 2 * t4];
        w01 *= sc[16 + 2 * t4 + 1];
        w10 *= sc[16 + 8 + 2 * t4];
        w11 *= sc[16 + 8 + 2 * t4 + 1];
      }
      pa[0] = MmaT<MT>::pack(w00, w01);  // (head g, tokens 2t, 2t+1)
      pa[1] = 0u;                       // heads g + 8: padding
      pa[2] = MmaT<MT>::pack(w10, w11);  // (head g, tokens 8 + 2t, +1)
      pa[3] = 0u;
    }
    m_run = m_new;
    // ---- O = O * corr + P V
#pragma unroll
    for (int nb2 = 0; nb2 < D / 16; ++nb2) {
      // matrices (transposed on load): (tokens 0-7, d 0-7), (tokens 8-15, d 0-7), (tokens 0-7, d 8-15), (tokens 8-15, d 8-15)
      uint32_t vb[4];
      const int mat = lane >> 3;
      const int r = (mat & 1) * 8 + (lane & 7);
      ldsm_x4_trans(vb, sV + r * kRowBytes + nb2 * 32 + (mat >> 1) * 16);
      float c0[4] = {o[2 * nb2][0] * corr, o[2 * nb2][1] * corr, 0.f, 0.f};
      float c1[4] = {o[2 * nb2 + 1][0] * corr, o[2 * nb2 + 1][1] * corr, 0.f, 0.f};
      MmaT<MT>::mma(c0, pa, vb[0], vb[1]);
      MmaT<MT>::mma(c1, pa, vb[2], vb[3]);
      o[2 * nb2][0] = c0[0];
      o[2 * nb2][1] = c0[1];
      o[2 * nb2 + 1][0] = c1[0];
      o[2 * nb2 + 1][1] = c1[1];
    }
    __syncwarp();  // the stage may be overwritten by the copies issued in the next iteration
  }
  cp_async_wait<0>();

  // ---- finish the row sums, merge the 4 warps through shared memory
  float l_run = l_part;
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  __syncthreads();  // every warp is done with its ring: reuse the front of the buffer
  float* sm_o = reinterpret_cast<float*>(smem);               // [kWarps][8][D]
  float* sm_m = sm_o + kWarps * 8 * D;                        // [kWarps][8]
  float* sm_l = sm_m + kWarps * 8;
  if (g < p.gh) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      sm_o[(warp * 8 + g) * D + i * 8 + 2 * t4] = o[i][0];
      sm_o[(warp * 8 + g) * D + i * 8 + 2 * t4 + 1] = o[i][1];
    }
    if (t4 == 0) {
      sm_m[warp * 8 + g] = m_run;
      sm_l[warp * 8 + g] = l_run;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.gh * D; idx += kWarps * 32) {
    const int hh = idx / D, d = idx % D;
    float nm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) nm = fmaxf(nm, sm_m[w * 8 + hh]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_m[w * 8 + hh];
      const float c = mw == -INFINITY ? 0.f : exp2f(mw - nm);
      acc += sm_o[(w * 8 + hh) * D + d] * c;
      ll += sm_l[w * 8 + hh] * c;
    }
    const int h = h0 + hh;
    if (p.splits == 1) {
      static_cast<T*>(p.out)[(static_cast<long long>(a) * p.H + h) * D + d] = from_f32<T>(ll > 0.f ? acc / ll : 0.f);
    } else {
      const long long pi = (static_cast<long long>(a) * p.H + h) * p.splits + split;
      p.part_o[pi * D + d] = acc;
      if (d == 0) {
        p.part_ml[pi * 2] = nm;
        p.part_ml[pi * 2 + 1] = ll;
      }
    }
  }
}

template <typename T, int D, bool INT8>
int launch_mma(const MmaDecParams& p, cudaStream_t s) {
  constexpr int kRowBytes = D * 2 + 16;
  constexpr int kTileBytes = kTile * kRowBytes;
  constexpr int kRawTile = kTile * (INT8 ? D : D * 2);
  constexpr int kStageBytes = INT8 ? (kTile * (D + 16) + kRawTile + 2 * kTile * 4) : 2 * kTileBytes;
  constexpr int ring = kWarps * (kStagesD * kStageBytes + (INT8 ? kTileBytes : 0));
  constexpr int merge = (kWarps * 8 * D + 2 * kWarps * 8) * 4;
  constexpr int smem = (ring > merge ? ring : merge) + 128;
  auto kern = paged_decode_mma_kernel<T, D, INT8>;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr.set();
  }
  const int G = p.H / p.Hkv;
  dim3 grid(p.splits, p.Hkv * (G / p.gh), p.A);
  launch_pdl(kern, grid, dim3(kWarps * 32), smem, s, pdl_all_enabled(), p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Called by tsb_paged_decode for bf16 / fp16 pools. Returns -100 when the shape is not covered here.
int paged_decode_mma_dispatch(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                              const float* v_scale, const int* tables, const int* lens,
                              void* out, float* part_o, float* part_ml, int A, int H, int Hkv, int D, int bs, int nb,
                              int max_logical, int splits, int gh, float scale_log2, int dtype, cudaStream_t s) {
  if (gh > 8 || (D != 64 && D != 128)) return -100;
  MmaDecParams p;
  p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.k_scale = k_scale; p.v_scale = v_scale;
  p.tables = tables; p.lens = lens; p.out = out;
  p.part_o = part_o; p.part_ml = part_ml;
  p.A = A; p.H = H; p.Hkv = Hkv; p.bs = bs; p.nb = nb; p.max_logical = max_logical; p.splits = splits; p.gh = gh;
  p.scale_log2 = scale_log2;
  p.status = device_status_word();
  const bool i8 = k_scale != nullptr;
  if (dtype == 1) {
    if (D == 128) return i8 ? launch_mma<__nv_bfloat16, 128, true>(p, s) : launch_mma<__nv_bfloat16, 128, false>(p, s);
    return i8 ? launch_mma<__nv_bfloat16, 64, true>(p, s) : launch_mma<__nv_bfloat16, 64, false>(p, s);
  }
  if (dtype == 2) {
    if (D == 128) return i8 ? launch_mma<__half, 128, true>(p, s) : launch_mma<__half, 128, false>(p, s);
    return i8 ? launch_mma<__half, 64, true>(p, s) : launch_mma<__half, 64, false>(p, s);
  }
  return -100;
}

}  // namespace tsb
