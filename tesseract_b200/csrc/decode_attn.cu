// Decode-time attention over a paged KV pool (split-K, GQA-grouped, bf16/fp16 or INT8 KV) and the
// fused RoPE + KV-append (+ INT8 quantisation) kernel that feeds it.
//
// Pool layout [num_blocks, Hkv, block_size, D] (+ fp32 scales [num_blocks, Hkv, block_size] for INT8),
// block_tables int32 [A, max_logical], lens int32 [A]: the reference's layout (src/nn/PagedKVPool.cpp:27-29,
// src/cuda/PagedAttention.cu:88-262). A contiguous cache [B, Hkv, max_len, D] is the special case
// block_size = max_len with block table {b}.
//
// Differences from the reference kernels (one CTA per (request, query head), no split over keys):
//   * one CTA per (split, KV head, request) serves all G = H / Hkv query heads of the group, so K and V
//     are read from HBM once per KV head instead of once per query head;
//   * the key range of a request is split across CTAs (flash-decoding) and merged by a second kernel, so
//     a few long requests still fill 148 SMs;
//   * 128-bit loads: 8 lanes cover one D = 128 row, 4 tokens per warp per step, two steps in flight.
// The INT8 path dequantises in registers: s = (q . kq) * k_scale, o += p * v_scale * vq
// (per-(token, head) symmetric scales, src/cuda/QuantizeKV.cu:51-72).
#include "common.cuh"
#include "tsb_no_alloc.h"

#include <cuda_fp8.h>

#include <atomic>
#include <mutex>

namespace tsb {

int paged_decode_mma_dispatch(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                              const float* v_scale, const int* tables, const int* lens, void* out, float* part_o, float* part_ml, int A, int H, int Hkv, int D, int bs, int nb,
                              int max_logical, int splits, int gh, float scale_log2, int dtype, cudaStream_t s);

namespace {

// Scratch of tsb_paged_decode_static: lives in the library image, one copy per GPU that loads it.
static __device__ __align__(256) float g_static_decode_scratch[TSB_STATIC_DECODE_SCRATCH_FLOATS];

constexpr int kDecThreads = 128;
constexpr int kDecWarps = 4;

template <typename T>
__device__ __forceinline__ void cvt16(const uint4& a, const uint4& b, float (&f)[16]) {
  const T* pa = reinterpret_cast<const T*>(&a);
  const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    f[i] = to_f32<T>(pa[i]);
    f[8 + i] = to_f32<T>(pb[i]);
  }
}
__device__ __forceinline__ void cvt16_i8(const uint4& a, float (&f)[16]) {
  const int8_t* p = reinterpret_cast<const int8_t*>(&a);
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = static_cast<float>(p[i]);
}

struct DecParams {
  const void* q;        // [A, H, D]
  const void* k_pool;   // [nb, Hkv, bs, D]
  const void* v_pool;
  const float* k_scale; // [nb, Hkv, bs] or null
  const float* v_scale;
  const int* tables;    // [A, max_logical]
  const int* lens;      // [A]
  void* out;            // [A, H, D]
  float* part_o;        // [A, H, splits, D]
  float* part_ml;       // [A, H, splits, 2]
  int A, H, Hkv, bs, nb, max_logical, splits;
  float scale_log2;
};

// EPL = elements per lane (D / 8): 16 for D = 128, 8 for D = 64. GH = query heads handled per CTA.
template <typename T, bool INT8, int D, int GH>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_kernel(DecParams p) {
  constexpr int EPL = D / 8;
  const int split = blockIdx.x;
  const int hgrp = blockIdx.y;  // index over Hkv * (G / GH)
  const int a = blockIdx.z;
  const int G = p.H / p.Hkv;
  const int sub = G / GH;
  const int hk = hgrp / sub;
  const int h0 = hk * G + (hgrp % sub) * GH;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3;   // token slot within the warp step (0..3)
  const int gl = lane & 7;     // lane within the 8-lane group: covers elements [gl*EPL, gl*EPL+EPL)

  const int len = p.lens[a];
  const int chunk = ((len + p.splits - 1) / p.splits + 15) & ~15;
  const int t_begin = split * chunk;
  const int t_end = min(len, t_begin + chunk);

  // q slices in registers (fp32), pre-scaled by softmax scale * log2(e)
  float qf[GH][EPL];
  {
    const T* qbase = static_cast<const T*>(p.q) + (static_cast<long long>(a) * p.H + h0) * D + gl * EPL;
#pragma unroll
    for (int g = 0; g < GH; ++g) {
#pragma unroll
      for (int i = 0; i < EPL; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(qbase + g * D + i);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < 8; ++j) qf[g][i + j] = to_f32<T>(e[j]) * p.scale_log2;
      }
    }
  }
  float o[GH][EPL];
  float m[GH], l[GH];
#pragma unroll
  for (int g = 0; g < GH; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[g][i] = 0.f;
  }

  const int* table = p.tables + static_cast<long long>(a) * p.max_logical;
  constexpr int kRaw = INT8 ? (EPL / 16 > 0 ? EPL / 16 : 1) : EPL / 8;  // 16-byte words per K (or V) slice
  constexpr int U = 2;                                                   // tokens in flight per lane group
  // Each warp iteration covers 8 tokens (two per 8-lane group). All loads of an iteration (K, V, scales, and
  // the block ids of the NEXT iteration) are issued before any arithmetic, so ~128 B per lane are in flight.
  auto block_of = [&](int t) -> int {
    int blk = t < t_end ? table[t / p.bs] : 0;
    return (blk < 0 || blk >= p.nb) ? 0 : blk;  // defence in depth, as in the reference kernels
  };
  int t0 = t_begin + warp * (4 * U);
  int blk_next[U];
#pragma unroll
  for (int u = 0; u < U; ++u) blk_next[u] = block_of(t0 + u * 4 + grp);
  for (; t0 < t_end; t0 += kDecWarps * 4 * U) {
    uint4 kraw[U][kRaw], vraw[U][kRaw];
    float ks[U], vs[U];
    bool valid[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * 4 + grp;
      valid[u] = t < t_end;
      ks[u] = vs[u] = 1.f;
      if (valid[u]) {
        const long long row = (static_cast<long long>(blk_next[u]) * p.Hkv + hk) * p.bs + (t % p.bs);
        const size_t off = (static_cast<size_t>(row) * D + gl * EPL) * (INT8 ? 1 : sizeof(T));
        const char* kp = static_cast<const char*>(p.k_pool) + off;
        const char* vp = static_cast<const char*>(p.v_pool) + off;
        if constexpr (INT8 && EPL == 8) {
          const uint2 k2 = *reinterpret_cast<const uint2*>(kp);
          const uint2 v2 = *reinterpret_cast<const uint2*>(vp);
          kraw[u][0] = make_uint4(k2.x, k2.y, 0, 0);
          vraw[u][0] = make_uint4(v2.x, v2.y, 0, 0);
        } else {
#pragma unroll
          for (int w = 0; w < kRaw; ++w) {
            kraw[u][w] = *reinterpret_cast<const uint4*>(kp + w * 16);
            vraw[u][w] = *reinterpret_cast<const uint4*>(vp + w * 16);
          }
        }
        if constexpr (INT8) {
          ks[u] = p.k_scale[row];
          vs[u] = p.v_scale[row];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) blk_next[u] = block_of(t0 + kDecWarps * 4 * U + u * 4 + grp);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float kf[EPL], vf[EPL];
      if constexpr (INT8) {
        const int8_t* k8 = reinterpret_cast<const int8_t*>(&kraw[u][0]);
        const int8_t* v8 = reinterpret_cast<const int8_t*>(&vraw[u][0]);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          kf[i] = valid[u] ? static_cast<float>(k8[i]) : 0.f;
          vf[i] = valid[u] ? static_cast<float>(v8[i]) : 0.f;
        }
      } else {
        const T* ke = reinterpret_cast<const T*>(&kraw[u][0]);
        const T* ve = reinterpret_cast<const T*>(&vraw[u][0]);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          kf[i] = valid[u] ? to_f32<T>(ke[i]) : 0.f;
          vf[i] = valid[u] ? to_f32<T>(ve[i]) : 0.f;
        }
      }
#pragma unroll
      for (int g = 0; g < GH; ++g) {
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; i += 2) {
          s0 = fmaf(qf[g][i], kf[i], s0);
          s1 = fmaf(qf[g][i + 1], kf[i + 1], s1);
        }
        float sc = s0 + s1;
        sc += __shfl_xor_sync(0xffffffffu, sc, 1);
        sc += __shfl_xor_sync(0xffffffffu, sc, 2);
        sc += __shfl_xor_sync(0xffffffffu, sc, 4);
        sc *= ks[u];
        if (valid[u]) {
          if (sc > m[g]) {
            const float corr = exp2f(m[g] - sc);  // 0 when m was -inf
            l[g] *= corr;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[g][i] *= corr;
            m[g] = sc;
          }
          const float pr = exp2f(sc - m[g]);
          l[g] += pr;
          const float pv = pr * vs[u];
#pragma unroll
          for (int i = 0; i < EPL; ++i) o[g][i] = fmaf(pv, vf[i], o[g][i]);
        }
      }
    }
  }

  // merge the 4 token groups of the warp (lanes with equal gl), then the 4 warps through shared memory
#pragma unroll
  for (int off = 8; off <= 16; off <<= 1) {
#pragma unroll
    for (int g = 0; g < GH; ++g) {
      const float om = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float ol = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float nm = fmaxf(m[g], om);
      const float c0 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - nm);
      const float c1 = (om == -INFINITY) ? 0.f : exp2f(om - nm);
      l[g] = l[g] * c0 + ol * c1;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const float oo = __shfl_xor_sync(0xffffffffu, o[g][i], off);
        o[g][i] = o[g][i] * c0 + oo * c1;
      }
      m[g] = nm;
    }
  }
  __shared__ float sm_o[kDecWarps][GH][D];
  __shared__ float sm_m[kDecWarps][GH];
  __shared__ float sm_l[kDecWarps][GH];
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < GH; ++g) {
#pragma unroll
      for (int i = 0; i < EPL; ++i) sm_o[warp][g][gl * EPL + i] = o[g][i];
      if (gl == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
    }
  }
  __syncthreads();
  // thread tid handles (g, d) pairs
  for (int idx = threadIdx.x; idx < GH * D; idx += kDecThreads) {
    const int g = idx / D, d = idx % D;
    float nm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) nm = fmaxf(nm, sm_m[w][g]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float c = (sm_m[w][g] == -INFINITY) ? 0.f : exp2f(sm_m[w][g] - nm);
      acc += sm_o[w][g][d] * c;
      ll += sm_l[w][g] * c;
    }
    const int h = h0 + g;
    if (p.splits == 1) {
      const float inv = ll > 0.f ? 1.f / ll : 0.f;
      static_cast<T*>(p.out)[(static_cast<long long>(a) * p.H + h) * D + d] = from_f32<T>(acc * inv);
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

template <typename T, int D>
__global__ void __launch_bounds__(D)
decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, T* __restrict__ out,
                    int splits) {
  pdl_trigger();
  pdl_grid_wait();
  const long long ah = blockIdx.x;  // a * H + h
  const int d = threadIdx.x;
  float nm = -INFINITY;
  for (int s = 0; s < splits; ++s) nm = fmaxf(nm, part_ml[(ah * splits + s) * 2]);
  float acc = 0.f, ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(ah * splits + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - nm);
    acc += part_o[(ah * splits + s) * D + d] * c;
    ll += part_ml[(ah * splits + s) * 2 + 1] * c;
  }
  out[ah * D + d] = from_f32<T>(ll > 0.f ? acc / ll : 0.f);
}

// The merge of the key splits for head_dim 128 that hands its result on as the MX operand of the output projection:
// the bf16-rounded head (what decode_merge_kernel stores) is quantised to E4M3 with one power-of-two scale per 32
// values -- a warp of this CTA is one such block -- and the four exponent bytes of a head are the scale word of
// (row a, 128-byte K chunk h), at sf[h * m_pad + a]: the layout quant_act_mx_kernel writes for a [A, H * 128] matrix.
__global__ void __launch_bounds__(128)
decode_merge_quant_mx_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                             uint8_t* __restrict__ xq, uint32_t* __restrict__ sf, int splits, int H, int m_pad) {
  constexpr int D = 128;
  pdl_trigger();
  pdl_grid_wait();
  __shared__ uint32_t s_exp[4];
  const long long ah = blockIdx.x;  // a * H + h
  const int d = threadIdx.x;
  float nm = -INFINITY;
  for (int s = 0; s < splits; ++s) nm = fmaxf(nm, part_ml[(ah * splits + s) * 2]);
  float acc = 0.f, ll = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[(ah * splits + s) * 2];
    const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - nm);
    acc += part_o[(ah * splits + s) * D + d] * c;
    ll += part_ml[(ah * splits + s) * 2 + 1] * c;
  }
  const float v = __bfloat162float(__float2bfloat16(ll > 0.f ? acc / ll : 0.f));
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int e = mx_exponent_byte(amax);
  xq[ah * D + d] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v * mx_inv_scale(e), __NV_SATFINITE, __NV_E4M3));
  if ((d & 31) == 0) s_exp[d >> 5] = static_cast<uint32_t>(e);
  __syncthreads();
  if (d == 0) {
    const int a = static_cast<int>(ah / H), h = static_cast<int>(ah % H);
    sf[static_cast<long long>(h) * m_pad + a] = s_exp[0] | (s_exp[1] << 8) | (s_exp[2] << 16) | (s_exp[3] << 24);
  }
}

int choose_splits(int A, int Hkv_groups, int max_len) {
  // enough CTAs for ~6 per SM (they are latency-bound and small), but never chunks shorter than 256 keys
  static const int per_sm = [] {
    const char* e = getenv("TESSERACT_DECODE_CTAS_PER_SM");
    const int v = e ? atoi(e) : 0;
    return v > 0 && v <= 64 ? v : 6;
  }();
  const int target = sm_count() * per_sm;
  int s = (target + A * Hkv_groups - 1) / (A * Hkv_groups);
  const int max_s = max_len / 256 > 0 ? max_len / 256 : 1;
  if (s > max_s) s = max_s;
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  return s;
}

// Query heads per CTA and number of key splits for a problem; shared by both entry points so that they always
// agree. Full-precision pools run on the tensor-core kernel (up to 8 heads per CTA), INT8 pools on the CUDA-core one.
void decode_plan(int A, int H, int Hkv, int max_len, bool int8, int* gh, int* splits) {
  const int G = H / Hkv;
  (void)int8;  // both KV formats run on the tensor-core kernel: up to 8 query heads per CTA
  int g = G >= 8 ? 8 : G;
  while (G % g) --g;
  *gh = g;
  *splits = choose_splits(A, Hkv * (G / g), max_len);
}

template <typename T, bool INT8, int D>
int launch_decode(DecParams p, int G, cudaStream_t s) {
  const int GH = (G % 4 == 0) ? 4 : ((G % 2 == 0) ? 2 : 1);  // heads per CTA (decode_plan uses the same rule)
  dim3 grid(p.splits, p.Hkv * (G / GH), p.A);
  switch (GH) {
    case 4: paged_decode_kernel<T, INT8, D, 4><<<grid, kDecThreads, 0, s>>>(p); break;
    case 2: paged_decode_kernel<T, INT8, D, 2><<<grid, kDecThreads, 0, s>>>(p); break;
    case 1: paged_decode_kernel<T, INT8, D, 1><<<grid, kDecThreads, 0, s>>>(p); break;
    default: return -2;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (p.splits > 1) {
    decode_merge_kernel<T, D><<<p.A * p.H, D, 0, s>>>(p.part_o, p.part_ml, static_cast<T*>(p.out), p.splits);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

// ------------------------------------------------------------------ RoPE + KV append (+ INT8 quant)
// One warp per (token, head) over the H + 2 Hkv heads of a packed projection row.
//   query heads: rotated, written to q_out (or in place);
//   key heads:   rotated, then stored to the pool slot of the token (quantised if the pool is INT8);
//   value heads: stored to the pool.
template <typename T, bool INT8, int D>
__global__ void __launch_bounds__(256)
kv_append_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                 const int* __restrict__ positions, const int* __restrict__ slots, void* __restrict__ k_pool,
                 void* __restrict__ v_pool, float* __restrict__ k_scale, float* __restrict__ v_scale,
                 T* __restrict__ q_out, int tokens, int H, int Hkv, int bs, int rotate) {
  pdl_trigger();
  pdl_grid_wait();
  constexpr int EPL = D / 32;  // 4 (D=128) or 2 (D=64): an even count, so rotation pairs stay in-lane
  const long long wid = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int HT = H + 2 * Hkv;
  if (wid >= static_cast<long long>(tokens) * HT) return;
  const int head = static_cast<int>(wid % HT);
  const int t = static_cast<int>(wid / HT);
  T* src = qkv + (static_cast<long long>(t) * HT + head) * D + lane * EPL;
  float x[EPL];
  if constexpr (EPL == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = to_f32<T>(e[i]);
  } else {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(src);
    const T* e = reinterpret_cast<const T*>(&raw);
    x[0] = to_f32<T>(e[0]);
    x[1] = to_f32<T>(e[1]);
  }
  const bool is_q = head < H;
  const bool is_k = !is_q && head < H + Hkv;
  if (rotate && (is_q || is_k)) {
    const int pos = positions[t];
    const float* c = cos_t + static_cast<long long>(pos) * (D / 2) + lane * (EPL / 2);
    const float* s = sin_t + static_cast<long long>(pos) * (D / 2) + lane * (EPL / 2);
#pragma unroll
    for (int i = 0; i < EPL; i += 2) {
      const float a = x[i], b = x[i + 1], cc = c[i / 2], ss = s[i / 2];
      x[i] = a * cc - b * ss;
      x[i + 1] = a * ss + b * cc;
    }
  }
  if (is_q) {
    T* dst = (q_out ? q_out + (static_cast<long long>(t) * H + head) * D : qkv + (static_cast<long long>(t) * HT + head) * D) +
             lane * EPL;
    if constexpr (EPL == 4) {
      uint2 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) e[i] = from_f32<T>(x[i]);
      *reinterpret_cast<uint2*>(dst) = o;
    } else {
      uint32_t o;
      T* e = reinterpret_cast<T*>(&o);
      e[0] = from_f32<T>(x[0]);
      e[1] = from_f32<T>(x[1]);
      *reinterpret_cast<uint32_t*>(dst) = o;
    }
    return;
  }
  const int slot = slots[t];
  if (slot < 0) return;  // token without a cache slot (padding)
  const int kvh = is_k ? head - H : head - H - Hkv;
  const int blk = slot / bs, off = slot % bs;
  const long long row = (static_cast<long long>(blk) * Hkv + kvh) * bs + off;
  void* pool = is_k ? k_pool : v_pool;
  if constexpr (INT8) {
    // the model dtype round trip first: what is quantised is what a full-precision cache would hold
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      x[i] = to_f32<T>(from_f32<T>(x[i]));
      amax = fmaxf(amax, fabsf(x[i]));
    }
    amax = warp_max(amax);
    const float scale = amax > 0.f ? amax / 127.f : 1.f;
    int8_t qv[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      float r = rintf(x[i] / scale);
      r = fminf(127.f, fmaxf(-127.f, r));
      qv[i] = static_cast<int8_t>(r);
    }
    int8_t* dst = static_cast<int8_t*>(pool) + row * D + lane * EPL;
    if constexpr (EPL == 4) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(qv);
    else *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<uint16_t*>(qv);
    if (lane == 0) (is_k ? k_scale : v_scale)[row] = scale;
  } else {
    T* dst = static_cast<T*>(pool) + row * D + lane * EPL;
    if constexpr (EPL == 4) {
      uint2 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) e[i] = from_f32<T>(x[i]);
      *reinterpret_cast<uint2*>(dst) = o;
    } else {
      uint32_t o;
      T* e = reinterpret_cast<T*>(&o);
      e[0] = from_f32<T>(x[0]);
      e[1] = from_f32<T>(x[1]);
      *reinterpret_cast<uint32_t*>(dst) = o;
    }
  }
}

}  // namespace
}  // namespace tsb

// fp32 scratch elements tsb_paged_decode may use for A requests, H query heads, head_dim D and a
// longest sequence of max_len tokens (split partials: A * H * splits * (D + 2)).
TSB_EXPORT long long tsb_paged_decode_scratch_floats(int A, int H, int D, int max_len) {
  const long long splits = 64;
  (void)max_len;
  return static_cast<long long>(A) * H * splits * (D + 2);
}

// out[a, h, :] = attention of query q[a, h, :] over the first lens[a] pooled tokens of request a.
//   dtype: 1 = bf16, 2 = fp16 (q, out, and the pool unless k_scale != NULL, in which case the pool is INT8).
//   max_len: upper bound of lens (sizes the key split); scratch: tsb_paged_decode_scratch_floats() floats.
TSB_EXPORT int tsb_paged_decode(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                                const float* v_scale, const int* tables, const int* lens, void* out, float* scratch,
                                int A, int H, int Hkv, int D, int bs, int nb, int max_logical, float scale,
                                int max_len, int dtype, void* stream) {
  using namespace tsb;
  if (A <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128) || bs <= 0) return -2;
  const int G = H / Hkv;
  const bool i8 = k_scale != nullptr;
  int gh = 1, splits = 1;
  decode_plan(A, H, Hkv, max_len, i8, &gh, &splits);
  float* part_o = scratch;
  float* part_ml = scratch + static_cast<long long>(A) * H * splits * D;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    int rc = paged_decode_mma_dispatch(q, k_pool, v_pool, k_scale, v_scale, tables, lens, out, part_o, part_ml, A, H, Hkv, D, bs, nb,
                                       max_logical, splits, gh, scale * 1.4426950408889634f, dtype, s);
    if (rc != -100) {
      if (rc != 0 || splits == 1) return rc;
      if (dtype == 1) {
        const bool pdl = pdl_all_enabled();
        if (D == 128) launch_pdl(decode_merge_kernel<__nv_bfloat16, 128>, dim3(A * H), dim3(128), 0, s, pdl, part_o, part_ml, static_cast<__nv_bfloat16*>(out), splits);
        else launch_pdl(decode_merge_kernel<__nv_bfloat16, 64>, dim3(A * H), dim3(64), 0, s, pdl, part_o, part_ml, static_cast<__nv_bfloat16*>(out), splits);
      } else {
        const bool pdl = pdl_all_enabled();
        if (D == 128) launch_pdl(decode_merge_kernel<__half, 128>, dim3(A * H), dim3(128), 0, s, pdl, part_o, part_ml, static_cast<__half*>(out), splits);
        else launch_pdl(decode_merge_kernel<__half, 64>, dim3(A * H), dim3(64), 0, s, pdl, part_o, part_ml, static_cast<__half*>(out), splits);
      }
      return static_cast<int>(cudaGetLastError());
    }
  }
  DecParams p;
  p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.k_scale = k_scale; p.v_scale = v_scale;
  p.tables = tables; p.lens = lens; p.out = out;
  p.A = A; p.H = H; p.Hkv = Hkv; p.bs = bs; p.nb = nb; p.max_logical = max_logical;
  p.splits = splits;
  p.part_o = part_o;
  p.part_ml = part_ml;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (dtype == 1) {
    if (D == 128) return i8 ? launch_decode<__nv_bfloat16, true, 128>(p, G, s) : launch_decode<__nv_bfloat16, false, 128>(p, G, s);
    return i8 ? launch_decode<__nv_bfloat16, true, 64>(p, G, s) : launch_decode<__nv_bfloat16, false, 64>(p, G, s);
  }
  if (dtype == 2) {
    if (D == 128) return i8 ? launch_decode<__half, true, 128>(p, G, s) : launch_decode<__half, false, 128>(p, G, s);
    return i8 ? launch_decode<__half, true, 64>(p, G, s) : launch_decode<__half, false, 64>(p, G, s);
  }
  return -2;
}

extern "C" int tsb_quant_act_mx_layout(const void* X, long long ldx, void* Xq, void* sf, int M, int K, int atoms,
                                       void* stream);
extern "C" int tsb_mx_m_pad(int M);

// tsb_paged_decode whose result also leaves as the E4M3 + power-of-two-scale operand of an MX GEMM: xq [A, H * D]
// bytes and sf [H * D / 128, tsb_mx_m_pad(A)] scale words (the layout of tsb_quant_act_mx). With head_dim 128, bf16
// and more than one key split the merge kernel writes the operand itself and `out` is left untouched; otherwise the
// attention runs as usual into `out` and the quantiser follows.
TSB_EXPORT int tsb_paged_decode_mx(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                                   const float* v_scale, const int* tables, const int* lens, void* out,
                                   float* scratch, void* xq, void* sf, int A, int H, int Hkv, int D, int bs, int nb,
                                   int max_logical, float scale, int max_len, int dtype, void* stream) {
  using namespace tsb;
  if (A <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128) || bs <= 0 || (H * D) % 128) return -2;
  int gh = 1, splits = 1;
  decode_plan(A, H, Hkv, max_len, k_scale != nullptr, &gh, &splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (D == 128 && dtype == 1 && splits > 1) {
    float* part_o = scratch;
    float* part_ml = scratch + static_cast<long long>(A) * H * splits * D;
    const int rc = paged_decode_mma_dispatch(q, k_pool, v_pool, k_scale, v_scale, tables, lens, out, part_o, part_ml, A, H,
                                             Hkv, D, bs, nb, max_logical, splits, gh, scale * 1.4426950408889634f,
                                             dtype, s);
    if (rc == 0) {
      launch_pdl(decode_merge_quant_mx_kernel, dim3(A * H), dim3(128), 0, s, pdl_all_enabled(), part_o, part_ml,
                 static_cast<uint8_t*>(xq), static_cast<uint32_t*>(sf), splits, H, tsb_mx_m_pad(A));
      return static_cast<int>(cudaGetLastError());
    }
    if (rc != -100) return rc;
  }
  const int rc = tsb_paged_decode(q, k_pool, v_pool, k_scale, v_scale, tables, lens, out, scratch, A, H, Hkv, D, bs, nb,
                                  max_logical, scale, max_len, dtype, stream);
  if (rc != 0) return rc;
  return tsb_quant_act_mx_layout(out, static_cast<long long>(H) * D, xq, sf, A, H * D, 0, stream);
}

// Rotate (adjacent-pair RoPE at positions[t]) the query and key heads of packed qkv [tokens, (H + 2 Hkv) * D],
// write queries to q_out [tokens, H, D] (in place when NULL) and scatter keys / values into the pool at
// slots[t] = block * block_size + offset (negative = skip). With k_scale != NULL the pool is INT8 and
// the per-(token, head) scales are written too. rotate = 0 skips RoPE.
TSB_EXPORT int tsb_kv_append_paged(void* qkv, const float* cos_t, const float* sin_t, const int* positions,
                                   const int* slots, void* k_pool, void* v_pool, float* k_scale, float* v_scale,
                                   void* q_out, int tokens, int H, int Hkv, int D, int bs, int dtype, int rotate,
                                   void* stream) {
  using namespace tsb;
  if (tokens <= 0 || (D != 64 && D != 128) || bs <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long warps = static_cast<long long>(tokens) * (H + 2 * Hkv);
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  const bool i8 = k_scale != nullptr;
#define TSB_KVA(TT, I8, DD)                                                                                      \
  launch_pdl(kv_append_kernel<TT, I8, DD>, dim3(blocks), dim3(256), 0, s, pdl_all_enabled(), static_cast<TT*>(qkv), \
             cos_t, sin_t, positions, slots, k_pool, v_pool, k_scale, v_scale, static_cast<TT*>(q_out), tokens, H, Hkv,  \
             bs, rotate)
  if (dtype == 1) {
    if (D == 128) { if (i8) TSB_KVA(__nv_bfloat16, true, 128); else TSB_KVA(__nv_bfloat16, false, 128); }
    else { if (i8) TSB_KVA(__nv_bfloat16, true, 64); else TSB_KVA(__nv_bfloat16, false, 64); }
  } else if (dtype == 2) {
    if (D == 128) { if (i8) TSB_KVA(__half, true, 128); else TSB_KVA(__half, false, 128); }
    else { if (i8) TSB_KVA(__half, true, 64); else TSB_KVA(__half, false, 64); }
  } else {
    return -2;
  }
#undef TSB_KVA
  return static_cast<int>(cudaGetLastError());
}

// See tsb_no_alloc.h for the contract. The address of the file-scope array is looked up once per device
// (with that device current) and cached; host code must never hand the symbol itself to a kernel.
TSB_EXPORT int tsb_paged_decode_static(const void* q, const void* k_pool, const void* v_pool, const float* k_scale,
                                       const float* v_scale, const int* tables, const int* lens, void* out, int A,
                                       int H, int Hkv, int D, int bs, int nb, int max_logical, float scale,
                                       int max_len, int dtype, void* stream) {
  using namespace tsb;
  static std::atomic<float*> scratch_of_device[64];   // zero-initialised; read without the lock on the fast path
  static std::mutex mu;
  if (A <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || (D != 64 && D != 128) || bs <= 0) return -2;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -2;
  float* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (!scratch) {
    std::lock_guard<std::mutex> lk(mu);
    scratch = scratch_of_device[dev].load(std::memory_order_relaxed);
    if (!scratch) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_decode_scratch);
      if (e != cudaSuccess) return static_cast<int>(e);
      scratch = static_cast<float*>(p);
      scratch_of_device[dev].store(scratch, std::memory_order_release);
    }
  }
  int gh = 1, splits = 1;
  decode_plan(A, H, Hkv, max_len, k_scale != nullptr, &gh, &splits);
  const long long need = splits > 1 ? static_cast<long long>(A) * H * splits * (D + 2) : 0;
  if (need > TSB_STATIC_DECODE_SCRATCH_FLOATS) return TSB_ERR_STATIC_SCRATCH_TOO_SMALL;
  // Same code path as tsb_paged_decode from here on: identical split count, identical kernels.
  return tsb_paged_decode(q, k_pool, v_pool, k_scale, v_scale, tables, lens, out, scratch, A, H, Hkv, D, bs, nb,
                          max_logical, scale, max_len, dtype, stream);
}

TSB_EXPORT long long tsb_paged_decode_static_capacity_floats() { return TSB_STATIC_DECODE_SCRATCH_FLOATS; }

// Host-only: the fp32 elements of split-K scratch the plan for this problem asks for on the current device (0 when
// one key split suffices). tsb_paged_decode_static refuses exactly when this exceeds the capacity above.
TSB_EXPORT long long tsb_paged_decode_static_need_floats(int A, int H, int Hkv, int D, int max_len, int kv_int8) {
  using namespace tsb;
  if (A <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || D <= 0) return -2;
  int gh = 1, splits = 1;
  decode_plan(A, H, Hkv, max_len, kv_int8 != 0, &gh, &splits);
  return splits > 1 ? static_cast<long long>(A) * H * splits * (D + 2) : 0;
}
