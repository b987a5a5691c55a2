// Mixture-of-experts routing on the device: one warp per token computes softmax over the E router logits, picks
// the top-k experts (value descending, index ascending on ties -- the reference's rule, src/nn/MoEFeedForward.cpp:
// 27-50), renormalises the selected probabilities to sum 1 and bumps the per-expert token counters, all in one
// pass and without a host round trip (the reference's kernel uses one CTA per token with the k argmax rounds on
// thread 0, src/cuda/MoeRoute.cu:31-105, and its fused forward synchronises the stream to build offsets on the
// host, src/cuda/MoeForward.cu:241-247). A second kernel turns the counts into offsets and scatters the
// (token, slot) assignments into expert-sorted order, which is the row order of the grouped expert GEMMs.
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kMaxE = 256;  // experts handled per warp: 8 per lane

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ logits, int* __restrict__ topk_idx, float* __restrict__ topk_gate,
                 float* __restrict__ probs_out, int* __restrict__ counts, int tokens, int E, int k) {
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= tokens) return;
  const T* row = logits + static_cast<long long>(warp_global) * E;
  float v[kMaxE / 32];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxE / 32; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? to_f32<T>(row[e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxE / 32; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kMaxE / 32; ++i) {
    v[i] *= inv;
    const int e = lane + 32 * i;
    if (probs_out && e < E) probs_out[static_cast<long long>(warp_global) * E + e] = v[i];
  }
  float gate_sum = 0.f;
  float my_gate = 0.f;
  int my_idx = 0;
  for (int r = 0; r < k; ++r) {
    // lane-local best (lowest index on ties because i ascends), then warp argmax with the same tie rule
    float bv = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxE / 32; ++i) {
      const int e = lane + 32 * i;
      if (e < E && v[i] > bv) {
        bv = v[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    gate_sum += bv;
    if (lane == r % 32) {
      my_gate = bv;
      my_idx = bi;
    }
    if ((bi & 31) == lane) v[bi >> 5] = -2.f;  // remove the winner
    if (r % 32 == 31 || r == k - 1) {
      // flush up to 32 selections held one per lane
      const int base = r - (r % 32);
      if (base + lane <= r) {
        topk_idx[static_cast<long long>(warp_global) * k + base + lane] = my_idx;
        topk_gate[static_cast<long long>(warp_global) * k + base + lane] = my_gate;  // renormalised below
        atomicAdd(&counts[my_idx], 1);
      }
    }
  }
  __syncwarp();
  const float ginv = 1.f / gate_sum;
  for (int r = lane; r < k; r += 32) topk_gate[static_cast<long long>(warp_global) * k + r] *= ginv;
}

// offsets[e] = exclusive prefix sum of counts (E <= 256, one CTA); cursor[e] = offsets[e] (scatter cursors).
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursor,
                                   int E) {
  __shared__ int s[kMaxE];
  const int e = threadIdx.x;
  s[e] = e < E ? counts[e] : 0;
  __syncthreads();
  if (e == 0) {
    int acc = 0;
    for (int i = 0; i < E; ++i) {
      const int c = s[i];
      s[i] = acc;
      acc += c;
    }
    offsets[E] = acc;
  }
  __syncthreads();
  if (e < E) {
    offsets[e] = s[e];
    cursor[e] = s[e];
  }
}

// sorted_pos[t * k + r] = row of assignment (t, r) in expert-sorted order; sorted_token[row] = t.
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const int* __restrict__ topk_idx, int* __restrict__ cursor, int* __restrict__ sorted_pos,
                   int* __restrict__ sorted_token, long long n_assign, int k) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n_assign) return;
  const int e = topk_idx[i];
  const int row = atomicAdd(&cursor[e], 1);
  sorted_pos[i] = row;
  sorted_token[row] = static_cast<int>(i / k);
}

// Padded variant: every expert's row block starts at a multiple of `pad` rows (so that a 128-row GEMM tile never
// holds rows of two experts). offsets[e] are the padded starts, offsets[E] the padded total.
__global__ void moe_offsets_padded_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                          int* __restrict__ cursor, int E, int pad) {
  if (threadIdx.x != 0) return;
  int acc = 0;
  for (int i = 0; i < E; ++i) {
    offsets[i] = acc;
    cursor[i] = acc;
    acc += (counts[i] + pad - 1) / pad * pad;
  }
  offsets[E] = acc;
}

// sorted_pos[i] = row of assignment i = t * k + r in the padded expert-sorted order; sorted_assign[row] = i.
__global__ void __launch_bounds__(256)
moe_scatter_assign_kernel(const int* __restrict__ topk_idx, int* __restrict__ cursor, int* __restrict__ sorted_pos,
                          int* __restrict__ sorted_assign, long long n_assign) {
  const long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (i >= n_assign) return;
  const int row = atomicAdd(&cursor[topk_idx[i]], 1);
  sorted_pos[i] = row;
  sorted_assign[row] = static_cast<int>(i);
}

// dst[row, :] = scale(row) * src[assign[row] / k, :] for rows with assign >= 0, zero otherwise (padding rows).
// scale(row) = row_scale[assign[row]] when row_scale is given. One warp per row, 16-byte accesses (D % 8 == 0).
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ assign,
                       const float* __restrict__ row_scale, __nv_bfloat16* __restrict__ dst, int rows, int D, int k) {
  const int row = static_cast<int>((blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int a = assign[row];
  uint4* out = reinterpret_cast<uint4*>(dst + static_cast<long long>(row) * D);
  const int nvec = D / 8;
  if (a < 0) {
    for (int v = lane; v < nvec; v += 32) out[v] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long long>(a / k) * D);
  if (!row_scale) {
    for (int v = lane; v < nvec; v += 32) out[v] = in[v];
    return;
  }
  const float sc = row_scale[a];
  for (int v = lane; v < nvec; v += 32) {
    uint4 x = in[v];
    __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(e[j]);
      e[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    out[v] = x;
  }
}

// out[t, :] = sum_r w(t, r) * ys[pos[t * k + r], :]; w = gates[t * k + r] or 1 when gates is null. One warp per token.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ pos, const float* __restrict__ gates,
                   __nv_bfloat16* __restrict__ out, int T, int D, int k) {
  const int t = static_cast<int>((blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const int nvec = D / 8;
  for (int v = lane; v < nvec; v += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < k; ++r) {
      const int row = pos[static_cast<long long>(t) * k + r];
      const float w = gates ? gates[static_cast<long long>(t) * k + r] : 1.f;
      const uint4 x = reinterpret_cast<const uint4*>(ys + static_cast<long long>(row) * D)[v];
      const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(e[j]);
        acc[2 * j] += w * f.x;
        acc[2 * j + 1] += w * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + static_cast<long long>(t) * D)[v] = o;
  }
}

// dgate[i] = <dout[i / k, :], ys[pos[i], :]> for every assignment i. One warp per assignment.
__global__ void __launch_bounds__(256)
moe_gate_grad_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ ys,
                     const int* __restrict__ pos, float* __restrict__ dgate, long long n_assign, int D, int k) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n_assign) return;
  const uint4* a = reinterpret_cast<const uint4*>(dout + (i / k) * D);
  const uint4* b = reinterpret_cast<const uint4*>(ys + static_cast<long long>(pos[i]) * D);
  float acc = 0.f;
  for (int v = lane; v < D / 8; v += 32) {
    const uint4 xa = a[v], xb = b[v];
    const __nv_bfloat162* ea = reinterpret_cast<const __nv_bfloat162*>(&xa);
    const __nv_bfloat162* eb = reinterpret_cast<const __nv_bfloat162*>(&xb);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(ea[j]), fb = __bfloat1622float2(eb[j]);
      acc += fa.x * fb.x + fa.y * fb.y;
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dgate[i] = acc;
}

}  // namespace
}  // namespace tsb

// Router: logits [tokens, E] (fp32 / bf16 / fp16, E <= 256) -> topk_idx int32 [tokens, k] (value desc, index asc),
// topk_gate fp32 [tokens, k] (renormalised), probs fp32 [tokens, E] (may be NULL), counts int32 [E] (+=; zero it first).
TSB_EXPORT int tsb_moe_route(const void* logits, int* topk_idx, float* topk_gate, float* probs, int* counts, int tokens,
                             int E, int k, int dtype, void* stream) {
  using namespace tsb;
  if (tokens <= 0 || E <= 0 || E > kMaxE || k <= 0 || k > E) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(tokens) * 32 + 255) / 256);
  switch (dtype) {
    case 0: moe_route_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(logits), topk_idx, topk_gate, probs, counts, tokens, E, k); break;
    case 1: moe_route_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), topk_idx, topk_gate, probs, counts, tokens, E, k); break;
    case 2: moe_route_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(logits), topk_idx, topk_gate, probs, counts, tokens, E, k); break;
    default: return -2;
  }
  return static_cast<int>(cudaGetLastError());
}

// counts [E] -> offsets [E + 1] (exclusive scan, total last) and the expert-sorted permutation of the
// tokens * k assignments: sorted_pos [tokens * k], sorted_token [tokens * k]. cursor: int32 [E] scratch.
TSB_EXPORT int tsb_moe_sort(const int* topk_idx, const int* counts, int* offsets, int* cursor, int* sorted_pos,
                            int* sorted_token, int tokens, int E, int k, void* stream) {
  using namespace tsb;
  if (tokens <= 0 || E <= 0 || E > kMaxE || k <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  moe_offsets_kernel<<<1, kMaxE, 0, s>>>(counts, offsets, cursor, E);
  const long long n = static_cast<long long>(tokens) * k;
  moe_scatter_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(topk_idx, cursor, sorted_pos, sorted_token, n, k);
  return static_cast<int>(cudaGetLastError());
}

// Padded expert sort: like tsb_moe_sort, but every expert's row block starts at a multiple of `pad` (128 for the
// grouped GEMM). sorted_assign: int32 [rows_cap], -1 for padding rows and the unused tail; rows_cap >= the padded
// total (tokens * k + E * (pad - 1) rounded up to pad always suffices).
TSB_EXPORT int tsb_moe_sort_padded(const int* topk_idx, const int* counts, int* offsets, int* cursor, int* sorted_pos,
                                   int* sorted_assign, int tokens, int E, int k, int pad, int rows_cap, void* stream) {
  using namespace tsb;
  if (tokens <= 0 || E <= 0 || E > kMaxE || k <= 0 || pad < 1) return -2;
  const long long n = static_cast<long long>(tokens) * k;
  if (rows_cap < n + static_cast<long long>(E) * (pad - 1)) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(sorted_assign, 0xFF, static_cast<size_t>(rows_cap) * sizeof(int), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  moe_offsets_padded_kernel<<<1, 32, 0, s>>>(counts, offsets, cursor, E, pad);
  moe_scatter_assign_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(topk_idx, cursor, sorted_pos,
                                                                                   sorted_assign, n);
  return static_cast<int>(cudaGetLastError());
}

// dst [rows, D] bf16: row r = (row_scale ? row_scale[assign[r]] : 1) * src[assign[r] / k] or zeros where assign[r] < 0.
TSB_EXPORT int tsb_moe_gather_rows(const void* src, const int* assign, const float* row_scale, void* dst, int rows,
                                   int D, int k, void* stream) {
  using namespace tsb;
  if (rows <= 0 || D <= 0 || D % 8 || k <= 0) return -2;
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(rows) * 32 + 255) / 256);
  moe_gather_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), assign, row_scale, static_cast<__nv_bfloat16*>(dst), rows, D, k);
  return static_cast<int>(cudaGetLastError());
}

// out [T, D] bf16 = sum over the k assignments of a token of (gates ? gates[t, r] : 1) * ys[pos[t, r]].
TSB_EXPORT int tsb_moe_combine(const void* ys, const int* pos, const float* gates, void* out, int T, int D, int k,
                               void* stream) {
  using namespace tsb;
  if (T <= 0 || D <= 0 || D % 8 || k <= 0) return -2;
  const unsigned blocks = static_cast<unsigned>((static_cast<long long>(T) * 32 + 255) / 256);
  moe_combine_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ys), pos, gates, static_cast<__nv_bfloat16*>(out), T, D, k);
  return static_cast<int>(cudaGetLastError());
}

// dgate [T * k] fp32 = <dout[t], ys[pos[t, r]]>.
TSB_EXPORT int tsb_moe_gate_grad(const void* dout, const void* ys, const int* pos, float* dgate, int T, int D, int k,
                                 void* stream) {
  using namespace tsb;
  if (T <= 0 || D <= 0 || D % 8 || k <= 0) return -2;
  const long long n = static_cast<long long>(T) * k;
  const unsigned blocks = static_cast<unsigned>((n * 32 + 255) / 256);
  moe_gate_grad_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(ys), pos, dgate, n, D, k);
  return static_cast<int>(cudaGetLastError());
}
