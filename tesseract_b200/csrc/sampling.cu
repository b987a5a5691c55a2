// Device-side token selection so that a decode step needs no logits transfer:
//   * tsb_argmax_rows        greedy: index of the row maximum (lowest index on ties, like the host sampler)
//   * tsb_sample_top_p_rows  temperature + nucleus sampling without sorting: the probability threshold of the
//                            nucleus is found by a four-pass radix descent over the row (kept hot in L2), then one
//                            uniform draw picks a token among the survivors in index order.
// The host sampler (repetition penalty -> temperature -> top-k -> top-p -> mt19937_64 draw,
// src/models/Sampler.cpp:29-116) stays the bit-exact path for seeded tests; these kernels are the serving fast
// path. The reference copies the whole logits row to the host for every token (src/models/Llama.cpp:481-509).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kSampThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kSampThreads)
argmax_rows_kernel(const T* __restrict__ logits, int* __restrict__ out, int V, long long ld,
                   __nv_bfloat16* __restrict__ packed = nullptr, int rank = 0, int world = 1) {
  __shared__ float sv[kSampThreads / 32];
  __shared__ int si[kSampThreads / 32];
  const T* x = logits + blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int j0 = 0;
  if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    // 16-byte loads, four of them in flight per thread; a thread visits its elements in increasing order, so the
    // strict comparison keeps the lowest index among equal values
    const int nvec = V / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int c0 = threadIdx.x; c0 < nvec; c0 += 4 * blockDim.x) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < nvec) v[u] = xv[c];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < nvec) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float f = to_f32<T>(e[k]);
            if (f > best) {
              best = f;
              bi = c * 8 + k;
            }
          }
        }
      }
    }
    j0 = nvec * 8;
  }
  for (int j = j0 + threadIdx.x; j < V; j += blockDim.x) {
    const float f = to_f32<T>(x[j]);
    if (f > best || (f == best && j < bi)) {
      best = f;
      bi = j;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < kSampThreads / 32 ? sv[lane] : -INFINITY;
    bi = lane < kSampThreads / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (out) out[blockIdx.x] = bi;
      if (packed) {
        // vocabulary-parallel head: this rank's (best value, index as three base-256 digits) in its slot of a
        // [4 * world] row, zeros in the other slots -- the element-wise sum over the ranks (a bf16 all-reduce; every
        // entry is exact in bf16) then holds every rank's candidate
        __nv_bfloat16* row = packed + static_cast<long long>(blockIdx.x) * 4 * world;
        for (int j = 0; j < 4 * world; ++j) row[j] = __float2bfloat16(0.f);
        const int i = bi == 0x7fffffff ? 0 : bi;
        row[4 * rank + 0] = __float2bfloat16(best);
        row[4 * rank + 1] = __float2bfloat16(static_cast<float>(i & 255));
        row[4 * rank + 2] = __float2bfloat16(static_cast<float>((i >> 8) & 255));
        row[4 * rank + 3] = __float2bfloat16(static_cast<float>((i >> 16) & 255));
      }
    }
  }
}

// The other half of the vocabulary-parallel arg-max: row r of `summed` holds (value, index digits) of every rank's
// shard; the winner is the largest value, the lowest rank (= lowest global index) on ties.
__global__ void argmax_unpack_kernel(const __nv_bfloat16* __restrict__ summed, int* __restrict__ out, int rows,
                                     int world, int shard) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const __nv_bfloat16* row = summed + static_cast<long long>(r) * 4 * world;
  float best = __bfloat162float(row[0]);
  int bw = 0;
  for (int w = 1; w < world; ++w) {
    const float v = __bfloat162float(row[4 * w]);
    if (v > best) {
      best = v;
      bw = w;
    }
  }
  const int i = static_cast<int>(__bfloat162float(row[4 * bw + 1])) + (static_cast<int>(__bfloat162float(row[4 * bw + 2])) << 8) +
                (static_cast<int>(__bfloat162float(row[4 * bw + 3])) << 16);
  out[r] = bw * shard + i;
}

__device__ __forceinline__ float block_reduce_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_reduce_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  return warp_max(t);
}

// splitmix64 -> uniform in [0, 1)
__device__ __forceinline__ float uniform_from(unsigned long long seed, unsigned long long row, unsigned long long step) {
  unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (row * 0x100000001B3ull + step + 1);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

// Order-preserving map of a float onto an unsigned integer (for bisection on exact element values).
__device__ __forceinline__ unsigned int float_key(float f) {
  const unsigned int u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(unsigned int k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// In place: logits[row, t] is divided (if positive) or multiplied (otherwise) by `penalty` once per OCCURRENCE of t
// among the row's first hist_len[row] history tokens (the host sampler's rule, src/models/Sampler.cpp:29-50). The
// thread that holds the first occurrence of a token counts the later ones and applies the power in one go.
template <typename T>
__global__ void __launch_bounds__(256)
repetition_penalty_kernel(T* __restrict__ logits, long long ld, int V, const int* __restrict__ history, long long hist_ld,
                          const int* __restrict__ hist_len, float penalty) {
  const int row = blockIdx.x;
  const int n = hist_len[row];
  const int* h = history + row * hist_ld;
  T* x = logits + row * ld;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int t = h[i];
    if (t < 0 || t >= V) continue;
    bool first = true;
    for (int j = 0; j < i; ++j)
      if (h[j] == t) {
        first = false;
        break;
      }
    if (!first) continue;
    int cnt = 1;
    for (int j = i + 1; j < n; ++j) cnt += (h[j] == t) ? 1 : 0;
    float v = to_f32<T>(x[t]);
    for (int c = 0; c < cnt; ++c) v = v > 0.f ? v / penalty : v * penalty;
    x[t] = from_f32<T>(v);
  }
}

// Visits every element of a row once: f(index, value). 16-byte loads (two in flight per thread) when the row allows.
template <typename T, typename F>
__device__ __forceinline__ void for_each_elem(const T* __restrict__ x, int V, F f) {
  int j0 = 0;
  if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int nvec = V / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int c0 = threadIdx.x; c0 < nvec; c0 += 2 * blockDim.x) {
      uint4 v[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < nvec) v[u] = xv[c];
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int c = c0 + u * blockDim.x;
        if (c < nvec) {
          const T* e = reinterpret_cast<const T*>(&v[u]);
#pragma unroll
          for (int k = 0; k < 8; ++k) f(c * 8 + k, to_f32<T>(e[k]));
        }
      }
    }
    j0 = nvec * 8;
  }
  for (int j = j0 + threadIdx.x; j < V; j += blockDim.x) f(j, to_f32<T>(x[j]));
}

// Temperature, top-k, top-p and the draw for one row per CTA, in a handful of passes over the row (which stays in
// L2). The nucleus threshold is found exactly by a radix descent over the bit pattern of the unnormalised
// probabilities e = exp(z - max) (positive floats order like their bits): four passes, each adding the mass of the
// still-undecided elements into 256 bins of the next byte and picking, from the top, the bin in which the cumulative
// mass reaches top_p * sum(e). (A bisection on the threshold needs two dozen passes for the same answer; on a
// 128 K-entry vocabulary that was 1.8 ms per decode step.)
template <typename T>
__global__ void __launch_bounds__(kSampThreads)
sample_top_p_kernel(const T* __restrict__ logits, int* __restrict__ out, int V, long long ld, float inv_temp,
                    float top_p, int top_k, unsigned long long seed, unsigned long long step,
                    const unsigned long long* __restrict__ step_ptr) {
  constexpr int kWarps = kSampThreads / 32;
  __shared__ float red[32];
  __shared__ float s_scan[kSampThreads];
  __shared__ float s_hist[kWarps][256];
  __shared__ float s_bins[256];
  __shared__ unsigned int s_prefix;
  __shared__ float s_above, s_sel;
  const T* x = logits + blockIdx.x * ld;
  const int warp = threadIdx.x >> 5;
  if (step_ptr) step = *step_ptr;       // a device-resident counter: the launch can sit in a CUDA graph
  float m = -INFINITY;
  for_each_elem(x, V, [&](int, float v) { m = fmaxf(m, v * inv_temp); });
  m = block_reduce_max(m, red);
  // top-k: the k-th largest scaled logit by bisection on the ordered integer image of the values (exact; ties at the
  // k-th value all survive, as in the host sampler). kth = -inf keeps everything.
  float kth = -INFINITY;
  if (top_k > 0 && top_k < V) {
    unsigned int lo_k = float_key(-INFINITY), hi_k = float_key(m);   // count(x >= key_float(lo_k)) >= k throughout
    while (lo_k < hi_k) {
      const unsigned int mid = lo_k + ((hi_k - lo_k + 1u) >> 1);
      const float t = key_float(mid);
      float cnt = 0.f;
      for_each_elem(x, V, [&](int, float v) { cnt += (v * inv_temp >= t) ? 1.f : 0.f; });
      cnt = block_reduce_sum(cnt, red);
      if (cnt >= static_cast<float>(top_k)) lo_k = mid; else hi_k = mid - 1u;
    }
    kth = key_float(lo_k);
  }
  float s = 0.f;
  for_each_elem(x, V, [&](int, float v) {
    const float z = v * inv_temp;
    if (z >= kth) s += __expf(z - m);
  });
  const float denom = block_reduce_sum(s, red);
  // nucleus: the smallest set {e >= thr} whose mass reaches top_p * denom
  unsigned int thr_key = 0u;            // bit pattern of the threshold; 0 keeps every element with e > 0
  float total = denom;
  if (top_p < 1.f) {
    const float goal = top_p * denom;
    if (threadIdx.x == 0) {
      s_prefix = 0u;
      s_above = 0.f;
    }
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      for (int i = threadIdx.x; i < kWarps * 256; i += blockDim.x) (&s_hist[0][0])[i] = 0.f;
      __syncthreads();
      const unsigned int prefix = s_prefix;
      for_each_elem(x, V, [&](int, float v) {
        const float z = v * inv_temp;
        if (z >= kth) {
          const float e = __expf(z - m);
          const unsigned int key = __float_as_uint(e);
          const bool undecided = level == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8));
          if (e > 0.f && undecided) atomicAdd(&s_hist[warp][(key >> shift) & 255u], e);
        }
      });
      __syncthreads();
      if (threadIdx.x < 256) {
        float h = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) h += s_hist[w][threadIdx.x];
        s_bins[threadIdx.x] = h;
      }
      __syncthreads();
      if (threadIdx.x == 0) {
        float above = s_above;
        int pick = -1, lowest = -1;
        for (int bin = 255; bin >= 0; --bin) {
          const float h = s_bins[bin];
          if (h > 0.f) lowest = bin;
          if (h > 0.f && above + h >= goal) {
            pick = bin;
            break;
          }
          above += h;
        }
        if (pick < 0) {                 // rounding left the goal just out of reach: everything undecided survives
          pick = lowest < 0 ? 0 : lowest;
          above -= s_bins[pick];
        }
        s_above = above;
        s_sel = s_bins[pick];
        s_prefix = prefix | (static_cast<unsigned int>(pick) << shift);
      }
      __syncthreads();
    }
    thr_key = s_prefix;
    total = s_above + s_sel;            // mass of {e >= thr}: everything above the last bin plus the bin itself
  }
  const float target = uniform_from(seed, blockIdx.x, step) * total;
  // inverse-CDF walk in index order: each thread owns a contiguous span
  const int per = (V + blockDim.x - 1) / blockDim.x;
  const int j0 = threadIdx.x * per, j1 = min(V, j0 + per);
  float mine = 0.f;
  for (int j = j0; j < j1; ++j) {
    const float z = to_f32<T>(x[j]) * inv_temp;
    const float e = z >= kth ? __expf(z - m) : 0.f;
    if (e > 0.f && __float_as_uint(e) >= thr_key) mine += e;
  }
  s_scan[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float acc = 0.f;
    int owner = blockDim.x - 1;
    for (int t = 0; t < static_cast<int>(blockDim.x); ++t) {
      if (acc + s_scan[t] >= target && s_scan[t] > 0.f) {
        owner = t;
        break;
      }
      acc += s_scan[t];
    }
    // walk inside the owner's span
    const int a0 = owner * per, a1 = min(V, a0 + per);
    int pick = -1, last = -1;
    for (int j = a0; j < a1; ++j) {
      const float z = to_f32<T>(x[j]) * inv_temp;
      const float e = z >= kth ? __expf(z - m) : 0.f;
      if (e > 0.f && __float_as_uint(e) >= thr_key) {
        last = j;
        acc += e;
        if (acc >= target) {
          pick = j;
          break;
        }
      }
    }
    if (pick < 0) pick = last >= 0 ? last : 0;
    out[blockIdx.x] = pick;
  }
}

}  // namespace
}  // namespace tsb

#define TSB_DISPATCH_FLOAT(dtype, ...)                      \
  switch (dtype) {                                          \
    case 0: { using T = float; __VA_ARGS__; } break;        \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    case 2: { using T = __half; __VA_ARGS__; } break;       \
    default: return -2;                                     \
  }

// out[row] = argmax_j logits[row, j] (int32), lowest index on ties.
TSB_EXPORT int tsb_argmax_rows(const void* logits, int* out, int rows, int V, long long ld, int dtype, void* stream) {
  if (rows <= 0 || V <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::argmax_rows_kernel<T><<<rows, tsb::kSampThreads, 0, s>>>(
                                static_cast<const T*>(logits), out, V, ld)));
  return static_cast<int>(cudaGetLastError());
}

// Vocabulary-parallel arg-max over a head whose rows are split over `world` ranks, `shard` rows per rank (the last
// rank may hold fewer). Step 1: packed [rows, 4 * world] bf16 receives this rank's candidate per row (see the kernel);
// the caller sums `packed` over the ranks. Step 2: out[row] = global index of the best candidate in the summed rows.
TSB_EXPORT int tsb_argmax_rows_pack(const void* logits, void* packed, int rows, int V, long long ld, int rank, int world,
                                    void* stream) {
  if (rows <= 0 || V <= 0 || V >= (1 << 24) || world < 1 || rank < 0 || rank >= world || !packed) return -2;
  tsb::argmax_rows_kernel<__nv_bfloat16><<<rows, tsb::kSampThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), nullptr, V, ld, static_cast<__nv_bfloat16*>(packed), rank, world);
  return static_cast<int>(cudaGetLastError());
}
TSB_EXPORT int tsb_argmax_rows_unpack(const void* summed, int* out, int rows, int world, int shard, void* stream) {
  if (rows <= 0 || world < 1 || shard <= 0 || !summed || !out) return -2;
  tsb::argmax_unpack_kernel<<<(rows + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(summed), out, rows, world, shard);
  return static_cast<int>(cudaGetLastError());
}

// out[row] ~ softmax(logits[row] / temperature) restricted to its top_p nucleus. The draw for (row, step) is a
// pure function of (seed, row, step).
TSB_EXPORT int tsb_sample_top_p_rows(const void* logits, int* out, int rows, int V, long long ld, float temperature,
                                     float top_p, unsigned long long seed, unsigned long long step, int dtype,
                                     void* stream) {
  if (rows <= 0 || V <= 0 || temperature <= 0.f || top_p <= 0.f) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::sample_top_p_kernel<T><<<rows, tsb::kSampThreads, 0, s>>>(
                                static_cast<const T*>(logits), out, V, ld, 1.f / temperature, top_p, 0, seed, step,
                                nullptr)));
  return static_cast<int>(cudaGetLastError());
}

// The full device sampler, in the host sampler's stage order (src/models/Sampler.cpp:29-116): temperature, top-k
// (0 = off; ties at the k-th value survive), top-p over the renormalised survivors, one uniform draw per row. The
// draw for (row, step) is a pure function of (seed, row, step); with step_ptr != null the step is read from that
// device counter at run time, so the launch can be captured in a CUDA graph and replayed.
TSB_EXPORT int tsb_sample_rows(const void* logits, int* out, int rows, int V, long long ld, float temperature, int top_k,
                               float top_p, unsigned long long seed, unsigned long long step,
                               const unsigned long long* step_ptr, int dtype, void* stream) {
  if (rows <= 0 || V <= 0 || temperature <= 0.f || top_p <= 0.f || top_k < 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::sample_top_p_kernel<T><<<rows, tsb::kSampThreads, 0, s>>>(
                                static_cast<const T*>(logits), out, V, ld, 1.f / temperature, top_p, top_k, seed, step,
                                step_ptr)));
  return static_cast<int>(cudaGetLastError());
}

// logits [rows, V] in place: repetition penalty over history [rows, hist_ld] int32 (hist_len[row] valid entries each).
TSB_EXPORT int tsb_repetition_penalty_rows(void* logits, int rows, int V, long long ld, const int* history,
                                           long long hist_ld, const int* hist_len, float penalty, int dtype,
                                           void* stream) {
  if (rows <= 0 || V <= 0 || penalty <= 0.f || !history || !hist_len) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::repetition_penalty_kernel<T><<<rows, 256, 0, s>>>(
                                static_cast<T*>(logits), ld, V, history, hist_ld, hist_len, penalty)));
  return static_cast<int>(cudaGetLastError());
}
