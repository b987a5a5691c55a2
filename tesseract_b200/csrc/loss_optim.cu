// Cross-entropy (vocab-parallel capable, gradient written in place over the logits) and the
// single-launch Adam update over a table of tensors or one flat arena, plus the sum-of-squares
// reduction used for gradient clipping.
//
// Reference counterparts: fused CE forward/backward, fp32 only, one CTA per row
// (src/cuda/Loss.cu:81-155) and one Adam launch per parameter tensor (src/cuda/Optim.cu:38-122,
// src/optim/Adam.cpp:24-92). Formulae are the reference's: loss = mean(logsumexp(row) - row[target]),
// dlogits = (softmax - onehot) * g / N;  m = b1 m + (1-b1) g, v = b2 v + (1-b2) g^2,
// p -= lr * (m / bc1) / (sqrt(v / bc2) + eps).
#include "common.cuh"

namespace tsb {
namespace {

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32<T>(e[i]);
  } else {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f32<T>(f[i]);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}

constexpr int kCeThreads = 512;

// Per-row statistics of a logits shard [rows, V] holding vocabulary ids [vocab_start, vocab_start + V):
//   stats[row] = {max, sum exp(x - max), logit of the target if it lies in this shard else 0}
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_stats_kernel(const T* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ stats,
                int V, long long ld, int vocab_start) {
  __shared__ float red_m[kCeThreads / 32];
  __shared__ float red_s[kCeThreads / 32];
  const long long row = blockIdx.x;
  const T* x = logits + row * ld;
  float m = -INFINITY, s = 0.f;
  const bool vec = (V % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  if (vec) {
    for (int v = threadIdx.x; v < V / 8; v += blockDim.x) {
      float f[8];
      ld8<T>(x + v * 8, f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > m) {
        s *= __expf(m - lm);
        m = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) s += __expf(f[j] - m);
    }
  } else {
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
      const float f = to_f32<T>(x[j]);
      if (f > m) {
        s *= __expf(m - f);
        m = f;
      }
      s += __expf(f - m);
    }
  }
  // combine (m, s) pairs: warp, then block
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    red_m[warp] = m;
    red_s[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < kCeThreads / 32 ? red_m[lane] : -INFINITY;
    s = lane < kCeThreads / 32 ? red_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const float os = __shfl_xor_sync(0xffffffffu, s, o);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    if (lane == 0) {
      const long long tgt = targets[row] - vocab_start;
      float tl = 0.f;
      if (tgt >= 0 && tgt < V) tl = to_f32<T>(x[tgt]);
      stats[row * 3 + 0] = m;
      stats[row * 3 + 1] = s;
      stats[row * 3 + 2] = tl;
    }
  }
}

// loss_row = log(sum) + max - target_logit (0 for ignored rows, target < 0); optionally overwrites the
// logits with (softmax - onehot) * grad_scale using the (already combined across shards) stats.
template <typename T>
__global__ void __launch_bounds__(kCeThreads)
ce_grad_kernel(T* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ stats,
               float* __restrict__ loss_rows, int V, long long ld, int vocab_start, float grad_scale,
               int write_grad) {
  const long long row = blockIdx.x;
  T* x = logits + row * ld;
  const float m = stats[row * 3 + 0];
  const float s = stats[row * 3 + 1];
  const long long tgt_global = targets[row];
  const bool ignored = tgt_global < 0;
  if (threadIdx.x == 0 && loss_rows) loss_rows[row] = ignored ? 0.f : (__logf(s) + m - stats[row * 3 + 2]);
  if (!write_grad) return;
  const long long tgt = tgt_global - vocab_start;
  const float inv = ignored ? 0.f : grad_scale / s;
  const float gs = ignored ? 0.f : grad_scale;
  const bool vec = (V % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  if (vec) {
    for (int v = threadIdx.x; v < V / 8; v += blockDim.x) {
      float f[8];
      ld8<T>(x + v * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        f[j] = __expf(f[j] - m) * inv;
        if (v * 8 + j == tgt) f[j] -= gs;
      }
      st8<T>(x + v * 8, f);
    }
  } else {
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
      float f = __expf(to_f32<T>(x[j]) - m) * inv;
      if (j == tgt) f -= gs;
      x[j] = from_f32<T>(f);
    }
  }
}

// ------------------------------------------------------------------ Adam
struct AdamHyper {
  float lr, beta1, beta2, eps, bc1, bc2, weight_decay;
};

template <typename P, typename G>
__device__ __forceinline__ void adam_elem(P* p, const G* g, float* m, float* v, float* master, long long i,
                                          const AdamHyper& h, float gscale) {
  const float grad = to_f32<G>(g[i]) * gscale;
  float w = master ? master[i] : to_f32<P>(p[i]);
  const float mi = h.beta1 * m[i] + (1.f - h.beta1) * grad;
  const float vi = h.beta2 * v[i] + (1.f - h.beta2) * grad * grad;
  m[i] = mi;
  v[i] = vi;
  const float mhat = mi / h.bc1;
  const float vhat = vi / h.bc2;
  w -= h.lr * (mhat / (sqrtf(vhat) + h.eps) + h.weight_decay * w);
  if (master) master[i] = w;
  p[i] = from_f32<P>(w);
}

template <typename P, typename G>
__global__ void __launch_bounds__(256)
adam_flat_kernel(P* __restrict__ p, const G* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                 float* __restrict__ master, long long n, AdamHyper h, const float* __restrict__ gscale_ptr) {
  const float gscale = gscale_ptr ? *gscale_ptr : 1.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x);
  // 4 elements per thread per step, contiguous per thread for 64/128-bit accesses by the compiler.
  for (long long base = i * 4; base < n; base += stride * 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (base + j < n) adam_elem<P, G>(p, g, m, v, master, base + j, h, gscale);
    }
  }
}

// Vector path for 16-bit parameters and gradients: 8 elements per thread and step, every operand moved with
// 16-byte accesses that are all issued before the arithmetic starts (six to eight loads in flight per thread).
template <typename P, typename G>
__global__ void __launch_bounds__(256)
adam_flat_vec8_kernel(P* __restrict__ p, const G* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                      float* __restrict__ master, long long nvec, AdamHyper h, const float* __restrict__ gscale_ptr) {
  static_assert(sizeof(P) == 2 && sizeof(G) == 2, "16-bit parameters and gradients");
  const float gscale = gscale_ptr ? *gscale_ptr : 1.f;
  const float inv_bc1 = 1.f / h.bc1, inv_bc2 = 1.f / h.bc2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
    uint4 pw = reinterpret_cast<const uint4*>(p)[i];
    const uint4 gw = reinterpret_cast<const uint4*>(g)[i];
    float4 m0 = reinterpret_cast<const float4*>(m)[2 * i], m1 = reinterpret_cast<const float4*>(m)[2 * i + 1];
    float4 v0 = reinterpret_cast<const float4*>(v)[2 * i], v1 = reinterpret_cast<const float4*>(v)[2 * i + 1];
    float4 w0, w1;
    if (master) {
      w0 = reinterpret_cast<const float4*>(master)[2 * i];
      w1 = reinterpret_cast<const float4*>(master)[2 * i + 1];
    }
    float w[8], gr[8], mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w},
                       vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    const P* pe = reinterpret_cast<const P*>(&pw);
    const G* ge = reinterpret_cast<const G*>(&gw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      gr[j] = to_f32<G>(ge[j]) * gscale;
      w[j] = to_f32<P>(pe[j]);
    }
    if (master) {
      w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w;
      w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
    }
    P po[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mm[j] = h.beta1 * mm[j] + (1.f - h.beta1) * gr[j];
      vv[j] = h.beta2 * vv[j] + (1.f - h.beta2) * gr[j] * gr[j];
      const float mhat = mm[j] * inv_bc1;
      const float vhat = vv[j] * inv_bc2;
      w[j] -= h.lr * (__fdividef(mhat, sqrtf(vhat) + h.eps) + h.weight_decay * w[j]);
      po[j] = from_f32<P>(w[j]);
    }
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    if (master) {
      reinterpret_cast<float4*>(master)[2 * i] = make_float4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<float4*>(master)[2 * i + 1] = make_float4(w[4], w[5], w[6], w[7]);
    }
    reinterpret_cast<uint4*>(p)[i] = *reinterpret_cast<const uint4*>(po);
  }
}

struct AdamTensorRef {
  void* p;
  const void* g;
  float* m;
  float* v;
  float* master;  // may be null
  long long n;
};
constexpr int kAdamChunk = 65536;  // elements per CTA work item

// One launch over a table of tensors. work[i] = {tensor index, chunk index within the tensor}.
template <typename P, typename G>
__global__ void __launch_bounds__(256)
adam_multi_kernel(const AdamTensorRef* __restrict__ table, const int2* __restrict__ work, int num_work, AdamHyper h,
                  const float* __restrict__ gscale_ptr) {
  const float gscale = gscale_ptr ? *gscale_ptr : 1.f;
  for (int wi = blockIdx.x; wi < num_work; wi += gridDim.x) {
    const int2 w = work[wi];
    const AdamTensorRef t = table[w.x];
    const long long begin = static_cast<long long>(w.y) * kAdamChunk;
    const long long end = min(begin + kAdamChunk, t.n);
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x)
      adam_elem<P, G>(static_cast<P*>(t.p), static_cast<const G*>(t.g), t.m, t.v, t.master, i, h, gscale);
  }
}

// out[0] += sum x^2 (fp32 atomics; caller zeroes out[0]).
template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, long long n, float* __restrict__ out) {
  __shared__ float red[8];
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += stride) {
    const float f = to_f32<T>(x[i]);
    acc += f * f;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(out, t);
  }
}

// coef[0] = min(1, max_norm / (sqrt(sumsq[0]) + 1e-6)) * extra_scale
__global__ void clip_coef_kernel(const float* sumsq, float* coef, float max_norm, float extra_scale) {
  const float norm = sqrtf(sumsq[0]);
  float c = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
  coef[0] = c * extra_scale;
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

// stats (fp32 [rows, 3]) = per-row {max, sum exp(x - max), target logit} of a logits shard.
TSB_EXPORT int tsb_ce_stats(const void* logits, const long long* targets, float* stats, long long rows, int V,
                            long long ld, int vocab_start, int dtype, void* stream) {
  if (rows <= 0 || V <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::ce_stats_kernel<T><<<static_cast<unsigned>(rows), tsb::kCeThreads, 0, s>>>(
                                static_cast<const T*>(logits), targets, stats, V, ld, vocab_start)));
  return static_cast<int>(cudaGetLastError());
}

// loss_rows[row] = logsumexp - target logit (from stats); when write_grad != 0 the logits are replaced
// by (softmax - onehot) * grad_scale. Rows whose target is negative are ignored (loss 0, zero gradient).
TSB_EXPORT int tsb_ce_loss_grad(void* logits, const long long* targets, const float* stats, float* loss_rows,
                                long long rows, int V, long long ld, int vocab_start, float grad_scale,
                                int write_grad, int dtype, void* stream) {
  if (rows <= 0 || V <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TSB_DISPATCH_FLOAT(dtype, (tsb::ce_grad_kernel<T><<<static_cast<unsigned>(rows), tsb::kCeThreads, 0, s>>>(
                                static_cast<T*>(logits), targets, stats, loss_rows, V, ld, vocab_start, grad_scale,
                                write_grad)));
  return static_cast<int>(cudaGetLastError());
}

#define TSB_DISPATCH_PG(pd, gd, ...)                                                          \
  if (pd == 0 && gd == 0) { using P = float; using G = float; __VA_ARGS__; }                  \
  else if (pd == 1 && gd == 1) { using P = __nv_bfloat16; using G = __nv_bfloat16; __VA_ARGS__; } \
  else if (pd == 1 && gd == 0) { using P = __nv_bfloat16; using G = float; __VA_ARGS__; }     \
  else if (pd == 2 && gd == 2) { using P = __half; using G = __half; __VA_ARGS__; }           \
  else if (pd == 2 && gd == 0) { using P = __half; using G = float; __VA_ARGS__; }            \
  else return -2;

// Adam over one flat arena: p (param dtype), g (grad dtype), fp32 m / v, optional fp32 master copy.
// gscale (device fp32 scalar, may be NULL) multiplies every gradient (loss-scale removal, clipping).
TSB_EXPORT int tsb_adam_flat(void* p, const void* g, float* m, float* v, float* master, long long n, float lr,
                             float beta1, float beta2, float eps, float bc1, float bc2, float weight_decay,
                             const float* gscale, int p_dtype, int g_dtype, void* stream) {
  if (n <= 0) return 0;
  tsb::AdamHyper h{lr, beta1, beta2, eps, bc1, bc2, weight_decay};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long cap = static_cast<long long>(tsb::sm_count()) * 16;
  auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  long long done = 0;
  if ((p_dtype == 1 || p_dtype == 2) && g_dtype == p_dtype && n >= 8 && aligned16(p) && aligned16(g) && aligned16(m) &&
      aligned16(v) && (!master || aligned16(master))) {
    const long long nvec = n / 8;
    long long blocks = (nvec + 255) / 256;
    if (blocks > cap) blocks = cap;
    if (p_dtype == 1)
      tsb::adam_flat_vec8_kernel<__nv_bfloat16, __nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<__nv_bfloat16*>(p), static_cast<const __nv_bfloat16*>(g), m, v, master, nvec, h, gscale);
    else
      tsb::adam_flat_vec8_kernel<__half, __half><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
          static_cast<__half*>(p), static_cast<const __half*>(g), m, v, master, nvec, h, gscale);
    done = nvec * 8;
    if (done == n) return static_cast<int>(cudaGetLastError());
  }
  // scalar path: other dtype pairs, unaligned arenas, and the tail of the vector path
  const long long rest = n - done;
  const int psz = (p_dtype == 0) ? 4 : 2, gsz = (g_dtype == 0) ? 4 : 2;
  void* p2 = static_cast<char*>(p) + done * psz;
  const void* g2 = static_cast<const char*>(g) + done * gsz;
  float* m2 = m + done;
  float* v2 = v + done;
  float* master2 = master ? master + done : nullptr;
  long long blocks = (rest / 4 + 255) / 256;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  TSB_DISPATCH_PG(p_dtype, g_dtype, (tsb::adam_flat_kernel<P, G><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
                                        static_cast<P*>(p2), static_cast<const G*>(g2), m2, v2, master2, rest, h, gscale)));
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_adam_chunk_elems() { return tsb::kAdamChunk; }

// Adam over a device-resident table of tensors in ONE launch. `table` holds num_tensors records of
// {p, g, m, v, master, n} (6 x 8 bytes each); `work` holds num_work int32 pairs {tensor, chunk}, one per
// tsb_adam_chunk_elems() elements.
TSB_EXPORT int tsb_adam_multi(const void* table, const int* work, int num_work, float lr, float beta1, float beta2,
                              float eps, float bc1, float bc2, float weight_decay, const float* gscale, int p_dtype,
                              int g_dtype, void* stream) {
  if (num_work <= 0) return 0;
  tsb::AdamHyper h{lr, beta1, beta2, eps, bc1, bc2, weight_decay};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int blocks = num_work;
  const int cap = tsb::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  TSB_DISPATCH_PG(p_dtype, g_dtype, (tsb::adam_multi_kernel<P, G><<<blocks, 256, 0, s>>>(
                                        static_cast<const tsb::AdamTensorRef*>(table),
                                        reinterpret_cast<const int2*>(work), num_work, h, gscale)));
  return static_cast<int>(cudaGetLastError());
}

// out[0] += sum of squares of x (caller zeroes out first; several calls accumulate a global norm).
TSB_EXPORT int tsb_sumsq(const void* x, long long n, float* out, int dtype, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  long long blocks = (n + 255) / 256 / 8 + 1;
  const long long cap = static_cast<long long>(tsb::sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  TSB_DISPATCH_FLOAT(dtype, (tsb::sumsq_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
                                static_cast<const T*>(x), n, out)));
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_clip_coef(const float* sumsq, float* coef, float max_norm, float extra_scale, void* stream) {
  tsb::clip_coef_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, coef, max_norm, extra_scale);
  return static_cast<int>(cudaGetLastError());
}
