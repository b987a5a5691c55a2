// Bandwidth-bound fused kernels of the transformer block: RMSNorm (+ residual add) forward / backward,
// SwiGLU forward / backward, adjacent-pair RoPE on a packed QKV buffer (forward / backward), embedding
// gather / scatter-add. All math in fp32; I/O in bf16, fp16 or fp32; 128-bit accesses.
//
// Counterparts in the reference (forward only, fp32/fp64, one CTA per row or one thread per element):
// src/cuda/RMSNorm.cu:89-128, src/cuda/SwiGLU.cu:80-110, src/cuda/RotaryEmbedding.cu:74-138. The backward
// kernels have no counterpart there (the reference trains through primitive composites).
#include <cstdlib>
#include "common.cuh"

namespace tsb {
namespace {

template <typename T>
struct Vec8 {  // 8 elements of T moved as one or two 128-bit words
  T v[8];
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) {
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
__device__ __forceinline__ void store8(T* p, const float (&f)[8]) {
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

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ RMSNorm forward
// One CTA per row (grid-stride over rows). MAXV = ceil(D / (8 * threads)) register-resident vectors.
// If `res` != nullptr: h = x + res is written to `h_out` and normalised; else x is normalised.
template <typename T, int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w, T* __restrict__ y,
                   T* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int D, float eps) {
  pdl_trigger();
  __shared__ float red[32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * D;
    float f[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        load8<T>(xr + v * 8, f[i]);
        if (res) {
          float g[8];
          load8<T>(res + static_cast<size_t>(row) * D + v * 8, g);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[i][j] += g[j];
          // The residual stream is carried in the storage dtype: normalise what is stored.
#pragma unroll
          for (int j = 0; j < 8; ++j) f[i][j] = to_f32<T>(from_f32<T>(f[i][j]));
          store8<T>(h_out + static_cast<size_t>(row) * D + v * 8, f[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[i][j] * f[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(D) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float g[8], o[8];
        load8<T>(w + v * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[i][j] * rstd * g[j];
        store8<T>(y + static_cast<size_t>(row) * D + v * 8, o);
      }
    }
  }
}

// Same computation with the NEXT row's loads issued before the current row is reduced and stored, so that every
// thread keeps 16-byte loads in flight across the block reduction (the packed words wait in registers).
template <typename T>
struct Raw8 {
  uint4 a;
  uint4 b;   // second half of 8 fp32 values; unused for 2-byte types
};
template <typename T>
__device__ __forceinline__ Raw8<T> ldraw8(const T* p) {
  Raw8<T> r;
  r.a = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 4) r.b = *reinterpret_cast<const uint4*>(p + 4);
  return r;
}
template <typename T>
__device__ __forceinline__ void unpack8(const Raw8<T>& r, float (&f)[8]) {
  if constexpr (sizeof(T) == 2) {
    const T* e = reinterpret_cast<const T*>(&r.a);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = to_f32<T>(e[i]);
  } else {
    f[0] = __uint_as_float(r.a.x); f[1] = __uint_as_float(r.a.y); f[2] = __uint_as_float(r.a.z); f[3] = __uint_as_float(r.a.w);
    f[4] = __uint_as_float(r.b.x); f[5] = __uint_as_float(r.b.y); f[6] = __uint_as_float(r.b.z); f[7] = __uint_as_float(r.b.w);
  }
}

template <typename T, int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_pf_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w, T* __restrict__ y,
                      T* __restrict__ h_out, float* __restrict__ rstd_out, int rows, int D, float eps) {
  pdl_trigger();
  __shared__ float red[32];
  const int nvec = D / 8;
  Raw8<T> nx[MAXV], nr[MAXV];
  auto fetch = [&](int row) {
    const size_t off = static_cast<size_t>(row) * D;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        nx[i] = ldraw8<T>(x + off + v * 8);
        if (res) nr[i] = ldraw8<T>(res + off + v * 8);
      }
    }
  };
  int row = blockIdx.x;
  if (row < rows) fetch(row);
  for (; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    float f[MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        unpack8<T>(nx[i], f[i]);
        if (res) {
          float g[8];
          unpack8<T>(nr[i], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[i][j] = to_f32<T>(from_f32<T>(f[i][j] + g[j]));   // normalise what is stored
          store8<T>(h_out + off + v * 8, f[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += f[i][j] * f[i][j];
      }
    }
    const int next = row + gridDim.x;
    if (next < rows) fetch(next);
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(D) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float g[8], o[8];
        load8<T>(w + v * 8, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = f[i][j] * rstd * g[j];
        store8<T>(y + off + v * 8, o);
      }
    }
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres);  dw partial sums per CTA into `dw_partial[grid, D]`.
template <typename T, int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                   const float* __restrict__ rstd_in, const T* __restrict__ dres, T* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int D) {
  __shared__ float red[32];
  const int nvec = D / 8;
  float dwacc[MAXV][8];
  float wv[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (v < nvec) load8<T>(w + v * 8, wv[i]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    const float rstd = rstd_in[row];
    float xh[MAXV][8], g[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        load8<T>(x + off + v * 8, xh[i]);
        load8<T>(dy + off + v * 8, g[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          dwacc[i][j] += g[i][j] * xh[i][j];
          g[i][j] *= wv[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    const float mean_dot = block_sum(dot, red) / static_cast<float>(D);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * mean_dot);
        if (dres) {
          float r[8];
          load8<T>(dres + off + v * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8<T>(dx + off + v * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float* dst = dw_partial + static_cast<size_t>(blockIdx.x) * D + v * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
    }
  }
}

// dw[d] (+)= sum_p partial[p, d]
template <typename T>
__global__ void colsum_partials_kernel(const float* __restrict__ partial, T* __restrict__ dw, int parts, int D,
                                       int accumulate) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[static_cast<size_t>(p) * D + d];
  if (accumulate) s += to_f32<T>(dw[d]);
  dw[d] = from_f32<T>(s);
}

// ------------------------------------------------------------------ SwiGLU
// gate_up is [rows, 2F] with gate in columns [0, F) and up in [F, 2F); out is [rows, F].
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const T* __restrict__ gate_up, T* __restrict__ out, long long rows, int F) {
  pdl_trigger();
  const long long nvec = rows * (F / 8);
  const int vpr = F / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / vpr;
    const int c = static_cast<int>(i - row * vpr) * 8;
    float g[8], u[8], o[8];
    load8<T>(gate_up + row * 2 * F + c, g);
    load8<T>(gate_up + row * 2 * F + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    store8<T>(out + row * F + c, o);
  }
}
// Row-wise form: no 64-bit division per vector, and UNR independent vector pairs in flight per thread.
template <typename T, int UNR>
__global__ void __launch_bounds__(256)
swiglu_fwd_rows_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int F) {
  pdl_trigger();
  const int vpr = F / 8;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const T* gp = gate_up + static_cast<size_t>(row) * 2 * F;
    T* op = out + static_cast<size_t>(row) * F;
    for (int v0 = (blockIdx.x * blockDim.x + threadIdx.x) * UNR; v0 < vpr; v0 += gridDim.x * blockDim.x * UNR) {
      float g[UNR][8], u[UNR][8];
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (v0 + k < vpr) {
          load8<T>(gp + (v0 + k) * 8, g[k]);
          load8<T>(gp + F + (v0 + k) * 8, u[k]);
        }
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (v0 + k < vpr) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = __fdividef(g[k][j], 1.f + __expf(-g[k][j])) * u[k][j];
          store8<T>(op + (v0 + k) * 8, o);
        }
    }
  }
}

// d(gate_up) from d(out): dg = dout*u*s*(1+g*(1-s)), du = dout*g*s with s = sigmoid(g).
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ gate_up, T* __restrict__ dgate_up, long long rows,
                  int F) {
  const long long nvec = rows * (F / 8);
  const int vpr = F / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / vpr;
    const int c = static_cast<int>(i - row * vpr) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8<T>(gate_up + row * 2 * F + c, g);
    load8<T>(gate_up + row * 2 * F + F + c, u);
    load8<T>(dout + row * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * s * (1.f + g[j] * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    store8<T>(dgate_up + row * 2 * F + c, dg);
    store8<T>(dgate_up + row * 2 * F + F + c, du);
  }
}

template <typename T, int UNR>
__global__ void __launch_bounds__(256)
swiglu_bwd_rows_kernel(const T* __restrict__ dout, const T* __restrict__ gate_up, T* __restrict__ dgate_up, int rows, int F) {
  const int vpr = F / 8;
  for (int row = blockIdx.y; row < rows; row += gridDim.y) {
    const T* gp = gate_up + static_cast<size_t>(row) * 2 * F;
    const T* dp = dout + static_cast<size_t>(row) * F;
    T* op = dgate_up + static_cast<size_t>(row) * 2 * F;
    for (int v0 = (blockIdx.x * blockDim.x + threadIdx.x) * UNR; v0 < vpr; v0 += gridDim.x * blockDim.x * UNR) {
      float g[UNR][8], u[UNR][8], d[UNR][8];
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (v0 + k < vpr) {
          load8<T>(gp + (v0 + k) * 8, g[k]);
          load8<T>(gp + F + (v0 + k) * 8, u[k]);
          load8<T>(dp + (v0 + k) * 8, d[k]);
        }
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (v0 + k < vpr) {
          float dg[8], du[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float sg = __fdividef(1.f, 1.f + __expf(-g[k][j]));
            dg[j] = d[k][j] * u[k][j] * sg * (1.f + g[k][j] * (1.f - sg));
            du[j] = d[k][j] * g[k][j] * sg;
          }
          store8<T>(op + (v0 + k) * 8, dg);
          store8<T>(op + F + (v0 + k) * 8, du);
        }
    }
  }
}

// ------------------------------------------------------------------ RoPE on packed QKV
// qkv is [T, (Hq + 2*Hkv) * D]; heads [0, Hq + Hkv) (queries then keys) are rotated in place using the
// cos/sin table row `pos[t]` (or pos_offset + t % seq_len when pos == nullptr). Adjacent pairs
// (x[2j], x[2j+1]); tables are [max_pos, D/2] fp32. `sign` = +1 forward, -1 backward (inverse rotation).
template <typename T>
__global__ void __launch_bounds__(256)
rope_qkv_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                const int* __restrict__ pos, long long tokens, int seq_len, int pos_offset, int heads_rot,
                int heads_total, int D, float sign) {
  const int vph = D / 8;  // vectors per head
  const long long nvec = tokens * heads_rot * vph;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(i % vph);
    const long long th = i / vph;
    const int h = static_cast<int>(th % heads_rot);
    const long long t = th / heads_rot;
    const int p = pos ? pos[t] : pos_offset + static_cast<int>(t % seq_len);
    T* ptr = qkv + (t * heads_total + h) * D + v * 8;
    float x[8], o[8];
    load8<T>(ptr, x);
    const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(p) * (D / 2) + v * 4);
    float4 s = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(p) * (D / 2) + v * 4);
    s.x *= sign; s.y *= sign; s.z *= sign; s.w *= sign;
    o[0] = x[0] * c.x - x[1] * s.x; o[1] = x[0] * s.x + x[1] * c.x;
    o[2] = x[2] * c.y - x[3] * s.y; o[3] = x[2] * s.y + x[3] * c.y;
    o[4] = x[4] * c.z - x[5] * s.z; o[5] = x[4] * s.z + x[5] * c.z;
    o[6] = x[6] * c.w - x[7] * s.w; o[7] = x[6] * s.w + x[7] * c.w;
    store8<T>(ptr, o);
  }
}

// ------------------------------------------------------------------ embedding
template <typename T>
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const long long* __restrict__ ids, const T* __restrict__ table, T* __restrict__ out,
                     long long tokens, int D, int vocab, int* status) {
  const int vpr = D / 8;
  const long long nvec = tokens * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vpr;
    const int c = static_cast<int>(i - t * vpr) * 8;
    long long id = ids[t];
    if (id < 0 || id >= vocab) {        // never read outside the table: row 0 instead, and the host hears of it
      if (c == 0 && status) atomicCAS(status, kStatusOk, kStatusBadIndex);
      id = 0;
    }
    float f[8];
    load8<T>(table + id * D + c, f);
    store8<T>(out + t * D + c, f);
  }
}
// dtable[ids[t]] += dy[t] with atomics; dtable is fp32 (G = float) or bf16 (G = __nv_bfloat16, paired atomics).
template <typename T, typename G>
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(const long long* __restrict__ ids, const T* __restrict__ dy, G* __restrict__ dtable,
                     long long tokens, int D, int vocab, int* status) {
  const int vpr = D / 8;
  const long long nvec = tokens * vpr;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vpr;
    const int c = static_cast<int>(i - t * vpr) * 8;
    const long long id = ids[t];
    if (id < 0 || id >= vocab) {
      if (status) atomicCAS(status, kStatusOk, kStatusBadIndex);
      continue;
    }
    float f[8];
    load8<T>(dy + t * D + c, f);
    G* dst = dtable + id * D + c;
    if constexpr (sizeof(G) == 4) {
#pragma unroll
      for (int j = 0; j < 8; ++j) atomicAdd(reinterpret_cast<float*>(dst) + j, f[j]);
    } else {
      __nv_bfloat162* d2 = reinterpret_cast<__nv_bfloat162*>(dst);
#pragma unroll
      for (int j = 0; j < 4; ++j) atomicAdd(d2 + j, __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]));
    }
  }
}

inline int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

template <typename T>
int rmsnorm_fwd_t(const void* x, const void* res, const void* w, void* y, void* h, float* rstd, int rows, int D,
                  float eps, cudaStream_t s) {
  // Rows up to 8192 wide take the prefetching kernel (0.96 of the copy bandwidth at 65536 x 4096 bf16, against 0.65
  // for the plain one); TESSERACT_RMS_PREFETCH=0 / TESSERACT_RMS_THREADS=128 are kept for A/B measurements.
  static const int forced = [] { const char* e = getenv("TESSERACT_RMS_THREADS"); return e ? atoi(e) : 0; }();
  static const int prefetch = [] { const char* e = getenv("TESSERACT_RMS_PREFETCH"); return e ? atoi(e) : 1; }();
  int threads = 256;
  if (forced == 128 || forced == 256) threads = forced;
  const int maxv = (D / 8 + threads - 1) / threads;
  const int per_sm = 2048 / threads;
  const int grid = rows < sm_count() * per_sm ? rows : sm_count() * per_sm;
#define TSB_RMS_PF(MV)                                                                                             \
  rmsnorm_fwd_pf_kernel<T, MV><<<grid, threads, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(res),       \
                                                        static_cast<const T*>(w), static_cast<T*>(y),               \
                                                        static_cast<T*>(h), rstd, rows, D, eps)
  if (prefetch && maxv <= 4) {
    if (maxv <= 1) TSB_RMS_PF(1);
    else if (maxv <= 2) TSB_RMS_PF(2);
    else TSB_RMS_PF(4);
    return static_cast<int>(cudaGetLastError());
  }
#undef TSB_RMS_PF
#define TSB_RMS_FWD(MV)                                                                                            \
  rmsnorm_fwd_kernel<T, MV><<<grid, threads, 0, s>>>(static_cast<const T*>(x), static_cast<const T*>(res),          \
                                                     static_cast<const T*>(w), static_cast<T*>(y),                  \
                                                     static_cast<T*>(h), rstd, rows, D, eps)
  if (maxv <= 1) TSB_RMS_FWD(1);
  else if (maxv <= 2) TSB_RMS_FWD(2);
  else if (maxv <= 4) TSB_RMS_FWD(4);
  else if (maxv <= 8) TSB_RMS_FWD(8);
  else return -2;
#undef TSB_RMS_FWD
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int rmsnorm_bwd_t(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                  void* dw, float* partial, int parts, int rows, int D, int accumulate, cudaStream_t s) {
  const int threads = 256;
  const int maxv = (D / 8 + threads - 1) / threads;
  const int grid = parts;
#define TSB_RMS_BWD(MV)                                                                                            \
  rmsnorm_bwd_kernel<T, MV><<<grid, threads, 0, s>>>(static_cast<const T*>(dy), static_cast<const T*>(x),          \
                                                     static_cast<const T*>(w), rstd, static_cast<const T*>(dres),   \
                                                     static_cast<T*>(dx), partial, rows, D)
  if (maxv <= 1) TSB_RMS_BWD(1);
  else if (maxv <= 2) TSB_RMS_BWD(2);
  else if (maxv <= 4) TSB_RMS_BWD(4);
  else return -2;
#undef TSB_RMS_BWD
  colsum_partials_kernel<T><<<(D + 255) / 256, 256, 0, s>>>(partial, static_cast<T*>(dw), parts, D, accumulate);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace
}  // namespace tsb

// dtype codes shared by every entry point: 0 = fp32, 1 = bf16, 2 = fp16.
#define TSB_DISPATCH_FLOAT(dtype, ...)                      \
  switch (dtype) {                                          \
    case 0: { using T = float; __VA_ARGS__; } break;        \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; } break; \
    case 2: { using T = __half; __VA_ARGS__; } break;       \
    default: return -2;                                     \
  }

// y = rmsnorm(x [+ res]) * w over rows of length D (D % 8 == 0, D <= 16384). If res != NULL the sum
// x + res is also written to h_out. rstd (fp32 [rows]) may be NULL.
TSB_EXPORT int tsb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                               int rows, int D, float eps, int dtype, void* stream) {
  if (rows <= 0 || D <= 0 || D % 8) return -2;
  int rc = -2;
  TSB_DISPATCH_FLOAT(dtype, rc = tsb::rmsnorm_fwd_t<T>(x, res, w, y, h_out, rstd, rows, D, eps,
                                                       static_cast<cudaStream_t>(stream)));
  return rc;
}

// Number of per-CTA partial rows tsb_rmsnorm_bwd needs in its fp32 scratch buffer [parts, D].
TSB_EXPORT int tsb_rmsnorm_bwd_parts(int rows) {
  const int cap = tsb::sm_count() * 2;
  return rows < cap ? rows : cap;
}

// Backward of y = rmsnorm(x) * w. dx = d(x) (+ dres when dres != NULL); dw (+)= column sums of dy * xhat.
// `partial` is caller-provided fp32 scratch of tsb_rmsnorm_bwd_parts(rows) * D elements.
TSB_EXPORT int tsb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, void* dw, float* partial, int rows, int D, int accumulate_dw, int dtype,
                               void* stream) {
  if (rows <= 0 || D <= 0 || D % 8 || D > 8192) return -2;
  const int parts = tsb_rmsnorm_bwd_parts(rows);
  int rc = -2;
  TSB_DISPATCH_FLOAT(dtype, rc = tsb::rmsnorm_bwd_t<T>(dy, x, w, rstd, dres, dx, dw, partial, parts, rows, D,
                                                       accumulate_dw, static_cast<cudaStream_t>(stream)));
  return rc;
}

TSB_EXPORT int tsb_swiglu_fwd(const void* gate_up, void* out, long long rows, int F, int dtype, void* stream) {
  if (rows <= 0 || F <= 0 || F % 8) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Row-wise kernel by default (0.93 of the copy bandwidth at 65536 x 4096 bf16, against 0.67 for the flat one);
  // TESSERACT_SWIGLU=0 keeps the flat kernel for A/B measurements.
  static const int mode = [] { const char* e = getenv("TESSERACT_SWIGLU"); return e ? atoi(e) : 2; }();
  if (mode == 0 || rows > 0x7fffffffLL) {
    const int grid = tsb::ew_grid(rows * (F / 8), 256);
    TSB_DISPATCH_FLOAT(dtype, (tsb::swiglu_fwd_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(gate_up),
                                                                             static_cast<T*>(out), rows, F)));
    return static_cast<int>(cudaGetLastError());
  }
  // grid.x covers one row's vectors (UNR per thread), grid.y strides the rows: about 8 CTAs per SM in total
  const int unr = 2;
  const int vpr = F / 8;
  int gx = (vpr + 256 * unr - 1) / (256 * unr);
  long long gy = (static_cast<long long>(tsb::sm_count()) * 8 + gx - 1) / gx;
  if (gy > rows) gy = rows;
  if (gy > 65535) gy = 65535;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  TSB_DISPATCH_FLOAT(dtype, (tsb::swiglu_fwd_rows_kernel<T, 2><<<grid, 256, 0, s>>>(
                                static_cast<const T*>(gate_up), static_cast<T*>(out), static_cast<int>(rows), F)));
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long rows, int F, int dtype,
                              void* stream) {
  if (rows <= 0 || F <= 0 || F % 8) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  static const int mode = [] { const char* e = getenv("TESSERACT_SWIGLU"); return e ? atoi(e) : 2; }();
  if (mode == 0 || rows > 0x7fffffffLL) {
    const int grid = tsb::ew_grid(rows * (F / 8), 256);
    TSB_DISPATCH_FLOAT(dtype, (tsb::swiglu_bwd_kernel<T><<<grid, 256, 0, s>>>(
                                  static_cast<const T*>(dout), static_cast<const T*>(gate_up),
                                  static_cast<T*>(dgate_up), rows, F)));
    return static_cast<int>(cudaGetLastError());
  }
  const int vpr = F / 8;
  int gx = (vpr + 256 * 2 - 1) / (256 * 2);
  long long gy = (static_cast<long long>(tsb::sm_count()) * 8 + gx - 1) / gx;
  if (gy > rows) gy = rows;
  if (gy > 65535) gy = 65535;
  const dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy));
  TSB_DISPATCH_FLOAT(dtype, (tsb::swiglu_bwd_rows_kernel<T, 2><<<grid, 256, 0, s>>>(
                                static_cast<const T*>(dout), static_cast<const T*>(gate_up),
                                static_cast<T*>(dgate_up), static_cast<int>(rows), F)));
  return static_cast<int>(cudaGetLastError());
}

// In-place adjacent-pair RoPE on the first `heads_rot` heads of every token of a packed [tokens,
// heads_total * D] buffer. pos (int32 [tokens]) may be NULL: position = pos_offset + t % seq_len.
// sign = +1 forward, -1 for the backward pass.
TSB_EXPORT int tsb_rope_qkv(void* qkv, const float* cos_t, const float* sin_t, const int* pos, long long tokens,
                            int seq_len, int pos_offset, int heads_rot, int heads_total, int D, float sign,
                            int dtype, void* stream) {
  if (tokens <= 0 || D % 8 || heads_rot > heads_total || seq_len <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = tsb::ew_grid(tokens * heads_rot * (D / 8), 256);
  TSB_DISPATCH_FLOAT(dtype, (tsb::rope_qkv_kernel<T><<<grid, 256, 0, s>>>(static_cast<T*>(qkv), cos_t, sin_t, pos,
                                                                         tokens, seq_len, pos_offset, heads_rot,
                                                                         heads_total, D, sign)));
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_embedding_fwd(const long long* ids, const void* table, void* out, long long tokens, int D,
                                 int vocab, int dtype, void* stream) {
  if (tokens <= 0 || D % 8) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = tsb::ew_grid(tokens * (D / 8), 256);
  TSB_DISPATCH_FLOAT(dtype, (tsb::embedding_fwd_kernel<T><<<grid, 256, 0, s>>>(ids, static_cast<const T*>(table),
                                                                              static_cast<T*>(out), tokens, D,
                                                                              vocab, tsb::device_status_word())));
  return static_cast<int>(cudaGetLastError());
}

// dtable ([vocab, D]; fp32 when grad_f32 != 0, else bf16) += scatter of dy rows by token id.
TSB_EXPORT int tsb_embedding_bwd(const long long* ids, const void* dy, void* dtable, long long tokens, int D,
                                 int vocab, int dtype, int grad_f32, void* stream) {
  if (tokens <= 0 || D % 8) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = tsb::ew_grid(tokens * (D / 8), 256);
  if (grad_f32) {
    TSB_DISPATCH_FLOAT(dtype, (tsb::embedding_bwd_kernel<T, float><<<grid, 256, 0, s>>>(
                                  ids, static_cast<const T*>(dy), static_cast<float*>(dtable), tokens, D, vocab,
                                  tsb::device_status_word())));
  } else {
    TSB_DISPATCH_FLOAT(dtype, (tsb::embedding_bwd_kernel<T, __nv_bfloat16><<<grid, 256, 0, s>>>(
                                  ids, static_cast<const T*>(dy), static_cast<__nv_bfloat16*>(dtable), tokens, D,
                                  vocab, tsb::device_status_word())));
  }
  return static_cast<int>(cudaGetLastError());
}
