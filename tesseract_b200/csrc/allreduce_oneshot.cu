// One-shot all-reduce for latency-bound messages (tensor-parallel decode: [batch, hidden] bf16 after o_proj and
// down_proj), over peer-mapped memory. Every rank leaves its partial in its own symmetric buffer; the kernel tells the
// peers "my partial is complete" (system-scope release of an epoch number into their flag arrays), waits (bounded)
// until every peer has said the same, then every rank reads all partials -- the remote ones straight over NVLink with
// 16-byte loads -- and sums them in rank order, so all ranks produce bit-identical results. The epoch lives in
// device memory and is advanced by the last CTA of each launch, so the kernel can be captured in a CUDA graph and
// replayed. Two input buffers used alternately make the scheme safe without a second barrier: a rank can only
// start call n + 1 after it finished reading in call n, and no rank overwrites the buffer of call n before every
// peer has started call n + 1.
// Replaces ncclAllReduce on the decode path of the reference's tensor-parallel layers
// (src/distributed/NcclCommBackend.cpp:134-164).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kMaxWorld = 8;

struct ArArgs {
  const __nv_bfloat16* peer_in[kMaxWorld];  // the input buffer of every rank for this call (peer mappings)
  int* peer_flags[kMaxWorld];               // flag array [world] of every rank
  int* state;                               // local: [0] epoch of the last finished call, [1] finished CTAs
};

__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(ArArgs a, __nv_bfloat16* __restrict__ out, long long nvec, int rank, int world, int* status) {
  pdl_trigger();
  __shared__ int s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const int e = *reinterpret_cast<volatile int*>(a.state) + 1;
    s_epoch = e;
    int ok = 1;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[r] + rank), "r"(e) : "memory");
    }
    const long long t0 = clock64();
    for (int r = 0; r < world && ok; ++r) {
      const int* f = a.peer_flags[rank] + r;
      while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v >= e) break;
        if (clock64() - t0 > kWaitCycleLimit) {
          if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
          ok = 0;
          break;
        }
        __nanosleep(40);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec; i += stride) {
      uint4 raw[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < world) raw[r] = reinterpret_cast<const uint4*>(a.peer_in[r])[i];   // all loads in flight together
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r) {
        if (r < world) {
          const __nv_bfloat162* e2 = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(e2[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out)[i] = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.state + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {  // the last CTA of this launch publishes the new epoch
      a.state[1] = 0;
      __threadfence();
      atomicExch(a.state, s_epoch);
    }
  }
}

// The same all-reduce fused with what follows it in a transformer block: h = bf16(sum over ranks + residual) is the
// new residual stream, y = rmsnorm(h) * weight the input of the next projection. One CTA per row, so the row
// statistics never leave the CTA; saves the separate norm launch and a round trip of the row through HBM.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;   // 16-byte vectors per thread: rows of up to 256 * 4 * 8 = 8192 elements

__global__ void __launch_bounds__(kNormThreads)
allreduce_norm_oneshot_kernel(ArArgs a, const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ weight,
                              __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h, int cols, float eps, int rank,
                              int world, int* status) {
  pdl_trigger();
  __shared__ int s_epoch;
  __shared__ int s_ok;
  __shared__ float s_red[kNormThreads / 32];
  if (threadIdx.x == 0) {
    const int e = *reinterpret_cast<volatile int*>(a.state) + 1;
    s_epoch = e;
    int ok = 1;
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[r] + rank), "r"(e) : "memory");
    }
    const long long t0 = clock64();
    for (int r = 0; r < world && ok; ++r) {
      const int* f = a.peer_flags[rank] + r;
      while (true) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v >= e) break;
        if (clock64() - t0 > kWaitCycleLimit) {
          if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
          ok = 0;
          break;
        }
        __nanosleep(40);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    const int nvec = cols / 8;
    const long long row_off = static_cast<long long>(blockIdx.x) * nvec;
    float vals[kNormMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < kNormMaxVec; ++u) {
      const int v = threadIdx.x + u * kNormThreads;
      if (v < nvec) {
        uint4 raw[kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
          if (r < world) raw[r] = reinterpret_cast<const uint4*>(a.peer_in[r])[row_off + v];
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r) {
          if (r < world) {
            const __nv_bfloat162* e2 = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 f = __bfloat1622float2(e2[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
        }
        if (residual) {
          const uint4 rr = reinterpret_cast<const uint4*>(residual)[row_off + v];
          const __nv_bfloat162* e2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(e2[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        // the residual stream is carried in bf16: normalise what is stored
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(h)[row_off + v] = o;
        const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(o2[j]);
          vals[u][2 * j] = f.x;
          vals[u][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < kNormThreads / 32; ++w) tot += s_red[w];
    const float rstd = rsqrtf(tot / static_cast<float>(cols) + eps);
#pragma unroll
    for (int u = 0; u < kNormMaxVec; ++u) {
      const int v = threadIdx.x + u * kNormThreads;
      if (v < nvec) {
        const uint4 wr = reinterpret_cast<const uint4*>(weight)[v];
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wf = __bfloat1622float2(w2[j]);
          op[j] = pack_bf16x2(vals[u][2 * j] * rstd * wf.x, vals[u][2 * j + 1] * rstd * wf.y);
        }
        reinterpret_cast<uint4*>(y)[row_off + v] = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int done = atomicAdd(a.state + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      a.state[1] = 0;
      __threadfence();
      atomicExch(a.state, s_epoch);
    }
  }
}

}  // namespace
}  // namespace tsb

// h [rows, cols] = bf16(sum over ranks of peer_in[r] + residual), y = rmsnorm(h) * weight (all bf16, local outputs).
// Same buffers, flags, state and calling discipline as tsb_allreduce_oneshot; residual may be null; cols % 8 == 0,
// cols <= 8192.
TSB_EXPORT int tsb_allreduce_norm_oneshot(void* const* peer_in, void* const* peer_flags, int* state, const void* residual,
                                          const void* weight, void* y, void* h, int rows, int cols, float eps, int rank,
                                          int world, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || rows <= 0 || cols <= 0 || cols % 8 || !state) return -2;
  if (cols > kNormThreads * kNormMaxVec * 8 || !weight || !y || !h) return -2;
  if ((reinterpret_cast<uintptr_t>(y) & 15) || (reinterpret_cast<uintptr_t>(h) & 15) ||
      (reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15))
    return -2;
  ArArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!peer_in[r] || !peer_flags[r] || (reinterpret_cast<uintptr_t>(peer_in[r]) & 15)) return -2;
    a.peer_in[r] = static_cast<const __nv_bfloat16*>(peer_in[r]);
    a.peer_flags[r] = static_cast<int*>(peer_flags[r]);
  }
  a.state = state;
  allreduce_norm_oneshot_kernel<<<rows, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      a, static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(weight),
      static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(h), cols, eps, rank, world, device_status_word());
  return static_cast<int>(cudaGetLastError());
}

// out [n] bf16 (local) = sum over ranks of peer_in[r][0 .. n) (bf16, fp32 accumulation, rank order).
//   peer_in[r]: rank r's input buffer for this call as mapped in this process (peer_in[rank] is local);
//   peer_flags[r]: rank r's int32 [world] flag array (zero at allocation); state: local int32 [2], zero at allocation.
//   n % 8 == 0. Every rank calls this the same number of times; inputs alternate between two buffers.
TSB_EXPORT int tsb_allreduce_oneshot(void* const* peer_in, void* const* peer_flags, int* state, void* out, long long n,
                                     int rank, int world, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0 || n % 8 || !state) return -2;
  if (reinterpret_cast<uintptr_t>(out) & 15) return -2;
  ArArgs a{};
  for (int r = 0; r < world; ++r) {
    if (!peer_in[r] || !peer_flags[r] || (reinterpret_cast<uintptr_t>(peer_in[r]) & 15)) return -2;
    a.peer_in[r] = static_cast<const __nv_bfloat16*>(peer_in[r]);
    a.peer_flags[r] = static_cast<int*>(peer_flags[r]);
  }
  a.state = state;
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  const long long cap = sm_count();
  if (blocks > cap) blocks = cap;
  allreduce_oneshot_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, static_cast<__nv_bfloat16*>(out), nvec, rank, world, device_status_word());
  return static_cast<int>(cudaGetLastError());
}
