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

}  // namespace
}  // namespace tsb

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
