// Two-shot all-reduce of a large bf16 / fp32 buffer that lives in peer-mapped ("symmetric") memory, in place:
// the data-parallel gradient all-reduce. One kernel per rank and bucket, launched on a side stream while the
// backward pass of the earlier layers is still running:
//
//   1. start barrier  every rank tells its peers "my copy of this bucket is final" (system-scope release of the call's
//                     epoch into their flag pads) and waits, bounded, until every peer has said the same;
//   2. reduce-scatter rank r owns the r-th slice of the bucket: it loads that slice from every rank (its own copy from
//                     local memory, the others over NVLink with 16-byte peer loads, all `world` loads of a vector in
//                     flight together), sums them in fp32 in rank order and applies the averaging factor;
//   3. all-gather     and stores the reduced vector straight back into the same place of EVERY rank's buffer (peer
//                     stores). A vector is read and rewritten by the same thread of one rank only, so no second
//                     buffer and no barrier between 2 and 3 is needed, and all ranks end up with identical bits;
//   4. end barrier    the last CTA of the launch (grid-wide counter) publishes "my slice is written everywhere" and
//                     waits, bounded, for the same from every peer, so when the kernel has finished on a rank, that
//                     rank's whole bucket is reduced.
//
// Bytes over NVLink per rank: (world-1)/world of the bucket in (loads) and the same out (stores) -- what a ring
// all-reduce moves, without its 2 (world-1) serial steps. The kernel runs on few CTAs on purpose (it shares the SMs
// with the backward GEMMs; each spinning CTA costs an SM some issue slots) and never touches NCCL.
// Every wait is bounded: when one runs out, kStatusFlagTimeout goes to the status word and the kernel returns.
//
// The reference has no data parallelism (a comment only, src/ops/cpu/Arithmetic.cpp:270); its one collective call is
// ncclAllReduce followed by a stream synchronise (src/distributed/NcclCommBackend.cpp:134-138).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kDoneOffset = 16;   // flag pad of a rank: [0, world) start epochs, [16, 16 + world) done epochs

struct Ar2Args {
  void* peer[kMaxWorld];        // the bucket in every rank's buffer (peer mappings; peer[rank] is local)
  int* peer_flags[kMaxWorld];   // flag pad of every rank (32 int32, zero at allocation)
  int* state;                   // local int32 [2]: [1] counts finished CTAs of the running launch
};

__device__ __forceinline__ bool epoch_behind(int value, int target) {
  return static_cast<int>(static_cast<unsigned>(value) - static_cast<unsigned>(target)) < 0;
}

// Waits until flags[0 .. world) have all reached `epoch`. Returns false when the limit ran out.
__device__ bool wait_epochs(const int* flags, int world, int epoch, long long limit, int* status) {
  const long long t0 = clock64();
  for (int r = 0; r < world; ++r) {
    while (true) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
      if (!epoch_behind(v, epoch)) break;
      if (clock64() - t0 > limit) {
        if (status) atomicCAS(status, kStatusOk, kStatusFlagTimeout);
        return false;
      }
      __nanosleep(100);
    }
  }
  return true;
}

template <typename T>
struct Vec16;   // 16 bytes of T, summed in fp32
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  static __device__ __forceinline__ void add(float* acc, const uint4& raw) {
    const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(e[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    uint4 o;
    o.x = pack_bf16x2(acc[0] * scale, acc[1] * scale);
    o.y = pack_bf16x2(acc[2] * scale, acc[3] * scale);
    o.z = pack_bf16x2(acc[4] * scale, acc[5] * scale);
    o.w = pack_bf16x2(acc[6] * scale, acc[7] * scale);
    return o;
  }
};
template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  static __device__ __forceinline__ void add(float* acc, const uint4& raw) {
    acc[0] += __uint_as_float(raw.x);
    acc[1] += __uint_as_float(raw.y);
    acc[2] += __uint_as_float(raw.z);
    acc[3] += __uint_as_float(raw.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* acc, float scale) {
    uint4 o;
    o.x = __float_as_uint(acc[0] * scale);
    o.y = __float_as_uint(acc[1] * scale);
    o.z = __float_as_uint(acc[2] * scale);
    o.w = __float_as_uint(acc[3] * scale);
    return o;
  }
};

// phase_mask: bit 0 start barrier, bit 1 reduce + broadcast of this rank's slice, bit 2 end barrier. 7 in production;
// single phases let one GPU stand in for all ranks, one launch per rank and phase (a test pre-sets the flags).
template <typename T>
__global__ void __launch_bounds__(256)
allreduce_twoshot_kernel(Ar2Args a, long long nvec, int rank, int world, int epoch, float scale, int phase_mask,
                         long long limit, int* status) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    if (phase_mask & 1) {
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < world; ++r)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[r] + rank), "r"(epoch) : "memory");
      }
      ok = wait_epochs(a.peer_flags[rank], world, epoch, limit, status) ? 1 : 0;
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok && (phase_mask & 2)) {
    const long long per = (nvec + world - 1) / world;
    const long long lo = rank * per;
    const long long hi = lo + per < nvec ? lo + per : nvec;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    // two vectors per thread and pass: 2 * world 16-byte loads are in flight before the first sum (NVLink latency is
    // a few microseconds; the kernel runs on few CTAs, so every thread has to keep several requests outstanding)
    for (long long i0 = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < hi; i0 += 2 * stride) {
      const long long i1 = i0 + stride;
      const bool two = i1 < hi;
      uint4 raw0[kMaxWorld], raw1[kMaxWorld];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < world) raw0[r] = reinterpret_cast<const uint4*>(a.peer[r])[i0];
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < world && two) raw1[r] = reinterpret_cast<const uint4*>(a.peer[r])[i1];
      float acc0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, acc1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < world) Vec16<T>::add(acc0, raw0[r]);
      const uint4 o0 = Vec16<T>::pack(acc0, scale);
#pragma unroll
      for (int r = 0; r < kMaxWorld; ++r)
        if (r < world) reinterpret_cast<uint4*>(a.peer[r])[i0] = o0;
      if (two) {
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
          if (r < world) Vec16<T>::add(acc1, raw1[r]);
        const uint4 o1 = Vec16<T>::pack(acc1, scale);
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
          if (r < world) reinterpret_cast<uint4*>(a.peer[r])[i1] = o1;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && (phase_mask & 4)) {
    __threadfence_system();                       // this CTA's peer stores, ordered before the counter
    const int done = atomicAdd(a.state + 1, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      a.state[1] = 0;
      __threadfence_system();
      if (s_ok) {
        for (int r = 0; r < world; ++r)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[r] + kDoneOffset + rank), "r"(epoch)
                       : "memory");
        wait_epochs(a.peer_flags[rank] + kDoneOffset, world, epoch, limit, status);
      }
    }
  }
}

}  // namespace
}  // namespace tsb

// In-place all-reduce (sum, then * scale) of n elements at peer[r] on every rank r.
//   peer[r]: the bucket inside rank r's symmetric buffer as mapped in this process (16-byte aligned);
//   peer_flags[r]: rank r's flag pad, int32 [32], zero at allocation, used by this call sequence only;
//   state: local int32 [2], zero at allocation; epoch: number of this call (1, 2, ...; compared modulo 2^32);
//   dtype: 1 bf16 (n % 8 == 0), 0 fp32 (n % 4 == 0); ctas: grid size (<= 0: 64); limit_cycles <= 0: about a second.
//   Every rank issues the same calls in the same order.
TSB_EXPORT int tsb_allreduce_twoshot(void* const* peer, void* const* peer_flags, int* state, long long n, int dtype,
                                     int rank, int world, int epoch, float scale, int ctas, int phase_mask,
                                     long long limit_cycles, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || n <= 0 || !state || (phase_mask & 7) == 0) return -2;
  if ((dtype != 0 && dtype != 1) || n % (dtype == 1 ? 8 : 4)) return -2;
  Ar2Args a{};
  for (int r = 0; r < world; ++r) {
    if (!peer[r] || !peer_flags[r] || (reinterpret_cast<uintptr_t>(peer[r]) & 15)) return -2;
    a.peer[r] = peer[r];
    a.peer_flags[r] = static_cast<int*>(peer_flags[r]);
  }
  a.state = state;
  const long long nvec = n / (dtype == 1 ? 8 : 4);
  int grid = ctas > 0 ? ctas : 64;
  const long long need = (nvec / world + 255) / 256;
  if (need < grid) grid = static_cast<int>(need > 0 ? need : 1);
  const long long limit = limit_cycles > 0 ? limit_cycles : kWaitCycleLimit;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 1)
    allreduce_twoshot_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, nvec, rank, world, epoch, scale, phase_mask, limit,
                                                                 device_status_word());
  else
    allreduce_twoshot_kernel<float><<<grid, 256, 0, s>>>(a, nvec, rank, world, epoch, scale, phase_mask, limit,
                                                         device_status_word());
  return static_cast<int>(cudaGetLastError());
}
