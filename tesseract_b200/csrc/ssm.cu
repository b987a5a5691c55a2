// State-space kernels for the Mamba block: chunkwise selective scan (S6 recurrence) and depthwise causal conv1d
// (optionally fused with SiLU).
//
//   h_t = exp(delta_t * A) * h_{t-1} + delta_t * B_t * u_t ;   y_t = <h_t, C_t> + D * u_t
// u, delta, y: [B, L, d] (fp32 or bf16); A: [d, N] fp32; Bm, Cm: [B, L, N]; D: [d] fp32; state: [B, d, N] fp32.
//
// The recurrence is linear in h, so a sequence is cut into chunks of 64 steps that are scanned in parallel:
//   pass 1  per (batch, chunk, channel): scan from a zero state -> local end state, sum of delta over the chunk
//           (the chunk's decay is exp(A * sum delta), so one float per channel replaces N decay factors);
//   pass 2  per (batch, channel, state): walk the chunks, turning local end states into chunk START states;
//   pass 3  per (batch, chunk, channel): rescan from the start state and emit y.
// Short sequences (decode steps, L <= 64) run as one pass with the state in registers; wide layers (batch x channels
// >= 2048, N <= 16) run the whole sequence as one pass too (scan_stream_pair_kernel below). The reference has the same
// three-pass structure with chunk 128 for fp32 prefill only (src/cuda/SelectiveScan.cu:95-228, N <= 32) and a
// one-thread-per-output conv (src/cuda/CausalConv1d.cu:16-36).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kChunk = 64;
constexpr int kScanThreads = 128;

// Scan `steps` time steps of channel `ch` starting at t0 from the state in h[]; optionally emit y.
template <typename T, int NMAX, bool EMIT>
__device__ __forceinline__ float scan_steps(const T* __restrict__ u, const T* __restrict__ delta,
                                            const float* __restrict__ Arow, const T* __restrict__ Bm,
                                            const T* __restrict__ Cm, float Dval, T* __restrict__ y, float (&h)[NMAX],
                                            long long base_bl, int t0, int steps, int d, int ch, int N) {
  float sum_delta = 0.f;
  float a[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) a[n] = n < N ? Arow[n] : 0.f;
  for (int s = 0; s < steps; ++s) {
    const long long bl = base_bl + t0 + s;  // flattened (batch, time)
    const float dt = to_f32<T>(delta[bl * d + ch]);
    const float uv = to_f32<T>(u[bl * d + ch]);
    sum_delta += dt;
    const float du = dt * uv;
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < NMAX; ++n) {
      if (n < N) {
        h[n] = __expf(dt * a[n]) * h[n] + du * to_f32<T>(Bm[bl * N + n]);
        if (EMIT) acc += h[n] * to_f32<T>(Cm[bl * N + n]);
      }
    }
    if (EMIT) y[bl * d + ch] = from_f32<T>(acc + Dval * uv);
  }
  return sum_delta;
}

// One pass: thread per (batch, channel); state in registers. Used for L <= kChunk.
template <typename T, int NMAX>
__global__ void __launch_bounds__(kScanThreads)
scan_direct_kernel(const T* u, const T* delta, const float* A, const T* Bm, const T* Cm, const float* Dv,
                   const float* state_in, T* y, float* state_out, int Bsz, int L, int d, int N) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= Bsz * d) return;
  const int b = idx / d, ch = idx % d;
  float h[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) h[n] = (state_in && n < N) ? state_in[(static_cast<long long>(b) * d + ch) * N + n] : 0.f;
  scan_steps<T, NMAX, true>(u, delta, A + static_cast<long long>(ch) * N, Bm, Cm, Dv[ch], y, h,
                            static_cast<long long>(b) * L, 0, L, d, ch, N);
#pragma unroll
  for (int n = 0; n < NMAX; ++n)
    if (n < N) state_out[(static_cast<long long>(b) * d + ch) * N + n] = h[n];
}

// pass 1: h_loc[b, c, n, ch] = end state of chunk c scanned from zero; sdelta[b, c, ch] = sum of delta.
template <typename T, int NMAX>
__global__ void __launch_bounds__(kScanThreads)
scan_local_kernel(const T* u, const T* delta, const float* A, const T* Bm, float* h_loc, float* sdelta, int Bsz, int L,
                  int d, int N, int nC) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(Bsz) * nC * d) return;
  const int ch = static_cast<int>(idx % d);
  const int c = static_cast<int>((idx / d) % nC);
  const int b = static_cast<int>(idx / (static_cast<long long>(d) * nC));
  float h[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) h[n] = 0.f;
  const int t0 = c * kChunk, steps = min(kChunk, L - t0);
  const float sd = scan_steps<T, NMAX, false>(u, delta, A + static_cast<long long>(ch) * N, Bm, nullptr, 0.f, nullptr, h,
                                              static_cast<long long>(b) * L, t0, steps, d, ch, N);
  const long long bc = static_cast<long long>(b) * nC + c;
  sdelta[bc * d + ch] = sd;
#pragma unroll
  for (int n = 0; n < NMAX; ++n)
    if (n < N) h_loc[(bc * N + n) * d + ch] = h[n];
}

// pass 2: sequential over chunks per (b, ch, n): local end states become chunk start states; final state out.
__global__ void __launch_bounds__(kScanThreads)
scan_combine_kernel(const float* A, float* h_loc, const float* sdelta, const float* state_in, float* state_out, int Bsz,
                    int d, int N, int nC) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(Bsz) * N * d) return;
  const int ch = static_cast<int>(idx % d);
  const int n = static_cast<int>((idx / d) % N);
  const int b = static_cast<int>(idx / (static_cast<long long>(d) * N));
  const float a = A[static_cast<long long>(ch) * N + n];
  float h = state_in ? state_in[(static_cast<long long>(b) * d + ch) * N + n] : 0.f;
  for (int c = 0; c < nC; ++c) {
    const long long bc = static_cast<long long>(b) * nC + c;
    const long long at = (bc * N + n) * d + ch;
    const float loc = h_loc[at];
    h_loc[at] = h;
    h = __expf(a * sdelta[bc * d + ch]) * h + loc;
  }
  state_out[(static_cast<long long>(b) * d + ch) * N + n] = h;
}

// pass 3: rescan every chunk from its start state and emit y.
template <typename T, int NMAX>
__global__ void __launch_bounds__(kScanThreads)
scan_output_kernel(const T* u, const T* delta, const float* A, const T* Bm, const T* Cm, const float* Dv,
                   const float* h_start, T* y, int Bsz, int L, int d, int N, int nC) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<long long>(Bsz) * nC * d) return;
  const int ch = static_cast<int>(idx % d);
  const int c = static_cast<int>((idx / d) % nC);
  const int b = static_cast<int>(idx / (static_cast<long long>(d) * nC));
  const long long bc = static_cast<long long>(b) * nC + c;
  float h[NMAX];
#pragma unroll
  for (int n = 0; n < NMAX; ++n) h[n] = n < N ? h_start[(bc * N + n) * d + ch] : 0.f;
  const int t0 = c * kChunk, steps = min(kChunk, L - t0);
  scan_steps<T, NMAX, true>(u, delta, A + static_cast<long long>(ch) * N, Bm, Cm, Dv[ch], y, h,
                            static_cast<long long>(b) * L, t0, steps, d, ch, N);
}

// Single pass for wide layers. The recurrence costs one exponential per (step, channel, state); the chunked passes
// above evaluate every one twice, this kernel once, with the state in registers for the whole sequence. A thread's
// steps are serial, so its inputs must be on chip before it gets there: u and delta travel through a four-stage
// shared-memory ring of 16-step tiles filled by cp.async (three tiles in flight per CTA). B_t and C_t are shared by
// all channels of a batch row: staged as floats, double buffered, the next tile held in registers while the current
// one is consumed. exp(delta * A) = 2^(delta * A * log2 e) with the constant folded into A.
// Two lanes share a channel, each owning eight of the (at most 16) states: a lane per channel leaves one warp per
// scheduler, which issues an instruction only every three cycles (dependent multiply-adds, the exponential unit's
// issue interval, shared-memory latency); two lanes keep the instruction count per channel and step and double the
// warps (four lanes double the instructions too: measured slower). The two partial sums of y meet in one shuffle; a
// full tile runs as straight-line code. 64 channels per CTA, 36 KB of shared memory in fp32.
// Measured on [4, 4096, 4096, 16] fp32: 0.66 ms against 2.6 ms for the three chunked passes (four lanes: 0.72 ms, one
// lane: 0.74 - 0.78 ms); the exponential unit is about 35 % busy.
constexpr int kStreamStages = 4;

__device__ __forceinline__ void scan_cp_async16(void* dst_smem, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src), "r"(src_bytes) : "memory");
}

// Requires d * sizeof(T) % 16 == 0 and 16-byte aligned u / delta (every 16-byte piece of a row is whole).
constexpr int kPairTile = 16;
constexpr int kPairThreads = 128;
constexpr int kPairCh = kPairThreads / 2;

template <typename T>
constexpr int pair_smem_bytes() {
  return 2 * kStreamStages * kPairTile * kPairCh * static_cast<int>(sizeof(T)) + 2 * 2 * kPairTile * 16 * 4;
}

template <typename T>
__global__ void __launch_bounds__(kPairThreads)
scan_stream_pair_kernel(const T* __restrict__ u, const T* __restrict__ delta, const float* __restrict__ A,
                        const T* __restrict__ Bm, const T* __restrict__ Cm, const float* __restrict__ Dv,
                        const float* __restrict__ state_in, T* __restrict__ y, float* __restrict__ state_out, int L,
                        int d, int N) {
  constexpr int NMAX = 16, SPL = 8;
  extern __shared__ __align__(16) uint8_t stream_smem[];
  constexpr int kStageElems = kPairTile * kPairCh;
  T* su = reinterpret_cast<T*>(stream_smem);                       // [stages][tile][channels]
  T* sd = su + kStreamStages * kStageElems;
  float* sB = reinterpret_cast<float*>(sd + kStreamStages * kStageElems);   // [2][tile][NMAX]
  float* sC = sB + 2 * kPairTile * NMAX;
  constexpr int kPerThread = kPairTile * NMAX / kPairThreads;      // staged B / C values per thread: 2
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));
  constexpr int kVecPerRow = kPairCh / kVec;
  constexpr int kPieces = kPairTile * kVecPerRow;
  const int tid = threadIdx.x;
  const int part = tid & 1;                         // states 8 * part .. 8 * part + 7
  const int cl = tid >> 1;
  const int b = blockIdx.y;
  const int ch0 = blockIdx.x * kPairCh;
  const bool active = ch0 + cl < d;
  const int ch = active ? ch0 + cl : d - 1;
  const long long base = static_cast<long long>(b) * L;
  float a2[SPL], h[SPL];
#pragma unroll
  for (int j = 0; j < SPL; ++j) {
    const int n = part * SPL + j;
    a2[j] = n < N ? A[static_cast<long long>(ch) * N + n] * 1.4426950408889634f : 0.f;
    h[j] = (state_in && n < N) ? state_in[(static_cast<long long>(b) * d + ch) * N + n] : 0.f;
  }
  const float Dval = Dv[ch];
  const int ntiles = (L + kPairTile - 1) / kPairTile;

  auto issue_tile = [&](int tile, int stage) {
    for (int idx = tid; idx < kPieces; idx += kPairThreads) {
      const int row = idx / kVecPerRow, v = idx % kVecPerRow;
      const int t = tile * kPairTile + row;
      const int c0 = ch0 + v * kVec;
      const bool ok = tile < ntiles && t < L && c0 < d;
      const long long off = ok ? (base + t) * d + c0 : 0;
      const int dst = (stage * kPairTile + row) * kPairCh + v * kVec;
      scan_cp_async16(su + dst, u + off, ok ? 16 : 0);
      scan_cp_async16(sd + dst, delta + off, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float rb[kPerThread], rc[kPerThread];
  auto fetch_bc = [&](int tile) {
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      const int idx = tid + k * kPairThreads;
      const int step = idx / NMAX, n = idx % NMAX;
      const int t = tile * kPairTile + step;
      const bool ok = n < N && t < L;
      rb[k] = ok ? to_f32<T>(Bm[(base + t) * N + n]) : 0.f;
      rc[k] = ok ? to_f32<T>(Cm[(base + t) * N + n]) : 0.f;
    }
  };
  auto park_bc = [&](int buf) {
#pragma unroll
    for (int k = 0; k < kPerThread; ++k) {
      const int idx = tid + k * kPairThreads;
      sB[buf * kPairTile * NMAX + idx] = rb[k];
      sC[buf * kPairTile * NMAX + idx] = rc[k];
    }
  };

#pragma unroll
  for (int st = 0; st < kStreamStages - 1; ++st) issue_tile(st, st);
  fetch_bc(0);
  park_bc(0);
  T* yp = y + base * d + ch;                        // advanced by d per step
  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile % kStreamStages;
    const int buf = tile & 1;
    asm volatile("cp.async.wait_group %0;" ::"n"(kStreamStages - 2) : "memory");
    __syncthreads();
    issue_tile(tile + kStreamStages - 1, (tile + kStreamStages - 1) % kStreamStages);
    if (tile + 1 < ntiles) fetch_bc(tile + 1);
    const T* tu = su + stage * kStageElems + cl;
    const T* td = sd + stage * kStageElems + cl;
    const float* tb = sB + buf * kPairTile * NMAX + part * SPL;
    const float* tc = sC + buf * kPairTile * NMAX + part * SPL;
    auto one_step = [&](int s) {
      const float uv = to_f32<T>(tu[s * kPairCh]);
      const float dt = to_f32<T>(td[s * kPairCh]);
      const float du = dt * uv;
      const float4 b0 = *reinterpret_cast<const float4*>(tb + s * NMAX);
      const float4 b1 = *reinterpret_cast<const float4*>(tb + s * NMAX + 4);
      const float4 c0 = *reinterpret_cast<const float4*>(tc + s * NMAX);
      const float4 c1 = *reinterpret_cast<const float4*>(tc + s * NMAX + 4);
      const float bb[SPL] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      const float cc[SPL] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int j = 0; j < SPL; j += 2) {
        float e0, e1;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(dt * a2[j]));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(dt * a2[j + 1]));
        h[j] = e0 * h[j] + du * bb[j];
        h[j + 1] = e1 * h[j + 1] + du * bb[j + 1];
        acc0 += h[j] * cc[j];
        acc1 += h[j + 1] * cc[j + 1];
      }
      float acc = acc0 + acc1;
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      if (active && part == 0) *yp = from_f32<T>(acc + Dval * uv);
      yp += d;
    };
    const int steps = min(kPairTile, L - tile * kPairTile);   // uniform over the CTA: the shuffles stay whole
    if (steps == kPairTile) {
#pragma unroll
      for (int s = 0; s < kPairTile; ++s) one_step(s);
    } else {
      for (int s = 0; s < steps; ++s) one_step(s);
    }
    if (tile + 1 < ntiles) park_bc(buf ^ 1);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (active) {
#pragma unroll
    for (int j = 0; j < SPL; ++j) {
      const int n = part * SPL + j;
      if (n < N) state_out[(static_cast<long long>(b) * d + ch) * N + n] = h[j];
    }
  }
}

template <typename T, int NMAX>
int run_scan(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm, const float* Dv,
             const float* state_in, void* y, float* state_out, float* scratch, int Bsz, int L, int d, int N,
             cudaStream_t s) {
  const T* u_ = static_cast<const T*>(u);
  const T* dl = static_cast<const T*>(delta);
  const T* b_ = static_cast<const T*>(Bm);
  const T* c_ = static_cast<const T*>(Cm);
  T* y_ = static_cast<T*>(y);
  if (L <= kChunk) {
    const int blocks = (Bsz * d + kScanThreads - 1) / kScanThreads;
    scan_direct_kernel<T, NMAX><<<blocks, kScanThreads, 0, s>>>(u_, dl, A, b_, c_, Dv, state_in, y_, state_out, Bsz, L, d, N);
    return static_cast<int>(cudaGetLastError());
  }
  if (NMAX == 16 && static_cast<long long>(Bsz) * d >= 2048 && Bsz <= 65535 && (d * sizeof(T)) % 16 == 0 &&
      ((reinterpret_cast<uintptr_t>(u) | reinterpret_cast<uintptr_t>(delta)) & 15) == 0) {
    static const int stream_on = [] { const char* e = getenv("TESSERACT_SCAN_STREAM"); return e ? atoi(e) : 1; }();
    if (stream_on) {
      constexpr int smem = pair_smem_bytes<T>();
      static_assert(smem <= 48 * 1024, "within the default dynamic shared-memory limit: no per-device attribute needed");
      dim3 grid((d + kPairCh - 1) / kPairCh, Bsz);
      scan_stream_pair_kernel<T><<<grid, kPairThreads, smem, s>>>(u_, dl, A, b_, c_, Dv, state_in, y_, state_out, L, d, N);
      return static_cast<int>(cudaGetLastError());
    }
  }
  const int nC = (L + kChunk - 1) / kChunk;
  float* h_loc = scratch;
  float* sdelta = scratch + static_cast<long long>(Bsz) * nC * N * d;
  const long long work = static_cast<long long>(Bsz) * nC * d;
  const unsigned blocks = static_cast<unsigned>((work + kScanThreads - 1) / kScanThreads);
  scan_local_kernel<T, NMAX><<<blocks, kScanThreads, 0, s>>>(u_, dl, A, b_, h_loc, sdelta, Bsz, L, d, N, nC);
  const long long work2 = static_cast<long long>(Bsz) * N * d;
  scan_combine_kernel<<<static_cast<unsigned>((work2 + kScanThreads - 1) / kScanThreads), kScanThreads, 0, s>>>(
      A, h_loc, sdelta, state_in, state_out, Bsz, d, N, nC);
  scan_output_kernel<T, NMAX><<<blocks, kScanThreads, 0, s>>>(u_, dl, A, b_, c_, Dv, h_loc, y_, Bsz, L, d, N, nC);
  return static_cast<int>(cudaGetLastError());
}

// y[b, t, c] = bias[c] + sum_k w[c, k] * x[b, t - (K - 1) + k, c]   (+ SiLU)
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv1d_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                     T* __restrict__ out, int Bsz, int L, int C, int K, int silu) {
  const long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long total = static_cast<long long>(Bsz) * L * C;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % C);
  const int t = static_cast<int>((idx / C) % L);
  const long long b = idx / (static_cast<long long>(C) * L);
  float acc = bias[c];
  for (int k = 0; k < K; ++k) {
    const int ts = t - (K - 1) + k;
    if (ts >= 0) acc += w[c * K + k] * to_f32<T>(x[(b * L + ts) * C + c]);
  }
  if (silu) acc = acc / (1.f + __expf(-acc));
  out[idx] = from_f32<T>(acc);
}

}  // namespace
}  // namespace tsb

// fp32 scratch elements tsb_selective_scan needs (0 for L <= 64).
TSB_EXPORT long long tsb_selective_scan_scratch_floats(int Bsz, int L, int d, int N) {
  if (L <= tsb::kChunk) return 0;
  const long long nC = (L + tsb::kChunk - 1) / tsb::kChunk;
  return static_cast<long long>(Bsz) * nC * d * (N + 1);
}

// dtype of u / delta / Bm / Cm / y: 0 = fp32, 1 = bf16. N <= 64. state_in may be NULL (zero state).
TSB_EXPORT int tsb_selective_scan(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm,
                                  const float* Dv, const float* state_in, void* y, float* state_out, float* scratch,
                                  int Bsz, int L, int d, int N, int dtype, int flags, void* stream) {
  using namespace tsb;
  (void)flags;
  if (Bsz <= 0 || L <= 0 || d <= 0 || N <= 0 || N > 64) return -2;
  if (L > kChunk && !scratch) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TSB_SCAN(TT)                                                                                              \
  (N <= 16 ? run_scan<TT, 16>(u, delta, A, Bm, Cm, Dv, state_in, y, state_out, scratch, Bsz, L, d, N, s)          \
           : N <= 32 ? run_scan<TT, 32>(u, delta, A, Bm, Cm, Dv, state_in, y, state_out, scratch, Bsz, L, d, N, s) \
                     : run_scan<TT, 64>(u, delta, A, Bm, Cm, Dv, state_in, y, state_out, scratch, Bsz, L, d, N, s))
  if (dtype == 0) return TSB_SCAN(float);
  if (dtype == 1) return TSB_SCAN(__nv_bfloat16);
#undef TSB_SCAN
  return -2;
}

// x, out: [B, L, C] (fp32 or bf16); w [C, K] fp32; bias [C] fp32. `state` is reserved (pass NULL).
TSB_EXPORT int tsb_causal_conv1d(const void* x, const float* w, const float* bias, const void* state, void* out,
                                 int Bsz, int L, int C, int K, int silu, int dtype, void* stream) {
  using namespace tsb;
  (void)state;
  if (Bsz <= 0 || L <= 0 || C <= 0 || K <= 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long total = static_cast<long long>(Bsz) * L * C;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (dtype == 0)
    causal_conv1d_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), w, bias, static_cast<float*>(out), Bsz, L, C, K, silu);
  else if (dtype == 1)
    causal_conv1d_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), w, bias,
                                                                static_cast<__nv_bfloat16*>(out), Bsz, L, C, K, silu);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
