// Expert-parallel token exchange over peer-mapped memory (NVLink P2P through NVSwitch), entirely on the device:
// no host read of the routing counts, no NCCL all-to-all.
//
// Ranks r = 0 .. world-1 each own E_local consecutive experts. For one MoE layer call every rank
//   1. publishes its per-expert assignment counts to all peers       (tsb_ep_publish_counts, then a flag barrier)
//   2. derives, from the full [world][E] count matrix that everyone now holds, the row layout of EVERY owner:
//      expert-major, source-rank-minor, every expert's block padded to 128 rows       (tsb_ep_plan)
//   3. pushes each of its (token, expert) rows straight into the owner's receive buffer at the row the plan
//      assigns, together with a tag (source rank, assignment index) for the way back  (tsb_ep_dispatch, barrier)
//   4. the owner runs the grouped GEMMs over its receive buffer, then pushes every result row back into the source
//      rank's return buffer at the assignment index                                     (tsb_ep_return, barrier)
// The backward pass uses the same two push kernels in the opposite roles (output gradients are dispatched with the
// rows remembered from the forward pass, input gradients are returned). Pushes are 16-byte stores to the peer
// mapping; visibility is established by the flag barrier kernel of gemm_fused_comm.cu that follows each phase.
// The reference has no expert parallelism; its single-GPU MoE reads the counts back on the host between two
// kernels (src/cuda/MoeForward.cu:241-247).
#include "common.cuh"

namespace tsb {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxE = 256;

struct PeerPtrs {
  void* p[kMaxWorld];
};

// cnt_all[r] (on every rank r) [src][E] <- this rank's counts
__global__ void ep_publish_counts_kernel(PeerPtrs cnt_all, const int* __restrict__ counts, int rank, int world, int E) {
  const int e = threadIdx.x;
  if (e >= E) return;
  const int c = counts[e];
  for (int r = 0; r < world; ++r) static_cast<int*>(cnt_all.p[r])[rank * E + e] = c;
}

// One CTA. From cnt [world][E]:
//   send_base[e]      row in the OWNER's receive buffer where this rank's rows for global expert e start
//   offsets_local[El + 1]  padded (128) starts of this rank's local experts in its own receive buffer
//   cursor[e] = 0
__global__ void ep_plan_kernel(const int* __restrict__ cnt, int* __restrict__ send_base, int* __restrict__ offsets_local,
                               int* __restrict__ cursor, int rank, int world, int E, int pad) {
  const int El = E / world;
  if (threadIdx.x == 0) {
    for (int o = 0; o < world; ++o) {
      int acc = 0;
      for (int el = 0; el < El; ++el) {
        const int e = o * El + el;
        if (o == rank) offsets_local[el] = acc;
        int before = 0, total = 0;
        for (int s = 0; s < world; ++s) {
          const int c = cnt[s * E + e];
          if (s < rank) before += c;
          total += c;
        }
        send_base[e] = acc + before;
        acc += (total + pad - 1) / pad * pad;
      }
      if (o == rank) offsets_local[El] = acc;
    }
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
}

// tags of the receive buffer: -1 everywhere (padding rows stay -1); rows of recv that are padding are zeroed later
// by the gather-style consumers through the tag test.
__global__ void __launch_bounds__(256) ep_fill_kernel(int* __restrict__ p, long long n, int v) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    p[i] = v;
}

// One warp per assignment i = t * k + r: row (scale ? scale[i] : 1) * src[t] -> owner's receive buffer.
// dest_row[i]: on FIRST use (assign_rows != 0) it is computed here from send_base + a per-expert cursor and stored;
// later uses (backward) read it. The owner's tag array gets (rank << 24 | i).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx, const float* __restrict__ scale,
                   PeerPtrs recv, PeerPtrs tags, const int* __restrict__ send_base, int* __restrict__ cursor,
                   int* __restrict__ dest_row, long long n_assign, int k, int D, int El, int rank, int assign_rows,
                   long long cap_rows, int* status) {
  const long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (i >= n_assign) return;
  const int e = idx[i];
  const int owner = e / El;
  int row;
  if (assign_rows) {
    row = 0;
    if (lane == 0) {
      row = send_base[e] + atomicAdd(&cursor[e], 1);
      dest_row[i] = row;
    }
    row = __shfl_sync(0xffffffffu, row, 0);
  } else {
    row = dest_row[i];
  }
  if (row < 0 || row >= cap_rows) {  // a plan / capacity mismatch: record it, never write out of bounds
    if (lane == 0 && status) atomicCAS(status, kStatusOk, kStatusBadArgument);
    return;
  }
  const uint4* in = reinterpret_cast<const uint4*>(src + (i / k) * D);
  uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(recv.p[owner]) + static_cast<long long>(row) * D);
  const int nvec = D / 8;
  if (!scale) {
    for (int v = lane; v < nvec; v += 32) out[v] = in[v];
  } else {
    const float sc = scale[i];
    for (int v = lane; v < nvec; v += 32) {
      uint4 x = in[v];
      __nv_bfloat162* e2 = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(e2[j]);
        e2[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
      }
      out[v] = x;
    }
  }
  if (lane == 0 && assign_rows) static_cast<int*>(tags.p[owner])[row] = (rank << 24) | static_cast<int>(i);
}

// One warp per row of the owner's buffer: rows with a tag go to ret[source rank][assignment index].
__global__ void __launch_bounds__(256)
ep_return_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ tags, PeerPtrs ret, long long rows,
                 const int* __restrict__ rows_used, int D, long long ret_rows, int* status) {
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows || (rows_used && r >= *rows_used)) return;
  const int tag = tags[r];
  if (tag < 0) return;
  const int srank = tag >> 24;
  const long long i = tag & 0xFFFFFF;
  if (i >= ret_rows) {
    if (lane == 0 && status) atomicCAS(status, kStatusOk, kStatusBadArgument);
    return;
  }
  const uint4* in = reinterpret_cast<const uint4*>(ys + r * D);
  uint4* out = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(ret.p[srank]) + i * D);
  for (int v = lane; v < D / 8; v += 32) out[v] = in[v];
}

// dst[r] = tags[r] >= 0 ? src[r] : 0   (local copy of the receive buffer with clean padding rows)
__global__ void __launch_bounds__(256)
ep_clean_copy_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ tags, __nv_bfloat16* __restrict__ dst,
                     long long rows, const int* __restrict__ rows_used, int D) {
  const long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (r >= rows || (rows_used && r >= *rows_used)) return;
  const bool live = tags[r] >= 0;
  const uint4* in = reinterpret_cast<const uint4*>(src + r * D);
  uint4* out = reinterpret_cast<uint4*>(dst + r * D);
  for (int v = lane; v < D / 8; v += 32) out[v] = live ? in[v] : make_uint4(0u, 0u, 0u, 0u);
}

PeerPtrs to_peers(void* const* p, int world) {
  PeerPtrs a;
  for (int i = 0; i < kMaxWorld; ++i) a.p[i] = i < world ? p[i] : nullptr;
  return a;
}

}  // namespace
}  // namespace tsb

// counts int32 [E] (this rank's assignments per global expert) -> row `rank` of every rank's cnt_all [world][E].
TSB_EXPORT int tsb_ep_publish_counts(void* const* cnt_all, const int* counts, int rank, int world, int E, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || E < 1 || E > kMaxE || E % world) return -2;
  ep_publish_counts_kernel<<<1, kMaxE, 0, static_cast<cudaStream_t>(stream)>>>(to_peers(cnt_all, world), counts, rank, world, E);
  return static_cast<int>(cudaGetLastError());
}

// cnt int32 [world][E] (complete) -> send_base [E], offsets_local [E / world + 1] (padded to `pad` rows), cursor [E] = 0.
TSB_EXPORT int tsb_ep_plan(const int* cnt, int* send_base, int* offsets_local, int* cursor, int rank, int world, int E,
                           int pad, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || E < 1 || E > kMaxE || E % world || pad < 1) return -2;
  ep_plan_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(cnt, send_base, offsets_local, cursor, rank, world, E, pad);
  return static_cast<int>(cudaGetLastError());
}

TSB_EXPORT int tsb_ep_fill_i32(int* p, long long n, int value, void* stream) {
  using namespace tsb;
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 2048) blocks = 2048;
  ep_fill_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(p, n, value);
  return static_cast<int>(cudaGetLastError());
}

// Push row (scale ? scale[i] : 1) * src[i / k] of every assignment i to the owner of expert idx[i].
//   recv[r] / tags[r]: rank r's receive buffer [cap_rows][D] bf16 and tag array [cap_rows] (peer mappings).
//   assign_rows != 0: first dispatch of a layer call: rows are assigned (send_base + cursor), stored in dest_row and
//   tagged at the owner; assign_rows == 0: reuse dest_row (backward), tags untouched.
TSB_EXPORT int tsb_ep_dispatch(const void* src, const int* idx, const float* scale, void* const* recv, void* const* tags,
                               const int* send_base, int* cursor, int* dest_row, long long n_assign, int k, int D,
                               int E_local, int rank, int world, int assign_rows, long long cap_rows, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || n_assign < 0 || D <= 0 || D % 8 || k < 1 || E_local < 1) return -2;
  if (n_assign == 0) return 0;
  if (n_assign >= (1 << 24)) return -2;  // the tag packs the assignment index into 24 bits
  const unsigned blocks = static_cast<unsigned>((n_assign * 32 + 255) / 256);
  ep_dispatch_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), idx, scale, to_peers(recv, world), to_peers(tags, world), send_base, cursor,
      dest_row, n_assign, k, D, E_local, rank, assign_rows, cap_rows, device_status_word());
  return static_cast<int>(cudaGetLastError());
}

// Push every tagged row of ys [rows][D] back to ret[source rank][assignment index] (ret_rows rows each).
// rows_used (device int, may be null): only rows below it are looked at (the padded total of the plan).
TSB_EXPORT int tsb_ep_return(const void* ys, const int* tags, void* const* ret, long long rows, const int* rows_used, int D,
                             long long ret_rows, int world, void* stream) {
  using namespace tsb;
  if (world < 1 || world > kMaxWorld || rows < 0 || D <= 0 || D % 8) return -2;
  if (rows == 0) return 0;
  const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
  ep_return_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ys), tags, to_peers(ret, world), rows, rows_used, D, ret_rows, device_status_word());
  return static_cast<int>(cudaGetLastError());
}

// dst [rows][D] = src [rows][D] where tags[r] >= 0, zeros elsewhere; rows at or beyond *rows_used are left alone.
TSB_EXPORT int tsb_ep_clean_copy(const void* src, const int* tags, void* dst, long long rows, const int* rows_used, int D,
                                 void* stream) {
  using namespace tsb;
  if (rows <= 0 || D <= 0 || D % 8) return -2;
  const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
  ep_clean_copy_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), tags, static_cast<__nv_bfloat16*>(dst), rows, rows_used, D);
  return static_cast<int>(cudaGetLastError());
}
