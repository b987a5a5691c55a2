// Weight-streaming GEMM for decode-sized batches with fp8 operands on BOTH sides and the scales applied by the tensor
// core:  Y[M, N] (bf16) = Xq[M, K] (E4M3, one power-of-two scale per row and 32 columns) * W[N, K]^T (E4M3, one
// power-of-two scale per 128 x 128 block), tcgen05.mma kind::mxf8f6f4.block_scale, fp32 accumulators in TMEM.
//
// Why this form: a decode step streams every weight once; with fp8 weights and 16-bit activations somebody has to
// widen the weights before the multiply (the sibling kernel gemm_decode_wq.cu does, with eight conversion warps, and
// is bound by them at about a quarter of the copy bandwidth). Here nothing is converted: TMA writes the E4M3 weight
// tile in the layout the tensor core reads, the activations were quantised once by a small kernel in front
// (quant_act_mx_kernel below: M x K bytes, instead of once per CTA), and the block scales -- UE8M0 bytes, i.e. bare
// exponents -- sit in tensor memory next to the accumulators where the MMA picks them up. Weight scales restricted to
// powers of two are still "one fp32 scale per 128 x 128 block"; the byte the hardware wants is the exponent field of
// that float. What remains is a copy of W through the tensor cores at half the bytes of bf16.
//
//   * One CTA owns BN weight rows (32 .. 240, multiple of 16) and one of S K slices; the S CTAs of a tile form a
//     cluster and reduce their fp32 partial tiles through distributed shared memory. RB = 2: the CTA multiplies both
//     128-row blocks of a 129 .. 256-row batch with the tile it streams (two accumulators).
//   * Warp 0 lane 0: TMA producer (weights of the first ring before griddepcontrol.wait, activations after it).
//     Warp 1 lane 0: MMA issuer, four K = 32 instructions per 128-byte stage and row block.
//     Warps 2 .. 5: during the main loop they put the scale bytes of each stage into tensor memory with tcgen05.st
//     (every warp its own lane quadrant: the MMA wants the scales replicated in all four), afterwards they are the
//     epilogue.
//   * Scale layout in tensor memory (4 x 32-bit columns per 128 rows and stage): lane r % 32, column r / 32, byte j =
//     exponent of K block j (32 elements) of the stage; the instruction descriptor names the byte (sf_id = j).
// All waits are bounded (common.cuh).
//
// The reference has no fp8 tensor-core path for small batches: its fp8 GEMM dequantises into cuBLASLt
// (src/cuda/Fp8MatMul.cu:93-157) and its quantised decode path is CUDA-core GEMV (src/cuda/DequantMatMul.cu:95-127).
#include <cuda_fp8.h>

#include "common.cuh"

namespace tsb {
namespace {

constexpr int BM = 128;            // batch rows per row block (MMA M)
constexpr int BK = 128;            // K elements (= bytes) per pipeline stage: four MMAs of K = 32
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 220 * 1024;
constexpr int kThreads = 192;      // producer, MMA, 4 scale / epilogue warps
constexpr int kMaxSteps = 256;     // stages of one CTA's K slice whose weight exponents are staged in shared memory
constexpr int kSfCols = 16;        // tensor-memory columns of one stage's scales: A at +0 (4 per row block), B at +8 (8)
constexpr int kTmemCols = 512;

__host__ __device__ constexpr int max_bn(int rb) { return rb == 2 ? 208 : 240; }
__host__ __device__ constexpr int d_stride(int rb) { return rb == 2 ? 208 : 240; }   // columns between accumulators
__host__ __device__ constexpr int sf_base(int rb) { return rb == 2 ? 416 : 256; }    // first scale column
__host__ __device__ constexpr int max_sf_slots(int rb) { return (kTmemCols - sf_base(rb)) / kSfCols; }

struct Layout {
  int x_rows;     // rows of the activation box (batch rows rounded up to 8, at most 128)
  int x_pitch;    // bytes between activation stages (RB blocks of x_rows x 128, each 1024-aligned)
  int w_pitch;    // bytes between weight stages ([BN][128 B], 1024-aligned)
  int stages;
};

inline Layout make_layout(int M, int bn, int rb) {
  Layout L{};
  const int rows = (M >= BM || rb > 1) ? BM : ((M + 7) / 8) * 8;
  L.x_rows = rows;
  L.x_pitch = rb * rows * BK;                        // rows is a multiple of 8: every block starts on 1024 bytes
  L.w_pitch = ((bn * BK + 1023) / 1024) * 1024;
  // The MMA reads 128 activation rows of a block whatever x_rows is; what lies past the box only reaches accumulator
  // rows that are never stored, but must be inside the allocation: the activation ring comes first, the weight ring
  // (always more than 16 KB) behind it.
  int st = (kSmemBudget - 1024) / (L.x_pitch + L.w_pitch);
  if (st > kMaxStages) st = kMaxStages;
  if (st > max_sf_slots(rb)) st = max_sf_slots(rb);
  L.stages = st;
  return L;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Instruction descriptor of kind::mxf8f6f4.block_scale: E4M3 x E4M3, both K-major, UE8M0 scales, M = 128, N = n;
// sf_id selects the byte of the scale columns (= K block of the stage) for both operands.
__device__ __forceinline__ uint32_t mx_idesc(uint32_t n, uint32_t sf_id) {
  return (sf_id << 4) | ((n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (sf_id << 29);
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// This warp's 32 lanes x 4 (8) consecutive 32-bit columns: thread t writes lane (lane base + t).
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x8(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]),
               "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------ activation quantisers
// X [M, K] bf16 -> Xq [M, K] E4M3 and one UE8M0 exponent per row and 32 columns: q = x * 2^-(e - 127) with the smallest
// e that keeps the block inside +-448. The exponents are stored as one 32-bit word per row and 128 columns (byte j =
// columns 32 j .. 32 j + 31), laid out [K / 128][m_pad]: the word a GEMM CTA needs for (stage, row) is one load, and
// the 32 rows a warp needs are contiguous. The GEMM reads no word of a row past M.
//
// All three kernels below give consecutive lanes consecutive 8-column vectors of one row, so four lanes share a
// 32-column block and sixteen lanes a scale word; every lane of a warp calls the two helpers (lanes without data pass
// zeros and writer = false).
__device__ __forceinline__ uint32_t mx_quant8(const float (&v)[8], uint2* packed) {
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const int e = mx_exponent_byte(amax);
  const float inv = mx_inv_scale(e);
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    w[j] = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * j] * inv, v[2 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
  packed->x = w[0] | (w[1] << 16);
  packed->y = w[2] | (w[3] << 16);
  return static_cast<uint32_t>(e);
}
// Assembles the scale word of every 16-lane group from its four exponent bytes; the group's first lane stores it.
__device__ __forceinline__ void mx_store_word(uint32_t byte, int lane, bool writer, uint32_t* dst) {
  const int base = lane & 16;
  const uint32_t b0 = __shfl_sync(0xffffffffu, byte, base);
  const uint32_t b1 = __shfl_sync(0xffffffffu, byte, base + 4);
  const uint32_t b2 = __shfl_sync(0xffffffffu, byte, base + 8);
  const uint32_t b3 = __shfl_sync(0xffffffffu, byte, base + 12);
  if (writer && (lane & 15) == 0) *dst = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
}
__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float block_sum(float v, float* red) {      // same order of additions as the RMSNorm kernel
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__global__ void __launch_bounds__(256)
quant_act_mx_kernel(const __nv_bfloat16* __restrict__ X, long long ldx, uint8_t* __restrict__ Xq,
                    uint32_t* __restrict__ sf, int M, int K, int m_pad, int atoms) {
  pdl_trigger();
  pdl_grid_wait();
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = K / 8;                         // threads per row: 8 elements each, a multiple of 16
  const int row = static_cast<int>(t / per_row);
  const int c8 = static_cast<int>(t - static_cast<long long>(row) * per_row);
  if (row >= m_pad) return;                          // whole warps only: m_pad * per_row is a multiple of 32
  const int lane = threadIdx.x & 31;
  float v[8];
  if (row < M) {
    unpack_bf16x8(*reinterpret_cast<const uint4*>(X + static_cast<long long>(row) * ldx + c8 * 8), v);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
  }
  uint2 o;
  const uint32_t byte = mx_quant8(v, &o);
  if (row < M) *reinterpret_cast<uint2*>(Xq + static_cast<long long>(row) * K + c8 * 8) = o;
  // atoms = 0: [K / 128][m_pad] words (the decode GEMM reads a word per row); atoms = 1: 512-byte atoms
  // [m_pad / 128][K / 128][128 words], word (row % 32) * 4 + (row % 128) / 32 (what tcgen05.cp wants, gemm_mx.cu)
  const long long kc = c8 / 16;
  uint32_t* dst = atoms ? sf + ((static_cast<long long>(row >> 7) * (K / 128) + kc) << 7) + ((row & 31) << 2) + ((row & 127) >> 5)
                        : sf + kc * m_pad + row;
  mx_store_word(byte, lane, true, dst);
}

// RMSNorm (+ residual add) whose bf16 result exists only as the quantised operand of the next GEMM: one CTA per row.
// h = x (+ res), rounded to bf16 and written to h_out when a residual is given; y = bf16(h * rstd * w) -> (Xq, sf).
// Same arithmetic as the stand-alone RMSNorm kernel followed by quant_act_mx_kernel.
template <int MAXV>
__global__ void __launch_bounds__(256)
rmsnorm_quant_mx_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ h_out,
                        uint8_t* __restrict__ Xq, uint32_t* __restrict__ sf, int D, int m_pad, float eps) {
  pdl_trigger();
  pdl_grid_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31;
  const int nvec = D / 8;
  const size_t off = static_cast<size_t>(row) * D;
  float f[MAXV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v < nvec) {
      unpack_bf16x8(*reinterpret_cast<const uint4*>(x + off + v * 8), f[i]);
      if (res) {
        float g[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(res + off + v * 8), g);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[i][j] = round_bf16(f[i][j] + g[j]);      // normalise what is stored
#pragma unroll
        for (int j = 0; j < 4; ++j) op[j] = pack_bf16x2(f[i][2 * j], f[i][2 * j + 1]);
        *reinterpret_cast<uint4*>(h_out + off + v * 8) = o;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[i][j] * f[i][j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[i][j] = 0.f;
    }
  }
  const float tot = block_sum(ss, red);
  const float rstd = rsqrtf(tot / static_cast<float>(D) + eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int v = threadIdx.x + i * 256;
    const bool have = v < nvec;
    float y[8];
    if (have) {
      float g[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(w + v * 8), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = round_bf16(f[i][j] * rstd * g[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = 0.f;
    }
    uint2 o;
    const uint32_t byte = mx_quant8(y, &o);
    if (have) *reinterpret_cast<uint2*>(Xq + off + v * 8) = o;
    mx_store_word(byte, lane, have, sf + static_cast<long long>(v / 16) * m_pad + row);
  }
}

// silu(gate) * up of a packed [rows, 2F] tensor, rounded to bf16 and quantised: grid (column chunks, rows).
__global__ void __launch_bounds__(256)
swiglu_quant_mx_kernel(const __nv_bfloat16* __restrict__ gate_up, uint8_t* __restrict__ Xq, uint32_t* __restrict__ sf,
                       int F, int m_pad) {
  pdl_trigger();
  pdl_grid_wait();
  const int row = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int v = blockIdx.x * 256 + threadIdx.x;
  const bool have = v < F / 8;
  const __nv_bfloat16* gp = gate_up + static_cast<size_t>(row) * 2 * F;
  float y[8];
  if (have) {
    float g[8], u[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(gp + v * 8), g);
    unpack_bf16x8(*reinterpret_cast<const uint4*>(gp + F + v * 8), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = round_bf16(__fdividef(g[j], 1.f + __expf(-g[j])) * u[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) y[j] = 0.f;
  }
  uint2 o;
  const uint32_t byte = mx_quant8(y, &o);
  if (have) *reinterpret_cast<uint2*>(Xq + static_cast<size_t>(row) * F + v * 8) = o;
  mx_store_word(byte, lane, have, sf + static_cast<long long>(v / 16) * m_pad + row);
}

// ------------------------------------------------------------------------------------------------ the GEMM
template <int S, int RB>
__global__ void __launch_bounds__(kThreads, 1)
gemm_decode_mx_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                      const uint32_t* __restrict__ sfa, const float* __restrict__ w_scale,
                      __nv_bfloat16* __restrict__ Y, int M, int N, int K, int m_pad, long long ldy, int BN,
                      int scale_cols, int scale_rows, const Layout L, int* status, long long* trace) {
  const int ST = L.stages;
  // diagnostics: per-CTA phase timestamps (ns) when the host installed a trace buffer [CTAs][8]
  auto stamp = [&](int slot) {
    if (trace) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)::"memory");   // the clobber keeps it behind the barriers
      trace[static_cast<long long>(blockIdx.y * gridDim.x + blockIdx.x) * 8 + slot] = static_cast<long long>(t);
    }
  };
  if (threadIdx.x == 0) stamp(0);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sW = sX + ST * L.x_pitch;
  __shared__ __align__(8) uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ uint8_t s_exp[3 * kMaxSteps];      // weight exponents of this CTA: [row block 0 .. 2][stage]
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_smem;
  __shared__ volatile int cta_abort;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slice = static_cast<int>(cluster_ctarank());
  const int tile = static_cast<int>(blockIdx.x) / S;
  const int n0 = tile * BN;
  const int m0 = static_cast<int>(blockIdx.y) * BM * RB;
  const int x_block = L.x_rows * BK;               // one row block inside an activation stage
  const int total_kb = K / BK;
  const int kb_per = (total_kb + S - 1) / S;
  const int kb0 = slice * kb_per;
  const int kb1 = min(total_kb, kb0 + kb_per);
  const int nk = max(0, kb1 - kb0);
  const uint32_t w_bytes = static_cast<uint32_t>(BN) * BK;
  const uint32_t x_bytes = static_cast<uint32_t>(RB * L.x_rows) * BK;

  if (threadIdx.x == 0) {
    cta_abort = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full[s], 2 + 4);                  // weights, activations, four scale warps
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
    pdl_trigger();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_smem, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_smem;
  if (threadIdx.x == 0) stamp(1);                  // set-up done

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int w_issued = 0, ws = 0, x_issued = 0, xs = 0;
      uint32_t wphase = 0, xphase = 0;
      auto issue_w = [&]() {
        mbar_expect_tx(&full[ws], w_bytes);
        tma_load_2d(sW + ws * L.w_pitch, &tmW, &full[ws], (kb0 + w_issued) * BK, n0);
        ++w_issued;
        if (++ws == ST) {
          ws = 0;
          wphase ^= 1u;
        }
      };
      // weights do not depend on the kernel before this one: fill the ring before waiting for it
      while (w_issued < nk && w_issued < ST) issue_w();
      pdl_wait();
      long long t0 = clock64();
      uint32_t spins = 0;
      while (x_issued < nk || w_issued < nk) {
        bool progress = false;
        if (w_issued < nk && mbar_test_wait(&empty[ws], wphase ^ 1u)) {
          issue_w();
          progress = true;
        }
        if (x_issued < nk && mbar_test_wait(&empty[xs], xphase ^ 1u)) {
          mbar_expect_tx(&full[xs], x_bytes);
#pragma unroll
          for (int rb = 0; rb < RB; ++rb)
            tma_load_2d(sX + xs * L.x_pitch + rb * x_block, &tmX, &full[xs], (kb0 + x_issued) * BK, m0 + rb * BM);
          ++x_issued;
          if (++xs == ST) {
            xs = 0;
            xphase ^= 1u;
          }
          progress = true;
        }
        if (progress) {
          t0 = clock64();
          spins = 0;
        } else if ((++spins & 255u) == 0u) {
          if (cta_abort) break;
          if (clock64() - t0 > kWaitCycleLimit) {
            cta_abort = 1;
            if (status) atomicCAS(status, kStatusOk, kStatusMbarTimeout);
            break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nk; ++i) {
        if (!mbar_wait(&full[s], phase, &cta_abort, status)) break;
        if (i == 0) stamp(2);                      // first stage complete (weights, activations, scales)
        tc_fence_after();
        const uint32_t a_base = smem_u32(sX + s * L.x_pitch);
        const uint32_t b_base = smem_u32(sW + s * L.w_pitch);
        const uint32_t sf_col = tmem_base + static_cast<uint32_t>(sf_base(RB) + s * kSfCols);
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8(tmem_base + static_cast<uint32_t>(rb * d_stride(RB)),
                      umma_smem_desc_sw128(a_base + rb * x_block + k * 32, 16, 1024),
                      umma_smem_desc_sw128(b_base + k * 32, 16, 1024), mx_idesc(static_cast<uint32_t>(BN), k),
                      sf_col + static_cast<uint32_t>(rb * 4), sf_col + 8u, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);
        if (++s == ST) {
          s = 0;
          phase ^= 1u;
        }
      }
      umma_commit(&acc_bar);
      stamp(3);                                    // last MMA issued
    }
  } else {
    // ------------------------------------------------------------ scale warps (2 .. 5): one lane quadrant each
    const int q = warp & 3;
    const int t = (warp - 2) * 32 + lane;
    const int rblk0 = n0 >> 7;
    // The weight exponents (cold: they come from HBM) and the first activation scale words (written by the kernel
    // before this one) are requested together; the exponents are parked in shared memory once both are under way.
    constexpr int kExpPerThread = 3 * kMaxSteps / 128;
    float w_sc[kExpPerThread];
#pragma unroll
    for (int j = 0; j < kExpPerThread; ++j) {
      const int e = t + j * 128;
      w_sc[j] = 1.f;
      if (e < 3 * nk && e < 3 * kMaxSteps) {
        const int b3 = e / nk, kk = e - b3 * nk;
        w_sc[j] = __ldg(w_scale + static_cast<long long>(min(rblk0 + b3, scale_rows - 1)) * scale_cols +
                        min(kb0 + kk, scale_cols - 1));
      }
    }
    // which of the CTA's (at most three) 128-row weight blocks each of this thread's eight scale rows belongs to
    int blk[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) blk[c] = min(((n0 + 32 * c + lane) >> 7) - rblk0, 2);
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    // Activation scale words come from global memory (L2): kDepth stages are kept in flight in registers, so that a
    // stage costs a quarter of a load latency instead of a whole one.
    constexpr int kDepth = 4;
    uint32_t ring[kDepth][RB][4];
    auto load_a = [&](int i, uint32_t (&dst)[RB][4]) {
      const uint32_t* src = sfa + static_cast<long long>(kb0 + i) * m_pad + m0 + lane;
#pragma unroll
      for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int r = rb * BM + 32 * c;
          dst[rb][c] = (m0 + r + lane < M) ? __ldg(src + r) : 0x7f7f7f7fu;   // rows past M: scale 1 on zeros
        }
    };
    pdl_wait();                                     // the activation scales come from the kernel before this one
#pragma unroll
    for (int d = 0; d < kDepth; ++d)
      if (d < nk) load_a(d, ring[d]);
#pragma unroll
    for (int j = 0; j < kExpPerThread; ++j) {
      const int e = t + j * 128;
      if (e < 3 * nk && e < 3 * kMaxSteps) {
        const int b3 = e / nk, kk = e - b3 * nk;
        s_exp[b3 * kMaxSteps + kk] = static_cast<uint8_t>((__float_as_uint(w_sc[j]) >> 23) & 0xffu);
      }
    }
    asm volatile("bar.sync 2, 128;" ::: "memory");
    int s = 0;
    uint32_t phase = 0;
    bool alive = true;
    for (int i0 = 0; i0 < nk && alive; i0 += kDepth) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        const int i = i0 + d;
        if (i >= nk || !alive) break;
        uint32_t a_cur[RB][4];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
          for (int c = 0; c < 4; ++c) a_cur[rb][c] = ring[d][rb][c];
        if (i + kDepth < nk) load_a(i + kDepth, ring[d]);
        const bool ok = mbar_wait(&empty[s], phase ^ 1u, &cta_abort, status);
        if (!__all_sync(0xffffffffu, ok ? 1 : 0)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const uint32_t col = lane_addr + static_cast<uint32_t>(sf_base(RB) + s * kSfCols);
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
          tmem_st_32x4(col + rb * 4, a_cur[rb][0], a_cur[rb][1], a_cur[rb][2], a_cur[rb][3]);
        const int kk = min(i, kMaxSteps - 1);
        uint32_t b[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) b[c] = static_cast<uint32_t>(s_exp[blk[c] * kMaxSteps + kk]) * 0x01010101u;
        tmem_st_32x8(col + 8, b);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
        if (i == 0 && threadIdx.x == 64) stamp(5);   // scales of the first stage in tensor memory
        if (++s == ST) {
          s = 0;
          phase ^= 1u;
        }
      }
    }
  }

  // ---------------------------------------------------------------- epilogue (warps 2..5)
  // Only the batch rows that exist are moved: a 16-row batch occupies one warp's lanes, the other three have nothing
  // to do. Without a K split the bf16 result goes from the accumulator registers straight to global memory; with one,
  // every CTA parks its fp32 partial rows in shared memory (over the idle rings) and sums an equal share of the rows
  // from all S partials through distributed shared memory, several vectors in flight per thread.
  const int part_pitch = BN * 4 + 16;            // fp32 partial row, padded against bank conflicts
  const int m_valid = min(M - m0, RB * BM);      // batch rows of this CTA that exist
  if (warp >= 2) {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool ok = mbar_wait(&acc_bar, 0, &cta_abort, status);
    const bool warp_ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    tc_fence_after();
    if (threadIdx.x == 64) stamp(4);               // accumulator complete
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
      const int rows_here = m_valid - rb * BM;
      if (q * 32 >= rows_here) continue;         // warp-uniform
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(rb * d_stride(RB));
      if (S == 1) {
        const int grow = m0 + rb * BM + row;
        __nv_bfloat16* yrow = Y + static_cast<long long>(grow) * ldy + n0;
        const bool vec_ok = (ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          if (warp_ok && nk > 0) {
            tmem_ld_32x16(t_row + static_cast<uint32_t>(c), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
          if (row < rows_here) {
            if (vec_ok && n0 + c + 16 <= N) {
              uint4 o0, o1;
              o0.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
              o0.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
              o0.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
              o0.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
              o1.x = pack_bf16x2(__uint_as_float(r[8]), __uint_as_float(r[9]));
              o1.y = pack_bf16x2(__uint_as_float(r[10]), __uint_as_float(r[11]));
              o1.z = pack_bf16x2(__uint_as_float(r[12]), __uint_as_float(r[13]));
              o1.w = pack_bf16x2(__uint_as_float(r[14]), __uint_as_float(r[15]));
              *reinterpret_cast<uint4*>(yrow + c) = o0;
              *reinterpret_cast<uint4*>(yrow + c + 8) = o1;
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (n0 + c + i < N) yrow[c + i] = __float2bfloat16(__uint_as_float(r[i]));
            }
          }
        }
      } else {
        uint8_t* prow = smem + (rb * BM + row) * part_pitch;
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          if (warp_ok && nk > 0) {
            tmem_ld_32x16(t_row + static_cast<uint32_t>(c), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = 0u;
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(prow + (c + i) * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (S > 1) {
    cluster_sync_all();
    if (threadIdx.x == 0) stamp(6);
    if (warp >= 2) {
      // CTA `slice` sums an equal share of the existing batch rows from all S partial tiles
      const int rows_per = (m_valid + S - 1) / S;
      const int row_lo = slice * rows_per;
      const int row_hi = min(m_valid, row_lo + rows_per);
      const int t = (warp - 2) * 32 + lane;        // 0 .. 127
      const int vec_per_row = BN / 4;
      const int total = max(0, row_hi - row_lo) * vec_per_row;
      const bool vec_ok = (ldy % 4 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 7) == 0);
      constexpr int U = S >= 8 ? 2 : 4;            // vectors per thread and pass: U * S remote loads in flight
      for (int it0 = t; it0 < total; it0 += 128 * U) {
        float4 v[U][S];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int it = it0 + u * 128;
          if (it < total) {
            const int rr = it / vec_per_row;
            const uint32_t local = smem_u32(smem + (row_lo + rr) * part_pitch + (it - rr * vec_per_row) * 16);
#pragma unroll
            for (int r = 0; r < S; ++r) v[u][r] = ld_cluster_f4(map_to_cta(local, static_cast<uint32_t>(r)));
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int it = it0 + u * 128;
          if (it >= total) break;
          const int rr = it / vec_per_row;
          const int cv = it - rr * vec_per_row;
          float4 acc = v[u][0];
#pragma unroll
          for (int r = 1; r < S; ++r) {
            acc.x += v[u][r].x;
            acc.y += v[u][r].y;
            acc.z += v[u][r].z;
            acc.w += v[u][r].w;
          }
          const int col = n0 + cv * 4;
          __nv_bfloat16* dst = Y + static_cast<long long>(m0 + row_lo + rr) * ldy + col;
          if (vec_ok && col + 4 <= N) {
            uint2 o;
            o.x = pack_bf16x2(acc.x, acc.y);
            o.y = pack_bf16x2(acc.z, acc.w);
            *reinterpret_cast<uint2*>(dst) = o;
          } else {
            const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
            for (int j = 0; j < 4; ++j)
              if (col + j < N) dst[j] = __float2bfloat16(a4[j]);
          }
        }
      }
    }
    // nobody leaves (and frees its shared memory) before every CTA of the cluster has finished reading
    cluster_sync_all();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) stamp(7);
  if (warp == 1) {
    if (cta_abort) {
      for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

long long* g_trace = nullptr;   // diagnostics: see tsb_gemm_decode_mx_trace

template <int S, int RB>
cudaError_t config_mx(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* at, int grid_x, int grid_y, int pdl, cudaStream_t s) {
  auto kern = gemm_decode_mx_kernel<S, RB>;
  static PerDeviceFlag attr;
  if (attr.unset()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return e;
    attr.set();
  }
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(static_cast<unsigned>(grid_x), static_cast<unsigned>(grid_y), 1);
  cfg->blockDim = dim3(kThreads, 1, 1);
  cfg->dynamicSmemBytes = kSmemBudget;
  cfg->stream = s;
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = S;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  int n_attr = 1;
  if (pdl) {
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    n_attr = 2;
  }
  cfg->attrs = at;
  cfg->numAttrs = n_attr;
  return cudaSuccess;
}

template <int S, int RB>
int launch_mx(const CUtensorMap& tx, const CUtensorMap& tw, const uint32_t* sfa, const float* w_scale, void* Y, int M,
              int N, int K, int m_pad, long long ldy, int BN, int scale_cols, int scale_rows, const Layout& L, int pdl,
              cudaStream_t s) {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute at[2];
  const int tiles = (N + BN - 1) / BN;
  cudaError_t e = config_mx<S, RB>(&cfg, at, tiles * S, (M + RB * BM - 1) / (RB * BM), pdl, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_decode_mx_kernel<S, RB>, tx, tw, sfa, w_scale,
                                             static_cast<__nv_bfloat16*>(Y), M, N, K, m_pad, ldy, BN, scale_cols,
                                             scale_rows, L, device_status_word(), g_trace));
}

// CTAs that can be resident at once when launched as clusters of S (a GPC takes whole clusters only).
template <int S>
int resident_ctas() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return sm_count();
  if (cached[dev] == 0) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    int clusters = 0;
    if (config_mx<S, 1>(&cfg, at, S * 64, 1, 0, nullptr) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&clusters, gemm_decode_mx_kernel<S, 1>, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sm_count() / S * 3 / 4;
    }
    cached[dev] = clusters * S;
  }
  return cached[dev];
}
int resident_ctas_for(int split) {
  switch (split) {
    case 1: return resident_ctas<1>();
    case 2: return resident_ctas<2>();
    case 4: return resident_ctas<4>();
    default: return resident_ctas<8>();
  }
}

bool layout_ok(const Layout& L, int bn, int rb) {
  return L.stages >= 2 && bn <= max_bn(rb) && rb * BM * (bn * 4 + 16) <= kSmemBudget - 1024;
}

// Best single-wave plan for `rb` row blocks per CTA (score < 0: none): the plan that keeps the most SMs streaming,
// fewer K stages per CTA at equal counts; short K slices, eight-way splits and narrow tiles are marked down.
double plan_family(int M, int N, int kb, int fixed_bn, int rb, int* bn_out, int* split_out) {
  const int row_ctas = (M + rb * BM - 1) / (rb * BM);
  double best = -1.0;
  for (int s : {1, 2, 4, 8}) {
    if (s > 1 && kb / s < 4) break;
    int cap = resident_ctas_for(s);
    const int sms = sm_count();
    const int safe = s == 1 ? sms : (s == 2 ? sms - sms % 16 : (s == 4 ? (sms / 18) * 16 : (sms / 18) * 16 - 16));
    if (cap <= 0 || cap > sms) cap = safe;
    for (int bn = max_bn(rb); bn >= 32; bn -= 16) {
      if (fixed_bn > 0 && bn != fixed_bn) continue;
      const Layout L = make_layout(M, bn, rb);
      if (!layout_ok(L, bn, rb)) continue;
      const int tiles = (N + bn - 1) / bn;
      const int ctas = tiles * s * row_ctas;
      if (ctas > cap) continue;
      const double useful = static_cast<double>(N) / (static_cast<double>(tiles) * bn);
      double score = static_cast<double>(ctas) * useful - 0.04 * ((kb + s - 1) / s);
      if (kb / s < 8) score *= 0.85;
      if (s == 8) score *= 0.9;
      if (bn < 64) score *= 0.85;
      if (score > best + 1e-9) {
        best = score;
        *bn_out = bn;
        *split_out = s;
      }
    }
  }
  return best;
}

void plan_tiles(int M, int N, int kb, int fixed_bn, int* bn_out, int* split_out, int* rb_out) {
  int bn = 128, s = 1, rb = 1;
  double best = -1.0;
  if (M > BM && M <= 2 * BM) {
    int b2 = 0, s2 = 0;
    const double sc2 = plan_family(M, N, kb, fixed_bn, 2, &b2, &s2);
    if (sc2 > 0.0) {
      best = sc2;
      bn = b2;
      s = s2;
      rb = 2;
    }
  }
  if (best < 0.0) {
    int b1 = 0, s1 = 0;
    const double sc1 = plan_family(M, N, kb, fixed_bn, 1, &b1, &s1);
    if (sc1 > 0.0) {
      best = sc1;
      bn = b1;
      s = s1;
      rb = 1;
    }
  }
  if (best < 0.0) {   // more tiles than resident CTAs at every width: several waves of the widest tile that has room
    rb = (M > BM && M <= 2 * BM) ? 2 : 1;
    bn = fixed_bn > 0 ? fixed_bn : 32;
    s = 1;
    for (int b = max_bn(rb); b >= 32 && fixed_bn <= 0; b -= 16) {
      if (layout_ok(make_layout(M, b, rb), b, rb)) {
        bn = b;
        break;
      }
    }
  }
  *bn_out = bn;
  *split_out = s;
  *rb_out = rb;
}

}  // namespace
}  // namespace tsb

// Rows of the scale array the two calls below share: M rounded up to a multiple of 128.
TSB_EXPORT int tsb_mx_m_pad(int M) { return (M + 127) / 128 * 128; }

// X [M, K] bf16 (row stride ldx) -> Xq [M, K] E4M3 (dense rows) and sf: uint32 [K / 128][tsb_mx_m_pad(M)], byte j of
// word (k / 128, m) = UE8M0 exponent of X[m, 128 (k / 128) + 32 j .. + 31]. K % 128 == 0, X 16-byte aligned, ldx % 8 == 0.
TSB_EXPORT int tsb_quant_act_mx_layout(const void* X, long long ldx, void* Xq, void* sf, int M, int K, int atoms,
                                       void* stream);
TSB_EXPORT int tsb_quant_act_mx(const void* X, long long ldx, void* Xq, void* sf, int M, int K, void* stream) {
  return tsb_quant_act_mx_layout(X, ldx, Xq, sf, M, K, 0, stream);
}
// atoms != 0: sf receives 512-byte scale atoms [tsb_mx_m_pad(M) / 128][K / 128][128 words] (the operand of tsb_gemm_mx).
TSB_EXPORT int tsb_quant_act_mx_layout(const void* X, long long ldx, void* Xq, void* sf, int M, int K, int atoms,
                                       void* stream) {
  using namespace tsb;
  if (M <= 0 || K <= 0 || K % 128 || !X || !Xq || !sf || (ldx % 8) || (reinterpret_cast<uintptr_t>(X) & 15) ||
      (reinterpret_cast<uintptr_t>(Xq) & 7))
    return -2;
  const int m_pad = tsb_mx_m_pad(M);
  const long long threads = static_cast<long long>(m_pad) * (K / 8);
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  return static_cast<int>(launch_pdl(quant_act_mx_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(stream),
                                     pdl_all_enabled(), static_cast<const __nv_bfloat16*>(X), ldx,
                                     static_cast<uint8_t*>(Xq), static_cast<uint32_t*>(sf), M, K, m_pad, atoms));
}

// Fused producers of the same (Xq, sf) pair, bf16 only, D (F) % 128 == 0, dense rows:
//   tsb_rmsnorm_quant_mx: y = rmsnorm(x + res) * w; h_out receives x + res when res is given (may alias x or res).
//   tsb_swiglu_quant_mx:  y = silu(gate_up[:, :F]) * gate_up[:, F:].
TSB_EXPORT int tsb_rmsnorm_quant_mx(const void* x, const void* res, const void* w, void* h_out, void* Xq, void* sf,
                                    int rows, int D, float eps, void* stream) {
  using namespace tsb;
  if (rows <= 0 || D <= 0 || D % 128 || D > 8 * 256 * 4 || !x || !w || !Xq || !sf || (res && !h_out)) return -2;
  const int m_pad = tsb_mx_m_pad(rows);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int maxv = (D / 8 + 255) / 256;
#define TSB_RQ(MV)                                                                                                  \
  return static_cast<int>(launch_pdl(rmsnorm_quant_mx_kernel<MV>, dim3(rows), dim3(256), 0, s, pdl_all_enabled(),    \
                                     static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),   \
                                     static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(h_out),       \
                                     static_cast<uint8_t*>(Xq), static_cast<uint32_t*>(sf), D, m_pad, eps))
  if (maxv <= 1) TSB_RQ(1);
  if (maxv <= 2) TSB_RQ(2);
  TSB_RQ(4);
#undef TSB_RQ
}

TSB_EXPORT int tsb_swiglu_quant_mx(const void* gate_up, void* Xq, void* sf, int rows, int F, void* stream) {
  using namespace tsb;
  if (rows <= 0 || rows > 65535 || F <= 0 || F % 128 || !gate_up || !Xq || !sf) return -2;
  const dim3 grid(static_cast<unsigned>((F / 8 + 255) / 256), static_cast<unsigned>(rows));
  return static_cast<int>(launch_pdl(swiglu_quant_mx_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream),
                                     pdl_all_enabled(), static_cast<const __nv_bfloat16*>(gate_up),
                                     static_cast<uint8_t*>(Xq), static_cast<uint32_t*>(sf), F, tsb_mx_m_pad(rows)));
}

// Y [M, N] bf16 (row stride ldy) = dequant(Xq, sf) * dequant(W, w_scale)^T.
//   Xq, sf: what tsb_quant_act_mx wrote for the same M and K (any M; 129 .. 256 rows run as two row blocks per CTA,
//           more as several CTA rows).
//   W: E4M3 bytes [N, K] (row stride ldw bytes, a multiple of 16); w_scale: fp32 [ceil(N/128), K/128] row-major, every
//      entry a power of two (only the exponent field is used).
//   K % 128 == 0. bn / split: 0 = chosen here; otherwise bn a multiple of 16 in [32, 240] (208 for more than 128 rows),
//   split in {1, 2, 4, 8}. pdl != 0: programmatic stream serialisation (the kernel starts under the tail of its
//   predecessor and waits for it before it reads Xq and sf).
TSB_EXPORT int tsb_gemm_decode_mx(const void* Xq, const void* sf, const void* W, const float* w_scale, void* Y, int M,
                                  int N, int K, long long ldw, long long ldy, int bn, int split, int pdl, void* stream) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || K % BK || !Xq || !sf || !W || !w_scale || !Y) return -2;
  if ((reinterpret_cast<uintptr_t>(Xq) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) || (ldw % 16)) return -2;
  const int kb = K / BK;
  int rb = 1;
  {
    int pbn = 0, ps = 0, prb = 1;
    plan_tiles(M, N, kb, bn > 0 ? bn : 0, &pbn, &ps, &prb);
    if (bn <= 0) bn = pbn;
    if (split <= 0) split = ps;
    rb = prb;
  }
  if (bn < 32 || bn % 16 || (split != 1 && split != 2 && split != 4 && split != 8)) return -2;
  if (rb == 2 && bn > max_bn(2)) rb = 1;
  Layout L = make_layout(M, bn, rb);
  if (!layout_ok(L, bn, rb) && rb == 2) {
    rb = 1;
    L = make_layout(M, bn, rb);
  }
  if (!layout_ok(L, bn, rb)) return -2;
  if ((kb + split - 1) / split > kMaxSteps) return -2;
  CUtensorMap tx, tw;
  if (!make_tmap_2d(&tx, Xq, 1, M, K, K, L.x_rows, BK, true)) return -3;
  if (!make_tmap_2d(&tw, W, 1, N, K, ldw, bn, BK, true)) return -3;
  const int scale_cols = K / 128, scale_rows = (N + 127) / 128;
  const int m_pad = tsb_mx_m_pad(M);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TSB_MX_ARGS tx, tw, static_cast<const uint32_t*>(sf), w_scale, Y, M, N, K, m_pad, ldy, bn, scale_cols, scale_rows, L, pdl & 1, s
#define TSB_MX(S_) return rb == 2 ? launch_mx<S_, 2>(TSB_MX_ARGS) : launch_mx<S_, 1>(TSB_MX_ARGS)
  switch (split) {
    case 1: TSB_MX(1);
    case 2: TSB_MX(2);
    case 4: TSB_MX(4);
    default: TSB_MX(8);
  }
#undef TSB_MX
#undef TSB_MX_ARGS
}

// Diagnostics: the launches that follow write eight nanosecond timestamps per CTA into `buf` (int64 [CTAs][8]: start,
// set-up done, first stage landed, last MMA issued, accumulator complete, first scales written, cluster synchronised, end);
// nullptr switches it off again.
TSB_EXPORT void tsb_gemm_decode_mx_trace(void* buf) { tsb::g_trace = static_cast<long long*>(buf); }

// The plan the call above makes (host only): *bn (a positive value fixes the width), *split, ring depth (negative: two
// row blocks per CTA), resident CTAs for that cluster size.
TSB_EXPORT int tsb_gemm_decode_mx_plan(int M, int N, int K, int* bn, int* split, int* stages, int* resident) {
  using namespace tsb;
  if (M <= 0 || N <= 0 || K <= 0 || K % BK || !bn || !split) return -2;
  const int fixed = *bn > 0 ? *bn : 0;
  int rb = 1;
  plan_tiles(M, N, K / BK, fixed, bn, split, &rb);
  const Layout L = make_layout(M, *bn, rb);
  if (stages) *stages = L.stages * (rb == 2 ? -1 : 1);
  if (resident) *resident = resident_ctas_for(*split);
  return 0;
}
