// Native CPU FP32 GEMM of the host runtime: C[M, N] = A[M, K] * op(B), row-major, B given as [K, N] or as
// [N, K] (transposed use, the layout of a Linear weight).
//
// Design: a register tile chosen at run time: 14 x 32 on AVX-512 (28 zmm accumulators + 2 loads of B + 1 broadcast
// of A = 31 of 32 registers), 6 x 16 on AVX2 (12 + 2 + 1 of 16).
// Up to 512^3 (AVX-512) nothing is packed: the tile reads A rows and B rows where they lie and one parallel loop walks
// the tiles of C; a weight-layout B is transposed once, by all threads, into a scratch that outlives the call.
// Above that the classic three-level blocking: B is packed once per (kc, nc) panel into NR-wide column strips -- by
// all threads, a strip each -- and A once per (mc, kc) block into MR-high row strips, so the microkernel streams both
// with unit stride; edge tiles go through the same kernel on a zero-padded pack and a masked write-back. Threads
// split the M range of every panel in row blocks sized so that every thread gets the same number of them (whole
// strips, at most 8 per block). The panel buffers are kept between calls (fresh megabytes per call cost more in page
// faults than a mid-sized product). Small problems stay on few threads, since waking a thread costs more than a share
// of a 64^3 product, and TESSERACT_GEMM_MAX_THREADS caps the count for co-located jobs.
// Counterpart in the reference: a 4 x 8 FMA microkernel with an adaptive thread cap (src/ops/cpu/GemmAvx2.cpp:25-150).
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <vector>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define TSBH_HAVE_AVX2 1
#endif
#ifdef _OPENMP
#include <omp.h>
#endif

#include "host_runtime.hpp"

namespace tsbh {
namespace {

constexpr int64_t NC = 2048;

// packs A[mc, kc] (row stride lda) into strips of MR rows: strip s holds kc columns of MR values each
void pack_a(const float* A, int64_t lda, int64_t mc, int64_t kc, int MR, float* out) {
  for (int64_t i0 = 0; i0 < mc; i0 += MR) {
    const int64_t mr = std::min<int64_t>(MR, mc - i0);
    // every source row is read once with unit stride; the writes are the strided side (MR floats apart)
    for (int64_t i = 0; i < mr; ++i) {
      const float* src = A + (i0 + i) * lda;
      float* dst = out + i;
      for (int64_t k = 0; k < kc; ++k) dst[k * MR] = src[k];
    }
    for (int64_t i = mr; i < MR; ++i) {
      float* dst = out + i;
      for (int64_t k = 0; k < kc; ++k) dst[k * MR] = 0.f;
    }
    out += kc * MR;
  }
}

// packs one NR-wide strip of op(B)[kc, nc] starting at column j0: kc rows of NR values each.
// b_nk = false: B is [K, N] (element (k, n) at B[k * ldb + n]); true: B is [N, K] (element at B[n * ldb + k]).
void pack_b_strip(const float* B, int64_t ldb, bool b_nk, int64_t kc, int64_t nc, int64_t j0, int NR, float* out) {
  const int64_t nr = std::min<int64_t>(NR, nc - j0);
  if (!b_nk) {
    for (int64_t k = 0; k < kc; ++k) {
      const float* src = B + k * ldb + j0;
      for (int64_t j = 0; j < nr; ++j) out[j] = src[j];
      for (int64_t j = nr; j < NR; ++j) out[j] = 0.f;
      out += NR;
    }
    return;
  }
  // [N, K] storage: walk each of the nr source rows once (unit stride reads), scatter into the strip
  for (int64_t j = 0; j < nr; ++j) {
    const float* src = B + (j0 + j) * ldb;
    for (int64_t k = 0; k < kc; ++k) out[k * NR + j] = src[k];
  }
  for (int64_t j = nr; j < NR; ++j)
    for (int64_t k = 0; k < kc; ++k) out[k * NR + j] = 0.f;
}

void write_back(const float* tmp, int ld_tmp, float* C, int64_t ldc, int64_t mr, int64_t nr, bool accumulate) {
  for (int64_t i = 0; i < mr; ++i)
    for (int64_t j = 0; j < nr; ++j) C[i * ldc + j] = accumulate ? C[i * ldc + j] + tmp[i * ld_tmp + j] : tmp[i * ld_tmp + j];
}

// C[mr, nr] (+)= Ap[kc x MR] * Bp[kc x NR]
using MicroKernel = void (*)(const float* Ap, const float* Bp, int64_t kc, float* C, int64_t ldc, int64_t mr, int64_t nr,
                             bool accumulate);

void micro_scalar(const float* Ap, const float* Bp, int64_t kc, float* C, int64_t ldc, int64_t mr, int64_t nr,
                  bool accumulate) {
  constexpr int MR = 6, NR = 16;
  float tmp[MR * NR];
  for (int i = 0; i < MR * NR; ++i) tmp[i] = 0.f;
  for (int64_t k = 0; k < kc; ++k)
    for (int i = 0; i < MR; ++i)
      for (int j = 0; j < NR; ++j) tmp[i * NR + j] += Ap[k * MR + i] * Bp[k * NR + j];
  write_back(tmp, NR, C, ldc, mr, nr, accumulate);
}

#ifdef TSBH_HAVE_AVX2
void micro_avx2(const float* Ap, const float* Bp, int64_t kc, float* C, int64_t ldc, int64_t mr, int64_t nr,
                bool accumulate) {
  constexpr int MR = 6, NR = 16;
  __m256 acc[MR][2];
  for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm256_setzero_ps();
  for (int64_t k = 0; k < kc; ++k) {
    const __m256 b0 = _mm256_loadu_ps(Bp + k * NR);
    const __m256 b1 = _mm256_loadu_ps(Bp + k * NR + 8);
    const float* a = Ap + k * MR;
#pragma GCC unroll 6
    for (int i = 0; i < MR; ++i) {
      const __m256 av = _mm256_broadcast_ss(a + i);
      acc[i][0] = _mm256_fmadd_ps(av, b0, acc[i][0]);
      acc[i][1] = _mm256_fmadd_ps(av, b1, acc[i][1]);
    }
  }
  if (mr == MR && nr == NR) {
    for (int i = 0; i < MR; ++i) {
      float* c = C + i * ldc;
      if (accumulate) {
        _mm256_storeu_ps(c, _mm256_add_ps(_mm256_loadu_ps(c), acc[i][0]));
        _mm256_storeu_ps(c + 8, _mm256_add_ps(_mm256_loadu_ps(c + 8), acc[i][1]));
      } else {
        _mm256_storeu_ps(c, acc[i][0]);
        _mm256_storeu_ps(c + 8, acc[i][1]);
      }
    }
    return;
  }
  alignas(32) float tmp[MR * NR];
  for (int i = 0; i < MR; ++i) {
    _mm256_store_ps(tmp + i * NR, acc[i][0]);
    _mm256_store_ps(tmp + i * NR + 8, acc[i][1]);
  }
  write_back(tmp, NR, C, ldc, mr, nr, accumulate);
}

// The same loop on 512-bit registers; compiled for AVX-512 whatever the translation unit's baseline, chosen at run time.
__attribute__((target("avx512f,fma"))) void micro_avx512(const float* Ap, const float* Bp, int64_t kc, float* C,
                                                         int64_t ldc, int64_t mr, int64_t nr, bool accumulate) {
  constexpr int MR = 14, NR = 32;
  __m512 acc[MR][2];
#pragma GCC unroll 14
  for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm512_setzero_ps();
  for (int64_t k = 0; k < kc; ++k) {
    const __m512 b0 = _mm512_loadu_ps(Bp + k * NR);
    const __m512 b1 = _mm512_loadu_ps(Bp + k * NR + 16);
    const float* a = Ap + k * MR;
#pragma GCC unroll 14
    for (int i = 0; i < MR; ++i) {
      const __m512 av = _mm512_set1_ps(a[i]);
      acc[i][0] = _mm512_fmadd_ps(av, b0, acc[i][0]);
      acc[i][1] = _mm512_fmadd_ps(av, b1, acc[i][1]);
    }
  }
  if (mr == MR && nr == NR) {
#pragma GCC unroll 14
    for (int i = 0; i < MR; ++i) {
      float* c = C + i * ldc;
      if (accumulate) {
        _mm512_storeu_ps(c, _mm512_add_ps(_mm512_loadu_ps(c), acc[i][0]));
        _mm512_storeu_ps(c + 16, _mm512_add_ps(_mm512_loadu_ps(c + 16), acc[i][1]));
      } else {
        _mm512_storeu_ps(c, acc[i][0]);
        _mm512_storeu_ps(c + 16, acc[i][1]);
      }
    }
    return;
  }
  alignas(64) float tmp[MR * NR];
#pragma GCC unroll 14
  for (int i = 0; i < MR; ++i) {
    _mm512_store_ps(tmp + i * NR, acc[i][0]);
    _mm512_store_ps(tmp + i * NR + 16, acc[i][1]);
  }
  write_back(tmp, NR, C, ldc, mr, nr, accumulate);
}

// Small products skip packing: the register tile reads A rows (one broadcast per row and k) and B rows (two vector
// loads per k) where they lie. Rows beyond mr shadow the last valid row (computed, not stored); columns beyond nr are
// masked out of the loads and stores.
__attribute__((target("avx512f,fma"))) void micro_avx512_direct(const float* A, int64_t lda, const float* B, int64_t ldb,
                                                                int64_t K, float* C, int64_t ldc, int64_t mr, int64_t nr) {
  constexpr int MR = 14;
  const __mmask16 m0 = static_cast<__mmask16>(nr >= 16 ? 0xFFFFu : ((1u << nr) - 1u));
  const __mmask16 m1 = static_cast<__mmask16>(nr >= 32 ? 0xFFFFu : (nr > 16 ? ((1u << (nr - 16)) - 1u) : 0u));
  const float* ar[MR];
#pragma GCC unroll 14
  for (int i = 0; i < MR; ++i) ar[i] = A + std::min<int64_t>(i, mr - 1) * lda;
  __m512 acc[MR][2];
#pragma GCC unroll 14
  for (int i = 0; i < MR; ++i) acc[i][0] = acc[i][1] = _mm512_setzero_ps();
  for (int64_t k = 0; k < K; ++k) {
    const __m512 b0 = _mm512_maskz_loadu_ps(m0, B + k * ldb);
    const __m512 b1 = _mm512_maskz_loadu_ps(m1, B + k * ldb + 16);
#pragma GCC unroll 14
    for (int i = 0; i < MR; ++i) {
      const __m512 av = _mm512_set1_ps(ar[i][k]);
      acc[i][0] = _mm512_fmadd_ps(av, b0, acc[i][0]);
      acc[i][1] = _mm512_fmadd_ps(av, b1, acc[i][1]);
    }
  }
#pragma GCC unroll 14
  for (int i = 0; i < MR; ++i) {
    if (i < mr) {
      _mm512_mask_storeu_ps(C + i * ldc, m0, acc[i][0]);
      _mm512_mask_storeu_ps(C + i * ldc + 16, m1, acc[i][1]);
    }
  }
}
#endif

struct Tile {
  int mr, nr;
  int64_t kc;          // depth of a packed panel: an A strip and a B strip together fit the L1 data cache
  MicroKernel kernel;
};

Tile pick_tile() {
#ifdef TSBH_HAVE_AVX2
  static const bool no512 = [] { const char* e = std::getenv("TESSERACT_GEMM_NO_AVX512"); return e && std::atoi(e) != 0; }();
  if (!no512 && __builtin_cpu_supports("avx512f")) return {14, 32, 192, micro_avx512};
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return {6, 16, 256, micro_avx2};
#endif
  return {6, 16, 256, micro_scalar};
}

}  // namespace

int gemm_num_threads(int64_t M, int64_t N, int64_t K, int requested) {
  int hw = 1;
#ifdef _OPENMP
  hw = omp_get_max_threads();
#endif
  int cap = hw;
  if (const char* e = std::getenv("TESSERACT_GEMM_MAX_THREADS")) {
    const int v = std::atoi(e);
    if (v > 0) cap = std::min(cap, v);
  }
  if (requested > 0) cap = std::min(cap, requested);
  // about half a MFLOP of work per thread before another one pays for itself
  const double flops = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
  const int by_work = static_cast<int>(std::max(1.0, flops / 0.5e6));
  const int by_rows = static_cast<int>((M + 5) / 6);
  return std::max(1, std::min({cap, by_work, by_rows}));
}

void gemm_f32(const float* A, int64_t lda, const float* B, int64_t ldb, bool b_nk, float* C, int64_t ldc, int64_t M,
              int64_t N, int64_t K, int threads) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) {
    for (int64_t i = 0; i < M; ++i) std::memset(C + i * ldc, 0, sizeof(float) * static_cast<size_t>(N));
    return;
  }
  static const Tile tile = pick_tile();
#ifdef TSBH_HAVE_AVX2
  // up to 512^3: no packed panels, one parallel loop over the register tiles of C. A weight-layout B ([N, K]) is
  // transposed once, by all threads, into a [K, N] scratch whose row stride avoids multiples of 4 KB.
  if (tile.kernel == micro_avx512 && static_cast<double>(M) * N * K <= 512.0 * 512.0 * 512.0 && K * N <= 512 * 512 &&
      M * K <= 512 * 512) {
    const int nt = gemm_num_threads(M, N, K, threads);
    const int64_t tm = (M + 13) / 14, tn = (N + 31) / 32;
    // scratch of the calling thread, kept between calls: a fresh megabyte per call costs more in page faults than
    // the product itself
    static thread_local std::vector<float> bt;
    const float* Bd = B;
    int64_t ldbd = ldb;
    if (b_nk) {
      ldbd = (N + 15) / 16 * 16;
      if (ldbd % 1024 == 0) ldbd += 16;
      if (bt.size() < static_cast<size_t>(K * ldbd)) bt.resize(static_cast<size_t>(K * ldbd));
      Bd = bt.data();
    }
    float* const dst = b_nk ? bt.data() : nullptr;     // the caller's buffer: `bt` names another vector in a worker
#pragma omp parallel num_threads(nt) if (nt > 1)
    {
      if (b_nk) {
        const int64_t kb = (K + 15) / 16;
#pragma omp for schedule(static)
        for (int64_t blk = 0; blk < kb * ((N + 15) / 16); ++blk) {     // 16 x 16 blocks: both sides stay in cache lines
          const int64_t k0 = (blk % kb) * 16, n0 = (blk / kb) * 16;
          const int64_t k1 = std::min(K, k0 + 16), n1 = std::min(N, n0 + 16);
          for (int64_t n = n0; n < n1; ++n)
            for (int64_t k = k0; k < k1; ++k) dst[k * ldbd + n] = B[n * ldb + k];
        }
      }
#pragma omp for schedule(static)
      for (int64_t t = 0; t < tm * tn; ++t) {
        const int64_t i0 = (t / tn) * 14, j0 = (t % tn) * 32;
        micro_avx512_direct(A + i0 * lda, lda, Bd + j0, ldbd, K, C + i0 * ldc + j0, ldc, std::min<int64_t>(14, M - i0),
                            std::min<int64_t>(32, N - j0));
      }
    }
    return;
  }
#endif
  const int MR = tile.mr, NR = tile.nr;
  const int64_t KC = tile.kc;
  const int nt = gemm_num_threads(M, N, K, threads);
  // one row block per thread where M allows it: whole strips, at most 8 of them (the packed block stays in L2)
  const int64_t strips = (M + MR - 1) / MR;
  const int64_t rounds = (strips + nt * 8 - 1) / (nt * 8);           // every thread takes `rounds` blocks of <= 8 strips
  const int64_t per_block = std::max<int64_t>(1, (strips + nt * rounds - 1) / (nt * rounds));
  const int64_t MC = per_block * MR;
  const int64_t m_blocks = (M + MC - 1) / MC;
  const int64_t max_strips_b = (std::min(N, NC) + NR - 1) / NR;
  // panels live in buffers that outlast the call (grow-only): the caller's for B, every worker's own for A
  static thread_local std::vector<float> bpack_store;
  if (bpack_store.size() < static_cast<size_t>(KC * max_strips_b * NR)) bpack_store.resize(static_cast<size_t>(KC * max_strips_b * NR));
  float* const bpack_ptr = bpack_store.data();
#pragma omp parallel num_threads(nt)
  {
    static thread_local std::vector<float> apack;
    if (apack.size() < static_cast<size_t>(MC * KC)) apack.resize(static_cast<size_t>(MC * KC));
    for (int64_t jc = 0; jc < N; jc += NC) {
      const int64_t nc = std::min(NC, N - jc);
      const int64_t b_strips = (nc + NR - 1) / NR;
      for (int64_t pc = 0; pc < K; pc += KC) {
        const int64_t kc = std::min(KC, K - pc);
        const float* Bpanel = b_nk ? B + jc * ldb + pc : B + pc * ldb + jc;
#pragma omp for schedule(static)
        for (int64_t sb = 0; sb < b_strips; ++sb)
          pack_b_strip(Bpanel, ldb, b_nk, kc, nc, sb * NR, NR, bpack_ptr + sb * kc * NR);
        // (the loop above ends with a barrier: the panel is complete before anyone multiplies)
        const bool accumulate = pc > 0;
        // few row blocks (a small M): the column strips of the panel are split over threads as well, each task
        // packing its own copy of the A block (cheap at these sizes)
        const int64_t n_splits = m_blocks < nt ? std::min<int64_t>(b_strips, (2 * nt + m_blocks - 1) / m_blocks) : 1;
        const int64_t strips_per_split = (b_strips + n_splits - 1) / n_splits;
#pragma omp for schedule(dynamic, 1)
        for (int64_t task = 0; task < m_blocks * n_splits; ++task) {
          const int64_t ib = task / n_splits, js = task % n_splits;
          const int64_t ic = ib * MC;
          const int64_t mc = std::min(MC, M - ic);
          const int64_t jr_begin = js * strips_per_split * NR;
          const int64_t jr_end = std::min(nc, (js + 1) * strips_per_split * NR);
          if (jr_begin >= jr_end) continue;
          pack_a(A + ic * lda + pc, lda, mc, kc, MR, apack.data());
          for (int64_t jr = jr_begin; jr < jr_end; jr += NR) {
            const int64_t nr = std::min<int64_t>(NR, nc - jr);
            const float* Bp = bpack_ptr + (jr / NR) * kc * NR;
            for (int64_t ir = 0; ir < mc; ir += MR) {
              const int64_t mr = std::min<int64_t>(MR, mc - ir);
              tile.kernel(apack.data() + (ir / MR) * kc * MR, Bp, kc, C + (ic + ir) * ldc + jc + jr, ldc, mr, nr,
                          accumulate);
            }
          }
        }
        // (barrier again: the next panel overwrites bpack)
      }
    }
  }
}

bool gemm_avx2_supported() {
#ifdef TSBH_HAVE_AVX2
  return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#else
  return false;
#endif
}

}  // namespace tsbh
