// Native CPU FP32 GEMM of the host runtime: C[M, N] = A[M, K] * op(B), row-major, B given as [K, N] or as
// [N, K] (transposed use, the layout of a Linear weight).
//
// Design: the classic three-level blocking around a 6 x 16 register tile (12 ymm accumulators + 2 loads of B + 1
// broadcast of A = 15 of the 16 AVX2 registers). B is packed once per (kc, nc) panel into 16-wide column strips,
// A once per (mc, kc) block into 6-high row strips, so the microkernel streams both with unit stride; edge tiles go
// through the same kernel on a zero-padded pack and a masked write-back. Threads split the M range of every panel
// (OpenMP); small problems stay on few threads, since waking 48 threads costs more than a 128^3 product, and
// TESSERACT_GEMM_MAX_THREADS caps the count for co-located jobs.
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

constexpr int MR = 6, NR = 16;
constexpr int64_t MC = 96, KC = 256, NC = 2048;

// packs A[mc, kc] (row stride lda) into strips of MR rows: strip s holds kc columns of MR values each
void pack_a(const float* A, int64_t lda, int64_t mc, int64_t kc, float* out) {
  for (int64_t i0 = 0; i0 < mc; i0 += MR) {
    const int64_t mr = std::min<int64_t>(MR, mc - i0);
    for (int64_t k = 0; k < kc; ++k) {
      for (int64_t i = 0; i < mr; ++i) out[i] = A[(i0 + i) * lda + k];
      for (int64_t i = mr; i < MR; ++i) out[i] = 0.f;
      out += MR;
    }
  }
}

// packs op(B)[kc, nc] into strips of NR columns: strip s holds kc rows of NR values each.
// b_nk = false: B is [K, N] (element (k, n) at B[k * ldb + n]); true: B is [N, K] (element at B[n * ldb + k]).
void pack_b(const float* B, int64_t ldb, bool b_nk, int64_t kc, int64_t nc, float* out) {
  for (int64_t j0 = 0; j0 < nc; j0 += NR) {
    const int64_t nr = std::min<int64_t>(NR, nc - j0);
    for (int64_t k = 0; k < kc; ++k) {
      if (!b_nk) {
        const float* src = B + k * ldb + j0;
        for (int64_t j = 0; j < nr; ++j) out[j] = src[j];
      } else {
        for (int64_t j = 0; j < nr; ++j) out[j] = B[(j0 + j) * ldb + k];
      }
      for (int64_t j = nr; j < NR; ++j) out[j] = 0.f;
      out += NR;
    }
  }
}

// C[mr, nr] (+)= Ap[kc x MR] * Bp[kc x NR]
void micro_kernel(const float* Ap, const float* Bp, int64_t kc, float* C, int64_t ldc, int64_t mr, int64_t nr,
                  bool accumulate) {
#ifdef TSBH_HAVE_AVX2
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
  alignas(32) float tmp[MR][NR];
  for (int i = 0; i < MR; ++i) {
    _mm256_store_ps(tmp[i], acc[i][0]);
    _mm256_store_ps(tmp[i] + 8, acc[i][1]);
  }
#else
  float tmp[MR][NR];
  for (int i = 0; i < MR; ++i)
    for (int j = 0; j < NR; ++j) tmp[i][j] = 0.f;
  for (int64_t k = 0; k < kc; ++k)
    for (int i = 0; i < MR; ++i)
      for (int j = 0; j < NR; ++j) tmp[i][j] += Ap[k * MR + i] * Bp[k * NR + j];
#endif
  for (int64_t i = 0; i < mr; ++i)
    for (int64_t j = 0; j < nr; ++j) C[i * ldc + j] = accumulate ? C[i * ldc + j] + tmp[i][j] : tmp[i][j];
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
  // about 2 MFLOP of work per thread before another one pays for itself
  const double flops = 2.0 * static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
  const int by_work = static_cast<int>(std::max(1.0, flops / 2.0e6));
  const int by_rows = static_cast<int>((M + MR - 1) / MR);
  return std::max(1, std::min({cap, by_work, by_rows}));
}

void gemm_f32(const float* A, int64_t lda, const float* B, int64_t ldb, bool b_nk, float* C, int64_t ldc, int64_t M,
              int64_t N, int64_t K, int threads) {
  if (M <= 0 || N <= 0) return;
  if (K <= 0) {
    for (int64_t i = 0; i < M; ++i) std::memset(C + i * ldc, 0, sizeof(float) * static_cast<size_t>(N));
    return;
  }
  const int nt = gemm_num_threads(M, N, K, threads);
  std::vector<float> bpack(static_cast<size_t>(KC * ((std::min(N, NC) + NR - 1) / NR) * NR));
  for (int64_t jc = 0; jc < N; jc += NC) {
    const int64_t nc = std::min(NC, N - jc);
    for (int64_t pc = 0; pc < K; pc += KC) {
      const int64_t kc = std::min(KC, K - pc);
      pack_b(b_nk ? B + jc * ldb + pc : B + pc * ldb + jc, ldb, b_nk, kc, nc, bpack.data());
      const bool accumulate = pc > 0;
      const int64_t m_blocks = (M + MC - 1) / MC;
#pragma omp parallel num_threads(nt)
      {
        std::vector<float> apack(static_cast<size_t>(MC * KC));
#pragma omp for schedule(dynamic, 1)
        for (int64_t ib = 0; ib < m_blocks; ++ib) {
          const int64_t ic = ib * MC;
          const int64_t mc = std::min(MC, M - ic);
          pack_a(A + ic * lda + pc, lda, mc, kc, apack.data());
          for (int64_t jr = 0; jr < nc; jr += NR) {
            const int64_t nr = std::min<int64_t>(NR, nc - jr);
            const float* Bp = bpack.data() + (jr / NR) * kc * NR;
            for (int64_t ir = 0; ir < mc; ir += MR) {
              const int64_t mr = std::min<int64_t>(MR, mc - ir);
              micro_kernel(apack.data() + (ir / MR) * kc * MR, Bp, kc, C + (ic + ir) * ldc + jc + jr, ldc, mr, nr,
                           accumulate);
            }
          }
        }
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
