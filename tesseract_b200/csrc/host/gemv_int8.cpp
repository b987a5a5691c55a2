// CPU decode GEMV with INT8 weights and INT8 activations (W8A8): y[n] = xscale * wscale[n] * sum_k xq[k] * W[n,k].
// The AVX-512-VNNI path feeds vpdpbusd, which multiplies UNSIGNED bytes by signed bytes, so the activation is
// biased by +128 into u8 and the bias is taken out again with the precomputed row sums of W:
//   sum_k (xq[k] + 128) * W[n,k] = sum_k xq[k] * W[n,k] + 128 * rowsum[n].
// A scalar path gives the same integers on CPUs without VNNI. Behaviour of the reference's CPU decode kernels
// (src/ops/cpu/GemvVnni.cpp:33-107; checked by tests/ops/test_gemv_vnni.cpp).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif

#ifdef _OPENMP
#include <omp.h>
#endif

#include "host_runtime.hpp"

namespace tsbh {

bool gemv_vnni_supported() {
#if defined(__x86_64__)
  static const bool ok = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
                         __builtin_cpu_supports("avx512vnni");
  return ok;
#else
  return false;
#endif
}

float quantize_row_int8(const float* x, int64_t K, int8_t* xq) {
  float amax = 0.f;
  for (int64_t k = 0; k < K; ++k) amax = std::max(amax, std::fabs(x[k]));
  if (amax <= 0.f) {   // all-zero vector: zeros with scale 0 (src/ops/cpu/GemvVnni.cpp:126-133), so y = 0 exactly
    for (int64_t k = 0; k < K; ++k) xq[k] = 0;
    return 0.f;
  }
  const float scale = amax / 127.f;
  const float inv = 1.f / scale;
  for (int64_t k = 0; k < K; ++k) {
    const float r = std::nearbyint(x[k] * inv);
    xq[k] = static_cast<int8_t>(std::min(127.f, std::max(-127.f, r)));
  }
  return scale;
}

void compute_row_sums(const int8_t* W, int64_t N, int64_t K, int32_t* rowsum) {
  for (int64_t n = 0; n < N; ++n) {
    int32_t s = 0;
    const int8_t* w = W + n * K;
    for (int64_t k = 0; k < K; ++k) s += w[k];
    rowsum[n] = s;
  }
}

static void rows_scalar(const int8_t* W, const float* wscale, const int8_t* xq, float xscale, float* y, int64_t n0,
                        int64_t n1, int64_t K) {
  for (int64_t n = n0; n < n1; ++n) {
    const int8_t* w = W + n * K;
    int32_t acc = 0;
    for (int64_t k = 0; k < K; ++k) acc += static_cast<int32_t>(xq[k]) * static_cast<int32_t>(w[k]);
    y[n] = xscale * wscale[n] * static_cast<float>(acc);
  }
}

#if defined(__x86_64__)
// xu = xq + 128 as unsigned bytes, padded with 128 (the bias of a zero activation, matched by zero weight bytes
// that the masked load supplies) so that the tail needs no scalar loop.
__attribute__((target("avx512f,avx512bw,avx512vnni"))) static void rows_vnni(const int8_t* W, const float* wscale,
                                                                             const int32_t* rowsum, const uint8_t* xu,
                                                                             float xscale, float* y, int64_t n0, int64_t n1,
                                                                             int64_t K) {
  const int64_t K256 = K & ~int64_t(255);
  const int64_t K64 = K & ~int64_t(63);
  const int tail = static_cast<int>(K - K64);
  const __mmask64 tail_mask = tail ? (~0ULL >> (64 - tail)) : 0;
  for (int64_t n = n0; n < n1; ++n) {
    const int8_t* w = W + n * K;
    __m512i a0 = _mm512_setzero_si512(), a1 = a0, a2 = a0, a3 = a0;
    int64_t k = 0;
    for (; k < K256; k += 256) {   // four independent chains hide the latency of vpdpbusd
      a0 = _mm512_dpbusd_epi32(a0, _mm512_loadu_si512(xu + k), _mm512_loadu_si512(w + k));
      a1 = _mm512_dpbusd_epi32(a1, _mm512_loadu_si512(xu + k + 64), _mm512_loadu_si512(w + k + 64));
      a2 = _mm512_dpbusd_epi32(a2, _mm512_loadu_si512(xu + k + 128), _mm512_loadu_si512(w + k + 128));
      a3 = _mm512_dpbusd_epi32(a3, _mm512_loadu_si512(xu + k + 192), _mm512_loadu_si512(w + k + 192));
    }
    for (; k < K64; k += 64) a0 = _mm512_dpbusd_epi32(a0, _mm512_loadu_si512(xu + k), _mm512_loadu_si512(w + k));
    if (tail) a1 = _mm512_dpbusd_epi32(a1, _mm512_loadu_si512(xu + k), _mm512_maskz_loadu_epi8(tail_mask, w + k));
    const int32_t biased = _mm512_reduce_add_epi32(_mm512_add_epi32(_mm512_add_epi32(a0, a1), _mm512_add_epi32(a2, a3)));
    y[n] = xscale * wscale[n] * static_cast<float>(biased - 128 * rowsum[n]);
  }
}
#endif

void gemv_w8a8_range(const int8_t* W, const float* wscale, const int32_t* rowsum, const int8_t* xq, float xscale, float* y,
                     int64_t n_begin, int64_t n_end, int64_t K) {
  if (n_begin >= n_end || K <= 0) return;
#if defined(__x86_64__)
  if (gemv_vnni_supported() && rowsum != nullptr) {
    const int64_t Kp = (K + 63) & ~int64_t(63);
    std::vector<uint8_t> xu(static_cast<size_t>(Kp), 128);
    for (int64_t k = 0; k < K; ++k) xu[k] = static_cast<uint8_t>(static_cast<int>(xq[k]) + 128);
    rows_vnni(W, wscale, rowsum, xu.data(), xscale, y, n_begin, n_end, K);
    return;
  }
#endif
  rows_scalar(W, wscale, xq, xscale, y, n_begin, n_end, K);
}

void gemv_w8a8(const int8_t* W, const float* wscale, const int32_t* rowsum, const int8_t* xq, float xscale, float* y,
               int64_t N, int64_t K, int threads) {
  const int64_t work = N * K;
  int t = threads > 0 ? threads : static_cast<int>(std::min<unsigned>(16, std::max(1u, std::thread::hardware_concurrency())));
#ifdef _OPENMP
  t = std::min(t, omp_get_max_threads());
#else
  t = 1;
#endif
  if (work < (int64_t(1) << 20) || N < 2 * t) t = 1;      // small matrices: one thread beats waking the others
  if (t == 1) {
    gemv_w8a8_range(W, wscale, rowsum, xq, xscale, y, 0, N, K);
    return;
  }
  // the OpenMP team persists between calls (a decode step makes hundreds of them; creating threads per call cost
  // several times the product itself); the biased activation vector is built once and shared
#if defined(__x86_64__)
  const bool vnni = gemv_vnni_supported() && rowsum != nullptr;
  std::vector<uint8_t> xu;
  if (vnni) {
    const int64_t Kp = (K + 63) & ~int64_t(63);
    xu.assign(static_cast<size_t>(Kp), 128);
    for (int64_t k = 0; k < K; ++k) xu[k] = static_cast<uint8_t>(static_cast<int>(xq[k]) + 128);
  }
#else
  const bool vnni = false;
#endif
  const int64_t per = (N + t - 1) / t;
#pragma omp parallel for schedule(static, 1) num_threads(t)
  for (int i = 0; i < t; ++i) {
    const int64_t a = i * per, b = std::min<int64_t>(N, a + per);
    if (a >= b) continue;
#if defined(__x86_64__)
    if (vnni) {
      rows_vnni(W, wscale, rowsum, xu.data(), xscale, y, a, b, K);
      continue;
    }
#endif
    rows_scalar(W, wscale, xq, xscale, y, a, b, K);
  }
}

}  // namespace tsbh
