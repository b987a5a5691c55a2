#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>
#include <stdexcept>

#include "host_runtime.hpp"

namespace tsbh {

double HostSampler::uniform_double() {
  // one 64-bit draw scaled by 2^-64, clamped below 1 (what libstdc++'s uniform_real_distribution<double> yields)
  double r = static_cast<double>(rng_()) / 18446744073709551616.0;
  if (r >= 1.0) r = std::nextafter(1.0, 0.0);
  return r;
}

int HostSampler::sample(const float* logits, int64_t V, const int64_t* prev, int64_t n_prev) {
  if (V <= 0) throw std::invalid_argument("sample: empty logits");
  work_.assign(logits, logits + V);
  float* w = work_.data();
  const float ninf = -std::numeric_limits<float>::infinity();
  auto argmax = [&]() {
    int64_t best = 0;
    for (int64_t i = 1; i < V; ++i)
      if (w[i] > w[best]) best = i;  // lowest index on ties
    return static_cast<int>(best);
  };
  if (params_.repetition_penalty != 1.f && n_prev > 0) {
    const float pen = params_.repetition_penalty;
    for (int64_t i = 0; i < n_prev; ++i) {
      const int64_t t = prev[i];
      if (t >= 0 && t < V) w[t] = w[t] > 0.f ? w[t] / pen : w[t] * pen;
    }
  }
  if (params_.temperature <= 1e-6f) return argmax();
  const float inv_t = 1.0f / params_.temperature;
  for (int64_t i = 0; i < V; ++i) w[i] *= inv_t;
  if (params_.top_k > 0 && params_.top_k < V) {
    std::vector<float>& tmp = tmp_;
    tmp.assign(work_.begin(), work_.end());
    std::nth_element(tmp.begin(), tmp.begin() + (V - params_.top_k), tmp.end());
    const float kth = tmp[V - params_.top_k];
    for (int64_t i = 0; i < V; ++i)
      if (w[i] < kth) w[i] = ninf;
  }
  bool have_e = false;
  if (params_.top_p < 1.f) {
    have_e = true;
    // The nucleus is a prefix of the order (value descending, index ascending on ties). Only that prefix is sorted:
    // candidates are all entries not below the K-th largest value (K grows until the prefix reaches top_p); the
    // probabilities come from one pass over the row in index order.
    float mx = w[0];
    for (int64_t i = 1; i < V; ++i) mx = std::max(mx, w[i]);
    e_.resize(V);
    double denom = 0.0;
    for (int64_t i = 0; i < V; ++i) {
      e_[i] = (w[i] != ninf) ? std::exp(static_cast<double>(w[i] - mx)) : 0.0;
      denom += e_[i];
    }
    int64_t cut = -1;
    for (int64_t K = 256;; K *= 8) {
      order_.clear();
      if (K >= V) {
        order_.resize(V);
        std::iota(order_.begin(), order_.end(), 0);
      } else {
        std::vector<float>& tmp = tmp_;
        tmp.assign(work_.begin(), work_.end());
        std::nth_element(tmp.begin(), tmp.begin() + (V - K), tmp.end());
        const float kth = tmp[V - K];
        for (int64_t i = 0; i < V; ++i)
          if (w[i] >= kth) order_.push_back(static_cast<int32_t>(i));
      }
      std::stable_sort(order_.begin(), order_.end(), [&](int32_t a, int32_t b) { return w[a] > w[b]; });
      double cum = 0.0;
      for (size_t i = 0; i < order_.size(); ++i) {
        cum += e_[order_[i]] / denom;
        if (w[order_[i]] != ninf && cum >= static_cast<double>(params_.top_p)) {
          cut = static_cast<int64_t>(i) + 1;
          break;
        }
      }
      if (cut >= 0 || static_cast<int64_t>(order_.size()) >= V) break;
    }
    if (cut >= 0) {
      std::vector<char>& keep = keep_;
      keep.assign(static_cast<size_t>(V), 0);
      for (int64_t i = 0; i < cut; ++i) keep[order_[i]] = 1;
      for (int64_t i = 0; i < V; ++i)
        if (!keep[i]) w[i] = ninf;
    }
  }
  double denom = 0.0;
  if (have_e) {
    // the largest entry always survives the nucleus cut, so the exponentials of the survivors are the ones already
    // computed; the dropped entries count as zero
    for (int64_t i = 0; i < V; ++i) {
      if (w[i] == ninf) e_[i] = 0.0;
      denom += e_[i];
    }
  } else {
    float maxv = w[0];
    for (int64_t i = 1; i < V; ++i) maxv = std::max(maxv, w[i]);
    e_.resize(V);
    for (int64_t i = 0; i < V; ++i) {
      e_[i] = (w[i] != ninf) ? std::exp(static_cast<double>(w[i] - maxv)) : 0.0;
      denom += e_[i];
    }
  }
  if (!(denom > 0.0)) throw std::runtime_error("sample: degenerate distribution");
  double rem = uniform_double() * denom;
  for (int64_t i = 0; i < V; ++i) {
    rem -= e_[i];
    if (w[i] != ninf && rem <= 0.0) return static_cast<int>(i);
  }
  return argmax();
}

// ---------------------------------------------------------------------------------------------- block allocator
BlockAllocator::BlockAllocator(int64_t num_blocks) : num_(num_blocks) {
  if (num_blocks <= 0) throw std::invalid_argument("BlockAllocator needs at least one block");
  free_.reserve(num_blocks);
  for (int64_t b = num_blocks - 1; b >= 0; --b) free_.push_back(b);
  used_.assign(num_blocks, 0);
}
int64_t BlockAllocator::allocate() {
  if (free_.empty()) throw std::runtime_error("BlockAllocator: out of KV blocks");
  const int64_t b = free_.back();
  free_.pop_back();
  used_[b] = 1;
  return b;
}
void BlockAllocator::free(int64_t block) {
  if (block < 0 || block >= num_ || !used_[block])
    throw std::runtime_error("BlockAllocator: double free or foreign block " + std::to_string(block));
  used_[block] = 0;
  free_.push_back(block);
}

// ---------------------------------------------------------------------------------------------- automaton mask
void token_mask(const int32_t* table, int64_t num_states, int32_t state, const uint8_t* bytes, const int64_t* offsets,
                int64_t n_tokens, uint8_t* allowed) {
  // tokens are independent: a large vocabulary is split over the OpenMP team
#pragma omp parallel for schedule(static) if (n_tokens >= 16384)
  for (int64_t i = 0; i < n_tokens; ++i) {
    int32_t s = state;
    const int64_t b0 = offsets[i], b1 = offsets[i + 1];
    if (b1 == b0) {
      allowed[i] = 0;
      continue;
    }
    for (int64_t j = b0; j < b1 && s >= 0; ++j) s = (s < num_states) ? table[static_cast<int64_t>(s) * 256 + bytes[j]] : -1;
    allowed[i] = s >= 0;
  }
}

}  // namespace tsbh
