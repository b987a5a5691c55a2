// Host-side runtime of tesseract_b200 (no CUDA): the parts of the serving / loading path that the reference keeps
// in C++ and that are slow or allocation-heavy in Python. Exposed to Python as the pybind11 module `_tsb_host`;
// every class here has a pure-Python twin with identical results that is used when the module is not built.
#pragma once

#include <cstdint>
#include <random>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

namespace tsbh {

// ---- sampling (src/models/Sampler.cpp of the reference: penalty -> greedy -> temperature -> top-k -> top-p -> draw)
struct SamplingParams {
  float temperature = 1.f;
  long long top_k = 0;
  float top_p = 1.f;
  float repetition_penalty = 1.f;
};

class HostSampler {
 public:
  explicit HostSampler(SamplingParams p, uint64_t seed) : params_(p), rng_(seed) {}
  void reseed(uint64_t seed) { rng_.seed(seed); }
  uint64_t next_u64() { return rng_(); }
  double uniform_double();
  // logits: V floats (copied); prev: token history for the repetition penalty. Returns the chosen token id.
  int sample(const float* logits, int64_t V, const int64_t* prev, int64_t n_prev);

 private:
  SamplingParams params_;
  std::mt19937_64 rng_;
  std::vector<float> work_, tmp_;      // scratch kept between calls: no half-megabyte allocation per sampled token
  std::vector<int32_t> order_;
  std::vector<double> e_;
  std::vector<char> keep_;
};

// ---- byte-level BPE merge loop (src/io/Tokenizer.cpp of the reference)
class BpeCore {
 public:
  // vocab: token string (in the byte-to-unicode alphabet, UTF-8) -> id; merges in rank order;
  // b2u[b] = UTF-8 string of the alphabet character that stands for byte b.
  BpeCore(const std::unordered_map<std::string, int32_t>& vocab,
          const std::vector<std::pair<std::string, std::string>>& merges, const std::vector<std::string>& b2u);
  std::vector<int32_t> encode_piece(const std::string& piece_bytes) const;

 private:
  struct PairHash {
    size_t operator()(const std::pair<int32_t, int32_t>& p) const {
      return (static_cast<uint64_t>(static_cast<uint32_t>(p.first)) << 32 | static_cast<uint32_t>(p.second)) *
             0x9E3779B97F4A7C15ull;
    }
  };
  int32_t intern(const std::string& s);
  std::vector<std::string> syms_;                          // interned symbol strings
  std::unordered_map<std::string, int32_t> sym_id_;
  std::vector<int32_t> sym_token_;                         // vocabulary id of a symbol or -1
  std::unordered_map<std::pair<int32_t, int32_t>, std::pair<int32_t, int32_t>, PairHash> ranks_;  // -> (rank, merged)
  std::unordered_map<std::string, int32_t> vocab_;
  int32_t byte_sym_[256];
};

// ---- KV block free list (LIFO, first allocation returns block 0)
class BlockAllocator {
 public:
  explicit BlockAllocator(int64_t num_blocks);
  int64_t allocate();
  void free(int64_t block);
  int64_t num_free() const { return static_cast<int64_t>(free_.size()); }
  int64_t num_blocks() const { return num_; }
  int64_t num_used() const { return num_ - num_free(); }

 private:
  int64_t num_;
  std::vector<int64_t> free_;
  std::vector<uint8_t> used_;
};

// ---- file IO: many byte ranges of one file read in parallel straight into caller memory (pinned buffers)
// Returns the number of bytes read; throws std::runtime_error on a short read.
int64_t read_ranges(const std::string& path, const std::vector<int64_t>& offsets, const std::vector<int64_t>& sizes,
                    const std::vector<uintptr_t>& dst, int threads);
// safetensors: returns (header JSON text, offset of the data section); validates the 8-byte length prefix.
std::pair<std::string, int64_t> safetensors_header(const std::string& path);

// ---- token mask of a byte automaton: allowed[i] = walking token i's bytes from `state` does not die
// table: states x 256 next-state ids (-1 = dead). tokens: concatenated bytes with offsets (n + 1 entries).
void token_mask(const int32_t* table, int64_t num_states, int32_t state, const uint8_t* bytes, const int64_t* offsets,
                int64_t n_tokens, uint8_t* allowed);

// ---- byte-level regex -> complete DFA (regex.cpp). table: states x 256 next-state ids (-1 = dead), state 0 is the
// start state, states numbered in breadth-first discovery order; accepting: one flag per state. Throws
// std::invalid_argument on a malformed pattern, std::length_error when the DFA would exceed max_states.
struct CompiledRegex {
  std::vector<int32_t> table;
  std::vector<uint8_t> accepting;
  int64_t num_nfa_states = 0;
};
CompiledRegex compile_regex(const std::string& pattern, int64_t max_states);

// ---- CPU FP32 GEMM (gemm_f32.cpp): C[M, N] = A[M, K] * op(B); b_nk = B stored [N, K] (a Linear weight)
bool gemm_avx2_supported();
int gemm_num_threads(int64_t M, int64_t N, int64_t K, int requested);
void gemm_f32(const float* A, int64_t lda, const float* B, int64_t ldb, bool b_nk, float* C, int64_t ldc, int64_t M,
              int64_t N, int64_t K, int threads);

// ---- CPU decode GEMV, INT8 weights x INT8 activations (gemv_int8.cpp)
bool gemv_vnni_supported();
// Per-vector symmetric quantisation: scale = absmax / 127 (1 for a zero vector); returns the scale.
float quantize_row_int8(const float* x, int64_t K, int8_t* xq);
void compute_row_sums(const int8_t* W, int64_t N, int64_t K, int32_t* rowsum);
// y[n] = xscale * wscale[n] * sum_k xq[k] * W[n,k] for rows [n_begin, n_end); rowsum may be null (scalar path).
void gemv_w8a8_range(const int8_t* W, const float* wscale, const int32_t* rowsum, const int8_t* xq, float xscale, float* y,
                     int64_t n_begin, int64_t n_end, int64_t K);
void gemv_w8a8(const int8_t* W, const float* wscale, const int32_t* rowsum, const int8_t* xq, float xscale, float* y,
               int64_t N, int64_t K, int threads);

}  // namespace tsbh
