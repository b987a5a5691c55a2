#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <stdexcept>
#include <thread>

#include "host_runtime.hpp"

namespace tsbh {

// ---------------------------------------------------------------------------------------------- BPE
int32_t BpeCore::intern(const std::string& s) {
  auto it = sym_id_.find(s);
  if (it != sym_id_.end()) return it->second;
  const int32_t id = static_cast<int32_t>(syms_.size());
  syms_.push_back(s);
  sym_id_.emplace(s, id);
  auto v = vocab_.find(s);
  sym_token_.push_back(v == vocab_.end() ? -1 : v->second);
  return id;
}

BpeCore::BpeCore(const std::unordered_map<std::string, int32_t>& vocab,
                 const std::vector<std::pair<std::string, std::string>>& merges, const std::vector<std::string>& b2u)
    : vocab_(vocab) {
  if (b2u.size() != 256) throw std::invalid_argument("BpeCore: the byte alphabet needs 256 entries");
  for (int b = 0; b < 256; ++b) byte_sym_[b] = intern(b2u[b]);
  for (size_t r = 0; r < merges.size(); ++r) {
    const int32_t a = intern(merges[r].first), b = intern(merges[r].second);
    const int32_t m = intern(merges[r].first + merges[r].second);
    ranks_.emplace(std::make_pair(a, b), std::make_pair(static_cast<int32_t>(r), m));  // first rank of a pair wins
  }
}

static size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : 4; }

std::vector<int32_t> BpeCore::encode_piece(const std::string& piece) const {
  std::vector<int32_t> syms(piece.size());
  for (size_t i = 0; i < piece.size(); ++i) syms[i] = byte_sym_[static_cast<unsigned char>(piece[i])];
  while (syms.size() > 1) {
    int32_t best_rank = -1, best_a = 0, best_b = 0, best_m = 0;
    for (size_t i = 0; i + 1 < syms.size(); ++i) {
      auto it = ranks_.find(std::make_pair(syms[i], syms[i + 1]));
      if (it != ranks_.end() && (best_rank < 0 || it->second.first < best_rank)) {
        best_rank = it->second.first;
        best_a = syms[i];
        best_b = syms[i + 1];
        best_m = it->second.second;
      }
    }
    if (best_rank < 0) break;
    std::vector<int32_t> merged;
    merged.reserve(syms.size());
    for (size_t i = 0; i < syms.size();) {
      if (i + 1 < syms.size() && syms[i] == best_a && syms[i + 1] == best_b) {
        merged.push_back(best_m);
        i += 2;
      } else {
        merged.push_back(syms[i]);
        i += 1;
      }
    }
    syms.swap(merged);
  }
  std::vector<int32_t> ids;
  ids.reserve(syms.size());
  for (int32_t s : syms) {
    if (sym_token_[s] >= 0) {
      ids.push_back(sym_token_[s]);
      continue;
    }
    const std::string& str = syms_[s];  // unknown merged symbol: fall back to its single characters
    for (size_t i = 0; i < str.size();) {
      const size_t n = utf8_len(static_cast<unsigned char>(str[i]));
      auto v = vocab_.find(str.substr(i, n));
      if (v != vocab_.end()) ids.push_back(v->second);
      i += n;
    }
  }
  return ids;
}

// ---------------------------------------------------------------------------------------------- file IO
int64_t read_ranges(const std::string& path, const std::vector<int64_t>& offsets, const std::vector<int64_t>& sizes,
                    const std::vector<uintptr_t>& dst, int threads) {
  if (offsets.size() != sizes.size() || offsets.size() != dst.size())
    throw std::invalid_argument("read_ranges: offsets, sizes and destinations differ in length");
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error("read_ranges: cannot open " + path);
  // cut the ranges into pieces of at most 8 MiB so that a few huge tensors still spread over all threads
  struct Piece {
    int64_t off, size;
    uintptr_t dst;
  };
  std::vector<Piece> pieces;
  constexpr int64_t kPiece = 8ll << 20;
  for (size_t i = 0; i < offsets.size(); ++i)
    for (int64_t o = 0; o < sizes[i]; o += kPiece) pieces.push_back({offsets[i] + o, std::min(kPiece, sizes[i] - o), dst[i] + static_cast<uintptr_t>(o)});
  std::atomic<size_t> next{0};
  std::atomic<int64_t> total{0};
  std::atomic<bool> failed{false};
  auto worker = [&]() {
    for (;;) {
      const size_t i = next.fetch_add(1);
      if (i >= pieces.size() || failed.load()) return;
      int64_t done = 0;
      while (done < pieces[i].size) {
        const ssize_t n = ::pread(fd, reinterpret_cast<char*>(pieces[i].dst) + done, static_cast<size_t>(pieces[i].size - done),
                                  static_cast<off_t>(pieces[i].off + done));
        if (n <= 0) {
          failed.store(true);
          return;
        }
        done += n;
      }
      total.fetch_add(done);
    }
  };
  const int nt = std::max(1, std::min<int>(threads, static_cast<int>(pieces.size())));
  std::vector<std::thread> pool;
  for (int t = 1; t < nt; ++t) pool.emplace_back(worker);
  worker();
  for (auto& t : pool) t.join();
  ::close(fd);
  if (failed.load()) throw std::runtime_error("read_ranges: short read from " + path);
  return total.load();
}

std::pair<std::string, int64_t> safetensors_header(const std::string& path) {
  const int fd = ::open(path.c_str(), O_RDONLY);
  if (fd < 0) throw std::runtime_error("safetensors: cannot open " + path);
  struct stat st;
  ::fstat(fd, &st);
  unsigned char len8[8];
  if (::pread(fd, len8, 8, 0) != 8) {
    ::close(fd);
    throw std::runtime_error("safetensors: file shorter than its 8-byte header length");
  }
  uint64_t n = 0;
  for (int i = 7; i >= 0; --i) n = (n << 8) | len8[i];
  if (n == 0 || n > static_cast<uint64_t>(st.st_size) - 8 || n > (100ull << 20)) {
    ::close(fd);
    throw std::runtime_error("safetensors: implausible header length");
  }
  std::string header(n, '\0');
  const ssize_t got = ::pread(fd, header.data(), n, 8);
  ::close(fd);
  if (got != static_cast<ssize_t>(n)) throw std::runtime_error("safetensors: truncated header");
  return {header, static_cast<int64_t>(8 + n)};
}

}  // namespace tsbh
