// Byte-level regular expressions compiled to a complete DFA table, for grammar-constrained decoding.
//
// The subset is the one the Python twin (models/structured.py) accepts: literals (UTF-8, a multi-byte character is a
// byte sequence), `.`, escapes \d \D \w \W \s \S \n \t \r \f \v and escaped punctuation, classes [a-z0-9] / [^...],
// groups, alternation, * + ? and counted {m} {m,} {m,n}. Matching is anchored at both ends.
//
// Thompson construction (byte sets as 256-bit masks on the edges), then eager subset construction in breadth-first
// order -- states numbered as they are discovered, bytes visited 0 .. 255 -- so the table is a pure function of the
// pattern and equals what the twin's dfa_table() builds. The table is what the token-mask kernel walks
// (token_mask in sampler.cpp): 256 next-state ids per state, -1 = dead.
// The reference compiles its grammars on the host in C++ as well (src/models/StructuredDecoding.cpp:400-468).
#include <algorithm>
#include <bitset>
#include <cctype>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "host_runtime.hpp"

namespace tsbh {
namespace {

using ByteSet = std::bitset<256>;

struct Nfa {
  std::vector<std::vector<int>> eps;
  std::vector<std::vector<std::pair<ByteSet, int>>> trans;
  int add() {
    eps.emplace_back();
    trans.emplace_back();
    return static_cast<int>(eps.size()) - 1;
  }
};

struct Frag {
  int s, e;
};

ByteSet range_set(int lo, int hi) {
  ByteSet b;
  for (int i = lo; i <= hi; ++i) b.set(static_cast<size_t>(i));
  return b;
}
ByteSet digit_set() { return range_set('0', '9'); }
ByteSet word_set() { return range_set('0', '9') | range_set('A', 'Z') | range_set('a', 'z') | range_set('_', '_'); }
ByteSet space_set() {
  ByteSet b;
  for (int c : {32, 9, 10, 13, 11, 12}) b.set(static_cast<size_t>(c));
  return b;
}

// Bytes of the UTF-8 character that starts at p[i] (1 .. 4; a stray continuation byte counts as one character).
int char_len(const std::string& p, size_t i) {
  const unsigned char c = static_cast<unsigned char>(p[i]);
  int n = c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1;
  if (i + static_cast<size_t>(n) > p.size()) n = static_cast<int>(p.size() - i);
  return n;
}

class Parser {
 public:
  Parser(const std::string& pattern, size_t begin, size_t end, Nfa& nfa) : p_(pattern), i_(begin), end_(end), nfa_(nfa) {}

  Frag parse() {
    const Frag f = alt();
    if (i_ != end_) throw std::invalid_argument("regex: unexpected '" + p_.substr(i_, 1) + "' at " + std::to_string(i_));
    return f;
  }
  Frag atom();

 private:
  bool more() const { return i_ < end_; }
  char peek() const { return p_[i_]; }

  Frag alt() {
    std::vector<Frag> frags{cat()};
    while (more() && peek() == '|') {
      ++i_;
      frags.push_back(cat());
    }
    if (frags.size() == 1) return frags[0];
    const int s = nfa_.add(), e = nfa_.add();
    for (const Frag& f : frags) {
      nfa_.eps[s].push_back(f.s);
      nfa_.eps[f.e].push_back(e);
    }
    return {s, e};
  }

  Frag cat() {
    const int s = nfa_.add();
    int cur = s;
    while (more() && peek() != '|' && peek() != ')') {
      const Frag f = rep();
      nfa_.eps[cur].push_back(f.s);
      cur = f.e;
    }
    return {s, cur};
  }

  static long parse_count(const std::string& text) {
    size_t a = 0, b = text.size();
    while (a < b && std::isspace(static_cast<unsigned char>(text[a]))) ++a;
    while (b > a && std::isspace(static_cast<unsigned char>(text[b - 1]))) --b;
    if (a == b) throw std::invalid_argument("regex: bad counted quantifier");
    long v = 0;
    for (size_t k = a; k < b; ++k) {
      if (!std::isdigit(static_cast<unsigned char>(text[k]))) throw std::invalid_argument("regex: bad counted quantifier");
      v = v * 10 + (text[k] - '0');
      if (v > 100000) throw std::invalid_argument("regex: counted quantifier too large");
    }
    return v;
  }

  Frag rep() {
    const size_t a0 = i_;
    Frag frag = atom();
    const size_t a1 = i_;
    while (more() && (peek() == '*' || peek() == '+' || peek() == '?' || peek() == '{')) {
      const char c = peek();
      if (c == '{') {
        const size_t j = p_.find('}', i_);
        if (j == std::string::npos || j >= end_) throw std::invalid_argument("regex: unterminated {");
        const std::string body = p_.substr(i_ + 1, j - i_ - 1);
        i_ = j + 1;
        long lo, hi;   // hi < 0: unbounded
        const size_t comma = body.find(',');
        if (comma != std::string::npos) {
          lo = parse_count(body.substr(0, comma));
          const std::string hs = body.substr(comma + 1);
          bool blank = true;
          for (char ch : hs) blank = blank && std::isspace(static_cast<unsigned char>(ch));
          hi = blank ? -1 : parse_count(hs);
        } else {
          lo = hi = parse_count(body);
        }
        if (hi >= 0 && hi < lo) throw std::invalid_argument("regex: bad counted quantifier");
        frag = counted(a0, a1, lo, hi);
        continue;
      }
      ++i_;
      const int s = nfa_.add(), e = nfa_.add();
      nfa_.eps[s].push_back(frag.s);
      nfa_.eps[frag.e].push_back(e);
      if (c == '*' || c == '?') nfa_.eps[s].push_back(e);
      if (c == '*' || c == '+') nfa_.eps[frag.e].push_back(frag.s);
      frag = {s, e};
    }
    return frag;
  }

  // A fresh copy of the atom whose source is p_[a0, a1): counted repetition unrolls the atom.
  Frag again(size_t a0, size_t a1) {
    Parser sub(p_, a0, a1, nfa_);
    return sub.atom();
  }

  Frag counted(size_t a0, size_t a1, long lo, long hi) {
    const int s = nfa_.add();
    int cur = s;
    for (long k = 0; k < lo; ++k) {
      const Frag f = again(a0, a1);
      nfa_.eps[cur].push_back(f.s);
      cur = f.e;
    }
    if (hi < 0) {
      const Frag f = again(a0, a1);
      nfa_.eps[cur].push_back(f.s);
      nfa_.eps[f.e].push_back(f.s);
      const int e = nfa_.add();
      nfa_.eps[cur].push_back(e);
      nfa_.eps[f.e].push_back(e);
      return {s, e};
    }
    const int e = nfa_.add();
    nfa_.eps[cur].push_back(e);
    for (long k = 0; k < hi - lo; ++k) {
      const Frag f = again(a0, a1);
      nfa_.eps[cur].push_back(f.s);
      cur = f.e;
      nfa_.eps[cur].push_back(e);
    }
    return {s, e};
  }

  // The set an escape stands for; `len` = bytes of the escaped character (a multi-byte one stands for nothing).
  ByteSet escape_set(size_t at, int len) const {
    if (len != 1) return ByteSet();
    const char c = p_[at];
    switch (c) {
      case 'd': return digit_set();
      case 'D': return ~digit_set();
      case 'w': return word_set();
      case 'W': return ~word_set();
      case 's': return space_set();
      case 'S': return ~space_set();
      case 'n': return range_set(10, 10);
      case 't': return range_set(9, 9);
      case 'r': return range_set(13, 13);
      case 'f': return range_set(12, 12);
      case 'v': return range_set(11, 11);
      default: return range_set(static_cast<unsigned char>(c), static_cast<unsigned char>(c));
    }
  }

  Frag byte_edge(const ByteSet& set) {
    const int s = nfa_.add(), e = nfa_.add();
    nfa_.trans[s].emplace_back(set, e);
    return {s, e};
  }

  static int first_of(const ByteSet& b) {
    for (int i = 0; i < 256; ++i)
      if (b.test(static_cast<size_t>(i))) return i;
    throw std::invalid_argument("regex: empty escape in class range");
  }

  ByteSet klass() {
    ++i_;   // [
    bool neg = false;
    if (more() && peek() == '^') {
      neg = true;
      ++i_;
    }
    ByteSet items;
    bool first = true;
    while (true) {
      if (!more()) throw std::invalid_argument("regex: unterminated [");
      const char c = peek();
      if (c == ']' && !first) {
        ++i_;
        break;
      }
      first = false;
      int lo;
      if (c == '\\') {
        if (i_ + 1 >= end_) throw std::invalid_argument("regex: dangling backslash");
        const int len = char_len(p_, i_ + 1);
        const ByteSet es = escape_set(i_ + 1, len);
        i_ += 1 + static_cast<size_t>(len);
        if (es.count() != 1) {
          items |= es;
          continue;
        }
        lo = first_of(es);
      } else {
        const int len = char_len(p_, i_);
        if (len != 1) {
          for (int k = 0; k < len; ++k) items.set(static_cast<unsigned char>(p_[i_ + static_cast<size_t>(k)]));
          i_ += static_cast<size_t>(len);
          continue;
        }
        lo = static_cast<unsigned char>(c);
        ++i_;
      }
      if (more() && peek() == '-' && i_ + 1 < end_ && p_[i_ + 1] != ']') {
        ++i_;
        int hi;
        if (peek() == '\\') {
          if (i_ + 1 >= end_) throw std::invalid_argument("regex: dangling backslash");
          const int len = char_len(p_, i_ + 1);
          hi = first_of(escape_set(i_ + 1, len));
          i_ += 1 + static_cast<size_t>(len);
        } else {
          hi = static_cast<unsigned char>(peek());
          i_ += static_cast<size_t>(char_len(p_, i_));
        }
        if (hi < lo) throw std::invalid_argument("regex: reversed range in class");
        items |= range_set(lo, hi);
      } else {
        items.set(static_cast<size_t>(lo));
      }
    }
    return neg ? ~items : items;
  }

  const std::string& p_;
  size_t i_, end_;
  Nfa& nfa_;
};

Frag Parser::atom() {
  if (!more()) throw std::invalid_argument("regex: unexpected end of pattern");
  const char c = peek();
  if (c == '(') {
    ++i_;
    const Frag f = alt();
    if (!more() || peek() != ')') throw std::invalid_argument("regex: missing )");
    ++i_;
    return f;
  }
  if (c == '[') return byte_edge(klass());
  if (c == '.') {
    ++i_;
    return byte_edge(~ByteSet());
  }
  if (c == '\\') {
    if (i_ + 1 >= end_) throw std::invalid_argument("regex: dangling backslash");
    const int len = char_len(p_, i_ + 1);
    const ByteSet es = escape_set(i_ + 1, len);
    i_ += 1 + static_cast<size_t>(len);
    return byte_edge(es);
  }
  if (c == '*' || c == '+' || c == '?' || c == '{') throw std::invalid_argument("regex: nothing to repeat at " + std::to_string(i_));
  const int len = char_len(p_, i_);
  const int s = nfa_.add();
  int cur = s;
  for (int k = 0; k < len; ++k) {
    const int nxt = nfa_.add();
    nfa_.trans[cur].emplace_back(range_set(static_cast<unsigned char>(p_[i_ + static_cast<size_t>(k)]),
                                           static_cast<unsigned char>(p_[i_ + static_cast<size_t>(k)])), nxt);
    cur = nxt;
  }
  i_ += static_cast<size_t>(len);
  return {s, cur};
}

// Epsilon closure of `seed` (any order), returned sorted: the canonical name of a DFA state.
std::vector<int> closure(const Nfa& nfa, std::vector<int> seed, std::vector<char>& mark) {
  std::vector<int> out;
  std::vector<int> stack;
  for (int s : seed)
    if (!mark[static_cast<size_t>(s)]) {
      mark[static_cast<size_t>(s)] = 1;
      out.push_back(s);
      stack.push_back(s);
    }
  while (!stack.empty()) {
    const int s = stack.back();
    stack.pop_back();
    for (int t : nfa.eps[static_cast<size_t>(s)])
      if (!mark[static_cast<size_t>(t)]) {
        mark[static_cast<size_t>(t)] = 1;
        out.push_back(t);
        stack.push_back(t);
      }
  }
  for (int s : out) mark[static_cast<size_t>(s)] = 0;
  std::sort(out.begin(), out.end());
  return out;
}

}  // namespace

CompiledRegex compile_regex(const std::string& pattern, int64_t max_states) {
  Nfa nfa;
  Parser parser(pattern, 0, pattern.size(), nfa);
  const Frag whole = parser.parse();
  std::vector<char> mark(nfa.eps.size(), 0);
  std::map<std::vector<int>, int32_t> ids;
  std::vector<std::vector<int>> sets;
  auto intern = [&](std::vector<int> st) -> int32_t {
    auto it = ids.find(st);
    if (it != ids.end()) return it->second;
    if (static_cast<int64_t>(sets.size()) >= max_states) throw std::length_error("regex: more DFA states than max_states");
    const int32_t id = static_cast<int32_t>(sets.size());
    ids.emplace(st, id);
    sets.push_back(std::move(st));
    return id;
  };
  intern(closure(nfa, {whole.s}, mark));
  CompiledRegex out;
  std::vector<std::vector<int>> by_byte(256);
  for (size_t q = 0; q < sets.size(); ++q) {          // breadth first: `sets` grows while it is walked
    for (auto& v : by_byte) v.clear();
    const std::vector<int> cur = sets[q];             // a copy: intern() may reallocate `sets`
    for (int s : cur)
      for (const auto& edge : nfa.trans[static_cast<size_t>(s)])
        for (int b = 0; b < 256; ++b)
          if (edge.first.test(static_cast<size_t>(b))) by_byte[static_cast<size_t>(b)].push_back(edge.second);
    out.table.resize((q + 1) * 256);
    for (int b = 0; b < 256; ++b) {
      auto& tg = by_byte[static_cast<size_t>(b)];
      out.table[q * 256 + static_cast<size_t>(b)] = tg.empty() ? -1 : intern(closure(nfa, tg, mark));
    }
  }
  out.accepting.resize(sets.size());
  for (size_t q = 0; q < sets.size(); ++q)
    out.accepting[q] = std::binary_search(sets[q].begin(), sets[q].end(), whole.e) ? 1 : 0;
  out.num_nfa_states = static_cast<int64_t>(nfa.eps.size());
  return out;
}

}  // namespace tsbh
