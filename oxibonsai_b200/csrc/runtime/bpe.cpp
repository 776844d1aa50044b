// Byte-pair-encoding merge engine (host).
//
// The reference ships a pure-Rust tokenizer (crates/oxibonsai-tokenizer/src/bpe.rs:19-216: merge table, greedy
// lowest-rank merging, `<0xHH>` byte fallback).  This is the same algorithm on integer ids: the caller
// pre-tokenises text and hands over the pieces (or the initial token ids of one piece); the engine repeatedly merges
// the adjacent pair with the lowest merge rank until none applies.  A piece cache makes
// repeated words O(1).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Bpe {
  std::unordered_map<uint64_t, std::pair<uint32_t, uint32_t>> merges;  // (a,b) -> (rank, merged id)
  std::unordered_map<std::string, std::vector<uint32_t>> cache;
  std::mutex mu;
  size_t cache_cap = 1 << 18;
};

inline uint64_t key(uint32_t a, uint32_t b) { return (uint64_t)a << 32 | b; }

// Lowest rank first, leftmost first among equals.  The tokens sit in a doubly linked list over their first positions and the
// candidate pairs in a heap; an entry that no longer describes its two neighbours is skipped when it comes up.  O(n log n)
// in the piece's length (a piece without a split point can be as long as the request).
void merge_piece(const Bpe& m, std::vector<uint32_t>& ids) {
  const size_t n = ids.size();
  if (n < 2) return;
  struct Cand { uint32_t rank, pos, a, b, merged; };
  auto later = [](const Cand& x, const Cand& y) { return x.rank != y.rank ? x.rank > y.rank : x.pos > y.pos; };
  std::vector<Cand> heap;
  heap.reserve(n);
  std::vector<int64_t> prev(n), next(n);
  for (size_t i = 0; i < n; ++i) {
    prev[i] = (int64_t)i - 1;
    next[i] = i + 1 < n ? (int64_t)i + 1 : -1;
  }
  auto consider = [&](int64_t i, bool sift) {
    if (i < 0 || next[i] < 0) return;
    auto it = m.merges.find(key(ids[i], ids[next[i]]));
    if (it == m.merges.end()) return;
    heap.push_back({it->second.first, (uint32_t)i, ids[i], ids[next[i]], it->second.second});
    if (sift) std::push_heap(heap.begin(), heap.end(), later);
  };
  for (size_t i = 0; i + 1 < n; ++i) consider((int64_t)i, false);
  std::make_heap(heap.begin(), heap.end(), later);
  std::vector<uint8_t> gone(n, 0);
  size_t left = n;
  while (!heap.empty()) {
    std::pop_heap(heap.begin(), heap.end(), later);
    const Cand c = heap.back();
    heap.pop_back();
    const int64_t i = c.pos, j = gone[c.pos] ? -1 : next[c.pos];
    if (j < 0 || ids[i] != c.a || ids[j] != c.b) continue;
    ids[i] = c.merged;
    gone[j] = 1;
    next[i] = next[j];
    if (next[j] >= 0) prev[next[j]] = i;
    --left;
    consider(prev[i], true);
    consider(i, true);
  }
  if (left == n) return;
  size_t w = 0;
  for (size_t i = 0; i < n; ++i)
    if (!gone[i]) ids[w++] = ids[i];
  ids.resize(w);
}

}  // namespace

extern "C" {

// pairs: n x {left id, right id, merged id}; rank = index
void* bbpe_new(const uint32_t* pairs, uint64_t n) {
  Bpe* m = new Bpe();
  m->merges.reserve(n * 2);
  for (uint64_t i = 0; i < n; ++i) {
    uint64_t k = key(pairs[3 * i], pairs[3 * i + 1]);
    if (!m->merges.count(k)) m->merges.emplace(k, std::make_pair((uint32_t)i, pairs[3 * i + 2]));
  }
  return m;
}
void bbpe_free(void* h) { delete static_cast<Bpe*>(h); }

// ids: initial ids of one pre-tokenised piece (in/out, capacity n).  Returns the merged length.
uint64_t bbpe_merge(void* h, uint32_t* ids, uint64_t n) {
  Bpe* m = static_cast<Bpe*>(h);
  std::string k(reinterpret_cast<const char*>(ids), n * 4);
  {
    std::lock_guard<std::mutex> g(m->mu);
    auto it = m->cache.find(k);
    if (it != m->cache.end()) {
      std::memcpy(ids, it->second.data(), it->second.size() * 4);
      return it->second.size();
    }
  }
  std::vector<uint32_t> v(ids, ids + n);
  merge_piece(*m, v);
  std::memcpy(ids, v.data(), v.size() * 4);
  {
    std::lock_guard<std::mutex> g(m->mu);
    if (m->cache.size() < m->cache_cap) m->cache.emplace(std::move(k), v);
  }
  return v.size();
}

// bytes: the UTF-8 text of one segment; ends[i]: the offset one past piece i (pieces tile the segment in order);
// byte_id[256]: the initial token of each byte (negative: the vocabulary lacks it, the byte is dropped).  Writes the token
// ids of all pieces to out (capacity cap: the segment's length always suffices) and returns their number.
uint64_t bbpe_encode(void* h, const uint8_t* bytes, const uint64_t* ends, uint64_t n_pieces, const int32_t* byte_id, uint32_t* out,
                     uint64_t cap) {
  Bpe* m = static_cast<Bpe*>(h);
  uint64_t w = 0, begin = 0;
  std::vector<uint32_t> v;
  std::string k;
  for (uint64_t p = 0; p < n_pieces; ++p) {
    const uint64_t end = ends[p];
    if (end < begin) return w;                                   // malformed offsets: stop rather than read backwards
    v.clear();
    for (uint64_t i = begin; i < end; ++i)
      if (byte_id[bytes[i]] >= 0) v.push_back((uint32_t)byte_id[bytes[i]]);
    begin = end;
    if (v.size() > 1) {
      const bool cached = v.size() <= 64;                        // words; a long run is not worth a cache entry
      bool hit = false;
      if (cached) {
        k.assign(reinterpret_cast<const char*>(v.data()), v.size() * 4);
        std::lock_guard<std::mutex> g(m->mu);
        auto it = m->cache.find(k);
        if (it != m->cache.end()) {
          v = it->second;
          hit = true;
        }
      }
      if (!hit) {
        merge_piece(*m, v);
        if (cached) {
          std::lock_guard<std::mutex> g(m->mu);
          if (m->cache.size() < m->cache_cap) m->cache.emplace(k, v);
        }
      }
    }
    if (w + v.size() > cap) return w;
    std::memcpy(out + w, v.data(), v.size() * 4);
    w += v.size();
  }
  return w;
}

}  // extern "C"
