// Byte-pair-encoding merge engine (host).
//
// The reference ships a pure-Rust tokenizer (crates/oxibonsai-tokenizer/src/bpe.rs:19-216: merge table, greedy
// lowest-rank merging, `<0xHH>` byte fallback).  This is the same algorithm on integer ids: the caller
// pre-tokenises text and maps every byte (or character) of a piece to its initial token id; the engine
// repeatedly merges the adjacent pair with the lowest merge rank until none applies.  A piece cache makes
// repeated words O(1).
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

void merge_piece(const Bpe& m, std::vector<uint32_t>& ids) {
  while (ids.size() > 1) {
    uint32_t best_rank = UINT32_MAX, best_id = 0;
    size_t best_pos = 0;
    for (size_t i = 0; i + 1 < ids.size(); ++i) {
      auto it = m.merges.find(key(ids[i], ids[i + 1]));
      if (it != m.merges.end() && it->second.first < best_rank) {
        best_rank = it->second.first;
        best_id = it->second.second;
        best_pos = i;
      }
    }
    if (best_rank == UINT32_MAX) break;
    // merge every occurrence of the winning pair, left to right
    uint32_t a = ids[best_pos], b = ids[best_pos + 1];
    std::vector<uint32_t> out;
    out.reserve(ids.size());
    for (size_t i = 0; i < ids.size();) {
      if (i + 1 < ids.size() && ids[i] == a && ids[i + 1] == b) {
        out.push_back(best_id);
        i += 2;
      } else {
        out.push_back(ids[i]);
        ++i;
      }
    }
    ids.swap(out);
  }
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

}  // extern "C"
