// Vocabulary masks for constrained decoding (host).
//
// The reference computes, before every sampled token, which vocabulary entries keep a constraint
// satisfiable (crates/oxibonsai-runtime/src/constrained_decoding/sampler.rs:19-94, grammar/constraint.rs:66,
// grammar/cache.rs:52).  The inner loop - run every token's bytes through an automaton - is the hot
// part, so it lives here: a token table (byte strings of the whole vocabulary, plus an index by first
// byte) and two mask builders, one for byte-level DFAs and one that prefilters by the set of bytes an
// arbitrary recogniser can accept next.  Masks are packed 32 tokens per word, bit set = allowed, which
// is the format the GPU sampler takes.
#include <atomic>
#include <cstdint>
#include <cstring>
#include <vector>

#include "token_table.hpp"

using bonsai_tok::TokenTable;

extern "C" {

void* btok_new(const uint32_t* offsets, const uint8_t* bytes, uint32_t n) {
  static std::atomic<uint64_t> next_serial{1};
  TokenTable* t = new TokenTable();
  t->serial = next_serial.fetch_add(1);
  t->n = n;
  t->off.assign(offsets, offsets + n + 1);
  t->bytes.assign(bytes, bytes + offsets[n]);
  for (uint32_t i = 0; i < n; ++i)
    if (t->off[i + 1] > t->off[i]) t->by_first[t->bytes[t->off[i]]].push_back(i);
  return t;
}
void btok_free(void* h) { delete static_cast<TokenTable*>(h); }
uint32_t btok_count(void* h) { return static_cast<TokenTable*>(h)->n; }

// trans: int32 [n_states][256], -1 = reject.  Sets bit i of mask when token i, fed from `state`, stays
// inside the automaton; next_state (may be null) receives the state after each allowed token.
// Returns the number of allowed tokens.
uint32_t btok_dfa_mask(void* h, const int32_t* trans, int32_t n_states, int32_t state, uint32_t* mask, int32_t* next_state) {
  TokenTable& t = *static_cast<TokenTable*>(h);
  const uint32_t words = (t.n + 31) / 32;
  std::memset(mask, 0, words * sizeof(uint32_t));
  if (state < 0 || state >= n_states) return 0;
  uint32_t allowed = 0;
  const int32_t* row0 = trans + (size_t)state * 256;
  for (int b = 0; b < 256; ++b) {
    if (row0[b] < 0) continue;
    for (uint32_t i : t.by_first[b]) {
      int32_t s = row0[b];
      for (uint32_t p = t.off[i] + 1; p < t.off[i + 1] && s >= 0; ++p) s = trans[(size_t)s * 256 + t.bytes[p]];
      if (s >= 0) {
        mask[i >> 5] |= 1u << (i & 31);
        if (next_state) next_state[i] = s;
        ++allowed;
      }
    }
  }
  return allowed;
}

// first_ok: 256 flags.  Writes the ids of the tokens whose first byte is allowed into out (capacity
// cap) and returns how many there are (possibly more than cap).
uint32_t btok_candidates(void* h, const uint8_t* first_ok, uint32_t* out, uint32_t cap) {
  TokenTable& t = *static_cast<TokenTable*>(h);
  uint32_t k = 0;
  for (int b = 0; b < 256; ++b) {
    if (!first_ok[b]) continue;
    for (uint32_t i : t.by_first[b]) {
      if (k < cap) out[k] = i;
      ++k;
    }
  }
  return k;
}

// Packs a list of token ids into a mask.
void btok_pack_ids(const uint32_t* ids, uint32_t n_ids, uint32_t n_tokens, uint32_t* mask) {
  std::memset(mask, 0, ((n_tokens + 31) / 32) * sizeof(uint32_t));
  for (uint32_t k = 0; k < n_ids; ++k)
    if (ids[k] < n_tokens) mask[ids[k] >> 5] |= 1u << (ids[k] & 31);
}

}  // extern "C"

// ---- byte trie ------------------------------------------------------------------------------------------------------------
#include <algorithm>
#include <numeric>

void bonsai_tok::TokenTable::build_trie() {
  // tokens sorted by their bytes: every trie node is a contiguous range of the sorted order at some depth
  std::vector<uint32_t> order(n);
  std::iota(order.begin(), order.end(), 0u);
  auto tok = [&](uint32_t i) { return std::pair<const uint8_t*, uint32_t>(bytes.data() + off[i], off[i + 1] - off[i]); };
  std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
    auto [pa, la] = tok(a);
    auto [pb, lb] = tok(b);
    int c = std::memcmp(pa, pb, std::min(la, lb));
    return c != 0 ? c < 0 : (la != lb ? la < lb : a < b);
  });
  struct Work {
    uint32_t node, lo, hi, depth;
  };
  nodes.clear();
  edges.clear();
  node_tokens.clear();
  nodes.emplace_back();
  std::vector<Work> stack{{0, 0, n, 0}};
  while (!stack.empty()) {
    Work w = stack.back();
    stack.pop_back();
    uint32_t i = w.lo;
    // tokens that end here come first in the sorted range (shorter sorts before longer with the same prefix)
    nodes[w.node].tok_begin = uint32_t(node_tokens.size());
    while (i < w.hi && tok(order[i]).second == w.depth) {
      if (w.depth > 0) node_tokens.push_back(order[i]);
      ++i;
    }
    nodes[w.node].tok_end = uint32_t(node_tokens.size());
    uint32_t first_edge = uint32_t(edges.size());
    std::vector<Work> kids;
    while (i < w.hi) {
      uint8_t b = tok(order[i]).first[w.depth];
      uint32_t j = i;
      while (j < w.hi && tok(order[j]).first[w.depth] == b) ++j;
      uint32_t child = uint32_t(nodes.size());
      nodes.emplace_back();
      edges.push_back({b, child});
      kids.push_back({child, i, j, w.depth + 1});
      i = j;
    }
    nodes[w.node].child_begin = first_edge;
    nodes[w.node].child_end = uint32_t(edges.size());
    // children's edge ranges must be contiguous per node: process kids after this node's edges were all appended
    for (auto it = kids.rbegin(); it != kids.rend(); ++it) stack.push_back(*it);
  }
}
