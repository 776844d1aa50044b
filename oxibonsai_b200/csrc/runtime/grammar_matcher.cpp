// Byte-level Earley recogniser and the vocabulary mask of a grammar constraint (host).
//
// The reference recognises grammar-constrained output with an Earley parser over bytes and computes, before every
// sampled token, which vocabulary entries keep the output inside the grammar (crates/oxibonsai-runtime/src/grammar/
// earley.rs:39-193, constraint.rs:66, cache.rs:52).  Doing that per token over a 150 K vocabulary is the cost of constrained
// decoding, so it lives here:
//   * the chart is a stack: feeding a byte pushes an item set, pop() removes it, so one recogniser walks the byte trie of
//     the vocabulary depth-first and every shared prefix is parsed once;
//   * a child of a trie node is only entered when its byte is in the set of bytes the current item set can scan;
//   * every chart position has a signature: a hash of its unfinished items with each origin replaced by the signature of
//     the set it points to.  Two positions with equal signatures accept the same continuations, so the finished mask is
//     cached under (vocabulary, signature) in the compiled grammar and shared by every matcher of that grammar - the
//     positions inside a JSON string all hit one entry.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <memory>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>
#include <vector>

#include "token_table.hpp"

namespace {

using bonsai_tok::TokenTable;

struct ByteSet {
  uint64_t w[4] = {0, 0, 0, 0};
  bool has(uint8_t b) const { return (w[b >> 6] >> (b & 63)) & 1; }
  void merge(const ByteSet& o) {
    for (int i = 0; i < 4; ++i) w[i] |= o.w[i];
  }
};

struct Prod {
  uint32_t lhs, begin, len;          // symbols at syms[begin .. begin + len)
};

struct MaskKey {
  uint64_t table;                    // the vocabulary's serial number (addresses are reused, serials are not)
  uint64_t sig;
  int32_t eos;
  bool complete;
  bool operator==(const MaskKey& o) const { return table == o.table && sig == o.sig && eos == o.eos && complete == o.complete; }
};
struct MaskKeyHash {
  size_t operator()(const MaskKey& k) const {
    return size_t(k.sig ^ (k.table * 0x9E3779B97F4A7C15ull) ^ (uint64_t(uint32_t(k.eos)) << 1) ^ uint64_t(k.complete));
  }
};

struct TransKey {
  uint64_t sig;
  uint8_t byte;
  bool operator==(const TransKey& o) const { return sig == o.sig && byte == o.byte; }
};
struct TransKeyHash {
  size_t operator()(const TransKey& k) const { return size_t((k.sig ^ (uint64_t(k.byte) * 0x9E3779B97F4A7C15ull)) * 0xff51afd7ed558ccdull); }
};

struct Grammar {
  std::vector<ByteSet> terms;
  std::vector<int32_t> syms;          // >= 0: rule id, < 0: terminal -(id + 1)
  std::vector<Prod> prods;
  std::vector<std::vector<uint32_t>> rule_prods;
  std::vector<uint8_t> nullable;
  uint32_t start = 0;
  // finished masks, shared by the matchers of this grammar
  std::mutex mu;
  std::unordered_map<MaskKey, std::shared_ptr<std::vector<uint32_t>>, MaskKeyHash> masks;
  uint64_t hits = 0, misses = 0;
  size_t cap_bytes = 32u << 20;        // finished masks kept per grammar (a 152 K-token mask is 19 KB: about 1700 states)
  // Lazily built automaton over chart signatures: (signature, byte) -> signature after the byte, and the bytes a signature
  // can scan.  A signature stands for everything that can still follow, so once a transition has been seen the trie walk
  // takes it without touching the chart; only unseen transitions run the recogniser.
  std::shared_mutex tmu;
  std::unordered_map<TransKey, uint64_t, TransKeyHash> trans;
  std::unordered_map<uint64_t, ByteSet> info;
  uint64_t walked_real = 0, walked_cached = 0;
};

// item = prod (24 bits) | dot (8 bits) | origin (32 bits)
inline uint64_t mk_item(uint32_t prod, uint32_t dot, uint32_t origin) { return (uint64_t(prod) << 40) | (uint64_t(dot) << 32) | origin; }
inline uint32_t it_prod(uint64_t it) { return uint32_t(it >> 40); }
inline uint32_t it_dot(uint64_t it) { return uint32_t(it >> 32) & 0xFF; }
inline uint32_t it_origin(uint64_t it) { return uint32_t(it); }

inline uint64_t mix(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

struct ItemSet {
  std::vector<uint64_t> items;                      // closed set, insertion order
  std::vector<std::pair<uint32_t, uint64_t>> waiting;   // (rule the item waits for, item), sorted by rule
  ByteSet next;                                     // bytes that some item can scan
  uint64_t sig = 0;
  bool complete = false;                            // a start production spanning the whole input is finished
  void clear() {
    items.clear();
    waiting.clear();
    next = ByteSet();
    sig = 0;
    complete = false;
  }
};

struct Matcher {
  Grammar* g;
  std::vector<ItemSet> chart;       // chart[0 .. depth]
  size_t depth = 0;                 // index of the last live set
  bool dead = false;
  std::vector<uint64_t> work;
  // open-addressing set used while closing one item set
  std::vector<uint64_t> seen;
  size_t seen_mask = 0, seen_count = 0;

  explicit Matcher(Grammar* gr) : g(gr) { begin(); }

  bool seen_insert(uint64_t it) {
    if ((seen_count + 1) * 2 > seen.size()) {
      std::vector<uint64_t> old;
      old.swap(seen);
      seen.assign(old.empty() ? 64 : old.size() * 2, ~0ull);
      seen_mask = seen.size() - 1;
      seen_count = 0;
      for (uint64_t v : old)
        if (v != ~0ull) seen_insert(v);
    }
    size_t h = size_t(mix(it)) & seen_mask;
    while (seen[h] != ~0ull) {
      if (seen[h] == it) return false;
      h = (h + 1) & seen_mask;
    }
    seen[h] = it;
    ++seen_count;
    return true;
  }

  void close_set(ItemSet& s, uint32_t pos) {
    std::fill(seen.begin(), seen.end(), ~0ull);
    seen_count = 0;
    work.clear();
    std::vector<uint64_t> seed;
    seed.swap(s.items);
    auto push = [&](uint64_t it) {
      if (seen_insert(it)) {
        s.items.push_back(it);
        work.push_back(it);
      }
    };
    for (uint64_t it : seed) push(it);
    while (!work.empty()) {
      uint64_t it = work.back();
      work.pop_back();
      const Prod& p = g->prods[it_prod(it)];
      uint32_t d = it_dot(it);
      if (d < p.len) {
        int32_t sym = g->syms[p.begin + d];
        if (sym >= 0) {
          for (uint32_t q : g->rule_prods[size_t(sym)]) push(mk_item(q, 0, pos));
          if (g->nullable[size_t(sym)]) push(mk_item(it_prod(it), d + 1, it_origin(it)));
        }
      } else {
        uint32_t o = it_origin(it);
        if (o == pos) {
          // an empty derivation: the predictor has advanced the waiting items already, but items added to this set
          // later may wait for the same rule, so the set as it stands is scanned too
          for (size_t k = 0; k < s.items.size(); ++k) {
            uint64_t w = s.items[k];
            const Prod& pw = g->prods[it_prod(w)];
            uint32_t dw = it_dot(w);
            if (dw < pw.len && g->syms[pw.begin + dw] == int32_t(p.lhs)) push(mk_item(it_prod(w), dw + 1, it_origin(w)));
          }
        } else {
          const auto& wt = chart[o].waiting;
          auto lo = std::lower_bound(wt.begin(), wt.end(), std::make_pair(p.lhs, uint64_t(0)));
          for (; lo != wt.end() && lo->first == p.lhs; ++lo) push(mk_item(it_prod(lo->second), it_dot(lo->second) + 1, it_origin(lo->second)));
        }
      }
    }
    // derived data: waiting index, scannable bytes, completeness, signature
    uint64_t acc = 0x243F6A8885A308D3ull;
    for (uint64_t it : s.items) {
      const Prod& p = g->prods[it_prod(it)];
      uint32_t d = it_dot(it);
      if (d == p.len) {
        if (p.lhs == g->start && it_origin(it) == 0) s.complete = true;
        continue;
      }
      int32_t sym = g->syms[p.begin + d];
      if (sym >= 0) {
        s.waiting.emplace_back(uint32_t(sym), it);
      } else {
        s.next.merge(g->terms[size_t(-sym - 1)]);
      }
      uint32_t o = it_origin(it);
      // "this set" and "the first set" are named apart from every other origin: completeness of the whole input is tied to
      // origin 0, whatever else carries the same signature
      uint64_t osig = o == pos ? 0x5851F42D4C957F2Dull : (o == 0 ? chart[0].sig ^ 0x1F83D9ABFB41BD6Bull : chart[o].sig);
      acc += mix(mix((uint64_t(it_prod(it)) << 8) | d) ^ (osig * 0x9E3779B97F4A7C15ull));     // order-independent sum
    }
    std::sort(s.waiting.begin(), s.waiting.end());
    s.sig = mix(acc ^ (s.complete ? 0xA5A5A5A5ull : 0));
  }

  void begin() {
    if (chart.empty()) chart.emplace_back();
    depth = 0;
    dead = false;
    ItemSet& s = chart[0];
    s.clear();
    for (uint32_t q : g->rule_prods[g->start]) s.items.push_back(mk_item(q, 0, 0));
    close_set(s, 0);
  }

  bool feed(uint8_t b) {
    if (dead) return false;
    const ItemSet& last = chart[depth];
    if (!last.next.has(b)) {
      dead = true;
      return false;
    }
    if (chart.size() <= depth + 1) chart.emplace_back();
    ItemSet& s = chart[depth + 1];
    s.clear();
    for (uint64_t it : chart[depth].items) {
      const Prod& p = g->prods[it_prod(it)];
      uint32_t d = it_dot(it);
      if (d < p.len) {
        int32_t sym = g->syms[p.begin + d];
        if (sym < 0 && g->terms[size_t(-sym - 1)].has(b)) s.items.push_back(mk_item(it_prod(it), d + 1, it_origin(it)));
      }
    }
    ++depth;
    close_set(chart[depth], uint32_t(depth));
    return true;
  }

  void pop() {
    if (depth > 0) --depth;
    dead = false;
  }
};

// Depth-first over the vocabulary trie from the matcher's current position; sets the bit of every token that can be fed.
// The walk moves through chart signatures: a transition that the grammar's automaton already knows costs a hash lookup; an
// unknown one materialises the chart at that trie node (replaying the bytes of the path that were taken virtually), feeds
// the byte for real and records where it led.
struct Walker {
  Matcher& m;
  const TokenTable& t;
  Grammar& g;
  uint32_t* mask;
  size_t root_depth;
  std::vector<uint8_t> path;          // bytes from the walk's root to the current trie node
  size_t real = 0;                    // how many of them the chart holds (chart depth = root_depth + real)
  std::unordered_map<TransKey, uint64_t, TransKeyHash> new_trans;
  std::unordered_map<uint64_t, ByteSet> new_info;
  uint32_t allowed = 0;
  uint64_t n_real = 0, n_cached = 0;

  const ByteSet* info(uint64_t sig) const {
    auto a = new_info.find(sig);
    if (a != new_info.end()) return &a->second;
    auto b = g.info.find(sig);
    return b == g.info.end() ? nullptr : &b->second;
  }
  bool transition(uint64_t sig, uint8_t byte, uint64_t& out) const {
    TransKey k{sig, byte};
    auto a = new_trans.find(k);
    if (a != new_trans.end()) {
      out = a->second;
      return true;
    }
    auto b = g.trans.find(k);
    if (b == g.trans.end()) return false;
    out = b->second;
    return true;
  }
  void materialise() {
    while (real < path.size()) {
      m.feed(path[real]);
      ++real;
    }
  }
  void visit(uint32_t node, uint64_t sig) {
    const auto& nd = t.nodes[node];
    for (uint32_t k = nd.tok_begin; k < nd.tok_end; ++k) {
      uint32_t id = t.node_tokens[k];
      mask[id >> 5] |= 1u << (id & 31);
      ++allowed;
    }
    if (nd.child_begin == nd.child_end) return;
    const ByteSet* known = info(sig);
    if (!known) return;                                   // cannot happen: every signature handed to visit() was registered
    const ByteSet next = *known;
    for (uint32_t e = nd.child_begin; e < nd.child_end; ++e) {
      uint8_t b = t.edges[e].byte;
      if (!next.has(b)) continue;
      uint64_t nsig;
      if (transition(sig, b, nsig)) {
        ++n_cached;
      } else {
        materialise();
        if (!m.feed(b)) continue;                         // (the byte was in the scannable set, so this does not happen)
        ++real;
        ++n_real;
        const ItemSet& s = m.chart[m.depth];
        nsig = s.sig;
        new_trans.emplace(TransKey{sig, b}, nsig);
        if (!info(nsig)) new_info.emplace(nsig, s.next);
      }
      path.push_back(b);
      visit(t.edges[e].node, nsig);
      path.pop_back();
      while (real > path.size()) {                        // the chart must stay a prefix of the path: drop what belonged to the child
        m.pop();
        --real;
      }
    }
  }
};

uint32_t walk(Matcher& m, const TokenTable& t, uint32_t* mask) {
  Grammar& g = *m.g;
  Walker w{m, t, g, mask, m.depth, {}, 0, {}, {}, 0, 0, 0};
  const uint64_t root_sig = m.chart[m.depth].sig;
  {
    std::shared_lock<std::shared_mutex> rd(g.tmu);
    if (!w.info(root_sig)) w.new_info.emplace(root_sig, m.chart[m.depth].next);
    w.visit(0, root_sig);
  }
  m.depth = w.root_depth;
  m.dead = false;
  std::unique_lock<std::shared_mutex> wr(g.tmu);
  if (g.trans.size() + w.new_trans.size() > (1u << 19)) {          // a plain bound on the automaton (tens of megabytes)
    g.trans.clear();
    g.info.clear();
  }
  for (auto& kv : w.new_trans) g.trans.emplace(kv.first, kv.second);
  for (auto& kv : w.new_info) g.info.emplace(kv.first, kv.second);
  g.walked_real += w.n_real;
  g.walked_cached += w.n_cached;
  return w.allowed;
}

}  // namespace

extern "C" {

// blob (int32): n_terms, n_rules, start, then n_terms x 8 words (256-bit sets, little end first), then per rule:
// n_alternatives, per alternative: length, symbols (>= 0 rule id, < 0 terminal -(id + 1)).  Returns nullptr on a malformed blob.
static void* compile_checked(const int32_t* blob, uint32_t n);

void* bgram_compile(const int32_t* blob, uint32_t n) {
  try {
    return blob ? compile_checked(blob, n) : nullptr;
  } catch (...) {                       // out of memory on an absurd but well-formed blob: refused like a malformed one
    return nullptr;
  }
}

static void* compile_checked(const int32_t* blob, uint32_t n) {
  auto g = std::make_unique<Grammar>();
  uint32_t p = 0;
  auto need = [&](uint64_t k) { return uint64_t(p) + k <= uint64_t(n); };
  if (!need(3)) return nullptr;
  if (blob[0] < 0 || blob[1] <= 0 || blob[2] < 0) return nullptr;
  uint32_t n_terms = uint32_t(blob[p++]), n_rules = uint32_t(blob[p++]);
  g->start = uint32_t(blob[p++]);
  // every terminal set takes 8 words and every rule at least one, so both counts are bounded by the blob's length
  if (g->start >= n_rules || n_rules > n || !need(uint64_t(n_terms) * 8)) return nullptr;
  g->terms.resize(n_terms);
  for (uint32_t t = 0; t < n_terms; ++t)
    for (int w = 0; w < 4; ++w) {
      uint64_t lo = uint32_t(blob[p++]);
      uint64_t hi = uint32_t(blob[p++]);
      g->terms[t].w[w] = lo | (hi << 32);
    }
  g->rule_prods.resize(n_rules);
  for (uint32_t r = 0; r < n_rules; ++r) {
    if (!need(1)) return nullptr;
    if (blob[p] < 0) return nullptr;
    uint32_t alts = uint32_t(blob[p++]);
    if (!need(alts)) return nullptr;                    // every alternative takes at least its length word
    for (uint32_t a = 0; a < alts; ++a) {
      if (!need(1) || blob[p] < 0) return nullptr;
      uint32_t len = uint32_t(blob[p++]);
      if (!need(len) || len > 255 || g->prods.size() >= (1u << 24)) return nullptr;
      Prod pr{r, uint32_t(g->syms.size()), len};
      for (uint32_t k = 0; k < len; ++k) {
        int32_t s = blob[p++];
        if (s >= int32_t(n_rules) || (s < 0 && uint32_t(-s - 1) >= n_terms)) return nullptr;
        g->syms.push_back(s);
      }
      g->rule_prods[r].push_back(uint32_t(g->prods.size()));
      g->prods.push_back(pr);
    }
  }
  // nullable rules: fixed point
  g->nullable.assign(n_rules, 0);
  for (bool changed = true; changed;) {
    changed = false;
    for (const Prod& pr : g->prods) {
      if (g->nullable[pr.lhs]) continue;
      bool all = true;
      for (uint32_t k = 0; k < pr.len && all; ++k) {
        int32_t s = g->syms[pr.begin + k];
        all = s >= 0 && g->nullable[size_t(s)];
      }
      if (all) {
        g->nullable[pr.lhs] = 1;
        changed = true;
      }
    }
  }
  return g.release();
}

void bgram_free(void* h) { delete static_cast<Grammar*>(h); }

void* bgram_matcher_new(void* grammar) { return new Matcher(static_cast<Grammar*>(grammar)); }
void bgram_matcher_free(void* h) { delete static_cast<Matcher*>(h); }
void bgram_matcher_reset(void* h) { static_cast<Matcher*>(h)->begin(); }

// Feeds bytes; returns 1 when all were accepted, 0 when the matcher died on the way (it stays dead until reset).
int bgram_matcher_feed(void* h, const uint8_t* bytes, uint32_t n) {
  Matcher& m = *static_cast<Matcher*>(h);
  for (uint32_t i = 0; i < n; ++i)
    if (!m.feed(bytes[i])) return 0;
  return m.dead ? 0 : 1;
}

int bgram_matcher_complete(void* h) {
  Matcher& m = *static_cast<Matcher*>(h);
  return !m.dead && m.chart[m.depth].complete ? 1 : 0;
}

int bgram_matcher_dead(void* h) { return static_cast<Matcher*>(h)->dead ? 1 : 0; }
uint32_t bgram_matcher_position(void* h) { return uint32_t(static_cast<Matcher*>(h)->depth); }
uint64_t bgram_matcher_signature(void* h) {
  Matcher& m = *static_cast<Matcher*>(h);
  return m.dead ? 0 : m.chart[m.depth].sig;
}
uint32_t bgram_matcher_items(void* h) { return uint32_t(static_cast<Matcher*>(h)->chart[static_cast<Matcher*>(h)->depth].items.size()); }

void bgram_matcher_next_bytes(void* h, uint8_t* out256) {
  Matcher& m = *static_cast<Matcher*>(h);
  for (int b = 0; b < 256; ++b) out256[b] = !m.dead && m.chart[m.depth].next.has(uint8_t(b)) ? 1 : 0;
}

// The packed mask of the tokens that can follow the matcher's position (bit i = token i); ``eos`` (>= 0) is allowed when the
// input so far is a complete sentence.  Returns the number of allowed tokens; *cached tells whether the mask came from the
// grammar's cache.
uint32_t bgram_matcher_mask(void* h, void* table, int32_t eos, uint32_t* mask, int* cached) {
  Matcher& m = *static_cast<Matcher*>(h);
  TokenTable& t = *static_cast<TokenTable*>(table);
  const uint32_t words = (t.n + 31) / 32;
  std::memset(mask, 0, words * sizeof(uint32_t));
  if (cached) *cached = 0;
  if (m.dead) return 0;
  std::call_once(t.trie_once, [&] { t.build_trie(); });
  const bool complete = m.chart[m.depth].complete;            // (the chart may be reallocated by the walk below)
  MaskKey key{t.serial, m.chart[m.depth].sig, eos, complete};
  {
    std::lock_guard<std::mutex> lk(m.g->mu);
    auto it = m.g->masks.find(key);
    if (it != m.g->masks.end()) {
      m.g->hits++;
      std::memcpy(mask, it->second->data(), words * sizeof(uint32_t));
      if (cached) *cached = 1;
      uint32_t c = 0;
      for (uint32_t w = 0; w < words; ++w) c += uint32_t(__builtin_popcount(mask[w]));
      return c;
    }
    m.g->misses++;
  }
  uint32_t allowed = walk(m, t, mask);
  if (eos >= 0 && uint32_t(eos) < t.n && complete && !((mask[uint32_t(eos) >> 5] >> (uint32_t(eos) & 31)) & 1)) {
    mask[uint32_t(eos) >> 5] |= 1u << (uint32_t(eos) & 31);
    ++allowed;
  }
  auto copy = std::make_shared<std::vector<uint32_t>>(mask, mask + words);
  std::lock_guard<std::mutex> lk(m.g->mu);
  if ((m.g->masks.size() + 1) * size_t(words) * sizeof(uint32_t) > m.g->cap_bytes) m.g->masks.clear();      // a plain bound: grammars rarely reach it
  m.g->masks.emplace(key, std::move(copy));
  return allowed;
}

// out[0..5]: mask-cache hits, misses, entries; automaton transitions known; trie edges taken through the recogniser and
// through the automaton.
void bgram_cache_stats(void* grammar, uint64_t* out) {
  Grammar* g = static_cast<Grammar*>(grammar);
  {
    std::lock_guard<std::mutex> lk(g->mu);
    out[0] = g->hits;
    out[1] = g->misses;
    out[2] = g->masks.size();
  }
  std::shared_lock<std::shared_mutex> rd(g->tmu);
  out[3] = g->trans.size();
  out[4] = g->walked_real;
  out[5] = g->walked_cached;
}

}  // extern "C"
