// The vocabulary as byte strings, indexed by first byte and (built on first use) as a byte trie.
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>

namespace bonsai_tok {

struct TrieNode {
  uint32_t child_begin = 0, child_end = 0;   // range in TokenTable::edges, sorted by byte
  uint32_t tok_begin = 0, tok_end = 0;       // range in TokenTable::node_tokens: the tokens that end at this node
};
struct TrieEdge {
  uint8_t byte;
  uint32_t node;
};

struct TokenTable {
  std::vector<uint32_t> off;     // n + 1
  std::vector<uint8_t> bytes;
  std::vector<uint32_t> by_first[256];
  uint32_t n = 0;
  uint64_t serial = 0;           // unique per table for the life of the process (cache keys)
  // byte trie over all tokens (node 0 is the root); empty tokens end at the root and are never offered
  std::vector<TrieNode> nodes;
  std::vector<TrieEdge> edges;
  std::vector<uint32_t> node_tokens;
  std::once_flag trie_once;
  void build_trie();
};

}  // namespace bonsai_tok
