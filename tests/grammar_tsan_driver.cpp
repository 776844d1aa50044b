// Race check of the grammar matcher's shared caches under ThreadSanitizer: compiled together with
// csrc/runtime/grammar_matcher.cpp and csrc/runtime/token_mask.cpp by tests/test_grammar_native.py.  Several threads, each
// with its own matcher over ONE compiled grammar and ONE vocabulary, feed random valid inputs and ask for masks, so the mask
// cache and the signature automaton are read and extended concurrently; the masks must agree with a single-threaded run.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* btok_new(const uint32_t* offsets, const uint8_t* bytes, uint32_t n);
void btok_free(void*);
void* bgram_compile(const int32_t* blob, uint32_t n);
void bgram_free(void*);
void* bgram_matcher_new(void*);
void bgram_matcher_free(void*);
void bgram_matcher_reset(void*);
int bgram_matcher_feed(void*, const uint8_t*, uint32_t);
uint32_t bgram_matcher_mask(void*, void*, int32_t, uint32_t*, int*);
void bgram_cache_stats(void*, uint64_t*);
}

static void term(std::vector<int32_t>& blob, uint8_t b) {
    uint32_t w[8] = {0};
    w[b >> 5] |= 1u << (b & 31);
    for (uint32_t x : w) blob.push_back(int32_t(x));
}

int main() {
    // root ::= rep ; rep ::= | rep item ; item ::= "(" root ")" | "a" | "b"
    std::vector<int32_t> blob{4, 3, 0};
    for (uint8_t b : {uint8_t('('), uint8_t(')'), uint8_t('a'), uint8_t('b')}) term(blob, b);
    const int32_t T_OPEN = -1, T_CLOSE = -2, T_A = -3, T_B = -4;
    blob.insert(blob.end(), {1, 1, 1});                              // root: one alternative: rep
    blob.insert(blob.end(), {2, 0, 2, 1, 2});                        // rep: empty | rep item
    blob.insert(blob.end(), {3, 3, T_OPEN, 0, T_CLOSE, 1, T_A, 1, T_B});
    void* g = bgram_compile(blob.data(), uint32_t(blob.size()));
    if (!g) return 2;
    // vocabulary: every string over "ab()" of length 1..4
    std::vector<std::string> toks;
    const char alpha[] = "ab()";
    for (int len = 1; len <= 4; ++len) {
        int total = 1;
        for (int i = 0; i < len; ++i) total *= 4;
        for (int v = 0; v < total; ++v) {
            std::string s;
            for (int i = 0, x = v; i < len; ++i, x /= 4) s += alpha[x % 4];
            toks.push_back(s);
        }
    }
    std::vector<uint32_t> off{0};
    std::vector<uint8_t> bytes;
    for (auto& s : toks) {
        bytes.insert(bytes.end(), s.begin(), s.end());
        off.push_back(uint32_t(bytes.size()));
    }
    void* table = btok_new(off.data(), bytes.data(), uint32_t(toks.size()));
    const uint32_t words = (uint32_t(toks.size()) + 31) / 32;
    auto inputs = [&alpha](unsigned seed) {
        std::mt19937 rng(seed);
        std::vector<std::string> out;
        for (int k = 0; k < 40; ++k) {
            std::string s;
            int depth = 0;
            for (int i = 0, n = int(rng() % 24); i < n; ++i) {
                int c = int(rng() % 4);
                if (c == 3 && depth == 0) c = 0;
                s += alpha[c];
                depth += c == 2 ? 1 : (c == 3 ? -1 : 0);
            }
            out.push_back(s);
        }
        return out;
    };
    auto run = [&](unsigned seed, std::vector<std::vector<uint32_t>>& masks) {
        void* m = bgram_matcher_new(g);
        std::vector<uint32_t> mask(words);
        for (auto& s : inputs(seed)) {
            bgram_matcher_reset(m);
            for (char ch : s) {
                uint8_t b = uint8_t(ch);
                if (!bgram_matcher_feed(m, &b, 1)) break;
                int cached = 0;
                bgram_matcher_mask(m, table, -1, mask.data(), &cached);
                masks.push_back(mask);
            }
        }
        bgram_matcher_free(m);
    };
    const int kThreads = 4;
    std::vector<std::vector<std::vector<uint32_t>>> got(kThreads);
    std::vector<std::thread> th;
    for (int t = 0; t < kThreads; ++t) th.emplace_back([&, t] { run(100u + unsigned(t % 2), got[size_t(t)]); });   // pairs of threads share inputs
    for (auto& t : th) t.join();
    // a fresh grammar, one thread: the reference for the masks
    void* g2 = bgram_compile(blob.data(), uint32_t(blob.size()));
    void* keep = g;
    g = g2;
    std::vector<std::vector<uint32_t>> want0, want1;
    run(100u, want0);
    run(101u, want1);
    bool same = got[0] == want0 && got[2] == want0 && got[1] == want1 && got[3] == want1;
    uint64_t st[6];
    bgram_cache_stats(keep, st);
    std::printf("grammar tsan driver %s: %zu masks per thread, cache hits %llu, misses %llu, transitions %llu\n", same ? "ok" : "MISMATCH", got[0].size(),
                (unsigned long long)st[0], (unsigned long long)st[1], (unsigned long long)st[3]);
    bgram_free(g2);
    bgram_free(keep);
    btok_free(table);
    return same ? 0 : 1;
}
