// Host-side stress of the KV slab manager (tm_cache_*, host-memory mode) meant to run under AddressSanitizer and
// UndefinedBehaviorSanitizer: a seeded sequence of create / fetch / update / erase calls with more sessions than
// entries, every slab handed out written over its full length, every stored token list read back.
// Built and run by tests/test_host_sanitizers.py; exits 0 when every check holds.
#include "tm_b200.h"

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <random>
#include <vector>

#define CHECK(cond)                                                                                                    \
    do {                                                                                                               \
        if (!(cond)) {                                                                                                 \
            std::fprintf(stderr, "check failed at line %d: %s\n", __LINE__, #cond);                                    \
            return 1;                                                                                                  \
        }                                                                                                              \
    } while (0)

int main()
{
    const size_t layers = 2, heads = 2, dim = 8, max_len = 16, bits = 16, entries = 5, chunk = 2;
    const size_t half_slab = layers * heads * max_len * dim * bits / 8;  // keys (or values) of one sequence
    tm_cache_manager* m = nullptr;
    CHECK(tm_cache_manager_create(&m, layers, heads, dim, max_len, bits, entries, chunk, -1) == TM_OK);

    std::mt19937                    rng(1234);
    std::map<uint64_t, std::vector<int>> known;   // what every live session stored last
    std::vector<tm_cache_sequence>       held;    // sequences fetched and not yet given back
    for (int step = 0; step < 4000; ++step) {
        const uint64_t id = 1 + rng() % 9;
        const int      op = (int)(rng() % 10);
        bool           id_held = false;
        for (const auto& h : held) id_held = id_held || h.id == id;
        if (op < 4) {
            if (id_held) continue;  // one holder per session at a time
            // fetch or create, write the whole slab, store some tokens, give it back
            tm_cache_sequence s{};
            const bool        exists = tm_cache_contains(m, id) != 0;
            const int         rc     = exists ? tm_cache_fetch(m, id, nullptr, &s) : tm_cache_create(m, id, nullptr, &s);
            if (rc != TM_OK) continue;  // every entry pinned by `held`: refused, nothing changed
            CHECK(s.k_cache != nullptr && s.v_cache != nullptr && s.max_seq_len == max_len);
            std::memset(s.k_cache, 0x5a, half_slab);
            std::memset(s.v_cache, 0xa5, half_slab);
            if (exists && s.cache_len == 0) {
                // the slab was taken by another session in between: the tokens survive, the rows do not
            }
            if (rng() % 3 == 0 && held.size() < 3) {
                held.push_back(s);  // stays pinned for a while
                continue;
            }
            std::vector<int> toks(rng() % (max_len + 1));
            for (auto& t : toks) t = (int)(rng() % 1000);
            s.cache_len = toks.empty() ? 0 : toks.size() - 1;
            CHECK(tm_cache_update(m, &s, toks.data(), toks.size()) == TM_OK);
            known[id] = toks;
        }
        else if (op < 6 && !held.empty()) {
            // give a pinned sequence back
            tm_cache_sequence s = held.back();
            held.pop_back();
            std::vector<int> toks(1 + rng() % max_len, 7);
            s.cache_len = toks.size() - 1;
            CHECK(tm_cache_update(m, &s, toks.data(), toks.size()) == TM_OK);
            known[s.id] = toks;
        }
        else if (op < 8) {
            // read the tokens back: exactly what was stored
            if (!tm_cache_contains(m, id)) continue;
            size_t n = 0;
            CHECK(tm_cache_tokens(m, id, nullptr, 0, &n) == TM_OK);
            std::vector<int> got(n + 4, -1);
            CHECK(tm_cache_tokens(m, id, got.data(), n, &n) == TM_OK);
            auto it = known.find(id);
            if (it != known.end()) {
                CHECK(n == it->second.size());
                CHECK(n == 0 || std::memcmp(got.data(), it->second.data(), n * sizeof(int)) == 0);
            }
            CHECK(got[n] == -1);  // nothing written past the count
        }
        else {
            if (id_held) continue;
            const int had = tm_cache_contains(m, id);
            const int rc  = tm_cache_erase(m, id);
            CHECK((rc == TM_OK) == (had != 0));
            known.erase(id);
            CHECK(tm_cache_contains(m, id) == 0);
        }
    }
    // bad arguments are refused, not dereferenced
    tm_cache_sequence s{};
    CHECK(tm_cache_fetch(m, 424242, nullptr, &s) != TM_OK);
    CHECK(tm_cache_create(nullptr, 1, nullptr, &s) != TM_OK);
    CHECK(tm_cache_tokens(m, 424242, nullptr, 0, nullptr) != TM_OK);
    CHECK(tm_cache_manager_destroy(m) == TM_OK);
    std::puts("cache manager stress ok");
    return 0;
}
