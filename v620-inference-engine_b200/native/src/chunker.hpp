// Content-defined chunking of a prompt (cuts where a rolling hash of the last 16 tokens hits, at message
// boundaries, and at a maximum length) - feeds the "reusable outside the prefix" statistics of the
// prefix cache (behaviour of the reference's src/session/chunker.cpp: min 128 / average 512 / max 2048).
#pragma once
#include <vector>

#include "common.hpp"

namespace qwh {

struct Chunk {
    int64_t start, len;
    uint64_t hash;
};
constexpr int CHUNK_MIN = 128, CHUNK_AVG = 512, CHUNK_MAX = 2048, CHUNK_WINDOW = 16;

inline uint64_t chunk_mix(uint64_t h, uint32_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h * 0xff51afd7ed558ccdull;
}

inline std::vector<Chunk> chunk_prompt(const int32_t *tok, int64_t n, int32_t boundary) {
    std::vector<Chunk> out;
    int64_t start = 0;
    uint64_t h = 0;
    auto cut = [&](int64_t end) {
        if (end > start) out.push_back({start, end - start, h});
        start = end;
        h = 0;
    };
    for (int64_t i = 0; i < n; ++i) {
        if (tok[i] == boundary && i > start) cut(i);
        h = chunk_mix(h, uint32_t(tok[i]));
        const int64_t len = i + 1 - start;
        if (len >= CHUNK_MAX) { cut(i + 1); continue; }
        if (len >= CHUNK_MIN && i + 1 >= CHUNK_WINDOW) {
            uint64_t w = 0;
            for (int64_t j = i + 1 - CHUNK_WINDOW; j <= i; ++j) w = chunk_mix(w, uint32_t(tok[j]));
            if (w % CHUNK_AVG == 0) cut(i + 1);
        }
    }
    cut(n);
    return out;
}

}  // namespace qwh
