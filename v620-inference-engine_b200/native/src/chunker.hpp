// Content-defined chunking of a prompt.  A prompt is cut into chunks whose borders depend on the text
// around them rather than on their distance from the start, so that the same passage met again after a
// different prefix falls into the same chunks; the session counts how many prompt tokens lie in chunks it
// has seen before (the "reusable outside the prefix" statistic of the prefix cache).
//
// A border is placed after a token when a cyclic-polynomial (buzhash) fingerprint of the last 16 tokens
// has its low nine bits clear - on average every 512 tokens - but not before a chunk has 128 tokens and
// at the latest at 2,048; a message-boundary token always starts a new chunk.  The fingerprint slides in
// constant time per token: the leaving token's table value, rotated by the window length, is xor-ed out
// as the entering one is xor-ed in.  A chunk's identity is an FNV-1a hash of its tokens.
// (Role of the reference's src/session/chunker.cpp:14-41: same size limits and boundary rule; the
// fingerprint and the identity hash are this implementation's own, nothing stores them.)
#pragma once
#include <vector>

#include "common.hpp"

namespace qwh {

struct Chunk {
    int64_t start, len;
    uint64_t hash;
};
constexpr int CHUNK_MIN = 128, CHUNK_AVG = 512, CHUNK_MAX = 2048, CHUNK_WINDOW = 16;

// The sliding fingerprint of the most recent CHUNK_WINDOW tokens.
class WindowPrint {
public:
    void push(int32_t tok) {
        ring_[n_ % CHUNK_WINDOW] = tok;
        const uint64_t in = spread(tok);
        if (n_ < CHUNK_WINDOW) {
            h_ = rotl(h_, 1) ^ in;
        } else {
            // the token that entered CHUNK_WINDOW pushes ago has been rotated that many times since
            h_ = rotl(h_, 1) ^ rotl(spread(leaving_), CHUNK_WINDOW) ^ in;
        }
        ++n_;
        leaving_ = ring_[n_ % CHUNK_WINDOW];
    }
    bool full() const { return n_ >= CHUNK_WINDOW; }
    bool at_border() const { return (h_ & uint64_t(CHUNK_AVG - 1)) == 0; }

private:
    static uint64_t rotl(uint64_t v, int k) { return (v << k) | (v >> (64 - k)); }
    static uint64_t spread(int32_t tok) {          // a fixed pseudo-random 64-bit value per token id
        uint64_t z = uint64_t(uint32_t(tok)) + 0x9e3779b97f4a7c15ull;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        return z ^ (z >> 31);
    }
    int32_t ring_[CHUNK_WINDOW] = {};
    int32_t leaving_ = 0;
    int64_t n_ = 0;
    uint64_t h_ = 0;
};

inline uint64_t chunk_identity(const int32_t *tok, int64_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (int64_t i = 0; i < n; ++i) {
        uint32_t v = uint32_t(tok[i]);
        for (int b = 0; b < 4; ++b, v >>= 8) h = (h ^ (v & 0xffu)) * 0x100000001b3ull;
    }
    return h;
}

inline std::vector<Chunk> chunk_prompt(const int32_t *tok, int64_t n, int32_t boundary) {
    static_assert((CHUNK_AVG & (CHUNK_AVG - 1)) == 0, "the border test masks the fingerprint's low bits");
    std::vector<Chunk> chunks;
    WindowPrint print;
    int64_t first = 0;                               // first token of the chunk being grown
    const auto close_at = [&](int64_t end) {         // [first, end) becomes a chunk
        if (end <= first) return;
        chunks.push_back(Chunk{first, end - first, chunk_identity(tok + first, end - first)});
        first = end;
    };
    for (int64_t pos = 0; pos < n; ++pos) {
        if (tok[pos] == boundary) close_at(pos);     // a message boundary opens a chunk of its own
        print.push(tok[pos]);
        const int64_t grown = pos + 1 - first;
        const bool content_border = grown >= CHUNK_MIN && print.full() && print.at_border();
        if (content_border || grown >= CHUNK_MAX) close_at(pos + 1);
    }
    close_at(n);
    return chunks;
}

}  // namespace qwh
