// Host-side basics shared by the native runtime: error type, logging, numeric conversions.
#pragma once
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>

namespace qwh {

struct Error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
[[noreturn]] inline void fail(const std::string &m) { throw Error(m); }
#define QWH_CHECK(c, msg) do { if (!(c)) ::qwh::fail(std::string("check failed: ") + (msg)); } while (0)

inline void logf(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    std::fputs("[qw] ", stderr);
    std::vfprintf(stderr, fmt, ap);
    std::fputc('\n', stderr);
    va_end(ap);
}

inline float bf16_to_f32(uint16_t v) {
    uint32_t u = uint32_t(v) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16(float f) {          // round to nearest even
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
    const uint32_t s = (h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = s;
        else {
            int sh = 0;
            uint32_t mm = m;
            while (!(mm & 0x400)) { mm <<= 1; ++sh; }
            u = s | ((uint32_t)(113 - sh) << 23) | ((mm & 0x3ff) << 13);
        }
    } else if (e == 31) u = s | 0x7f800000u | (m << 13);
    else u = s | ((e + 112) << 23) | (m << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline float f8e4m3_to_f32(uint8_t b) {          // finite-only "fn" variant; 0x7f / 0xff are NaN -> 0
    const int s = b >> 7, e = (b >> 3) & 0xf, m = b & 7;
    if (e == 15 && m == 7) return 0.f;
    float v = e == 0 ? std::ldexp(float(m), -9) : std::ldexp(float(8 + m), e - 10);
    return s ? -v : v;
}

}  // namespace qwh
