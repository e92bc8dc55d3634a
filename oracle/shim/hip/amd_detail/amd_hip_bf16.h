// Stand-in for ROCm's <hip/amd_detail/amd_hip_bf16.h>, which the reference's utils.h
// includes (utils.h:6) only for the __hip_bfloat16 type.  Just enough of that type for
// utils.h to compile with g++: construction from float (round to nearest even),
// conversion back to float, and subtraction (used by allClose, utils.h:41).
// Test infrastructure only; lets the reference's own host helpers be built unmodified.
#pragma once
#include <cstdint>
#include <cstring>
#include <cmath>

struct __hip_bfloat16 {
    uint16_t bits;
    __hip_bfloat16() : bits(0) {}
    __hip_bfloat16(float f) {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if ((u & 0x7fffffffu) > 0x7f800000u) { bits = 0x7fc0; }
        else { u += 0x7fffu + ((u >> 16) & 1u); bits = (uint16_t)(u >> 16); }
    }
    operator float() const {
        uint32_t u = (uint32_t)bits << 16;
        float f;
        std::memcpy(&f, &u, 4);
        return f;
    }
};
inline __hip_bfloat16 operator-(const __hip_bfloat16& a, const __hip_bfloat16& b) {
    return __hip_bfloat16((float)a - (float)b);
}
