// Last-bit tables for the three single-precision libm functions the projection needs per node.
//
// The reference computes acosf, sinf and tanf with the host's libm, whose results are within one ulp of the exact
// value but not always the correctly rounded one (about 2-5 % of inputs differ in the last bit). The device evaluates
// the same functions in double precision and rounds once, which lands within one ulp of whatever the host libm
// returns. To return exactly what the host libm returns - on this machine, whichever libm version it runs - the
// engine tabulates, once per process and function, the low two bits of libm's result for every float in the input
// range that can occur for an on-screen node (2 bits per input, 57-59 MB per function). The device then picks, among
// its own result and its two neighbouring floats, the one whose low two bits match: three consecutive bit patterns have
// distinct residues modulo four, so the choice is unique whenever the two sides are within one ulp.
// The tables start at 2^-27. Below that, sin(t) = tan(t) = t and acos(x) = float(pi / 2) in single precision for any
// libm that is within one ulp (glibc 2.39 was checked over every float below 2^-24: its only results that differ from
// the correctly rounded ones are acosf at five inputs near 1.59e-8, which the table covers). Inputs outside the tables
// keep the device's correctly rounded value: x <= 0 for acos (a ray in or behind the plane perpendicular to the optical
// axis, on screen only for a lens whose field of view exceeds 180 degrees) and theta / 2 >= 2 for sin (never: theta
// is at most pi). There the pixel coordinate can differ from the reference's by one ulp of theta (2.4e-7 rad, under
// 3e-4 px for the focal lengths of a megapixel camera), inside the 1e-3 px tolerance.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace vm {
namespace libm {

    enum Function { ACOS = 0, SIN = 1, TAN = 2, N_FUNCTIONS = 3 };

    // [first, first + count) in float bit patterns: positive floats only, whole binades
    constexpr uint32_t TABLE_FIRST     = 0x32000000u;  // 2^-27
    constexpr uint32_t TABLE_END_ONE   = 0x3F800000u;  // 1
    constexpr uint32_t TABLE_END_TWO   = 0x40000000u;  // 2
    constexpr uint32_t FIRST_BITS[N_FUNCTIONS] = {
      TABLE_FIRST,  // acos: x in [2^-27, 1)
      TABLE_FIRST,  // sin:  t in [2^-27, 2)   (t = theta / 2 <= pi / 2)
      TABLE_FIRST,  // tan:  t in [2^-27, 2)   (t = theta clamped to [0, pi/2])
    };
    constexpr uint32_t END_BITS[N_FUNCTIONS] = {TABLE_END_ONE, TABLE_END_TWO, TABLE_END_TWO};

    inline uint32_t count(int fn) {
        return END_BITS[fn] - FIRST_BITS[fn];
    }
    inline size_t words(int fn) {
        return (static_cast<size_t>(count(fn)) + 15) / 16;
    }

    // Evaluated through the same overloads the reference's templates resolve to for Scalar = float
    // (cpp/visualmesh/utility/projection.hpp:41,53,167).
    inline float evaluate(int fn, float x) {
        switch (fn) {
            case ACOS: return std::acos(x);
            case SIN: return std::sin(x);
            default: return std::tan(x);
        }
    }

    inline std::vector<uint32_t> build(int fn) {
        std::vector<uint32_t> packed(words(fn), 0u);
        const uint32_t first = FIRST_BITS[fn];
        const size_t n_words = packed.size();
        unsigned n_threads   = std::thread::hardware_concurrency();
        n_threads            = n_threads == 0 ? 4 : (n_threads > 32 ? 32 : n_threads);
        std::vector<std::thread> workers;
        const size_t per = (n_words + n_threads - 1) / n_threads;
        for (unsigned t = 0; t < n_threads; ++t) {
            const size_t w0 = t * per;
            const size_t w1 = w0 + per < n_words ? w0 + per : n_words;
            if (w0 >= w1) break;
            workers.emplace_back([fn, first, w0, w1, &packed] {
                for (size_t w = w0; w < w1; ++w) {
                    uint32_t word = 0;
                    for (uint32_t j = 0; j < 16; ++j) {
                        const uint32_t bits = first + static_cast<uint32_t>(w) * 16u + j;
                        float x;
                        std::memcpy(&x, &bits, sizeof(x));
                        const float y = evaluate(fn, x);
                        uint32_t yb;
                        std::memcpy(&yb, &y, sizeof(yb));
                        word |= (yb & 3u) << (2u * j);
                    }
                    packed[w] = word;
                }
            });
        }
        for (auto& w : workers) w.join();
        return packed;
    }

}  // namespace libm
}  // namespace vm
