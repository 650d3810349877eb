// Device-side arithmetic of the Visual Mesh hot path: lens projection and image sampling.
//
// Every function follows the operation order and rounding of the reference CPU engine so that the on-screen set
// and the pixel coordinates come out the same. This translation unit must be compiled with -fmad=false: the
// reference is only self-consistent without FMA contraction, and a fused multiply-add in the ray rotation or in
// 1 - x*x moves nodes across the image border.
#pragma once

#include <cstdint>

#include "../../include/vmcuda.h"

namespace vm {

// Per-frame constants, computed on the host with the host's libm exactly as the reference computes them.
struct FrameParams {
    float Rco[9];       // Rco[i][j] = Hoc[j][i]            cpp/visualmesh/engine/cpu/engine.hpp:95
    float focal_length;
    float centre[2];
    float half_dims[2]; // float(dimensions) * 0.5f         cpp/visualmesh/utility/projection.hpp:186
    float ik[4];        // inverse_coefficients(lens.k)     cpp/visualmesh/utility/projection.hpp:80-87
    int32_t dims[2];
    int32_t projection;
    uint32_t format;
    float cos_fov;      // cos(fov / 2), sin(fov / 2)       cpp/visualmesh/mesh.hpp:503-504
    float sin_fov;
    float edges[4][5];  // screen edge cones axis, cos, sin  cpp/visualmesh/mesh.hpp:265-349
    const float4* rays;       // mesh rays (x, y, z, 0)
    const int32_t* neighbours; // mesh neighbour table [n_nodes][N]
    const float4* bsp_cones_a; // per BSP element: axis xyz, cos
    const float* bsp_cones_s;  // per BSP element: sin
    const int4* bsp_topology;  // per BSP element: child0, child1 (-1 leaf), first node of child1, unused
    const uint8_t* image;
    const int2* ranges;        // host lookup ranges of this frame (device copy), or nullptr for device lookup
    const int32_t* range_starts; // exclusive prefix sum of the range lengths
    int32_t n_ranges;
    int32_t n_nodes;
    int32_t n_bsp;
    int32_t n_candidates; // sum of range lengths, or n_nodes for device lookup
    int32_t cand_off;     // first candidate slot of this frame inside the chunk
    int32_t node_off;     // first entry of this frame's node -> local index table inside the chunk
    int32_t bsp_off;      // first entry of this frame's BSP state table inside the chunk
    int32_t image_row_bytes;
    // low two bits of the host libm's acosf / sinf / tanf per input float (libm_tables.hpp); nullptr = not tabulated
    const uint32_t* libm_acos;
    const uint32_t* libm_sin;
    const uint32_t* libm_tan;
};

__device__ __forceinline__ float dot3(float a0, float a1, float a2, float b0, float b1, float b2) {
    // cpp/visualmesh/utility/math.hpp:160-177: a[2]*b[2] + (a[1]*b[1] + a[0]*b[0]), every operation rounded
    return __fadd_rn(__fmul_rn(a2, b2), __fadd_rn(__fmul_rn(a1, b1), __fmul_rn(a0, b0)));
}

// The host libm's acosf/sinf/tanf are within 1 ulp of the exact result; evaluating in double and rounding once gives
// the correctly rounded float, which is within one ulp of the host's. `as_host_libm` then moves it by at most one
// ulp onto the host libm's own result, using the tabulated low two bits of that result (libm_tables.hpp).
__device__ __forceinline__ float as_host_libm(float approx, float x, const uint32_t* table, uint32_t first_bits, uint32_t end_bits) {
    const uint32_t bx = __float_as_uint(x);
    if (table == nullptr || bx < first_bits || bx >= end_bits) return approx;
    const uint32_t i    = bx - first_bits;
    const uint32_t code = (__ldg(table + (i >> 4)) >> ((i & 15u) * 2u)) & 3u;
    uint32_t ba         = __float_as_uint(approx);
    const uint32_t d    = (code - (ba & 3u)) & 3u;  // 0: same, 1: one ulp up, 3: one ulp down
    ba += (d == 1u) ? 1u : (d == 3u) ? 0xFFFFFFFFu : 0u;
    return __uint_as_float(ba);
}
// Input ranges of the tables as float bit patterns, [first, end): 2^-27 up to 1 (acos) or 2 (sin, tan). The host side
// builds the tables over the same ranges (libm_tables.hpp; the engine checks the two at compile time).
constexpr uint32_t LIBM_FIRST_BITS = 0x32000000u;
constexpr uint32_t LIBM_ONE_BITS   = 0x3F800000u;
constexpr uint32_t LIBM_TWO_BITS   = 0x40000000u;
__device__ __forceinline__ float acos_rn(float x, const uint32_t* table) {
    return as_host_libm(__double2float_rn(acos(static_cast<double>(x))), x, table, LIBM_FIRST_BITS, LIBM_ONE_BITS);
}
__device__ __forceinline__ float sin_rn(float x, const uint32_t* table) {
    return as_host_libm(__double2float_rn(sin(static_cast<double>(x))), x, table, LIBM_FIRST_BITS, LIBM_TWO_BITS);
}
__device__ __forceinline__ float tan_rn(float x, const uint32_t* table) {
    return as_host_libm(__double2float_rn(tan(static_cast<double>(x))), x, table, LIBM_FIRST_BITS, LIBM_TWO_BITS);
}

// cpp/visualmesh/utility/projection.hpp:105-120: float products, double running sum, one rounding at the end
__device__ __forceinline__ float distort(float r, const float* ik) {
    const float r2 = __fmul_rn(r, r);
    const float r4 = __fmul_rn(r2, r2);
    const float t0 = __fmul_rn(ik[0], r2);
    const float t1 = __fmul_rn(ik[1], r4);
    const float t2 = __fmul_rn(__fmul_rn(ik[2], r4), r2);
    const float t3 = __fmul_rn(__fmul_rn(ik[3], r4), r4);
    double s       = __dadd_rn(1.0, static_cast<double>(t0));
    s              = __dadd_rn(s, static_cast<double>(t1));
    s              = __dadd_rn(s, static_cast<double>(t2));
    s              = __dadd_rn(s, static_cast<double>(t3));
    return __double2float_rn(__dmul_rn(static_cast<double>(r), s));
}

// cpp/visualmesh/utility/projection.hpp:163-187 on a camera-space unit vector
__device__ __forceinline__ float2 project(float rx, float ry, float rz, const FrameParams& p) {
    const float f          = p.focal_length;
    const float theta      = acos_rn(rx, p.libm_acos);
    const float rsin_theta = __fdiv_rn(1.0f, __fsqrt_rn(__fsub_rn(1.0f, __fmul_rn(rx, rx))));
    float r_u;
    if (p.projection == VM_RECTILINEAR) {
        // std::min(std::max(theta, 0), float(pi/2)) with std::min/max's NaN behaviour (projection.hpp:52-54)
        const float pi_2 = 1.57079637050628662109375f;
        float t          = (theta < 0.0f) ? 0.0f : theta;
        t                = (pi_2 < t) ? pi_2 : t;
        r_u              = __fmul_rn(f, tan_rn(t, p.libm_tan));
    }
    else if (p.projection == VM_EQUISOLID) {
        r_u = __fmul_rn(__fmul_rn(2.0f, f), sin_rn(__fmul_rn(theta, 0.5f), p.libm_sin));
    }
    else {
        r_u = __fmul_rn(f, theta);
    }
    const float r_d = distort(r_u, p.ik);
    float sx = 0.0f, sy = 0.0f;
    if (!(rx >= 1.0f)) {
        sx = __fmul_rn(__fmul_rn(r_d, ry), rsin_theta);
        sy = __fmul_rn(__fmul_rn(r_d, rz), rsin_theta);
    }
    float2 px;
    px.x = __fsub_rn(__fsub_rn(p.half_dims[0], sx), p.centre[0]);
    px.y = __fsub_rn(__fsub_rn(p.half_dims[1], sy), p.centre[1]);
    return px;
}

// Rotates an observation-plane ray into camera space: multiply(Rco, ray), cpp/visualmesh/utility/math.hpp:254-257
__device__ __forceinline__ void rotate(const FrameParams& p, float x, float y, float z, float& cx, float& cy, float& cz) {
    cx = dot3(p.Rco[0], p.Rco[1], p.Rco[2], x, y, z);
    cy = dot3(p.Rco[3], p.Rco[4], p.Rco[5], x, y, z);
    cz = dot3(p.Rco[6], p.Rco[7], p.Rco[8], x, y, z);
}

// The engine's keep test (strict, cpp/visualmesh/engine/cpu/engine.hpp:116-117); NaN fails.
__device__ __forceinline__ bool on_screen_strict(float2 px, const FrameParams& p) {
    return 0.0f <= px.x && __fadd_rn(px.x, 1.0f) < static_cast<float>(p.dims[0]) && 0.0f <= px.y
           && __fadd_rn(px.y, 1.0f) < static_cast<float>(p.dims[1]);
}
// The lookup's test (non-strict, cpp/visualmesh/mesh.hpp:374-375, :562-565)
__device__ __forceinline__ bool on_screen_loose(float2 px, const FrameParams& p) {
    return 0.0f <= px.x && __fadd_rn(px.x, 1.0f) <= static_cast<float>(p.dims[0]) && 0.0f <= px.y
           && __fadd_rn(px.y, 1.0f) <= static_cast<float>(p.dims[1]);
}

// ---- image sampling ---------------------------------------------------------------------------------------------

__host__ __device__ constexpr uint32_t fcc(char a, char b, char c, char d) {
    return uint32_t(uint8_t(a)) | (uint32_t(uint8_t(b)) << 8) | (uint32_t(uint8_t(c)) << 16) | (uint32_t(uint8_t(d)) << 24);
}

enum : int { FMT_UNKNOWN = 0, FMT_RGBA, FMT_BGRA, FMT_RGB3, FMT_BGR3, FMT_GREY, FMT_RGGB, FMT_GRBG, FMT_GBRG, FMT_BGGR };

__host__ __device__ inline int format_class(uint32_t f) {
    switch (f) {
        case fcc('R', 'G', 'B', 'A'): return FMT_RGBA;
        case fcc('B', 'G', 'R', 'A'): return FMT_BGRA;
        case fcc('R', 'G', 'B', '3'):
        case fcc('R', 'G', 'B', '8'): return FMT_RGB3;
        case fcc('B', 'G', 'R', '3'):
        case fcc('B', 'G', 'R', '8'): return FMT_BGR3;
        case fcc('G', 'R', 'A', 'Y'):
        case fcc('G', 'R', 'E', 'Y'):
        case fcc('Y', '8', ' ', ' '): return FMT_GREY;
        case fcc('R', 'G', 'G', 'B'): return FMT_RGGB;
        case fcc('G', 'R', 'B', 'G'): return FMT_GRBG;
        case fcc('G', 'B', 'R', 'G'): return FMT_GBRG;
        case fcc('B', 'G', 'G', 'R'): return FMT_BGGR;
        default: return FMT_UNKNOWN;
    }
}
__host__ __device__ inline int format_bytes_per_pixel(int cls) {
    return (cls == FMT_RGBA || cls == FMT_BGRA) ? 4 : (cls == FMT_RGB3 || cls == FMT_BGR3) ? 3 : 1;
}

// Malvar-He-Cutler kernels scaled by 64, cpp/visualmesh/engine/cpu/bayer.hpp:45-83. Four distinct matrices:
// 0 = G at R/B, 1 = R at B / B at R, 2 = R at G on red rows / B at G on blue rows, 3 = R at G on blue rows / B at G on
// red rows.
__device__ __forceinline__ int mhc(const int* p, int which) {
    switch (which) {
        case 0: return -8 * p[2] + 16 * p[7] - 8 * p[10] + 16 * p[11] + 32 * p[12] + 16 * p[13] - 8 * p[14] + 16 * p[17] - 8 * p[22];
        case 1:
            return -12 * p[2] + 16 * p[6] + 16 * p[8] - 12 * p[10] + 48 * p[12] - 12 * p[14] + 16 * p[16] + 16 * p[18]
                   - 12 * p[22];
        case 2:
            return 4 * p[2] - 8 * p[6] - 8 * p[8] - 8 * p[10] + 32 * p[11] + 40 * p[12] + 32 * p[13] - 8 * p[14] - 8 * p[16]
                   - 8 * p[18] + 4 * p[22];
        default:
            return -8 * p[2] - 8 * p[6] + 32 * p[7] - 8 * p[8] + 4 * p[10] + 40 * p[12] + 4 * p[14] - 8 * p[16] + 32 * p[17]
                   - 8 * p[18] - 8 * p[22];
    }
}

// cpp/visualmesh/engine/cpu/bayer.hpp:96-158: integer demosaic of the clamped 5x5 patch, /64 truncating toward zero,
// no clamp of the result, alpha 255.
__device__ __forceinline__ float4 bayer_pixel(int x, int y, const uint8_t* image, int W, int H, int cls) {
    int p[25];
#pragma unroll
    for (int dy = 0; dy < 5; ++dy) {
        const int yc          = min(max(y - 2 + dy, 0), H - 1);
        const uint8_t* row    = image + static_cast<size_t>(yc) * W;
#pragma unroll
        for (int dx = 0; dx < 5; ++dx) { p[dy * 5 + dx] = __ldg(row + min(max(x - 2 + dx, 0), W - 1)); }
    }
    const bool col = (x % 2) == 1;
    const bool row = (y % 2) == 1;
    // 0 = R, 1 = GR (green on a red row), 2 = GB, 3 = B
    int type;
    switch (cls) {
        case FMT_GRBG: type = row ? (col ? 2 : 3) : (col ? 0 : 1); break;
        case FMT_RGGB: type = row ? (col ? 3 : 2) : (col ? 1 : 0); break;
        case FMT_GBRG: type = row ? (col ? 1 : 0) : (col ? 3 : 2); break;
        default: type = row ? (col ? 0 : 1) : (col ? 2 : 3); break;  // BGGR
    }
    int r, g, b;
    switch (type) {
        case 0: r = p[12]; g = mhc(p, 0) / 64; b = mhc(p, 1) / 64; break;
        case 1: r = mhc(p, 2) / 64; g = p[12]; b = mhc(p, 3) / 64; break;
        case 2: r = mhc(p, 3) / 64; g = p[12]; b = mhc(p, 2) / 64; break;
        default: r = mhc(p, 1) / 64; g = mhc(p, 0) / 64; b = p[12]; break;
    }
    const float s = static_cast<float>(1.0 / 255.0);
    return make_float4(__fmul_rn(static_cast<float>(r), s), __fmul_rn(static_cast<float>(g), s),
                       __fmul_rn(static_cast<float>(b), s), __fmul_rn(255.0f, s));
}

// cpp/visualmesh/engine/cpu/pixel.hpp:44-58: the two formats of four bytes per pixel
__device__ __forceinline__ float4 get_pixel_packed4(int x, int y, const uint8_t* image, int W, bool bgra) {
    const float s    = static_cast<float>(1.0 / 255.0);
    const uint8_t* c = image + (static_cast<size_t>(y) * W + x) * 4;
    uchar4 v;
    if ((reinterpret_cast<uintptr_t>(image) & 3) == 0) { v = __ldg(reinterpret_cast<const uchar4*>(c)); }
    else {
        v = make_uchar4(__ldg(c), __ldg(c + 1), __ldg(c + 2), __ldg(c + 3));
    }
    const float a0 = __fmul_rn(static_cast<float>(v.x), s);
    const float a1 = __fmul_rn(static_cast<float>(v.y), s);
    const float a2 = __fmul_rn(static_cast<float>(v.z), s);
    const float a3 = __fmul_rn(static_cast<float>(v.w), s);
    return bgra ? make_float4(a2, a1, a0, a3) : make_float4(a0, a1, a2, a3);
}

// cpp/visualmesh/engine/cpu/pixel.hpp:44-102
__device__ __forceinline__ float4 get_pixel(int x, int y, const uint8_t* image, int W, int H, int cls) {
    const float s = static_cast<float>(1.0 / 255.0);
    switch (cls) {
        case FMT_RGBA:
        case FMT_BGRA: return get_pixel_packed4(x, y, image, W, cls == FMT_BGRA);
        case FMT_RGB3:
        case FMT_BGR3: {
            const uint8_t* c = image + (static_cast<size_t>(y) * W + x) * 3;
            const float a0   = __fmul_rn(static_cast<float>(__ldg(c)), s);
            const float a1   = __fmul_rn(static_cast<float>(__ldg(c + 1)), s);
            const float a2   = __fmul_rn(static_cast<float>(__ldg(c + 2)), s);
            return cls == FMT_RGB3 ? make_float4(a0, a1, a2, 1.0f) : make_float4(a2, a1, a0, 1.0f);
        }
        case FMT_GREY: {
            const float a = __fmul_rn(static_cast<float>(__ldg(image + static_cast<size_t>(y) * W + x)), s);
            return make_float4(a, a, a, 1.0f);
        }
        default: return bayer_pixel(x, y, image, W, H, cls);
    }
}

// cpp/visualmesh/engine/cpu/pixel.hpp:116-144; fetch(x, y) returns the pixel at integer coordinates
template <class Fetch>
__device__ __forceinline__ float4 interpolate_with(float2 P, int W, int H, Fetch fetch) {
    const float x = P.x;
    const float y = P.y;
    const int x1  = max(static_cast<int>(floorf(x)), 0);
    const int y1  = max(static_cast<int>(floorf(y)), 0);
    const int x2  = min(x1 + 1, W - 1);
    const int y2  = min(y1 + 1, H - 1);
    const float4 Q1 = fetch(x1, y1);
    const float4 Q2 = fetch(x2, y1);
    const float4 Q3 = fetch(x1, y2);
    const float4 Q4 = fetch(x2, y2);
    const float dx  = static_cast<float>(x2 - x1);
    const float dy  = static_cast<float>(y2 - y1);
    const float wx0 = __fdiv_rn(__fsub_rn(static_cast<float>(x2), x), dx);
    const float wx1 = __fdiv_rn(__fsub_rn(x, static_cast<float>(x1)), dx);
    const float wy0 = __fdiv_rn(__fsub_rn(static_cast<float>(y2), y), dy);
    const float wy1 = __fdiv_rn(__fsub_rn(y, static_cast<float>(y1)), dy);
#define VM_BLEND(c)                                                                                       \
    __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(Q1.c, wx0), __fmul_rn(Q2.c, wx1)), wy0),                      \
              __fmul_rn(__fadd_rn(__fmul_rn(Q3.c, wx0), __fmul_rn(Q4.c, wx1)), wy1))
    const float4 out = make_float4(VM_BLEND(x), VM_BLEND(y), VM_BLEND(z), VM_BLEND(w));
#undef VM_BLEND
    return out;
}
__device__ __forceinline__ float4 interpolate(float2 P, const uint8_t* image, int W, int H, int cls) {
    return interpolate_with(P, W, H, [=](int x, int y) { return get_pixel(x, y, image, W, H, cls); });
}
// the same for an image that is known to be RGBA or BGRA: a fraction of the registers of the general sampler
__device__ __forceinline__ float4 interpolate_packed4(float2 P, const uint8_t* image, int W, int H, bool bgra) {
    return interpolate_with(P, W, H, [=](int x, int y) { return get_pixel_packed4(x, y, image, W, bgra); });
}

}  // namespace vm
