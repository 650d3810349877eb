// Host-side float arithmetic shared by the engine (per-frame constants) and the host mesh tables (lookup).
//
// These are the small pieces of the reference that run once per frame or per BSP element on the host. They follow
// the reference's operation order in single precision and use the host libm, so their results are the reference's
// bit for bit. Compile with -ffp-contract=off.
#pragma once

#include <array>
#include <cmath>
#include <cstdint>

#include "../../include/vmcuda.h"

namespace vm {
namespace host {

    using v2 = std::array<float, 2>;
    using v3 = std::array<float, 3>;
    using m3 = std::array<v3, 3>;

    struct Cone {
        v3 axis;
        float cos_t;
        float sin_t;
    };

    // cpp/visualmesh/utility/math.hpp:160-177: the last product is added to the sum of the ones before it
    inline float dot(const v3& a, const v3& b) {
        return a[2] * b[2] + (a[1] * b[1] + a[0] * b[0]);
    }
    inline float dot(const v2& a, const v2& b) {
        return a[1] * b[1] + a[0] * b[0];
    }
    inline v3 mul(const m3& m, const v3& v) {
        return v3{{dot(m[0], v), dot(m[1], v), dot(m[2], v)}};
    }
    inline v3 normalise(const v3& a) {
        const float len = 1.0f / std::sqrt(dot(a, a));
        return v3{{a[0] * len, a[1] * len, a[2] * len}};
    }
    inline v3 cross(const v3& a, const v3& b) {
        return v3{{a[1] * b[2] - a[2] * b[1], a[2] * b[0] - a[0] * b[2], a[0] * b[1] - a[1] * b[0]}};
    }
    // cpp/visualmesh/utility/math.hpp:280-305
    inline m3 invert(const m3& m) {
        const float det = (m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) - m[0][1] * (m[1][0] * m[2][2] - m[1][2] * m[2][0])
                           + m[0][2] * (m[1][0] * m[2][1] - m[1][1] * m[2][0]));
        if (det == 0) {
            const float nan = std::nanf("");
            return m3{{v3{{nan, nan, nan}}, v3{{nan, nan, nan}}, v3{{nan, nan, nan}}}};
        }
        const float idet = 1.0f / det;
        return m3{{v3{{(m[1][1] * m[2][2] - m[2][1] * m[1][2]) * idet,
                       (m[0][2] * m[2][1] - m[0][1] * m[2][2]) * idet,
                       (m[0][1] * m[1][2] - m[0][2] * m[1][1]) * idet}},
                   v3{{(m[1][2] * m[2][0] - m[1][0] * m[2][2]) * idet,
                       (m[0][0] * m[2][2] - m[0][2] * m[2][0]) * idet,
                       (m[1][0] * m[0][2] - m[0][0] * m[1][2]) * idet}},
                   v3{{(m[1][0] * m[2][1] - m[2][0] * m[1][1]) * idet,
                       (m[2][0] * m[0][1] - m[0][0] * m[2][1]) * idet,
                       (m[0][0] * m[1][1] - m[1][0] * m[0][1]) * idet}}}};
    }

    // cpp/visualmesh/utility/cone.hpp:33-99
    inline std::pair<v3, float> cone_from_points() {
        return {v3{{0, 0, 0}}, 1.0f};
    }
    inline std::pair<v3, float> cone_from_points(const v3& p1) {
        return {p1, 1.0f};
    }
    inline std::pair<v3, float> cone_from_points(const v3& p1, const v3& p2) {
        const v3 axis = normalise(v3{{p1[0] + p2[0], p1[1] + p2[1], p1[2] + p2[2]}});
        return {axis, dot(axis, p1)};
    }
    inline std::pair<v3, float> cone_from_points(const v3& p1, const v3& p2, const v3& p3) {
        const m3 imat = invert(m3{{p1, p2, p3}});
        const v3 ones{{1.0f, 1.0f, 1.0f}};
        const v3 axis = normalise(v3{{dot(imat[0], ones), dot(imat[1], ones), dot(imat[2], ones)}});
        return {axis, dot(axis, p1)};
    }

    // cpp/visualmesh/utility/projection.hpp:80-87
    inline void inverse_coefficients(const float* k, float* ik) {
        ik[0] = -k[0];
        ik[1] = 3.0f * (k[0] * k[0]) - k[1];
        ik[2] = -12.0f * (k[0] * k[0]) * k[0] + 8.0f * k[0] * k[1];
        ik[3] = 55.0f * (k[0] * k[0]) * (k[0] * k[0]) - 55.0f * (k[0] * k[0]) * k[1] + 5.0f * (k[1] * k[1]);
    }
    // cpp/visualmesh/utility/projection.hpp:105-120 - the literal 1.0 makes the bracket a double sum
    inline float distort(float r, const float* k) {
        float ik[4];
        inverse_coefficients(k, ik);
        return static_cast<float>(r
                                  * (1.0 + ik[0] * (r * r) + ik[1] * ((r * r) * (r * r))
                                     + ik[2] * ((r * r) * (r * r)) * (r * r) + ik[3] * ((r * r) * (r * r)) * ((r * r) * (r * r))));
    }
    // cpp/visualmesh/utility/projection.hpp:138-143
    inline float undistort(float r, const float* k) {
        return static_cast<float>(r * (1.0 + k[0] * (r * r) + k[1] * ((r * r) * (r * r))));
    }

    // cpp/visualmesh/utility/projection.hpp:163-187; false for an unknown projection
    inline bool project(const v3& ray, const vm_lens& lens, v2& px) {
        const float f          = lens.focal_length;
        const float theta      = std::acos(ray[0]);
        const float rsin_theta = 1.0f / std::sqrt(1.0f - ray[0] * ray[0]);
        float r_u;
        switch (lens.projection) {
            case VM_RECTILINEAR: r_u = f * std::tan(std::min(std::max(theta, 0.0f), float(M_PI_2))); break;
            case VM_EQUISOLID: r_u = 2.0f * f * std::sin(theta * 0.5f); break;
            case VM_EQUIDISTANT: r_u = f * theta; break;
            default: return false;
        }
        const float r_d = distort(r_u, lens.k);
        const v2 screen = ray[0] >= 1 ? v2{{0.0f, 0.0f}} : v2{{r_d * ray[1] * rsin_theta, r_d * ray[2] * rsin_theta}};
        px[0]           = (float(lens.dimensions[0]) * 0.5f - screen[0]) - lens.centre[0];
        px[1]           = (float(lens.dimensions[1]) * 0.5f - screen[1]) - lens.centre[1];
        return true;
    }

    // cpp/visualmesh/utility/projection.hpp:205-225
    inline bool unproject(const v2& px, const vm_lens& lens, v3& ray) {
        const v2 screen{{float(lens.dimensions[0]) * 0.5f - (px[0] + lens.centre[0]),
                         float(lens.dimensions[1]) * 0.5f - (px[1] + lens.centre[1])}};
        const float f   = lens.focal_length;
        const float r_d = std::sqrt(dot(screen, screen));
        if (r_d == 0) {
            ray = v3{{1.0f, 0.0f, 0.0f}};
            return true;
        }
        const float r_u = undistort(r_d, lens.k);
        float theta;
        switch (lens.projection) {
            case VM_RECTILINEAR: theta = std::atan(r_u / f); break;
            case VM_EQUISOLID: theta = 2.0f * std::asin(r_u / (2.0f * f)); break;
            case VM_EQUIDISTANT: theta = r_u / f; break;
            default: return false;
        }
        const float sin_theta = std::sin(theta);
        ray                   = v3{{std::cos(theta), sin_theta * screen[0] / r_d, sin_theta * screen[1] / r_d}};
        return true;
    }

    // cpp/visualmesh/mesh.hpp:265-349: the four screen-edge cones (planes for a rectilinear lens) in world space
    inline bool screen_edges(const float* Hoc, const vm_lens& lens, std::array<Cone, 4>& edges) {
        const m3 Roc{{v3{{Hoc[0], Hoc[1], Hoc[2]}}, v3{{Hoc[4], Hoc[5], Hoc[6]}}, v3{{Hoc[8], Hoc[9], Hoc[10]}}}};
        const v2 dims{{float(lens.dimensions[0]) - 1.0f, float(lens.dimensions[1]) - 1.0f}};
        const std::array<v2, 4> corners{{v2{{1.0f, 1.0f}}, v2{{dims[0], 1.0f}}, v2{{dims[0], dims[1]}}, v2{{1.0f, dims[1]}}}};
        std::array<v3, 4> rNCo;
        for (int i = 0; i < 4; ++i) {
            v3 cam;
            if (!unproject(corners[i], lens, cam)) return false;
            rNCo[i] = mul(Roc, cam);
        }
        if (lens.projection == VM_RECTILINEAR) {
            for (int i = 0; i < 4; ++i) {
                edges[i].axis  = normalise(cross(rNCo[(i + 1) & 3], rNCo[i]));
                edges[i].cos_t = 0.0f;
                edges[i].sin_t = 1.0f;
            }
            return true;
        }
        const v2 centre{{dims[0] * 0.5f + lens.centre[0], dims[1] * 0.5f + lens.centre[1]}};
        const std::array<v2, 4> mids{{v2{{centre[0], 1.0f}}, v2{{dims[0], centre[1]}}, v2{{centre[0], dims[1]}}, v2{{1.0f, centre[1]}}}};
        for (int i = 0; i < 4; ++i) {
            v3 cam;
            if (!unproject(mids[i], lens, cam)) return false;
            const v3 rECo  = mul(Roc, cam);
            const auto c   = cone_from_points(rNCo[(i + 1) & 3], rECo, rNCo[i]);
            edges[i].axis  = c.first;
            edges[i].cos_t = c.second;
            edges[i].sin_t = std::sqrt(1.0f - c.second * c.second);
        }
        return true;
    }

}  // namespace host
}  // namespace vm
