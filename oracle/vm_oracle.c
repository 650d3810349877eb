/*
 * TEST INFRASTRUCTURE - not part of the product. Only tests/, the smoke check and the CPU-baseline leg of the
 * benchmark may load this file's library; the CUDA engine never does.
 *
 * A plain-C, single-threaded restatement of the reference CPU path, function by function, with the reference's
 * operation order and rounding (build with -ffp-contract=off; float expressions stay in float, the one
 * double-promoted sum of distort()/undistort() stays in double). Transcendentals are the host libm's, as in the
 * reference.
 *
 * Parity of this restatement is PINNED: the reference publishes no golden vectors for this path, so it is checked
 * bit for bit against the reference itself compiled in place (oracle/_ref/libvmref.so) by tests/test_oracle.py, and
 * against fixtures generated from that library (tests/golden/).
 */
#define _GNU_SOURCE
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "vmcuda.h"

#define VMO_EXPORT __attribute__((visibility("default")))

/* ---- cpp/visualmesh/utility/math.hpp -------------------------------------------------------------------------- */

/* math.hpp:160-177: dot = a[L-1]*b[L-1] + (... + a[0]*b[0]) */
static float dot3(const float* a, const float* b) {
    return a[2] * b[2] + (a[1] * b[1] + a[0] * b[0]);
}
static float dot2(const float* a, const float* b) {
    return a[1] * b[1] + a[0] * b[0];
}
/* math.hpp:254-257 */
static void matvec3(const float m[3][3], const float* v, float* out) {
    out[0] = dot3(m[0], v);
    out[1] = dot3(m[1], v);
    out[2] = dot3(m[2], v);
}
/* math.hpp:182-195 */
static void normalise3(const float* a, float* out) {
    const float len = 1.0f / sqrtf(dot3(a, a));
    out[0]          = a[0] * len;
    out[1]          = a[1] * len;
    out[2]          = a[2] * len;
}
/* math.hpp:200-207 */
static void cross3(const float* a, const float* b, float* out) {
    out[0] = a[1] * b[2] - a[2] * b[1];
    out[1] = a[2] * b[0] - a[0] * b[2];
    out[2] = a[0] * b[1] - a[1] * b[0];
}
/* math.hpp:280-305 */
static void invert3(const float m[3][3], float o[3][3]) {
    const float det = (m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) - m[0][1] * (m[1][0] * m[2][2] - m[1][2] * m[2][0])
                       + m[0][2] * (m[1][0] * m[2][1] - m[1][1] * m[2][0]));
    if (det == 0) {
        for (int i = 0; i < 3; ++i)
            for (int j = 0; j < 3; ++j) o[i][j] = NAN;
        return;
    }
    const float idet = 1.0f / det;
    o[0][0]          = (m[1][1] * m[2][2] - m[2][1] * m[1][2]) * idet;
    o[0][1]          = (m[0][2] * m[2][1] - m[0][1] * m[2][2]) * idet;
    o[0][2]          = (m[0][1] * m[1][2] - m[0][2] * m[1][1]) * idet;
    o[1][0]          = (m[1][2] * m[2][0] - m[1][0] * m[2][2]) * idet;
    o[1][1]          = (m[0][0] * m[2][2] - m[0][2] * m[2][0]) * idet;
    o[1][2]          = (m[1][0] * m[0][2] - m[0][0] * m[1][2]) * idet;
    o[2][0]          = (m[1][0] * m[2][1] - m[2][0] * m[1][1]) * idet;
    o[2][1]          = (m[2][0] * m[0][1] - m[0][0] * m[2][1]) * idet;
    o[2][2]          = (m[0][0] * m[1][1] - m[1][0] * m[0][1]) * idet;
}

/* ---- cpp/visualmesh/utility/projection.hpp -------------------------------------------------------------------- */

/* projection.hpp:80-87 */
static void inverse_coefficients(const float* k, float* ik) {
    ik[0] = -k[0];
    ik[1] = 3.0f * (k[0] * k[0]) - k[1];
    ik[2] = -12.0f * (k[0] * k[0]) * k[0] + 8.0f * k[0] * k[1];
    ik[3] = 55.0f * (k[0] * k[0]) * (k[0] * k[0]) - 55.0f * (k[0] * k[0]) * k[1] + 5.0f * (k[1] * k[1]);
}

/* projection.hpp:105-120. The literal 1.0 is a double: each ik[j] * (r...) product is a float, the running sum and
 * the final product with r are double, rounded to float once on return. */
static float distort(float r, const float* k) {
    float ik[4];
    inverse_coefficients(k, ik);
    return (float) (r
                    * (1.0 + ik[0] * (r * r) + ik[1] * ((r * r) * (r * r)) + ik[2] * ((r * r) * (r * r)) * (r * r)
                       + ik[3] * ((r * r) * (r * r)) * ((r * r) * (r * r))));
}

/* projection.hpp:138-143 */
static float undistort(float r, const float* k) {
    return (float) (r * (1.0 + k[0] * (r * r) + k[1] * ((r * r) * (r * r))));
}

/* projection.hpp:163-187. Returns 0, or -1 for an unknown projection. */
static int project(const float* ray, const vm_lens* lens, float* px) {
    const float f          = lens->focal_length;
    const float theta      = acosf(ray[0]);
    const float rsin_theta = 1.0f / sqrtf(1.0f - ray[0] * ray[0]);
    float r_u;
    switch (lens->projection) {
        case VM_RECTILINEAR: {
            /* std::min(std::max(theta, 0), pi/2) with std::min/max's NaN behaviour (projection.hpp:52-54) */
            float t          = (theta < 0.0f) ? 0.0f : theta;
            const float pi_2 = (float) M_PI_2;
            t                = (pi_2 < t) ? pi_2 : t;
            r_u              = f * tanf(t);
        } break;
        case VM_EQUISOLID: r_u = 2.0f * f * sinf(theta * 0.5f); break; /* projection.hpp:40-42 */
        case VM_EQUIDISTANT: r_u = f * theta; break;                    /* projection.hpp:28-30 */
        default: return -1;
    }
    const float r_d = distort(r_u, lens->k);
    float screen[2];
    if (ray[0] >= 1) {
        screen[0] = 0.0f;
        screen[1] = 0.0f;
    }
    else {
        screen[0] = r_d * ray[1] * rsin_theta;
        screen[1] = r_d * ray[2] * rsin_theta;
    }
    px[0] = ((float) lens->dimensions[0] * 0.5f - screen[0]) - lens->centre[0];
    px[1] = ((float) lens->dimensions[1] * 0.5f - screen[1]) - lens->centre[1];
    return 0;
}

/* projection.hpp:205-225 */
static int unproject(const float* px, const vm_lens* lens, float* ray) {
    float screen[2];
    screen[0]       = (float) lens->dimensions[0] * 0.5f - (px[0] + lens->centre[0]);
    screen[1]       = (float) lens->dimensions[1] * 0.5f - (px[1] + lens->centre[1]);
    const float f   = lens->focal_length;
    const float r_d = sqrtf(dot2(screen, screen));
    if (r_d == 0) {
        ray[0] = 1.0f;
        ray[1] = 0.0f;
        ray[2] = 0.0f;
        return 0;
    }
    const float r_u = undistort(r_d, lens->k);
    float theta;
    switch (lens->projection) {
        case VM_RECTILINEAR: theta = atanf(r_u / f); break;
        case VM_EQUISOLID: theta = 2.0f * asinf(r_u / (2.0f * f)); break;
        case VM_EQUIDISTANT: theta = r_u / f; break;
        default: return -1;
    }
    const float sin_theta = sinf(theta);
    ray[0]                = cosf(theta);
    ray[1]                = sin_theta * screen[0] / r_d;
    ray[2]                = sin_theta * screen[1] / r_d;
    return 0;
}

VMO_EXPORT int vmo_project_rays(const float* rays, int n, const vm_lens* lens, float* px) {
    for (int i = 0; i < n; ++i)
        if (project(rays + 3 * i, lens, px + 2 * i) != 0) return -1;
    return 0;
}

VMO_EXPORT int vmo_unproject(const float* px, int n, const vm_lens* lens, float* rays) {
    for (int i = 0; i < n; ++i)
        if (unproject(px + 2 * i, lens, rays + 3 * i) != 0) return -1;
    return 0;
}

/* ---- cpp/visualmesh/utility/cone.hpp -------------------------------------------------------------------------- */

/* cone.hpp:79-99: the cone through three unit vectors: axis xyz and cos of the half angle */
static void cone_from_3(const float* p1, const float* p2, const float* p3, float* axis, float* cos_theta) {
    const float mat[3][3] = {{p1[0], p1[1], p1[2]}, {p2[0], p2[1], p2[2]}, {p3[0], p3[1], p3[2]}};
    float imat[3][3];
    invert3(mat, imat);
    const float ones[3] = {1.0f, 1.0f, 1.0f};
    const float raw[3]  = {dot3(imat[0], ones), dot3(imat[1], ones), dot3(imat[2], ones)};
    normalise3(raw, axis);
    *cos_theta = dot3(axis, p1);
}

/* ---- cpp/visualmesh/mesh.hpp: per-frame lookup ------------------------------------------------------------------ */

typedef struct {
    float axis[3];
    float cs[2]; /* cos, sin */
} vmo_cone;

/* mesh.hpp:265-349 */
static int screen_edges(const float* Hoc, const vm_lens* lens, vmo_cone edges[4]) {
    const float Roc[3][3] = {{Hoc[0], Hoc[1], Hoc[2]}, {Hoc[4], Hoc[5], Hoc[6]}, {Hoc[8], Hoc[9], Hoc[10]}};
    const float dims[2]   = {(float) lens->dimensions[0] - 1.0f, (float) lens->dimensions[1] - 1.0f};
    const float corners[4][2] = {{1.0f, 1.0f}, {dims[0], 1.0f}, {dims[0], dims[1]}, {1.0f, dims[1]}};
    float rNCo[4][3];
    for (int i = 0; i < 4; ++i) {
        float cam[3];
        if (unproject(corners[i], lens, cam) != 0) return -1;
        matvec3(Roc, cam, rNCo[i]);
    }
    switch (lens->projection) {
        case VM_RECTILINEAR: {
            const int a[4] = {1, 2, 3, 0};
            const int b[4] = {0, 1, 2, 3};
            for (int i = 0; i < 4; ++i) {
                float c[3];
                cross3(rNCo[a[i]], rNCo[b[i]], c);
                normalise3(c, edges[i].axis);
                edges[i].cs[0] = 0.0f;
                edges[i].cs[1] = 1.0f;
            }
            return 0;
        }
        case VM_EQUIDISTANT:
        case VM_EQUISOLID: {
            const float centre[2]   = {dims[0] * 0.5f + lens->centre[0], dims[1] * 0.5f + lens->centre[1]};
            const float mids[4][2]  = {{centre[0], 1.0f}, {dims[0], centre[1]}, {centre[0], dims[1]}, {1.0f, centre[1]}};
            float rECo[4][3];
            for (int i = 0; i < 4; ++i) {
                float cam[3];
                if (unproject(mids[i], lens, cam) != 0) return -1;
                matvec3(Roc, cam, rECo[i]);
            }
            const int a[4] = {1, 2, 3, 0};
            const int b[4] = {0, 1, 2, 3};
            for (int i = 0; i < 4; ++i) {
                float c;
                cone_from_3(rNCo[a[i]], rECo[i], rNCo[b[i]], edges[i].axis, &c);
                edges[i].cs[0] = c;
                edges[i].cs[1] = sqrtf(1.0f - c * c);
            }
            return 0;
        }
        default: return -1;
    }
}

/* mesh.hpp:362-406 */
static void check_on_screen(const float Rco[3][3],
                            const float* axis,
                            const float* cs,
                            const vm_lens* lens,
                            const vmo_cone edges[4],
                            int* inside,
                            int* outside) {
    float cam[3], px[2];
    matvec3(Rco, axis, cam);
    project(cam, lens, px);
    const int axis_on_screen =
      0 <= px[0] && px[0] + 1 <= lens->dimensions[0] && 0 <= px[1] && px[1] + 1 <= lens->dimensions[1];
    float angles[4];
    int contains = 0;
    for (int i = 0; i < 4; ++i) {
        angles[i] = dot3(axis, edges[i].axis);
        contains |= angles[i] > edges[i].cs[0] * cs[0] + edges[i].cs[1] * cs[1];
    }
    if (!axis_on_screen && contains) {
        *inside  = 0;
        *outside = 1;
        return;
    }
    int intersects = 1;
    for (int i = 0; i < 4; ++i) { intersects &= angles[i] < edges[i].cs[0] * cs[0] - edges[i].cs[1] * cs[1]; }
    *inside  = axis_on_screen && intersects;
    *outside = 0;
}

/* mesh.hpp:499-595. BSP given as flat arrays: element ranges [n][2], children [n][2], cones [n][5] = axis, cos, sin.
 * Writes up to capacity [start,end) pairs and returns the number of ranges (which may exceed capacity), or -1. */
VMO_EXPORT int vmo_lookup(const float* rays,
                          const int32_t* bsp_ranges,
                          const int32_t* bsp_children,
                          const float* bsp_cones,
                          int n_bsp,
                          const float* Hoc,
                          const vm_lens* lens,
                          int32_t* out_ranges,
                          int capacity) {
    const float cos_fov = cosf(lens->fov * 0.5f);
    const float sin_fov = sinf(lens->fov * 0.5f);
    /* Rco = block<3,3>(transpose(Hoc)): Rco[i][j] = Hoc[j][i] */
    const float Rco[3][3] = {{Hoc[0], Hoc[4], Hoc[8]}, {Hoc[1], Hoc[5], Hoc[9]}, {Hoc[2], Hoc[6], Hoc[10]}};
    const float* rXCo     = Rco[0];
    vmo_cone edges[4];
    if (screen_edges(Hoc, lens, edges) != 0) return -1;

    int cap_stack = 64, top = 0;
    int* stack    = (int*) malloc(sizeof(int) * cap_stack);
    int n_out = 0, building = 0, range_start = 0, range_end = 0;
    if (n_bsp > 0) stack[top++] = 0;

#define EMIT()                                        \
    do {                                              \
        if (n_out < capacity) {                       \
            out_ranges[2 * n_out + 0] = range_start;  \
            out_ranges[2 * n_out + 1] = range_end;    \
        }                                             \
        ++n_out;                                      \
    } while (0)

    while (top > 0) {
        const int e       = stack[--top];
        const float* cone = bsp_cones + 5 * e;
        const float delta = dot3(rXCo, cone);
        int outside       = delta < cos_fov * cone[3] - sin_fov * cone[4];
        int inside        = delta > cos_fov * cone[3] + sin_fov * cone[4];
        if (!outside && inside) { check_on_screen(Rco, cone, cone + 3, lens, edges, &inside, &outside); }

        if (inside) {
            if (building) { range_end = bsp_ranges[2 * e + 1]; }
            else {
                range_start = bsp_ranges[2 * e + 0];
                range_end   = bsp_ranges[2 * e + 1];
                building    = 1;
            }
        }
        else if (outside) {
            if (building) {
                EMIT();
                building = 0;
            }
        }
        else if (bsp_children[2 * e + 0] < 0) {
            for (int i = bsp_ranges[2 * e + 0]; i < bsp_ranges[2 * e + 1]; ++i) {
                float cam[3], px[2];
                matvec3(Rco, rays + 3 * i, cam);
                project(cam, lens, px);
                const int on_screen = dot3(rXCo, rays + 3 * i) > cos_fov && 0 <= px[0]
                                      && px[0] + 1 <= lens->dimensions[0] && 0 <= px[1]
                                      && px[1] + 1 <= lens->dimensions[1];
                if (on_screen && building) { range_end = i + 1; }
                else if (!on_screen && building) {
                    EMIT();
                    building = 0;
                }
                else if (on_screen && !building) {
                    range_start = i;
                    range_end   = i + 1;
                    building    = 1;
                }
            }
        }
        else {
            if (top + 2 > cap_stack) {
                cap_stack *= 2;
                stack = (int*) realloc(stack, sizeof(int) * cap_stack);
            }
            stack[top++] = bsp_children[2 * e + 1];
            stack[top++] = bsp_children[2 * e + 0];
        }
    }
    if (building) { EMIT(); }
#undef EMIT
    free(stack);
    return n_out;
}

/* ---- cpp/visualmesh/engine/cpu/engine.hpp:85-147: project, filter, remap -------------------------------------- */

/* rays [n_nodes][3], neighbours [n_nodes][N]. Outputs sized for the sum of the range lengths: px [n][2],
 * global_indices [n], neighbourhood [n+1][N]. Returns n, or -1. */
VMO_EXPORT int vmo_project_mesh(const float* rays,
                                const int32_t* neighbours,
                                int n_nodes,
                                int N,
                                const int32_t* ranges,
                                int n_ranges,
                                const float* Hoc,
                                const vm_lens* lens,
                                float* px_out,
                                int32_t* global_indices,
                                int32_t* neighbourhood) {
    const float Rco[3][3] = {{Hoc[0], Hoc[4], Hoc[8]}, {Hoc[1], Hoc[5], Hoc[9]}, {Hoc[2], Hoc[6], Hoc[10]}};
    int n                 = 0;
    for (int r = 0; r < n_ranges; ++r) {
        for (int i = ranges[2 * r]; i < ranges[2 * r + 1]; ++i) {
            float cam[3], px[2];
            matvec3(Rco, rays + 3 * i, cam);
            if (project(cam, lens, px) != 0) return -1;
            if (0 <= px[0] && px[0] + 1 < lens->dimensions[0] && 0 <= px[1] && px[1] + 1 < lens->dimensions[1]) {
                global_indices[n] = i;
                px_out[2 * n]     = px[0];
                px_out[2 * n + 1] = px[1];
                ++n;
            }
        }
    }
    int32_t* r_lookup = (int32_t*) malloc(sizeof(int32_t) * ((size_t) n_nodes + 1));
    for (int i = 0; i <= n_nodes; ++i) r_lookup[i] = n;
    for (int i = 0; i < n; ++i) r_lookup[global_indices[i]] = i;
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < N; ++j) neighbourhood[(size_t) i * N + j] = r_lookup[neighbours[(size_t) global_indices[i] * N + j]];
    for (int j = 0; j < N; ++j) neighbourhood[(size_t) n * N + j] = n;
    free(r_lookup);
    return n;
}

/* ---- cpp/visualmesh/engine/cpu/bayer.hpp, pixel.hpp ------------------------------------------------------------ */

#define FCC(a, b, c, d) ((uint32_t) (a) | ((uint32_t) (b) << 8) | ((uint32_t) (c) << 16) | ((uint32_t) (d) << 24))

/* bayer.hpp:45-83, scaled by 64 */
static const int G_R[25]  = {0, 0, -8, 0, 0, 0, 0, 16, 0, 0, -8, 16, 32, 16, -8, 0, 0, 16, 0, 0, 0, 0, -8, 0, 0};
static const int R_B[25]  = {0, 0, -12, 0, 0, 0, 16, 0, 16, 0, -12, 0, 48, 0, -12, 0, 16, 0, 16, 0, 0, 0, -12, 0, 0};
static const int R_GR[25] = {0, 0, 4, 0, 0, 0, -8, 0, -8, 0, -8, 32, 40, 32, -8, 0, -8, 0, -8, 0, 0, 0, 4, 0, 0};
static const int R_GB[25] = {0, 0, -8, 0, 0, 0, -8, 32, -8, 0, 4, 0, 40, 0, 4, 0, -8, 32, -8, 0, 0, 0, -8, 0, 0};
#define G_B G_R
#define B_R R_B
#define B_GB R_GR
#define B_GR R_GB

static int idot25(const int* p, const int* k) {
    int s = 0;
    for (int i = 0; i < 25; ++i) s += p[i] * k[i];
    return s;
}

enum { PX_R, PX_GR, PX_GB, PX_B };

/* bayer.hpp:96-108 (integer division truncates toward zero; no clamp) and :123-158 */
static int bayer_pixel(int x, int y, const uint8_t* image, int W, int H, uint32_t format, float* out) {
    int p[25];
    for (int dy = 0; dy < 5; ++dy) {
        int yc = y - 2 + dy;
        yc     = yc < 0 ? 0 : (yc > H - 1 ? H - 1 : yc);
        for (int dx = 0; dx < 5; ++dx) {
            int xc = x - 2 + dx;
            xc     = xc < 0 ? 0 : (xc > W - 1 ? W - 1 : xc);
            p[dy * 5 + dx] = image[(size_t) yc * W + xc];
        }
    }
    const int col = x % 2 == 1;
    const int row = y % 2 == 1;
    int type;
    switch (format) {
        case FCC('G', 'R', 'B', 'G'): type = row ? (col ? PX_GB : PX_B) : (col ? PX_R : PX_GR); break;
        case FCC('R', 'G', 'G', 'B'): type = row ? (col ? PX_B : PX_GB) : (col ? PX_GR : PX_R); break;
        case FCC('G', 'B', 'R', 'G'): type = row ? (col ? PX_GR : PX_R) : (col ? PX_B : PX_GB); break;
        case FCC('B', 'G', 'G', 'R'): type = row ? (col ? PX_R : PX_GR) : (col ? PX_GB : PX_B); break;
        default: return -1;
    }
    int o[4];
    switch (type) {
        case PX_R: o[0] = p[12]; o[1] = idot25(p, G_R) / 64; o[2] = idot25(p, B_R) / 64; break;
        case PX_GR: o[0] = idot25(p, R_GR) / 64; o[1] = p[12]; o[2] = idot25(p, B_GR) / 64; break;
        case PX_GB: o[0] = idot25(p, R_GB) / 64; o[1] = p[12]; o[2] = idot25(p, B_GB) / 64; break;
        default: o[0] = idot25(p, R_B) / 64; o[1] = idot25(p, G_B) / 64; o[2] = p[12]; break;
    }
    o[3] = 255;
    for (int c = 0; c < 4; ++c) out[c] = (float) o[c] * (float) (1.0 / 255.0);
    return 0;
}

/* pixel.hpp:44-102 */
static int get_pixel(int x, int y, const uint8_t* image, int W, int H, uint32_t format, float* out) {
    const float s = (float) (1.0 / 255.0);
    switch (format) {
        case FCC('G', 'R', 'B', 'G'):
        case FCC('R', 'G', 'G', 'B'):
        case FCC('G', 'B', 'R', 'G'):
        case FCC('B', 'G', 'G', 'R'): return bayer_pixel(x, y, image, W, H, format, out);
        case FCC('B', 'G', 'R', '3'):
        case FCC('B', 'G', 'R', '8'): {
            const size_t c = ((size_t) y * W + x) * 3;
            out[0] = image[c + 2] * s; out[1] = image[c + 1] * s; out[2] = image[c + 0] * s; out[3] = 1.0f;
            return 0;
        }
        case FCC('B', 'G', 'R', 'A'): {
            const size_t c = ((size_t) y * W + x) * 4;
            out[0] = image[c + 2] * s; out[1] = image[c + 1] * s; out[2] = image[c + 0] * s; out[3] = image[c + 3] * s;
            return 0;
        }
        case FCC('R', 'G', 'B', '3'):
        case FCC('R', 'G', 'B', '8'): {
            const size_t c = ((size_t) y * W + x) * 3;
            out[0] = image[c + 0] * s; out[1] = image[c + 1] * s; out[2] = image[c + 2] * s; out[3] = 1.0f;
            return 0;
        }
        case FCC('R', 'G', 'B', 'A'): {
            const size_t c = ((size_t) y * W + x) * 4;
            out[0] = image[c + 0] * s; out[1] = image[c + 1] * s; out[2] = image[c + 2] * s; out[3] = image[c + 3] * s;
            return 0;
        }
        case FCC('G', 'R', 'A', 'Y'):
        case FCC('G', 'R', 'E', 'Y'):
        case FCC('Y', '8', ' ', ' '): {
            const size_t c = (size_t) y * W + x;
            out[0] = image[c] * s; out[1] = image[c] * s; out[2] = image[c] * s; out[3] = 1.0f;
            return 0;
        }
        default: return -1;
    }
}

/* pixel.hpp:116-144 */
static int interpolate(const float* P, const uint8_t* image, int W, int H, uint32_t format, float* out) {
    const float x = P[0];
    const float y = P[1];
    int x1        = (int) floorf(P[0]);
    int y1        = (int) floorf(P[1]);
    x1            = x1 < 0 ? 0 : x1;
    y1            = y1 < 0 ? 0 : y1;
    const int x2  = (x1 + 1 < W - 1) ? x1 + 1 : W - 1;
    const int y2  = (y1 + 1 < H - 1) ? y1 + 1 : H - 1;
    float Q1[4], Q2[4], Q3[4], Q4[4];
    if (get_pixel(x1, y1, image, W, H, format, Q1) != 0) return -1;
    get_pixel(x2, y1, image, W, H, format, Q2);
    get_pixel(x1, y2, image, W, H, format, Q3);
    get_pixel(x2, y2, image, W, H, format, Q4);
    const float wx0 = ((float) x2 - x) / (float) (x2 - x1);
    const float wx1 = (x - (float) x1) / (float) (x2 - x1);
    const float wy0 = ((float) y2 - y) / (float) (y2 - y1);
    const float wy1 = (y - (float) y1) / (float) (y2 - y1);
    for (int c = 0; c < 4; ++c) {
        const float R1 = Q1[c] * wx0 + Q2[c] * wx1;
        const float R2 = Q3[c] * wx0 + Q4[c] * wx1;
        out[c]         = R1 * wy0 + R2 * wy1;
    }
    return 0;
}

VMO_EXPORT int vmo_interpolate(const float* px, int n, const void* image, int W, int H, uint32_t format, float* out) {
    for (int i = 0; i < n; ++i)
        if (interpolate(px + 2 * i, (const uint8_t*) image, W, H, format, out + 4 * i) != 0) return -1;
    return 0;
}

/* ---- cpp/visualmesh/engine/cpu/engine.hpp:206-265 and apply_activation.hpp ----------------------------------- */

/* apply_activation.hpp:35-64 over rows x dims values */
static void apply_activation(int fn, float* data, size_t rows, int dims) {
    const size_t total = rows * (size_t) dims;
    switch (fn) {
        case VM_SELU: {
            const float lambda = 1.0507009873554804934193349852946;
            const float alpha  = 1.6732632423543772848170429916717;
            for (size_t i = 0; i < total; ++i) {
                const float s = data[i];
                data[i]       = lambda * (s >= 0 ? s : alpha * expf(s) - alpha);
            }
        } break;
        case VM_RELU:
            for (size_t i = 0; i < total; ++i) data[i] = (data[i] < 0.0f) ? 0.0f : data[i]; /* std::max(s, 0) */
            break;
        case VM_TANH:
            for (size_t i = 0; i < total; ++i) data[i] = tanhf(data[i]);
            break;
        case VM_SOFTMAX:
            for (size_t i = 0; i < total; ++i) data[i] = expf(data[i]);
            for (size_t r = 0; r < rows; ++r) {
                float* row  = data + r * dims;
                float total_ = 0.0f;
                for (int j = 0; j < dims; ++j) total_ = total_ + row[j];
                for (int j = 0; j < dims; ++j) row[j] = row[j] / total_;
            }
            break;
        default: break;
    }
}

/* engine.hpp:213-265. input: n_rows x 4 (last row = off-screen row). Returns the output width, writes
 * n_rows x width floats to out (which must hold n_rows * max layer width), or -1 on a shape error. */
VMO_EXPORT int vmo_network(const float* input,
                           const int32_t* neighbourhood,
                           int n_rows,
                           int N,
                           const vm_layer* layers,
                           const int32_t* layers_per_group,
                           int n_groups,
                           float* out) {
    int dims   = 4;
    float* cur = (float*) malloc(sizeof(float) * (size_t) n_rows * 4);
    memcpy(cur, input, sizeof(float) * (size_t) n_rows * 4);
    int l = 0;
    for (int g = 0; g < n_groups; ++g) {
        /* gather: self then the neighbours in stored order (engine.hpp:222-231) */
        const int gdims = dims * (N + 1);
        float* gathered = (float*) malloc(sizeof(float) * (size_t) n_rows * gdims);
        for (int i = 0; i < n_rows; ++i) {
            float* dst = gathered + (size_t) i * gdims;
            memcpy(dst, cur + (size_t) i * dims, sizeof(float) * dims);
            for (int j = 0; j < N; ++j) {
                const int nb = neighbourhood[(size_t) i * N + j];
                memcpy(dst + (size_t) (j + 1) * dims, cur + (size_t) nb * dims, sizeof(float) * dims);
            }
        }
        free(cur);
        cur  = gathered;
        dims = gdims;
        for (int k = 0; k < layers_per_group[g]; ++k, ++l) {
            const vm_layer* L = &layers[l];
            if (L->n_in != dims) {
                free(cur);
                return -1;
            }
            const int od = L->n_out;
            float* next  = (float*) malloc(sizeof(float) * (size_t) n_rows * od);
            for (int i = 0; i < n_rows; ++i) {
                const float* in = cur + (size_t) i * dims;
                for (int j = 0; j < od; ++j) {
                    /* std::inner_product(in, in + dims, W^T[j], bias[j]) (engine.hpp:250-256) */
                    float acc = L->biases[j];
                    for (int q = 0; q < dims; ++q) acc = acc + in[q] * L->weights[(size_t) q * od + j];
                    next[(size_t) i * od + j] = acc;
                }
            }
            apply_activation(L->activation, next, (size_t) n_rows, od);
            free(cur);
            cur  = next;
            dims = od;
        }
    }
    memcpy(out, cur, sizeof(float) * (size_t) n_rows * dims);
    free(cur);
    return dims;
}

/* The whole call: engine.hpp:181-273. Returns n (0 = empty result), or -1. classifications gets (n+1) x n_classes. */
VMO_EXPORT int vmo_classify(const float* rays,
                            const int32_t* neighbours,
                            int n_nodes,
                            int N,
                            const int32_t* ranges,
                            int n_ranges,
                            const float* Hoc,
                            const vm_lens* lens,
                            const void* image,
                            uint32_t format,
                            const vm_layer* layers,
                            const int32_t* layers_per_group,
                            int n_groups,
                            float* px_out,
                            int32_t* global_indices,
                            int32_t* neighbourhood,
                            float* classifications,
                            int* n_classes) {
    const int n = vmo_project_mesh(rays, neighbours, n_nodes, N, ranges, n_ranges, Hoc, lens, px_out, global_indices, neighbourhood);
    if (n <= 0) return n;
    float* input = (float*) malloc(sizeof(float) * ((size_t) n + 1) * 4);
    if (vmo_interpolate(px_out, n, image, lens->dimensions[0], lens->dimensions[1], format, input) != 0) {
        free(input);
        return -1;
    }
    for (int c = 0; c < 4; ++c) input[(size_t) n * 4 + c] = -1.0f; /* engine.hpp:206 */
    int max_w = 4;
    int l     = 0;
    for (int g = 0; g < n_groups; ++g)
        for (int k = 0; k < layers_per_group[g]; ++k, ++l) max_w = layers[l].n_out > max_w ? layers[l].n_out : max_w;
    float* tmp = (float*) malloc(sizeof(float) * ((size_t) n + 1) * max_w);
    const int w = vmo_network(input, neighbourhood, n + 1, N, layers, layers_per_group, n_groups, tmp);
    if (w > 0) memcpy(classifications, tmp, sizeof(float) * ((size_t) n + 1) * w);
    if (n_classes != NULL) *n_classes = w;
    free(tmp);
    free(input);
    return w < 0 ? -1 : n;
}
