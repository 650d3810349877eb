// Host-side mesh tables behind the vm_hostmesh_* entry points of include/vmcuda.h.
//
// The engine consumes a mesh as plain tables: unit rays in BSP order, a neighbour table and the BSP itself. C++
// callers take them from the reference's own visualmesh::Mesh object; this file builds the same tables for callers
// that cannot instantiate those templates. It restates, in single precision with the host libm and the same
// standard-library algorithms (so the same permutations), what the reference does once per camera height:
//   model generation   cpp/visualmesh/model/ring_base.hpp:53-115, ring{4,6,8}.hpp, grid_base.hpp:78-144,
//                      xygrid_map.hpp:40-48, xmgrid_map.hpp:42-50, nmgrid_map.hpp:30-127, polar_map.hpp:41-72
//   shapes             cpp/visualmesh/geometry/Sphere.hpp:55-134, Circle.hpp:64-139, plus a Cylinder
//   BSP construction   cpp/visualmesh/mesh.hpp:97-248, :425-467
//   per-frame lookup   cpp/visualmesh/mesh.hpp:265-406, :499-595
// Host code only; nothing here runs per node per frame on the hot path once the device lookup is used.
#include <algorithm>
#include <cmath>
#include <limits>
#include <map>
#include <memory>
#include <numeric>
#include <set>
#include <stack>
#include <string>
#include <utility>
#include <vector>

#include "../../include/vmcuda.h"
#include "host_math.hpp"

namespace vm {
namespace host {

    // ---- shapes --------------------------------------------------------------------------------------------------
    struct Shape {
        enum Kind { SPHERE, CIRCLE, CYLINDER } kind;
        float r;
        float half;  // cylinder: half its height = height of its centre disc

        // phi(n, h): angle from straight down to the centre of the n-th stacked object
        float phi(float n, float h) const {
            switch (kind) {
                case SPHERE: return -std::atan(std::sinh(n * std::log1p(-2.0f * r / h)));  // Sphere.hpp:75-77
                case CIRCLE: return std::atan((2.0f * n * r) / h);                           // Circle.hpp:64-66
                default: return std::atan((2.0f * n * r) / (h - half));
            }
        }
        // n(phi, h): the inverse of phi - how many objects are stacked up to that angle
        float n(float phi, float h) const {
            switch (kind) {
                case SPHERE: return std::asinh(std::tan(-phi)) / std::log1p(-2.0f * r / h);  // Sphere.hpp:79-81
                case CIRCLE: return (h * std::tan(phi)) / (2.0f * r);                          // Circle.hpp:82-84
                default: return ((h - half) * std::tan(phi)) / (2.0f * r);
            }
        }
        // height of the object's centre above the observation plane
        float c() const {
            return kind == SPHERE ? r : kind == CIRCLE ? 0.0f : half;
        }
        // angular width of the object around the phi circle; the first branch is evaluated in double because of
        // the 1.0 literal and the whole expression is rounded to float on return (Sphere.hpp:126-131)
        float theta(float n, float h) const {
            if (n <= 0.5) { return static_cast<float>(float(2.0 * M_PI) / (1.0 + n * 2.0f)); }
            const float hh = kind == CYLINDER ? h - half : h;
            return 2.0f * std::asin(r / ((hh - r) * std::tan(phi(n, h))));
        }
    };

    struct Node {
        v3 ray;
        std::vector<int> nb;
    };

    // ---- ring models ---------------------------------------------------------------------------------------------
    // polar_map.hpp:41-43, :57-72
    static v3 polar_map(const Shape& shape, float h, float n, float m) {
        const float phi     = shape.phi(std::abs(n), h);
        const float d_theta = shape.theta(std::abs(n), h);
        const float theta   = static_cast<float>(d_theta * m + (n < 0 ? M_PI : 0.0));
        return v3{{std::cos(theta) * std::sin(phi), std::sin(theta) * std::sin(phi), -std::cos(phi)}};
    }

    // ring4.hpp:50-67, ring6.hpp:50-69, ring8.hpp:50-73: neighbour offsets relative to the start of the ring
    static void ring_neighbours(int N, int i, int p, int c, int n, int* out) {
        const float f = float(i) / float(c);
        const int l   = i > 0 ? i - 1 : c - 1;
        const int r   = i + 1 < c ? i + 1 : 0;
        if (N == 4) {
            const int t = (static_cast<int>(std::round(f * n)) % n) + c;
            const int b = (static_cast<int>(std::round(f * p)) % p) - p;
            out[0] = l; out[1] = t; out[2] = r; out[3] = b;
        }
        else if (N == 6) {
            const int tl = (static_cast<int>(f * n) % n) + c;
            const int tr = ((static_cast<int>(f * n) + 1) % n) + c;
            const int bl = (static_cast<int>(f * p) % p) - p;
            const int br = ((static_cast<int>(f * p) + 1) % p) - p;
            out[0] = l; out[1] = tl; out[2] = tr; out[3] = r; out[4] = br; out[5] = bl;
        }
        else {
            const int t  = static_cast<int>(std::round(f * n)) % n;
            const int tl = (t + n - 1) % n;
            const int tr = (t + 1) % n;
            const int b  = static_cast<int>(std::round(f * p)) % p;
            const int bl = (b + p - 1) % p;
            const int br = (b + 1) % p;
            out[0] = l; out[1] = tl + c; out[2] = t + c; out[3] = tr + c; out[4] = r; out[5] = br - p; out[6] = b - p; out[7] = bl - p;
        }
    }

    // ring_base.hpp:53-115
    static std::vector<Node> generate_ring(int N, const Shape& shape, float h, float k, float max_distance) {
        std::vector<Node> nodes;
        const float jump = static_cast<float>(1.0 / k);
        int start        = 1;
        nodes.push_back(Node{v3{{0.0f, 0.0f, -1.0f}}, std::vector<int>(N, 0)});
        const int n_first      = int(std::ceil((k * float(2.0 * M_PI)) / shape.theta(jump, h)));
        const float first_jump = float(n_first) / float(N);
        for (unsigned int i = 0; i < static_cast<unsigned int>(N); ++i) { nodes.front().nb[i] = int(i * first_jump) + start; }

        for (int i = 1; h * std::tan(shape.phi(i * jump, h)) < max_distance; ++i) {
            const float n_p = (i - 1) * jump;
            const float n_c = i * jump;
            const float n_n = (i + 1) * jump;
            const float s_p = i == 1 ? 1.0f : k * float(2.0 * M_PI) / shape.theta(n_p, h);
            const float s_c = k * float(2.0 * M_PI) / shape.theta(n_c, h);
            const float s_n = k * float(2.0 * M_PI) / shape.theta(n_n, h);
            const float m_jump = s_c / (k * std::ceil(s_c));
            start              = int(nodes.size());
            const int ip = static_cast<int>(std::ceil(s_p)), ic = static_cast<int>(std::ceil(s_c)), in = static_cast<int>(std::ceil(s_n));
            for (int j = 0; j < int(std::ceil(s_c)); ++j) {
                Node n;
                n.ray = polar_map(shape, h, n_c, j * m_jump);
                n.nb.assign(N, start);
                int rel[8];
                ring_neighbours(N, j, ip, ic, in, rel);
                for (int q = 0; q < N; ++q) n.nb[q] += rel[q];
                nodes.push_back(std::move(n));
            }
        }
        for (int i = start - 1; i < int(nodes.size()); ++i) {
            for (auto& n : nodes[i].nb) n = std::min(n, int(nodes.size()));
        }
        return nodes;
    }

    // ---- grid models ---------------------------------------------------------------------------------------------
    enum class GridMap { XY, XM, NM };

    // nmgrid_map.hpp:30-62: the point on the observation plane when the plane through the first axis stands at height
    // h_n, and the second coordinate that point would have
    static v3 nm_xyz(const Shape& shape, float h, float n, float h_n) {
        const float c = shape.c();
        const float x = (h_n - c) * std::tan(shape.phi(n, h_n));
        const float y = std::sqrt((h_n - c) * (h_n - c) - (h - c) * (h - c));
        return v3{{x, y, c - h}};
    }
    static float nm_guess_m(const Shape& shape, float h, float n, float h_n) {
        const float c     = shape.c();
        const v3 v        = nm_xyz(shape, h, n, h_n);
        const float h_m   = std::sqrt(v[0] * v[0] + v[2] * v[2]) + c;
        const float phi_m = std::acos(std::sqrt((v[0] * v[0] + v[2] * v[2]) / (v[0] * v[0] + v[1] * v[1] + v[2] * v[2])));
        return shape.n(phi_m, h_m);
    }
    // nmgrid_map.hpp:91-127: bisection on the height of the first axis' plane until the second coordinate fits; it ends
    // when the interval cannot be halved any more in float
    static v3 nm_map(const Shape& shape, float h, const v2& nm) {
        const float n = std::abs(nm[0]);
        const float m = std::abs(nm[1]);
        const float c = shape.c();
        float lo      = h;
        float hi      = (h - c) / std::cos(shape.phi(m, h)) + c;
        float h_n     = (lo + hi) * 0.5f;
        while (true) {
            if (h_n == lo || h_n == hi) break;
            const float m_g = nm_guess_m(shape, h, n, h_n);
            (m_g > m ? hi : lo) = h_n;
            if (h_n == (lo + hi) * 0.5f) break;
            h_n = (lo + hi) * 0.5f;
        }
        v3 vec = nm_xyz(shape, h, n, h_n);
        vec[0] *= nm[0] >= 0 ? 1 : -1;
        vec[1] *= nm[1] >= 0 ? 1 : -1;
        return vec;
    }

    // xygrid_map.hpp:40-48, xmgrid_map.hpp:42-50
    static v3 grid_map(GridMap map, const Shape& shape, float h, const v2& nm) {
        if (map == GridMap::NM) return nm_map(shape, h, nm);
        const float phi_x = shape.phi(nm[0], h);
        const float x     = (h - shape.c()) * std::tan(phi_x);
        float y;
        if (map == GridMap::XY) {
            const float phi_y = shape.phi(nm[1], h);
            y                 = (h - shape.c()) * std::tan(phi_y);
        }
        else {
            const float h_p = (h - shape.c()) / std::cos(phi_x);
            y               = h_p * std::tan(shape.phi(nm[1], h_p + shape.c()));
        }
        return v3{{x, y, shape.c() - h}};
    }

    // grid_base.hpp:36-76 neighbour offsets, :78-144 flood fill
    static std::vector<Node> generate_grid(GridMap map, int N, const Shape& shape, float h, float k, float max_distance) {
        using I2 = std::array<int, 2>;
        static const I2 off4[4] = {{{-1, 0}}, {{0, 1}}, {{1, 0}}, {{0, -1}}};
        static const I2 off6[6] = {{{-1, 0}}, {{-1, 1}}, {{0, 1}}, {{1, 0}}, {{1, -1}}, {{0, -1}}};
        static const I2 off8[8] = {{{-1, 0}}, {{-1, 1}}, {{0, 1}}, {{1, 1}}, {{1, 0}}, {{1, -1}}, {{0, -1}}, {{-1, -1}}};
        const I2* offsets       = N == 4 ? off4 : N == 6 ? off6 : off8;

        const float jump = static_cast<float>(1.0 / k);
        std::vector<Node> output;
        std::map<I2, int> locations;
        std::set<I2> seen;
        std::stack<I2> stack;
        seen.insert(I2{{0, 0}});
        stack.push(I2{{0, 0}});
        while (!stack.empty()) {
            const I2 e = stack.top();
            stack.pop();
            v2 nm;
            if (N == 6) {
                nm = v2{{(e[0] + 0.5f * e[1]) * jump, (std::sqrt(3.0f) * 0.5f * e[1]) * jump}};
            }
            else {
                nm = v2{{float(e[0]) * jump, float(e[1]) * jump}};
            }
            const v3 vec         = grid_map(map, shape, h, nm);
            const float distance = std::sqrt(vec[1] * vec[1] + vec[0] * vec[0]);
            if (distance <= max_distance) {
                Node node;
                node.ray = normalise(vec);
                node.nb.assign(N, 0);
                locations.emplace(e, int(output.size()));
                output.push_back(std::move(node));
                for (int q = 0; q < N; ++q) {
                    const I2 n{{e[0] + offsets[q][0], e[1] + offsets[q][1]}};
                    if (seen.count(n) == 0) {
                        seen.insert(n);
                        stack.push(n);
                    }
                }
            }
        }
        for (const auto& loc : locations) {
            Node& node = output[loc.second];
            for (int q = 0; q < N; ++q) {
                const I2 target{{loc.first[0] + offsets[q][0], loc.first[1] + offsets[q][1]}};
                const auto it = locations.find(target);
                node.nb[q]    = it != locations.end() ? it->second : int(output.size());
            }
        }
        return output;
    }

    // ---- the mesh: nodes in BSP order + BSP + lookup -------------------------------------------------------------
    struct BSP {
        std::pair<int, int> range;
        std::array<int, 2> children;
        Cone cone;
    };

    class HostMesh {
    public:
        int N = 0;
        std::vector<Node> nodes;
        std::vector<BSP> bsp;

        // mesh.hpp:425-467
        HostMesh(int n_neighbours, std::vector<Node>&& generated) : N(n_neighbours), nodes(std::move(generated)) {
            std::vector<int> sorting(nodes.size());
            std::iota(sorting.begin(), sorting.end(), 0);
            uint32_t x = 0x4d657368;
            for (int i = int(sorting.size()) - 1; i > 0; i -= 5) {
                x ^= x << 13;
                x ^= x >> 17;
                x ^= x << 5;
                std::swap(sorting[i], sorting[x % i]);
            }
            bsp.reserve(nodes.size() * 2);
            build_bsp(sorting.begin(), sorting.end(), 8, 0);

            std::vector<int> r_sorting(nodes.size() + 1);
            r_sorting[nodes.size()] = int(nodes.size());
            for (unsigned int i = 0; i < nodes.size(); ++i) r_sorting[sorting[i]] = int(i);
            std::vector<Node> sorted;
            sorted.reserve(nodes.size());
            for (const auto& i : sorting) {
                sorted.push_back(nodes[i]);
                for (int& n : sorted.back().nb) n = r_sorting[n];
            }
            nodes = std::move(sorted);
        }

        // mesh.hpp:499-595
        bool lookup(const float* Hoc, const vm_lens& lens, std::vector<std::pair<int, int>>& ranges) const {
            const float cos_fov = std::cos(lens.fov * 0.5f);
            const float sin_fov = std::sin(lens.fov * 0.5f);
            const m3 Rco{{v3{{Hoc[0], Hoc[4], Hoc[8]}}, v3{{Hoc[1], Hoc[5], Hoc[9]}}, v3{{Hoc[2], Hoc[6], Hoc[10]}}}};
            const v3& rXCo = Rco[0];
            std::array<Cone, 4> edges;
            if (!screen_edges(Hoc, lens, edges)) return false;

            std::vector<int> stack(1, 0);
            bool building   = false;
            int range_start = 0;
            int range_end   = 0;
            while (!stack.empty()) {
                const int i = stack.back();
                stack.pop_back();
                const BSP& elem   = bsp[i];
                const Cone& cone  = elem.cone;
                const float delta = dot(rXCo, cone.axis);
                bool outside      = delta < cos_fov * cone.cos_t - sin_fov * cone.sin_t;
                bool inside       = delta > cos_fov * cone.cos_t + sin_fov * cone.sin_t;
                if (!outside && inside) check_on_screen(Rco, cone, lens, edges, inside, outside);

                if (inside) {
                    if (building) { range_end = elem.range.second; }
                    else {
                        range_start = elem.range.first;
                        range_end   = elem.range.second;
                        building    = true;
                    }
                }
                else if (outside) {
                    if (building) {
                        ranges.emplace_back(range_start, range_end);
                        building = false;
                    }
                }
                else if (elem.children[0] < 0) {
                    for (int j = elem.range.first; j < elem.range.second; ++j) {
                        v2 px;
                        project(mul(Rco, nodes[j].ray), lens, px);
                        const bool on_screen = dot(rXCo, nodes[j].ray) > cos_fov && 0 <= px[0]
                                               && px[0] + 1 <= lens.dimensions[0] && 0 <= px[1]
                                               && px[1] + 1 <= lens.dimensions[1];
                        if (on_screen && building) { range_end = j + 1; }
                        else if (!on_screen && building) {
                            ranges.emplace_back(range_start, range_end);
                            building = false;
                        }
                        else if (on_screen && !building) {
                            range_start = j;
                            range_end   = j + 1;
                            building    = true;
                        }
                    }
                }
                else {
                    stack.push_back(elem.children[1]);
                    stack.push_back(elem.children[0]);
                }
            }
            if (building) ranges.emplace_back(range_start, range_end);
            return true;
        }

    private:
        using It = std::vector<int>::iterator;

        // mesh.hpp:362-406
        static void check_on_screen(const m3& Rco,
                                    const Cone& cone,
                                    const vm_lens& lens,
                                    const std::array<Cone, 4>& edges,
                                    bool& inside,
                                    bool& outside) {
            v2 px;
            project(mul(Rco, cone.axis), lens, px);
            const bool axis_on_screen =
              0 <= px[0] && px[0] + 1 <= lens.dimensions[0] && 0 <= px[1] && px[1] + 1 <= lens.dimensions[1];
            float angles[4];
            bool contains = false;
            for (int i = 0; i < 4; ++i) {
                angles[i] = dot(cone.axis, edges[i].axis);
                contains  = contains || angles[i] > edges[i].cos_t * cone.cos_t + edges[i].sin_t * cone.sin_t;
            }
            if (!axis_on_screen && contains) {
                inside  = false;
                outside = true;
                return;
            }
            bool intersects = true;
            for (int i = 0; i < 4; ++i) {
                intersects = intersects && angles[i] < edges[i].cos_t * cone.cos_t - edges[i].sin_t * cone.sin_t;
            }
            inside  = axis_on_screen && intersects;
            outside = false;
        }

        // mesh.hpp:97-122: Welzl's algorithm on cones
        Cone bounding_cone(It start, It end) const {
            std::pair<v3, float> cone = cone_from_points();
            for (auto i = start; i < end; ++i) {
                if (dot(cone.first, nodes[*i].ray) < cone.second) {
                    cone = cone_from_points(nodes[*i].ray);
                    for (auto j = start; j < i; ++j) {
                        if (dot(cone.first, nodes[*j].ray) < cone.second) {
                            cone = cone_from_points(nodes[*i].ray, nodes[*j].ray);
                            for (auto k = start; k < j; ++k) {
                                if (dot(cone.first, nodes[*k].ray) < cone.second) {
                                    cone = cone_from_points(nodes[*i].ray, nodes[*j].ray, nodes[*k].ray);
                                }
                            }
                        }
                    }
                }
            }
            return Cone{cone.first, cone.second, std::sqrt(1.0f - cone.second * cone.second)};
        }

        // mesh.hpp:136-248
        int build_bsp(It start, It end, int min_points, int offset) {
            if (std::distance(start, end) <= min_points) {
                const int elem = int(bsp.size());
                bsp.push_back(BSP{{offset, static_cast<int>(offset + std::distance(start, end))}, {{-1, -1}}, bounding_cone(start, end)});
                std::sort(start, end);
                return elem;
            }
            if (bsp.empty()) {
                auto max_phi_element = std::max_element(
                  start, end, [this](const int& a, const int& b) { return nodes[a].ray[2] < nodes[b].ray[2]; });
                const float cone_cos = -nodes[*max_phi_element].ray[2];
                const float cone_sin = std::sqrt(1 - cone_cos * cone_cos);
                const Cone cone{v3{{0, 0, -1}}, cone_cos, cone_sin};
                It mid = std::partition(start, end, [this](const int& a) { return nodes[a].ray[1] > 0; });
                bsp.push_back(BSP{{offset, static_cast<int>(std::distance(start, end))}, {{-1, -1}}, cone});
                const int c0 = build_bsp(start, mid, min_points, 0);
                const int c1 = build_bsp(mid, end, min_points, int(std::distance(start, mid)));
                bsp.front().children = {{c0, c1}};
                return 0;
            }
            const Cone cone = bounding_cone(start, end);
            float min_phi   = std::numeric_limits<float>::max();
            float max_phi   = std::numeric_limits<float>::lowest();
            float min_theta = std::numeric_limits<float>::max();
            float max_theta = std::numeric_limits<float>::lowest();
            float sum_theta = 0;
            float sum_phi   = 0;
            int count_theta = 0;
            int count_phi   = 0;
            for (auto it = start; it != end; ++it) {
                const v3& ray     = nodes[*it].ray;
                const float phi   = ray[2];
                const float theta = ray[0] / std::sqrt(1 - ray[2] * ray[2]);
                min_phi           = std::min(min_phi, phi);
                max_phi           = std::max(max_phi, phi);
                sum_phi += phi;
                count_phi += 1;
                if (std::isfinite(theta)) {
                    min_theta = std::min(min_theta, theta);
                    max_theta = std::max(max_theta, theta);
                    sum_theta += theta;
                    count_theta += 1;
                }
            }
            const float split_phi   = sum_phi / count_phi;
            const float split_theta = sum_theta / count_theta;
            It mid = max_phi - min_phi > max_theta - min_theta
                       ? std::partition(start, end, [this, &split_phi](const int& a) { return nodes[a].ray[2] > split_phi; })
                       : std::partition(start, end, [this, &split_theta](const int& a) {
                             return nodes[a].ray[0] / std::sqrt(1 - nodes[a].ray[2] * nodes[a].ray[2]) < split_theta;
                         });
            const int elem = int(bsp.size());
            bsp.push_back(BSP{{offset, static_cast<int>(offset + std::distance(start, end))}, {{-1, -1}}, cone});
            const int c0 = build_bsp(start, mid, min_points, offset);
            const int c1 = build_bsp(mid, end, min_points, offset + int(std::distance(start, mid)));
            bsp[elem].children = {{c0, c1}};
            return elem;
        }
    };

}  // namespace host
}  // namespace vm

struct vm_hostmesh {
    std::unique_ptr<vm::host::HostMesh> mesh;
};

namespace {
thread_local std::string g_hostmesh_error;
}

extern "C" {

// defined in engine.cu; the host mesh reports through the same channel
const char* vm_last_error(void);
void vm_set_last_error_(const char* message);

vm_status vm_hostmesh_create(const char* model, const char* shape, float a, float b, float h, float k, float max_distance, vm_hostmesh** out) {
    using namespace vm::host;
    if (model == nullptr || shape == nullptr || out == nullptr) {
        vm_set_last_error_("null argument");
        return VM_ERR_INVALID_ARGUMENT;
    }
    *out = nullptr;
    const std::string m(model), s(shape);
    Shape sh{};
    if (s == "SPHERE") sh = Shape{Shape::SPHERE, a, 0.0f};
    else if (s == "CIRCLE") sh = Shape{Shape::CIRCLE, a, 0.0f};
    else if (s == "CYLINDER") sh = Shape{Shape::CYLINDER, a, b * 0.5f};
    else {
        vm_set_last_error_("unknown shape (SPHERE, CIRCLE, CYLINDER)");
        return VM_ERR_INVALID_ARGUMENT;
    }
    if (!(h > 0) || !(k > 0) || !(max_distance > 0) || !(a > 0)) {
        vm_set_last_error_("shape size, h, k and max_distance must be positive");
        return VM_ERR_INVALID_ARGUMENT;
    }
    try {
        std::vector<Node> nodes;
        int N = 0;
        if (m == "RING4" || m == "RING6" || m == "RING8") {
            N     = m[4] - '0';
            nodes = generate_ring(N, sh, h, k, max_distance);
        }
        else if (m == "XYGRID4" || m == "XYGRID6" || m == "XYGRID8") {
            N     = m[6] - '0';
            nodes = generate_grid(GridMap::XY, N, sh, h, k, max_distance);
        }
        else if (m == "XMGRID4" || m == "XMGRID6" || m == "XMGRID8") {
            N     = m[6] - '0';
            nodes = generate_grid(GridMap::XM, N, sh, h, k, max_distance);
        }
        else if (m == "NMGRID4" || m == "NMGRID6" || m == "NMGRID8") {
            N     = m[6] - '0';
            nodes = generate_grid(GridMap::NM, N, sh, h, k, max_distance);
        }
        else {
            vm_set_last_error_("unknown model (RING4/6/8, XYGRID4/6/8, XMGRID4/6/8, NMGRID4/6/8)");
            return VM_ERR_INVALID_ARGUMENT;
        }
        std::unique_ptr<vm_hostmesh> hm(new vm_hostmesh());
        hm->mesh.reset(new HostMesh(N, std::move(nodes)));
        *out = hm.release();
        return VM_OK;
    }
    catch (const std::exception& e) {
        vm_set_last_error_(e.what());
        return VM_ERR_OUT_OF_MEMORY;
    }
}

void vm_hostmesh_destroy(vm_hostmesh* mesh) {
    delete mesh;
}
int32_t vm_hostmesh_n_nodes(const vm_hostmesh* mesh) {
    return mesh == nullptr ? 0 : int32_t(mesh->mesh->nodes.size());
}
int32_t vm_hostmesh_n_neighbours(const vm_hostmesh* mesh) {
    return mesh == nullptr ? 0 : mesh->mesh->N;
}
int32_t vm_hostmesh_n_bsp(const vm_hostmesh* mesh) {
    return mesh == nullptr ? 0 : int32_t(mesh->mesh->bsp.size());
}

vm_status vm_hostmesh_nodes(const vm_hostmesh* mesh, float* rays, int32_t* neighbours) {
    if (mesh == nullptr || rays == nullptr || neighbours == nullptr) {
        vm_set_last_error_("null argument");
        return VM_ERR_INVALID_ARGUMENT;
    }
    const auto& m = *mesh->mesh;
    for (size_t i = 0; i < m.nodes.size(); ++i) {
        for (int c = 0; c < 3; ++c) rays[i * 3 + c] = m.nodes[i].ray[c];
        for (int j = 0; j < m.N; ++j) neighbours[i * m.N + j] = m.nodes[i].nb[j];
    }
    return VM_OK;
}

vm_status vm_hostmesh_bsp(const vm_hostmesh* mesh, int32_t* ranges, int32_t* children, float* cones) {
    if (mesh == nullptr || ranges == nullptr || children == nullptr || cones == nullptr) {
        vm_set_last_error_("null argument");
        return VM_ERR_INVALID_ARGUMENT;
    }
    const auto& m = *mesh->mesh;
    for (size_t i = 0; i < m.bsp.size(); ++i) {
        ranges[2 * i]       = m.bsp[i].range.first;
        ranges[2 * i + 1]   = m.bsp[i].range.second;
        children[2 * i]     = m.bsp[i].children[0];
        children[2 * i + 1] = m.bsp[i].children[1];
        cones[5 * i]        = m.bsp[i].cone.axis[0];
        cones[5 * i + 1]    = m.bsp[i].cone.axis[1];
        cones[5 * i + 2]    = m.bsp[i].cone.axis[2];
        cones[5 * i + 3]    = m.bsp[i].cone.cos_t;
        cones[5 * i + 4]    = m.bsp[i].cone.sin_t;
    }
    return VM_OK;
}

vm_status vm_hostmesh_lookup(const vm_hostmesh* mesh, const float Hoc[16], const vm_lens* lens, int32_t* ranges, int32_t capacity, int32_t* n_ranges) {
    if (mesh == nullptr || Hoc == nullptr || lens == nullptr || n_ranges == nullptr || (capacity > 0 && ranges == nullptr)) {
        vm_set_last_error_("null argument");
        return VM_ERR_INVALID_ARGUMENT;
    }
    std::vector<std::pair<int, int>> out;
    if (!mesh->mesh->lookup(Hoc, *lens, out)) {
        vm_set_last_error_("Unknown lens type");
        return VM_ERR_UNSUPPORTED_LENS;
    }
    *n_ranges = int32_t(out.size());
    for (size_t i = 0; i < out.size() && int32_t(i) < capacity; ++i) {
        ranges[2 * i]     = out[i].first;
        ranges[2 * i + 1] = out[i].second;
    }
    return VM_OK;
}

}  // extern "C"
