/*
 * TEST INFRASTRUCTURE - not part of the product.
 *
 * A C ABI around the UNMODIFIED reference implementation, compiled from the reference's own headers where they lie
 * (-I<reference>/cpp; nothing is copied). It exposes, for the parity tests and for the timed CPU baseline:
 *   - visualmesh::Mesh<float, Model> construction and lookup      cpp/visualmesh/mesh.hpp:425-467, :499-595
 *   - visualmesh::engine::cpu::Engine<float>::operator()          cpp/visualmesh/engine/cpu/engine.hpp:85-147, :181-273
 *   - visualmesh::project / cpu::interpolate as unit functions    cpp/visualmesh/utility/projection.hpp:163-187,
 *                                                                 cpp/visualmesh/engine/cpu/pixel.hpp:116-144
 *   - the drop-in visualmesh::engine::cuda::Engine<float> called exactly like the CPU engine, on the same Mesh object
 *
 * Build rules that matter for parity:
 *   - -ffp-contract=off: with FMA contraction the reference changes its own on-screen set.
 *   - a FRESH cpu::Engine per frame: the reference never clears its `input` scratch vector
 *     (cpp/visualmesh/engine/cpu/engine.hpp:196-206), so an instance is only right on its first call.
 *   - <stdexcept>, <string>, <cmath> first: the reference headers use std::runtime_error without including it.
 */
#include <cmath>
#include <cstring>
#include <map>
#include <set>
#include <stack>
#include <stdexcept>
#include <string>
#include <thread>
#include <chrono>
#include <atomic>
#include <memory>
#include <limits>
#include <algorithm>

#include "visualmesh/engine/cpu/engine.hpp"
#include "visualmesh/geometry/Circle.hpp"
#include "visualmesh/geometry/Sphere.hpp"
#include "visualmesh/model/nmgrid4.hpp"
#include "visualmesh/model/nmgrid6.hpp"
#include "visualmesh/model/nmgrid8.hpp"
#include "visualmesh/model/ring4.hpp"
#include "visualmesh/model/ring6.hpp"
#include "visualmesh/model/ring8.hpp"
#include "visualmesh/model/xmgrid4.hpp"
#include "visualmesh/model/xmgrid6.hpp"
#include "visualmesh/model/xmgrid8.hpp"
#include "visualmesh/model/xygrid4.hpp"
#include "visualmesh/model/xygrid6.hpp"
#include "visualmesh/model/xygrid8.hpp"

#include "vmcuda.h"
#ifdef VMREF_WITH_CUDA_ENGINE
#include "visualmesh/engine/cuda/engine.hpp"
#endif

namespace vmref {

// A shape the reference does not have: an upright cylinder of radius r and height H standing on the observation
// plane, measured at the horizontal disc through its centre (height H/2). Shapes are duck-typed template
// parameters of Mesh (cpp/visualmesh/mesh.hpp:424-426), so the reference's own generator accepts it. The formulas
// are Circle's (cpp/visualmesh/geometry/Circle.hpp:64-139) with the camera height measured from that disc.
template <typename Scalar>
struct Cylinder {
    Cylinder(const Scalar& radius, const Scalar& height) : r(radius), half(height * Scalar(0.5)) {}
    Scalar phi(const Scalar& n, const Scalar& h) const {
        return std::atan((Scalar(2.0) * n * r) / (h - half));
    }
    Scalar n(const Scalar& phi, const Scalar& h) const {
        return ((h - half) * std::tan(phi)) / (Scalar(2.0) * r);
    }
    Scalar k(const Scalar& h_0, const Scalar& h_1) const {
        return (h_0 - half) / (h_1 - half);
    }
    Scalar c() const {
        return half;
    }
    Scalar theta(const Scalar& n, const Scalar& h) const {
        return n <= 0.5 ? Scalar(2.0 * M_PI) / (1.0 + n * Scalar(2.0))
                        : Scalar(2.0) * std::asin(r / ((h - half - r) * std::tan(phi(n, h))));
    }
    Scalar r;
    Scalar half;
};

template <typename S>
struct Peek {};

}  // namespace vmref

namespace visualmesh {
// Mesh befriends every specialisation of itself (cpp/visualmesh/mesh.hpp:611-612), so a specialisation on a tag of
// our own may read the private BSP of any other Mesh without touching the reference.
template <>
class Mesh<float, vmref::Peek> {
public:
    template <template <typename> class Model>
    static int size(const Mesh<float, Model>& m) {
        return int(m.bsp.size());
    }
    template <template <typename> class Model>
    static void dump(const Mesh<float, Model>& m, int* ranges, int* children, float* cones) {
        for (size_t i = 0; i < m.bsp.size(); ++i) {
            const auto& e       = m.bsp[i];
            ranges[2 * i + 0]   = e.range.first;
            ranges[2 * i + 1]   = e.range.second;
            children[2 * i + 0] = e.children[0];
            children[2 * i + 1] = e.children[1];
            cones[5 * i + 0]    = e.cone.first[0];
            cones[5 * i + 1]    = e.cone.first[1];
            cones[5 * i + 2]    = e.cone.first[2];
            cones[5 * i + 3]    = e.cone.second[0];
            cones[5 * i + 4]    = e.cone.second[1];
        }
    }
};
}  // namespace visualmesh

namespace vmref {

using visualmesh::Lens;
using visualmesh::mat4;
using visualmesh::NetworkStructure;

static Lens<float> to_lens(const vm_lens* l) {
    Lens<float> lens;
    lens.dimensions   = {{l->dimensions[0], l->dimensions[1]}};
    lens.projection   = static_cast<visualmesh::LensProjection>(l->projection);
    lens.focal_length = l->focal_length;
    lens.centre       = {{l->centre[0], l->centre[1]}};
    lens.k            = {{l->k[0], l->k[1]}};
    lens.fov          = l->fov;
    return lens;
}

static mat4<float> to_mat4(const float* H) {
    mat4<float> m;
    for (int i = 0; i < 4; ++i)
        for (int j = 0; j < 4; ++j) m[i][j] = H[i * 4 + j];
    return m;
}

static NetworkStructure<float> to_network(const vm_layer* layers, const int32_t* layers_per_group, int n_groups) {
    NetworkStructure<float> net;
    int l = 0;
    for (int g = 0; g < n_groups; ++g) {
        visualmesh::ConvolutionalGroup<float> group;
        for (int i = 0; i < layers_per_group[g]; ++i, ++l) {
            visualmesh::Layer<float> layer;
            layer.weights.resize(layers[l].n_in);
            for (int r = 0; r < layers[l].n_in; ++r) {
                layer.weights[r].assign(layers[l].weights + size_t(r) * layers[l].n_out,
                                        layers[l].weights + size_t(r + 1) * layers[l].n_out);
            }
            layer.biases.assign(layers[l].biases, layers[l].biases + layers[l].n_out);
            layer.activation = static_cast<visualmesh::ActivationFunction>(layers[l].activation);
            group.push_back(std::move(layer));
        }
        net.push_back(std::move(group));
    }
    return net;
}

struct Out {
    float* px;
    int32_t* neighbourhood;
    int32_t* global_indices;
    float* classifications;
    int32_t capacity_points;
    int32_t capacity_class_floats;
};

struct IMesh {
    virtual ~IMesh()                                                                        = default;
    virtual int n_nodes() const                                                             = 0;
    virtual int n_neighbours() const                                                        = 0;
    virtual void nodes(float* rays, int32_t* nbrs) const                                    = 0;
    virtual int n_bsp() const                                                               = 0;
    virtual void bsp(int* ranges, int* children, float* cones) const                        = 0;
    virtual int lookup(const float* Hoc, const vm_lens* lens, int32_t* ranges, int cap) const = 0;
    virtual int project(const float* Hoc, const vm_lens* lens, Out& out) const              = 0;
    virtual int classify(const NetworkStructure<float>& net,
                         const float* Hoc,
                         const vm_lens* lens,
                         const void* image,
                         uint32_t format,
                         Out* out,
                         int* n_classes) const                                              = 0;
#ifdef VMREF_WITH_CUDA_ENGINE
    virtual int cuda_classify(const NetworkStructure<float>& net,
                              const float* Hoc,
                              const vm_lens* lens,
                              const void* image,
                              uint32_t format,
                              int project_only,
                              Out* out,
                              int* n_classes) const = 0;
#endif
};

template <typename PM>
static int store_projected(const PM& p, Out& out) {
    const int n = int(p.global_indices.size());
    const int N = int(p.neighbourhood.empty() ? 0 : p.neighbourhood[0].size());
    if (n > out.capacity_points) return -2;
    for (int i = 0; i < n; ++i) {
        out.px[2 * i + 0]     = p.pixel_coordinates[i][0];
        out.px[2 * i + 1]     = p.pixel_coordinates[i][1];
        out.global_indices[i] = p.global_indices[i];
    }
    for (size_t i = 0; i < p.neighbourhood.size(); ++i)
        for (int j = 0; j < N; ++j) out.neighbourhood[i * N + j] = p.neighbourhood[i][j];
    return n;
}

template <template <typename> class Model>
struct MeshImpl : IMesh {
    static constexpr int N = Model<float>::N_NEIGHBOURS;
    visualmesh::Mesh<float, Model> mesh;

    template <typename Shape>
    MeshImpl(const Shape& shape, float h, float k, float d) : mesh(shape, h, k, d) {}

    int n_nodes() const override {
        return int(mesh.nodes.size());
    }
    int n_neighbours() const override {
        return N;
    }
    void nodes(float* rays, int32_t* nbrs) const override {
        for (size_t i = 0; i < mesh.nodes.size(); ++i) {
            for (int c = 0; c < 3; ++c) rays[i * 3 + c] = mesh.nodes[i].ray[c];
            for (int j = 0; j < N; ++j) nbrs[i * N + j] = mesh.nodes[i].neighbours[j];
        }
    }
    int n_bsp() const override {
        return visualmesh::Mesh<float, Peek>::size(mesh);
    }
    void bsp(int* ranges, int* children, float* cones) const override {
        visualmesh::Mesh<float, Peek>::dump(mesh, ranges, children, cones);
    }
    int lookup(const float* Hoc, const vm_lens* lens, int32_t* ranges, int cap) const override {
        auto r = mesh.lookup(to_mat4(Hoc), to_lens(lens));
        for (size_t i = 0; i < r.size() && int(i) < cap; ++i) {
            ranges[2 * i + 0] = r[i].first;
            ranges[2 * i + 1] = r[i].second;
        }
        return int(r.size());
    }
    int project(const float* Hoc, const vm_lens* lens, Out& out) const override {
        visualmesh::engine::cpu::Engine<float> engine;
        auto p = engine(mesh, to_mat4(Hoc), to_lens(lens));
        return store_projected(p, out);
    }
    int classify(const NetworkStructure<float>& net,
                 const float* Hoc,
                 const vm_lens* lens,
                 const void* image,
                 uint32_t format,
                 Out* out,
                 int* n_classes) const override {
        // A fresh engine for every frame: see the header of this file
        visualmesh::engine::cpu::Engine<float> engine(net);
        auto c      = engine(mesh, to_mat4(Hoc), to_lens(lens), image, format);
        const int n = int(c.global_indices.size());
        if (n_classes != nullptr) { *n_classes = n == 0 ? 0 : int(c.classifications.size() / (n + 1)); }
        if (out == nullptr) return n;
        int r = store_projected(c, *out);
        if (r < 0) return r;
        if (int(c.classifications.size()) > out->capacity_class_floats) return -2;
        std::copy(c.classifications.begin(), c.classifications.end(), out->classifications);
        return n;
    }
#ifdef VMREF_WITH_CUDA_ENGINE
    int cuda_classify(const NetworkStructure<float>& net,
                      const float* Hoc,
                      const vm_lens* lens,
                      const void* image,
                      uint32_t format,
                      int project_only,
                      Out* out,
                      int* n_classes) const override {
        visualmesh::engine::cuda::Engine<float> engine(net);
        if (project_only) {
            auto p = engine(mesh, to_mat4(Hoc), to_lens(lens));
            if (n_classes != nullptr) *n_classes = 0;
            return store_projected(p, *out);
        }
        auto c      = engine(mesh, to_mat4(Hoc), to_lens(lens), image, format);
        const int n = int(c.global_indices.size());
        if (n_classes != nullptr) { *n_classes = n == 0 ? 0 : int(c.classifications.size() / (n + 1)); }
        int r = store_projected(c, *out);
        if (r < 0) return r;
        if (int(c.classifications.size()) > out->capacity_class_floats) return -2;
        std::copy(c.classifications.begin(), c.classifications.end(), out->classifications);
        return n;
    }
#endif
};

template <template <typename> class Model>
static IMesh* make_with_shape(const std::string& shape, float a, float b, float h, float k, float d) {
    if (shape == "SPHERE") return new MeshImpl<Model>(visualmesh::geometry::Sphere<float>(a), h, k, d);
    if (shape == "CIRCLE") return new MeshImpl<Model>(visualmesh::geometry::Circle<float>(a), h, k, d);
    if (shape == "CYLINDER") return new MeshImpl<Model>(Cylinder<float>(a, b), h, k, d);
    return nullptr;
}

static thread_local std::string g_error;

}  // namespace vmref

using namespace vmref;

extern "C" {

const char* vmref_last_error() {
    return g_error.c_str();
}

void* vmref_mesh_create(const char* model, const char* shape, float a, float b, float h, float k, float d) {
    try {
        const std::string m(model);
        const std::string s(shape);
        using namespace visualmesh::model;
        IMesh* out = nullptr;
        if (m == "RING4") out = make_with_shape<Ring4>(s, a, b, h, k, d);
        else if (m == "RING6") out = make_with_shape<Ring6>(s, a, b, h, k, d);
        else if (m == "RING8") out = make_with_shape<Ring8>(s, a, b, h, k, d);
        else if (m == "XYGRID4") out = make_with_shape<XYGrid4>(s, a, b, h, k, d);
        else if (m == "XYGRID6") out = make_with_shape<XYGrid6>(s, a, b, h, k, d);
        else if (m == "XYGRID8") out = make_with_shape<XYGrid8>(s, a, b, h, k, d);
        else if (m == "XMGRID4") out = make_with_shape<XMGrid4>(s, a, b, h, k, d);
        else if (m == "XMGRID6") out = make_with_shape<XMGrid6>(s, a, b, h, k, d);
        else if (m == "XMGRID8") out = make_with_shape<XMGrid8>(s, a, b, h, k, d);
        else if (m == "NMGRID4") out = make_with_shape<NMGrid4>(s, a, b, h, k, d);
        else if (m == "NMGRID6") out = make_with_shape<NMGrid6>(s, a, b, h, k, d);
        else if (m == "NMGRID8") out = make_with_shape<NMGrid8>(s, a, b, h, k, d);
        if (out == nullptr) g_error = "unknown model or shape";
        return out;
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}

void vmref_mesh_destroy(void* mesh) {
    delete static_cast<IMesh*>(mesh);
}
int vmref_mesh_n_nodes(const void* mesh) {
    return static_cast<const IMesh*>(mesh)->n_nodes();
}
int vmref_mesh_n_neighbours(const void* mesh) {
    return static_cast<const IMesh*>(mesh)->n_neighbours();
}
void vmref_mesh_nodes(const void* mesh, float* rays, int32_t* nbrs) {
    static_cast<const IMesh*>(mesh)->nodes(rays, nbrs);
}
int vmref_mesh_n_bsp(const void* mesh) {
    return static_cast<const IMesh*>(mesh)->n_bsp();
}
void vmref_mesh_bsp(const void* mesh, int32_t* ranges, int32_t* children, float* cones) {
    static_cast<const IMesh*>(mesh)->bsp(ranges, children, cones);
}
int vmref_mesh_lookup(const void* mesh, const float* Hoc, const vm_lens* lens, int32_t* ranges, int capacity) {
    try {
        return static_cast<const IMesh*>(mesh)->lookup(Hoc, lens, ranges, capacity);
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// cpu::Engine::operator()(mesh, Hoc, lens). Returns the number of on-screen points, -1 on exception, -2 if the
// output arrays are too small. neighbourhood gets n + 1 rows.
int vmref_project(const void* mesh,
                  const float* Hoc,
                  const vm_lens* lens,
                  float* px,
                  int32_t* neighbourhood,
                  int32_t* global_indices,
                  int capacity_points) {
    try {
        Out out{px, neighbourhood, global_indices, nullptr, capacity_points, 0};
        return static_cast<const IMesh*>(mesh)->project(Hoc, lens, out);
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// cpu::Engine::operator()(mesh, Hoc, lens, image, format) on a fresh engine.
int vmref_classify(const void* mesh,
                   const float* Hoc,
                   const vm_lens* lens,
                   const void* image,
                   uint32_t format,
                   const vm_layer* layers,
                   const int32_t* layers_per_group,
                   int n_groups,
                   float* px,
                   int32_t* neighbourhood,
                   int32_t* global_indices,
                   float* classifications,
                   int capacity_points,
                   int capacity_class_floats,
                   int* n_classes) {
    try {
        Out out{px, neighbourhood, global_indices, classifications, capacity_points, capacity_class_floats};
        auto net = to_network(layers, layers_per_group, n_groups);
        return static_cast<const IMesh*>(mesh)->classify(net, Hoc, lens, image, format, &out, n_classes);
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

#ifdef VMREF_WITH_CUDA_ENGINE
// The same call through visualmesh::engine::cuda::Engine<float> on the same reference Mesh object.
int vmref_cuda_classify(const void* mesh,
                        const float* Hoc,
                        const vm_lens* lens,
                        const void* image,
                        uint32_t format,
                        const vm_layer* layers,
                        const int32_t* layers_per_group,
                        int n_groups,
                        int project_only,
                        float* px,
                        int32_t* neighbourhood,
                        int32_t* global_indices,
                        float* classifications,
                        int capacity_points,
                        int capacity_class_floats,
                        int* n_classes) {
    try {
        Out out{px, neighbourhood, global_indices, classifications, capacity_points, capacity_class_floats};
        auto net = to_network(layers, layers_per_group, n_groups);
        return static_cast<const IMesh*>(mesh)->cuda_classify(
          net, Hoc, lens, image, format, project_only, &out, n_classes);
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}
#endif

// visualmesh::project on n camera-space unit vectors (cpp/visualmesh/utility/projection.hpp:163-187)
int vmref_project_rays(const float* rays, int n, const vm_lens* lens, float* px) {
    try {
        const auto l = to_lens(lens);
        for (int i = 0; i < n; ++i) {
            auto p = visualmesh::project(visualmesh::vec3<float>{{rays[3 * i], rays[3 * i + 1], rays[3 * i + 2]}}, l);
            px[2 * i]     = p[0];
            px[2 * i + 1] = p[1];
        }
        return 0;
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// cpu::interpolate at n pixel coordinates (cpp/visualmesh/engine/cpu/pixel.hpp:116-144)
int vmref_interpolate(const float* px, int n, const void* image, int width, int height, uint32_t format, float* out) {
    try {
        const visualmesh::vec2<int> dims{{width, height}};
        for (int i = 0; i < n; ++i) {
            auto v = visualmesh::engine::cpu::interpolate(
              visualmesh::vec2<float>{{px[2 * i], px[2 * i + 1]}}, static_cast<const uint8_t*>(image), dims, format);
            for (int c = 0; c < 4; ++c) out[4 * i + c] = v[c];
        }
        return 0;
    }
    catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}

// The timed CPU baseline: n_threads workers, frames dealt round-robin, one fresh cpu::Engine per frame, a shared
// const Mesh - the shape of example/benchmark.cpp:86-101,142. Returns wall-clock seconds, total on-screen points
// through *total_points. Frame f uses meshes[f], Hocs + 16 f, lenses[f], images[f], formats[f].
double vmref_run_stream(const void* const* meshes,
                        const float* Hocs,
                        const vm_lens* lenses,
                        const void* const* images,
                        const uint32_t* formats,
                        int n_frames,
                        const vm_layer* layers,
                        const int32_t* layers_per_group,
                        int n_groups,
                        int n_threads,
                        long long* total_points) {
    auto net = to_network(layers, layers_per_group, n_groups);
    std::atomic<long long> points(0);
    std::atomic<int> failed(0);
    auto start = std::chrono::steady_clock::now();
    std::vector<std::thread> workers;
    for (int t = 0; t < n_threads; ++t) {
        workers.emplace_back([&, t] {
            try {
                for (int f = t; f < n_frames; f += n_threads) {
                    int n = static_cast<const IMesh*>(meshes[f])->classify(
                      net, Hocs + 16 * f, &lenses[f], images[f], formats[f], nullptr, nullptr);
                    points += n;
                }
            }
            catch (...) {
                failed = 1;
            }
        });
    }
    for (auto& w : workers) w.join();
    auto end = std::chrono::steady_clock::now();
    if (total_points != nullptr) *total_points = points.load();
    if (failed.load()) return -1.0;
    return std::chrono::duration<double>(end - start).count();
}

}  // extern "C"
