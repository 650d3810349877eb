/*
 * visualmesh::engine::cuda::Engine - a CUDA (sm_100a) engine beside the reference's cpu and opencl engines.
 *
 * Drop-in: include this header next to the reference's headers, link libvmcuda.so, and replace
 *     visualmesh::engine::cpu::Engine<float> engine(network);
 * by
 *     visualmesh::engine::cuda::Engine<float> engine(network);
 * The four call operators have the reference's signatures and return types
 * (cpp/visualmesh/engine/cpu/engine.hpp:84-87, :160-165, :180-185, :289-296):
 *     ProjectedMesh<float, N>  operator()(const Mesh<float, Model>&,       const mat4<float>& Hoc, const Lens<float>&) const
 *     ProjectedMesh<float, N>  operator()(const VisualMesh<float, Model>&, const mat4<float>& Hoc, const Lens<float>&) const
 *     ClassifiedMesh<float, N> operator()(const Mesh<float, Model>&,       Hoc, lens, const void* image, const uint32_t& format) const
 *     ClassifiedMesh<float, N> operator()(const VisualMesh<float, Model>&, Hoc, lens, const void* image, const uint32_t& format) const
 * plus clear_cache() as on the OpenCL engine (cpp/visualmesh/engine/opencl/engine.hpp:559-572).
 *
 * Only the reference's public headers are used, unmodified. Mesh tables are uploaded once per Mesh object and cached by
 * its address, as the OpenCL engine does (cpp/visualmesh/engine/opencl/engine.hpp:603-625): keep the Mesh alive and
 * unchanged, or call clear_cache(). Like the reference engines an instance is not thread-safe; make one per thread.
 * Errors are thrown as std::system_error with cuda_error_category(), std::runtime_error for an unknown lens or
 * image format as the reference does (cpp/visualmesh/engine/cpu/pixel.hpp:100, utility/projection.hpp:174).
 */
#ifndef VISUALMESH_ENGINE_CUDA_ENGINE_HPP
#define VISUALMESH_ENGINE_CUDA_ENGINE_HPP

#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <system_error>
#include <vector>

#include "visualmesh/classified_mesh.hpp"
#include "visualmesh/lens.hpp"
#include "visualmesh/mesh.hpp"
#include "visualmesh/network_structure.hpp"
#include "visualmesh/projected_mesh.hpp"
#include "visualmesh/utility/math.hpp"
#include "visualmesh/visualmesh.hpp"
#include "vmcuda.h"

namespace visualmesh {
namespace engine {
    namespace cuda {

        /// Error category for vm_status codes, the counterpart of opencl_error_category()
        /// (cpp/visualmesh/engine/opencl/operation/opencl_error_category.hpp)
        class error_category_t : public std::error_category {
        public:
            const char* name() const noexcept override {
                return "visualmesh_cuda";
            }
            std::string message(int code) const override {
                switch (code) {
                    case VM_OK: return "ok";
                    case VM_ERR_INVALID_ARGUMENT: return "invalid argument";
                    case VM_ERR_UNSUPPORTED_FORMAT: return "unsupported image format";
                    case VM_ERR_UNSUPPORTED_LENS: return "unknown lens type";
                    case VM_ERR_NETWORK_SHAPE: return "network layer shapes do not chain";
                    case VM_ERR_CUDA: return "CUDA error";
                    case VM_ERR_OUT_OF_MEMORY: return "out of device or pinned memory";
                    case VM_ERR_DEVICE_ABORT: return "a kernel aborted on a bounded loop";
                    case VM_ERR_NO_BSP: return "mesh has no BSP on the device";
                    default: return "unknown error";
                }
            }
        };
        inline const std::error_category& cuda_error_category() {
            static error_category_t instance;
            return instance;
        }

        namespace detail {
            template <typename S>
            struct BspAccess {};
        }  // namespace detail
    }      // namespace cuda
}  // namespace engine

// Mesh declares every specialisation of itself a friend (cpp/visualmesh/mesh.hpp:611-612). This specialisation on a tag
// type of our own reads the otherwise private BSP of any Mesh so that the lookup can run on the device; the reference
// header stays untouched.
template <>
class Mesh<float, engine::cuda::detail::BspAccess> {
public:
    template <template <typename> class Model>
    static void flatten(const Mesh<float, Model>& m,
                        std::vector<int32_t>& ranges,
                        std::vector<int32_t>& children,
                        std::vector<float>& cones) {
        const std::size_t n = m.bsp.size();
        ranges.resize(2 * n);
        children.resize(2 * n);
        cones.resize(5 * n);
        for (std::size_t i = 0; i < n; ++i) {
            const auto& e       = m.bsp[i];
            ranges[2 * i]       = e.range.first;
            ranges[2 * i + 1]   = e.range.second;
            children[2 * i]     = e.children[0];
            children[2 * i + 1] = e.children[1];
            cones[5 * i]        = e.cone.first[0];
            cones[5 * i + 1]    = e.cone.first[1];
            cones[5 * i + 2]    = e.cone.first[2];
            cones[5 * i + 3]    = e.cone.second[0];
            cones[5 * i + 4]    = e.cone.second[1];
        }
    }
};

namespace engine {
    namespace cuda {

        template <typename Scalar>
        class Engine {
            static_assert(std::is_same<Scalar, float>::value, "the CUDA engine computes in float");

        public:
            /**
             * @param structure      the network to classify with (may be empty for projection only)
             * @param device         CUDA device ordinal, -1 for the current device
             * @param device_lookup  true: Mesh::lookup runs on the GPU from the mesh's BSP; false: it runs on the host
             *                       through mesh.lookup() as in the OpenCL engine
             *                       (cpp/visualmesh/engine/opencl/engine.hpp:581)
             */
            explicit Engine(const NetworkStructure<Scalar>& structure = {}, int device = -1, bool device_lookup = true)
              : device_lookup(device_lookup) {
                std::vector<vm_layer> layers;
                std::vector<int32_t> per_group;
                std::vector<std::vector<float>> flat;
                for (const auto& group : structure) {
                    per_group.push_back(int32_t(group.size()));
                    for (const auto& layer : group) {
                        const int n_in  = int(layer.weights.size());
                        const int n_out = int(layer.biases.size());
                        flat.emplace_back();
                        auto& w = flat.back();
                        w.reserve(std::size_t(n_in) * n_out);
                        for (const auto& row : layer.weights) {
                            if (int(row.size()) != n_out) { throw_status(VM_ERR_NETWORK_SHAPE, "ragged weights matrix"); }
                            w.insert(w.end(), row.begin(), row.end());
                        }
                        layers.push_back(vm_layer{nullptr, layer.biases.data(), n_in, n_out, int32_t(layer.activation)});
                    }
                }
                for (std::size_t i = 0; i < layers.size(); ++i) layers[i].weights = flat[i].data();
                check(vm_engine_create(device, layers.data(), per_group.data(), int32_t(per_group.size()), &engine));
                has_network = !layers.empty();
            }
            ~Engine() {
                vm_engine_destroy(engine);
            }
            Engine(const Engine&) = delete;
            Engine& operator=(const Engine&) = delete;

            /// Drops the device copies of all meshes seen so far
            void clear_cache() {
                for (auto& m : meshes) vm_mesh_release(engine, m.second.handle);
                meshes.clear();
            }

            /// Bounds the number of meshes kept on the device (0 = unbounded, the default, like the OpenCL engine's
            /// grow-only cache): beyond it the least recently used mesh is released. For a VisualMesh with many
            /// heights in a long-running process (the role of tensorflow/mesh_cache.hpp:119-159 in training).
            void set_cache_limit(std::size_t n_meshes) {
                cache_limit = n_meshes;
                evict();
            }

            template <template <typename> class Model>
            ProjectedMesh<Scalar, Model<Scalar>::N_NEIGHBOURS> operator()(const Mesh<Scalar, Model>& mesh,
                                                                          const mat4<Scalar>& Hoc,
                                                                          const Lens<Scalar>& lens) const {
                static constexpr int N = Model<Scalar>::N_NEIGHBOURS;
                vm_batch_result r;
                run(mesh, Hoc, lens, nullptr, 0, r);
                ProjectedMesh<Scalar, N> out;
                fill_projection<N>(r, out.pixel_coordinates, out.neighbourhood, out.global_indices);
                return out;
            }

            template <template <typename> class Model>
            inline ProjectedMesh<Scalar, Model<Scalar>::N_NEIGHBOURS> operator()(const VisualMesh<Scalar, Model>& mesh,
                                                                                 const mat4<Scalar>& Hoc,
                                                                                 const Lens<Scalar>& lens) const {
                return operator()(mesh.height(Hoc[2][3]), Hoc, lens);
            }

            template <template <typename> class Model>
            ClassifiedMesh<Scalar, Model<Scalar>::N_NEIGHBOURS> operator()(const Mesh<Scalar, Model>& mesh,
                                                                           const mat4<Scalar>& Hoc,
                                                                           const Lens<Scalar>& lens,
                                                                           const void* image,
                                                                           const uint32_t& format) const {
                static constexpr int N = Model<Scalar>::N_NEIGHBOURS;
                if (!has_network) throw_status(VM_ERR_NETWORK_SHAPE, "engine was constructed without a network");
                vm_batch_result r;
                run(mesh, Hoc, lens, image, format, r);
                ClassifiedMesh<Scalar, N> out;
                // an empty on-screen set gives a default-constructed result (cpp/visualmesh/engine/cpu/engine.hpp:193)
                if (r.offsets[1] == 0) return out;
                fill_projection<N>(r, out.pixel_coordinates, out.neighbourhood, out.global_indices);
                const std::size_t rows = std::size_t(r.offsets[1]) + 1;
                out.classifications.assign(r.classifications, r.classifications + rows * r.n_classes);
                return out;
            }

            template <template <typename> class Model>
            ClassifiedMesh<Scalar, Model<Scalar>::N_NEIGHBOURS> operator()(const VisualMesh<Scalar, Model>& mesh,
                                                                           const mat4<Scalar>& Hoc,
                                                                           const Lens<Scalar>& lens,
                                                                           const void* image,
                                                                           const uint32_t& format) const {
                return operator()(mesh.height(Hoc[2][3]), Hoc, lens, image, format);
            }

        private:
            [[noreturn]] static void throw_status(vm_status s, const std::string& what) {
                if (s == VM_ERR_UNSUPPORTED_FORMAT || s == VM_ERR_UNSUPPORTED_LENS) throw std::runtime_error(what);
                throw std::system_error(int(s), cuda_error_category(), what);
            }
            static void check(vm_status s) {
                if (s != VM_OK) throw_status(s, vm_last_error());
            }

            template <template <typename> class Model>
            vm_mesh* device_mesh(const Mesh<Scalar, Model>& mesh) const {
                auto it = meshes.find(&mesh);
                if (it != meshes.end()) {
                    it->second.last_use = ++use_counter;
                    return it->second.handle;
                }
                static constexpr int N = Model<Scalar>::N_NEIGHBOURS;
                const std::size_t n    = mesh.nodes.size();
                std::vector<float> rays(3 * n);
                std::vector<int32_t> nbrs(std::size_t(N) * n);
                for (std::size_t i = 0; i < n; ++i) {
                    for (int c = 0; c < 3; ++c) rays[3 * i + c] = mesh.nodes[i].ray[c];
                    for (int j = 0; j < N; ++j) nbrs[N * i + j] = mesh.nodes[i].neighbours[j];
                }
                vm_mesh* handle = nullptr;
                check(vm_mesh_upload(engine, rays.data(), nbrs.data(), int32_t(n), N, &handle));
                if (device_lookup) {
                    std::vector<int32_t> ranges, children;
                    std::vector<float> cones;
                    Mesh<float, detail::BspAccess>::flatten(mesh, ranges, children, cones);
                    check(vm_mesh_set_bsp(engine, handle, int32_t(ranges.size() / 2), ranges.data(), children.data(), cones.data()));
                }
                meshes[&mesh] = CachedMesh{handle, ++use_counter};
                evict();
                return handle;
            }

            void evict() const {
                while (cache_limit != 0 && meshes.size() > cache_limit) {
                    auto oldest = meshes.begin();
                    for (auto it = meshes.begin(); it != meshes.end(); ++it) {
                        if (it->second.last_use < oldest->second.last_use) oldest = it;
                    }
                    vm_mesh_release(engine, oldest->second.handle);
                    meshes.erase(oldest);
                }
            }

            template <template <typename> class Model>
            void run(const Mesh<Scalar, Model>& mesh,
                     const mat4<Scalar>& Hoc,
                     const Lens<Scalar>& lens,
                     const void* image,
                     uint32_t format,
                     vm_batch_result& r) const {
                vm_lens l;
                l.dimensions[0] = lens.dimensions[0];
                l.dimensions[1] = lens.dimensions[1];
                l.projection    = int32_t(lens.projection);
                l.focal_length  = lens.focal_length;
                l.centre[0]     = lens.centre[0];
                l.centre[1]     = lens.centre[1];
                l.k[0]          = lens.k[0];
                l.k[1]          = lens.k[1];
                l.fov           = lens.fov;
                float H[16];
                for (int i = 0; i < 4; ++i)
                    for (int j = 0; j < 4; ++j) H[4 * i + j] = Hoc[i][j];
                vm_mesh* handle = device_mesh(mesh);
                std::vector<int32_t> flat;
                const int32_t* ranges = nullptr;
                int32_t n_ranges      = 0;
                static const int32_t none[2] = {0, 0};
                if (!device_lookup) {
                    const auto looked = mesh.lookup(Hoc, lens);
                    flat.reserve(2 * looked.size());
                    for (const auto& p : looked) {
                        flat.push_back(p.first);
                        flat.push_back(p.second);
                    }
                    ranges   = flat.empty() ? none : flat.data();
                    n_ranges = int32_t(looked.size());
                }
                if (image == nullptr) { check(vm_project(engine, handle, ranges, n_ranges, H, &l, &r)); }
                else {
                    check(vm_classify(engine, handle, ranges, n_ranges, H, &l, image, format, &r));
                }
            }

            template <int N>
            static void fill_projection(const vm_batch_result& r,
                                        std::vector<vec2<Scalar>>& px,
                                        std::vector<std::array<int, N>>& nb,
                                        std::vector<int>& gi) {
                const std::size_t n = std::size_t(r.offsets[1]);
                px.resize(n);
                gi.resize(n);
                nb.resize(n + 1);
                for (std::size_t i = 0; i < n; ++i) {
                    px[i] = vec2<Scalar>{{r.pixel_coordinates[2 * i], r.pixel_coordinates[2 * i + 1]}};
                    gi[i] = r.global_indices[i];
                }
                for (std::size_t i = 0; i <= n; ++i)
                    for (int j = 0; j < N; ++j) nb[i][j] = r.neighbourhood[i * N + j];
            }

            vm_engine* engine = nullptr;
            bool has_network  = false;
            bool device_lookup;
            /// Device meshes by the address of the Mesh they were uploaded from
            struct CachedMesh {
                vm_mesh* handle;
                std::uint64_t last_use;
            };
            mutable std::map<const void*, CachedMesh> meshes;
            mutable std::uint64_t use_counter = 0;
            std::size_t cache_limit           = 0;
        };

    }  // namespace cuda
}  // namespace engine
}  // namespace visualmesh

#endif  // VISUALMESH_ENGINE_CUDA_ENGINE_HPP
