/*
 * vmcuda.h - C ABI of the B200 (sm_100a) Visual Mesh inference engine.
 *
 * The library behind this header replaces, for one path only, what the reference's interchangeable engines do:
 *   visualmesh::engine::cpu::Engine<float>::operator()(mesh, Hoc, lens)                  cpp/visualmesh/engine/cpu/engine.hpp:85-147
 *   visualmesh::engine::cpu::Engine<float>::operator()(mesh, Hoc, lens, image, format)   cpp/visualmesh/engine/cpu/engine.hpp:181-273
 * (the OpenCL engine has the same two calls: cpp/visualmesh/engine/opencl/engine.hpp:283-333, :348-534).
 *
 * Plain pointers and sizes only. All matrices are row-major. Every function returns a vm_status; a failing call
 * leaves a message readable through vm_last_error(). There is no CPU fallback: without a CUDA device every compute
 * entry point fails with VM_ERR_CUDA.
 */
#ifndef VMCUDA_H
#define VMCUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define VM_API __attribute__((visibility("default")))
#else
#define VM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum vm_status {
    VM_OK                     = 0,
    VM_ERR_INVALID_ARGUMENT   = 1,
    /* unknown fourcc; the reference throws std::runtime_error (cpp/visualmesh/engine/cpu/pixel.hpp:100) */
    VM_ERR_UNSUPPORTED_FORMAT = 2,
    /* unknown lens projection; the reference throws std::runtime_error (cpp/visualmesh/utility/projection.hpp:174) */
    VM_ERR_UNSUPPORTED_LENS   = 3,
    /* layer shapes that do not chain: weights rows != (N+1) * previous width, biases != weights columns */
    VM_ERR_NETWORK_SHAPE      = 4,
    VM_ERR_CUDA               = 5,
    VM_ERR_OUT_OF_MEMORY      = 6,
    /* a kernel gave up on a bounded loop and raised its abort flag */
    VM_ERR_DEVICE_ABORT       = 7,
    /* device-side lookup asked for (ranges == NULL) on a mesh that has no BSP uploaded */
    VM_ERR_NO_BSP             = 8
} vm_status;

/* cpp/visualmesh/lens.hpp:28 - same order as enum LensProjection */
enum { VM_RECTILINEAR = 0, VM_EQUISOLID = 1, VM_EQUIDISTANT = 2 };
/* cpp/visualmesh/network_structure.hpp:32-37 - same order as enum ActivationFunction */
enum { VM_SELU = 0, VM_RELU = 1, VM_SOFTMAX = 2, VM_TANH = 3 };

/* Mirrors visualmesh::Lens<float> (cpp/visualmesh/lens.hpp:35-52). k is applied to radii in pixels. */
typedef struct vm_lens {
    int32_t dimensions[2]; /* width, height */
    int32_t projection;    /* VM_RECTILINEAR | VM_EQUISOLID | VM_EQUIDISTANT */
    float focal_length;    /* pixels */
    float centre[2];       /* pixels */
    float k[2];
    float fov;             /* radians */
} vm_lens;

/* One dense layer: visualmesh::Layer<float> (cpp/visualmesh/network_structure.hpp:40-45).
 * weights is row-major [n_in][n_out] exactly as the reference hands them over (:25-27). */
typedef struct vm_layer {
    const float* weights;
    const float* biases;
    int32_t n_in;
    int32_t n_out;
    int32_t activation; /* VM_SELU | VM_RELU | VM_SOFTMAX | VM_TANH */
} vm_layer;

typedef struct vm_engine vm_engine;
typedef struct vm_mesh vm_mesh;

/* One camera frame: the arguments of Engine::operator() (cpp/visualmesh/engine/cpu/engine.hpp:181-185). */
typedef struct vm_frame {
    const vm_mesh* mesh;
    /* n_ranges [start,end) pairs as returned by Mesh::lookup (cpp/visualmesh/mesh.hpp:499-595), or NULL to have
     * the device walk the mesh's BSP itself (needs vm_mesh_set_bsp) */
    const int32_t* ranges;
    int32_t n_ranges;
    float Hoc[16];
    vm_lens lens;
    const void* image; /* NULL: projection only */
    uint32_t format;   /* fourcc code of image */
    int32_t image_on_device;
} vm_frame;

/* Results of a batch, frames concatenated. Frame f has n_f = offsets[f+1] - offsets[f] on-screen points.
 * pixel_coordinates and global_indices hold n_f entries per frame starting at offsets[f].
 * neighbourhood and classifications hold n_f + 1 rows per frame (the last is the off-screen row, as in
 * cpp/visualmesh/engine/cpu/engine.hpp:134-143, :206, :269-272) starting at row offsets[f] + f.
 * Neighbour indices are local to their frame (0..n_f, n_f = off-screen row).
 * Host pointers address pinned memory owned by the engine, valid until its next call. */
typedef struct vm_batch_result {
    int32_t n_frames;
    int32_t n_neighbours;
    int32_t n_classes; /* 0 for projection only */
    int32_t on_device; /* 1: the four data pointers are device pointers */
    const int32_t* offsets; /* host, n_frames + 1 */
    const float* pixel_coordinates;
    const int32_t* global_indices;
    const int32_t* neighbourhood;
    const float* classifications;
} vm_batch_result;

/* flags of vm_run_batch */
enum {
    VM_RESULTS_ON_DEVICE = 1, /* leave results in device memory: no device-to-host copies except offsets */
    VM_TIME_STAGES       = 2  /* bracket every kernel with events; read them with vm_stage_times */
};

/* Replaces the engine constructor Engine(const NetworkStructure<float>&) (cpp/visualmesh/engine/cpu/engine.hpp:57-72,
 * OpenCL: cpp/visualmesh/engine/opencl/engine.hpp:189). layers holds the dense layers of all groups in order;
 * layers_per_group[g] of them belong to ConvolutionalGroup g (cpp/visualmesh/network_structure.hpp:47-52): the first
 * layer of a group consumes the (N+1)-row gather, the others follow without one. n_groups == 0 gives a
 * projection-only engine. device < 0 selects the current device. */
VM_API vm_status vm_engine_create(int device,
                           const vm_layer* layers,
                           const int32_t* layers_per_group,
                           int32_t n_groups,
                           vm_engine** out);
VM_API void vm_engine_destroy(vm_engine* engine);

/* Uploads one mesh (one camera height) once, as the OpenCL engine caches rays per mesh
 * (cpp/visualmesh/engine/opencl/engine.hpp:603-625). rays is n_nodes x 3, neighbours n_nodes x n_neighbours
 * (visualmesh::Node, cpp/visualmesh/node.hpp:40-46); neighbour value n_nodes = no such node. n_neighbours in {4,6,8}. */
VM_API vm_status vm_mesh_upload(vm_engine* engine,
                         const float* rays,
                         const int32_t* neighbours,
                         int32_t n_nodes,
                         int32_t n_neighbours,
                         vm_mesh** out);
/* Adds the mesh's binary space partition (cpp/visualmesh/mesh.hpp:66-83): per element its node range [start,end),
 * its two children (-1,-1 for a leaf) and its bounding cone (axis xyz, cos, sin). With it frames may pass
 * ranges == NULL and Mesh::lookup (cpp/visualmesh/mesh.hpp:499-595) runs on the device. */
VM_API vm_status vm_mesh_set_bsp(vm_engine* engine,
                          vm_mesh* mesh,
                          int32_t n_elements,
                          const int32_t* element_ranges,
                          const int32_t* element_children,
                          const float* element_cones);
/* Counterpart of clear_cache() (cpp/visualmesh/engine/opencl/engine.hpp:559-572) for one mesh. */
VM_API void vm_mesh_release(vm_engine* engine, vm_mesh* mesh);

/* The hot path over a batch of independent frames in one set of kernel launches.
 * All frames of a batch must use meshes with the same n_neighbours. */
VM_API vm_status vm_run_batch(vm_engine* engine, const vm_frame* frames, int32_t n_frames, uint32_t flags, vm_batch_result* out);

/* Single-frame forms of the two reference calls (batches of one).
 * vm_project  = operator()(mesh, Hoc, lens)                cpp/visualmesh/engine/cpu/engine.hpp:85-147
 * vm_classify = operator()(mesh, Hoc, lens, image, format) cpp/visualmesh/engine/cpu/engine.hpp:181-273 */
VM_API vm_status vm_project(vm_engine* engine,
                     const vm_mesh* mesh,
                     const int32_t* ranges,
                     int32_t n_ranges,
                     const float Hoc[16],
                     const vm_lens* lens,
                     vm_batch_result* out);
VM_API vm_status vm_classify(vm_engine* engine,
                      const vm_mesh* mesh,
                      const int32_t* ranges,
                      int32_t n_ranges,
                      const float Hoc[16],
                      const vm_lens* lens,
                      const void* image,
                      uint32_t format,
                      vm_batch_result* out);

/* No counterpart in the reference.
 * Projection of one frame (operator()(mesh, Hoc, lens) with the lookup on the device) for callers that must not
 * allocate device memory while they run: a camera thread inside a fixed-period control loop, where the driver lock and
 * the implicit device synchronisation of cudaMalloc/cudaFree show up as missed frame deadlines, or a process in which
 * another framework's caching allocator already owns all of the GPU's memory so that a fresh allocation fails.
 * Every intermediate of the call (frame constants, BSP element states, per-candidate pixels and node ids, per-block
 * counts, the node -> point table, the point count) lives in one array that is part of the library image itself,
 * about 4.3 MB, resident on every GPU that loads the library until the process exits. The call makes no
 * cudaMalloc/cudaFree and uses no allocating library routine; inputs (a mesh uploaded earlier with its BSP) and
 * outputs (device buffers of the caller) are passed in.
 * Limits: mesh->n_nodes <= VM_STATIC_MAX_NODES and its BSP <= VM_STATIC_MAX_BSP elements; larger meshes are
 * rejected with VM_ERR_INVALID_ARGUMENT and a message naming the limit.
 * Outputs, all DEVICE pointers sized for the whole mesh: pixel_coordinates n_nodes x 2, global_indices n_nodes,
 * neighbourhood (n_nodes + 1) x n_neighbours; the first n (+1 for neighbourhood) entries are written. n is stored to
 * *d_n_points (device, may be NULL) and to *n_points (host, may be NULL). The call returns after its work has finished.
 * The last-bit correction tables of acosf/sinf/tanf (built, with an allocation, by the first vm_run_batch/vm_project/
 * vm_classify on a device) are used when they already exist and never built here; without them a pixel coordinate can
 * differ from the reference's in its last bit.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) - make that first call
 * during set-up, before any stream capture. All calls share the one array and it keeps the previous call's contents
 * (the cells that must start at zero are cleared by each call): two calls whose GPU work overlaps - from two engines,
 * threads or processes' streams on the same device within one process - race on it, so serialise them. */
#define VM_STATIC_MAX_NODES 262144
#define VM_STATIC_MAX_BSP 131072
VM_API vm_status vm_project_static(vm_engine* engine,
                                   const vm_mesh* mesh,
                                   const float Hoc[16],
                                   const vm_lens* lens,
                                   float* d_pixel_coordinates,
                                   int32_t* d_global_indices,
                                   int32_t* d_neighbourhood,
                                   int32_t* d_n_points,
                                   int32_t* n_points);

/* Stand-alone stages on caller-provided HOST arrays, for testing a stage against the reference function it
 * replaces with identical inputs.
 * vm_sample: cpu::interpolate (cpp/visualmesh/engine/cpu/pixel.hpp:116-144) at n pixel coordinates -> n x 4 floats.
 * vm_network: the gather/dense/activation loop (cpp/visualmesh/engine/cpu/engine.hpp:213-265) over n_rows rows
 *             (last row = off-screen row) of 4 input floats with an n_rows x n_neighbours neighbourhood. */
VM_API vm_status vm_sample(vm_engine* engine,
                    const float* pixel_coordinates,
                    int32_t n,
                    const void* image,
                    int32_t width,
                    int32_t height,
                    uint32_t format,
                    float* out);
VM_API vm_status vm_network(vm_engine* engine,
                     const float* input,
                     const int32_t* neighbourhood,
                     int32_t n_rows,
                     int32_t n_neighbours,
                     float* out);

/* Kernel time of the last vm_run_batch called with VM_TIME_STAGES, one entry per launched kernel in launch order.
 * Returns the number of stages through *n; names[i] points at a static string. */
VM_API vm_status vm_stage_times(vm_engine* engine, const char** names, float* milliseconds, int32_t capacity, int32_t* n);

/* Device-side stopwatch over any number of calls: vm_timer_start records a CUDA event on the engine's first stream
 * (after draining its streams), vm_timer_stop records one that follows all of the engine's streams, waits for it and
 * returns the elapsed device time. */
VM_API vm_status vm_timer_start(vm_engine* engine);
VM_API vm_status vm_timer_stop(vm_engine* engine, float* milliseconds);

/* No counterpart in the reference. Every wait of one thread block on another agent inside the tensor-core kernels (an
 * mbarrier armed by the tensor core or by another warp) polls at most `polls` times, then the kernel raises its abort
 * flag, leaves through its normal tear-down and the call returns VM_ERR_DEVICE_ABORT with the engine still usable.
 * The default (4,000,000 polls, a few seconds) is never reached by a healthy run. 0 makes every such wait give up at
 * once: the way to exercise the error path without hanging or faulting the device. */
VM_API vm_status vm_set_wait_limit(vm_engine* engine, uint32_t polls);

/* Number of kernels launched by this engine since creation. */
VM_API int64_t vm_launch_count(const vm_engine* engine);

/* Pinned host memory for callers that want zero-staging copies of their frames. */
VM_API vm_status vm_host_alloc(void** ptr, size_t bytes);
VM_API void vm_host_free(void* ptr);

/* Message of the last failing call on this thread. */
VM_API const char* vm_last_error(void);

/* ------------------------------------------------------------------------------------------------------------------
 * Host-side mesh tables for callers that are not C++ and cannot instantiate the reference's templates:
 * a restatement of visualmesh::Mesh (cpp/visualmesh/mesh.hpp:425-467 construction, :499-595 lookup) over the ring
 * and grid models (cpp/visualmesh/model/) and shapes (cpp/visualmesh/geometry/). Host code only.
 * ------------------------------------------------------------------------------------------------------------------ */
typedef struct vm_hostmesh vm_hostmesh;

/* model: "RING4" "RING6" "RING8", "XYGRID4" "XYGRID6" "XYGRID8", "XMGRID4" "XMGRID6" "XMGRID8", "NMGRID4" "NMGRID6"
 * "NMGRID8" (every model of cpp/visualmesh/model/); shape: "SPHERE" (a = radius), "CIRCLE" (a = radius), "CYLINDER"
 * (a = radius, b = height). */
VM_API vm_status vm_hostmesh_create(const char* model,
                             const char* shape,
                             float shape_a,
                             float shape_b,
                             float h,
                             float k,
                             float max_distance,
                             vm_hostmesh** out);
VM_API void vm_hostmesh_destroy(vm_hostmesh* mesh);
VM_API int32_t vm_hostmesh_n_nodes(const vm_hostmesh* mesh);
VM_API int32_t vm_hostmesh_n_neighbours(const vm_hostmesh* mesh);
VM_API int32_t vm_hostmesh_n_bsp(const vm_hostmesh* mesh);
/* rays: n_nodes x 3, neighbours: n_nodes x n_neighbours */
VM_API vm_status vm_hostmesh_nodes(const vm_hostmesh* mesh, float* rays, int32_t* neighbours);
/* ranges: n_bsp x 2, children: n_bsp x 2, cones: n_bsp x 5 */
VM_API vm_status vm_hostmesh_bsp(const vm_hostmesh* mesh, int32_t* ranges, int32_t* children, float* cones);
/* Mesh::lookup on the host; writes up to capacity pairs, returns the number of ranges through *n_ranges. */
VM_API vm_status vm_hostmesh_lookup(const vm_hostmesh* mesh,
                             const float Hoc[16],
                             const vm_lens* lens,
                             int32_t* ranges,
                             int32_t capacity,
                             int32_t* n_ranges);

#ifdef __cplusplus
}
#endif

#endif /* VMCUDA_H */
