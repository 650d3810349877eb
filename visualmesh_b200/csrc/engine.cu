// Host side of the engine and its C ABI (include/vmcuda.h).
//
// One engine instance owns its streams, its grow-only device scratch and its pinned result buffers; like the
// reference engines it is not thread-safe - use one instance per host thread. A batch is cut into chunks of frames;
// chunks rotate over a few lanes (stream + scratch) so that the host-to-device copy of one chunk's images, the
// kernels of another and the device-to-host copy of a third overlap.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/vmcuda.h"
#include "host_math.hpp"
#include "kernels.cuh"
#include "conv_dispatch.hpp"
#include "libm_tables.hpp"

namespace vm {

static thread_local std::string g_error;

static vm_status fail(vm_status s, const std::string& msg) {
    g_error = msg;
    return s;
}

// the per-frame constants could not be computed: a projection the lens math does not know (the reference throws from
// unproject, cpp/visualmesh/utility/projection.hpp:224)
struct UnsupportedLens {};

// Grow-only device and pinned-host arrays (the reference's OpenCL engine keeps the same kind of caches,
// cpp/visualmesh/engine/opencl/engine.hpp:740-835).
template <typename T>
struct DeviceArray {
    T* p       = nullptr;
    size_t cap = 0;
    void ensure(size_t n) {
        if (n <= cap) return;
        if (p != nullptr) VM_CUDA(cudaFree(p));
        p   = nullptr;
        cap = 0;
        const size_t want = n + n / 8 + 64;
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&p), want * sizeof(T)));
        cap = want;
    }
    void release() {
        if (p != nullptr) cudaFree(p);
        p   = nullptr;
        cap = 0;
    }
};

template <typename T>
struct PinnedArray {
    T* p       = nullptr;
    size_t cap = 0;
    void ensure(size_t n) {
        if (n <= cap) return;
        if (p != nullptr) VM_CUDA(cudaFreeHost(p));
        p   = nullptr;
        cap = 0;
        const size_t want = n + n / 8 + 64;
        VM_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&p), want * sizeof(T), cudaHostAllocDefault));
        cap = want;
    }
    void release() {
        if (p != nullptr) cudaFreeHost(p);
        p   = nullptr;
        cap = 0;
    }
};

static_assert(libm::FIRST_BITS[libm::ACOS] == LIBM_FIRST_BITS && libm::END_BITS[libm::ACOS] == LIBM_ONE_BITS
                && libm::FIRST_BITS[libm::SIN] == LIBM_FIRST_BITS && libm::END_BITS[libm::SIN] == LIBM_TWO_BITS
                && libm::FIRST_BITS[libm::TAN] == LIBM_FIRST_BITS && libm::END_BITS[libm::TAN] == LIBM_TWO_BITS,
              "the device reads the last-bit tables over the ranges the host builds them for");

// Device copies of the libm last-bit tables, built on first use and shared by all engines of a process (per device).
constexpr int LIBM_MAX_DEVICES = 64;
static uint32_t* g_libm_device[LIBM_MAX_DEVICES][libm::N_FUNCTIONS] = {};
static std::mutex g_libm_mutex;

static const uint32_t* libm_table(int device, int fn, bool build_if_missing) {
    static const bool disabled = [] {
        const char* v = std::getenv("VMCUDA_LIBM_TABLES");
        return v != nullptr && v[0] == '0';
    }();
    if (disabled || device < 0 || device >= LIBM_MAX_DEVICES) return nullptr;
    std::lock_guard<std::mutex> lock(g_libm_mutex);
    if (g_libm_device[device][fn] == nullptr && build_if_missing) {
        const std::vector<uint32_t> packed = libm::build(fn);
        uint32_t* d = nullptr;
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&d), packed.size() * sizeof(uint32_t)));
        VM_CUDA(cudaMemcpy(d, packed.data(), packed.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
        g_libm_device[device][fn] = d;
    }
    return g_libm_device[device][fn];
}

constexpr int MAX_LANES = 3;

struct Lane {
    cudaStream_t stream   = nullptr;
    cudaEvent_t ev_staged = nullptr;   // host staging of this lane has been consumed
    cudaEvent_t ev_scan   = nullptr;   // this chunk's offsets are on the device
    cudaEvent_t ev_offsets = nullptr;  // ... and on the host
    cudaEvent_t ev_done   = nullptr;   // everything of this chunk, copies included, has finished
    bool busy             = false;
    int f0 = 0, f1 = 0;
    PinnedArray<FrameParams> h_frames;
    DeviceArray<FrameParams> d_frames;
    PinnedArray<int32_t> h_ranges;  // int2 ranges then range starts
    DeviceArray<int32_t> d_ranges;
    DeviceArray<uint8_t> d_state;
    DeviceArray<float2> d_cand_px;
    DeviceArray<int32_t> d_cand_node;
    DeviceArray<int32_t> d_block_counts;
    DeviceArray<int32_t> d_node_rank;
    DeviceArray<float> d_feat[2];
    DeviceArray<uint8_t> d_images;
    // tile plan of the chunk for the staged tensor-core layers (conv_staged.cuh)
    DeviceArray<uint16_t> d_nbl;
    DeviceArray<int32_t> d_halo_rows;
    DeviceArray<int32_t> d_halo_count;
    bool plan_valid = false;
};

struct StageTimer {
    const char* name;
    cudaEvent_t start, stop;
};

}  // namespace vm

struct vm_mesh {
    const vm_engine* owner = nullptr;  // the engine it was uploaded through (and whose device holds it)
    int32_t n_nodes = 0, n_neighbours = 0, n_bsp = 0;
    float4* d_rays        = nullptr;
    int32_t* d_neighbours = nullptr;
    float4* d_cones_a     = nullptr;
    float* d_cones_s      = nullptr;
    int4* d_topology      = nullptr;
};

struct vm_engine {
    int device = 0;
    std::vector<vm::DenseLayer> layers;
    int max_width = 4;
    int n_classes = 0;
    vm::Lane lanes[vm::MAX_LANES];
    int n_lanes = vm::MAX_LANES;
    int64_t chunk_candidates = 2 << 20;
    int chunk_frames         = 16;
    bool chunk_override      = false;  // set by the environment: use the limits above for every batch
    // batch-wide results
    vm::DeviceArray<int32_t> d_offsets;
    vm::PinnedArray<int32_t> h_offsets;
    vm::DeviceArray<float2> d_px;
    vm::DeviceArray<int32_t> d_gi;
    vm::DeviceArray<int32_t> d_nb;
    vm::DeviceArray<float> d_cls;
    vm::PinnedArray<float2> h_px;
    vm::PinnedArray<int32_t> h_gi;
    vm::PinnedArray<int32_t> h_nb;
    vm::PinnedArray<float> h_cls;
    int32_t* d_abort = nullptr;
    int32_t* h_abort = nullptr;
    std::vector<vm_mesh*> meshes;
    // stage timing
    std::vector<vm::StageTimer> timers;
    std::vector<cudaEvent_t> event_pool;
    size_t events_used = 0;
    bool timing        = false;
    std::vector<std::pair<const char*, float>> stage_ms;
    int64_t launches = 0;
    bool use_tc      = true;
    int tc_mode      = 1;
    int tc_min_product = 512;   // mode 1: layers with C_in x C_out at least this run on the tensor cores
    bool tc_no_split = false;   // debugging: never use the split feature layout
    bool staged          = true;    // tensor-core layers read their gather from shared-memory windows (conv_staged.cuh)
    bool may_stage       = false;   // some layer could run as a staged tensor-core layer under the engine's policy
    uint32_t tc_wait_limit = vm::TC_DEFAULT_WAIT_LIMIT;  // polls of one mbarrier wait in the tensor-core kernels (vm_set_wait_limit)
    cudaEvent_t ev_timer_start = nullptr, ev_timer_stop = nullptr;
    cudaEvent_t ev_batch_start = nullptr;  // the start-of-batch clears (offsets[0], abort flag) are done
    cudaEvent_t ev_batch_done  = nullptr;  // everything of the batch, the abort flag's copy included, has finished
    bool blocking_sync         = false;    // host waits sleep instead of spinning
    bool nvtx                  = false;    // NVTX ranges around every kernel launch and batch (VMCUDA_NVTX=1)
};

namespace vm {

// A stage is one kernel launch. With VMCUDA_NVTX=1 every launch sits in an NVTX range of the stage's name (the header-only
// NVTX does nothing unless a profiler is attached); with stage timing on, between two CUDA events.
static void begin_stage(vm_engine* e, cudaStream_t s, const char* name) {
    ++e->launches;
    if (e->nvtx) nvtxRangePushA(name);
    if (!e->timing) return;
    while (e->event_pool.size() < e->events_used + 2) {
        cudaEvent_t ev;
        VM_CUDA(cudaEventCreate(&ev));
        e->event_pool.push_back(ev);
    }
    StageTimer t{name, e->event_pool[e->events_used], e->event_pool[e->events_used + 1]};
    e->events_used += 2;
    VM_CUDA(cudaEventRecord(t.start, s));
    e->timers.push_back(t);
}
static void end_stage(vm_engine* e, cudaStream_t s) {
    if (e->nvtx) nvtxRangePop();
    if (!e->timing) return;
    VM_CUDA(cudaEventRecord(e->timers.back().stop, s));
}

enum ConvKind { CONV_FFMA = 0, CONV_TC_GATHER = 1, CONV_TC_SPLIT = 2, CONV_TC_STAGED = 3 };

// Whether the kernel that runs layer L as `kind` honours ConvArgs::out_split. The tensor-core kernels write the split
// layout when their tile is exactly as wide as the layer; the specialised FFMA kernels when the width is a multiple
// of 8; the generic kernel never does.
static bool producer_writes_split(const DenseLayer& L, ConvKind kind) {
    if (kind == CONV_TC_STAGED) return L.cout % 8 == 0;
    if (kind != CONV_FFMA) return L.cout == L.tc_np;
    return has_fast_ffma_kernel(L.cin, L.cout) && L.cout % 8 == 0;
}

// Scratch of a chunk's tile plan (tile_plan.cuh): neighbour positions per row, halo lists per super-tile.
static st::PlanOut ensure_tile_plan(Lane& lane, size_t rows_cap, size_t supertiles_cap) {
    lane.d_nbl.ensure(rows_cap * STAGED_NBL_STRIDE + 64);
    lane.d_halo_rows.ensure(supertiles_cap * STAGED_HALO + 64);
    lane.d_halo_count.ensure(supertiles_cap + 64);
    return st::PlanOut{lane.d_nbl.p, lane.d_halo_rows.p, lane.d_halo_count.p};
}

static void launch_conv(vm_engine* e, const DenseLayer& L, ConvArgs a, int n_frames, int max_rows, cudaStream_t s, ConvKind kind, const StagedPlan& plan) {
    a.weights     = L.d_weights;
    a.biases      = L.d_weights + static_cast<size_t>(L.n_slots) * L.cin * L.coutp;
    a.n_slots     = L.n_slots;
    a.activation  = L.activation;
    begin_stage(e, s, L.stage.c_str());
    if (kind == CONV_TC_STAGED && launch_conv_staged(L, a, plan, n_frames, max_rows, e->d_abort, e->tc_wait_limit, s)) {}
    else if ((kind == CONV_TC_SPLIT || kind == CONV_TC_STAGED) && launch_conv_tc_split(L, a, n_frames, max_rows, e->d_abort, e->tc_wait_limit, s)) {}
    else if (kind == CONV_TC_GATHER && launch_conv_tc_gather(L, a, n_frames, max_rows, e->d_abort, e->tc_wait_limit, s)) {}
    else {
        launch_conv_ffma(L, a, n_frames, max_rows, s);
    }
    VM_CUDA(cudaGetLastError());
    end_stage(e, s);
}

// Runs all layers over a chunk whose input features are in feat[0]; the last layer writes out_final.
static void run_network(vm_engine* e,
                        Lane& lane,
                        const int32_t* d_offsets,
                        const int32_t* d_nb,
                        int n_neighbours,
                        int f0,
                        int n_frames,
                        int max_rows,
                        float* out_final,
                        bool final_global,
                        int feature_stride) {
    // Which kernel runs each layer (VMCUDA_TC: 0 = CUDA cores only; 1, the default, and 2 = tensor cores too).
    // A 16- or 32-channel layer whose producer can write the split layout runs as a staged layer (conv_staged.cuh,
    // VMCUDA_STAGED=0 turns it off). Otherwise the tcgen05 kernels take a layer when its contraction is dense enough to
    // pay (mode 1: C_in x C_out >= 512) or whenever one exists (mode 2): fed by plain copies from the split layout
    // (CONV_TC_SPLIT) or gathering and splitting fp32 themselves (CONV_TC_GATHER).
    const size_t n_layers = e->layers.size();
    std::vector<ConvKind> kind(n_layers, CONV_FFMA);
    for (size_t l = 0; l < n_layers; ++l) {
        const DenseLayer& L = e->layers[l];
        if (!e->use_tc || L.tc_np == 0 || L.n_slots == 1 || n_frames > TC_MAX_FRAMES) continue;
        const bool producer_can_split = l > 0 && producer_writes_split(e->layers[l - 1], kind[l - 1]) && !e->tc_no_split;
        // the staged kernel wherever it exists (it writes features, not results: never the last layer)
        if (e->staged && lane.plan_valid && producer_can_split && has_staged_kernel(L) && l + 1 < n_layers) {
            kind[l] = CONV_TC_STAGED;
            continue;
        }
        // the tcgen05 kernels where the contraction is dense enough for them to pay (mode 1) or wherever they exist (mode 2)
        if (e->tc_mode == 1 && L.cin * L.cout < e->tc_min_product) continue;
        if (has_tc_split_kernel(L) && producer_can_split) kind[l] = CONV_TC_SPLIT;
        else if (has_tc_gather_kernel(L)) kind[l] = CONV_TC_GATHER;
        // anything else (dense-only layers, shapes without a tensor-core instantiation) stays on the FFMA kernels
    }
    const StagedPlan plan{lane.d_nbl.p, lane.d_halo_rows.p, lane.d_halo_count.p};
    int cur = 0;
    for (size_t l = 0; l < n_layers; ++l) {
        const bool last = l + 1 == n_layers;
        ConvArgs a{};
        a.in           = lane.d_feat[cur].p;
        a.out          = last ? out_final : lane.d_feat[cur ^ 1].p;
        a.nb           = d_nb;
        a.offsets      = d_offsets;
        a.n_neighbours = n_neighbours;
        a.f0           = f0;
        a.out_global   = (last && final_global) ? 1 : 0;
        a.in_stride    = feature_stride;
        a.out_stride   = feature_stride;
        a.out_planar   = (!last && e->layers[l].cout % 4 == 0) ? 1 : 0;
        a.out_split    = (!last && (kind[l + 1] == CONV_TC_SPLIT || kind[l + 1] == CONV_TC_STAGED)) ? 1 : 0;
        a.range_flag   = e->d_abort;
        launch_conv(e, e->layers[l], a, n_frames, max_rows, lane.stream, kind[l], plan);
        cur ^= 1;
    }
}

// ---- per-frame constants -----------------------------------------------------------------------------------------

static bool fill_frame_params(const vm_frame& fr, FrameParams& p, int device, bool may_allocate = true) {
    const float* H = fr.Hoc;
    // Rco = block<3,3>(transpose(Hoc)), cpp/visualmesh/engine/cpu/engine.hpp:95
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) p.Rco[i * 3 + j] = H[j * 4 + i];
    p.focal_length = fr.lens.focal_length;
    p.centre[0]    = fr.lens.centre[0];
    p.centre[1]    = fr.lens.centre[1];
    p.half_dims[0] = float(fr.lens.dimensions[0]) * 0.5f;
    p.half_dims[1] = float(fr.lens.dimensions[1]) * 0.5f;
    host::inverse_coefficients(fr.lens.k, p.ik);
    p.dims[0]    = fr.lens.dimensions[0];
    p.dims[1]    = fr.lens.dimensions[1];
    p.projection = fr.lens.projection;
    p.format     = fr.format;
    // cpp/visualmesh/mesh.hpp:503-504
    p.cos_fov = std::cos(fr.lens.fov * 0.5f);
    p.sin_fov = std::sin(fr.lens.fov * 0.5f);
    if (fr.ranges == nullptr) {
        std::array<host::Cone, 4> edges;
        if (!host::screen_edges(H, fr.lens, edges)) return false;
        for (int i = 0; i < 4; ++i) {
            p.edges[i][0] = edges[i].axis[0];
            p.edges[i][1] = edges[i].axis[1];
            p.edges[i][2] = edges[i].axis[2];
            p.edges[i][3] = edges[i].cos_t;
            p.edges[i][4] = edges[i].sin_t;
        }
    }
    p.libm_acos = libm_table(device, libm::ACOS, may_allocate);
    p.libm_sin  = fr.lens.projection == VM_EQUISOLID ? libm_table(device, libm::SIN, may_allocate) : nullptr;
    p.libm_tan  = fr.lens.projection == VM_RECTILINEAR ? libm_table(device, libm::TAN, may_allocate) : nullptr;
    const vm_mesh* m = fr.mesh;
    p.rays           = m->d_rays;
    p.neighbours     = m->d_neighbours;
    p.bsp_cones_a    = m->d_cones_a;
    p.bsp_cones_s    = m->d_cones_s;
    p.bsp_topology   = m->d_topology;
    p.n_nodes        = m->n_nodes;
    p.n_bsp          = m->n_bsp;
    return true;
}

static size_t image_bytes(const vm_frame& fr) {
    const int cls = format_class(fr.format);
    return static_cast<size_t>(fr.lens.dimensions[0]) * fr.lens.dimensions[1] * format_bytes_per_pixel(cls);
}

static int64_t frame_candidates(const vm_frame& fr) {
    if (fr.ranges == nullptr) return fr.mesh->n_nodes;
    int64_t n = 0;
    for (int r = 0; r < fr.n_ranges; ++r) n += std::max(0, fr.ranges[2 * r + 1] - fr.ranges[2 * r]);
    return n;
}

// ---- one chunk: enqueue everything up to the last kernel -----------------------------------------------------

static void enqueue_chunk(vm_engine* e, Lane& lane, Lane* prev, const vm_frame* frames, int f0, int f1, bool classify) {
    const int nf = f1 - f0;
    cudaStream_t s = lane.stream;
    lane.f0 = f0;
    lane.f1 = f1;

    // host staging: frame constants and the concatenated ranges
    lane.h_frames.ensure(nf);
    lane.d_frames.ensure(nf);
    size_t n_ranges_total = 0;
    for (int f = f0; f < f1; ++f) n_ranges_total += frames[f].ranges != nullptr ? frames[f].n_ranges : 0;
    lane.h_ranges.ensure(3 * n_ranges_total + 4);
    lane.d_ranges.ensure(3 * n_ranges_total + 4);

    int64_t cand_total = 0, node_total = 0, bsp_total = 0, image_total = 0;
    const int plan_st     = STAGED_ST;
    size_t supertiles_cap = 0;
    lane.plan_valid       = false;
    int32_t max_cand = 0;
    bool any_device_lookup = false, any_host_ranges = false;
    size_t range_cursor = 0;
    for (int f = f0; f < f1; ++f) {
        const vm_frame& fr = frames[f];
        FrameParams& p     = lane.h_frames.p[f - f0];
        std::memset(&p, 0, sizeof(p));
        if (!fill_frame_params(fr, p, e->device)) throw UnsupportedLens{};
        const int64_t nc = frame_candidates(fr);
        p.n_candidates   = static_cast<int32_t>(nc);
        p.cand_off       = static_cast<int32_t>(cand_total);
        p.node_off       = static_cast<int32_t>(node_total);
        p.bsp_off        = static_cast<int32_t>(bsp_total);
        if (fr.ranges != nullptr) {
            any_host_ranges = true;
            // device layout: [int2 ranges of all frames][starts of all frames]; pointers are patched below
            p.n_ranges = fr.n_ranges;
        }
        else {
            any_device_lookup = true;
            bsp_total += fr.mesh->n_bsp;
        }
        cand_total += nc;
        supertiles_cap += static_cast<size_t>((nc + 1 + plan_st - 1) / plan_st);
        node_total += fr.mesh->n_nodes;
        max_cand = std::max<int32_t>(max_cand, static_cast<int32_t>(nc));
        if (classify && !fr.image_on_device) image_total += (image_bytes(fr) + 255) & ~size_t(255);
    }
    // ranges and their exclusive prefix sums
    {
        int32_t* pairs  = lane.h_ranges.p;
        int32_t* starts = lane.h_ranges.p + 2 * n_ranges_total;
        for (int f = f0; f < f1; ++f) {
            const vm_frame& fr = frames[f];
            if (fr.ranges == nullptr) continue;
            FrameParams& p = lane.h_frames.p[f - f0];
            p.ranges       = reinterpret_cast<const int2*>(lane.d_ranges.p + 2 * range_cursor);
            p.range_starts = lane.d_ranges.p + 2 * n_ranges_total + range_cursor;
            int32_t run    = 0;
            for (int r = 0; r < fr.n_ranges; ++r) {
                pairs[2 * (range_cursor + r) + 0] = fr.ranges[2 * r];
                pairs[2 * (range_cursor + r) + 1] = fr.ranges[2 * r + 1];
                starts[range_cursor + r]          = run;
                run += std::max(0, fr.ranges[2 * r + 1] - fr.ranges[2 * r]);
            }
            if (fr.n_ranges == 0) {
                // keep the "host ranges" marker non-null for an empty frame
                p.ranges       = reinterpret_cast<const int2*>(lane.d_ranges.p);
                p.range_starts = lane.d_ranges.p;
            }
            range_cursor += fr.n_ranges;
        }
    }

    lane.d_cand_px.ensure(cand_total + 1);
    lane.d_cand_node.ensure(cand_total + 1);
    lane.d_node_rank.ensure(node_total + 1);
    if (any_device_lookup) lane.d_state.ensure(bsp_total + 1);
    const int blocks_per_frame = std::max(1, (max_cand + SELECT_THREADS - 1) / SELECT_THREADS);
    const int n_blocks         = blocks_per_frame * nf;
    lane.d_block_counts.ensure(n_blocks + 1);
    const int64_t rows_cap = cand_total + nf;
    if (classify) {
        lane.d_feat[0].ensure(static_cast<size_t>(rows_cap) * e->max_width);
        lane.d_feat[1].ensure(static_cast<size_t>(rows_cap) * e->max_width);
        lane.d_images.ensure(image_total + 256);
    }

    // images: host frames go through the lane's device buffer, device frames are read in place. Frames that follow
    // one another in host memory (a caller's ring of camera buffers, the rows of one big array) travel as ONE copy:
    // sixteen 5 MB copies per chunk cost measurably more host time and bus turn-around than one 84 MB copy.
    if (classify) {
        size_t cursor = 0;
        const uint8_t* run_src = nullptr;
        size_t run_dst = 0, run_bytes = 0;
        auto flush = [&] {
            if (run_bytes > 0) VM_CUDA(cudaMemcpyAsync(lane.d_images.p + run_dst, run_src, run_bytes, cudaMemcpyHostToDevice, s));
            run_bytes = 0;
        };
        for (int f = f0; f < f1; ++f) {
            const vm_frame& fr = frames[f];
            FrameParams& p     = lane.h_frames.p[f - f0];
            if (fr.image_on_device) {
                p.image = static_cast<const uint8_t*>(fr.image);
                continue;
            }
            const size_t bytes = image_bytes(fr);
            const uint8_t* src = static_cast<const uint8_t*>(fr.image);
            if (run_bytes > 0 && src == run_src + run_bytes && cursor == run_dst + run_bytes) { run_bytes += bytes; }
            else {
                flush();
                run_src   = src;
                run_dst   = cursor;
                run_bytes = bytes;
            }
            p.image = lane.d_images.p + cursor;
            cursor += (bytes + 255) & ~size_t(255);
        }
        flush();
    }
    VM_CUDA(cudaMemcpyAsync(lane.d_frames.p, lane.h_frames.p, sizeof(FrameParams) * nf, cudaMemcpyHostToDevice, s));
    if (n_ranges_total > 0) {
        VM_CUDA(cudaMemcpyAsync(lane.d_ranges.p, lane.h_ranges.p, sizeof(int32_t) * 3 * n_ranges_total, cudaMemcpyHostToDevice, s));
    }
    VM_CUDA(cudaEventRecord(lane.ev_staged, s));

    if (any_host_ranges) VM_CUDA(cudaMemsetAsync(lane.d_node_rank.p, 0xFF, sizeof(int32_t) * node_total, s));

    if (any_device_lookup) {
        int32_t max_bsp = 0;
        for (int f = f0; f < f1; ++f)
            if (frames[f].ranges == nullptr) max_bsp = std::max(max_bsp, frames[f].mesh->n_bsp);
        dim3 g((max_bsp + SELECT_THREADS - 1) / SELECT_THREADS, nf);
        begin_stage(e, s, "bsp_state");
        k_bsp_state<<<g, SELECT_THREADS, 0, s>>>(lane.d_frames.p, lane.d_state.p);
        VM_CUDA(cudaGetLastError());
        end_stage(e, s);
    }
    {
        dim3 g(blocks_per_frame, nf);
        begin_stage(e, s, "select_project");
        k_select<<<g, SELECT_THREADS, 0, s>>>(lane.d_frames.p, lane.d_state.p, lane.d_cand_px.p, lane.d_cand_node.p,
                                              lane.d_block_counts.p, e->d_abort);
        VM_CUDA(cudaGetLastError());
        end_stage(e, s);
    }
    // the scan continues the batch-wide offsets from the previous chunk's scan
    if (prev != nullptr && prev != &lane) VM_CUDA(cudaStreamWaitEvent(s, prev->ev_scan, 0));
    begin_stage(e, s, "scan");
    k_scan<<<1, 1024, 0, s>>>(lane.d_block_counts.p, n_blocks, blocks_per_frame, nf, e->d_offsets.p, f0);
    VM_CUDA(cudaGetLastError());
    end_stage(e, s);
    VM_CUDA(cudaEventRecord(lane.ev_scan, s));
    VM_CUDA(cudaMemcpyAsync(e->h_offsets.p + f0 + 1, e->d_offsets.p + f0 + 1, sizeof(int32_t) * nf, cudaMemcpyDeviceToHost, s));
    VM_CUDA(cudaEventRecord(lane.ev_offsets, s));
    {
        dim3 g((blocks_per_frame + SCATTER_UNITS - 1) / SCATTER_UNITS, nf);
        begin_stage(e, s, "scatter_compact");
        k_scatter<SCATTER_UNITS><<<g, SELECT_THREADS, 0, s>>>(lane.d_frames.p, lane.d_cand_px.p, lane.d_cand_node.p, lane.d_block_counts.p,
                                                              blocks_per_frame, e->d_offsets.p, f0, e->d_px.p, e->d_gi.p, lane.d_node_rank.p);
        VM_CUDA(cudaGetLastError());
        end_stage(e, s);
    }
    const int max_rows = max_cand + 1;
    {
        dim3 g((max_rows + ROW_THREADS - 1) / ROW_THREADS, nf);
        const int N = frames[f0].mesh->n_neighbours;
        begin_stage(e, s, "remap_neighbours");
        // the staged layer kernels want a tile plan of the chunk: the remap makes it while it has the indices in hand
        const bool with_plan = classify && e->staged && e->use_tc && e->may_stage && nf <= TC_MAX_FRAMES;
        const st::PlanOut plan = with_plan ? ensure_tile_plan(lane, static_cast<size_t>(rows_cap), supertiles_cap) : st::PlanOut{nullptr, nullptr, nullptr};
#define VM_REMAP(NN)                                                                                                                    \
    if (N == NN) {                                                                                                                      \
        if (with_plan) k_remap<NN, true><<<g, ROW_THREADS, 0, s>>>(lane.d_frames.p, e->d_offsets.p, f0, e->d_gi.p, lane.d_node_rank.p, e->d_nb.p, plan); \
        else k_remap<NN, false><<<g, ROW_THREADS, 0, s>>>(lane.d_frames.p, e->d_offsets.p, f0, e->d_gi.p, lane.d_node_rank.p, e->d_nb.p, plan); \
    }
        VM_REMAP(4) VM_REMAP(6) VM_REMAP(8)
#undef VM_REMAP
        lane.plan_valid = with_plan;
        VM_CUDA(cudaGetLastError());
        end_stage(e, s);
        if (classify) {
            begin_stage(e, s, "sample_image");
            bool packed4 = true;
            for (int f = f0; f < f1; ++f) {
                const int cls = format_class(frames[f].format);
                packed4 &= cls == FMT_RGBA || cls == FMT_BGRA;
            }
            const dim3 gs((max_rows + ROW_THREADS * SAMPLE_ROWS - 1) / (ROW_THREADS * SAMPLE_ROWS), nf);
            if (packed4) {
                k_sample<true><<<gs, ROW_THREADS, 0, s>>>(lane.d_frames.p, e->d_offsets.p, f0, e->d_px.p,
                                                         reinterpret_cast<float4*>(lane.d_feat[0].p));
            }
            else {
                k_sample<false><<<gs, ROW_THREADS, 0, s>>>(lane.d_frames.p, e->d_offsets.p, f0, e->d_px.p,
                                                          reinterpret_cast<float4*>(lane.d_feat[0].p));
            }
            VM_CUDA(cudaGetLastError());
            end_stage(e, s);
            run_network(e, lane, e->d_offsets.p, e->d_nb.p, N, f0, nf, max_rows, e->d_cls.p, true, static_cast<int>(rows_cap));
        }
    }
    lane.busy = true;
}

// Copies a finished chunk's results to the host. Needs the chunk's offsets on the host first.
static void enqueue_chunk_readback(vm_engine* e, Lane& lane, int N, bool classify, bool to_host) {
    VM_CUDA(cudaEventSynchronize(lane.ev_offsets));
    if (to_host) {
        const int32_t* off = e->h_offsets.p;
        const size_t p0 = off[lane.f0], p1 = off[lane.f1];
        const size_t r0 = p0 + lane.f0, r1 = p1 + lane.f1;
        cudaStream_t s = lane.stream;
        if (p1 > p0) {
            VM_CUDA(cudaMemcpyAsync(e->h_px.p + p0, e->d_px.p + p0, sizeof(float2) * (p1 - p0), cudaMemcpyDeviceToHost, s));
            VM_CUDA(cudaMemcpyAsync(e->h_gi.p + p0, e->d_gi.p + p0, sizeof(int32_t) * (p1 - p0), cudaMemcpyDeviceToHost, s));
        }
        VM_CUDA(cudaMemcpyAsync(e->h_nb.p + r0 * N, e->d_nb.p + r0 * N, sizeof(int32_t) * (r1 - r0) * N, cudaMemcpyDeviceToHost, s));
        if (classify) {
            const size_t C = e->n_classes;
            VM_CUDA(cudaMemcpyAsync(e->h_cls.p + r0 * C, e->d_cls.p + r0 * C, sizeof(float) * (r1 - r0) * C, cudaMemcpyDeviceToHost, s));
        }
    }
    VM_CUDA(cudaEventRecord(lane.ev_done, lane.stream));
}

static vm_status run_batch(vm_engine* e, const vm_frame* frames, int32_t n_frames, uint32_t flags, vm_batch_result* out) {
    if (e == nullptr || out == nullptr || n_frames < 0 || (n_frames > 0 && frames == nullptr)) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null engine, frames or result");
    }
    std::memset(out, 0, sizeof(*out));
    if (n_frames == 0) return VM_OK;
    struct BatchRange {  // one NVTX range per batch, closed on every way out
        bool on;
        explicit BatchRange(bool enabled) : on(enabled) {
            if (on) nvtxRangePushA("vm_run_batch");
        }
        ~BatchRange() {
            if (on) nvtxRangePop();
        }
    } batch_range(e->nvtx);

    // validation, before any device work - the reference throws from inside the call for the same conditions
    bool classify = frames[0].image != nullptr && !e->layers.empty();
    const int N   = frames[0].mesh != nullptr ? frames[0].mesh->n_neighbours : 0;
    int64_t cand_all = 0;
    for (int f = 0; f < n_frames; ++f) {
        const vm_frame& fr = frames[f];
        if (fr.mesh == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "frame without a mesh");
        if (fr.mesh->owner != e) return fail(VM_ERR_INVALID_ARGUMENT, "mesh was uploaded through another engine");
        if (fr.mesh->n_neighbours != N) return fail(VM_ERR_INVALID_ARGUMENT, "frames of one batch must share n_neighbours");
        if (fr.lens.projection != VM_RECTILINEAR && fr.lens.projection != VM_EQUISOLID && fr.lens.projection != VM_EQUIDISTANT) {
            return fail(VM_ERR_UNSUPPORTED_LENS, "Cannot project: Unknown lens type");
        }
        if (fr.lens.dimensions[0] <= 0 || fr.lens.dimensions[1] <= 0) return fail(VM_ERR_INVALID_ARGUMENT, "lens dimensions must be positive");
        if (fr.ranges == nullptr && fr.n_ranges != 0) return fail(VM_ERR_INVALID_ARGUMENT, "n_ranges without ranges");
        if (fr.ranges == nullptr && fr.mesh->n_bsp == 0) return fail(VM_ERR_NO_BSP, "device lookup needs vm_mesh_set_bsp");
        if (fr.n_ranges < 0) return fail(VM_ERR_INVALID_ARGUMENT, "negative n_ranges");
        for (int r = 0; r < fr.n_ranges; ++r) {
            if (fr.ranges[2 * r] < 0 || fr.ranges[2 * r + 1] > fr.mesh->n_nodes || fr.ranges[2 * r] > fr.ranges[2 * r + 1]) {
                return fail(VM_ERR_INVALID_ARGUMENT, "range outside the mesh");
            }
        }
        if ((fr.image != nullptr) != (frames[0].image != nullptr)) return fail(VM_ERR_INVALID_ARGUMENT, "either all frames carry an image or none");
        if (classify && format_class(fr.format) == FMT_UNKNOWN) {
            char code[5] = {char(fr.format & 0xFF), char(fr.format >> 8 & 0xFF), char(fr.format >> 16 & 0xFF), char(fr.format >> 24 & 0xFF), 0};
            return fail(VM_ERR_UNSUPPORTED_FORMAT, std::string("Unsupported image format ") + code);
        }
        cand_all += frame_candidates(fr);
    }
    if (classify && e->layers.front().cin != 4) return fail(VM_ERR_NETWORK_SHAPE, "first layer must take 4 channels");
    if (classify && e->layers.front().n_slots != N + 1) return fail(VM_ERR_NETWORK_SHAPE, "network was built for a different n_neighbours");
    if (cand_all + n_frames > (int64_t(1) << 31) - 1024) return fail(VM_ERR_INVALID_ARGUMENT, "batch too large: split it");

    try {
        VM_CUDA(cudaSetDevice(e->device));
        e->timing = (flags & VM_TIME_STAGES) != 0;
        e->timers.clear();
        e->events_used = 0;
        e->stage_ms.clear();
        const bool to_host = (flags & VM_RESULTS_ON_DEVICE) == 0;
        const int n_lanes  = e->timing ? 1 : e->n_lanes;

        const size_t rows_all = static_cast<size_t>(cand_all) + n_frames;
        e->d_offsets.ensure(n_frames + 1);
        e->h_offsets.ensure(n_frames + 1);
        e->d_px.ensure(cand_all + 1);
        e->d_gi.ensure(cand_all + 1);
        e->d_nb.ensure(rows_all * N);
        if (classify) e->d_cls.ensure(rows_all * e->n_classes);
        if (to_host) {
            e->h_px.ensure(cand_all + 1);
            e->h_gi.ensure(cand_all + 1);
            e->h_nb.ensure(rows_all * N);
            if (classify) e->h_cls.ensure(rows_all * e->n_classes);
        }
        e->h_offsets.p[0] = 0;
        *e->h_abort       = 0;
        VM_CUDA(cudaMemsetAsync(e->d_offsets.p, 0, sizeof(int32_t), e->lanes[0].stream));
        VM_CUDA(cudaMemsetAsync(e->d_abort, 0, sizeof(int32_t), e->lanes[0].stream));
        // kernels of the other lanes raise the same abort flag: their first chunk must not start before the clear
        VM_CUDA(cudaEventRecord(e->ev_batch_start, e->lanes[0].stream));
        for (int l = 1; l < n_lanes; ++l) VM_CUDA(cudaStreamWaitEvent(e->lanes[l].stream, e->ev_batch_start, 0));

        // chunks: runs of frames bounded by a candidate budget and a frame count. Small chunks let the copies of one
        // chunk overlap the kernels of another; when there is nothing to copy in (frames already on the device, or
        // projection only) larger chunks mean fewer, fuller launches.
        bool host_images = false;
        for (int f = 0; f < n_frames; ++f) host_images = host_images || (classify && !frames[f].image_on_device);
        const int64_t max_chunk_candidates = (e->chunk_override || host_images) ? e->chunk_candidates : 4 * e->chunk_candidates;
        const int max_chunk_frames         = (e->chunk_override || host_images) ? e->chunk_frames : std::min(4 * e->chunk_frames, static_cast<int>(TC_MAX_FRAMES));
        int f0 = 0, chunk = 0;
        Lane* prev = nullptr;
        std::vector<Lane*> order;
        while (f0 < n_frames) {
            int f1 = f0;
            int64_t c = 0;
            while (f1 < n_frames && (f1 == f0 || (c + frame_candidates(frames[f1]) <= max_chunk_candidates && f1 - f0 < max_chunk_frames))) {
                c += frame_candidates(frames[f1]);
                ++f1;
            }
            Lane& lane = e->lanes[chunk % n_lanes];
            if (lane.busy) {
                // its previous chunk must have left the lane's staging and scratch
                VM_CUDA(cudaEventSynchronize(lane.ev_done));
                lane.busy = false;
            }
            enqueue_chunk(e, lane, prev, frames, f0, f1, classify);
            // while this chunk runs, read back the one before it
            if (prev != nullptr) enqueue_chunk_readback(e, *prev, N, classify, to_host);
            if (n_lanes == 1) {
                enqueue_chunk_readback(e, lane, N, classify, to_host);
                prev = nullptr;
                // a single lane still has to chain its scans: same stream, already ordered
            }
            else {
                prev = &lane;
            }
            f0 = f1;
            ++chunk;
        }
        if (prev != nullptr) enqueue_chunk_readback(e, *prev, N, classify, to_host);
        // the abort flag is read once, after the last kernel of EVERY lane: the chunks before the last one run on
        // other streams and may still be in their network layers when the last chunk's stream gets here
        cudaStream_t last_stream = e->lanes[(chunk - 1) % n_lanes].stream;
        for (int l = 0; l < n_lanes; ++l) {
            if (e->lanes[l].busy && e->lanes[l].stream != last_stream) VM_CUDA(cudaStreamWaitEvent(last_stream, e->lanes[l].ev_done, 0));
        }
        VM_CUDA(cudaMemcpyAsync(e->h_abort, e->d_abort, sizeof(int32_t), cudaMemcpyDeviceToHost, last_stream));
        // the last stream has waited for every other lane: one event behind the flag's copy marks the end of the batch
        VM_CUDA(cudaEventRecord(e->ev_batch_done, last_stream));
        VM_CUDA(cudaEventSynchronize(e->ev_batch_done));
        for (int l = 0; l < n_lanes; ++l) e->lanes[l].busy = false;
        if (*e->h_abort == ABORT_TC_RANGE && e->use_tc) {
            // a feature value beyond the range of the fp16 split: this engine goes back to the FFMA kernels for good and
            // the batch is computed again
            e->use_tc = false;
            return run_batch(e, frames, n_frames, flags, out);
        }
        if (*e->h_abort == ABORT_TC_TIMEOUT) return fail(VM_ERR_DEVICE_ABORT, "a tensor-core kernel gave up waiting on an mbarrier");
        if (*e->h_abort != 0) return fail(VM_ERR_DEVICE_ABORT, "a kernel gave up on a bounded loop (BSP deeper than 128 levels)");

        if (e->timing) {
            for (const auto& t : e->timers) {
                float ms = 0.0f;
                VM_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop));
                e->stage_ms.emplace_back(t.name, ms);
            }
        }

        out->n_frames     = n_frames;
        out->n_neighbours = N;
        out->n_classes    = classify ? e->n_classes : 0;
        out->on_device    = to_host ? 0 : 1;
        out->offsets      = e->h_offsets.p;
        if (to_host) {
            out->pixel_coordinates = reinterpret_cast<const float*>(e->h_px.p);
            out->global_indices    = e->h_gi.p;
            out->neighbourhood     = e->h_nb.p;
            out->classifications   = classify ? e->h_cls.p : nullptr;
        }
        else {
            out->pixel_coordinates = reinterpret_cast<const float*>(e->d_px.p);
            out->global_indices    = e->d_gi.p;
            out->neighbourhood     = e->d_nb.p;
            out->classifications   = classify ? e->d_cls.p : nullptr;
        }
        return VM_OK;
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        const vm_status s = f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA;
        return fail(s, std::string(cudaGetErrorName(f.code)) + ": " + cudaGetErrorString(f.code) + " in " + f.what);
    }
    catch (const UnsupportedLens&) {
        // work already enqueued for earlier chunks finishes on its own; the lanes are drained before the next batch
        for (int l = 0; l < MAX_LANES; ++l) {
            cudaStreamSynchronize(e->lanes[l].stream);
            e->lanes[l].busy = false;
        }
        return fail(VM_ERR_UNSUPPORTED_LENS, "Cannot project: Unknown lens type");
    }
}

}  // namespace vm

using namespace vm;

extern "C" {

const char* vm_last_error(void) {
    return g_error.c_str();
}

// lets the host mesh translation unit report through the same per-thread message
void vm_set_last_error_(const char* message) {
    g_error = message != nullptr ? message : "";
}

vm_status vm_engine_create(int device, const vm_layer* layers, const int32_t* layers_per_group, int32_t n_groups, vm_engine** out) {
    if (out == nullptr || n_groups < 0 || (n_groups > 0 && (layers == nullptr || layers_per_group == nullptr))) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    }
    *out = nullptr;
    // shape check: cpp/visualmesh/engine/cpu/engine.hpp:213-256 multiplies whatever it is given; a mismatch there is
    // undefined behaviour, here it is an error
    {
        int l = 0, width = 4, slots_first = 0;
        for (int g = 0; g < n_groups; ++g) {
            if (layers_per_group[g] <= 0) return fail(VM_ERR_NETWORK_SHAPE, "a group needs at least one layer");
            for (int i = 0; i < layers_per_group[g]; ++i, ++l) {
                const vm_layer& L = layers[l];
                if (L.weights == nullptr || L.biases == nullptr || L.n_in <= 0 || L.n_out <= 0) return fail(VM_ERR_NETWORK_SHAPE, "empty layer");
                if (L.activation < VM_SELU || L.activation > VM_TANH) return fail(VM_ERR_NETWORK_SHAPE, "unknown activation");
                if (i == 0) {
                    if (L.n_in % width != 0) return fail(VM_ERR_NETWORK_SHAPE, "gather layer rows must be (N+1) x previous width");
                    const int slots = L.n_in / width;
                    if (slots != 5 && slots != 7 && slots != 9) return fail(VM_ERR_NETWORK_SHAPE, "gather layer rows must be (N+1) x previous width, N in {4,6,8}");
                    if (slots_first == 0) slots_first = slots;
                    if (slots != slots_first) return fail(VM_ERR_NETWORK_SHAPE, "all groups must gather the same number of neighbours");
                }
                else if (L.n_in != width) {
                    return fail(VM_ERR_NETWORK_SHAPE, "dense layer rows must equal the previous width");
                }
                width = L.n_out;
            }
        }
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(VM_ERR_CUDA, "no CUDA device: this engine has no CPU fallback");
    }
    std::unique_ptr<vm_engine> e(new vm_engine());
    try {
        if (device < 0) VM_CUDA(cudaGetDevice(&device));
        if (device >= count) return fail(VM_ERR_INVALID_ARGUMENT, "no such device");
        e->device = device;
        VM_CUDA(cudaSetDevice(device));
        if (const char* v = std::getenv("VMCUDA_CHUNK_FRAMES")) {
            e->chunk_frames   = std::max(1, std::atoi(v));
            e->chunk_override = true;
        }
        if (const char* v = std::getenv("VMCUDA_CHUNK_CANDIDATES")) {
            e->chunk_candidates = std::max<long long>(1, std::atoll(v));
            e->chunk_override   = true;
        }
        if (const char* v = std::getenv("VMCUDA_TC")) {
            e->tc_mode = std::atoi(v);
            e->use_tc  = e->tc_mode != 0;
        }
        if (const char* v = std::getenv("VMCUDA_TC_MIN_PRODUCT")) e->tc_min_product = std::atoi(v);
        if (const char* v = std::getenv("VMCUDA_TC_NO_SPLIT")) e->tc_no_split = std::atoi(v) != 0;
        if (const char* v = std::getenv("VMCUDA_STAGED")) e->staged = std::atoi(v) != 0;
        if (const char* v = std::getenv("VMCUDA_BLOCKING_SYNC")) e->blocking_sync = std::atoi(v) != 0;
        if (const char* v = std::getenv("VMCUDA_NVTX")) e->nvtx = std::atoi(v) != 0;
        if (const char* v = std::getenv("VMCUDA_LANES")) e->n_lanes = std::min(MAX_LANES, std::max(1, std::atoi(v)));
        for (int l = 0; l < MAX_LANES; ++l) {
            Lane& lane = e->lanes[l];
            VM_CUDA(cudaStreamCreateWithFlags(&lane.stream, cudaStreamNonBlocking));
            VM_CUDA(cudaEventCreateWithFlags(&lane.ev_staged, cudaEventDisableTiming));
            VM_CUDA(cudaEventCreateWithFlags(&lane.ev_scan, cudaEventDisableTiming));
            // the two events the host waits on: spinning (lowest latency) or, with VMCUDA_BLOCKING_SYNC=1, sleeping - for
            // boxes where several engines' host threads share few cores
            const unsigned wait_flags = cudaEventDisableTiming | (e->blocking_sync ? cudaEventBlockingSync : 0);
            VM_CUDA(cudaEventCreateWithFlags(&lane.ev_offsets, wait_flags));
            VM_CUDA(cudaEventCreateWithFlags(&lane.ev_done, wait_flags));
        }
        VM_CUDA(cudaEventCreate(&e->ev_timer_start));
        VM_CUDA(cudaEventCreate(&e->ev_timer_stop));
        VM_CUDA(cudaEventCreateWithFlags(&e->ev_batch_start, cudaEventDisableTiming));
        VM_CUDA(cudaEventCreateWithFlags(&e->ev_batch_done, cudaEventDisableTiming | (e->blocking_sync ? cudaEventBlockingSync : 0)));
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&e->d_abort), sizeof(int32_t)));
        VM_CUDA(cudaHostAlloc(reinterpret_cast<void**>(&e->h_abort), sizeof(int32_t), cudaHostAllocDefault));
        int l = 0;
        int width = 4;
        for (int g = 0; g < n_groups; ++g) {
            for (int i = 0; i < layers_per_group[g]; ++i, ++l) {
                const vm_layer& L = layers[l];
                DenseLayer d;
                d.n_slots    = i == 0 ? L.n_in / width : 1;
                d.cin        = width;
                d.cout       = L.n_out;
                d.coutp      = (L.n_out + 3) & ~3;
                d.activation = L.activation;
                d.stage      = std::string(i == 0 ? "graph_conv_" : "dense_") + std::to_string(width) + "x" + std::to_string(L.n_out);
                // [n_in][n_out] as handed over (cpp/visualmesh/network_structure.hpp:25-27), padded to coutp columns
                std::vector<float> packed((static_cast<size_t>(L.n_in) + 1) * d.coutp, 0.0f);
                for (int r = 0; r < L.n_in; ++r)
                    for (int c = 0; c < L.n_out; ++c) packed[static_cast<size_t>(r) * d.coutp + c] = L.weights[static_cast<size_t>(r) * L.n_out + c];
                for (int c = 0; c < L.n_out; ++c) packed[static_cast<size_t>(L.n_in) * d.coutp + c] = L.biases[c];
                VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&d.d_weights), packed.size() * sizeof(float)));
                VM_CUDA(cudaMemcpy(d.d_weights, packed.data(), packed.size() * sizeof(float), cudaMemcpyHostToDevice));
                d.host_packed = packed;
                // tensor-core copy of the weights: per 16-byte K chunk, NP rows of hi parts then NP rows of lo parts
                if ((width == 8 || width == 16 || width == 32) && L.n_out <= 32 && i == 0) {
                    const int np    = L.n_out <= 16 ? 16 : 32;
                    const int K     = L.n_in;
                    const bool half = width != 8;
                    const int kch   = half ? 8 : 4;
                    float w_max     = 0.0f;
                    for (size_t q = 0; q < size_t(K) * L.n_out; ++q) w_max = std::max(w_max, std::fabs(L.weights[q]));
                    const size_t smem_need = 256 + size_t(9) * 2 * (width / kch) * 128 * 16 + size_t(K / kch) * 2 * np * 16;
                    if (smem_need <= 200 * 1024 && (!half || w_max < 60000.0f)) {
                        const size_t chunks = size_t(K / kch);
                        std::vector<unsigned char> cat(chunks * 2 * np * 16, 0);
                        std::vector<float> bias(np, 0.0f);
                        for (int k = 0; k < K; ++k) {
                            for (int n = 0; n < L.n_out; ++n) {
                                const float w     = L.weights[size_t(k) * L.n_out + n];
                                const size_t base = size_t(k / kch) * 2 * np * 16;
                                if (half) {
                                    const __half h = __float2half_rn(w);
                                    const __half l = __float2half_rn(w - __half2float(h));
                                    std::memcpy(&cat[base + size_t(n) * 16 + (k % kch) * 2], &h, 2);
                                    std::memcpy(&cat[base + size_t(np + n) * 16 + (k % kch) * 2], &l, 2);
                                }
                                else {
                                    uint32_t bits;
                                    std::memcpy(&bits, &w, sizeof(bits));
                                    bits &= 0xFFFFE000u;
                                    float h;
                                    std::memcpy(&h, &bits, sizeof(h));
                                    const float l = w - h;
                                    std::memcpy(&cat[base + size_t(n) * 16 + (k % kch) * 4], &h, 4);
                                    std::memcpy(&cat[base + size_t(np + n) * 16 + (k % kch) * 4], &l, 4);
                                }
                            }
                        }
                        for (int n = 0; n < L.n_out; ++n) bias[n] = L.biases[n];
                        VM_CUDA(cudaMalloc(&d.d_tc_cat, cat.size()));
                        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&d.d_tc_bias), bias.size() * sizeof(float)));
                        VM_CUDA(cudaMemcpy(d.d_tc_cat, cat.data(), cat.size(), cudaMemcpyHostToDevice));
                        VM_CUDA(cudaMemcpy(d.d_tc_bias, bias.data(), bias.size() * sizeof(float), cudaMemcpyHostToDevice));
                        d.tc_np   = np;
                        d.tc_half = half;
                    }
                }
                e->layers.push_back(d);
                width        = L.n_out;
                e->max_width = std::max(e->max_width, width);
            }
        }
        e->n_classes = e->layers.empty() ? 0 : e->layers.back().cout;
        for (size_t l = 1; l + 1 < e->layers.size(); ++l) e->may_stage = e->may_stage || has_staged_kernel(e->layers[l]);
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA,
                    std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    *out = e.release();
    return VM_OK;
}

static void free_mesh(vm_mesh* m) {
    if (m == nullptr) return;
    cudaFree(m->d_rays);
    cudaFree(m->d_neighbours);
    cudaFree(m->d_cones_a);
    cudaFree(m->d_cones_s);
    cudaFree(m->d_topology);
    delete m;
}

void vm_engine_destroy(vm_engine* e) {
    if (e == nullptr) return;
    cudaSetDevice(e->device);
    cudaDeviceSynchronize();
    for (auto* m : e->meshes) free_mesh(m);
    for (auto& L : e->layers) {
        cudaFree(L.d_weights);
        cudaFree(L.d_tc_cat);
        cudaFree(L.d_tc_bias);
    }
    for (auto& lane : e->lanes) {
        lane.h_frames.release();
        lane.d_frames.release();
        lane.h_ranges.release();
        lane.d_ranges.release();
        lane.d_state.release();
        lane.d_cand_px.release();
        lane.d_cand_node.release();
        lane.d_block_counts.release();
        lane.d_node_rank.release();
        lane.d_feat[0].release();
        lane.d_feat[1].release();
        lane.d_images.release();
        lane.d_nbl.release();
        lane.d_halo_rows.release();
        lane.d_halo_count.release();
        if (lane.stream) cudaStreamDestroy(lane.stream);
        if (lane.ev_staged) cudaEventDestroy(lane.ev_staged);
        if (lane.ev_scan) cudaEventDestroy(lane.ev_scan);
        if (lane.ev_offsets) cudaEventDestroy(lane.ev_offsets);
        if (lane.ev_done) cudaEventDestroy(lane.ev_done);
    }
    e->d_offsets.release();
    e->h_offsets.release();
    e->d_px.release();
    e->d_gi.release();
    e->d_nb.release();
    e->d_cls.release();
    e->h_px.release();
    e->h_gi.release();
    e->h_nb.release();
    e->h_cls.release();
    for (auto ev : e->event_pool) cudaEventDestroy(ev);
    if (e->ev_timer_start) cudaEventDestroy(e->ev_timer_start);
    if (e->ev_timer_stop) cudaEventDestroy(e->ev_timer_stop);
    if (e->ev_batch_start) cudaEventDestroy(e->ev_batch_start);
    if (e->ev_batch_done) cudaEventDestroy(e->ev_batch_done);
    cudaFree(e->d_abort);
    cudaFreeHost(e->h_abort);
    delete e;
}

vm_status vm_mesh_upload(vm_engine* e, const float* rays, const int32_t* neighbours, int32_t n_nodes, int32_t n_neighbours, vm_mesh** out) {
    if (e == nullptr || rays == nullptr || neighbours == nullptr || out == nullptr || n_nodes <= 0) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument or empty mesh");
    }
    if (n_neighbours != 4 && n_neighbours != 6 && n_neighbours != 8) return fail(VM_ERR_INVALID_ARGUMENT, "n_neighbours must be 4, 6 or 8");
    *out = nullptr;
    std::unique_ptr<vm_mesh> m(new vm_mesh());
    try {
        VM_CUDA(cudaSetDevice(e->device));
        m->owner        = e;
        m->n_nodes      = n_nodes;
        m->n_neighbours = n_neighbours;
        // rays padded to float4 as the OpenCL engine does (cpp/visualmesh/engine/opencl/engine.hpp:611-615)
        std::vector<float4> padded(n_nodes);
        for (int i = 0; i < n_nodes; ++i) padded[i] = make_float4(rays[3 * i], rays[3 * i + 1], rays[3 * i + 2], 0.0f);
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->d_rays), sizeof(float4) * n_nodes));
        VM_CUDA(cudaMemcpy(m->d_rays, padded.data(), sizeof(float4) * n_nodes, cudaMemcpyHostToDevice));
        const size_t nb_bytes = sizeof(int32_t) * static_cast<size_t>(n_nodes) * n_neighbours;
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->d_neighbours), nb_bytes));
        VM_CUDA(cudaMemcpy(m->d_neighbours, neighbours, nb_bytes, cudaMemcpyHostToDevice));
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        free_mesh(m.release());
        return fail(f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    e->meshes.push_back(m.get());
    *out = m.release();
    return VM_OK;
}

vm_status vm_mesh_set_bsp(vm_engine* e, vm_mesh* m, int32_t n, const int32_t* ranges, const int32_t* children, const float* cones) {
    if (e == nullptr || m == nullptr || n <= 0 || ranges == nullptr || children == nullptr || cones == nullptr) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument or empty BSP");
    }
    std::vector<float4> a(n);
    std::vector<float> s(n);
    std::vector<int4> t(n);
    for (int i = 0; i < n; ++i) {
        a[i] = make_float4(cones[5 * i], cones[5 * i + 1], cones[5 * i + 2], cones[5 * i + 3]);
        s[i] = cones[5 * i + 4];
        const int c0 = children[2 * i], c1 = children[2 * i + 1];
        if (c0 >= n || c1 >= n || (c0 < 0) != (c1 < 0)) return fail(VM_ERR_INVALID_ARGUMENT, "BSP child out of range");
        if (ranges[2 * i] < 0 || ranges[2 * i + 1] > m->n_nodes) return fail(VM_ERR_INVALID_ARGUMENT, "BSP range outside the mesh");
        t[i] = make_int4(c0, c1, c1 >= 0 ? ranges[2 * c1] : 0, 0);
    }
    try {
        VM_CUDA(cudaSetDevice(e->device));
        cudaFree(m->d_cones_a);
        cudaFree(m->d_cones_s);
        cudaFree(m->d_topology);
        m->d_cones_a = nullptr;
        m->d_cones_s = nullptr;
        m->d_topology = nullptr;
        m->n_bsp = 0;
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->d_cones_a), sizeof(float4) * n));
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->d_cones_s), sizeof(float) * n));
        VM_CUDA(cudaMalloc(reinterpret_cast<void**>(&m->d_topology), sizeof(int4) * n));
        VM_CUDA(cudaMemcpy(m->d_cones_a, a.data(), sizeof(float4) * n, cudaMemcpyHostToDevice));
        VM_CUDA(cudaMemcpy(m->d_cones_s, s.data(), sizeof(float) * n, cudaMemcpyHostToDevice));
        VM_CUDA(cudaMemcpy(m->d_topology, t.data(), sizeof(int4) * n, cudaMemcpyHostToDevice));
        m->n_bsp = n;
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    return VM_OK;
}

void vm_mesh_release(vm_engine* e, vm_mesh* m) {
    if (e == nullptr || m == nullptr) return;
    cudaSetDevice(e->device);
    cudaDeviceSynchronize();
    e->meshes.erase(std::remove(e->meshes.begin(), e->meshes.end(), m), e->meshes.end());
    free_mesh(m);
}

vm_status vm_run_batch(vm_engine* e, const vm_frame* frames, int32_t n_frames, uint32_t flags, vm_batch_result* out) {
    return run_batch(e, frames, n_frames, flags, out);
}

vm_status vm_project(vm_engine* e, const vm_mesh* mesh, const int32_t* ranges, int32_t n_ranges, const float Hoc[16], const vm_lens* lens, vm_batch_result* out) {
    if (Hoc == nullptr || lens == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null Hoc or lens");
    vm_frame fr{};
    fr.mesh     = mesh;
    fr.ranges   = ranges;
    fr.n_ranges = n_ranges;
    std::memcpy(fr.Hoc, Hoc, sizeof(fr.Hoc));
    fr.lens = *lens;
    return run_batch(e, &fr, 1, 0, out);
}

vm_status vm_classify(vm_engine* e, const vm_mesh* mesh, const int32_t* ranges, int32_t n_ranges, const float Hoc[16], const vm_lens* lens, const void* image, uint32_t format, vm_batch_result* out) {
    if (Hoc == nullptr || lens == nullptr || image == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null Hoc, lens or image");
    if (e != nullptr && e->layers.empty()) return fail(VM_ERR_NETWORK_SHAPE, "this engine was created without a network");
    vm_frame fr{};
    fr.mesh     = mesh;
    fr.ranges   = ranges;
    fr.n_ranges = n_ranges;
    std::memcpy(fr.Hoc, Hoc, sizeof(fr.Hoc));
    fr.lens   = *lens;
    fr.image  = image;
    fr.format = format;
    return run_batch(e, &fr, 1, 0, out);
}

vm_status vm_sample(vm_engine* e, const float* px, int32_t n, const void* image, int32_t width, int32_t height, uint32_t format, float* out) {
    if (e == nullptr || px == nullptr || image == nullptr || out == nullptr || n < 0 || width <= 0 || height <= 0) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    }
    const int cls = format_class(format);
    if (cls == FMT_UNKNOWN) return fail(VM_ERR_UNSUPPORTED_FORMAT, "Unsupported image format");
    if (n == 0) return VM_OK;
    // The reference reads whatever address a coordinate outside the image leads to (cpp/visualmesh/engine/cpu/
    // pixel.hpp:131-134 clamp only one side); the engine itself only samples points that passed the on-screen test.
    // Here the coordinates come from the caller, so they are checked: a read outside the image would be a GPU fault.
    for (int32_t i = 0; i < n; ++i) {
        const float x = px[2 * i], y = px[2 * i + 1];
        if (!(x >= 0.0f && x <= static_cast<float>(width - 1) && y >= 0.0f && y <= static_cast<float>(height - 1))) {
            return fail(VM_ERR_INVALID_ARGUMENT, "pixel coordinate " + std::to_string(i) + " is outside the image (or not finite)");
        }
    }
    try {
        VM_CUDA(cudaSetDevice(e->device));
        Lane& lane        = e->lanes[0];
        const size_t bytes = static_cast<size_t>(width) * height * format_bytes_per_pixel(cls);
        lane.d_images.ensure(bytes);
        lane.d_cand_px.ensure(n);
        lane.d_feat[0].ensure(static_cast<size_t>(n) * 4);
        VM_CUDA(cudaMemcpyAsync(lane.d_images.p, image, bytes, cudaMemcpyHostToDevice, lane.stream));
        VM_CUDA(cudaMemcpyAsync(lane.d_cand_px.p, px, sizeof(float2) * n, cudaMemcpyHostToDevice, lane.stream));
        ++e->launches;
        k_sample_flat<<<(n + ROW_THREADS - 1) / ROW_THREADS, ROW_THREADS, 0, lane.stream>>>(
          lane.d_cand_px.p, n, lane.d_images.p, width, height, cls, reinterpret_cast<float4*>(lane.d_feat[0].p));
        VM_CUDA(cudaGetLastError());
        VM_CUDA(cudaMemcpyAsync(out, lane.d_feat[0].p, sizeof(float) * 4 * n, cudaMemcpyDeviceToHost, lane.stream));
        VM_CUDA(cudaStreamSynchronize(lane.stream));
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    return VM_OK;
}

vm_status vm_network(vm_engine* e, const float* input, const int32_t* neighbourhood, int32_t n_rows, int32_t n_neighbours, float* out) {
    if (e == nullptr || input == nullptr || neighbourhood == nullptr || out == nullptr || n_rows <= 0) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    }
    if (e->layers.empty()) return fail(VM_ERR_NETWORK_SHAPE, "this engine was created without a network");
    if (e->layers.front().n_slots != n_neighbours + 1) return fail(VM_ERR_NETWORK_SHAPE, "network was built for a different n_neighbours");
    for (size_t i = 0; i < static_cast<size_t>(n_rows) * n_neighbours; ++i) {
        if (neighbourhood[i] < 0 || neighbourhood[i] >= n_rows) return fail(VM_ERR_INVALID_ARGUMENT, "neighbour index outside the rows");
    }
    try {
        VM_CUDA(cudaSetDevice(e->device));
        Lane& lane = e->lanes[0];
        const size_t rows = n_rows;
        e->d_offsets.ensure(2);
        e->d_nb.ensure(rows * n_neighbours);
        e->d_cls.ensure(rows * e->n_classes);
        lane.d_feat[0].ensure(rows * e->max_width);
        lane.d_feat[1].ensure(rows * e->max_width);
        const int32_t offsets[2] = {0, n_rows - 1};
        VM_CUDA(cudaMemcpyAsync(e->d_offsets.p, offsets, sizeof(offsets), cudaMemcpyHostToDevice, lane.stream));
        VM_CUDA(cudaMemcpyAsync(e->d_nb.p, neighbourhood, sizeof(int32_t) * rows * n_neighbours, cudaMemcpyHostToDevice, lane.stream));
        e->timing = false;
        for (int attempt = 0; attempt < 2; ++attempt) {
            // the layers ping-pong over the feature buffers, so a second attempt needs the input again
            VM_CUDA(cudaMemcpyAsync(lane.d_feat[0].p, input, sizeof(float) * rows * 4, cudaMemcpyHostToDevice, lane.stream));
            VM_CUDA(cudaMemsetAsync(e->d_abort, 0, sizeof(int32_t), lane.stream));
            lane.plan_valid = false;
            if (e->staged && e->use_tc && e->may_stage) {
                const st::PlanOut plan = ensure_tile_plan(lane, rows, (rows + STAGED_ST - 1) / STAGED_ST + 1);
                ++e->launches;
                launch_tile_plan_kernel(n_neighbours, e->d_offsets.p, e->d_nb.p, plan.nbl, plan.halo_rows, plan.halo_count, 0, 1, n_rows, lane.stream);
                VM_CUDA(cudaGetLastError());
                lane.plan_valid = true;
            }
            run_network(e, lane, e->d_offsets.p, e->d_nb.p, n_neighbours, 0, 1, n_rows, e->d_cls.p, true, n_rows);
            VM_CUDA(cudaMemcpyAsync(out, e->d_cls.p, sizeof(float) * rows * e->n_classes, cudaMemcpyDeviceToHost, lane.stream));
            VM_CUDA(cudaMemcpyAsync(e->h_abort, e->d_abort, sizeof(int32_t), cudaMemcpyDeviceToHost, lane.stream));
            VM_CUDA(cudaStreamSynchronize(lane.stream));
            if (*e->h_abort == ABORT_TC_RANGE && e->use_tc) {
                e->use_tc = false;  // a value beyond the fp16 split's range: recompute with the FFMA kernels
                continue;
            }
            if (*e->h_abort != 0) return fail(VM_ERR_DEVICE_ABORT, "a kernel gave up on a bounded wait");
            break;
        }
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(f.code == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    return VM_OK;
}

// ---- projection without any allocation ----------------------------------------------------------------------------
// All scratch of this entry point is one array inside the library image. In host code `g_static_scratch` is only a
// stand-in for the symbol; the address the kernels need comes from cudaGetSymbolAddress, looked up once per device.
namespace {
constexpr size_t align256(size_t v) {
    return (v + 255) & ~size_t(255);
}
constexpr size_t ST_FRAME   = 0;
constexpr size_t ST_CELLS   = ST_FRAME + align256(sizeof(vm::FrameParams));  // offsets[2], abort flag
constexpr size_t ST_BLOCKS  = ST_CELLS + 256;
constexpr size_t ST_STATE   = ST_BLOCKS + align256(sizeof(int32_t) * (VM_STATIC_MAX_NODES / vm::SELECT_THREADS + 2));
constexpr size_t ST_CAND_PX = ST_STATE + align256(VM_STATIC_MAX_BSP);
constexpr size_t ST_CAND_ID = ST_CAND_PX + align256(sizeof(float2) * VM_STATIC_MAX_NODES);
constexpr size_t ST_RANK    = ST_CAND_ID + align256(sizeof(int32_t) * VM_STATIC_MAX_NODES);
constexpr size_t ST_BYTES   = ST_RANK + align256(sizeof(int32_t) * VM_STATIC_MAX_NODES);

static __device__ __align__(256) unsigned char g_static_scratch[ST_BYTES];

constexpr int ST_MAX_DEVICES = 64;
unsigned char* g_static_address[ST_MAX_DEVICES] = {};
std::once_flag g_static_once[ST_MAX_DEVICES];
}  // namespace

vm_status vm_project_static(vm_engine* e,
                            const vm_mesh* mesh,
                            const float Hoc[16],
                            const vm_lens* lens,
                            float* d_px,
                            int32_t* d_gi,
                            int32_t* d_nb,
                            int32_t* d_n_points,
                            int32_t* n_points) {
    if (e == nullptr || mesh == nullptr || Hoc == nullptr || lens == nullptr || d_px == nullptr || d_gi == nullptr || d_nb == nullptr) {
        return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    }
    if (lens->projection != VM_RECTILINEAR && lens->projection != VM_EQUISOLID && lens->projection != VM_EQUIDISTANT) {
        return fail(VM_ERR_UNSUPPORTED_LENS, "Cannot project: Unknown lens type");
    }
    if (lens->dimensions[0] <= 0 || lens->dimensions[1] <= 0) return fail(VM_ERR_INVALID_ARGUMENT, "lens dimensions must be positive");
    if (mesh->owner != e) return fail(VM_ERR_INVALID_ARGUMENT, "mesh was uploaded through another engine");
    if (mesh->n_bsp == 0) return fail(VM_ERR_NO_BSP, "vm_project_static looks up on the device: the mesh needs vm_mesh_set_bsp");
    if (mesh->n_nodes > VM_STATIC_MAX_NODES) {
        return fail(VM_ERR_INVALID_ARGUMENT, "mesh has " + std::to_string(mesh->n_nodes) + " nodes; vm_project_static holds at most VM_STATIC_MAX_NODES = "
                                               + std::to_string(VM_STATIC_MAX_NODES));
    }
    if (mesh->n_bsp > VM_STATIC_MAX_BSP) {
        return fail(VM_ERR_INVALID_ARGUMENT, "mesh BSP has " + std::to_string(mesh->n_bsp) + " elements; vm_project_static holds at most VM_STATIC_MAX_BSP = "
                                               + std::to_string(VM_STATIC_MAX_BSP));
    }
    if (e->device < 0 || e->device >= ST_MAX_DEVICES) return fail(VM_ERR_INVALID_ARGUMENT, "device ordinal out of range");
    try {
        VM_CUDA(cudaSetDevice(e->device));
        // once per device, with that device current; engines of several host threads may get here together
        cudaError_t lookup = cudaSuccess;
        std::call_once(g_static_once[e->device], [&] {
            unsigned char* address = nullptr;
            lookup = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
            if (lookup == cudaSuccess) g_static_address[e->device] = address;
        });
        if (lookup != cudaSuccess) throw CudaFailure{lookup, "cudaGetSymbolAddress(g_static_scratch)"};
        unsigned char* base = g_static_address[e->device];
        if (base == nullptr) return fail(VM_ERR_CUDA, "the address of the static scratch array could not be looked up on this device");
        auto* d_frame         = reinterpret_cast<FrameParams*>(base + ST_FRAME);
        auto* d_cells         = reinterpret_cast<int32_t*>(base + ST_CELLS);  // [0], [1] offsets, [2] abort
        auto* d_blocks        = reinterpret_cast<int32_t*>(base + ST_BLOCKS);
        auto* d_state         = reinterpret_cast<uint8_t*>(base + ST_STATE);
        auto* d_cand_px       = reinterpret_cast<float2*>(base + ST_CAND_PX);
        auto* d_cand_node     = reinterpret_cast<int32_t*>(base + ST_CAND_ID);
        auto* d_rank          = reinterpret_cast<int32_t*>(base + ST_RANK);

        vm_frame fr{};
        fr.mesh = mesh;
        std::memcpy(fr.Hoc, Hoc, sizeof(fr.Hoc));
        fr.lens = *lens;
        FrameParams p;
        std::memset(&p, 0, sizeof(p));
        // never builds the libm last-bit tables here (that allocates): they are used only if an earlier call built them
        if (!fill_frame_params(fr, p, e->device, false)) return fail(VM_ERR_UNSUPPORTED_LENS, "Cannot project: Unknown lens type");
        p.n_candidates = mesh->n_nodes;

        cudaStream_t s = e->lanes[0].stream;
        VM_CUDA(cudaMemcpyAsync(d_frame, &p, sizeof(p), cudaMemcpyHostToDevice, s));
        // the array keeps the last call's contents: the running offset and the abort flag must start at zero
        VM_CUDA(cudaMemsetAsync(d_cells, 0, 4 * sizeof(int32_t), s));
        const int blocks = (mesh->n_nodes + SELECT_THREADS - 1) / SELECT_THREADS;
        k_bsp_state<<<dim3((mesh->n_bsp + SELECT_THREADS - 1) / SELECT_THREADS, 1), SELECT_THREADS, 0, s>>>(d_frame, d_state);
        k_select<<<dim3(blocks, 1), SELECT_THREADS, 0, s>>>(d_frame, d_state, d_cand_px, d_cand_node, d_blocks, d_cells + 2);
        k_scan<<<1, 1024, 0, s>>>(d_blocks, blocks, blocks, 1, d_cells, 0);
        k_scatter<1><<<dim3(blocks, 1), SELECT_THREADS, 0, s>>>(d_frame, d_cand_px, d_cand_node, d_blocks, blocks, d_cells, 0,
                                                             reinterpret_cast<float2*>(d_px), d_gi, d_rank);
        dim3 g((mesh->n_nodes + 1 + ROW_THREADS - 1) / ROW_THREADS, 1);
        const st::PlanOut no_plan{nullptr, nullptr, nullptr};
        if (mesh->n_neighbours == 4) k_remap<4, false><<<g, ROW_THREADS, 0, s>>>(d_frame, d_cells, 0, d_gi, d_rank, d_nb, no_plan);
        else if (mesh->n_neighbours == 6) k_remap<6, false><<<g, ROW_THREADS, 0, s>>>(d_frame, d_cells, 0, d_gi, d_rank, d_nb, no_plan);
        else k_remap<8, false><<<g, ROW_THREADS, 0, s>>>(d_frame, d_cells, 0, d_gi, d_rank, d_nb, no_plan);
        VM_CUDA(cudaGetLastError());
        e->launches += 5;
        if (d_n_points != nullptr) VM_CUDA(cudaMemcpyAsync(d_n_points, d_cells + 1, sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
        int32_t cells[3] = {0, 0, 0};
        VM_CUDA(cudaMemcpyAsync(cells, d_cells, sizeof(cells), cudaMemcpyDeviceToHost, s));
        VM_CUDA(cudaStreamSynchronize(s));
        if (cells[2] != 0) return fail(VM_ERR_DEVICE_ABORT, "a kernel gave up on a bounded loop (BSP deeper than 128 levels)");
        if (n_points != nullptr) *n_points = cells[1];
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + ": " + cudaGetErrorString(f.code) + " in " + f.what);
    }
    return VM_OK;
}

vm_status vm_stage_times(vm_engine* e, const char** names, float* ms, int32_t capacity, int32_t* n) {
    if (e == nullptr || n == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    *n = static_cast<int32_t>(e->stage_ms.size());
    for (int i = 0; i < *n && i < capacity; ++i) {
        if (names != nullptr) names[i] = e->stage_ms[i].first;
        if (ms != nullptr) ms[i] = e->stage_ms[i].second;
    }
    return VM_OK;
}

vm_status vm_timer_start(vm_engine* e) {
    if (e == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null engine");
    try {
        VM_CUDA(cudaSetDevice(e->device));
        for (int l = 0; l < MAX_LANES; ++l) VM_CUDA(cudaStreamSynchronize(e->lanes[l].stream));
        VM_CUDA(cudaEventRecord(e->ev_timer_start, e->lanes[0].stream));
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    return VM_OK;
}

vm_status vm_timer_stop(vm_engine* e, float* milliseconds) {
    if (e == nullptr || milliseconds == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    try {
        VM_CUDA(cudaSetDevice(e->device));
        // lane 0 waits for the other lanes, then stamps the end
        for (int l = 1; l < MAX_LANES; ++l) {
            VM_CUDA(cudaEventRecord(e->lanes[l].ev_staged, e->lanes[l].stream));
            VM_CUDA(cudaStreamWaitEvent(e->lanes[0].stream, e->lanes[l].ev_staged, 0));
        }
        VM_CUDA(cudaEventRecord(e->ev_timer_stop, e->lanes[0].stream));
        VM_CUDA(cudaEventSynchronize(e->ev_timer_stop));
        VM_CUDA(cudaEventElapsedTime(milliseconds, e->ev_timer_start, e->ev_timer_stop));
    }
    catch (const CudaFailure& f) {
        cudaGetLastError();
        return fail(VM_ERR_CUDA, std::string(cudaGetErrorName(f.code)) + " in " + f.what);
    }
    return VM_OK;
}

vm_status vm_set_wait_limit(vm_engine* e, uint32_t polls) {
    if (e == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null engine");
    e->tc_wait_limit = polls;
    return VM_OK;
}

int64_t vm_launch_count(const vm_engine* e) {
    return e == nullptr ? 0 : e->launches;
}

vm_status vm_host_alloc(void** ptr, size_t bytes) {
    if (ptr == nullptr) return fail(VM_ERR_INVALID_ARGUMENT, "null argument");
    const cudaError_t err = cudaHostAlloc(ptr, bytes, cudaHostAllocDefault);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(err == cudaErrorMemoryAllocation ? VM_ERR_OUT_OF_MEMORY : VM_ERR_CUDA, cudaGetErrorString(err));
    }
    return VM_OK;
}

void vm_host_free(void* ptr) {
    if (ptr != nullptr) cudaFreeHost(ptr);
}

}  // extern "C"
