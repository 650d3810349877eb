// Host-side interface between the engine (engine.cu) and the translation units that hold the graph-convolution layer
// kernels with their launchers (conv_ffma.cu, conv_tc.cu, conv_staged.cu). Splitting them keeps every kernel family in
// a translation unit of its own, compiled in parallel.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "conv_args.hpp"

namespace vm {

struct CudaFailure {
    cudaError_t code;
    const char* what;
};
#define VM_CUDA(expr)                                        \
    do {                                                     \
        cudaError_t vm_e_ = (expr);                          \
        if (vm_e_ != cudaSuccess) throw CudaFailure{vm_e_, #expr}; \
    } while (0)

struct DenseLayer {
    float* d_weights = nullptr;  // [n_slots * cin][coutp] then [coutp] biases
    int cin = 0, cout = 0, coutp = 0, n_slots = 1, activation = 0;
    std::string stage;  // name under which this layer's kernel is timed, e.g. "graph_conv_16x16"
    std::vector<float> host_packed;  // [K][coutp] weights then biases, as on the device (for parameter-space kernels)
    // tensor-core path (conv_tc.cuh): weights split into TF32 hi/lo parts in the UMMA K-major layout, padded bias
    void* d_tc_cat   = nullptr;  // [K / KCH chunks][2 * NP rows][16 B]: hi rows then lo rows
    float* d_tc_bias = nullptr;
    int tc_np        = 0;      // padded output width of the tensor-core tile, 0 = no tensor-core path for this shape
    bool tc_half     = false;  // fp16 hi/lo split (16- and 32-channel inputs) or TF32 split (8-channel inputs)
};

// What a launcher works out once per kernel instantiation and device: function attributes are per device, and engine
// instances of several host threads may reach a launcher at the same time.
struct LaunchPlan {
    int ctas_per_sm = 0;
    int n_sms       = 0;
};
constexpr int MAX_DEVICES = 64;
struct LaunchPlans {
    LaunchPlan plan[MAX_DEVICES];
    std::once_flag once[MAX_DEVICES];
    template <typename Init>
    const LaunchPlan& get(Init init) {
        int dev = 0;
        VM_CUDA(cudaGetDevice(&dev));
        dev = std::min(std::max(dev, 0), MAX_DEVICES - 1);
        std::call_once(once[dev], [&] { plan[dev] = init(dev); });
        return plan[dev];
    }
};

// ---- conv_ffma.cu: layers on the CUDA cores ----------------------------------------------------------------------
// a specialised kernel exists for this shape (anything else runs the generic kernel, which ignores ConvArgs::out_split)
bool has_fast_ffma_kernel(int cin, int cout);
void launch_conv_ffma(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, cudaStream_t s);

// ---- conv_tc.cu: layers on the tensor cores, gather by global loads ----------------------------------------------
constexpr int TC_MAX_FRAMES    = 64;  // frames per launch of a tensor-core layer (shared table of tile counts)
constexpr int ABORT_TC_TIMEOUT = 2;   // abort flag: a bounded wait of a tensor-core kernel ran out
constexpr int ABORT_TC_RANGE   = 3;   // abort flag: a feature value too large for the fp16 split
constexpr uint32_t TC_DEFAULT_WAIT_LIMIT = 4000000;
bool has_tc_gather_kernel(const DenseLayer& L);  // gathers fp32 rows and splits them itself
bool has_tc_split_kernel(const DenseLayer& L);   // fed from the split feature layout
bool launch_conv_tc_gather(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s);
bool launch_conv_tc_split(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s);

// ---- conv_staged.cu: layers on the tensor cores, gather from shared-memory windows --------------------------------
// What the tile plan of a chunk holds (device pointers), see conv_staged.cuh.
struct StagedPlan {
    const uint16_t* nbl;
    const int32_t* halo_rows;
    const int32_t* halo_count;
};
constexpr int STAGED_NBL_STRIDE = 8;    // 16-bit neighbour positions per row
constexpr int STAGED_ST         = 256;  // rows of a super-tile
constexpr int STAGED_HALO       = 192;  // halo slots of a super-tile
bool has_staged_kernel(const DenseLayer& L);
bool launch_conv_staged(const DenseLayer& L, const ConvArgs& a, const StagedPlan& plan, int n_frames, int max_rows, int32_t* abort_flag,
                        uint32_t wait_limit, cudaStream_t s);
// the plan for a neighbourhood that is already in memory (the hot path makes it inside the neighbour-remap kernel)
void launch_tile_plan_kernel(int n_neighbours, const int32_t* offsets, const int32_t* nb, uint16_t* nbl, int32_t* halo_rows, int32_t* halo_count,
                             int f0, int n_frames, int max_rows, cudaStream_t s);

}  // namespace vm
