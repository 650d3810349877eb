// Launchers of the CUDA-core graph-convolution layer kernels (conv_ffma.cuh).
#include <cstdlib>
#include <cstring>

#include "conv_dispatch.hpp"
#include "conv_ffma.cuh"

namespace vm {

// layer shapes (C_in, C_out, rows per thread) with a specialised FFMA kernel
#define VM_CONV_SHAPES(X)                                                                                   \
    X(4, 2, 4) X(4, 3, 4) X(4, 4, 4) X(4, 8, 4) X(4, 12, 4) X(4, 16, 4) X(4, 32, 2)                         \
    X(8, 2, 4) X(8, 3, 4) X(8, 4, 4) X(8, 5, 4) X(8, 8, 4) X(8, 12, 4) X(8, 16, 4)                          \
    X(12, 2, 4) X(12, 3, 4) X(12, 4, 4) X(12, 8, 4) X(12, 12, 4) X(12, 16, 4)                               \
    X(16, 2, 4) X(16, 3, 4) X(16, 4, 4) X(16, 5, 4) X(16, 8, 4) X(16, 12, 4) X(16, 16, 4) X(16, 32, 2)      \
    X(32, 2, 4) X(32, 3, 4) X(32, 4, 4) X(32, 8, 4) X(32, 16, 4) X(32, 32, 2)

bool has_fast_ffma_kernel(int cin, int cout) {
#define VM_IS(CI, CO, RR) if (cin == CI && cout == CO) return true;
    VM_CONV_SHAPES(VM_IS)
#undef VM_IS
    return false;
}

template <int CIN, int COUT, int R, int T = CONV_THREADS, int MINB = 1>
static void launch_conv_t(const ConvArgs& a, dim3 grid_rows, int max_rows, cudaStream_t s) {
    constexpr int COUTP = (COUT + 3) & ~3;
    const size_t smem   = (static_cast<size_t>(a.n_slots) * CIN * COUTP + COUTP) * sizeof(float);
    static LaunchPlans plans;
    plans.get([](int) {
        VM_CUDA(cudaFuncSetAttribute(k_graph_conv<CIN, COUT, R, T, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        return LaunchPlan{};
    });
    dim3 grid((max_rows + T * R - 1) / (T * R), grid_rows.y);
    k_graph_conv<CIN, COUT, R, T, MINB><<<grid, T, smem, s>>>(a);
}

constexpr int CW_MAX = 2320;  // floats: a 16 -> 16 layer with 8 neighbours and its biases

template <int CIN, int COUT, int R, int WMAX, int T = CONV_THREADS>
static bool launch_conv_cw(const DenseLayer& L, const ConvArgs& a, dim3 grid_rows, int max_rows, cudaStream_t s) {
    if (L.host_packed.size() > static_cast<size_t>(WMAX)) return false;
    ConvWeights<WMAX> wp;
    std::memcpy(wp.w, L.host_packed.data(), L.host_packed.size() * sizeof(float));
    dim3 grid((max_rows + T * R - 1) / (T * R), grid_rows.y);
    // Layers bound by the latency of their gather rather than by the FP32 pipe - 4-channel first layers, 8 -> 8, and
    // the narrow last layers - run with the slot loop unrolled (slot count as a template parameter): the loads of the
    // next slots are then issued ahead of the current slot's arithmetic. Measured on 4.4 M rows: 4 -> 16 183 -> 114 us
    // (with the weights in the parameter space instead of shared memory), 8 -> 8 133 -> 112 us, 32 -> 4 448 -> 413 us;
    // the 16- and 32-channel layers in between, bound by the FP32 pipe, measured 3-6 % slower unrolled and stay rolled.
    constexpr bool LATENCY_BOUND = (CIN == 8 && COUT == 8) || CIN == 4 || COUT <= 4;
    if (LATENCY_BOUND && a.n_slots == 5) { k_graph_conv_cw<CIN, COUT, R, WMAX, T, LATENCY_BOUND ? 5 : 0><<<grid, T, 0, s>>>(a, wp); }
    else if (LATENCY_BOUND && a.n_slots == 7) {
        k_graph_conv_cw<CIN, COUT, R, WMAX, T, LATENCY_BOUND ? 7 : 0><<<grid, T, 0, s>>>(a, wp);
    }
    else if (LATENCY_BOUND && a.n_slots == 9) {
        k_graph_conv_cw<CIN, COUT, R, WMAX, T, LATENCY_BOUND ? 9 : 0><<<grid, T, 0, s>>>(a, wp);
    }
    else {
        k_graph_conv_cw<CIN, COUT, R, WMAX, T><<<grid, T, 0, s>>>(a, wp);
    }
    return true;
}

// Shapes with a specialised kernel; anything else takes the generic one.
static bool launch_conv_fast(const DenseLayer& L, const ConvArgs& a, dim3 grid, int max_rows, cudaStream_t s) {
    const size_t smem = (static_cast<size_t>(a.n_slots) * L.cin * L.coutp + L.coutp) * sizeof(float);
    if (smem > 96 * 1024) return false;
    // weights small enough for the kernel parameter space are read through the constant cache (measured 15-40 %
    // faster than the shared-memory copy: the weight reads leave the L1/shared data path to the gather)
    static const bool const_weights = [] {
        const char* v = std::getenv("VMCUDA_CONST_WEIGHTS");
        return v == nullptr || v[0] != '0';
    }();
    // the 16 -> 16 layer measured best with two rows per thread and 256 threads
    if (const_weights && L.cin == 16 && L.cout == 16 && launch_conv_cw<16, 16, 2, CW_MAX, 256>(L, a, grid, max_rows, s)) return true;
#define VM_CONV(CI, CO, RR)                                                                       \
    if (L.cin == CI && L.cout == CO) {                                                            \
        /* parameter-space weights: two rows per thread and 256 threads measured best for every shape tried */ \
        if (const_weights && launch_conv_cw<CI, CO, 2, CW_MAX, 256>(L, a, grid, max_rows, s)) return true; \
        launch_conv_t<CI, CO, RR>(a, grid, max_rows, s);                                          \
        return true;                                                                              \
    }
    VM_CONV_SHAPES(VM_CONV)
#undef VM_CONV
    return false;
}


void launch_conv_ffma(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, cudaStream_t s) {
    dim3 grid(1, n_frames);
    if (!launch_conv_fast(L, a, grid, max_rows, s)) {
        dim3 g((max_rows + CONV_THREADS - 1) / CONV_THREADS, n_frames);
        k_graph_conv_generic<<<g, CONV_THREADS, 0, s>>>(a, L.cin, L.cout, L.coutp);
    }
}

}  // namespace vm
