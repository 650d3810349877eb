// Launchers of the staged tensor-core graph-convolution layers and of their tile plan (conv_staged.cuh).
#include <cstdlib>

#include "conv_dispatch.hpp"
#include "../../include/vmcuda.h"
#include "conv_staged.cuh"

namespace vm {

static_assert(STAGED_NBL_STRIDE == st::NBL_STRIDE && STAGED_ST == st::ST && STAGED_HALO == st::HALO,
              "the engine sizes the plan with the kernels' own constants");

template <int CIN, int COUT, int NSLOTS>
static void launch_conv_staged_t(const DenseLayer& L, const ConvArgs& a, const st::Plan& plan, int n_frames, int max_rows, int32_t* abort_flag,
                                 uint32_t wait_limit, cudaStream_t s) {
    constexpr int THREADS = (CIN == 16 ? 8 : 16) * 32 + 32;  // compute warps + the loader warp
    constexpr auto kernel = st::k_graph_conv_mma<CIN, COUT, NSLOTS, THREADS>;
    constexpr size_t smem = st::smem_bytes<CIN, COUT, NSLOTS, THREADS>();
    static LaunchPlans plans;
    const LaunchPlan& lp = plans.get([](int dev) {
        LaunchPlan p;
        VM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        VM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        VM_CUDA(cudaDeviceGetAttribute(&p.n_sms, cudaDevAttrMultiProcessorCount, dev));
        int by_occupancy = 0;
        VM_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&by_occupancy, kernel, THREADS, smem));
        p.ctas_per_sm = std::max(1, by_occupancy);
        if (const char* v = std::getenv("VMCUDA_TC_CTAS")) p.ctas_per_sm = std::max(1, std::min(p.ctas_per_sm, std::atoi(v)));
        return p;
    });
    st::Args t{};
    t.n_frames   = n_frames;
    t.cout       = L.cout;
    t.abort_flag = abort_flag;
    t.wait_limit = wait_limit;
    const int tiles_upper = n_frames * ((max_rows + st::ST - 1) / st::ST);
    const int grid        = std::max(1, std::min(tiles_upper, lp.n_sms * lp.ctas_per_sm));
    kernel<<<grid, THREADS, smem, s>>>(a, t, plan);
}

bool has_staged_kernel(const DenseLayer& L) {
    // tc_half: the layer's weights are within the range of the fp16 split
    // 16-channel inputs: on 32-channel layers the tcgen05 kernel of conv_tc.cuh measured faster (94 against 102 ms for the
    // eight 32 -> 32 layers of 64 frames with 0.93 M rows each), the warp-level MMA rate being what bounds this one there
    return L.tc_np != 0 && L.tc_half && L.cin == 16 && (L.cout == 8 || L.cout == 16 || L.cout == 32)
           && (L.n_slots == 5 || L.n_slots == 7 || L.n_slots == 9) && L.activation != VM_SOFTMAX;
}

bool launch_conv_staged(const DenseLayer& L, const ConvArgs& a, const StagedPlan& plan, int n_frames, int max_rows, int32_t* abort_flag,
                        uint32_t wait_limit, cudaStream_t s) {
    const st::Plan p{plan.nbl, plan.halo_rows, plan.halo_count};
#define VM_STG(CI, CO, NS)                                                                             \
    if (L.cin == CI && L.cout == CO && L.n_slots == NS) {                                                \
        launch_conv_staged_t<CI, CO, NS>(L, a, p, n_frames, max_rows, abort_flag, wait_limit, s);        \
        return true;                                                                                     \
    }
    VM_STG(16, 8, 5) VM_STG(16, 8, 7) VM_STG(16, 8, 9) VM_STG(16, 16, 5) VM_STG(16, 16, 7) VM_STG(16, 16, 9)
    VM_STG(16, 32, 5) VM_STG(16, 32, 7) VM_STG(16, 32, 9)
#undef VM_STG
    return false;
}

void launch_tile_plan_kernel(int n_neighbours, const int32_t* offsets, const int32_t* nb, uint16_t* nbl, int32_t* halo_rows, int32_t* halo_count,
                             int f0, int n_frames, int max_rows, cudaStream_t s) {
    st::PlanArgs p{};
    p.offsets = offsets;
    p.nb      = nb;
    p.out     = st::PlanOut{nbl, halo_rows, halo_count};
    p.f0      = f0;
    dim3 g((max_rows + st::ST - 1) / st::ST, n_frames);
    if (n_neighbours == 4) st::k_tile_plan<4><<<g, st::ST, 0, s>>>(p);
    else if (n_neighbours == 6) st::k_tile_plan<6><<<g, st::ST, 0, s>>>(p);
    else st::k_tile_plan<8><<<g, st::ST, 0, s>>>(p);
}

}  // namespace vm

#ifdef VM_PROFILE_STAGED
extern "C" __attribute__((visibility("default"))) int vm_debug_staged_profile(long long* out, int n) {
    return (int)cudaMemcpyFromSymbol(out, vm::st::g_prof, sizeof(long long) * n);
}
#endif
