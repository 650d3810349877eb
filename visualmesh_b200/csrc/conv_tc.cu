// Launchers of the tensor-core graph-convolution layer kernels that gather with global loads (conv_tc.cuh).
#include <cstdlib>

#include "conv_dispatch.hpp"
#include "conv_tc.cuh"

namespace vm {

static_assert(TC_MAX_FRAMES == tc::MAX_FRAMES && ABORT_TC_TIMEOUT == tc::ABORT_TC_TIMEOUT && ABORT_TC_RANGE == tc::ABORT_TC_RANGE
                && TC_DEFAULT_WAIT_LIMIT == tc::WAIT_LIMIT,
              "the constants the engine sees are the kernels' own");

template <int CIN, int NP, int NSLOTS, bool HALF>
static void launch_conv_tc_t(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s) {
    constexpr int STAGES = CIN >= 32 ? 2 : 3;  // 32-channel stages are 16 KB: two of them leave room for a third CTA per SM
    const size_t smem    = tc::smem_bytes<CIN, NP, STAGES, HALF>(NSLOTS);
    static LaunchPlans plans;
    const LaunchPlan& plan = plans.get([smem](int dev) {
        LaunchPlan p;
        VM_CUDA(cudaFuncSetAttribute(tc::k_graph_conv_tc<CIN, NP, STAGES, NSLOTS, HALF>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        VM_CUDA(cudaDeviceGetAttribute(&p.n_sms, cudaDevAttrMultiProcessorCount, dev));
        // resident CTAs per SM: shared memory (about 220 KB usable, some per CTA reserved) and tensor memory (512 columns)
        const int by_smem = static_cast<int>((220 * 1024) / (smem + 2048));
        const int by_tmem = 512 / (4 * NP);
        cudaFuncAttributes attr;
        VM_CUDA(cudaFuncGetAttributes(&attr, tc::k_graph_conv_tc<CIN, NP, STAGES, NSLOTS, HALF>));
        const int regs_per_warp = (((attr.numRegs + 7) / 8 * 8) * 32 + 511) / 512 * 512;
        const int by_regs       = 65536 / std::max(1, regs_per_warp * (tc::CTA_THREADS / 32));
        p.ctas_per_sm           = std::max(1, std::min(std::min(by_smem, by_tmem), std::min(by_regs, 8)));
        return p;
    });
    tc::Args t{};
    t.w_cat      = L.d_tc_cat;
    t.bias       = L.d_tc_bias;
    t.n_frames   = n_frames;
    t.cout       = L.cout;
    t.abort_flag = abort_flag;
    t.wait_limit = wait_limit;
    const int tiles_upper = n_frames * ((max_rows + tc::TILE_ROWS - 1) / tc::TILE_ROWS);
    const int grid        = std::max(1, std::min(tiles_upper, plan.n_sms * plan.ctas_per_sm));
    tc::k_graph_conv_tc<CIN, NP, STAGES, NSLOTS, HALF><<<grid, tc::CTA_THREADS, smem, s>>>(a, t);
}

template <int CIN, int NP, int NSLOTS>
static void launch_conv_tc_tmem_t(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s) {
    const size_t smem = tc::smem_bytes_tmem<CIN, NP>(NSLOTS);
    static LaunchPlans plans;
    const LaunchPlan& plan = plans.get([smem](int dev) {
        LaunchPlan p;
        if (smem > 48 * 1024) {
            VM_CUDA(cudaFuncSetAttribute(tc::k_graph_conv_tc_tmem<CIN, NP, NSLOTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        }
        VM_CUDA(cudaDeviceGetAttribute(&p.n_sms, cudaDevAttrMultiProcessorCount, dev));
        const int by_smem = static_cast<int>((220 * 1024) / (smem + 2048));
        const int by_tmem = 512 / tc::tmem_columns<NP>();
        cudaFuncAttributes attr;
        VM_CUDA(cudaFuncGetAttributes(&attr, tc::k_graph_conv_tc_tmem<CIN, NP, NSLOTS>));
        // registers: 8 per thread at a time, 512 per warp at a time, 64 K per SM
        const int regs_per_warp = (((attr.numRegs + 7) / 8 * 8) * 32 + 511) / 512 * 512;
        const int by_regs       = 65536 / std::max(1, regs_per_warp * (tc::CTA_THREADS / 32));
        p.ctas_per_sm           = std::max(1, std::min(std::min(by_smem, by_tmem), std::min(by_regs, 8)));
        if (const char* v = std::getenv("VMCUDA_TC_CTAS")) p.ctas_per_sm = std::max(1, std::min(p.ctas_per_sm, std::atoi(v)));
        return p;
    });
    tc::Args t{};
    t.w_cat      = L.d_tc_cat;
    t.bias       = L.d_tc_bias;
    t.n_frames   = n_frames;
    t.cout       = L.cout;
    t.abort_flag = abort_flag;
    t.wait_limit = wait_limit;
    const int tiles_upper = n_frames * ((max_rows + tc::TILE_ROWS - 1) / tc::TILE_ROWS);
    const int grid        = std::max(1, std::min(tiles_upper, plan.n_sms * plan.ctas_per_sm));
    tc::k_graph_conv_tc_tmem<CIN, NP, NSLOTS><<<grid, tc::CTA_THREADS, smem, s>>>(a, t);
}

// The tensor-core kernel fed from the split feature layout exists for these shapes.
bool has_tc_split_kernel(const DenseLayer& L) {
    return L.tc_np != 0 && L.tc_half && (L.cin == 16 || L.cin == 32) && (L.n_slots == 5 || L.n_slots == 7 || L.n_slots == 9);
}

bool launch_conv_tc_split(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s) {
#define VM_TCS(CI, NPAD, NS)                                                              \
    if (L.cin == CI && L.tc_np == NPAD && L.n_slots == NS) {                               \
        launch_conv_tc_tmem_t<CI, NPAD, NS>(L, a, n_frames, max_rows, abort_flag, wait_limit, s);       \
        return true;                                                                       \
    }
    VM_TCS(16, 16, 5) VM_TCS(16, 16, 7) VM_TCS(16, 16, 9) VM_TCS(16, 32, 5) VM_TCS(16, 32, 7) VM_TCS(16, 32, 9)
    VM_TCS(32, 16, 5) VM_TCS(32, 16, 7) VM_TCS(32, 16, 9) VM_TCS(32, 32, 5) VM_TCS(32, 32, 7) VM_TCS(32, 32, 9)
#undef VM_TCS
    return false;
}

bool launch_conv_tc_gather(const DenseLayer& L, const ConvArgs& a, int n_frames, int max_rows, int32_t* abort_flag, uint32_t wait_limit, cudaStream_t s) {
    if (L.tc_np == 0 || n_frames > tc::MAX_FRAMES) return false;
#define VM_TC(CI, NPAD, NS, HF)                                                      \
    if (L.cin == CI && L.tc_np == NPAD && L.n_slots == NS && L.tc_half == HF) {        \
        launch_conv_tc_t<CI, NPAD, NS, HF>(L, a, n_frames, max_rows, abort_flag, wait_limit, s);   \
        return true;                                                                  \
    }
    VM_TC(8, 16, 5, false) VM_TC(8, 16, 7, false) VM_TC(8, 16, 9, false)
    VM_TC(16, 16, 5, true) VM_TC(16, 16, 7, true) VM_TC(16, 16, 9, true)
    VM_TC(16, 32, 7, true) VM_TC(16, 32, 9, true)
    VM_TC(32, 16, 7, true) VM_TC(32, 16, 9, true)
    VM_TC(32, 32, 7, true) VM_TC(32, 32, 9, true)
#undef VM_TC
    return false;
}

// The tensor-core kernel that gathers fp32 rows itself exists for these shapes (the VM_TC list of launch_conv_tc).
bool has_tc_gather_kernel(const DenseLayer& L) {
    if (L.tc_np == 0) return false;
    const int ns = L.n_slots;
    if (!L.tc_half) return L.cin == 8 && L.tc_np == 16 && (ns == 5 || ns == 7 || ns == 9);
    if (L.cin == 16 && L.tc_np == 16) return ns == 5 || ns == 7 || ns == 9;
    if ((L.cin == 16 && L.tc_np == 32) || (L.cin == 32 && (L.tc_np == 16 || L.tc_np == 32))) return ns == 7 || ns == 9;
    return false;
}


}  // namespace vm
