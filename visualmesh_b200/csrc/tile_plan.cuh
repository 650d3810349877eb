// The tile plan of a chunk of frames for the staged graph-convolution layers (conv_staged.cuh).
//
// The rows of a frame are cut into super-tiles of ST consecutive rows. For every super-tile the plan lists the rows
// outside it that its rows have as neighbours (its halo, at most HALO rows - mesh nodes are stored in the order of the
// reference's BSP, cpp/visualmesh/mesh.hpp:450-466, which is spatially compact, so a 256-row super-tile has ~95 of
// them), and for every row its neighbours as 16-bit positions inside "super-tile rows, then halo slots". A neighbour
// whose halo slot did not fit is marked NBL_GLOBAL and fetched from global memory by the layer kernels.
// The neighbourhood does not change between layers, so the plan is made once per chunk: by the neighbour-remap kernel
// itself (kernels.cuh) on the hot path, by k_tile_plan for a caller-supplied neighbourhood.
#pragma once

#include <cstdint>

namespace vm {
namespace st {

    constexpr int ST               = 256;     // rows of a super-tile = threads of the block that plans it
    constexpr int HALO             = 192;     // halo slots of a super-tile
    constexpr int HASH_SIZE        = 1024;    // open-addressing table of a super-tile's outside rows
    constexpr uint32_t NBL_GLOBAL  = 0xFFFFu; // neighbour position: not staged, fetch from global memory
    constexpr int NBL_STRIDE       = 8;       // 16-bit positions per row (N <= 8), one 16-byte load

    // What the plan leaves behind for the layers of a chunk.
    struct Plan {
        const uint16_t* nbl;        // [chunk rows][NBL_STRIDE]: neighbour j of a row as a position in its super-tile's window
        const int32_t* halo_rows;   // [super-tiles][HALO]: chunk-local feature row of every halo slot
        const int32_t* halo_count;  // [super-tiles]
    };
    struct PlanOut {
        uint16_t* nbl;
        int32_t* halo_rows;
        int32_t* halo_count;
    };

    __device__ __forceinline__ uint32_t hash_row(int32_t v) {
        return (static_cast<uint32_t>(v) * 2654435761u) >> 22;  // top 10 bits: [0, HASH_SIZE)
    }

    // Called by all ST threads of a block for super-tile blockIdx.x of frame f (the f-th of the launch, frames f0 ...):
    // thread tid holds the frame-local neighbour indices idx[0..N) of row t0 + tid (valid: the row exists).
    template <int N>
    __device__ __forceinline__ void plan_super_tile(const int (&idx)[N], bool valid, int t0, int f, const int32_t* offsets, int f0, const PlanOut& out) {
        static_assert(HASH_SIZE % ST == 0 && HASH_SIZE == 1024, "table entries are dealt evenly to the threads, the hash has 10 bits");
        static_assert(N <= NBL_STRIDE, "one 16-byte row of positions");
        constexpr int PER = HASH_SIZE / ST;
        __shared__ int32_t keys[HASH_SIZE];
        __shared__ uint16_t slot_of[HASH_SIZE];
        __shared__ int32_t warp_sums[ST / 32];
        __shared__ int32_t tiles_before;
        const int tid = threadIdx.x;
        if (tid == 0) tiles_before = 0;
        for (int i = tid; i < HASH_SIZE; i += ST) keys[i] = -1;
        __syncthreads();
        // super-tiles of the frames before this one (at most 64 frames per launch)
        if (tid < f) {
            const int r = offsets[f0 + tid + 1] - offsets[f0 + tid] + 1;
            atomicAdd(&tiles_before, (r + ST - 1) / ST);
        }
        const int local_base = offsets[f0 + f] - offsets[f0] + f;
        // ---- 1: the set of outside rows ----
        if (valid) {
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const int i = idx[j];
                if (i >= t0 && i < t0 + ST) continue;
                uint32_t h = hash_row(i);
                for (int probe = 0; probe < HASH_SIZE; ++probe) {
                    const int prev = atomicCAS(&keys[h], -1, i);
                    if (prev == -1 || prev == i) break;
                    h = (h + 1) & (HASH_SIZE - 1);
                }
                // a full table leaves the row out: it is then fetched from global memory by the layer kernels
            }
        }
        __syncthreads();
        // ---- 2: halo slots in table order ----
        int mine = 0;
#pragma unroll
        for (int q = 0; q < PER; ++q) mine += keys[tid * PER + q] >= 0 ? 1 : 0;
        const int lane = tid & 31, warp = tid >> 5;
        int incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_sums[w];
        int total = 0;
        for (int w = 0; w < ST / 32; ++w) total += warp_sums[w];
        const int st_id = tiles_before + blockIdx.x;
        int slot        = before + incl - mine;
#pragma unroll
        for (int q = 0; q < PER; ++q) {
            const int e = tid * PER + q;
            if (keys[e] >= 0) {
                slot_of[e] = static_cast<uint16_t>(slot < HALO ? slot : NBL_GLOBAL);
                if (slot < HALO) out.halo_rows[static_cast<size_t>(st_id) * HALO + slot] = local_base + keys[e];
                ++slot;
            }
        }
        if (tid == 0) out.halo_count[st_id] = total < HALO ? total : HALO;
        __syncthreads();
        // ---- 3: every neighbour as a position in the window ----
        if (valid) {
            uint32_t v[NBL_STRIDE];
#pragma unroll
            for (int j = 0; j < NBL_STRIDE; ++j) v[j] = 0;
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const int i = idx[j];
                if (i >= t0 && i < t0 + ST) {
                    v[j] = static_cast<uint32_t>(i - t0);
                    continue;
                }
                uint32_t h   = hash_row(i);
                uint32_t pos = NBL_GLOBAL;
                for (int probe = 0; probe < HASH_SIZE; ++probe) {
                    const int k = keys[h];
                    if (k == i) {
                        const uint32_t s = slot_of[h];
                        pos              = s == NBL_GLOBAL ? NBL_GLOBAL : static_cast<uint32_t>(ST) + s;
                        break;
                    }
                    if (k == -1) break;
                    h = (h + 1) & (HASH_SIZE - 1);
                }
                v[j] = pos;
            }
            uint4 packed;
            packed.x = v[0] | (v[1] << 16);
            packed.y = v[2] | (v[3] << 16);
            packed.z = v[4] | (v[5] << 16);
            packed.w = v[6] | (v[7] << 16);
            reinterpret_cast<uint4*>(out.nbl)[static_cast<size_t>(local_base + t0 + tid)] = packed;
        }
    }

}  // namespace st
}  // namespace vm
