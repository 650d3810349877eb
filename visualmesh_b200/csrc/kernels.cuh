// Kernels of the Visual Mesh hot path for sm_100a.
//
// A chunk is a run of frames of one batch processed by one set of launches. Grids are two-dimensional:
// blockIdx.y is the frame within the chunk, blockIdx.x walks that frame's candidates (or rows). Blocks past the end of
// their frame exit at once, so no launch needs a count that only the device knows and the host never waits in the
// middle of a chunk. No kernel waits on another block: compaction is count -> scan -> scatter in three launches.
//
// Row spaces: points of frame f start at offsets[f] in the batch-wide result arrays; rows (points + one off-screen
// row per frame) start at offsets[f] + f. Feature buffers are chunk-local: rows start at
// offsets[f] - offsets[f0] + (f - f0) where f0 is the chunk's first frame.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_math.cuh"
#include "tile_plan.cuh"

namespace vm {

constexpr int SELECT_THREADS = 256;
constexpr int ROW_THREADS    = 256;
constexpr int SCATTER_UNITS  = 4;    // runs of SELECT_THREADS candidates per block of k_scatter
constexpr int SAMPLE_ROWS    = 2;    // points per thread of k_sample

enum : uint8_t { BSP_DESCEND = 0, BSP_INSIDE = 1, BSP_OUTSIDE = 2 };

// ---- device-side Mesh::lookup, part 1: classify every BSP element ----------------------------------------------
// cpp/visualmesh/mesh.hpp:521-539 (field-of-view cone test) and :362-406 (check_on_screen), evaluated for every
// element independently of its ancestors; the descent in k_select applies them top-down.
__global__ void __launch_bounds__(SELECT_THREADS) k_bsp_state(const FrameParams* __restrict__ frames, uint8_t* __restrict__ state) {
    const FrameParams& p = frames[blockIdx.y];
    const int e          = blockIdx.x * SELECT_THREADS + threadIdx.x;
    if (p.ranges != nullptr || e >= p.n_bsp) return;
    const float4 a  = __ldg(p.bsp_cones_a + e);
    const float sn  = __ldg(p.bsp_cones_s + e);
    const float cs  = a.w;
    const float delta = dot3(p.Rco[0], p.Rco[1], p.Rco[2], a.x, a.y, a.z);
    bool outside = delta < __fsub_rn(__fmul_rn(p.cos_fov, cs), __fmul_rn(p.sin_fov, sn));
    bool inside  = delta > __fadd_rn(__fmul_rn(p.cos_fov, cs), __fmul_rn(p.sin_fov, sn));
    if (!outside && inside) {
        float cx, cy, cz;
        rotate(p, a.x, a.y, a.z, cx, cy, cz);
        const bool axis_on_screen = on_screen_loose(project(cx, cy, cz, p), p);
        float angles[4];
        bool contains = false;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            angles[i] = dot3(a.x, a.y, a.z, p.edges[i][0], p.edges[i][1], p.edges[i][2]);
            contains |= angles[i] > __fadd_rn(__fmul_rn(p.edges[i][3], cs), __fmul_rn(p.edges[i][4], sn));
        }
        if (!axis_on_screen && contains) {
            inside  = false;
            outside = true;
        }
        else {
            bool intersects = true;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                intersects &= angles[i] < __fsub_rn(__fmul_rn(p.edges[i][3], cs), __fmul_rn(p.edges[i][4], sn));
            }
            inside  = axis_on_screen && intersects;
            outside = false;
        }
    }
    state[p.bsp_off + e] = inside ? BSP_INSIDE : (outside ? BSP_OUTSIDE : BSP_DESCEND);
}

// ---- select + project + count -----------------------------------------------------------------------------------
// One thread per candidate. With host ranges (cpp/visualmesh/engine/cpu/engine.hpp:110-122) a candidate is the c-th
// node of the concatenated ranges. With device lookup every node is a candidate and the thread first walks the BSP
// from the root: an INSIDE ancestor selects the node, an OUTSIDE one drops it, a leaf tests the node itself
// (cpp/visualmesh/mesh.hpp:559-583: inside the field of view and loosely on screen). Selected nodes then take the
// engine's strict on-screen test. Writes the pixel and node id (-1 = dropped) per candidate and the number kept per
// block.
__global__ void __launch_bounds__(SELECT_THREADS) k_select(const FrameParams* __restrict__ frames,
                                                           const uint8_t* __restrict__ state,
                                                           float2* __restrict__ cand_px,
                                                           int32_t* __restrict__ cand_node,
                                                           int32_t* __restrict__ block_counts,
                                                           int32_t* __restrict__ abort_flag) {
    const FrameParams& p = frames[blockIdx.y];
    const int c          = blockIdx.x * SELECT_THREADS + threadIdx.x;
    bool keep            = false;
    if (c < p.n_candidates) {
        int g          = c;
        bool selected  = true;
        bool test_fov  = false;
        if (p.ranges != nullptr) {
            // binary search for the last range whose start is <= c
            int lo = 0, hi = p.n_ranges - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (__ldg(p.range_starts + mid) <= c) { lo = mid; }
                else {
                    hi = mid - 1;
                }
            }
            g = __ldg(p.ranges + lo).x + (c - __ldg(p.range_starts + lo));
        }
        else {
            int e = 0;
            int steps = 0;
            for (; steps < 128; ++steps) {
                // both loads of a step are issued together: the walk is a chain of dependent loads, and the element's
                // topology is in bounds whatever its state turns out to be
                const uint8_t s = state[p.bsp_off + e];
                const int4 t    = __ldg(p.bsp_topology + e);
                if (s == BSP_INSIDE) break;
                if (s == BSP_OUTSIDE) {
                    selected = false;
                    break;
                }
                if (t.x < 0) {
                    test_fov = true;
                    break;
                }
                e = (g < t.z) ? t.x : t.y;
            }
            if (steps == 128) {
                // a tree deeper than any the builder makes: give up on this node and report it
                atomicExch(abort_flag, 1);
                selected = false;
            }
        }
        float2 px = make_float2(0.0f, 0.0f);
        if (selected) {
            const float4 r = __ldg(p.rays + g);
            float cx, cy, cz;
            rotate(p, r.x, r.y, r.z, cx, cy, cz);
            px   = project(cx, cy, cz, p);
            keep = on_screen_strict(px, p) && (!test_fov || cx > p.cos_fov);
        }
        if (keep) cand_px[p.cand_off + c] = px;  // the scatter reads the pixels of kept candidates only
        cand_node[p.cand_off + c] = keep ? g : -1;
    }
    const int n = __syncthreads_count(keep);
    if (threadIdx.x == 0) block_counts[blockIdx.y * gridDim.x + blockIdx.x] = n;
}

// ---- scan of the per-block counts --------------------------------------------------------------------------------
// One block. Turns block_counts into exclusive block offsets relative to the chunk's first point and extends the
// batch-wide offsets array: offsets[f0 + y + 1] for every frame y of the chunk, continuing from offsets[f0].
// Each warp owns a contiguous run of the counts and walks it 32 at a time, so every load and store is one coalesced
// line; the first pass sums the runs, the second redoes each run as a shuffle scan carried from line to line.
__global__ void __launch_bounds__(1024) k_scan(int32_t* __restrict__ block_counts,
                                               int32_t n_blocks,
                                               int32_t blocks_per_frame,
                                               int32_t n_frames,
                                               int32_t* __restrict__ offsets,
                                               int32_t f0) {
    __shared__ int32_t warp_base[33];
    const int t     = threadIdx.x;
    const int lane  = t & 31;
    const int warp  = t >> 5;
    const int lines = (n_blocks + 1023) / 1024;  // 32-count lines per warp
    const int begin = min(warp * lines * 32, n_blocks);
    const int end   = min(begin + lines * 32, n_blocks);
    int sum         = 0;
#pragma unroll 4
    for (int i = begin + lane; i < end; i += 32) sum += block_counts[i];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane == 0) warp_base[warp + 1] = sum;
    __syncthreads();
    if (warp == 0) {
        // exclusive scan of the 32 run totals; warp_base[32] keeps the grand total
        int v = warp_base[lane + 1];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += u;
        }
        warp_base[lane + 1] = v;
        if (lane == 0) warp_base[0] = 0;
    }
    __syncthreads();
    const int total = warp_base[32];
    int run         = warp_base[warp];
    for (int i0 = begin; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const int c = (i < end) ? block_counts[i] : 0;
        int v       = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, v, d);
            if (lane >= d) v += u;
        }
        if (i < end) block_counts[i] = run + v - c;
        run += __shfl_sync(0xffffffffu, v, 31);
    }
    __syncthreads();
    // frame y starts at block y * blocks_per_frame
    const int base = offsets[f0];
    for (int y = t; y < n_frames; y += 1024) {
        const int first = (y + 1) * blocks_per_frame;
        const int upto  = (first < n_blocks) ? block_counts[first] : total;
        offsets[f0 + y + 1] = base + upto;
    }
}

// ---- scatter: stable compaction ----------------------------------------------------------------------------------
// Kept candidates, in candidate order, become the frame's points: global_indices ascending
// (cpp/visualmesh/engine/cpu/engine.hpp:110-120). Also fills the node -> local index table that k_remap reads in
// place of the reference's r_lookup (engine.hpp:128-131); with device lookup every entry is written, with host
// ranges the table was cleared to -1 beforehand.
template <int UNITS>
__global__ void __launch_bounds__(SELECT_THREADS) k_scatter(const FrameParams* __restrict__ frames,
                                                            const float2* __restrict__ cand_px,
                                                            const int32_t* __restrict__ cand_node,
                                                            const int32_t* __restrict__ block_offsets,
                                                            int32_t blocks_per_frame,
                                                            const int32_t* __restrict__ offsets,
                                                            int32_t f0,
                                                            float2* __restrict__ out_px,
                                                            int32_t* __restrict__ out_gi,
                                                            int32_t* __restrict__ node_rank) {
    // a block compacts UNITS runs of SELECT_THREADS candidates (the unit k_select counted and k_scan scanned); their
    // loads are issued together
    __shared__ int32_t warp_counts[UNITS][SELECT_THREADS / 32];
    const FrameParams& p = frames[blockIdx.y];
    const int lane       = threadIdx.x & 31;
    const int warp       = threadIdx.x >> 5;
    const int frame      = f0 + blockIdx.y;
    int c[UNITS], g[UNITS];
    unsigned mask[UNITS];
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        c[u] = (blockIdx.x * UNITS + u) * SELECT_THREADS + threadIdx.x;
        g[u] = (c[u] < p.n_candidates) ? cand_node[p.cand_off + c[u]] : -1;
    }
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        mask[u] = __ballot_sync(0xffffffffu, g[u] >= 0);
        if (lane == 0) warp_counts[u][warp] = __popc(mask[u]);
    }
    __syncthreads();
    const int chunk_base = offsets[f0];
    const int frame_base = offsets[frame];
#pragma unroll
    for (int u = 0; u < UNITS; ++u) {
        const int unit = blockIdx.x * UNITS + u;
        if (unit >= blocks_per_frame) break;
        int before = 0;
        for (int w = 0; w < warp; ++w) before += warp_counts[u][w];
        const int in_chunk = block_offsets[blockIdx.y * blocks_per_frame + unit] + before + __popc(mask[u] & ((1u << lane) - 1u));
        if (g[u] >= 0) {
            const int o  = chunk_base + in_chunk;
            out_px[o]    = cand_px[p.cand_off + c[u]];
            out_gi[o]    = g[u];
            node_rank[p.node_off + g[u]] = o - frame_base;
        }
        else if (c[u] < p.n_candidates && p.ranges == nullptr) {
            node_rank[p.node_off + c[u]] = -1;
        }
    }
}

// ---- neighbour remap ---------------------------------------------------------------------------------------------
// cpp/visualmesh/engine/cpu/engine.hpp:134-143: neighbours into the frame's compact index space; a neighbour that is
// off the mesh or not on screen becomes n (the off-screen row); row n is all n.
// With PLAN the block - which owns 256 consecutive rows, exactly one super-tile of the staged layer kernels - also makes
// that super-tile's part of the tile plan (tile_plan.cuh) from the indices it has just computed.
template <int N, bool PLAN>
__global__ void __launch_bounds__(ROW_THREADS) k_remap(const FrameParams* __restrict__ frames,
                                                       const int32_t* __restrict__ offsets,
                                                       int32_t f0,
                                                       const int32_t* __restrict__ out_gi,
                                                       const int32_t* __restrict__ node_rank,
                                                       int32_t* __restrict__ out_nb,
                                                       const st::PlanOut plan) {
    static_assert(!PLAN || ROW_THREADS == st::ST, "a block of the remap is a super-tile of the plan");
    const FrameParams& p = frames[blockIdx.y];
    const int frame      = f0 + blockIdx.y;
    const int start      = offsets[frame];
    const int n          = offsets[frame + 1] - start;
    const int t0         = blockIdx.x * ROW_THREADS;
    if (t0 > n) return;  // the whole block is past the frame's n + 1 rows
    const int i      = t0 + threadIdx.x;
    const bool valid = i <= n;
    int v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = n;
    if (valid) {
        int32_t* row = out_nb + static_cast<size_t>(start + frame + i) * N;
        if (i < n) {
            const int g         = out_gi[start + i];
            const int32_t* nbrs = p.neighbours + static_cast<size_t>(g) * N;
#pragma unroll
            for (int j = 0; j < N; ++j) {
                const int t = __ldg(nbrs + j);
                if (t >= 0 && t < p.n_nodes) {
                    const int k = node_rank[p.node_off + t];
                    v[j]        = (k < 0) ? n : k;
                }
            }
        }
#pragma unroll
        for (int j = 0; j < N; ++j) row[j] = v[j];
    }
    if (PLAN) st::plan_super_tile<N>(v, valid, t0, static_cast<int>(blockIdx.y), offsets, f0, plan);
}

// ---- image sampling ----------------------------------------------------------------------------------------------
// cpp/visualmesh/engine/cpu/engine.hpp:198-206: bilinear sample at every point, four -1 for the off-screen row.
// PACKED4: every frame of the launch is RGBA or BGRA. The general sampler carries the 5x5 Bayer patch in its register
// count (66), which holds it to three blocks per SM although it waits on memory; the packed one fills the SM.
template <bool PACKED4>
__global__ void __launch_bounds__(ROW_THREADS) k_sample(const FrameParams* __restrict__ frames,
                                                        const int32_t* __restrict__ offsets,
                                                        int32_t f0,
                                                        const float2* __restrict__ out_px,
                                                        float4* __restrict__ features) {
    // a thread samples SAMPLE_ROWS points, ROW_THREADS apart: the pixel coordinates of all of them are loaded before
    // the first texel, so that many independent chains of two dependent loads are in flight per thread
    const FrameParams& p = frames[blockIdx.y];
    const int frame      = f0 + blockIdx.y;
    const int start      = offsets[frame];
    const int n          = offsets[frame + 1] - start;
    const int first      = blockIdx.x * (ROW_THREADS * SAMPLE_ROWS) + threadIdx.x;
    if (first > n) return;
    const int row0 = start - offsets[f0] + blockIdx.y;
    float2 px[SAMPLE_ROWS];
#pragma unroll
    for (int q = 0; q < SAMPLE_ROWS; ++q) {
        const int i = first + q * ROW_THREADS;
        px[q]       = (i < n) ? out_px[start + i] : make_float2(0.0f, 0.0f);
    }
#pragma unroll
    for (int q = 0; q < SAMPLE_ROWS; ++q) {
        const int i = first + q * ROW_THREADS;
        if (i > n) break;
        float4 v = make_float4(-1.0f, -1.0f, -1.0f, -1.0f);
        if (i < n) {
            if (PACKED4) { v = interpolate_packed4(px[q], p.image, p.dims[0], p.dims[1], p.format == fcc('B', 'G', 'R', 'A')); }
            else {
                v = interpolate(px[q], p.image, p.dims[0], p.dims[1], format_class(p.format));
            }
        }
        features[row0 + i] = v;
    }
}

// The same sampler on a flat list of pixel coordinates (stand-alone stage for unit parity tests).
__global__ void __launch_bounds__(ROW_THREADS) k_sample_flat(const float2* __restrict__ px,
                                                             int32_t n,
                                                             const uint8_t* __restrict__ image,
                                                             int32_t W,
                                                             int32_t H,
                                                             int32_t cls,
                                                             float4* __restrict__ out) {
    const int i = blockIdx.x * ROW_THREADS + threadIdx.x;
    if (i < n) out[i] = interpolate(px[i], image, W, H, cls);
}

}  // namespace vm
