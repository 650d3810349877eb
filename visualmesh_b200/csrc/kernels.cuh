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

namespace vm {

constexpr int SELECT_THREADS = 256;
constexpr int ROW_THREADS    = 256;
constexpr int CONV_THREADS   = 128;

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
                const uint8_t s = state[p.bsp_off + e];
                if (s == BSP_INSIDE) break;
                if (s == BSP_OUTSIDE) {
                    selected = false;
                    break;
                }
                const int4 t = __ldg(p.bsp_topology + e);
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
        cand_px[p.cand_off + c]   = px;
        cand_node[p.cand_off + c] = keep ? g : -1;
    }
    const int n = __syncthreads_count(keep);
    if (threadIdx.x == 0) block_counts[blockIdx.y * gridDim.x + blockIdx.x] = n;
}

// ---- scan of the per-block counts --------------------------------------------------------------------------------
// One block. Turns block_counts into exclusive block offsets relative to the chunk's first point and extends the
// batch-wide offsets array: offsets[f0 + y + 1] for every frame y of the chunk, continuing from offsets[f0].
__global__ void __launch_bounds__(1024) k_scan(int32_t* __restrict__ block_counts,
                                               int32_t n_blocks,
                                               int32_t blocks_per_frame,
                                               int32_t n_frames,
                                               int32_t* __restrict__ offsets,
                                               int32_t f0) {
    __shared__ int32_t partial[1024];
    const int t     = threadIdx.x;
    const int per   = (n_blocks + 1023) / 1024;
    const int begin = min(t * per, n_blocks);
    const int end   = min(begin + per, n_blocks);
    int sum         = 0;
    for (int i = begin; i < end; ++i) sum += block_counts[i];
    partial[t] = sum;
    __syncthreads();
    // Hillis-Steele inclusive scan over the 1024 partials
    for (int d = 1; d < 1024; d <<= 1) {
        const int v = (t >= d) ? partial[t - d] : 0;
        __syncthreads();
        partial[t] += v;
        __syncthreads();
    }
    int run = partial[t] - sum;
    for (int i = begin; i < end; ++i) {
        const int v     = block_counts[i];
        block_counts[i] = run;
        run += v;
    }
    __syncthreads();
    // frame y starts at block y * blocks_per_frame
    const int base = offsets[f0];
    for (int y = t; y < n_frames; y += 1024) {
        const int first = (y + 1) * blocks_per_frame;
        const int upto  = (first < n_blocks) ? block_counts[first] : partial[1023];
        offsets[f0 + y + 1] = base + upto;
    }
}

// ---- scatter: stable compaction ----------------------------------------------------------------------------------
// Kept candidates, in candidate order, become the frame's points: global_indices ascending
// (cpp/visualmesh/engine/cpu/engine.hpp:110-120). Also fills the node -> local index table that k_remap reads in
// place of the reference's r_lookup (engine.hpp:128-131); with device lookup every entry is written, with host
// ranges the table was cleared to -1 beforehand.
__global__ void __launch_bounds__(SELECT_THREADS) k_scatter(const FrameParams* __restrict__ frames,
                                                            const float2* __restrict__ cand_px,
                                                            const int32_t* __restrict__ cand_node,
                                                            const int32_t* __restrict__ block_offsets,
                                                            const int32_t* __restrict__ offsets,
                                                            int32_t f0,
                                                            float2* __restrict__ out_px,
                                                            int32_t* __restrict__ out_gi,
                                                            int32_t* __restrict__ node_rank) {
    __shared__ int32_t warp_counts[SELECT_THREADS / 32];
    const FrameParams& p = frames[blockIdx.y];
    const int c          = blockIdx.x * SELECT_THREADS + threadIdx.x;
    int g                = -1;
    if (c < p.n_candidates) g = cand_node[p.cand_off + c];
    const bool keep      = g >= 0;
    const unsigned mask  = __ballot_sync(0xffffffffu, keep);
    const int lane       = threadIdx.x & 31;
    const int warp       = threadIdx.x >> 5;
    if (lane == 0) warp_counts[warp] = __popc(mask);
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_counts[w];
    const int in_chunk = block_offsets[blockIdx.y * gridDim.x + blockIdx.x] + before + __popc(mask & ((1u << lane) - 1u));
    const int frame    = f0 + blockIdx.y;
    if (keep) {
        const int o  = offsets[f0] + in_chunk;
        out_px[o]    = cand_px[p.cand_off + c];
        out_gi[o]    = g;
        node_rank[p.node_off + g] = o - offsets[frame];
    }
    else if (c < p.n_candidates && p.ranges == nullptr) {
        node_rank[p.node_off + c] = -1;
    }
}

// ---- neighbour remap ---------------------------------------------------------------------------------------------
// cpp/visualmesh/engine/cpu/engine.hpp:134-143: neighbours into the frame's compact index space; a neighbour that is
// off the mesh or not on screen becomes n (the off-screen row); row n is all n.
template <int N>
__global__ void __launch_bounds__(ROW_THREADS) k_remap(const FrameParams* __restrict__ frames,
                                                       const int32_t* __restrict__ offsets,
                                                       int32_t f0,
                                                       const int32_t* __restrict__ out_gi,
                                                       const int32_t* __restrict__ node_rank,
                                                       int32_t* __restrict__ out_nb) {
    const FrameParams& p = frames[blockIdx.y];
    const int frame      = f0 + blockIdx.y;
    const int start      = offsets[frame];
    const int n          = offsets[frame + 1] - start;
    const int i          = blockIdx.x * ROW_THREADS + threadIdx.x;
    if (i > n) return;
    int32_t* row = out_nb + static_cast<size_t>(start + frame + i) * N;
    if (i == n) {
#pragma unroll
        for (int j = 0; j < N; ++j) row[j] = n;
        return;
    }
    const int g          = out_gi[start + i];
    const int32_t* nbrs  = p.neighbours + static_cast<size_t>(g) * N;
    int v[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
        const int t = __ldg(nbrs + j);
        int r       = n;
        if (t >= 0 && t < p.n_nodes) {
            const int k = node_rank[p.node_off + t];
            r           = (k < 0) ? n : k;
        }
        v[j] = r;
    }
#pragma unroll
    for (int j = 0; j < N; ++j) row[j] = v[j];
}

// ---- image sampling ----------------------------------------------------------------------------------------------
// cpp/visualmesh/engine/cpu/engine.hpp:198-206: bilinear sample at every point, four -1 for the off-screen row.
__global__ void __launch_bounds__(ROW_THREADS) k_sample(const FrameParams* __restrict__ frames,
                                                        const int32_t* __restrict__ offsets,
                                                        int32_t f0,
                                                        const float2* __restrict__ out_px,
                                                        float4* __restrict__ features) {
    const FrameParams& p = frames[blockIdx.y];
    const int frame      = f0 + blockIdx.y;
    const int start      = offsets[frame];
    const int n          = offsets[frame + 1] - start;
    const int i          = blockIdx.x * ROW_THREADS + threadIdx.x;
    if (i > n) return;
    const int local_row = start - offsets[f0] + blockIdx.y + i;
    float4 v            = make_float4(-1.0f, -1.0f, -1.0f, -1.0f);
    if (i < n) { v = interpolate(out_px[start + i], p.image, p.dims[0], p.dims[1], format_class(p.format)); }
    features[local_row] = v;
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

// ---- activations -------------------------------------------------------------------------------------------------
// cpp/visualmesh/engine/cpu/apply_activation.hpp:35-64
__device__ __forceinline__ float selu(float s) {
    const float lambda = 1.0507009873554804934193349852946f;
    const float alpha  = 1.6732632423543772848170429916717f;
    // exp is evaluated on min(s, 0) for every value and the result selected: straight-line code, so the chains of a
    // row's outputs overlap instead of running one branch after the other; the value is the same bit for bit
    const float negative = __fsub_rn(__fmul_rn(alpha, expf(fminf(s, 0.0f))), alpha);
    return __fmul_rn(lambda, (s >= 0.0f) ? s : negative);
}

template <int COUT>
__device__ __forceinline__ void activate(float* v, int act) {
    if (act == VM_SELU) {
#pragma unroll
        for (int j = 0; j < COUT; ++j) v[j] = selu(v[j]);
    }
    else if (act == VM_RELU) {
#pragma unroll
        for (int j = 0; j < COUT; ++j) v[j] = (v[j] < 0.0f) ? 0.0f : v[j];
    }
    else if (act == VM_TANH) {
#pragma unroll
        for (int j = 0; j < COUT; ++j) v[j] = tanhf(v[j]);
    }
    else if (act == VM_SOFTMAX) {
        // exp of each, summed in index order from 0, no max subtraction
        float total = 0.0f;
#pragma unroll
        for (int j = 0; j < COUT; ++j) {
            v[j]  = expf(v[j]);
            total = __fadd_rn(total, v[j]);
        }
#pragma unroll
        for (int j = 0; j < COUT; ++j) v[j] = __fdiv_rn(v[j], total);
    }
}

// ---- fused graph convolution layer -------------------------------------------------------------------------------
// gather (cpp/visualmesh/engine/cpu/engine.hpp:216-235) + dense with the accumulator started at the bias and k
// ascending (engine.hpp:250-256) + activation (engine.hpp:259), one launch per dense layer, nothing materialised.
// Feature layout between layers. A width that is a multiple of 4 is stored "chunk-planar": float4 chunk c of row r at
// float4 index c * stride + r, so that the 32 threads of a warp, which own 32 consecutive rows, read and write
// consecutive 16-byte pieces (one 512-byte request per instruction instead of 32 pieces scattered over 16 cache
// lines). Other widths, and the final classifications, are row-major [row][width].
struct ConvArgs {
    const float* in;        // chunk-local features (planar when CIN % 4 == 0, else row-major)
    float* out;             // chunk-local features, or the batch-wide row-major classifications when out_global
    const int32_t* nb;      // batch-wide neighbourhood rows (frame-local indices)
    const int32_t* offsets; // batch-wide point offsets
    const float* weights;   // [n_slots * CIN][COUTP] row-major, COUTP = COUT rounded up to 4, zero padded
    const float* biases;    // [COUTP]
    int32_t n_slots;        // N + 1 for the first layer of a group, 1 for the layers that follow it
    int32_t n_neighbours;   // N
    int32_t activation;
    int32_t f0;
    int32_t out_global;
    int32_t in_stride;      // rows per planar chunk of `in`
    int32_t out_stride;     // rows per planar chunk of `out`
    int32_t out_planar;     // write `out` chunk-planar (needs COUT % 4 == 0 and !out_global)
    int32_t out_split;      // write `out` as fp16 hi/lo planes for a tensor-core consumer (needs COUT % 8 == 0)
    int32_t* range_flag;    // raised (to 3) when a value is too large for the fp16 split
};

// The "split" feature layout, produced for a layer that runs on the tensor cores. Every fp32 value x is stored as two
// fp16 values, hi = fp16(x) and lo = fp16(x - hi) (x = hi + lo to ~2^-22 relative, absolute error <= 3e-8 for small
// x), in the shape the tensor-core kernel copies straight into shared memory: 16-byte chunks of 8 channels, chunk
// plane p of row r at byte ((p * stride + r) * 16), the C/8 hi planes first, then the C/8 lo planes. Same footprint as
// fp32. Values beyond the fp16 range raise the range flag; the host then recomputes without the tensor-core path.
constexpr int ABORT_RANGE = 3;

template <int COUT>
__device__ __forceinline__ void store_split(float* out, int stride, size_t row, const float* v, int32_t* range_flag) {
    static_assert(COUT % 8 == 0, "split layout needs whole 8-channel chunks");
    constexpr int P = COUT / 8;
    unsigned char* base = reinterpret_cast<unsigned char*>(out);
    bool bad            = false;
#pragma unroll
    for (int p = 0; p < P; ++p) {
        uint32_t h[4], l[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float x0 = v[8 * p + 2 * q], x1 = v[8 * p + 2 * q + 1];
            bad |= fabsf(x0) > 60000.0f || fabsf(x1) > 60000.0f;
            const __half h0 = __float2half_rn(x0);
            const __half h1 = __float2half_rn(x1);
            const __half l0 = __float2half_rn(x0 - __half2float(h0));
            const __half l1 = __float2half_rn(x1 - __half2float(h1));
            h[q] = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
            l[q] = static_cast<uint32_t>(__half_as_ushort(l0)) | (static_cast<uint32_t>(__half_as_ushort(l1)) << 16);
        }
        *reinterpret_cast<uint4*>(base + (static_cast<size_t>(p) * stride + row) * 16)     = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(base + (static_cast<size_t>(P + p) * stride + row) * 16) = make_uint4(l[0], l[1], l[2], l[3]);
    }
    if (bad) atomicCAS(range_flag, 0, ABORT_RANGE);
}

// Each thread owns R rows strided by the block size, so a warp's loads and stores of one row index are contiguous.
// The layer's weights sit in shared memory; every weight read is a 128-bit broadcast shared by the R rows.
template <int CIN, int COUT, int R, int T = CONV_THREADS, int MINB = 1>
__global__ void __launch_bounds__(T, MINB) k_graph_conv(const ConvArgs a) {
    constexpr int COUTP = (COUT + 3) & ~3;
    extern __shared__ float4 smem4[];
    float* w_s = reinterpret_cast<float*>(smem4);

    const int frame_in_chunk = blockIdx.y;
    const int frame          = a.f0 + frame_in_chunk;
    const int start          = a.offsets[frame];
    const int rows           = a.offsets[frame + 1] - start + 1;
    const int first          = blockIdx.x * (T * R);
    if (first >= rows) return;

    const int K = a.n_slots * CIN;
    {
        const float4* src = reinterpret_cast<const float4*>(a.weights);
        const int total4  = (K * COUTP + COUTP) / 4;  // weights then biases, contiguous on the device
        for (int i = threadIdx.x; i < total4; i += T) smem4[i] = __ldg(src + i);
    }
    __syncthreads();
    const float* b_s = w_s + K * COUTP;

    const int local_base  = start - a.offsets[a.f0] + frame_in_chunk;  // chunk-local row of this frame's row 0
    const size_t nb_base  = static_cast<size_t>(start + frame);        // batch-wide row of this frame's row 0

    int row[R];
    float acc[R][COUTP];
#pragma unroll
    for (int q = 0; q < R; ++q) {
        row[q] = min(first + q * T + static_cast<int>(threadIdx.x), rows - 1);
#pragma unroll
        for (int j = 0; j < COUTP; ++j) acc[q][j] = b_s[j];
    }

    const float4* in4 = reinterpret_cast<const float4*>(a.in);
    for (int s = 0; s < a.n_slots; ++s) {
        const float* src[R];
        int src_row[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int idx = (s == 0) ? row[q] : __ldg(a.nb + (nb_base + row[q]) * a.n_neighbours + (s - 1));
            src_row[q]    = local_base + idx;
            src[q]        = a.in + static_cast<size_t>(local_base + idx) * CIN;
        }
        const float* w_slot = w_s + s * CIN * COUTP;
        if (CIN % 4 == 0) {
#pragma unroll
            for (int c4 = 0; c4 < CIN / 4; ++c4) {
                float4 x[R];
#pragma unroll
                for (int q = 0; q < R; ++q) x[q] = in4[static_cast<size_t>(c4) * a.in_stride + src_row[q]];
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const float* w_row = w_slot + (c4 * 4 + kk) * COUTP;
#pragma unroll
                    for (int j4 = 0; j4 < COUTP / 4; ++j4) {
                        const float4 w = *reinterpret_cast<const float4*>(w_row + j4 * 4);
#pragma unroll
                        for (int q = 0; q < R; ++q) {
                            const float xv = kk == 0 ? x[q].x : kk == 1 ? x[q].y : kk == 2 ? x[q].z : x[q].w;
                            acc[q][j4 * 4 + 0] = fmaf(xv, w.x, acc[q][j4 * 4 + 0]);
                            acc[q][j4 * 4 + 1] = fmaf(xv, w.y, acc[q][j4 * 4 + 1]);
                            acc[q][j4 * 4 + 2] = fmaf(xv, w.z, acc[q][j4 * 4 + 2]);
                            acc[q][j4 * 4 + 3] = fmaf(xv, w.w, acc[q][j4 * 4 + 3]);
                        }
                    }
                }
            }
        }
        else {
#pragma unroll
            for (int c = 0; c < CIN; ++c) {
                float x[R];
#pragma unroll
                for (int q = 0; q < R; ++q) x[q] = src[q][c];
                const float* w_row = w_slot + c * COUTP;
#pragma unroll
                for (int j4 = 0; j4 < COUTP / 4; ++j4) {
                    const float4 w = *reinterpret_cast<const float4*>(w_row + j4 * 4);
#pragma unroll
                    for (int q = 0; q < R; ++q) {
                        acc[q][j4 * 4 + 0] = fmaf(x[q], w.x, acc[q][j4 * 4 + 0]);
                        acc[q][j4 * 4 + 1] = fmaf(x[q], w.y, acc[q][j4 * 4 + 1]);
                        acc[q][j4 * 4 + 2] = fmaf(x[q], w.z, acc[q][j4 * 4 + 2]);
                        acc[q][j4 * 4 + 3] = fmaf(x[q], w.w, acc[q][j4 * 4 + 3]);
                    }
                }
            }
        }
    }

    const size_t out_base = a.out_global ? nb_base : static_cast<size_t>(local_base);
#pragma unroll
    for (int q = 0; q < R; ++q) {
        const int i = first + q * T + static_cast<int>(threadIdx.x);
        if (i >= rows) continue;
        activate<COUT>(acc[q], a.activation);
        float* dst = a.out + (out_base + i) * COUT;
        if (COUT % 8 == 0 && a.out_split) { store_split<(COUT % 8 == 0 ? COUT : 8)>(a.out, a.out_stride, out_base + i, acc[q], a.range_flag); }
        else if (COUT % 4 == 0 && a.out_planar) {
            float4* out4 = reinterpret_cast<float4*>(a.out);
#pragma unroll
            for (int j4 = 0; j4 < COUT / 4; ++j4) {
                out4[static_cast<size_t>(j4) * a.out_stride + out_base + i] =
                  make_float4(acc[q][j4 * 4], acc[q][j4 * 4 + 1], acc[q][j4 * 4 + 2], acc[q][j4 * 4 + 3]);
            }
        }
        else if (COUT % 4 == 0) {
#pragma unroll
            for (int j4 = 0; j4 < COUT / 4; ++j4) {
                *reinterpret_cast<float4*>(dst + j4 * 4) =
                  make_float4(acc[q][j4 * 4], acc[q][j4 * 4 + 1], acc[q][j4 * 4 + 2], acc[q][j4 * 4 + 3]);
            }
        }
        else {
#pragma unroll
            for (int j = 0; j < COUT; ++j) dst[j] = acc[q][j];
        }
    }
}

// The same layer with the weights in the kernel's parameter space (constant bank) instead of shared memory: every
// weight read is a constant-cache load that all lanes share and does not touch the L1/shared data path that the
// gather loads. Layers whose weights fit the parameter space (WMAX floats).
template <int WMAX>
struct ConvWeights {
    float w[WMAX];
};

// Packed single-precision FMA of sm_100 (two independent IEEE fused multiply-adds per instruction): halves the
// number of FMA instructions of a kernel that is bound by instruction issue, not by the FMA pipe.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void ffma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// Accumulators live as pairs of adjacent output columns, each weight pair is one 64-bit constant load shared by the R
// rows, each input value is duplicated into a pair once per row and k.
template <int CIN, int COUT, int R, int WMAX, int T = CONV_THREADS, int NS = 0>
__global__ void __launch_bounds__(T) k_graph_conv_cw(const ConvArgs a, const __grid_constant__ ConvWeights<WMAX> wp) {
    static_assert(CIN % 4 == 0, "vector loads of the input rows");
    constexpr int COUTP = (COUT + 3) & ~3;
    const int frame_in_chunk = blockIdx.y;
    const int frame          = a.f0 + frame_in_chunk;
    const int start          = a.offsets[frame];
    const int rows           = a.offsets[frame + 1] - start + 1;
    const int first          = blockIdx.x * (T * R);
    if (first >= rows) return;
    const int n_slots     = NS ? NS : a.n_slots;  // NS != 0: the slot loop is unrolled and its loads scheduled across slots
    const int K           = n_slots * CIN;
    const int local_base  = start - a.offsets[a.f0] + frame_in_chunk;
    const size_t nb_base  = static_cast<size_t>(start + frame);

    int row[R];
    unsigned long long acc[R][COUTP / 2];
#pragma unroll
    for (int q = 0; q < R; ++q) {
        row[q] = min(first + q * T + static_cast<int>(threadIdx.x), rows - 1);
#pragma unroll
        for (int j = 0; j < COUTP / 2; ++j) acc[q][j] = pack2(wp.w[K * COUTP + 2 * j], wp.w[K * COUTP + 2 * j + 1]);
    }
    const float4* in4 = reinterpret_cast<const float4*>(a.in);
#pragma unroll(NS ? NS : 1)
    for (int s = 0; s < n_slots; ++s) {
        int src_row[R];
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int idx = (s == 0) ? row[q] : __ldg(a.nb + (nb_base + row[q]) * a.n_neighbours + (s - 1));
            src_row[q]    = local_base + idx;
        }
        const int w_slot = s * CIN * COUTP;
#pragma unroll
        for (int c4 = 0; c4 < CIN / 4; ++c4) {
            float4 x[R];
#pragma unroll
            for (int q = 0; q < R; ++q) x[q] = in4[static_cast<size_t>(c4) * a.in_stride + src_row[q]];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                unsigned long long xx[R];
#pragma unroll
                for (int q = 0; q < R; ++q) {
                    const float xv = kk == 0 ? x[q].x : kk == 1 ? x[q].y : kk == 2 ? x[q].z : x[q].w;
                    xx[q]          = pack2(xv, xv);
                }
#pragma unroll
                for (int j = 0; j < COUTP / 2; ++j) {
                    const int at               = w_slot + (c4 * 4 + kk) * COUTP + 2 * j;
                    const unsigned long long w = pack2(wp.w[at], wp.w[at + 1]);
#pragma unroll
                    for (int q = 0; q < R; ++q) ffma2(acc[q][j], xx[q], w);
                }
            }
        }
    }
    const size_t out_base = a.out_global ? nb_base : static_cast<size_t>(local_base);
#pragma unroll
    for (int q = 0; q < R; ++q) {
        const int i = first + q * T + static_cast<int>(threadIdx.x);
        if (i >= rows) continue;
        float v[COUTP];
#pragma unroll
        for (int j = 0; j < COUTP / 2; ++j) unpack2(acc[q][j], v[2 * j], v[2 * j + 1]);
        activate<COUT>(v, a.activation);
        float* dst = a.out + (out_base + i) * COUT;
        if (COUT % 8 == 0 && a.out_split) { store_split<(COUT % 8 == 0 ? COUT : 8)>(a.out, a.out_stride, out_base + i, v, a.range_flag); }
        else if (COUT % 4 == 0 && a.out_planar) {
            float4* out4 = reinterpret_cast<float4*>(a.out);
#pragma unroll
            for (int j4 = 0; j4 < COUT / 4; ++j4) {
                out4[static_cast<size_t>(j4) * a.out_stride + out_base + i] = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
            }
        }
        else if (COUT % 4 == 0) {
#pragma unroll
            for (int j4 = 0; j4 < COUT / 4; ++j4) {
                *reinterpret_cast<float4*>(dst + j4 * 4) = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
            }
        }
        else {
#pragma unroll
            for (int j = 0; j < COUT; ++j) dst[j] = v[j];
        }
    }
}

// Any layer shape: one row per thread, outputs in tiles of 8, weights read through the read-only cache.
__global__ void __launch_bounds__(CONV_THREADS) k_graph_conv_generic(const ConvArgs a, int32_t cin, int32_t cout, int32_t coutp) {
    const int frame_in_chunk = blockIdx.y;
    const int frame          = a.f0 + frame_in_chunk;
    const int start          = a.offsets[frame];
    const int rows           = a.offsets[frame + 1] - start + 1;
    const int i              = blockIdx.x * CONV_THREADS + threadIdx.x;
    if (i >= rows) return;
    const int local_base  = start - a.offsets[a.f0] + frame_in_chunk;
    const size_t nb_base  = static_cast<size_t>(start + frame);
    const size_t out_base = a.out_global ? nb_base : static_cast<size_t>(local_base);
    const bool in_planar  = (cin % 4) == 0;
    const bool out_planar = a.out_planar != 0;
    // element c of a row in either layout
    auto in_at = [&](size_t r, int c) -> float {
        return in_planar ? a.in[((static_cast<size_t>(c >> 2) * a.in_stride + r) << 2) + (c & 3)] : a.in[r * cin + c];
    };
    auto out_ptr = [&](int c) -> float* {
        return out_planar ? a.out + ((static_cast<size_t>(c >> 2) * a.out_stride + out_base + i) << 2) + (c & 3)
                          : a.out + (out_base + i) * cout + c;
    };
    const float* biases   = a.weights + static_cast<size_t>(a.n_slots) * cin * coutp;
    for (int j0 = 0; j0 < cout; j0 += 8) {
        float acc[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc[jj] = (j0 + jj < cout) ? __ldg(biases + j0 + jj) : 0.0f;
        for (int s = 0; s < a.n_slots; ++s) {
            const int idx    = (s == 0) ? i : __ldg(a.nb + (nb_base + i) * a.n_neighbours + (s - 1));
            const size_t src = static_cast<size_t>(local_base + idx);
            for (int c = 0; c < cin; ++c) {
                const float x      = in_at(src, c);
                const float* w_row = a.weights + static_cast<size_t>(s * cin + c) * coutp + j0;
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    if (j0 + jj < coutp) acc[jj] = fmaf(x, __ldg(w_row + jj), acc[jj]);
                }
            }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
            if (j0 + jj < cout) *out_ptr(j0 + jj) = acc[jj];
        }
    }
    // activation over the row this thread has just written
    if (a.activation == VM_SELU) {
        for (int j = 0; j < cout; ++j) *out_ptr(j) = selu(*out_ptr(j));
    }
    else if (a.activation == VM_RELU) {
        for (int j = 0; j < cout; ++j) *out_ptr(j) = (*out_ptr(j) < 0.0f) ? 0.0f : *out_ptr(j);
    }
    else if (a.activation == VM_TANH) {
        for (int j = 0; j < cout; ++j) *out_ptr(j) = tanhf(*out_ptr(j));
    }
    else if (a.activation == VM_SOFTMAX) {
        float total = 0.0f;
        for (int j = 0; j < cout; ++j) {
            const float e = expf(*out_ptr(j));
            *out_ptr(j)   = e;
            total         = __fadd_rn(total, e);
        }
        for (int j = 0; j < cout; ++j) *out_ptr(j) = __fdiv_rn(*out_ptr(j), total);
    }
}

}  // namespace vm
