// Arguments of one graph-convolution layer launch, shared by every layer kernel and by the host code that fills them.
#pragma once

#include <cstdint>

namespace vm {

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

constexpr int CONV_THREADS = 128;

}  // namespace vm
