// Device code shared by the graph-convolution layer kernels: activations and the split (fp16 hi/lo) feature layout.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/vmcuda.h"
#include "conv_args.hpp"

namespace vm {

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

}  // namespace vm
