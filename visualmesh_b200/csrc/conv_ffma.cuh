// Graph-convolution layer kernels on the CUDA cores (fused gather + dense + activation).
#pragma once

#include "conv_common.cuh"

namespace vm {

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
// The narrow 8-channel layers wait on their gather: six blocks of 256 threads per SM (42 registers) instead of five
// measured 102 -> 98 us on the 8 -> 3 layer over 4.4 M rows, eight (32 registers) spill. 0 = no bound for the others.
template <int CIN, int COUT, int R, int WMAX, int T = CONV_THREADS, int NS = 0>
__global__ void __launch_bounds__(T, (CIN == 8 && COUT <= 8 && T == 256) ? 6 : 0) k_graph_conv_cw(const ConvArgs a, const __grid_constant__ ConvWeights<WMAX> wp) {
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
