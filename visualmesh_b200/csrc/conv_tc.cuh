// Graph-convolution layer on the 5th-generation tensor cores (tcgen05) with fp32-grade accuracy.
//
// out[row] = act(bias + sum_s  X[nbr_s(row)] . W_s)  is a [rows x K] x [K x COUT] product whose A operand is a GATHER:
// K = (N+1) * CIN, slot s of row r is the feature row of r's s-th neighbour. A CTA owns 128-row tiles. For every slot
// its 128 threads (thread = row) read the neighbour's feature chunks (coalesced in the chunk-planar layout), split
// each fp32 value x into two parts x = hi + lo (two fp16 values, or a TF32 and its remainder for 8-channel layers) and
// store both into shared memory in the canonical K-major no-swizzle UMMA layout; one thread then issues
//     D[:, 0:2NP] += A_hi . [B_hi | B_lo]      D[:, 0:NP] += A_lo . B_hi        (tcgen05.mma, M = 128)
// against the layer's weights, which sit in shared memory pre-split the same way; the epilogue adds the two halves
// of D. Dropping only lo*lo keeps the product within ~2^-21 relative of fp32, far inside the 1e-4 tolerance that
// rules out a single reduced-precision pass.
// The accumulator lives in tensor memory (two buffers, so a tile's epilogue never meets the next tile's first MMA);
// the epilogue reads it with tcgen05.ld (thread = row again), adds the bias, applies the activation and writes the
// output row. Shared-memory stages are recycled through mbarriers armed by tcgen05.commit.
//
// Every wait is bounded: a wait that runs out raises the abort flag, the CTA stops issuing work, frees its tensor
// memory and returns, and the host reports VM_ERR_DEVICE_ABORT.
#pragma once

#include <cuda_fp16.h>
#include <type_traits>
#include <cuda_runtime.h>

#include "conv_common.cuh"

namespace vm {
namespace tc {

    constexpr int TILE_ROWS     = 128;
    constexpr int MAX_FRAMES    = 64;       // frames per launch whose tile counts fit the shared prefix table
    constexpr uint32_t WAIT_LIMIT = 4000000;  // default polls of mbarrier.try_wait before giving up (Args::wait_limit)
    constexpr int ABORT_TC_TIMEOUT = 2;

    __device__ __forceinline__ uint32_t smem_u32(const void* p) {
        return static_cast<uint32_t>(__cvta_generic_to_shared(p));
    }
    __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
    }
    __device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
        uint32_t ok;
        asm volatile(
          "{\n\t"
          ".reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t"
          "}\n"
          : "=r"(ok)
          : "r"(bar), "r"(parity)
          : "memory");
        return ok != 0;
    }
    // false when the limit ran out
    __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
        for (uint32_t i = 0; i < limit; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        return false;
    }

    // K-major, no swizzle: 8-row x 16-byte core matrices; LBO = distance between the two 16-byte K chunks of one MMA,
    // SBO = distance between 8-row groups. Version 1 = Blackwell descriptor.
    __device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
        return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16)
               | (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
    }

    __device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
        asm volatile(
          "{\n\t"
          ".reg .pred p;\n\t"
          "setp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
          "}\n" ::"r"(tmem_d),
          "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
          : "memory");
    }
    __device__ __forceinline__ void commit(uint32_t bar) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }

    struct Args {
        const void* w_cat;  // [K / KCH chunks][2 * NP rows][16 bytes]: rows 0..NP-1 = hi parts, NP..2NP-1 = lo parts
        const float* bias;  // [NP]
        int32_t n_frames;
        int32_t cout;
        int32_t* abort_flag;
        uint32_t wait_limit;  // polls of one mbarrier wait before the kernel gives up (0: every wait fails at once)
    };

    constexpr int ABORT_TC_RANGE = ABORT_RANGE;  // a feature value too large for the fp16 split: the host falls back to FFMA

    // Element formats of the split. HALF: x = h + l with h, l fp16 (kind::f16, 8 channels per 16-byte chunk, K = 16
    // per MMA) - half the shared-memory traffic of the fp32 container formats, needs |x| < 65504. Otherwise TF32:
    // h = x with 13 mantissa bits cleared, l = x - h (kind::tf32, 4 channels per chunk, K = 8 per MMA).
    template <bool HALF>
    struct Format {
        static constexpr int KCH          = HALF ? 8 : 4;  // channels per 16-byte chunk
        static constexpr uint32_t AB_CODE = HALF ? 0u : 2u;  // instruction-descriptor format code of A and B
    };

    template <bool HALF>
    __device__ __forceinline__ void mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
        if (HALF) {
            asm volatile(
              "{\n\t"
              ".reg .pred p;\n\t"
              "setp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
              "}\n" ::"r"(tmem_d),
              "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
              : "memory");
        }
        else {
            mma_tf32(tmem_d, desc_a, desc_b, idesc, accumulate);
        }
    }

    // shared memory: [stages][hi, lo][planes][128 rows][16 B], then the concatenated weights
    template <int CIN, int NP, int STAGES, bool HALF>
    constexpr size_t smem_bytes(int n_slots) {
        return 256 + static_cast<size_t>(STAGES) * 2 * (CIN / Format<HALF>::KCH) * TILE_ROWS * 16
               + static_cast<size_t>(n_slots) * (CIN / Format<HALF>::KCH) * 2 * NP * 16;
    }

    __device__ __forceinline__ void mbar_arrive(uint32_t bar) {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
    }
    // bounded wait that also gives up as soon as another role of the CTA has failed
    // Bounded wait that also gives up as soon as another role of the CTA has failed. The first poll is inline (it
    // usually succeeds, or blocks in hardware for a while and then succeeds); the polling loop is one shared function,
    // not a copy per call site: these kernels are unrolled over K steps and phases, and the layer's time moved by 10 to
    // 30 % with the size of the code around the waits.
    static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int32_t* failed, uint32_t limit) {
        for (uint32_t i = 1; i < limit; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if ((i & 1023u) == 1023u && *failed) return false;
        }
        return false;
    }
    __device__ __forceinline__ bool mbar_wait_or_fail(uint32_t bar, uint32_t parity, volatile int32_t* failed, uint32_t limit) {
        if (limit != 0 && mbar_try_wait(bar, parity)) return true;
        return mbar_wait_slow(bar, parity, failed, limit);
    }

    constexpr int PRODUCER_WARPS = 4;
    constexpr int CTA_THREADS    = (PRODUCER_WARPS + 1) * 32;

    // The two products of one K step:  D[:, 0:2NP] += A_hi . [B_hi | B_lo]   and   D[:, 0:NP] += A_lo . B_hi ;
    // the epilogue adds the two halves of D. A is read twice per K step instead of three times.
    //
    // Roles. Warps 0-3 (thread = row of the tile): gather, split, store into the stage, signal full[stage]; after the
    // last slot of a tile they wait for its accumulator, read it, release it and write the output rows.
    // Warp 4, one lane: waits full[stage], issues the stage's MMAs, commits to empty[stage] (the stage may be
    // overwritten once they have read it) and after a tile's last slot to acc_full. No block-wide barrier in the loop.
    template <int CIN, int NP, int STAGES, int NSLOTS, bool HALF>
    __global__ void __launch_bounds__(CTA_THREADS) k_graph_conv_tc(const ConvArgs a, const Args t) {
        static_assert(NP == 16 || NP == 32, "unsupported tile width");
        constexpr int KCH        = Format<HALF>::KCH;
        static_assert(CIN % (2 * KCH) == 0, "a slot must hold whole K steps");
        constexpr int PLANES     = CIN / KCH;            // 16-byte chunks per row and slot
        constexpr int PLANE      = TILE_ROWS * 16;       // bytes of one chunk over the 128 rows
        constexpr int SLOT_BYTES = PLANES * PLANE;       // one slot, hi or lo
        constexpr int WCHUNK     = 2 * NP * 16;          // bytes of one weight chunk: hi rows then lo rows
        constexpr int TMEM_COLS  = 4 * NP;               // two accumulator buffers of 2 * NP columns
        constexpr int DEPTH      = CIN <= 16 ? 2 : 1;    // slots whose loads are in flight ahead of the one being stored

        extern __shared__ __align__(1024) unsigned char smem_raw[];
        // full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], drain
        __shared__ uint64_t bars[2 * STAGES + 5];
        __shared__ uint32_t tmem_base_slot;
        __shared__ int32_t tile_prefix[MAX_FRAMES + 1];
        __shared__ int32_t failed_s;
        volatile int32_t* failed = &failed_s;

        const int tid  = threadIdx.x;
        const int warp = tid >> 5;
        const int lane = tid & 31;
        unsigned char* stage_base = smem_raw;
        unsigned char* w_s        = smem_raw + static_cast<size_t>(STAGES) * 2 * SLOT_BYTES;
        const uint32_t bar_full      = smem_u32(&bars[0]);
        const uint32_t bar_empty     = smem_u32(&bars[STAGES]);
        const uint32_t bar_acc_full  = smem_u32(&bars[2 * STAGES]);
        const uint32_t bar_acc_empty = smem_u32(&bars[2 * STAGES + 2]);
        const uint32_t bar_drain     = smem_u32(&bars[2 * STAGES + 4]);

        // ---- set-up ----
        if (tid == 0) {
            failed_s = 0;
            for (int i = 0; i < STAGES; ++i) {
                mbar_init(bar_full + 8 * i, PRODUCER_WARPS);
                mbar_init(bar_empty + 8 * i, 1);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(bar_acc_full + 8 * i, 1);
                mbar_init(bar_acc_empty + 8 * i, PRODUCER_WARPS);
            }
            mbar_init(bar_drain, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            int run = 0;
            for (int f = 0; f < t.n_frames; ++f) {
                tile_prefix[f] = run;
                const int rows = a.offsets[a.f0 + f + 1] - a.offsets[a.f0 + f] + 1;
                run += (rows + TILE_ROWS - 1) / TILE_ROWS;
            }
            tile_prefix[t.n_frames] = run;
        }
        if (warp == 0) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        {
            const uint4* g = reinterpret_cast<const uint4*>(t.w_cat);
            uint4* sw      = reinterpret_cast<uint4*>(w_s);
            for (int i = tid; i < NSLOTS * PLANES * 2 * NP; i += CTA_THREADS) sw[i] = __ldg(g + i);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = tmem_base_slot;
        const int total_tiles    = tile_prefix[t.n_frames];
        // tiles are dealt round-robin: a contiguous run per CTA was measured 10 % slower (the tail is less balanced)
        bool out_of_range        = false;

        if (warp == PRODUCER_WARPS) {
            // ================= MMA issuer =================
            if (lane == 0) {
                constexpr uint32_t IDESC_BASE = (1u << 4) | (Format<HALF>::AB_CODE << 7) | (Format<HALF>::AB_CODE << 10) | (static_cast<uint32_t>(TILE_ROWS >> 4) << 24);
                constexpr uint32_t IDESC_CAT  = IDESC_BASE | (static_cast<uint32_t>((2 * NP) >> 3) << 17);
                constexpr uint32_t IDESC_HI   = IDESC_BASE | (static_cast<uint32_t>(NP >> 3) << 17);
                const uint32_t w_addr = smem_u32(w_s);
                const uint32_t a_addr = smem_u32(stage_base);
                uint32_t it = 0, tile_count = 0;
                bool ok = true;
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_count) {
                    const uint32_t ab  = tile_count & 1u;
                    const uint32_t acc = tmem_base + ab * (2 * NP);
                    // the epilogue of the tile that used this accumulator two tiles ago must have read it
                    if (tile_count >= 2 && !mbar_wait_or_fail(bar_acc_empty + 8 * ab, ((tile_count >> 1) - 1) & 1u, failed, t.wait_limit)) {
                        ok = false;
                        break;
                    }
                    for (int s = 0; s < NSLOTS; ++s, ++it) {
                        const uint32_t stage = it % STAGES;
                        const uint32_t use   = it / STAGES;
                        if (!mbar_wait_or_fail(bar_full + 8 * stage, use & 1u, failed, t.wait_limit)) {
                            ok = false;
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_hi = a_addr + stage * 2 * SLOT_BYTES;
                        const uint32_t a_lo = a_hi + SLOT_BYTES;
#pragma unroll
                        for (int ks = 0; ks < PLANES / 2; ++ks) {
                            const uint64_t da_hi = smem_desc(a_hi + ks * 2 * PLANE, PLANE, 128);
                            const uint64_t da_lo = smem_desc(a_lo + ks * 2 * PLANE, PLANE, 128);
                            const uint64_t db    = smem_desc(w_addr + (s * PLANES + ks * 2) * WCHUNK, WCHUNK, 128);
                            mma<HALF>(acc, da_hi, db, IDESC_CAT, (s == 0 && ks == 0) ? 0u : 1u);
                            mma<HALF>(acc, da_lo, db, IDESC_HI, 1u);
                        }
                        commit(bar_empty + 8 * stage);
                        if (s == NSLOTS - 1) commit(bar_acc_full + 8 * ab);
                    }
                }
                if (!ok) {
                    failed_s = 1;
                    // Giving up: MMAs issued so far may still be running against this CTA's tensor memory and stages.
                    // One more commit tracks them all; the tear-down below frees the tensor memory only after it (the
                    // wait uses the full default limit whatever the kernel was told, and is itself bounded).
                    if (it > 0) {
                        commit(bar_drain);
                        mbar_wait(bar_drain, 0u, WAIT_LIMIT);
                    }
                }
            }
        }
        else {
            // ================= producers + epilogue =================
            const float4* in4 = reinterpret_cast<const float4*>(a.in);
            uint32_t it = 0, tile_count = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_count) {
                int f = 0;
                while (f + 1 < t.n_frames && tile_prefix[f + 1] <= tile) ++f;
                const int frame      = a.f0 + f;
                const int start      = a.offsets[frame];
                const int rows       = a.offsets[frame + 1] - start + 1;
                const int row        = (tile - tile_prefix[f]) * TILE_ROWS + tid;
                const int rowc       = min(row, rows - 1);
                const int local_base = start - a.offsets[a.f0] + f;
                const size_t nb_base = static_cast<size_t>(start + frame);
                const uint32_t ab    = tile_count & 1u;
                const uint32_t acc   = tmem_base + ab * (2 * NP);

                // all neighbour indices of this row up front; the loads of the next DEPTH slots are in flight while a slot
                // is split and stored
                int src_rows[NSLOTS];
                src_rows[0] = local_base + rowc;
#pragma unroll
                for (int s = 1; s < NSLOTS; ++s) src_rows[s] = local_base + __ldg(a.nb + (nb_base + rowc) * a.n_neighbours + (s - 1));
                float4 ring[DEPTH][CIN / 4];
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) {
                    if (d < NSLOTS) {
#pragma unroll
                        for (int c = 0; c < CIN / 4; ++c) ring[d][c] = in4[static_cast<size_t>(c) * a.in_stride + src_rows[d]];
                    }
                }

#pragma unroll
                for (int s = 0; s < NSLOTS; ++s, ++it) {
                    const uint32_t stage = it % STAGES;
                    const uint32_t use   = it / STAGES;
                    float4 cur[CIN / 4];
#pragma unroll
                    for (int c = 0; c < CIN / 4; ++c) cur[c] = ring[s % DEPTH][c];
                    if (s + DEPTH < NSLOTS) {
#pragma unroll
                        for (int c = 0; c < CIN / 4; ++c) ring[s % DEPTH][c] = in4[static_cast<size_t>(c) * a.in_stride + src_rows[s + DEPTH]];
                    }
                    // the MMAs that read this stage on its previous use must be done
                    if (use > 0 && !mbar_wait_or_fail(bar_empty + 8 * stage, (use - 1) & 1u, failed, t.wait_limit)) {
                        ok      = false;
                        *failed = 1;
                    }
                    unsigned char* hi_p = stage_base + static_cast<size_t>(stage) * 2 * SLOT_BYTES;
                    unsigned char* lo_p = hi_p + SLOT_BYTES;
                    if (!ok) {
                        // the stage may still be read by the tensor core: nothing is written into it any more
                    }
                    else if (HALF) {
#pragma unroll
                        for (int p = 0; p < PLANES; ++p) {
                            const float x[8] = {cur[2 * p].x, cur[2 * p].y, cur[2 * p].z, cur[2 * p].w,
                                                cur[2 * p + 1].x, cur[2 * p + 1].y, cur[2 * p + 1].z, cur[2 * p + 1].w};
                            uint32_t h[4], l[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                out_of_range |= fabsf(x[2 * q]) > 60000.0f || fabsf(x[2 * q + 1]) > 60000.0f;
                                const __half h0 = __float2half_rn(x[2 * q]);
                                const __half h1 = __float2half_rn(x[2 * q + 1]);
                                const __half l0 = __float2half_rn(x[2 * q] - __half2float(h0));
                                const __half l1 = __float2half_rn(x[2 * q + 1] - __half2float(h1));
                                h[q] = static_cast<uint32_t>(__half_as_ushort(h0)) | (static_cast<uint32_t>(__half_as_ushort(h1)) << 16);
                                l[q] = static_cast<uint32_t>(__half_as_ushort(l0)) | (static_cast<uint32_t>(__half_as_ushort(l1)) << 16);
                            }
                            *reinterpret_cast<uint4*>(hi_p + p * PLANE + tid * 16) = make_uint4(h[0], h[1], h[2], h[3]);
                            *reinterpret_cast<uint4*>(lo_p + p * PLANE + tid * 16) = make_uint4(l[0], l[1], l[2], l[3]);
                        }
                    }
                    else {
#pragma unroll
                        for (int c = 0; c < CIN / 4; ++c) {
                            const float4 x = cur[c];
                            float4 h, l;
                            h.x = __uint_as_float(__float_as_uint(x.x) & 0xFFFFE000u);
                            h.y = __uint_as_float(__float_as_uint(x.y) & 0xFFFFE000u);
                            h.z = __uint_as_float(__float_as_uint(x.z) & 0xFFFFE000u);
                            h.w = __uint_as_float(__float_as_uint(x.w) & 0xFFFFE000u);
                            l.x = x.x - h.x;
                            l.y = x.y - h.y;
                            l.z = x.z - h.z;
                            l.w = x.w - h.w;
                            *reinterpret_cast<float4*>(hi_p + c * PLANE + tid * 16) = h;
                            *reinterpret_cast<float4*>(lo_p + c * PLANE + tid * 16) = l;
                        }
                    }
                    // make this warp's stores visible to the tensor core, then one arrival per warp
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                }
                ok = __all_sync(0xffffffffu, ok) && !*failed;
                if (!ok) break;

                // ---- epilogue: accumulator -> registers -> bias, activation -> global ----
                // the tensor-memory load is warp-collective: the warp decides together whether to go on
                const bool arrived = mbar_wait_or_fail(bar_acc_full + 8 * ab, (tile_count >> 1) & 1u, failed, t.wait_limit);
                ok                 = __all_sync(0xffffffffu, arrived);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float v[NP];
#pragma unroll
                for (int j0 = 0; j0 < 2 * NP; j0 += 16) {
                    uint32_t r[16];
                    const uint32_t taddr = acc + (static_cast<uint32_t>(warp * 32) << 16) + j0;
                    asm volatile(
                      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                      : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        // columns NP..2NP-1 hold A_hi . B_lo of output column j0 + j - NP
                        if (j0 < NP) { v[j0 + j] = __uint_as_float(r[j]); }
                        else {
                            v[j0 + j - NP] = v[j0 + j - NP] + __uint_as_float(r[j]);
                        }
                    }
                }
                // the accumulator buffer may be overwritten from here on
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
#pragma unroll
                for (int j = 0; j < NP; ++j) v[j] = v[j] + __ldg(t.bias + j);
                if (row < rows) {
                    const size_t out_row = (a.out_global ? nb_base : static_cast<size_t>(local_base)) + row;
                    if (a.activation == VM_SOFTMAX) {
                        float total = 0.0f;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            if (j < t.cout) {
                                v[j]  = expf(v[j]);
                                total = __fadd_rn(total, v[j]);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < NP; ++j) v[j] = __fdiv_rn(v[j], total);
                    }
                    else {
                        activate<NP>(v, a.activation);  // one branch on the activation, then NP independent chains
                    }
                    if (a.out_split && t.cout == NP) { store_split<NP>(a.out, a.out_stride, out_row, v, a.range_flag); }
                    else if (a.out_planar) {
                        float4* out4 = reinterpret_cast<float4*>(a.out);
#pragma unroll
                        for (int j4 = 0; j4 < NP / 4; ++j4) {
                            if (j4 * 4 < t.cout) {
                                out4[static_cast<size_t>(j4) * a.out_stride + out_row] = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
                            }
                        }
                    }
                    else {
                        float* dst = a.out + out_row * t.cout;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            if (j < t.cout) dst[j] = v[j];
                        }
                    }
                }
            }
            if (!ok && lane == 0) failed_s = 1;
        }

        // ---- tear-down: nothing of this CTA may still be running on the tensor core when its memory goes away ----
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        const int any_range = __syncthreads_or(out_of_range ? 1 : 0);
        if (tid == 0) {
            if (failed_s) { atomicExch(t.abort_flag, ABORT_TC_TIMEOUT); }
            else if (any_range) {
                atomicCAS(t.abort_flag, 0, ABORT_TC_RANGE);
            }
        }
        if (warp == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        }
    }

    // ---- the same layer with the A operand in tensor memory -------------------------------------------------------
    // The split layout holds every feature row as fp16 hi chunks and lo chunks, which is exactly what the MMA wants of
    // one row of A. Here a gather thread (thread = row) loads its neighbour's chunks with 16-byte loads and writes them
    // straight into tensor-memory columns of its own lane (tcgen05.st); the MMA takes A from tensor memory and only the
    // weights from shared memory. The gathered tile never passes through shared memory, so the load/store data pipe
    // carries the gather once (as in the FFMA kernels) instead of three times (copy in, tensor-core read, conflicts).
    // The unit of work is one K step: 16 channels of one slot = two hi and two lo chunks = 16 columns of tensor memory.
    // Loads run DEPTH - 1 units ahead in registers, across tile boundaries; the register buffer of a unit is chosen at
    // compile time, so the tile body exists once per phase of the (units per tile) mod DEPTH cycle.
    __device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint4& x, const uint4& y) {
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(x.x), "r"(x.y),
                     "r"(x.z), "r"(x.w), "r"(y.x), "r"(y.y), "r"(y.z), "r"(y.w)
                     : "memory");
    }
    // A read-only 16-byte load that stays where it is written: the compiler may sink a plain __ldg down to its first
    // use, which would undo the software pipelining; volatile asm statements keep their order.
    __device__ __forceinline__ uint4 load_early(const uint4* p) {
        uint4 v;
        asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
        return v;
    }
    __device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
        asm volatile(
          "{\n\t"
          ".reg .pred p;\n\t"
          "setp.ne.b32 p, %4, 0;\n\t"
          "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
          "}\n" ::"r"(tmem_d),
          "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
          : "memory");
    }

    constexpr int LOAD_DEPTH = 3;  // register buffers of gathered units per thread

    // two accumulators of 2 NP columns, then the stages of A: 8 columns of hi pairs and 8 of lo pairs per K step
    template <int NP>
    __host__ __device__ constexpr int tmem_a_stages() {
        return NP == 16 ? 4 : 8;
    }
    template <int NP>
    __host__ __device__ constexpr int tmem_columns() {
        return 4 * NP + tmem_a_stages<NP>() * 16;  // 128 or 256: powers of two as the allocator wants
    }
    template <int CIN, int NP>
    constexpr size_t smem_bytes_tmem(int n_slots) {
        return 256 + static_cast<size_t>(n_slots) * (CIN / 8) * 2 * NP * 16;
    }

    template <int CIN, int NP, int NSLOTS>
    __global__ void __launch_bounds__(CTA_THREADS, NP == 16 ? 3 : 2) k_graph_conv_tc_tmem(const ConvArgs a, const Args t) {
        static_assert(NP == 16 || NP == 32, "unsupported tile width");
        static_assert(CIN % 16 == 0, "a slot must hold whole K steps of 16 fp16 channels");
        constexpr int PLANES    = CIN / 8;   // 16-byte chunks of the hi (or lo) half of a row
        constexpr int KSTEPS    = CIN / 16;  // K steps (units) per slot
        constexpr int UNITS     = NSLOTS * KSTEPS;
        constexpr int STAGES    = tmem_a_stages<NP>();
        constexpr int DEPTH     = LOAD_DEPTH;
        constexpr int WCHUNK    = 2 * NP * 16;
        constexpr int D_COLS    = 4 * NP;
        constexpr int TMEM_COLS = tmem_columns<NP>();
        static_assert(UNITS >= DEPTH - 1, "the prologue loads DEPTH - 1 units of the first tile");
        static_assert(DEPTH == 2 || DEPTH == 3, "the tile loop below is written out for two or three phases");

        extern __shared__ __align__(1024) unsigned char smem_raw[];
        __shared__ uint64_t bars[2 * STAGES + 5];
        __shared__ uint32_t tmem_base_slot;
        __shared__ int32_t tile_prefix[MAX_FRAMES + 1];
        __shared__ int32_t frame_start[MAX_FRAMES + 1];  // offsets[f0 + f]: first compact node of frame f
        __shared__ int32_t failed_s;
        volatile int32_t* failed = &failed_s;

        const int tid  = threadIdx.x;
        const int warp = tid >> 5;
        const int lane = tid & 31;
        unsigned char* w_s           = smem_raw;
        const uint32_t bar_full      = smem_u32(&bars[0]);
        const uint32_t bar_empty     = smem_u32(&bars[STAGES]);
        const uint32_t bar_acc_full  = smem_u32(&bars[2 * STAGES]);
        const uint32_t bar_acc_empty = smem_u32(&bars[2 * STAGES + 2]);
        const uint32_t bar_drain     = smem_u32(&bars[2 * STAGES + 4]);

        if (tid == 0) {
            failed_s = 0;
            for (int i = 0; i < STAGES; ++i) {
                mbar_init(bar_full + 8 * i, PRODUCER_WARPS);
                mbar_init(bar_empty + 8 * i, 1);
            }
            for (int i = 0; i < 2; ++i) {
                mbar_init(bar_acc_full + 8 * i, 1);
                mbar_init(bar_acc_empty + 8 * i, PRODUCER_WARPS);
            }
            mbar_init(bar_drain, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        for (int f = tid; f <= t.n_frames; f += CTA_THREADS) frame_start[f] = a.offsets[a.f0 + f];
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int f = 0; f < t.n_frames; ++f) {
                tile_prefix[f] = run;
                const int rows = frame_start[f + 1] - frame_start[f] + 1;
                run += (rows + TILE_ROWS - 1) / TILE_ROWS;
            }
            tile_prefix[t.n_frames] = run;
        }
        if (warp == 0) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        {
            const uint4* g = reinterpret_cast<const uint4*>(t.w_cat);
            uint4* sw      = reinterpret_cast<uint4*>(w_s);
            for (int i = tid; i < NSLOTS * PLANES * 2 * NP; i += CTA_THREADS) sw[i] = __ldg(g + i);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = tmem_base_slot;
        const uint32_t a_base    = tmem_base + D_COLS;
        const int total_tiles    = tile_prefix[t.n_frames];

        if (warp == PRODUCER_WARPS) {
            // ================= MMA issuer =================
            if (lane == 0) {
                constexpr uint32_t IDESC_BASE = (1u << 4) | (static_cast<uint32_t>(TILE_ROWS >> 4) << 24);  // fp16 x fp16 -> fp32, K-major
                constexpr uint32_t IDESC_CAT  = IDESC_BASE | (static_cast<uint32_t>((2 * NP) >> 3) << 17);
                constexpr uint32_t IDESC_HI   = IDESC_BASE | (static_cast<uint32_t>(NP >> 3) << 17);
                const uint32_t w_addr = smem_u32(w_s);
                uint32_t it = 0, tile_count = 0;
                bool ok = true;
                for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tile_count) {
                    const uint32_t ab  = tile_count & 1u;
                    const uint32_t acc = tmem_base + ab * (2 * NP);
                    if (tile_count >= 2 && !mbar_wait_or_fail(bar_acc_empty + 8 * ab, ((tile_count >> 1) - 1) & 1u, failed, t.wait_limit)) {
                        ok = false;
                        break;
                    }
                    for (int u = 0; u < UNITS; ++u, ++it) {
                        const uint32_t stage = it % STAGES;
                        const uint32_t use   = it / STAGES;
                        if (!mbar_wait_or_fail(bar_full + 8 * stage, use & 1u, failed, t.wait_limit)) {
                            ok = false;
                            break;
                        }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_hi = a_base + stage * 16;
                        const uint64_t db   = smem_desc(w_addr + u * 2 * WCHUNK, WCHUNK, 128);  // chunks 2u and 2u + 1 of K
                        mma_f16_ts(acc, a_hi, db, IDESC_CAT, u == 0 ? 0u : 1u);
                        mma_f16_ts(acc, a_hi + 8, db, IDESC_HI, 1u);
                        commit(bar_empty + 8 * stage);
                        if (u == UNITS - 1) commit(bar_acc_full + 8 * ab);
                    }
                }
                if (!ok) {
                    failed_s = 1;
                    // Giving up: MMAs issued so far may still be running against this CTA's tensor memory and stages.
                    // One more commit tracks them all; the tear-down below frees the tensor memory only after it (the
                    // wait uses the full default limit whatever the kernel was told, and is itself bounded).
                    if (it > 0) {
                        commit(bar_drain);
                        mbar_wait(bar_drain, 0u, WAIT_LIMIT);
                    }
                }
            }
        }
        else {
            // ================= gather + epilogue =================
            const uint4* in4         = reinterpret_cast<const uint4*>(a.in);
            const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;  // this warp's quarter of the 128 lanes
            uint32_t tile_count = 0;
            bool ok = true;

            struct TileRef {
                int rows;        // rows of the tile's frame, sentinel row included
                int row;         // this thread's row within the frame
                int local_base;  // first feature row of the frame in this launch
                size_t nb_base;  // first neighbourhood / global output row of the frame
            };
            int frame_hint = 0;  // tiles only move forward: the search resumes at the frame of the last tile located
            auto locate = [&](int tile) {
                int f = frame_hint;
                while (f + 1 < t.n_frames && tile_prefix[f + 1] <= tile) ++f;
                frame_hint      = f;
                const int start = frame_start[f];
                TileRef r;
                r.rows       = frame_start[f + 1] - start + 1;
                r.row        = (tile - tile_prefix[f]) * TILE_ROWS + tid;
                r.local_base = start - frame_start[0] + f;
                r.nb_base    = static_cast<size_t>(start + a.f0 + f);
                return r;
            };
            // Source rows relative to the frame's first feature row. The neighbour indices come from HBM and nothing
            // may touch them before they are needed (an add right behind the load would stall the thread for the whole
            // memory latency): the frame's base is added where the row is used.
            auto fetch_rows = [&](const TileRef& r, int (&src)[NSLOTS]) {
                const int rowc = min(r.row, r.rows - 1);
                src[0]         = rowc;
#pragma unroll
                for (int s = 1; s < NSLOTS; ++s) src[s] = __ldg(a.nb + (r.nb_base + rowc) * a.n_neighbours + (s - 1));
            };
            auto arrived_value = [](int x) {
                asm volatile("" : "+r"(x));  // pins the first use of a loaded value to this point of the program
                return x;
            };
            uint4 buf[DEPTH][4];  // two hi chunks and two lo chunks of up to DEPTH gathered units
            auto load = [&](uint4 (&b)[4], int src_row, int ks) {
                b[0] = load_early(in4 + static_cast<size_t>(2 * ks) * a.in_stride + src_row);
                b[1] = load_early(in4 + static_cast<size_t>(2 * ks + 1) * a.in_stride + src_row);
                b[2] = load_early(in4 + static_cast<size_t>(PLANES + 2 * ks) * a.in_stride + src_row);
                b[3] = load_early(in4 + static_cast<size_t>(PLANES + 2 * ks + 1) * a.in_stride + src_row);
            };

            int cur[NSLOTS], nxt[NSLOTS];
            TileRef cr = {1, 0, 0, 0}, nr = {1, 0, 0, 0};
            int tile = blockIdx.x;
            if (tile < total_tiles) {
                cr = locate(tile);
                fetch_rows(cr, cur);
#pragma unroll
                for (int u = 0; u < DEPTH - 1; ++u) load(buf[u], cr.local_base + arrived_value(cur[u / KSTEPS]), u % KSTEPS);
            }

            // one tile; PH = (units handled before this tile) mod DEPTH selects the register buffers at compile time
            auto do_tile = [&](auto phase) -> bool {
                constexpr int PH = decltype(phase)::value;
                if (tile >= total_tiles || !ok) return false;
                const uint32_t ab   = tile_count & 1u;
                const uint32_t acc  = tmem_base + ab * (2 * NP);
                const uint32_t it0  = tile_count * UNITS;
                const bool has_next = tile + static_cast<int>(gridDim.x) < total_tiles;
                if (has_next) {
                    nr = locate(tile + gridDim.x);
                    fetch_rows(nr, nxt);
                }
#pragma unroll
                for (int u = 0; u < UNITS; ++u) {
                    constexpr int AHEAD = DEPTH - 1;
                    const int ua        = u + AHEAD;  // the unit whose loads start now
                    if (ua < UNITS) { load(buf[(PH + ua) % DEPTH], cr.local_base + arrived_value(cur[ua / KSTEPS]), ua % KSTEPS); }
                    else if (has_next) {
                        load(buf[(PH + ua) % DEPTH], nr.local_base + arrived_value(nxt[(ua - UNITS) / KSTEPS]), (ua - UNITS) % KSTEPS);
                    }
                    const uint32_t it    = it0 + u;
                    const uint32_t stage = it % STAGES;
                    const uint32_t use   = it / STAGES;
                    // After a wait that ran out the warp still finishes the tile's stores (they are warp-collective, and a
                    // vote per K step measured 10 % of the layer's time): the stage may then be overwritten while an MMA reads
                    // it, which only garbles results of a launch that is reported as failed; the issuer waits for every
                    // MMA in flight before the tensor memory is freed.
                    if (use > 0 && !mbar_wait_or_fail(bar_empty + 8 * stage, (use - 1) & 1u, failed, t.wait_limit)) ok = false;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint4(&b)[4]  = buf[(PH + u) % DEPTH];
                    const uint32_t a_hi = a_base + lane_base + stage * 16;
                    tmem_st8(a_hi, b[0], b[1]);
                    tmem_st8(a_hi + 8, b[2], b[3]);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * stage);
                }
                ok = __all_sync(0xffffffffu, ok) && !*failed;
                if (!ok) return false;
                const bool arrived = mbar_wait_or_fail(bar_acc_full + 8 * ab, (tile_count >> 1) & 1u, failed, t.wait_limit);
                ok                 = __all_sync(0xffffffffu, arrived);
                if (!ok) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float v[NP];
#pragma unroll
                for (int j0 = 0; j0 < 2 * NP; j0 += 16) {
                    uint32_t r[16];
                    const uint32_t taddr = acc + lane_base + j0;
                    asm volatile(
                      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                      : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (j0 < NP) { v[j0 + j] = __uint_as_float(r[j]); }
                        else {
                            v[j0 + j - NP] = v[j0 + j - NP] + __uint_as_float(r[j]);
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * ab);
#pragma unroll
                for (int j = 0; j < NP; ++j) v[j] = v[j] + __ldg(t.bias + j);
                if (cr.row < cr.rows) {
                    const size_t out_row = (a.out_global ? cr.nb_base : static_cast<size_t>(cr.local_base)) + cr.row;
                    if (a.activation == VM_SOFTMAX) {
                        float total = 0.0f;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            if (j < t.cout) {
                                v[j]  = expf(v[j]);
                                total = __fadd_rn(total, v[j]);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < NP; ++j) v[j] = __fdiv_rn(v[j], total);
                    }
                    else {
                        activate<NP>(v, a.activation);  // one branch on the activation, then NP independent chains
                    }
                    if (a.out_split && t.cout == NP) { store_split<NP>(a.out, a.out_stride, out_row, v, a.range_flag); }
                    else if (a.out_planar) {
                        float4* out4 = reinterpret_cast<float4*>(a.out);
#pragma unroll
                        for (int j4 = 0; j4 < NP / 4; ++j4) {
                            if (j4 * 4 < t.cout) {
                                out4[static_cast<size_t>(j4) * a.out_stride + out_row] = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
                            }
                        }
                    }
                    else {
                        float* dst = a.out + out_row * t.cout;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            if (j < t.cout) dst[j] = v[j];
                        }
                    }
                }
                cr = nr;
#pragma unroll
                for (int s = 0; s < NSLOTS; ++s) cur[s] = nxt[s];
                tile += gridDim.x;
                ++tile_count;
                return true;
            };
            // DEPTH tiles bring the phase back to where it started
            while (do_tile(std::integral_constant<int, 0>{}) && do_tile(std::integral_constant<int, UNITS % DEPTH>{})
                   && (DEPTH == 2 || do_tile(std::integral_constant<int, (2 * UNITS) % DEPTH>{}))) {}
            if (!ok && lane == 0) failed_s = 1;
        }

        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && failed_s) atomicExch(t.abort_flag, ABORT_TC_TIMEOUT);
        if (warp == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        }
    }

}  // namespace tc
}  // namespace vm
