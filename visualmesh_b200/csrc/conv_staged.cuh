// Graph-convolution layer on the tensor cores with the gather served from shared memory.
//
// The other layer kernels gather every neighbour row with per-thread global loads; a quarter of them miss the L1 cache
// (the first touch of every row), each miss stalls its warp for a full memory latency, and the layers end up bound by
// that latency (tensor-core kernels of conv_tc.cuh) or by the FP32 pipe (conv_ffma.cuh). Mesh nodes are stored in the
// order of the reference's BSP (cpp/visualmesh/mesh.hpp:450-466), which is spatially compact: of the neighbour
// references of 256 consecutive on-screen rows about 87 % point inside the same 256 rows, and the rest touch ~95
// distinct rows outside.
//
// So the rows of a frame are cut into super-tiles of consecutive rows and a tile plan (tile_plan.cuh) is made once per
// chunk of frames: the list of outside rows each super-tile needs (its halo) and every row's neighbours as 16-bit
// positions inside "super-tile + halo". A layer then runs as a persistent kernel whose loader warp brings a
// super-tile's own rows into shared memory with one bulk asynchronous copy per 16-byte plane and its halo rows with
// 16-byte asynchronous copies - every byte of the feature buffer is requested once per super-tile that needs it, in
// large contiguous pieces, a super-tile ahead of its use - and whose compute warps read neighbour rows from shared
// memory only: ldmatrix takes one row address per lane, so the gather of sixteen neighbour rows IS the load of an MMA
// operand fragment. The product runs on the warp-level tensor-core path (mma.sync m16n8k16, fp16 hi/lo parts of both
// operands, fp32 accumulators in registers) rather than tcgen05: a 16-channel slot is a 16x16x16 product per sixteen
// rows, far too little work per instruction to amortise moving a gathered tile into tensor memory and a single-thread
// issue pipeline, while here every warp is an independent worker with nothing to hand over (measured on the 16 -> 16
// layer over 4.4 M rows: tcgen05 with global-load gather 337 us, tcgen05 with this staging 740 us at one CTA per SM,
// this kernel 222 us; the FFMA kernel 308 us). The epilogue runs on the accumulator registers.
// A neighbour whose halo slot did not fit (more outside rows than halo slots) is marked and fetched from global memory
// by its warp, so any neighbourhood is computed correctly, only slower.
//
// The only waits are for a window's copies (compute warps) and for a window to be handed back (loader), and they are
// bounded. No multicast of any kind; all copies read this GPU's own memory.
#pragma once

#include "conv_tc.cuh"
#include "tile_plan.cuh"

namespace vm {
namespace st {

    struct PlanArgs {
        const int32_t* offsets;  // batch-wide point offsets
        const int32_t* nb;       // batch-wide neighbourhood rows (frame-local indices)
        PlanOut out;
        int32_t f0;
    };

    // The plan for a neighbourhood that is already in memory: one block per super-tile (blockIdx.x) and frame
    // (blockIdx.y), one thread per row. (On the hot path the neighbour-remap kernel makes the plan as it writes the
    // neighbourhood.)
    template <int N>
    __global__ void __launch_bounds__(ST) k_tile_plan(const PlanArgs a) {
        const int f     = blockIdx.y;
        const int frame = a.f0 + f;
        const int start = a.offsets[frame];
        const int rows  = a.offsets[frame + 1] - start + 1;
        const int t0    = blockIdx.x * ST;
        if (t0 >= rows) return;
        const int row    = t0 + static_cast<int>(threadIdx.x);
        const bool valid = row < rows;
        int idx[N];
#pragma unroll
        for (int j = 0; j < N; ++j) idx[j] = 0;
        if (valid) {
            const int32_t* src = a.nb + static_cast<size_t>(start + frame + row) * N;
#pragma unroll
            for (int j = 0; j < N; ++j) idx[j] = __ldg(src + j);
        }
        plan_super_tile<N>(idx, valid, t0, f, a.offsets, a.f0, a.out);
    }

    // ---- asynchronous copies ------------------------------------------------------------------------------------------
    __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
    }
    // contiguous global -> shared, completion counted in bytes on the mbarrier; no multicast
    __device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                     "r"(bytes), "r"(bar)
                     : "memory");
    }
    __device__ __forceinline__ void copy16(uint32_t dst, const void* src) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    }
    // one arrival on the mbarrier once all earlier 16-byte copies of this thread have landed (counted at init)
    __device__ __forceinline__ void copies_arrive(uint32_t bar) {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
    }
    // ---- warp-level tensor-core pieces ----------------------------------------------------------------------------------
    // Four 8x8 fp16 matrices, one 16-byte row address per lane: the A fragment of mma.m16n8k16 for sixteen ARBITRARY
    // rows of shared memory - the gather of a slot is this one instruction.
    __device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
    }
    // D += A . B, A 16x16 fp16 (row), B 16x8 fp16 (col), D 16x8 fp32
    __device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
    __device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    // x = h + l with h = fp16(x), l = fp16(x - h), for two values at once
    __device__ __forceinline__ void split_pair(float x0, float x1, uint32_t& h, uint32_t& l) {
        h               = pack_half2(x0, x1);
        const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&h));
        l               = pack_half2(x0 - hf.x, x1 - hf.y);
    }

    struct Args {
        int32_t n_frames;
        int32_t cout;
        int32_t* abort_flag;
        uint32_t wait_limit;  // polls of one wait for a window before the kernel gives up (0: the first wait fails at once)
    };

    constexpr uint32_t WAIT_LIMIT  = tc::WAIT_LIMIT;
    constexpr int MAX_FRAMES       = tc::MAX_FRAMES;
    constexpr int TILE             = 16;  // rows of one warp-level MMA tile

    constexpr int PAIR = 2;  // 16-row tiles a warp works on at a time: two independent chains of MMAs to interleave

    template <int CIN, int COUT, int NSLOTS, int THREADS>
    __host__ __device__ constexpr size_t smem_bytes() {
        return static_cast<size_t>(2) * (2 * (CIN / 8)) * (ST + HALO) * 16                     // two windows
               + static_cast<size_t>(THREADS / 32 - 1) * (2 * (CIN / 8)) * TILE * 16           // per-warp rows fetched from global memory
               + static_cast<size_t>(NSLOTS) * (CIN / 16) * (COUT / 8) * 2 * 32 * 8;           // B fragments, hi and lo
    }
    template <int CIN, int COUT>
    __host__ __device__ constexpr int ctas_per_sm_wanted() {
        return CIN == 16 ? (COUT <= 16 ? 3 : 2) : 1;
    }

    // One CTA walks super-tiles; while it computes on one window the next is on its way. Every warp owns pairs of 16-row
    // tiles of the super-tile: for each slot one ldmatrix per fp16 part and tile gathers the sixteen neighbour rows from
    // the window, three MMAs per 8 output columns add hi.hi, hi.lo and lo.hi into fp32 accumulators in registers
    // (dropping only lo.lo keeps ~2^-21 relative accuracy), and the epilogue (bias, activation, store as fp32 chunks or
    // split again for the next such layer) runs on the accumulator registers. The weights sit in shared memory as
    // ready-made B fragments (8 bytes per lane, read once per slot for both tiles). The last warp of the CTA is the
    // loader; a compute warp waits only for a window to land and tells the loader when it is done with one, so no
    // compute warp ever waits for another.
    template <int CIN, int COUT, int NSLOTS, int THREADS>
    __global__ void __launch_bounds__(THREADS, ctas_per_sm_wanted<CIN, COUT>()) k_graph_conv_mma(const ConvArgs a, const Args t, const Plan plan) {
        static_assert(CIN % 16 == 0 && COUT % 8 == 0 && ST % (PAIR * TILE) == 0, "whole K steps, whole column blocks, whole tile pairs");
        constexpr int PLANES    = CIN / 8;   // 16-byte chunks of the hi (or lo) half of a row
        constexpr int ALLP      = 2 * PLANES;
        constexpr int KSTEPS    = CIN / 16;
        constexpr int NBLK      = COUT / 8;
        constexpr int WARPS     = THREADS / 32 - 1;       // compute warps; the last warp of the CTA is the loader
        constexpr int WROWS     = ST + HALO;
        constexpr int PSTRIDE   = WROWS * 16;             // bytes between planes of a window
        constexpr int WIN_BYTES = ALLP * PSTRIDE;
        constexpr int SCR_BYTES = ALLP * TILE * 16;       // per warp: rows of one tile that were not staged
        constexpr int NFRAG     = NSLOTS * KSTEPS * NBLK; // B fragments per part

        extern __shared__ __align__(1024) unsigned char smem_raw[];
        __shared__ uint64_t bars[4];                      // full[2]: a window has landed; empty[2]: every compute warp is done with it
        __shared__ int32_t tile_prefix[MAX_FRAMES + 1];   // in super-tiles
        __shared__ int32_t frame_start[MAX_FRAMES + 1];   // offsets[f0 + f]
        __shared__ int32_t failed_s;
        volatile int32_t* failed = &failed_s;

        const int tid  = threadIdx.x;
        const int warp = tid >> 5;
        const int lane = tid & 31;
        const int g    = lane >> 2;  // row of the accumulator fragment (and g + 8)
        const int tq   = lane & 3;   // column pair of the accumulator fragment
        const uint32_t win_addr = tc::smem_u32(smem_raw);
        const uint32_t scr_addr = win_addr + 2 * WIN_BYTES + warp * SCR_BYTES;
        unsigned char* scr_ptr  = smem_raw + 2 * WIN_BYTES + warp * SCR_BYTES;
        const uint32_t frag_addr = win_addr + 2 * WIN_BYTES + WARPS * SCR_BYTES + lane * 8;  // this lane's 8 bytes of fragment 0, hi part
        const uint32_t bar_full  = tc::smem_u32(&bars[0]);
        const uint32_t bar_empty = tc::smem_u32(&bars[2]);

        if (tid == 0) {
            failed_s = 0;
            for (int i = 0; i < 2; ++i) {
                tc::mbar_init(bar_full + 8 * i, 1 + 32);  // the bulk copies' byte count + one arrival per loader lane
                tc::mbar_init(bar_empty + 8 * i, WARPS);
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        for (int f = tid; f <= t.n_frames; f += THREADS) frame_start[f] = a.offsets[a.f0 + f];
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int f = 0; f < t.n_frames; ++f) {
                tile_prefix[f] = run;
                const int rows = frame_start[f + 1] - frame_start[f] + 1;
                run += (rows + ST - 1) / ST;
            }
            tile_prefix[t.n_frames] = run;
        }

        // ---- B fragments: weights [k][n] split into fp16 hi and lo, in the register layout of mma.m16n8k16 ----
        // fragment of (slot s, K step ks, column block nb), lane (g, tq): b0 = {W[k0 + 2 tq][n], W[k0 + 2 tq + 1][n]} and b1 =
        // the same 8 rows further, with k0 = s * CIN + ks * 16 and n = nb * 8 + g
        {
            constexpr int COUTP = (COUT + 3) & ~3;
            uint2* w_frag       = reinterpret_cast<uint2*>(smem_raw + 2 * WIN_BYTES + WARPS * SCR_BYTES);  // [part][fragment][lane]
            for (int frag = warp; frag < NFRAG; frag += WARPS + 1) {
                const int nb = frag % NBLK, ks = (frag / NBLK) % KSTEPS, sl = frag / (NBLK * KSTEPS);
                const int n  = nb * 8 + g;
                const int k0 = sl * CIN + ks * 16 + 2 * tq;
                uint32_t h[2], l[2];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const float w0 = __ldg(a.weights + static_cast<size_t>(k0 + 8 * half) * COUTP + n);
                    const float w1 = __ldg(a.weights + static_cast<size_t>(k0 + 8 * half + 1) * COUTP + n);
                    split_pair(w0, w1, h[half], l[half]);
                }
                w_frag[frag * 32 + lane]           = make_uint2(h[0], h[1]);
                w_frag[(NFRAG + frag) * 32 + lane] = make_uint2(l[0], l[1]);
            }
        }
        float bias[NBLK][2];
#pragma unroll
        for (int nb = 0; nb < NBLK; ++nb) {
            bias[nb][0] = __ldg(a.biases + nb * 8 + 2 * tq);
            bias[nb][1] = __ldg(a.biases + nb * 8 + 2 * tq + 1);
        }
        __syncthreads();
        const int total_st = tile_prefix[t.n_frames];

        struct StRef {
            int rows;        // rows of the frame, off-screen row included
            int t0;          // first row of the super-tile within the frame
            int local_base;  // first feature row of the frame in this launch
            size_t nb_base;  // first neighbourhood row of the frame
        };
        int frame_hint = 0;
        auto locate = [&](int s) {
            int f = frame_hint;
            while (f + 1 < t.n_frames && tile_prefix[f + 1] <= s) ++f;
            frame_hint      = f;
            const int start = frame_start[f];
            StRef r;
            r.rows       = frame_start[f + 1] - start + 1;
            r.t0         = (s - tile_prefix[f]) * ST;
            r.local_base = start - frame_start[0] + f;
            r.nb_base    = static_cast<size_t>(start + a.f0 + f);
            return r;
        };
        const unsigned char* in_bytes = reinterpret_cast<const unsigned char*>(a.in);
        const uint4* in4              = reinterpret_cast<const uint4*>(a.in);
        const uint4* nbl4             = reinterpret_cast<const uint4*>(plan.nbl);

        if (warp == WARPS) {
            // ================= loader warp: one window ahead of the compute warps per buffer =================
            // The halo list of a super-tile (its length, then this lane's entries) is read one super-tile ahead, while
            // the loader waits for a buffer anyway: the copies of a window then start the moment its buffer is free
            // instead of two dependent trips to global memory later.
            constexpr int PER_LANE = (HALO + 31) / 32;
            int n_halo = 0;
            int32_t halo_row[PER_LANE];
            auto fetch_halo_list = [&](int st) {
                n_halo                = __ldg(plan.halo_count + st);
                const int32_t* h_rows = plan.halo_rows + static_cast<size_t>(st) * HALO;
#pragma unroll
                for (int k = 0; k < PER_LANE; ++k) halo_row[k] = __ldg(h_rows + min(lane + 32 * k, HALO - 1));  // entries past n_halo are never used
            };
            uint32_t n = 0;
            bool ok    = true;
            if (static_cast<int>(blockIdx.x) < total_st) fetch_halo_list(blockIdx.x);
            for (int s = blockIdx.x; s < total_st; s += gridDim.x, ++n) {
                const uint32_t b = n & 1u;
                // every compute warp must be done with the super-tile that used this buffer before
                if (n >= 2 && !tc::mbar_wait_or_fail(bar_empty + 8 * b, ((n >> 1) - 1) & 1u, failed, t.wait_limit)) {
                    ok = false;
                    break;
                }
                const StRef r      = locate(s);
                const int own      = min(ST, r.rows - r.t0);
                const uint32_t dst = win_addr + b * WIN_BYTES;
                const uint32_t bar = bar_full + 8 * b;
                if (lane == 0) {
                    mbar_expect_tx(bar, static_cast<uint32_t>(ALLP * own * 16));
#pragma unroll
                    for (int p = 0; p < ALLP; ++p) {
                        bulk_copy(dst + p * PSTRIDE, in_bytes + (static_cast<size_t>(p) * a.in_stride + r.local_base + r.t0) * 16,
                                  static_cast<uint32_t>(own * 16), bar);
                    }
                }
#pragma unroll
                for (int k = 0; k < PER_LANE; ++k) {
                    const int h = lane + 32 * k;
                    if (h < n_halo) {
                        const size_t src_row = static_cast<size_t>(halo_row[k]);
#pragma unroll
                        for (int p = 0; p < ALLP; ++p) copy16(dst + p * PSTRIDE + (ST + h) * 16, in_bytes + (static_cast<size_t>(p) * a.in_stride + src_row) * 16);
                    }
                }
                if (s + static_cast<int>(gridDim.x) < total_st) fetch_halo_list(s + gridDim.x);
                copies_arrive(bar);
            }
            if (!ok) *failed = 1;
            // Nothing may still be writing this CTA's shared memory when it exits. On the normal path the compute warps have
            // waited for every window; after a wait ran out the last windows may still be on their way: this lane's own
            // 16-byte copies are waited for here, the bulk copies through the windows' barriers (a window is the last one
            // issued into its buffer, so its barrier phase can only be pending or complete), with the full default limit.
            asm volatile("cp.async.wait_all;" ::: "memory");
            if (lane == 0) {
                for (uint32_t m = n > 2 ? n - 2 : 0; m < n; ++m) tc::mbar_wait(bar_full + 8 * (m & 1u), (m >> 1) & 1u, WAIT_LIMIT);
            }
        }
        else {
        // ================= compute warps =================
        uint32_t n = 0;
        bool ok    = true;
        for (int s = blockIdx.x; s < total_st; s += gridDim.x, ++n) {
            const uint32_t b  = n & 1u;
            const StRef r     = locate(s);
            const int own     = min(ST, r.rows - r.t0);
            const int n_pairs = (own + PAIR * TILE - 1) / (PAIR * TILE);
            // neighbour positions of this warp's first pair of tiles, fetched while the window is on its way
            // (lanes 0-15 and 16-31 address the same sixteen rows; tile i of the pair is rows 16 i .. 16 i + 15)
            int arow[PAIR];
            uint4 pos[PAIR];
            auto fetch_positions = [&](int pair, int (&rows_out)[PAIR], uint4 (&pos_out)[PAIR]) {
#pragma unroll
                for (int i = 0; i < PAIR; ++i) {
                    rows_out[i] = min((pair * PAIR + i) * TILE + (lane & 15), own - 1);
                    pos_out[i]  = __ldg(nbl4 + r.local_base + r.t0 + rows_out[i]);
                }
            };
            if (warp < n_pairs) fetch_positions(warp, arow, pos);
            ok = __all_sync(0xffffffffu, tc::mbar_wait_or_fail(bar_full + 8 * b, (n >> 1) & 1u, failed, t.wait_limit));
            if (!ok) {
                *failed = 1;
                break;
            }
            const uint32_t win = win_addr + b * WIN_BYTES;
            for (int pair = warp; pair < n_pairs; pair += WARPS) {
                int cur_row[PAIR];
                uint4 cur_pos[PAIR];
#pragma unroll
                for (int i = 0; i < PAIR; ++i) {
                    cur_row[i] = arow[i];
                    cur_pos[i] = pos[i];
                }
                if (pair + WARPS < n_pairs) fetch_positions(pair + WARPS, arow, pos);  // for the next round, in flight during this one
                float acc[PAIR][NBLK][4];
#pragma unroll
                for (int i = 0; i < PAIR; ++i) {
#pragma unroll
                    for (int nb = 0; nb < NBLK; ++nb) {
                        acc[i][nb][0] = bias[nb][0];
                        acc[i][nb][1] = bias[nb][1];
                        acc[i][nb][2] = bias[nb][0];
                        acc[i][nb][3] = bias[nb][1];
                    }
                }
#pragma unroll
                for (int sl = 0; sl < NSLOTS; ++sl) {
                    uint32_t base[PAIR], pstride[PAIR];
                    bool miss[PAIR];
                    bool any_miss = false;
#pragma unroll
                    for (int i = 0; i < PAIR; ++i) {
                        uint32_t p;
                        if (sl == 0) { p = static_cast<uint32_t>(cur_row[i]); }
                        else {
                            const uint4& q      = cur_pos[i];
                            const uint32_t word = ((sl - 1) >> 1) == 0 ? q.x : ((sl - 1) >> 1) == 1 ? q.y : ((sl - 1) >> 1) == 2 ? q.z : q.w;
                            p                   = ((sl - 1) & 1) ? (word >> 16) : (word & 0xFFFFu);
                        }
                        // address of this lane's row in plane 0 of the window, and the distance between planes
                        base[i]    = win + p * 16;
                        pstride[i] = PSTRIDE;
                        miss[i]    = sl > 0 && p == NBL_GLOBAL;
                        any_miss |= miss[i];
                    }
                    // the slot's products for tiles [I0, I1) of the pair: one B fragment load serves all of them
                    auto products = [&](auto i0, auto i1) {
                        constexpr int I0 = decltype(i0)::value, I1 = decltype(i1)::value;
#pragma unroll
                        for (int ks = 0; ks < KSTEPS; ++ks) {
                            uint32_t a_hi[PAIR][4], a_lo[PAIR][4];
#pragma unroll
                            for (int i = I0; i < I1; ++i) {
                                // lanes 16-31 address the second 16-byte chunk of the K step
                                const uint32_t at = base[i] + (2 * ks + (lane >> 4)) * pstride[i];
                                ldmatrix_x4(a_hi[i], at);
                                ldmatrix_x4(a_lo[i], at + PLANES * pstride[i]);
                            }
#pragma unroll
                            for (int nb = 0; nb < NBLK; ++nb) {
                                const int frag = (sl * KSTEPS + ks) * NBLK + nb;
                                uint32_t h0, h1, l0, l1;
                                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(h0), "=r"(h1) : "r"(frag_addr + frag * 256));
                                asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(l0), "=r"(l1) : "r"(frag_addr + (NFRAG + frag) * 256));
#pragma unroll
                                for (int i = I0; i < I1; ++i) {
                                    mma_16816(acc[i][nb], a_hi[i], h0, h1);
                                    mma_16816(acc[i][nb], a_hi[i], l0, l1);
                                    mma_16816(acc[i][nb], a_lo[i], h0, h1);
                                }
                            }
                        }
                    };
                    if (!__any_sync(0xffffffffu, any_miss)) { products(std::integral_constant<int, 0>{}, std::integral_constant<int, PAIR>{}); }
                    else {
                        // Some neighbour of this slot was not staged (more outside rows than halo slots): one tile at a time,
                        // its missing rows are fetched from global memory into the warp's scratch rows and addressed there.
                        auto one_tile = [&](auto which) {
                            constexpr int I = decltype(which)::value;
                            __syncwarp();
                            if (miss[I] && lane < 16) {
                                const int idx        = __ldg(a.nb + (r.nb_base + r.t0 + cur_row[I]) * a.n_neighbours + (sl - 1));
                                const size_t src_row = static_cast<size_t>(r.local_base + idx);
#pragma unroll
                                for (int pl = 0; pl < ALLP; ++pl) {
                                    *reinterpret_cast<uint4*>(scr_ptr + (pl * TILE + lane) * 16) = __ldg(in4 + static_cast<size_t>(pl) * a.in_stride + src_row);
                                }
                            }
                            __syncwarp();
                            if (miss[I]) {
                                base[I]    = scr_addr + (lane & 15) * 16;
                                pstride[I] = TILE * 16;
                            }
                            products(std::integral_constant<int, I>{}, std::integral_constant<int, I + 1>{});
                        };
                        one_tile(std::integral_constant<int, 0>{});
                        one_tile(std::integral_constant<int, 1>{});
                        static_assert(PAIR == 2, "the fallback above is written out for two tiles");
                    }
                }
                // ---- epilogue on the accumulator fragments: rows g and g + 8 of each tile, columns nb * 8 + 2 tq, + 1 ----
                bool bad = false;
#pragma unroll
                for (int i = 0; i < PAIR; ++i) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int row = r.t0 + (pair * PAIR + i) * TILE + g + 8 * half;  // within the frame
                        float v[NBLK][2];
#pragma unroll
                        for (int nb = 0; nb < NBLK; ++nb) {
                            v[nb][0] = acc[i][nb][2 * half];
                            v[nb][1] = acc[i][nb][2 * half + 1];
                            if (a.activation == VM_SELU) {
                                v[nb][0] = selu(v[nb][0]);
                                v[nb][1] = selu(v[nb][1]);
                            }
                            else if (a.activation == VM_RELU) {
                                v[nb][0] = v[nb][0] < 0.0f ? 0.0f : v[nb][0];
                                v[nb][1] = v[nb][1] < 0.0f ? 0.0f : v[nb][1];
                            }
                            else if (a.activation == VM_TANH) {
                                v[nb][0] = tanhf(v[nb][0]);
                                v[nb][1] = tanhf(v[nb][1]);
                            }
                        }
                        if (row >= r.rows) continue;
                        const size_t out_row = static_cast<size_t>(r.local_base) + row;
                        unsigned char* out_b = reinterpret_cast<unsigned char*>(a.out);
                        if (a.out_split) {
                            // column block nb is 16-byte chunk nb of the row's hi part (and of its lo part): this thread's two
                            // values are 4 bytes of it, the four threads of a row write the chunk, eight rows 128 contiguous bytes
#pragma unroll
                            for (int nb = 0; nb < NBLK; ++nb) {
                                uint32_t h, l;
                                split_pair(v[nb][0], v[nb][1], h, l);
                                bad |= fabsf(v[nb][0]) > 60000.0f || fabsf(v[nb][1]) > 60000.0f;
                                *reinterpret_cast<uint32_t*>(out_b + (static_cast<size_t>(nb) * a.out_stride + out_row) * 16 + tq * 4)        = h;
                                *reinterpret_cast<uint32_t*>(out_b + (static_cast<size_t>(NBLK + nb) * a.out_stride + out_row) * 16 + tq * 4) = l;
                            }
                        }
                        else {
                            // chunk-planar fp32: this thread's two values are half of 16-byte chunk 2 nb + tq / 2
#pragma unroll
                            for (int nb = 0; nb < NBLK; ++nb) {
                                *reinterpret_cast<float2*>(out_b + (static_cast<size_t>(2 * nb + (tq >> 1)) * a.out_stride + out_row) * 16 + (tq & 1) * 8) =
                                  make_float2(v[nb][0], v[nb][1]);
                            }
                        }
                    }
                }
                if (bad) atomicCAS(a.range_flag, 0, ABORT_RANGE);
            }
            // this warp is done with the window: the loader may refill it once every compute warp has said so
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar_empty + 8 * b);
        }
        }
        __syncthreads();
        if (tid == 0 && failed_s) atomicExch(t.abort_flag, tc::ABORT_TC_TIMEOUT);
    }

}  // namespace st
}  // namespace vm
