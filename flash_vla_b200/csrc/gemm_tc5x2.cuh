// Two-SM tcgen05 GEMMs: the gated FFN of the prefix encoder, out = gelu(A @ Wg) * (A @ Wu), and the
// residual projections out += A @ W (optionally with K split over several work items).
//
// A pair of CTAs (a cluster of 2) computes a 256-row x 128-column tile of `out` with
// tcgen05.mma.cta_group::2: one MMA of shape M = 256, N = 256, K = 16 whose first 128 B columns are
// gate columns held in the leader CTA's shared memory and whose last 128 are the matching up
// columns held in the peer's. Each CTA therefore stages only its own 128 rows of A (16 KB) and ONE
// 128-column weight tile (16 KB) per 64-wide k step - 32 KB per 512 tensor-core clocks, which is
// what the L2 -> SM path can deliver (about 64 B/clk/SM); the one-SM kernel needs 48 KB for the
// same work and is fill-bound. Each CTA ends up with gate and up accumulators for its own 128 rows
// in its own TMEM and runs the GeGLU epilogue on them. In the plain (residual) form the pair computes a
// 256 x 256 tile: the leader stages B columns [n0, n0+128), the peer [n0+128, n0+256).
//
// Synchronisation (all waits bounded, as in the one-SM kernel):
//   full[s]      in the leader only; the leader's producer expects the bytes of BOTH CTAs, and both
//                CTAs' TMA loads complete on it (cta_group::2 load with the leader's barrier address)
//   empty[s]     in both CTAs, released by the leader's tcgen05.commit multicast to both
//   accfull[a]   in both CTAs, same multicast commit after the last k step of a tile
//   accempty[a]  in the leader only, 16 arrivals: the 8 epilogue warps of each CTA
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "gemm_tc5.cuh"

namespace fvla {
namespace tc5x2 {

using namespace tc5;

constexpr int STAGES = 6;
constexpr int STAGE_BYTES = 32768;                 // A 128 x 64 + B 64 x 128, bf16
constexpr int EPI_WARPS = 8;
constexpr int EPI_STAGE_BYTES = 32 * 80;
constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + BAR_BYTES + EPI_WARPS * EPI_STAGE_BYTES;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;      // clears the CTA-rank bit: address in the leader CTA

__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t leader_bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {      // arrives on `bar` in both CTAs
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// kind::f16, fp32 accumulate, bf16 A (K-major) and B (MN-major), M = 256 over the CTA pair, N = 256.
__host__ __device__ constexpr uint32_t pair_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <bool DUAL>
__global__ void __launch_bounds__(320, 1)
tc5x2_gemm_kernel(const Tc5Args args, const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmG,
                   const __grid_constant__ CUtensorMap tmU) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bars = smem_base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + s * 8; };
    auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
    auto accfull_bar = [&](int a) { return bars + (2 * STAGES + a) * 8; };
    auto accempty_bar = [&](int a) { return bars + (2 * STAGES + 2 + a) * 8; };
    const uint32_t tmem_slot = bars + (2 * STAGES + 4) * 8;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const GemmArgs& p = args.g;
    constexpr int TILE_N = DUAL ? 128 : 256;                      // output columns of a pair tile
    const int num_tiles = args.tiles_m * args.tiles_n * args.splits;   // work items: (pair tile, k-split)
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), 2 * EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    // both CTAs' barriers exist before either side signals the other
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tmA);
            const CUtensorMap* tmB = (DUAL && rank == 1) ? &tmU : &tmG;
            prefetch_tensormap(tmB);
            // the B columns this CTA stages: gated form, both CTAs the same 128 (gate / up matrix); plain form, its half of 256
            auto b_col = [&](int t_idx) { return (t_idx / args.tiles_m) * TILE_N + (DUAL ? 0 : (int)rank * 128); };
            // Weights are never written inside a forward pass: the B halves of the first stages are requested
            // before waiting for the previous kernel, the A halves (its output) after.
            uint32_t early = 0;
            if (pair < num_tiles) {
                const int t_idx = pair / args.splits, split = pair % args.splits;
                const int n0 = b_col(t_idx);
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end && early < (uint32_t)STAGES; ++kt, ++early) {
                    if (rank == 0) mbar_expect_tx(full_bar(early), 2 * STAGE_BYTES);
                    const uint32_t sB = smem_base + early * STAGE_BYTES + 16384;
                    const uint32_t leader_full = full_bar(early) & kPeerBitMask;
                    tma_load_2d_pair(sB, tmB, leader_full, n0, kt * BK);
                    tma_load_2d_pair(sB + 8192, tmB, leader_full, n0 + 64, kt * BK);
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t it = 0;
            for (int tile = pair; tile < num_tiles; tile += pairs) {
                const int t_idx = tile / args.splits, split = tile % args.splits;
                const int m0 = (t_idx % args.tiles_m) * 256 + (int)rank * 128;
                const int n0 = b_col(t_idx);
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    const bool fresh = it >= early;               // stages below `early` already hold their B request
                    if (fresh) {
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) goto producer_done;
                        if (rank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);      // the bytes of both CTAs
                    }
                    const uint32_t sA = smem_base + s * STAGE_BYTES;
                    const uint32_t leader_full = full_bar(s) & kPeerBitMask;
                    tma_load_2d_pair(sA, &tmA, leader_full, kt * BK, m0);
                    if (fresh) {
                        tma_load_2d_pair(sA + 16384, tmB, leader_full, n0, kt * BK);
                        tma_load_2d_pair(sA + 16384 + 8192, tmB, leader_full, n0 + 64, kt * BK);
                    }
                }
            }
        }
    producer_done:;
        __syncwarp();
        if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // every thread of the CTA signals at the end of its role
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = pair_idesc();
            uint32_t it = 0, tcount = 0;
            for (int tile = pair; tile < num_tiles; tile += pairs, ++tcount) {
                const int acc = tcount & 1;
                const uint32_t acc_ph = (tcount >> 1) & 1u;
                if (!mbar_wait(accempty_bar(acc), acc_ph ^ 1u, abort_flag)) goto mma_done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * 256;
                const int split = tile % args.splits;
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag)) goto mma_done;
                    tc_fence_after();
                    const uint32_t sA = smem_base + s * STAGE_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint64_t adesc = smem_desc(sA + k16 * 32, 16, 1024);
                        const uint64_t bdesc = smem_desc(sA + 16384 + k16 * 2048, 8192, 1024);
                        umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kt > kt_beg || k16 > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar(s));
                }
                umma_commit_pair(accfull_bar(acc));
            }
        }
    mma_done:;
        __syncwarp();
        if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    } else {
        // 8 epilogue warps per CTA: warp w reads TMEM lanes [32 (w % 4), +32) and owns half of the tile's
        // output columns (64 in the gated form, 128 in the plain form), 32 at a time.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const int ew = warp - 2, quad = warp & 3, chalf = ew >> 2;
        constexpr int SPAN = TILE_N / 2, CHUNKS = SPAN / 32;
        uint8_t* stg = smem_gen + STAGES * STAGE_BYTES + BAR_BYTES + ew * EPI_STAGE_BYTES;
        const int sr = lane >> 2, sp = lane & 3;
        auto release_acc = [&](int acc) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                uint32_t leader_bar;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(leader_bar) : "r"(accempty_bar(acc)), "r"(0));
                mbar_arrive_cluster(leader_bar);
            }
        };
        uint32_t tcount = 0;
        for (int tile = pair; tile < num_tiles; tile += pairs, ++tcount) {
            const int acc = tcount & 1;
            const uint32_t acc_ph = (tcount >> 1) & 1u;
            const int t_idx = tile / args.splits, split = tile % args.splits;
            const int m0 = (t_idx % args.tiles_m) * 256 + (int)rank * 128, n0 = (t_idx / args.tiles_m) * TILE_N + chalf * SPAN;
            // the residual of this warp's rows, fetched (coalesced) while the MMAs still run
            uint4 rco[DUAL ? 1 : CHUNKS][4];
            if (!DUAL) {
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        rco[DUAL ? 0 : c][i] = make_uint4(0, 0, 0, 0);
                        const int grow = m0 + quad * 32 + sr + 8 * i, gcol = n0 + c * 32 + sp * 8;
                        if (p.R && !p.c_f32 && grow < p.M && gcol < p.N && (chalf * CHUNKS + c) % args.splits == split)
                            rco[DUAL ? 0 : c][i] = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.R) + (size_t)grow * p.ldr + gcol);
                    }
            }
            if (!mbar_wait(accfull_bar(acc), acc_ph, abort_flag)) break;
            if (tile + (int)pairs >= num_tiles) { if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }      // last accumulator complete
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * 256 + chalf * SPAN;
            bool from_partials = false;
            if (!DUAL && args.splits > 1) {
                // K split over `splits` work items of one tile. The 8 chunks (32 columns each) of this CTA's 128 rows
                // are shared out: chunk g is finished by the item whose split index is g % splits. An item publishes
                // the partial sums of the chunks it does NOT finish (layout [item][rank][column quad][row][4],
                // coalesced), announces itself on the tile's arrival counter, waits until all items of the tile
                // have done so (all of them are resident or will be: items run in index order and publish before
                // they wait), and then sums its own chunks in split order, taking its own addend from TMEM.
                int* arrive = args.counters + (t_idx * 2 + rank) * 2;
#pragma unroll 1
                for (int c = 0; c < CHUNKS; ++c) {
                    if ((chalf * CHUNKS + c) % args.splits == split) continue;
                    float a[32];
                    tmem_ld32(t_row + c * 32, a);
                    float* dst = args.partial + ((size_t)((t_idx * args.splits + split) * 2 + rank) * 64 + (chalf * CHUNKS + c) * 8) * 512 +
                                 (quad * 32 + lane) * 4;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        __stcg(reinterpret_cast<float4*>(dst + (j / 4) * 512), make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]));
                }
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
                int* flag = reinterpret_cast<int*>(smem_gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 12);
                if (ew == 0 && lane == 0) {
                    atomicAdd(arrive, 1);
                    int ok = 0;
                    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
                        int seen;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(arrive) : "memory");
                        if (seen >= args.splits) { ok = 1; break; }
                        if ((spin & 1023u) == 1023u && *abort_flag) break;
                    }
                    if (!ok) *abort_flag = 1;
                    *flag = ok;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
                const int all_here = *reinterpret_cast<volatile int*>(flag);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");   // flag may be rewritten by the next item
                if (!all_here) break;
                __threadfence();
                from_partials = true;
            }
#pragma unroll 1
            for (int c = 0; c < CHUNKS; ++c) {
                float a[32];
                if (from_partials) {
                    if ((chalf * CHUNKS + c) % args.splits != split) continue;      // another item of the tile finishes this chunk
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = 0.f;
                    for (int sp_i = 0; sp_i < args.splits; ++sp_i) {
                        if (sp_i == split) {
                            float own[32];
                            tmem_ld32(t_row + c * 32, own);
#pragma unroll
                            for (int j = 0; j < 32; ++j) a[j] += own[j];
                            continue;
                        }
                        const float* src = args.partial + ((size_t)((t_idx * args.splits + sp_i) * 2 + rank) * 64 + (chalf * CHUNKS + c) * 8) * 512 +
                                           (quad * 32 + lane) * 4;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (j / 4) * 512));
                            a[j] += v.x; a[j + 1] += v.y; a[j + 2] += v.z; a[j + 3] += v.w;
                        }
                    }
                } else {
                    tmem_ld32(t_row + c * 32, a);
                }
                if (!DUAL && p.bias) {
                    // bias of this chunk's 32 columns (the same for every row: broadcast loads)
                    const int col0 = n0 + c * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 8)
                        if (col0 + j + 8 <= p.N) {
                            const uint4 bv = __ldg(reinterpret_cast<const uint4*>(p.bias + col0 + j));
                            const float2 b0 = unpack_bf16x2(bv.x), b1 = unpack_bf16x2(bv.y), b2 = unpack_bf16x2(bv.z), b3 = unpack_bf16x2(bv.w);
                            a[j] += b0.x; a[j + 1] += b0.y; a[j + 2] += b1.x; a[j + 3] += b1.y;
                            a[j + 4] += b2.x; a[j + 5] += b2.y; a[j + 6] += b3.x; a[j + 7] += b3.y;
                        }
                }
                if (!DUAL && p.act == 1) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = gelu_f(a[j]);
                }
                if (!DUAL && p.c_f32) {
                    // fp32 destination (and fp32 residual, usually the destination itself): this thread owns 32
                    // consecutive floats of its row, 128 contiguous bytes, read and written as float4
                    const int grow = m0 + quad * 32 + lane, col0 = n0 + c * 32;
                    if (grow < p.M) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (col0 + j + 4 > p.N) break;
                            float4 v = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
                            if (p.R) {
                                const float4 r = *reinterpret_cast<const float4*>(static_cast<const float*>(p.R) + (size_t)grow * p.ldr + col0 + j);
                                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
                            }
                            *reinterpret_cast<float4*>(static_cast<float*>(p.C) + (size_t)grow * p.ldc + col0 + j) = v;
                        }
                    }
                    continue;
                }
                if (DUAL) {
                    float u[32];
                    tmem_ld32(t_row + 128 + c * 32, u);      // matching up columns
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = gelu_f(a[j]) * u[j];
                } else if (p.R) {
                    // hand each thread the residual of its own row (arrived as 8 rows x 64 B per request)
                    uint4 mine[4];
#pragma unroll
                    for (int cc = 0; cc < CHUNKS; ++cc)
                        if (cc == c) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) mine[i] = rco[DUAL ? 0 : cc][i];
                        }
#pragma unroll
                    for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(stg + (sr + 8 * i) * 80 + sp * 16) = mine[i];
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 r = *reinterpret_cast<const uint4*>(stg + lane * 80 + j * 16);
                        const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
                        a[8 * j] += r0.x; a[8 * j + 1] += r0.y; a[8 * j + 2] += r1.x; a[8 * j + 3] += r1.y;
                        a[8 * j + 4] += r2.x; a[8 * j + 5] += r2.y; a[8 * j + 6] += r3.x; a[8 * j + 7] += r3.y;
                    }
                    __syncwarp();
                }
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    *reinterpret_cast<uint4*>(stg + lane * 80 + j * 16) =
                        make_uint4(pack_bf16x2(a[8 * j], a[8 * j + 1]), pack_bf16x2(a[8 * j + 2], a[8 * j + 3]),
                                   pack_bf16x2(a[8 * j + 4], a[8 * j + 5]), pack_bf16x2(a[8 * j + 6], a[8 * j + 7]));
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int grow = m0 + quad * 32 + sr + 8 * i, gcol = n0 + c * 32 + sp * 8;
                    if (grow < p.M && gcol < p.N)
                        *reinterpret_cast<uint4*>(static_cast<bf16*>(p.C) + (size_t)grow * p.ldc + gcol) =
                            *reinterpret_cast<const uint4*>(stg + (sr + 8 * i) * 80 + sp * 16);
                }
                __syncwarp();
            }
            release_acc(acc);
            if (from_partials) {
                // the last item to leave the tile zeroes both counters for the next launch: by then every item has seen
                // the full arrival count
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");
                if (ew == 0 && lane == 0) {
                    int* arrive = args.counters + (t_idx * 2 + rank) * 2;
                    if (atomicAdd(arrive + 1, 1) == args.splits - 1) { arrive[1] = 0; arrive[0] = 0; __threadfence(); }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    // neither CTA may leave while the other can still signal its barriers or read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
    if (threadIdx.x == 0 && *abort_flag && args.status) atomicExch(args.status, 4);
}

struct PairPlan { bool ok; int splits; size_t ws_bytes; float est_us; };

// Plain residual GEMM on CTA pairs: 256 x 256 tiles; K is split so that the work items fill the 74 pairs.
inline PairPlan plan_pair_plain(int M, int N, int K, bool ws_ok) {
    PairPlan pl{false, 1, 0, 1e30f};
    if (M <= 128 || N % 8 || K % 8) return pl;
    const int tiles = ((M + 255) / 256) * ((N + 255) / 256), pairs = num_sms() / 2, k_iters = (K + BK - 1) / BK;
    for (int s = 1; s <= (ws_ok ? 6 : 1); ++s) {
        if (s > 1 && k_iters / s < 8) break;
        const int per = (k_iters + s - 1) / s;
        const int waves = (tiles * s + pairs - 1) / pairs;
        float t = waves * (per * 0.28f + 5.0f);
        if (s > 1) t += 3.0f + (float)s * M * N * 8.0f / 4.0e6f;
        if (t < pl.est_us) { pl.est_us = t; pl.splits = s; pl.ok = true; }
    }
    if (pl.splits > 1) pl.ws_bytes = (((size_t)tiles * 4 * sizeof(int) + 255) / 256) * 256 + (size_t)tiles * pl.splits * 2 * 128 * 256 * sizeof(float);
    return pl;
}

template <bool DUAL>
inline int launch_pair(const GemmArgs& g, int splits, void* ws, int* status, cudaStream_t st) {
    auto kern = tc5x2_gemm_kernel<DUAL>;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    CUtensorMap tmA, tmG, tmU;
    int rc = make_map(&tmA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, 128);
    if (rc) return rc;
    rc = make_map(&tmG, g.B, (uint64_t)g.N, (uint64_t)g.Kb, (uint64_t)g.ldb, 64, BK);
    if (rc) return rc;
    rc = make_map(&tmU, DUAL ? g.B2 : g.B, (uint64_t)g.N, (uint64_t)g.Kb, (uint64_t)g.ldb, 64, BK);
    if (rc) return rc;
    Tc5Args a{};
    a.g = g;
    a.tiles_m = (g.M + 255) / 256;
    a.tiles_n = DUAL ? g.N / 128 : (g.N + 255) / 256;
    a.k_iters = (g.K + BK - 1) / BK;
    a.splits = splits; a.k_per_split = (a.k_iters + splits - 1) / splits;
    if (splits > 1) {
        const size_t counters = (((size_t)a.tiles_m * a.tiles_n * 4 * sizeof(int) + 255) / 256) * 256;
        a.counters = reinterpret_cast<int*>(ws);
        a.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + counters);
    }
    a.status = status;
    const int items = a.tiles_m * a.tiles_n * splits;
    const int pairs = balanced_grid(items, num_sms() / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(320, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[3];
    int n_attr = 0;
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = 2; attr[n_attr].val.clusterDim.y = 1; attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
    // Nsight Compute reports a launch failure for this cooperative cluster launch: when the process runs under it (it
    // exports NV_COMPUTE_PROFILER_PERFWORKS_DIR), or with FVLA_COOP=0, the attribute is dropped; the waits stay bounded.
    static int coop = -1;
    if (coop < 0) {
        const char* v = getenv("FVLA_COOP");
        coop = v != nullptr ? (v[0] == '0' ? 0 : 1) : (getenv("NV_COMPUTE_PROFILER_PERFWORKS_DIR") != nullptr ? 0 : 1);
    }
    if (splits > 1 && coop) {
        // The items of a tile wait for one another (shared-out final sum): a cooperative launch makes the whole grid
        // resident at once, so no item can wait for a mate that another grid keeps off the SMs.
        attr[n_attr].id = cudaLaunchAttributeCooperative;
        attr[n_attr].val.cooperative = 1;
        ++n_attr;
    }
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, tmA, tmG, tmU);
    if (e != cudaSuccess) { set_error("tc5x2_gemm_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("tc5x2_gemm_kernel");
}

// Gated FFN with M > 128 rows, N a multiple of 128: returns FVLA_ERR_UNSUPPORTED otherwise.
inline int launch_geglu_pair(const GemmArgs& g, int* status, cudaStream_t st) {
    if (g.B2 == nullptr || g.N % 128 != 0 || g.M <= 128 || g.rope != nullptr || g.c_f32 || g.bias != nullptr || g.R != nullptr ||
        g.act != 0)
        return FVLA_ERR_UNSUPPORTED;
    return launch_pair<true>(g, 1, nullptr, status, st);
}

// What the plain form of the pair kernel can take: out = act(A @ W + bias) + residual, destination and residual
// both bf16 or both fp32, act none or GELU, no RoPE, no per-row scale, residual laid out like the destination.
inline bool pair_plain_supports(const GemmArgs& g) {
    return g.B2 == nullptr && g.rope == nullptr && (g.act == 0 || g.act == 1) && g.res_mod == 0 && g.row_scale == nullptr &&
           (!g.c_f32 || (g.N % 4 == 0 && g.ldc % 4 == 0 && aligned16(g.C))) &&
           (g.bias == nullptr || aligned16(g.bias)) && (g.R == nullptr || g.ldr == g.ldc) && g.M > 128 && g.N % 8 == 0 && g.K % 8 == 0;
}

// FVLA_ERR_UNSUPPORTED when the epilogue is outside `pair_plain_supports`.
inline int launch_plain_pair(const GemmArgs& g, void* ws, size_t ws_bytes, int* status, cudaStream_t st) {
    if (!pair_plain_supports(g)) return FVLA_ERR_UNSUPPORTED;
    PairPlan pl = plan_pair_plain(g.M, g.N, g.K, ws != nullptr);
    if (pl.ok && pl.splits > 1 && ws_bytes < pl.ws_bytes) pl = plan_pair_plain(g.M, g.N, g.K, false);
    if (!pl.ok) return FVLA_ERR_UNSUPPORTED;
    return launch_pair<false>(g, pl.splits, ws, status, st);
}

// Scratch bytes of the pair kernel's K split.
inline size_t pair_split_bytes(int M, int N, int splits) {
    const size_t tiles = (size_t)((M + 255) / 256) * ((N + 255) / 256);
    return splits > 1 ? ((tiles * 4 * sizeof(int) + 255) / 256) * 256 + tiles * splits * 2 * 128 * 256 * sizeof(float) : 0;
}

// A pinned K split (1..6) for the plain form of the pair kernel; errors out when it cannot be honoured.
inline int launch_plain_pair_pinned(const GemmArgs& g, int splits, void* ws, size_t ws_bytes, int* status, cudaStream_t st) {
    if (!pair_plain_supports(g)) {
        set_error("pinned plan: the pair kernel's plain form takes bias, GELU and a residual of the destination's type only");
        return FVLA_ERR_UNSUPPORTED;
    }
    const int k_iters = (g.K + BK - 1) / BK;
    if (splits < 1 || splits > 6 || (splits > 1 && k_iters / splits < 2)) { set_error("pinned plan: pair split %d", splits); return FVLA_ERR_UNSUPPORTED; }
    if (splits > 1 && (ws == nullptr || ws_bytes < pair_split_bytes(g.M, g.N, splits))) {
        set_error("pinned plan: scratch of %zu bytes needed", pair_split_bytes(g.M, g.N, splits));
        return FVLA_ERR_WORKSPACE;
    }
    return launch_pair<false>(g, splits, ws, status, st);
}

}  // namespace tc5x2
}  // namespace fvla
