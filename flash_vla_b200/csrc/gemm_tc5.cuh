// Blackwell-native bf16 GEMM: TMA -> shared memory -> tcgen05.mma -> TMEM -> fused epilogue.
//
//   C[M,N] = epilogue(A[M,K] @ B[K,N])   (optionally two B operands: gated FFN)
//
// A is row-major with K contiguous ("K-major" operand); B is the checkpoint's (K, N) layout with
// N contiguous, consumed in place as an "MN-major" operand, so no weight is ever re-packed.
// One CTA computes 128 x BN output tiles in a persistent loop. Warp roles:
//   warp 0     TMA producer: 128B-swizzled boxes of A (64 k x 128 rows) and B (64 n x 64 k rows)
//              into a STAGES-deep ring, completion counted on mbarriers.
//   warp 1     allocates TMEM; one elected lane issues tcgen05.mma (M=128, N=BN, K=16, fp32
//              accumulate) and commits ring slots / accumulator stages back through mbarriers.
//   warps 2-5  epilogue: tcgen05.ld of the accumulator (one TMEM lane = one output row per
//              thread), bias / GELU / GeGLU / residual / RoPE+scatter in fp32, bf16 stores.
// Accumulators are double-buffered in TMEM, so the epilogue of tile i overlaps the MMAs of
// tile i+1. Every wait is bounded: when a limit is hit the kernel records a code in `status`
// and every role leaves its loop; TMEM is released on all paths.
#pragma once

#include <cuda.h>

#include <cstdio>

#include "common.cuh"
#include "gemm_mma.cuh"

namespace fvla {
namespace tc5 {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait; false when the limit ran out (the caller then abandons its loop). `limit` is the number
// of polls; the default is far beyond any legitimate wait of these kernels (tens of microseconds).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = kSpinLimit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; kind::f16 covers bf16 inputs with fp32 accumulation.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets
// (all >> 4), version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;            // descriptor version for tcgen05
    d |= (uint64_t)2 << 61;            // SWIZZLE_128B
    return d;
}
// Instruction descriptor for kind::f16: fp32 accumulator, bf16 A (K-major) and B (MN-major).
__host__ __device__ constexpr uint32_t instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(BM >> 4) << 24);
}

struct Tc5Args {
    GemmArgs g;                // epilogue description, shapes, C / R / bias / rope pointers
    int tiles_m, tiles_n, k_iters;
    int splits, k_per_split;   // K split over `splits` work items per tile (k_per_split 64-wide steps each)
    float* partial;            // [tile][split][BN/4 column quads][128 rows][4] fp32 partial products (splits > 1)
    int* counters;             // one self-resetting arrival counter per tile (splits > 1)
    int* status;               // device word: set non-zero when a bounded wait ran out
    FVLA_DBG_MEMBER
};

// Epilogue for 8 adjacent columns of one row (a: first / gate accumulator, u: up accumulator).
// `rpre`: the bf16 residual of these 8 columns, loaded by the caller before any store of the tile
// (the residual may alias the destination, so loads issued after a store would each wait for it).
template <bool DUAL>
__device__ __forceinline__ void epilogue8(const GemmArgs& p, int row, int col, float (&a)[8], const float (&u)[8],
                                          uint4 rpre, bool use_pre) {
    if (DUAL) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = gelu_f(a[i]) * u[i];
    }
    if (p.bias_f32) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += __ldg(p.bias_f32 + col + i);
    } else if (p.bias) {
        uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
        float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y), b2 = unpack_bf16x2(b.z), b3 = unpack_bf16x2(b.w);
        a[0] += b0.x; a[1] += b0.y; a[2] += b1.x; a[3] += b1.y; a[4] += b2.x; a[5] += b2.y; a[6] += b3.x; a[7] += b3.y;
    }
    if (p.act == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = gelu_f(a[i]);
    } else if (p.act == 2) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = silu_f(a[i]);
    }
    if (p.R) {
        int rr = p.res_mod > 0 ? row % p.res_mod : row;
        if (p.c_f32) {
            const float4* r = reinterpret_cast<const float4*>(static_cast<const float*>(p.R) + (size_t)rr * p.ldr + col);
            float4 r0 = r[0], r1 = r[1];
            a[0] += r0.x; a[1] += r0.y; a[2] += r0.z; a[3] += r0.w; a[4] += r1.x; a[5] += r1.y; a[6] += r1.z; a[7] += r1.w;
        } else {
            uint4 r = use_pre ? rpre : *reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.R) + (size_t)rr * p.ldr + col);
            float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
            a[0] += r0.x; a[1] += r0.y; a[2] += r1.x; a[3] += r1.y; a[4] += r2.x; a[5] += r2.y; a[6] += r3.x; a[7] += r3.y;
        }
    }
    bf16* dst;
    if (p.rope) {
        const int hd = p.head_dim, qd = p.heads * hd;
        if (col < qd + hd) {
            uint4 cs = __ldg(reinterpret_cast<const uint4*>(p.rope + (size_t)rope_row(p, row) * hd + (col % hd)));
            const uint32_t csw[4] = {cs.x, cs.y, cs.z, cs.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float x0 = a[2 * i], x1 = a[2 * i + 1];
                if (p.round_first) { x0 = round_bf16(x0); x1 = round_bf16(x1); }
                float2 c = unpack_bf16x2(csw[i]);
                a[2 * i] = x0 * c.x - x1 * c.y;
                a[2 * i + 1] = x1 * c.x + x0 * c.y;
            }
            dst = col < qd ? p.q + (size_t)row * qd + col : p.k + kv_row(p, row) * hd + (col - qd);
        } else {
            dst = p.v + kv_row(p, row) * hd + (col - qd - hd);
        }
    } else if (p.c_f32) {
        float4* d = reinterpret_cast<float4*>(static_cast<float*>(p.C) + (size_t)row * p.ldc + col);
        d[0] = make_float4(a[0], a[1], a[2], a[3]);
        d[1] = make_float4(a[4], a[5], a[6], a[7]);
        return;
    } else {
        dst = static_cast<bf16*>(p.C) + (size_t)row * p.ldc + col;
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]),
                                                pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
}

template <int BN, bool DUAL, int STAGES>
struct Tc5Cfg {
    static constexpr int NB = DUAL ? 2 : 1;
    static constexpr int A_BYTES = BM * BK * 2;                 // 16 KB: 128 rows x 128 B
    static constexpr int SLAB = BK * 128;                       // 8 KB: 64 k-rows x (64 n = 128 B)
    static constexpr int B_BYTES = (BN / 64) * SLAB;
    static constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
    static constexpr int ACC_COLS = NB * BN;                    // TMEM columns per accumulator stage
    static constexpr int TMEM_COLS = 2 * ACC_COLS <= 32 ? 32 : (2 * ACC_COLS <= 64 ? 64 : (2 * ACC_COLS <= 128 ? 128 : (2 * ACC_COLS <= 256 ? 256 : 512)));
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16 + 16;     // pipeline barriers, TMEM slot / flags, cluster split-K barriers
    static constexpr int EPI_WARPS = 8;                         // two warps per TMEM lane quadrant, half the columns each
    static constexpr int EPI_STAGE_BYTES = 32 * 80;             // per warp: 32 rows x (64 B + 16 B pad)
    static constexpr int THREADS = 64 + 32 * EPI_WARPS;
    static constexpr int NORM_BYTES = 2 * BM * 2 * 4;           // fused row norm: (sum, sum of squares) of each row from each of its two threads
    static constexpr int COLC_BYTES = 2 * 2 * BN * 4;           // per-column epilogue constants (bias, column sums) as fp32, one set per accumulator stage
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + BAR_BYTES + EPI_WARPS * EPI_STAGE_BYTES + NORM_BYTES + COLC_BYTES;
    static_assert(2 * ACC_COLS <= 512, "two accumulator stages must fit in TMEM");
    static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");
    static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "BN");
};

// ROPE: the staged (coalesced) epilogue also handles the RoPE + Q/K/V scatter form; without it that form
// takes the per-row path. A template switch so that the other instantiations do not carry its registers.
// CLUSTER: split-K inside a thread-block cluster. The `splits` CTAs of a tile are cluster mates; the ones
// with split > 0 stage their fp32 partial tile in their own (by then idle) pipeline shared memory and push
// it with one bulk copy into the idle pipeline memory of the split-0 CTA, which adds the partials in
// split order and runs the epilogue. No global scratch, no semaphore; needs one work item per CTA.
// NORM: the row norm of A is folded in (GemmArgs::norm_mode): the epilogue warps also consume every operand stage,
// so a stage returns to the producer after the MMAs AND the eight epilogue warps have read it. Meant for one tile
// per CTA; with more, a tile's statistics wait for the previous tile's epilogue (correct, but the overlap is lost).
template <int BN, bool DUAL, int STAGES, bool ROPE = false, bool CLUSTER = false, bool NORM = false>
__global__ void __launch_bounds__(320, 1)
tc5_gemm_kernel(const Tc5Args args, const __grid_constant__ CUtensorMap tmA,
                const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmB2) {
    using Cfg = Tc5Cfg<BN, DUAL, STAGES>;
    constexpr int NB = Cfg::NB;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = smem_base + STAGES * Cfg::STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + s * 8; };
    auto empty_bar = [&](int s) { return bars + (STAGES + s) * 8; };
    auto accfull_bar = [&](int a) { return bars + (2 * STAGES + a) * 8; };
    auto accempty_bar = [&](int a) { return bars + (2 * STAGES + 2 + a) * 8; };
    const uint32_t tmem_slot = bars + (2 * STAGES + 4) * 8;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_gen + STAGES * Cfg::STAGE_BYTES + (2 * STAGES + 4) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + STAGES * Cfg::STAGE_BYTES + (2 * STAGES + 4) * 8 + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const GemmArgs& p = args.g;
    const int num_tiles = args.tiles_m * args.tiles_n * args.splits;      // work items: (tile, k-split)
    FVLA_DBG_CTA(args, blockIdx.x);
    if (threadIdx.x == 0) FVLA_STAMP_ANY(0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), NORM ? 1 + Cfg::EPI_WARPS : 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(accfull_bar(a), 1); mbar_init(accempty_bar(a), Cfg::EPI_WARPS); }
        mbar_init(bars + (2 * STAGES + 4) * 8 + 16, 1);          // cluster split-K: "the leader's pipeline memory is free"
        mbar_init(bars + (2 * STAGES + 4) * 8 + 24, 1);          // cluster split-K: "the peers' partial tiles have arrived"
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    // cluster split-K: tell the cluster mates that this CTA's barriers exist (the fence after their
    // initialisation already published them; the matching wait sits where the first remote access is)
    if (CLUSTER) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    // Set-up above touched only this CTA's own shared memory and TMEM.
    if (threadIdx.x == 0) FVLA_STAMP_ANY(1);

    if (warp == 0) {
        if (lane == 0) {
            prefetch_tensormap(&tmA);
            prefetch_tensormap(&tmB);
            if (DUAL) prefetch_tensormap(&tmB2);
            auto load_b = [&](int s, int n0, int kt) {
                const uint32_t sB = smem_base + s * Cfg::STAGE_BYTES + Cfg::A_BYTES;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_2d(sB + nb * Cfg::B_BYTES + j * Cfg::SLAB, nb == 0 ? &tmB : &tmB2, full_bar(s), n0 + j * 64, kt * BK);
            };
            // Weights are never written inside a forward pass, so the B halves of the first stages are
            // requested before waiting for the previous kernel; the A halves (its output) follow the wait.
            uint32_t early = 0;
            if ((int)blockIdx.x < num_tiles) {
                const int t_idx = blockIdx.x / args.splits, split = blockIdx.x % args.splits;
                const int n0 = (t_idx / args.tiles_m) * BN;
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end && early < (uint32_t)STAGES; ++kt, ++early) {
                    mbar_expect_tx(full_bar(early), Cfg::STAGE_BYTES);
                    load_b(early, n0, kt);
                }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
                const int t_idx = tile / args.splits, split = tile % args.splits;
                const int m0 = (t_idx % args.tiles_m) * BM, n0 = (t_idx / args.tiles_m) * BN;
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    const bool fresh = it >= early;               // stages below `early` already hold their B request
                    if (fresh) {
                        if (!mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) goto producer_done;
                        mbar_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
                    }
                    tma_load_2d(smem_base + s * Cfg::STAGE_BYTES, &tmA, full_bar(s), kt * BK, m0);
                    if (fresh) load_b(s, n0, kt);
                }
            }
        }
    producer_done:;
        __syncwarp();
        if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // every thread of the CTA signals at the end of its role
    } else if (warp == 1) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BN);
            uint32_t it = 0, tcount = 0;
            for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
                const int acc = tcount & 1;
                const uint32_t acc_ph = (tcount >> 1) & 1u;
                if (!mbar_wait(accempty_bar(acc), acc_ph ^ 1u, abort_flag)) goto mma_done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_COLS;
                const int split = tile % args.splits;
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                for (int kt = kt_beg; kt < kt_end; ++kt, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag)) goto mma_done;
                    tc_fence_after();
                    if (it == 0) FVLA_STAMP_ANY(2);
                    const uint32_t sA = smem_base + s * Cfg::STAGE_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        const uint64_t adesc = smem_desc(sA + k16 * 32, 16, 1024);
#pragma unroll
                        for (int nb = 0; nb < NB; ++nb) {
                            const uint64_t bdesc = smem_desc(sA + Cfg::A_BYTES + nb * Cfg::B_BYTES + k16 * 2048, Cfg::SLAB, 1024);
                            umma_bf16(d_tmem + nb * BN, adesc, bdesc, idesc, (kt > kt_beg || k16 > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(empty_bar(s));              // slot reusable once these MMAs have read it
                }
                umma_commit(accfull_bar(acc));              // accumulator complete
                if (tcount == 0) FVLA_STAMP_ANY(3);
            }
        }
    mma_done:;
        __syncwarp();
        if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    } else {
        // Eight epilogue warps: warp w reads TMEM lanes [32 (w % 4), +32) and owns one half of the
        // tile's columns. One thread = one output row; results go through a small per-warp staging
        // area so that global loads and stores touch 64 contiguous bytes per row (8 rows per request)
        // instead of 16 bytes in each of 32 rows.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (CLUSTER) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const int ew = warp - 2, quad = warp & 3, whalf = ew >> 2;
        constexpr int HALF = BN / 2, CHUNKS = HALF / 32;
        uint8_t* stg = smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES + ew * Cfg::EPI_STAGE_BYTES;
        // staged path: bf16 destination(s); the preloaded operand is the bf16 residual or, for the RoPE +
        // scatter epilogue, the cos/sin entries of the chunk (one or the other)
        const bool plain = !p.c_f32 && (ROPE ? !(p.R != nullptr || p.bias != nullptr || p.act != 0) : p.rope == nullptr);
        const int rope_qd = p.heads * p.head_dim;            // RoPE epilogue: columns [0, qd) are Q, then K, then V
        const int sr = lane >> 2, sp = lane & 3;              // staged access: row sr + 8 i, 16-byte piece sp
        uint32_t tcount = 0;
        uint32_t nit = 0;                                     // fused row norm: stages consumed so far
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
            const int acc = tcount & 1;
            const uint32_t acc_ph = (tcount >> 1) & 1u;
            const int t_idx = tile / args.splits, split = tile % args.splits;
            // Two cluster mates that split K between them share the epilogue as well: each finishes the column half
            // of its own rank (after receiving the other's partial sums for it), and inside that half the warp's
            // `whalf` picks one of the two 32-column chunks. In every other case `whalf` picks the column half.
            const bool sym = CLUSTER && CHUNKS == 2 && args.splits == 2;
            const int chalf = sym ? split : whalf;
            const int m0 = (t_idx % args.tiles_m) * BM, n0 = (t_idx / args.tiles_m) * BN + chalf * HALF;
            const int row = m0 + quad * 32 + lane;
            // operands that do not depend on the accumulator, fetched while the MMAs still run
            // Per-column constants of this tile (bias; column sums for the folded LayerNorm) go to shared memory
            // as fp32, one column per thread; the chunk loop reads them back as broadcast 16-byte loads. Two sets,
            // alternating with the accumulator stage, so a warp that runs ahead never overwrites values in use.
            const bool has_bias = p.bias != nullptr || p.bias_f32 != nullptr;
            float* colc = reinterpret_cast<float*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES + Cfg::EPI_WARPS * Cfg::EPI_STAGE_BYTES + Cfg::NORM_BYTES) + acc * 2 * BN;
            {
                const int t = (int)threadIdx.x - 64, col = (t_idx / args.tiles_m) * BN + t;
                if (t < BN && (has_bias || NORM)) {
                    float bv = 0.f, cv = 0.f;
                    if (col < p.N) {
                        bv = p.bias_f32 ? __ldg(p.bias_f32 + col) : (p.bias ? __bfloat162float(__ldg(p.bias + col)) : 0.f);
                        if (NORM && p.colsum) cv = __ldg(p.colsum + col);
                    }
                    colc[t] = bv;
                    if (NORM) colc[BN + t] = cv;
                }
            }
            uint4 rco[CHUNKS][4];
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    rco[c][i] = make_uint4(0, 0, 0, 0);
                    if (sym && c != whalf) continue;
                    const int grow = m0 + quad * 32 + sr + 8 * i, gcol = n0 + c * 32 + sp * 8;
                    if (ROPE && plain && p.rope) {
                        if (grow < p.M && gcol < rope_qd + p.head_dim)
                            rco[c][i] = __ldg(reinterpret_cast<const uint4*>(p.rope + (size_t)rope_row(p, grow) * p.head_dim + (gcol % p.head_dim)));
                    } else if (plain && p.R && grow < p.M && gcol < p.N) {
                        const int rr = p.res_mod > 0 ? grow % p.res_mod : grow;
                        rco[c][i] = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.R) + (size_t)rr * p.ldr + gcol);
                    }
                }
            }
            float nrm_mean = 0.f, nrm_rstd = 1.f;
            if (NORM) {
                // This thread adds up half of its row: four of the eight 16-byte pieces of each 128-byte operand
                // row. Sums do not depend on the order of the pieces, so the 128-byte swizzle needs no undoing;
                // the piece index rotates with the lane so that a quarter warp touches eight different bank groups.
                float s1 = 0.f, s2 = 0.f;
                const int kt_beg = split * args.k_per_split, kt_end = min(args.k_iters, kt_beg + args.k_per_split);
                bool alive = true;
                for (int kt = kt_beg; kt < kt_end; ++kt, ++nit) {
                    const int s = nit % STAGES;
                    const uint32_t ph = (nit / STAGES) & 1u;
                    if (!mbar_wait(full_bar(s), ph, abort_flag)) { alive = false; break; }
                    const uint8_t* arow = smem_gen + s * Cfg::STAGE_BYTES + (quad * 32 + lane) * 128;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 v = *reinterpret_cast<const uint4*>(arow + (((lane + 2 * j + whalf) & 7) << 4));
                        const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y), f2 = unpack_bf16x2(v.z), f3 = unpack_bf16x2(v.w);
                        s1 += (f0.x + f0.y) + (f1.x + f1.y) + (f2.x + f2.y) + (f3.x + f3.y);
                        s2 += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar(s));      // this warp has read the stage
                }
                if (!alive) break;
                float2* nstat = reinterpret_cast<float2*>(smem_gen + STAGES * Cfg::STAGE_BYTES + Cfg::BAR_BYTES + Cfg::EPI_WARPS * Cfg::EPI_STAGE_BYTES);
                nstat[whalf * BM + quad * 32 + lane] = make_float2(s1, s2);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");
                const float2 other = nstat[(whalf ^ 1) * BM + quad * 32 + lane];
                // both threads of a row add the two halves in the same order
                const float t1 = whalf == 0 ? s1 + other.x : other.x + s1, t2 = whalf == 0 ? s2 + other.y : other.y + s2;
                const float invk = 1.f / (float)p.K;
                if (p.norm_mode == 2) {
                    nrm_mean = t1 * invk;
                    nrm_rstd = rsqrtf(t2 * invk - nrm_mean * nrm_mean + 1e-5f);
                } else {
                    nrm_rstd = rsqrtf(t2 * invk + 1e-6f);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");      // the statistics area may be rewritten for the next tile
            } else if (has_bias) {
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");      // the column constants are in place
            }
            if (!mbar_wait(accfull_bar(acc), acc_ph, abort_flag)) break;
            if (tile + (int)gridDim.x >= num_tiles) { if (p.trigger_early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }      // last accumulator complete
            tc_fence_after();
            if (tcount == 0 && threadIdx.x == 64) FVLA_STAMP_ANY(4);
            const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * Cfg::ACC_COLS + chalf * HALF;
            bool from_partials = false;
            bool from_cluster = false;
            if (CLUSTER && args.splits > 1) {
                const uint32_t free_bar = bars + (2 * STAGES + 4) * 8 + 16, red_bar = bars + (2 * STAGES + 4) * 8 + 24;
                constexpr uint32_t TILE_BYTES = BM * BN * 4;
                if (sym) {
                    // Reduce-scatter between the two mates. This CTA's pipeline memory is idle (its MMAs are done):
                    // [0, 32 KB) stages the partial sums of the MATE's column half as [column quad][row][4],
                    // [32 KB, 64 KB) receives the mate's partial sums of THIS CTA's half in the same layout.
                    constexpr uint32_t HALF_BYTES = BM * HALF * 4;
                    if (ew == 0 && lane == 0) {
                        mbar_expect_tx(red_bar, HALF_BYTES);
                        uint32_t fb;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(fb) : "r"(free_bar), "r"(split ^ 1));
                        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(fb) : "memory");      // "send when ready"
                    }
                    {
                        float a[32];
                        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * Cfg::ACC_COLS + (split ^ 1) * HALF + whalf * 32, a);
                        float* dst = reinterpret_cast<float*>(smem_gen) + (whalf * 8) * (BM * 4) + (quad * 32 + lane) * 4;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(dst + (j / 4) * (BM * 4)) = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // staged half -> visible to the bulk copy
                    asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");
                    if (ew == 0 && lane == 0) {
                        if (mbar_wait(free_bar, 0, abort_flag)) {      // the mate's pipeline memory is idle
                            uint32_t dst0, rbar;
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst0) : "r"(smem_base + HALF_BYTES), "r"(split ^ 1));
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(red_bar), "r"(split ^ 1));
#pragma unroll
                            for (uint32_t off = 0; off < HALF_BYTES; off += 16384)
                                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                             ::"r"(dst0 + off), "r"(smem_base + off), "r"(16384), "r"(rbar) : "memory");
                        }
                    }
                    mbar_wait(red_bar, 0, abort_flag);      // a wait that gives up sets the abort flag; the sums are then garbage and reported
                } else if (split > 0) {
                    // stage the partial tile as [column quad][row][4] in this CTA's idle pipeline memory, then push it
#pragma unroll
                    for (int c = 0; c < CHUNKS; ++c) {
                        float a[32];
                        tmem_ld32(t_row + c * 32, a);
                        float* dst = reinterpret_cast<float*>(smem_gen) + ((chalf * CHUNKS + c) * 8) * (BM * 4) + (quad * 32 + lane) * 4;
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(dst + (j / 4) * (BM * 4)) = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
                    }
                    tc_fence_before();
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // staged tile -> visible to the bulk copy
                    asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");
                    if (ew == 0 && lane == 0) {
                        mbar_arrive(accempty_bar(acc));
                        if (mbar_wait(free_bar, 0, abort_flag)) {      // the leader's pipeline memory is idle
                            uint32_t dst0, rbar;
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst0) : "r"(smem_base + (uint32_t)(split - 1) * TILE_BYTES), "r"(0));
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(red_bar), "r"(0));
#pragma unroll
                            for (uint32_t off = 0; off < TILE_BYTES; off += 16384)
                                asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                             ::"r"(dst0 + off), "r"(smem_base + off), "r"(16384), "r"(rbar) : "memory");
                        }
                    }
                    continue;
                }
                if (!sym && ew == 0 && lane == 0) {
                    mbar_expect_tx(red_bar, (uint32_t)(args.splits - 1) * TILE_BYTES);
                    for (int sp_i = 1; sp_i < args.splits; ++sp_i) {
                        uint32_t fb;
                        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(fb) : "r"(free_bar), "r"(sp_i));
                        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(fb) : "memory");
                    }
                }
                if (!sym) mbar_wait(red_bar, 0, abort_flag);      // a wait that gives up sets the abort flag; the sums are then garbage and reported
                from_cluster = true;
            }
            if (!CLUSTER && !DUAL && args.splits > 1) {
                // Publish this item's partial tile, then let the last-arriving item of the tile sum all
                // of them (in split order, so the result does not depend on arrival order) and finish.
#pragma unroll
                for (int c = 0; c < CHUNKS; ++c) {
                    float a[32];
                    tmem_ld32(t_row + c * 32, a);
                    // Partials use a tile-private layout [item][column quad][row][4] so that the 32 rows of a
                    // warp write (and later read) 512 contiguous bytes per request.
                    float* dst = args.partial + ((size_t)(t_idx * args.splits + split) * (BN / 4) + (chalf * CHUNKS + c) * 8) * (BM * 4) +
                                 (quad * 32 + lane) * 4;
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        __stcg(reinterpret_cast<float4*>(dst + (j / 4) * (BM * 4)), make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(accempty_bar(acc));          // the accumulator stage is free again
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");
                int* flag = reinterpret_cast<int*>(smem_gen + STAGES * Cfg::STAGE_BYTES + (2 * STAGES + 4) * 8 + 12);
                if (ew == 0 && lane == 0) {
                    const int prev = atomicAdd(args.counters + t_idx, 1);
                    const int last = prev == args.splits - 1;
                    if (last) args.counters[t_idx] = 0;                  // self-reset: the graph replays this kernel
                    *flag = last;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");
                const int last = *reinterpret_cast<volatile int*>(flag);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * Cfg::EPI_WARPS) : "memory");   // flag may be rewritten by the next item
                if (!last) continue;
                __threadfence();
                from_partials = true;
            }
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                float a[32], u[32];
                if (sym && c != whalf) continue;
                if (from_partials) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) a[j] = 0.f;
                    for (int sp_i = 0; sp_i < args.splits; ++sp_i) {
                        const float* src = args.partial + ((size_t)(t_idx * args.splits + sp_i) * (BN / 4) + (chalf * CHUNKS + c) * 8) * (BM * 4) +
                                           (quad * 32 + lane) * 4;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (j / 4) * (BM * 4)));
                            a[j] += v.x; a[j + 1] += v.y; a[j + 2] += v.z; a[j + 3] += v.w;
                        }
                    }
                } else {
                    tmem_ld32(t_row + c * 32, a);
                    if (DUAL) tmem_ld32(t_row + BN + c * 32, u);
                }
                if (CLUSTER && from_cluster && sym) {
                    // the mate's partial sums of this chunk (two addends: the order does not matter)
                    const float* src = reinterpret_cast<const float*>(smem_gen + BM * HALF * 4) + (c * 8) * (BM * 4) + (quad * 32 + lane) * 4;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(src + (j / 4) * (BM * 4));
                        a[j] += v.x; a[j + 1] += v.y; a[j + 2] += v.z; a[j + 3] += v.w;
                    }
                } else if (CLUSTER && from_cluster) {
                    // split 0 is this CTA's own accumulator; the others arrived in split order
                    for (int sp_i = 1; sp_i < args.splits; ++sp_i) {
                        const float* src = reinterpret_cast<const float*>(smem_gen + (size_t)(sp_i - 1) * (BM * BN * 4)) +
                                           ((chalf * CHUNKS + c) * 8) * (BM * 4) + (quad * 32 + lane) * 4;
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 v = *reinterpret_cast<const float4*>(src + (j / 4) * (BM * 4));
                            a[j] += v.x; a[j + 1] += v.y; a[j + 2] += v.z; a[j + 3] += v.w;
                        }
                    }
                }
                if (plain) {
                    float res[32];
                    if (p.R || (ROPE && p.rope)) {
                        // residual arrives coalesced (8 rows x 64 B per request); hand each thread its own row
#pragma unroll
                        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(stg + (sr + 8 * i) * 80 + sp * 16) = rco[c][i];
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint4 r = *reinterpret_cast<const uint4*>(stg + lane * 80 + j * 16);
                            const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y), r2 = unpack_bf16x2(r.z), r3 = unpack_bf16x2(r.w);
                            res[8 * j] = r0.x; res[8 * j + 1] = r0.y; res[8 * j + 2] = r1.x; res[8 * j + 3] = r1.y;
                            res[8 * j + 4] = r2.x; res[8 * j + 5] = r2.y; res[8 * j + 6] = r3.x; res[8 * j + 7] = r3.y;
                        }
                        __syncwarp();
                    }
                    // the activation is chosen once per chunk, outside the element loop: inside it the compiler
                    // evaluates every branch for every element and selects
                    const float* colc_chunk = colc + chalf * HALF + c * 32;
                    if (NORM) {
                        // the norm of this thread's row, applied to the raw product
                        if (p.norm_mode == 2) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 cs = *reinterpret_cast<const float4*>(colc_chunk + BN + j);
                                a[j] = nrm_rstd * (a[j] - nrm_mean * cs.x); a[j + 1] = nrm_rstd * (a[j + 1] - nrm_mean * cs.y);
                                a[j + 2] = nrm_rstd * (a[j + 2] - nrm_mean * cs.z); a[j + 3] = nrm_rstd * (a[j + 3] - nrm_mean * cs.w);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) a[j] *= nrm_rstd;
                        }
                    }
                    auto finish = [&](auto act) {
                        if (DUAL) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) a[j] = gelu_f(a[j]) * u[j];
                        }
                        if (has_bias) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                const float4 b4 = *reinterpret_cast<const float4*>(colc_chunk + j);
                                a[j] += b4.x; a[j + 1] += b4.y; a[j + 2] += b4.z; a[j + 3] += b4.w;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float v = act(a[j]);
                            a[j] = p.R ? v + res[j] : v;
                        }
                    };
                    const int col0 = n0 + c * 32;                  // first column of this chunk
                    bf16* out_base = static_cast<bf16*>(p.C);
                    int out_ld = p.ldc, out_col = col0;
                    bool kv_dst = false;                           // K / V destination: rows follow the sequence-group mapping
                    if (ROPE && p.rope) {
                        // res[] holds this row's 16 (cos, sin) pairs for the chunk's 16 column pairs
                        if (col0 < rope_qd + p.head_dim) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                float x0 = a[2 * i], x1 = a[2 * i + 1];
                                if (p.round_first) { x0 = round_bf16(x0); x1 = round_bf16(x1); }
                                a[2 * i] = x0 * res[2 * i] - x1 * res[2 * i + 1];
                                a[2 * i + 1] = x1 * res[2 * i] + x0 * res[2 * i + 1];
                            }
                        }
                        if (col0 < rope_qd) { out_base = p.q; out_ld = rope_qd; }
                        else if (col0 < rope_qd + p.head_dim) { out_base = p.k; out_ld = p.head_dim; out_col = col0 - rope_qd; kv_dst = true; }
                        else { out_base = p.v; out_ld = p.head_dim; out_col = col0 - rope_qd - p.head_dim; kv_dst = true; }
                    } else if (p.act == 1) finish([](float v) { return gelu_f(v); });
                    else if (p.act == 2) finish([](float v) { return silu_f(v); });
                    else finish([](float v) { return v; });
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
                            *reinterpret_cast<uint4*>(out_base + (kv_dst ? kv_row(p, grow) : (size_t)grow) * out_ld + out_col + sp * 8) =
                                *reinterpret_cast<const uint4*>(stg + (sr + 8 * i) * 80 + sp * 16);
                    }
                    __syncwarp();
                } else if (row < p.M) {
                    // RoPE scatter or fp32 destination: direct per-row stores
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const int col = n0 + c * 32 + j;
                        if (col < p.N) {
                            float a8[8], u8[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) { a8[i] = a[j + i]; u8[i] = DUAL ? u[j + i] : 0.f; }
                            uint4 rdirect = make_uint4(0, 0, 0, 0);
                            epilogue8<DUAL>(p, row, col, a8, u8, rdirect, false);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (tcount == 0 && threadIdx.x == 64) FVLA_STAMP_ANY(5);
            if (!from_partials && lane == 0) mbar_arrive(accempty_bar(acc));
        }
    }

    if (CLUSTER) {
        // nobody leaves while a bulk copy may still read its shared memory or signal its barriers
        if (warp < 2) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // pairs with the arrive after set-up
        asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
    if (threadIdx.x == 0) FVLA_STAMP_ANY(6);
    if (threadIdx.x == 0 && *abort_flag && args.status) atomicExch(args.status, 1);
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows of pitch `ld` elements;
// box = box_inner x box_outer, 128-byte swizzle, out-of-bounds reads give zero.
inline int make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
                    uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return FVLA_ERR_LAUNCH; }
    cuuint64_t gdim[2] = {inner, outer};
    cuuint64_t gstride[1] = {ld * sizeof(bf16)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return FVLA_ERR_ARG; }
    return FVLA_OK;
}

inline int num_sms() {
    static std::atomic<int> cached[kMaxDevices];
    const int dev = current_device();
    int sms = cached[dev].load(std::memory_order_relaxed);
    if (sms == 0) {
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
        cached[dev].store(sms, std::memory_order_relaxed);
    }
    return sms;
}

// Persistent kernels walk `items` work items with stride gridDim: the smallest grid that needs no more rounds than
// `max_ctas` would. Same critical path, fewer CTAs competing for the L2 -> SM path, no nearly empty last round.
inline int balanced_grid(int items, int max_ctas) {
    if (items <= max_ctas) return items;
    const int rounds = (items + max_ctas - 1) / max_ctas;
    return (items + rounds - 1) / rounds;
}

// 3-D bf16 tensor map: `inner` contiguous elements per row, `rows` rows of pitch `ld` elements, `slabs` such matrices
// `slab_stride` elements apart (a batch of sequences, each with its own row count limit: rows past `rows` read as
// zero instead of running into the next slab); box = box_inner x box_rows x 1, 128-byte swizzle.
inline int make_map3d(CUtensorMap* map, const void* base, uint64_t inner, uint64_t rows, uint64_t slabs, uint64_t ld,
                      uint64_t slab_stride, uint32_t box_inner, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return FVLA_ERR_LAUNCH; }
    cuuint64_t gdim[3] = {inner, rows, slabs};
    cuuint64_t gstride[2] = {ld * sizeof(bf16), (slabs > 1 ? slab_stride : rows * ld) * sizeof(bf16)};
    cuuint32_t box[3] = {box_inner, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), gdim, gstride, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (3-D) failed with CUresult %d", (int)r); return FVLA_ERR_ARG; }
    return FVLA_OK;
}

struct Tc5Plan { int bn, splits; size_t ws_bytes; float est_us; };

// Per-step times (us) of one 64-wide k step at tile width 64 / 128 / 192 / 256, as measured on B200: the
// shared-memory traffic of a step (every operand byte written once by TMA and read once by the tensor core, at
// 128 B/clk), not the MMA, sets them.
inline float k_step_us(int bn) { return bn == 64 ? 0.26f : (bn == 128 ? 0.30f : (bn == 192 ? 0.37f : 0.43f)); }

// Tile width and K split for a plain (non-gated) GEMM: minimise the estimated time of the slowest SM,
// (waves of work items) x (k steps per item) x (time per step), plus, for a split, the cost of writing
// and re-reading the fp32 partials. A split needs caller scratch and is only offered when `ws_ok`.
inline Tc5Plan plan_tc5(int M, int N, int K, bool ws_ok) {
    const int tiles_m = (M + BM - 1) / BM, sms = num_sms(), k_iters = (K + BK - 1) / BK;
    Tc5Plan best{128, 1, 0, 1e30f};
    float best_t = 1e30f;
    for (int bn = 64; bn <= 256; bn += 64) {
        const int tiles = tiles_m * ((N + bn - 1) / bn);
        for (int s = 1; s <= (ws_ok ? 4 : 1); ++s) {
            if (s > 1 && k_iters / s < 16) break;
            const int per = (k_iters + s - 1) / s;
            const int waves = (tiles * s + sms - 1) / sms;
            float t = waves * (per * k_step_us(bn) + 4.0f);
            if (s > 1) t += 3.0f + (float)s * M * N * 8.0f / 4.0e6f;      // partial traffic at about 4 TB/s
            if (t < best_t) { best_t = t; best = Tc5Plan{bn, s, 0, t}; }
        }
    }
    if (best.splits > 1)
        best.ws_bytes = (((size_t)tiles_m * ((N + best.bn - 1) / best.bn) * sizeof(int) + 255) / 256) * 256 +
                        (size_t)best.splits * tiles_m * ((N + best.bn - 1) / best.bn) * BM * best.bn * sizeof(float);
    return best;
}

template <int BN, bool DUAL, int STAGES, bool ROPE = false, bool CLUSTER = false, bool NORM = false>
inline int launch_tc5_cfg(const GemmArgs& g, int* status, cudaStream_t st, int splits = 1, void* ws = nullptr) {
    using Cfg = Tc5Cfg<BN, DUAL, STAGES>;
    auto kern = tc5_gemm_kernel<BN, DUAL, STAGES, ROPE, CLUSTER, NORM>;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    CUtensorMap tmA, tmB, tmB2;
    int rc = make_map(&tmA, g.A, (uint64_t)g.K, (uint64_t)g.M, (uint64_t)g.lda, BK, BM);
    if (rc) return rc;
    rc = make_map(&tmB, g.B, (uint64_t)g.N, (uint64_t)g.Kb, (uint64_t)g.ldb, 64, BK);
    if (rc) return rc;
    rc = make_map(&tmB2, DUAL ? g.B2 : g.B, (uint64_t)g.N, (uint64_t)g.Kb, (uint64_t)g.ldb, 64, BK);
    if (rc) return rc;
    Tc5Args a;
    a.g = g;
    a.tiles_m = (g.M + BM - 1) / BM;
    a.tiles_n = (g.N + BN - 1) / BN;
    a.k_iters = (g.K + BK - 1) / BK;
    a.splits = splits;
    a.k_per_split = (a.k_iters + splits - 1) / splits;
    a.partial = nullptr; a.counters = nullptr;
    if (splits > 1 && !CLUSTER) {
        const size_t counters = (((size_t)a.tiles_m * a.tiles_n * sizeof(int) + 255) / 256) * 256;
        a.counters = reinterpret_cast<int*>(ws);
        a.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + counters);
    }
    a.status = status;
    FVLA_DBG_ATTACH(a);
    int tiles = a.tiles_m * a.tiles_n * splits;
    int grid = balanced_grid(tiles, num_sms());
    cudaError_t e;
    if (CLUSTER) {
        // one work item per CTA, the splits of a tile adjacent in the grid = one cluster
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(tiles); cfg.blockDim = dim3(Cfg::THREADS); cfg.dynamicSmemBytes = Cfg::SMEM_BYTES; cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, kern, a, tmA, tmB, tmB2);
    } else {
        e = launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, st, a, tmA, tmB, tmB2);
    }
    if (e != cudaSuccess) { set_error("tc5_gemm_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("tc5_gemm_kernel");
}

// Shapes this path takes: at least one full 128-row tile of work and 16-byte aligned rows.
inline bool tc5_supports(const GemmArgs& g) {
    return g.M > 64 && g.N % 8 == 0 && g.K % 8 == 0 && g.lda % 8 == 0 && g.ldb % 8 == 0 && g.row_scale == nullptr &&
           aligned16(g.A) && aligned16(g.B) && (g.B2 == nullptr || aligned16(g.B2));
}

// Scratch bytes of a split through global partials at tile width bn.
inline size_t scratch_split_bytes(int M, int N, int bn, int splits) {
    const size_t tiles = (size_t)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    return splits > 1 ? ((tiles * sizeof(int) + 255) / 256) * 256 + (size_t)splits * tiles * BM * bn * sizeof(float) : 0;
}

// A pinned plan for a plain GEMM on the one-SM kernel: `engine` ENGINE_TC5_SCRATCH (tile width bn, K split
// through caller scratch) or ENGINE_TC5_CLUSTER (128-wide tiles, K split inside a cluster). Errors out when
// the launch cannot honour it.
inline int launch_gemm_tc5_pinned(GemmArgs g, const PlanChoice& pc, int* status, cudaStream_t st, void* ws, size_t ws_bytes) {
    if (g.Kb == 0) g.Kb = g.K;
    if (g.B2 != nullptr || g.rope != nullptr) { set_error("pinned plan: only plain GEMMs take a tile / split choice"); return FVLA_ERR_UNSUPPORTED; }
    const int k_iters = (g.K + BK - 1) / BK;
    if (pc.engine == ENGINE_TC5_CLUSTER) {
        const int tiles = ((g.M + BM - 1) / BM) * ((g.N + 127) / 128);
        if (pc.splits < 2 || pc.splits > 4 || tiles * pc.splits > num_sms() || k_iters / pc.splits < 2) {
            set_error("pinned plan: cluster split %d does not fit %d tiles / %d k steps", pc.splits, tiles, k_iters);
            return FVLA_ERR_UNSUPPORTED;
        }
        return launch_tc5_cfg<128, false, 6, false, true>(g, status, st, pc.splits, nullptr);
    }
    if (pc.splits < 1 || pc.splits > 4 || (pc.splits > 1 && (g.c_f32 || k_iters / pc.splits < 2))) {
        set_error("pinned plan: scratch split %d not possible here", pc.splits);
        return FVLA_ERR_UNSUPPORTED;
    }
    if (pc.splits > 1 && (ws == nullptr || ws_bytes < scratch_split_bytes(g.M, g.N, pc.bn, pc.splits))) {
        set_error("pinned plan: scratch of %zu bytes needed", scratch_split_bytes(g.M, g.N, pc.bn, pc.splits));
        return FVLA_ERR_WORKSPACE;
    }
    switch (pc.bn) {
        case 256: return launch_tc5_cfg<256, false, 4>(g, status, st, pc.splits, ws);
        case 192: return launch_tc5_cfg<192, false, 5>(g, status, st, pc.splits, ws);
        case 128: return launch_tc5_cfg<128, false, 6>(g, status, st, pc.splits, ws);
        case 64: return launch_tc5_cfg<64, false, 8>(g, status, st, pc.splits, ws);
        default: set_error("pinned plan: tile width %d (64, 128, 192 or 256)", pc.bn); return FVLA_ERR_ARG;
    }
}

inline int launch_gemm_tc5(GemmArgs g, int* status, cudaStream_t st, void* ws = nullptr, size_t ws_bytes = 0) {
    if (g.Kb == 0) g.Kb = g.K;
    if (g.B2 != nullptr) return launch_tc5_cfg<128, true, 4>(g, status, st);
    if (g.rope != nullptr) return launch_tc5_cfg<128, false, 6, true>(g, status, st);
    // an fp32 destination cannot take the split through global scratch, so it is planned without one
    Tc5Plan pl = plan_tc5(g.M, g.N, g.K, ws != nullptr && !g.c_f32);
    // Split-K reduced inside clusters (128-wide tiles, one work item per CTA, no scratch): taken when its
    // estimate (mainloop + epilogue + one 64 KB push per extra split) beats the plan above. An fp32
    // destination (the decoder's residual stream at M > 64) takes it as well: the split-0 CTA sums the
    // partials before either epilogue form runs.
    if (g.rope == nullptr) {
        const int tiles = ((g.M + BM - 1) / BM) * ((g.N + 127) / 128), k_iters = (g.K + BK - 1) / BK;
        int best_s = 0;
        float best_t = pl.est_us;
        for (int sp = 2; sp <= 4; ++sp) {
            if (tiles * sp > num_sms() || k_iters / sp < 8) break;
            // two mates reduce-scatter their halves (about 1.5 us); more splits gather one 64 KB tile each into the split-0 CTA
            const float t = ((k_iters + sp - 1) / sp) * k_step_us(128) + 4.0f + (sp == 2 ? 1.5f : 2.5f + (sp - 1) * 2.1f);
            if (t < best_t) { best_t = t; best_s = sp; }
        }
        if (best_s) return launch_tc5_cfg<128, false, 6, false, true>(g, status, st, best_s, nullptr);
    }
    if (pl.splits > 1 && (ws_bytes < pl.ws_bytes || g.rope != nullptr || g.c_f32)) pl = plan_tc5(g.M, g.N, g.K, false);
    switch (pl.bn) {
        case 256: return launch_tc5_cfg<256, false, 4>(g, status, st, pl.splits, ws);
        case 192: return launch_tc5_cfg<192, false, 5>(g, status, st, pl.splits, ws);
        case 64: return launch_tc5_cfg<64, false, 8>(g, status, st, pl.splits, ws);
        default: return launch_tc5_cfg<128, false, 6>(g, status, st, pl.splits, ws);
    }
}

// GEMM with the row norm of A folded in (GemmArgs::norm_mode != 0): one tile per CTA, no K split, bf16 destination,
// and either the RoPE + scatter epilogue alone or the plain one. FVLA_ERR_UNSUPPORTED otherwise; the caller then
// normalises A with a kernel of its own and calls the plain GEMM.
// Tile width at which the fused-norm GEMM takes an M x N x K problem (0: it does not): every CTA gets one tile.
inline int normed_tile_width(int M, int N, int K, bool rope) {
    if (M <= 64 || N % 8 != 0 || K % BK != 0) return 0;
    const int tiles_m = (M + BM - 1) / BM, sms = num_sms();
    if (rope) return tiles_m * ((N + 127) / 128) <= sms ? 128 : 0;
    int bn = plan_tc5(M, N, K, false).bn;      // the widest tile that still gives every CTA exactly one, starting from the plain kernel's plan
    if (bn < 128) bn = 128;                    // the fused-norm variants start at 128 columns
    while (bn < 256 && tiles_m * ((N + bn - 1) / bn) > sms) bn += 64;
    return tiles_m * ((N + bn - 1) / bn) <= sms ? bn : 0;
}

inline int launch_gemm_tc5_normed(GemmArgs g, int* status, cudaStream_t st) {
    if (g.Kb == 0) g.Kb = g.K;
    if (!tc5_supports(g) || g.B2 != nullptr || g.c_f32 || g.norm_mode < 1 || g.norm_mode > 2 || g.K % BK != 0 ||
        (g.norm_mode == 2 && g.colsum == nullptr))
        return FVLA_ERR_UNSUPPORTED;
    const int bn = normed_tile_width(g.M, g.N, g.K, g.rope != nullptr);
    if (bn == 0) return FVLA_ERR_UNSUPPORTED;
    if (g.rope != nullptr) {
        if (g.R != nullptr || g.bias != nullptr || g.bias_f32 != nullptr || g.act != 0) return FVLA_ERR_UNSUPPORTED;
        return launch_tc5_cfg<128, false, 6, true, false, true>(g, status, st);
    }
    switch (bn) {
        case 256: return launch_tc5_cfg<256, false, 4, false, false, true>(g, status, st);
        case 192: return launch_tc5_cfg<192, false, 5, false, false, true>(g, status, st);
        default: return launch_tc5_cfg<128, false, 6, false, false, true>(g, status, st);
    }
}

}  // namespace tc5
}  // namespace fvla
