// tcgen05 flash attention for the prefix encoder: unmasked multi-query attention over flat queries
// (token x head rows, one shared K/V head), head dimension 256.
//
// One CTA owns 128 query rows (= the 128 TMEM lanes) and walks the keys in blocks of 128:
//   * warp 0 (one lane) is the TMA producer: the Q tile once, then K and V blocks, each into its own
//     single buffer (K is free again as soon as S = Q K^T has been issued, V once P V has);
//   * warp 1 (one lane) issues the MMAs: S_j = Q K_j^T (16 x m128 n128 k16) into one of two TMEM score
//     buffers, always one block ahead of O += P_j V_j (8 x m128 n256 k16) into a TMEM accumulator;
//   * warps 2-5 are the softmax: thread = query row. They read S_j from TMEM, keep a running maximum,
//     write P_j = exp2(S_j - m) as bf16 into the K-major operand layout in shared memory and track the
//     row sum. The accumulator is rescaled only when the maximum has grown by more than 2^8 since the
//     value P is expressed against (rare after the first block), so P V seldom waits for a correction.
// All operands are used where TMA puts them (128-byte swizzle): Q and K are K-major, V is the
// MN-major B operand exactly as the weights of the GEMM kernels.
//
// When one CTA per query tile would leave most SMs idle, two CTAs (a cluster) share a tile: each walks half of
// the key blocks, then the two reduce-scatter: a CTA stages the other's half of its unnormalised accumulator
// (128 of the 256 columns, fp32) in its idle K buffer and pushes it, with its rows' running maximum and sum,
// into the mate's idle V buffer by bulk copy; each then merges the two partial results for its own 128
// columns (log-sum-exp) and stores them.
#pragma once

#include "common.cuh"
#include "gemm_tc5.cuh"

namespace fvla {
namespace attn5 {

using tc5::mbar_init;
using tc5::mbar_expect_tx;
using tc5::mbar_wait;
using tc5::tma_load_2d;
using tc5::tma_load_3d;
using tc5::smem_desc;

constexpr int HD = 256, BQ = 128, BKEY = 128, THREADS = 192;
constexpr int Q_BYTES = BQ * HD * 2, K_BYTES = BKEY * HD * 2, V_BYTES = BKEY * HD * 2, P_BYTES = BQ * BKEY * 2;
constexpr int OFF_Q = 0, OFF_K = OFF_Q + Q_BYTES, OFF_V = OFF_K + K_BYTES, OFF_P = OFF_V + V_BYTES;
constexpr int OFF_BAR = OFF_P + P_BYTES;
constexpr int SMEM = 1024 + OFF_BAR + 192;
constexpr uint32_t S_COLS = 128, O_COL = 256;         // TMEM: S buffers at columns 0 and 128, O at 256..511
constexpr float RESCALE_THRESHOLD = 8.0f;              // log2 units

struct Args {
    bf16* out;
    int nq, nk;
    float scale_log2;
    int* status;
    int split;          // 1: launched as clusters of two CTAs per query tile, each walking half of the key blocks
    // A batch of sequences (grid.y): sequence e reads slab e of the Q / K / V tensor maps and writes `out` at
    // e * out_stride elements. Rows below `mask_rows` only see keys up to `mask_key_le` (the action expert's
    // state token must not see the action tokens); mask_rows = 0: no mask.
    long long out_stride;
    int mask_rows, mask_key_le;
};

// S = Q K^T: both operands K-major.
__host__ __device__ constexpr uint32_t idesc_qk() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(BKEY >> 3) << 17) |
           ((uint32_t)(BQ >> 4) << 24);
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// 128 consecutive TMEM columns of this thread's lane: four 32-column loads issued back to back, one wait.
__device__ __forceinline__ void ld_row128(uint32_t taddr, float (&v)[128]) {
    uint32_t r[128];
#pragma unroll
    for (int c = 0; c < 4; ++c)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[c * 32 + 0]), "=r"(r[c * 32 + 1]), "=r"(r[c * 32 + 2]), "=r"(r[c * 32 + 3]), "=r"(r[c * 32 + 4]), "=r"(r[c * 32 + 5]),
              "=r"(r[c * 32 + 6]), "=r"(r[c * 32 + 7]), "=r"(r[c * 32 + 8]), "=r"(r[c * 32 + 9]), "=r"(r[c * 32 + 10]), "=r"(r[c * 32 + 11]),
              "=r"(r[c * 32 + 12]), "=r"(r[c * 32 + 13]), "=r"(r[c * 32 + 14]), "=r"(r[c * 32 + 15]), "=r"(r[c * 32 + 16]), "=r"(r[c * 32 + 17]),
              "=r"(r[c * 32 + 18]), "=r"(r[c * 32 + 19]), "=r"(r[c * 32 + 20]), "=r"(r[c * 32 + 21]), "=r"(r[c * 32 + 22]), "=r"(r[c * 32 + 23]),
              "=r"(r[c * 32 + 24]), "=r"(r[c * 32 + 25]), "=r"(r[c * 32 + 26]), "=r"(r[c * 32 + 27]), "=r"(r[c * 32 + 28]), "=r"(r[c * 32 + 29]),
              "=r"(r[c * 32 + 30]), "=r"(r[c * 32 + 31])
            : "r"(taddr + c * 32) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 128; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tc5_kernel(const Args p, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V, sP = base + OFF_P;
    const uint32_t bars = base + OFF_BAR;
    const uint32_t q_full = bars, k_full = bars + 8, k_empty = bars + 16, v_full = bars + 24, v_empty = bars + 32;
    const uint32_t p_full = bars + 40, p_empty = bars + 48, o_done = bars + 56;
    auto s_full = [&](int b) { return bars + 64 + b * 8; };
    auto s_empty = [&](int b) { return bars + 80 + b * 8; };
    const uint32_t tmem_slot = bars + 96;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + OFF_BAR + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + OFF_BAR + 104);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nblk_all = (p.nk + BKEY - 1) / BKEY;
    uint32_t rank = 0;
    if (p.split) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int q0 = (p.split ? blockIdx.x >> 1 : blockIdx.x) * BQ;
    const int seq = blockIdx.y;                                                 // which sequence of the batch
    const int half_blks = (nblk_all + 1) / 2;
    const int jb0 = p.split ? (int)rank * half_blks : 0;                        // first key block of this CTA
    const int nblk = p.split ? min(half_blks, nblk_all - jb0) : nblk_all;      // and how many it walks
    const uint32_t x_ready = bars + 112, x_recv = bars + 120;                   // key split: "mate may send", "mate's half has arrived"

    if (tid == 0) {
        for (int i = 0; i < 12; ++i) mbar_init(bars + i * 8, 1);
        mbar_init(x_ready, 1);
        mbar_init(x_recv, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tc5::tmem_alloc(tmem_slot, 512);
        tc5::tmem_relinquish();
    }
    tc5::tc_fence_before();
    __syncthreads();
    tc5::tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;
    if (p.split) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");   // the mate's barriers exist
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");       // Q, K and V come from the preceding kernel

    if (warp == 0) {
        // two independent streams: lane 0 feeds Q and the K blocks, lane 1 the V blocks, so that the next K
        // block is requested as soon as S = Q K^T has been issued, whatever the state of P V
        if (lane == 0) {
            tc5::prefetch_tensormap(&tmQ);
            tc5::prefetch_tensormap(&tmK);
            mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
            for (int a = 0; a < 4; ++a) tma_load_3d(sQ + a * 16384, &tmQ, q_full, a * 64, q0, seq);
            for (int j = 0; j < nblk; ++j) {
                if (!mbar_wait(k_empty, (uint32_t)(j & 1) ^ 1u, abort_flag)) break;
                mbar_expect_tx(k_full, K_BYTES);
#pragma unroll
                for (int a = 0; a < 4; ++a) tma_load_3d(sK + a * 16384, &tmK, k_full, a * 64, (jb0 + j) * BKEY, seq);
            }
        } else if (lane == 1) {
            tc5::prefetch_tensormap(&tmV);
            for (int j = 0; j < nblk; ++j) {
                if (!mbar_wait(v_empty, (uint32_t)(j & 1) ^ 1u, abort_flag)) break;
                mbar_expect_tx(v_full, V_BYTES);
#pragma unroll
                for (int kb = 0; kb < 2; ++kb)
#pragma unroll
                    for (int a = 0; a < 4; ++a)
                        tma_load_3d(sV + kb * 32768 + a * 8192, &tmV, v_full, a * 64, (jb0 + j) * BKEY + kb * 64, seq);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t id_qk = idesc_qk();
            constexpr uint32_t id_pv = tc5::instr_desc(256);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            tc5::tc_fence_after();
            auto issue_qk = [&](int j) -> bool {
                const int b = j & 1;
                if (!mbar_wait(k_full, (uint32_t)(j & 1), abort_flag)) return false;
                if (!mbar_wait(s_empty(b), (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag)) return false;
                tc5::tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const uint64_t adesc = smem_desc(sQ + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t bdesc = smem_desc(sK + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    tc5::umma_bf16(tmem + b * S_COLS, adesc, bdesc, id_qk, kk > 0 ? 1u : 0u);
                }
                tc5::umma_commit(k_empty);
                tc5::umma_commit(s_full(b));
                return true;
            };
            if (ok && nblk > 0) ok = issue_qk(0);
            for (int j = 0; j < nblk && ok; ++j) {
                if (j + 1 < nblk) { ok = issue_qk(j + 1); if (!ok) break; }
                if (!mbar_wait(p_full, (uint32_t)(j & 1), abort_flag)) break;
                if (!mbar_wait(v_full, (uint32_t)(j & 1), abort_flag)) break;
                tc5::tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < BKEY / 16; ++k16) {
                    const uint64_t adesc = smem_desc(sP + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024);
                    const uint64_t bdesc = smem_desc(sV + (k16 >> 2) * 32768 + (k16 & 3) * 2048, 8192, 1024);
                    tc5::umma_bf16(tmem + O_COL, adesc, bdesc, id_pv, (j > 0 || k16 > 0) ? 1u : 0u);
                }
                tc5::umma_commit(v_empty);
                tc5::umma_commit(p_empty);
                tc5::umma_commit(o_done);
            }
        }
    } else {
        // softmax / correction / epilogue: one thread per query row. Every thread runs every iteration and
        // every named barrier even after a wait has given up (`ok` false), so nobody is left behind.
        const int quad = warp & 3;                           // TMEM lane group this warp may access
        const int row = quad * 32 + lane;
        const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
        bool ok = true;
        float m_used = 0.f, l = 0.f;
        // keys this row may see: all of them, or (masked rows) those up to mask_key_le
        const int key_limit = (q0 + row < p.mask_rows) ? min(p.nk, p.mask_key_le + 1) : p.nk;
        bool seen_any = false;                               // a block with at least one visible key has been processed
        for (int j = 0; j < nblk; ++j) {
            const int b = j & 1;
            ok = ok && mbar_wait(s_full(b), (uint32_t)((j >> 1) & 1), abort_flag);
            __syncwarp();                                    // the TMEM accesses below are warp-collective
            tc5::tc_fence_after();
            const uint32_t t_s = tmem + t_lane + b * S_COLS;
            // the whole 128-key score row of this thread, read once (four loads in flight, one wait)
            float v[BKEY];
            ld_row128(t_s, v);
            const int key0 = (jb0 + j) * BKEY;              // first key of this block
            const bool ragged = key0 + BKEY > key_limit;    // a block that holds keys this row does not see (past the end, or masked)
            float mx = -INFINITY;
            if (!ragged) {
#pragma unroll
                for (int i = 0; i < BKEY; ++i) mx = fmaxf(mx, v[i]);
            } else {
#pragma unroll
                for (int i = 0; i < BKEY; ++i)
                    if (key0 + i < key_limit) mx = fmaxf(mx, v[i]);
            }
            mx *= p.scale_log2;                              // the scale is positive
            if (j == 0) {
                m_used = mx == -INFINITY ? 0.f : mx;
            } else {
                // a row that has not seen a key yet (masked so far) has nothing accumulated: it adopts this block's
                // maximum as it is; the others rescale when their maximum has grown enough
                const bool first = !seen_any;
                const bool grow = !first && mx > m_used + RESCALE_THRESHOLD;
                if (__any_sync(0xffffffffu, grow)) {
                    // the accumulator must be quiet while it is rescaled: P_{j-1} V_{j-1} has to be complete
                    ok = ok && mbar_wait(o_done, (uint32_t)((j - 1) & 1), abort_flag);
                    __syncwarp();
                    tc5::tc_fence_after();
                    const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
#pragma unroll 1
                    for (int c = 0; c < HD / 32; ++c) {
                        float o[32];
                        tc5::tmem_ld32(tmem + t_lane + O_COL + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] *= alpha;
                        tmem_st32(tmem + t_lane + O_COL + c * 32, o);
                    }
                    l *= alpha;
                    if (grow) m_used = mx;
                    tc5::tc_fence_before();
                }
                if (first && mx != -INFINITY) m_used = mx;
            }
            // P = 2^(scale * S - m): one fused multiply-add and one special-function op per key
            float psum = 0.f;
            if (!ragged) {
#pragma unroll
                for (int i = 0; i < BKEY; ++i) { v[i] = fast_exp2(fmaf(v[i], p.scale_log2, -m_used)); psum += v[i]; }
            } else {
#pragma unroll
                for (int i = 0; i < BKEY; ++i) { v[i] = key0 + i < key_limit ? fast_exp2(fmaf(v[i], p.scale_log2, -m_used)) : 0.f; psum += v[i]; }
            }
            ok = ok && mbar_wait(p_empty, (uint32_t)(j & 1) ^ 1u, abort_flag);      // P_{j-1} has been consumed
            __syncwarp();
            // 8 keys = 16 bytes = one piece of this row's 128 bytes in atom (keys / 64), 128-byte swizzle
#pragma unroll
            for (int piece = 0; piece < BKEY / 8; ++piece) {
                uint8_t* prow = gen + OFF_P + (piece >> 3) * 16384 + row * 128;
                *reinterpret_cast<uint4*>(prow + (((piece & 7) ^ (row & 7)) << 4)) =
                    make_uint4(pack_bf16x2(v[8 * piece], v[8 * piece + 1]), pack_bf16x2(v[8 * piece + 2], v[8 * piece + 3]),
                               pack_bf16x2(v[8 * piece + 4], v[8 * piece + 5]), pack_bf16x2(v[8 * piece + 6], v[8 * piece + 7]));
            }
            l += psum;
            seen_any = seen_any || mx != -INFINITY;
            tc5::tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P stores -> visible to the MMA
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2 && lane == 0) {
                mbar_arrive_local(p_full);
                mbar_arrive_local(s_empty(b));
            }
        }
        if (nblk > 0) ok = ok && mbar_wait(o_done, (uint32_t)((nblk - 1) & 1), abort_flag);
        __syncwarp();
        tc5::tc_fence_after();
        const int grow = q0 + row;
        const bool store = ok && grow < p.nq;              // the TMEM loads are warp-collective: only the stores are predicated
        bf16* dst = p.out + (size_t)seq * p.out_stride + (size_t)(grow < p.nq ? grow : 0) * HD;
        if (p.split) {
            // Reduce-scatter with the mate. All of this CTA's MMAs are complete, so its K, V and P buffers are idle:
            // K stages the mate's column half of the accumulator as [column quad][row][4], P holds the rows'
            // (maximum, sum) for sending (first 1 KB) and the mate's (second 1 KB), V receives the mate's partial
            // sums of THIS CTA's column half.
            constexpr uint32_t HALF_BYTES = BQ * (HD / 2) * 4, STAT_BYTES = BQ * 8;
            const int mine = (int)rank, other = mine ^ 1;
            if (warp == 2 && lane == 0) {
                mbar_expect_tx(x_recv, HALF_BYTES + STAT_BYTES);
                uint32_t rb;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(x_ready), "r"(other));
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(rb) : "memory");
            }
            reinterpret_cast<float2*>(gen + OFF_P)[row] = make_float2(l > 0.f ? m_used : -INFINITY, l);      // a side that saw no key drops out of the merge
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                float o[32];
                tc5::tmem_ld32(tmem + t_lane + O_COL + other * (HD / 2) + c * 32, o);
                float* stage = reinterpret_cast<float*>(gen + OFF_K) + (c * 8) * (BQ * 4) + row * 4;
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(stage + (i / 4) * (BQ * 4)) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // staged values -> visible to the bulk copies
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (warp == 2 && lane == 0) {
                if (mbar_wait(x_ready, 0, abort_flag)) {      // the mate's V and P buffers are idle
                    uint32_t dv, dp, rb;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dv) : "r"(sV), "r"(other));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dp) : "r"(sP + STAT_BYTES), "r"(other));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(x_recv), "r"(other));
#pragma unroll
                    for (uint32_t off = 0; off < HALF_BYTES; off += 16384)
                        asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(dv + off), "r"(sK + off), "r"(16384), "r"(rb) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(dp), "r"(sP), "r"(STAT_BYTES), "r"(rb) : "memory");
                }
            }
            ok = mbar_wait(x_recv, 0, abort_flag) && ok;
            const float2 theirs = reinterpret_cast<const float2*>(gen + OFF_P + STAT_BYTES)[row];
            // both partial results against the larger maximum
            const float m_own = l > 0.f ? m_used : -INFINITY;
            const float m_all = fmaxf(m_own, theirs.x);
            const float s_own = l > 0.f ? fast_exp2(m_own - m_all) : 0.f, s_their = theirs.y > 0.f ? fast_exp2(theirs.x - m_all) : 0.f;
            const float l_all = l * s_own + theirs.y * s_their;
            const float inv_all = l_all > 0.f ? 1.0f / l_all : 0.f;
            const float w_own = s_own * inv_all, w_their = s_their * inv_all;
            const bool st = ok && grow < p.nq;
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                float o[32];
                tc5::tmem_ld32(tmem + t_lane + O_COL + mine * (HD / 2) + c * 32, o);
                const float* recv = reinterpret_cast<const float*>(gen + OFF_V) + (c * 8) * (BQ * 4) + row * 4;
                if (st) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 r0 = *reinterpret_cast<const float4*>(recv + (2 * q) * (BQ * 4));
                        const float4 r1 = *reinterpret_cast<const float4*>(recv + (2 * q + 1) * (BQ * 4));
                        *reinterpret_cast<uint4*>(dst + mine * (HD / 2) + c * 32 + q * 8) =
                            make_uint4(pack_bf16x2(o[8 * q] * w_own + r0.x * w_their, o[8 * q + 1] * w_own + r0.y * w_their),
                                       pack_bf16x2(o[8 * q + 2] * w_own + r0.z * w_their, o[8 * q + 3] * w_own + r0.w * w_their),
                                       pack_bf16x2(o[8 * q + 4] * w_own + r1.x * w_their, o[8 * q + 5] * w_own + r1.y * w_their),
                                       pack_bf16x2(o[8 * q + 6] * w_own + r1.z * w_their, o[8 * q + 7] * w_own + r1.w * w_their));
                    }
                }
                __syncwarp();
            }
        }
        const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll 1
        for (int c = 0; c < (p.split ? 0 : HD / 32); ++c) {
            float o[32];
            tc5::tmem_ld32(tmem + t_lane + O_COL + c * 32, o);
            if (store) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) =
                        make_uint4(pack_bf16x2(o[8 * q] * inv, o[8 * q + 1] * inv), pack_bf16x2(o[8 * q + 2] * inv, o[8 * q + 3] * inv),
                                   pack_bf16x2(o[8 * q + 4] * inv, o[8 * q + 5] * inv), pack_bf16x2(o[8 * q + 6] * inv, o[8 * q + 7] * inv));
            }
            __syncwarp();
        }
    }

    tc5::tc_fence_before();
    __syncthreads();
    // neither mate leaves while the other's bulk copies may still read its shared memory or signal its barrier
    if (p.split) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        tc5::tc_fence_after();
        tc5::tmem_dealloc(tmem, 512);
    }
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 4);
}

// `seqs` sequences of nq flat query rows x nk keys each (grid.y); Q / K / V of sequence e start q_stride / kv_stride
// elements after those of e - 1, `out` like Q. mask_rows / mask_key_le: see Args.
inline int launch_attention_tc5(const void* Q, const void* K, const void* V, void* out, int nq, int nk, float scale_log2,
                                int* status, cudaStream_t st, int seqs = 1, long long q_stride = 0, long long kv_stride = 0,
                                int mask_rows = 0, int mask_key_le = 0) {
    auto kern = attention_tc5_kernel;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    CUtensorMap tmQ, tmK, tmV;
    int rc = tc5::make_map3d(&tmQ, Q, HD, (uint64_t)nq, (uint64_t)seqs, HD, (uint64_t)q_stride, 64, BQ);
    if (rc) return rc;
    rc = tc5::make_map3d(&tmK, K, HD, (uint64_t)nk, (uint64_t)seqs, HD, (uint64_t)kv_stride, 64, BKEY);
    if (rc) return rc;
    rc = tc5::make_map3d(&tmV, V, HD, (uint64_t)nk, (uint64_t)seqs, HD, (uint64_t)kv_stride, 64, 64);
    if (rc) return rc;
    // Two CTAs per query tile (each half of the key blocks) when that still fits one CTA per SM and both get a block.
    const int q_tiles = (nq + BQ - 1) / BQ;
    const int split = (2 * q_tiles * seqs <= tc5::num_sms() && (nk + BKEY - 1) / BKEY >= 2) ? 1 : 0;
    Args a{static_cast<bf16*>(out), nq, nk, scale_log2, status, split, q_stride, mask_rows, mask_key_le};
    cudaError_t e;
    if (split) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * q_tiles, seqs); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM; cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 2 : 1;
        e = cudaLaunchKernelEx(&cfg, kern, a, tmQ, tmK, tmV);
    } else {
        e = launch_pdl(kern, dim3(q_tiles, seqs), dim3(THREADS), SMEM, st, a, tmQ, tmK, tmV);
    }
    if (e != cudaSuccess) { set_error("attention_tc5_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("attention_tc5_kernel");
}

// ---------------------------------------------------------------------------------------------
// SigLIP attention on tcgen05: one CTA per (view, head, half of the 256 query tokens). The whole key
// range (256 tokens) is one S tile, so there is no loop and no rescale: S = Q K^T (5 x m128 n256 k16:
// head dim 72 padded to 80), softmax by two threads per row (128 keys each, maxima and sums swapped
// through shared memory), O = P V (16 x m128 n80 k16). Q, K and V are read by TMA straight from the
// packed QKV activation ([views * tokens, 3 * heads * 72], head slices of 144 bytes); the 64-wide boxes
// that cover dims 64..127 of a slice pick up 56 columns that belong to the next slice: dims 72..79 of
// the Q tile are zeroed in shared memory before the MMA (so the matching K columns do not matter), and
// output columns 72..79 are simply not stored.
// ---------------------------------------------------------------------------------------------
namespace vis {
constexpr int TOK = 256, HDIM = 72, THREADS = 320;
constexpr int OFF_Q = 0;                       // 2 atoms x [128 rows x 128 B]
constexpr int OFF_K = 32768;                   // 2 atoms x [256 rows x 128 B]
constexpr int OFF_V = 98304;                   // [key block 4][dim atom 2][64 rows x 128 B]
constexpr int OFF_P = 163840;                  // 4 atoms x [128 rows x 128 B]
constexpr int OFF_BAR = 229376;
constexpr int SMEM = 1024 + OFF_BAR + 128;
constexpr uint32_t O_COL = 256;                // TMEM: S at columns 0..255, O at 256..335

__host__ __device__ constexpr uint32_t idesc_qk() {      // m128 n256, both operands K-major
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_pv() {      // m128 n80, A K-major, B MN-major
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((uint32_t)(80 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

struct Args {
    bf16* out;
    int heads;
    float scale_log2;
    int* status;
};

__global__ void __launch_bounds__(THREADS, 1)
vision_attention_tc5_kernel(const Args p, const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sQ = base + OFF_Q, sK = base + OFF_K, sV = base + OFF_V, sP = base + OFF_P;
    const uint32_t bars = base + OFF_BAR;
    const uint32_t qk_full = bars, v_full = bars + 8, q_fixed = bars + 16, s_full = bars + 24, p_full = bars + 32, o_full = bars + 40;
    const uint32_t tmem_slot = bars + 48;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gen + OFF_BAR + 48);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + OFF_BAR + 56);
    float* xch = reinterpret_cast<float*>(gen + OFF_Q);      // [2 groups][128 rows] maxima, then sums: Q is dead by then

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int qh = blockIdx.x, head = blockIdx.y, view = blockIdx.z;
    const int width = p.heads * HDIM;

    if (tid == 0) {
        mbar_init(qk_full, 1); mbar_init(v_full, 1); mbar_init(q_fixed, 128);
        mbar_init(s_full, 1); mbar_init(p_full, 1); mbar_init(o_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tc5::tmem_alloc(tmem_slot, 512);
        tc5::tmem_relinquish();
    }
    tc5::tc_fence_before();
    __syncthreads();
    tc5::tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the QKV activation comes from the preceding kernel

    if (warp == 0) {
        if (lane == 0) {
            tc5::prefetch_tensormap(&tmQ);
            tc5::prefetch_tensormap(&tmK);
            tc5::prefetch_tensormap(&tmV);
            mbar_expect_tx(qk_full, 32768 + 65536);
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                tma_load_2d(sQ + a * 16384, &tmQ, qk_full, head * HDIM + a * 64, view * TOK + qh * 128);
                tma_load_2d(sK + a * 32768, &tmK, qk_full, width + head * HDIM + a * 64, view * TOK);
            }
            mbar_expect_tx(v_full, 65536);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb)
#pragma unroll
                for (int a = 0; a < 2; ++a)
                    tma_load_2d(sV + kb * 16384 + a * 8192, &tmV, v_full, 2 * width + head * HDIM + a * 64, view * TOK + kb * 64);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = mbar_wait(qk_full, 0, abort_flag) && mbar_wait(q_fixed, 0, abort_flag);
            if (ok) {
                tc5::tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < 5; ++kk) {
                    const uint64_t adesc = smem_desc(sQ + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
                    const uint64_t bdesc = smem_desc(sK + (kk >> 2) * 32768 + (kk & 3) * 32, 16, 1024);
                    tc5::umma_bf16(tmem, adesc, bdesc, idesc_qk(), kk > 0 ? 1u : 0u);
                }
                tc5::umma_commit(s_full);
                ok = mbar_wait(p_full, 0, abort_flag) && mbar_wait(v_full, 0, abort_flag);
            }
            if (ok) {
                tc5::tc_fence_after();
#pragma unroll
                for (int k16 = 0; k16 < TOK / 16; ++k16) {
                    const uint64_t adesc = smem_desc(sP + (k16 >> 2) * 16384 + (k16 & 3) * 32, 16, 1024);
                    const uint64_t bdesc = smem_desc(sV + (k16 >> 2) * 16384 + (k16 & 3) * 2048, 8192, 1024);
                    tc5::umma_bf16(tmem + O_COL, adesc, bdesc, idesc_pv(), k16 > 0 ? 1u : 0u);
                }
                tc5::umma_commit(o_full);
            }
        }
    } else {
        // softmax / epilogue: group g (warps 2-5, 6-9) takes keys [128 g, +128) of row = 32 (warp & 3) + lane
        const int g = (warp - 2) >> 2, quad = warp & 3;
        const int row = quad * 32 + lane;
        const uint32_t t_lane = (uint32_t)(quad * 32) << 16;
        bool ok = true;
        if (g == 0) {
            // dims 72..79 of the Q tile hold the next slice's data: zero them (16-byte piece 1 of atom 1)
            ok = mbar_wait(qk_full, 0, abort_flag);
            *reinterpret_cast<uint4*>(gen + OFF_Q + 16384 + row * 128 + ((1 ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive_local(q_fixed);
        }
        ok = mbar_wait(s_full, 0, abort_flag) && ok;
        __syncwarp();
        tc5::tc_fence_after();
        float v[128];
        ld_row128(tmem + t_lane + g * 128, v);
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; ++i) mx = fmaxf(mx, v[i]);
        xch[g * 128 + row] = mx;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        const float m = fmaxf(xch[row], xch[128 + row]) * p.scale_log2;      // the scale is positive
        asm volatile("bar.sync 1, 256;" ::: "memory");                           // maxima read before the sums overwrite them
        float psum = 0.f;
#pragma unroll
        for (int i = 0; i < 128; ++i) { v[i] = fast_exp2(fmaf(v[i], p.scale_log2, -m)); psum += v[i]; }
#pragma unroll
        for (int piece = 0; piece < 16; ++piece) {
            uint8_t* prow = gen + OFF_P + (2 * g + (piece >> 3)) * 16384 + row * 128;
            *reinterpret_cast<uint4*>(prow + (((piece & 7) ^ (row & 7)) << 4)) =
                make_uint4(pack_bf16x2(v[8 * piece], v[8 * piece + 1]), pack_bf16x2(v[8 * piece + 2], v[8 * piece + 3]),
                           pack_bf16x2(v[8 * piece + 4], v[8 * piece + 5]), pack_bf16x2(v[8 * piece + 6], v[8 * piece + 7]));
        }
        xch[g * 128 + row] = psum;
        tc5::tc_fence_before();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // P stores -> visible to the MMA
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (warp == 2 && lane == 0) mbar_arrive_local(p_full);
        const float l = xch[row] + xch[128 + row];
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        ok = mbar_wait(o_full, 0, abort_flag) && ok;
        __syncwarp();
        tc5::tc_fence_after();
        // group 0 stores dims 0..39, group 1 dims 40..71 (TMEM columns 32..63 and 64..79 are read in both)
        float a[32], b[16];
        tc5::tmem_ld32(tmem + t_lane + O_COL + (g == 0 ? 0 : 32), a);
        tc5::tmem_ld16(tmem + t_lane + O_COL + (g == 0 ? 32 : 64), b);
        if (ok) {
            bf16* dst = p.out + ((size_t)(view * TOK + qh * 128 + row)) * width + head * HDIM;
            auto pack8 = [&](const float* s) {
                return make_uint4(pack_bf16x2(s[0] * inv, s[1] * inv), pack_bf16x2(s[2] * inv, s[3] * inv),
                                  pack_bf16x2(s[4] * inv, s[5] * inv), pack_bf16x2(s[6] * inv, s[7] * inv));
            };
            if (g == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = pack8(a + q * 8);
                *reinterpret_cast<uint4*>(dst + 32) = pack8(b);
            } else {
                // a = dims 32..63, b = dims 64..79
#pragma unroll
                for (int q = 1; q < 4; ++q) *reinterpret_cast<uint4*>(dst + 32 + q * 8) = pack8(a + q * 8);
                *reinterpret_cast<uint4*>(dst + 64) = pack8(b);
            }
        }
    }

    tc5::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc5::tc_fence_after();
        tc5::tmem_dealloc(tmem, 512);
    }
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 5);
}

// qkv: [views * 256, 3 * heads * 72] bf16; out: [views * 256, heads * 72] bf16.
inline int launch_vision_attention_tc5(const void* qkv, void* out, int views, int heads, int* status, cudaStream_t st) {
    auto kern = vision_attention_tc5_kernel;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    const uint64_t cols = (uint64_t)3 * heads * HDIM, rows = (uint64_t)views * TOK;
    CUtensorMap tmQ, tmK, tmV;
    int rc = tc5::make_map(&tmQ, qkv, cols, rows, cols, 64, 128);
    if (rc) return rc;
    rc = tc5::make_map(&tmK, qkv, cols, rows, cols, 64, 256);
    if (rc) return rc;
    rc = tc5::make_map(&tmV, qkv, cols, rows, cols, 64, 64);
    if (rc) return rc;
    Args a{static_cast<bf16*>(out), heads, kLog2e / sqrtf((float)HDIM), status};
    cudaError_t e = launch_pdl(kern, dim3(2, heads, views), dim3(THREADS), SMEM, st, a, tmQ, tmK, tmV);
    if (e != cudaSuccess) { set_error("vision_attention_tc5_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("vision_attention_tc5_kernel");
}
}  // namespace vis

}  // namespace attn5
}  // namespace fvla
