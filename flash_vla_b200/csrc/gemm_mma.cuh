// General bf16 GEMM with fused epilogues on the warp-level tensor path (mma.sync m16n8k16).
//
// C[M,N] = epilogue(A[M,K] @ B[K,N]) with A row-major (K contiguous) and B row-major
// (N contiguous, the checkpoint's (in, out) layout). This kernel covers every ragged or tiny
// shape in the model (K = 588, N = 4304, M = 1 / 50 / 51) and is the fallback for shapes the
// tcgen05 kernels do not take. Split-K spreads the M <= 64 decoder GEMMs over all SMs; the
// last-arriving CTA of a tile sums the partials in fixed split order, so results are
// deterministic, and resets its semaphore so a captured graph can be replayed.
#pragma once

#include <cstdlib>

#include "common.cuh"

namespace fvla {

struct GemmArgs {
    const bf16* A = nullptr; int lda = 0;
    const bf16* B = nullptr; const bf16* B2 = nullptr; int ldb = 0;
    void* C = nullptr; int ldc = 0; int c_f32 = 0;           // C (and R) are fp32 when c_f32 != 0
    const bf16* bias = nullptr;
    const void* R = nullptr; int ldr = 0; int res_mod = 0;   // residual row = row % res_mod if > 0
    const float* row_scale = nullptr;                        // per-row factor on the accumulator
    int act = 0;                                             // 0 none, 1 gelu, 2 silu
    int M = 0, N = 0, K = 0, Kb = 0;                         // Kb: valid rows of B (<= K)
    // RoPE + scatter epilogue (used when rope != nullptr; C is ignored)
    const bf16* rope = nullptr; bf16* q = nullptr; bf16* k = nullptr; bf16* v = nullptr;
    int heads = 0, head_dim = 0, round_first = 0;
    // Rows may be several sequences of `group_rows` tokens laid end to end (a batch of episodes): the RoPE
    // entry of a row is then that of its position inside its sequence, and sequence g's K / V rows go to
    // rows [g * kv_group_pitch, + group_rows) of the K / V destinations (each sequence's cache also holds
    // rows this GEMM does not write). group_rows = 0: one sequence, contiguous K / V.
    int group_rows = 0, kv_group_pitch = 0;
    // split-K
    int splits = 1, k_per_split = 0; float* partial = nullptr; int* counters = nullptr;
    // Programmatic dependent launch: 1 = let the next kernel be scheduled once this CTA's last
    // accumulator is complete (its set-up then overlaps the last epilogue); 0 = only at exit. Set 1
    // only when the next kernel runs one CTA per SM: a kernel with several small CTAs per SM (row
    // norm, SigLIP attention) would be packed onto the few SMs that are idle at that moment.
    int trigger_early = 0;
    // Row norm of A folded into the GEMM (tcgen05 one-SM kernel only, one tile per CTA): A holds the raw rows, the
    // epilogue warps add up each row's sum and sum of squares from the operand stages while the MMAs run, and the
    // accumulator is corrected before bias / activation / RoPE. 1: RMS norm, acc * rstd (eps 1e-6). 2: LayerNorm
    // whose scale and shift were folded into B, colsum and bias_f32 beforehand: rstd * (acc - mean * colsum[n])
    // (eps 1e-5). bias_f32, when set, replaces `bias`.
    int norm_mode = 0;
    const float* colsum = nullptr;
    const float* bias_f32 = nullptr;
};

__device__ __forceinline__ int rope_row(const GemmArgs& p, int row) { return p.group_rows > 0 ? row % p.group_rows : row; }
__device__ __forceinline__ size_t kv_row(const GemmArgs& p, int row) {
    return p.group_rows > 0 ? (size_t)(row / p.group_rows) * p.kv_group_pitch + row % p.group_rows : (size_t)row;
}

// Residual values of one (row, col..col+1) pair. Loaded for every fragment BEFORE any store of
// the epilogue: the residual may alias the destination, so the compiler cannot move a load above
// an earlier store, and interleaving them would serialise one memory latency per fragment.
__device__ __forceinline__ float2 load_residual_pair(const GemmArgs& p, int row, int col) {
    int rr = p.res_mod > 0 ? row % p.res_mod : row;
    return p.c_f32
        ? *reinterpret_cast<const float2*>(static_cast<const float*>(p.R) + (size_t)rr * p.ldr + col)
        : unpack_bf16x2(*reinterpret_cast<const uint32_t*>(static_cast<const bf16*>(p.R) + (size_t)rr * p.ldr + col));
}

template <bool DUAL>
__device__ __forceinline__ void gemm_epilogue_pair(const GemmArgs& p, int row, int col, float a0,
                                                   float a1, float u0, float u1, float2 res) {
    if (p.row_scale) {
        float s = p.row_scale[row];
        a0 *= s; a1 *= s;
        if (DUAL) { u0 *= s; u1 *= s; }
    }
    if (DUAL) { a0 = gelu_f(a0) * u0; a1 = gelu_f(a1) * u1; }
    if (p.bias) {
        float2 b = unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(p.bias + col)));
        a0 += b.x; a1 += b.y;
    }
    if (p.act == 1) { a0 = gelu_f(a0); a1 = gelu_f(a1); }
    else if (p.act == 2) { a0 = silu_f(a0); a1 = silu_f(a1); }
    a0 += res.x; a1 += res.y;
    if (p.rope) {
        const int hd = p.head_dim, qd = p.heads * hd;
        bf16* dst;
        if (col < qd + hd) {
            if (p.round_first) { a0 = round_bf16(a0); a1 = round_bf16(a1); }
            float2 cs = unpack_bf16x2(
                __ldg(reinterpret_cast<const uint32_t*>(p.rope + (size_t)rope_row(p, row) * hd + (col % hd))));
            float r0 = a0 * cs.x - a1 * cs.y, r1 = a1 * cs.x + a0 * cs.y;
            a0 = r0; a1 = r1;
            dst = col < qd ? p.q + (size_t)row * qd + col : p.k + kv_row(p, row) * hd + (col - qd);
        } else {
            dst = p.v + kv_row(p, row) * hd + (col - qd - hd);
        }
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(a0, a1);
        return;
    }
    if (p.c_f32)
        *reinterpret_cast<float2*>(static_cast<float*>(p.C) + (size_t)row * p.ldc + col) = make_float2(a0, a1);
    else
        *reinterpret_cast<uint32_t*>(static_cast<bf16*>(p.C) + (size_t)row * p.ldc + col) = pack_bf16x2(a0, a1);
}

template <int BM, int BN, int STAGES, int WM, int WN, bool DUAL>
__global__ void __launch_bounds__(WM * WN * 32) gemm_mma_kernel(const GemmArgs p) {
    constexpr int BK = 64;
    constexpr int THREADS = WM * WN * 32;
    constexpr int TM = BM / WM, TN = BN / WN;
    constexpr int MI = TM / 16, NI = TN / 8;
    constexpr int NB = DUAL ? 2 : 1;
    constexpr int A_BYTES = BM * BK * 2, B_BYTES = BK * BN * 2;
    constexpr int STAGE_BYTES = A_BYTES + NB * B_BYTES;
    static_assert(TM % 16 == 0 && TN % 16 == 0 && BN >= 64, "tile shape");

    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = smem_u32(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WN, wn = warp % WN;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kbeg = blockIdx.z * p.k_per_split;
    const int kend = min(p.K, kbeg + p.k_per_split);
    const int kb_end = min(kend, p.Kb);
    const int ktiles = (kend - kbeg + BK - 1) / BK;

    auto load_stage = [&](int stage, int kt) {
        const int k0 = kbeg + kt * BK;
        const uint32_t sA = smem_base + stage * STAGE_BYTES;
        for (int idx = tid; idx < BM * 8; idx += THREADS) {
            int r = idx >> 3, c = idx & 7;
            int grow = m0 + r, gk = k0 + c * 8;
            bool ok = grow < p.M && gk < kend;
            const bf16* src = ok ? p.A + (size_t)grow * p.lda + gk : p.A;
            cp_async16(sA + r * 128 + ((c ^ (r & 7)) << 4), src, ok ? 16 : 0);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const bf16* Bp = nb == 0 ? p.B : p.B2;
            const uint32_t sB = sA + A_BYTES + nb * B_BYTES;
            constexpr int CH = BN / 8;
            for (int idx = tid; idx < BK * CH; idx += THREADS) {
                int r = idx / CH, c = idx % CH;
                int gk = k0 + r, gn = n0 + c * 8;
                bool ok = gk < kb_end && gn < p.N;
                const bf16* src = ok ? Bp + (size_t)gk * p.ldb + gn : Bp;
                cp_async16(sB + r * (BN * 2) + ((c ^ (r & 7)) << 4), src, ok ? 16 : 0);
            }
        }
    };

    float acc[NB][MI][NI][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int mi = 0; mi < MI; ++mi)
#pragma unroll
            for (int ni = 0; ni < NI; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nb][mi][ni][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < ktiles) load_stage(s, s);
        cp_async_commit();
    }

    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            int nk = kt + STAGES - 1;
            if (nk < ktiles) load_stage(nk % STAGES, nk);
            cp_async_commit();
        }
        const uint32_t sA = smem_base + (kt % STAGES) * STAGE_BYTES;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t af[MI][4];
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
                int row = wm * TM + mi * 16 + (lane & 15);
                int ch = kk * 2 + (lane >> 4);
                ldmatrix_x4(af[mi], sA + row * 128 + ((ch ^ (row & 7)) << 4));
            }
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const uint32_t sB = sA + A_BYTES + nb * B_BYTES;
#pragma unroll
                for (int nj = 0; nj < NI / 2; ++nj) {
                    int krow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    int ch = (wn * TN + nj * 16) / 8 + (lane >> 4);
                    uint32_t bfr[4];
                    ldmatrix_x4_trans(bfr, sB + krow * (BN * 2) + ((ch ^ (krow & 7)) << 4));
#pragma unroll
                    for (int mi = 0; mi < MI; ++mi) {
                        mma_bf16_16816(acc[nb][mi][2 * nj], af[mi], bfr[0], bfr[1]);
                        mma_bf16_16816(acc[nb][mi][2 * nj + 1], af[mi], bfr[2], bfr[3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();

    const int row_base = m0 + wm * TM + (lane >> 2);
    const int col_base = n0 + wn * TN + (lane & 3) * 2;

    if (p.splits > 1) {
        // Publish this split's partial tile, then let the last-arriving CTA reduce all of them.
        const size_t plane = (size_t)p.splits * p.M * p.N;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < NI; ++ni)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        int row = row_base + mi * 16 + h * 8, col = col_base + ni * 8;
                        if (row < p.M && col < p.N) {
                            float2 v = make_float2(acc[nb][mi][ni][2 * h], acc[nb][mi][ni][2 * h + 1]);
                            __stcg(reinterpret_cast<float2*>(
                                       p.partial + nb * plane + ((size_t)blockIdx.z * p.M + row) * p.N + col), v);
                        }
                    }
        __threadfence();
        __syncthreads();
        __shared__ int s_last;
        if (tid == 0) {
            int tile = blockIdx.y * gridDim.x + blockIdx.x;
            int prev = atomicAdd(p.counters + tile, 1);
            s_last = (prev == p.splits - 1);
            if (s_last) p.counters[tile] = 0;      // self-reset: the graph replays this kernel
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
        // Sum the splits in fixed order 0..splits-1 (deterministic). The split loop is the outer
        // one so that each iteration issues all of this thread's loads before any is consumed.
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                for (int ni = 0; ni < NI; ++ni)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[nb][mi][ni][e] = 0.f;
#pragma unroll 4
        for (int s = 0; s < p.splits; ++s) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int mi = 0; mi < MI; ++mi)
#pragma unroll
                    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            int row = row_base + mi * 16 + h * 8, col = col_base + ni * 8;
                            if (row < p.M && col < p.N) {
                                float2 v = __ldcg(reinterpret_cast<const float2*>(
                                    p.partial + nb * plane + ((size_t)s * p.M + row) * p.N + col));
                                acc[nb][mi][ni][2 * h] += v.x; acc[nb][mi][ni][2 * h + 1] += v.y;
                            }
                        }
        }
    }

    float2 res[MI][NI][2];
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int row = row_base + mi * 16 + h * 8, col = col_base + ni * 8;
                res[mi][ni][h] = (p.R && row < p.M && col < p.N) ? load_residual_pair(p, row, col)
                                                                 : make_float2(0.f, 0.f);
            }
#pragma unroll
    for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < NI; ++ni)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                int row = row_base + mi * 16 + h * 8, col = col_base + ni * 8;
                if (row < p.M && col < p.N)
                    gemm_epilogue_pair<DUAL>(p, row, col, acc[0][mi][ni][2 * h],
                                             acc[0][mi][ni][2 * h + 1],
                                             DUAL ? acc[NB - 1][mi][ni][2 * h] : 0.f,
                                             DUAL ? acc[NB - 1][mi][ni][2 * h + 1] : 0.f, res[mi][ni][h]);
            }
}

// Host side -----------------------------------------------------------------------------------
struct GemmPlan { int skinny; int bn; int tiles_n, tiles_m, splits, k_per_split; size_t ws_bytes; };

inline GemmPlan plan_gemm_mma(int M, int N, int K, bool dual) {
    GemmPlan g{};
    g.skinny = M <= 64;
    g.bn = g.skinny ? 64 : (dual ? 64 : 128);
    g.tiles_n = (N + g.bn - 1) / g.bn;
    g.tiles_m = g.skinny ? 1 : (M + 127) / 128;
    g.splits = 1; g.k_per_split = (K + 63) / 64 * 64;
    if (g.skinny) {
        int ktiles = (K + 63) / 64;
        int want = (160 + g.tiles_n - 1) / g.tiles_n;          // about one CTA per SM
        int max_splits = ktiles / 2 > 0 ? ktiles / 2 : 1;      // at least 128 of K per split
        int s = want < max_splits ? want : max_splits;
        if (s < 1) s = 1;
        int per = (ktiles + s - 1) / s;
        g.k_per_split = per * 64;
        g.splits = (ktiles + per - 1) / per;
    }
    size_t counters = ((size_t)g.tiles_n * g.tiles_m * sizeof(int) + 255) / 256 * 256;
    g.ws_bytes = g.splits > 1 ? counters + (size_t)(dual ? 2 : 1) * g.splits * M * N * sizeof(float) : 0;
    return g;
}

template <int BM, int BN, int STAGES, int WM, int WN, bool DUAL>
inline int launch_gemm_cfg(const GemmArgs& a, dim3 grid, cudaStream_t st) {
    constexpr int smem = STAGES * (BM * 64 * 2 + (DUAL ? 2 : 1) * 64 * BN * 2);
    auto kern = gemm_mma_kernel<BM, BN, STAGES, WM, WN, DUAL>;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    kern<<<grid, WM * WN * 32, smem, st>>>(a);
    return check_launch("gemm_mma_kernel");
}

// Validates, plans and launches. `ws` is only needed when the plan uses split-K.
inline int launch_gemm_mma(GemmArgs a, void* ws, size_t ws_bytes, cudaStream_t st) {
    const bool dual = a.B2 != nullptr;
    if (a.Kb == 0) a.Kb = a.K;
    if (a.M <= 0 || a.N <= 0 || a.K <= 0) { set_error("gemm: empty shape %dx%dx%d", a.M, a.N, a.K); return FVLA_ERR_ARG; }
    if ((a.K % 8) || (a.N % 8) || (a.lda % 8) || (a.ldb % 8)) {
        set_error("gemm: K, N, lda, ldb must be multiples of 8 (got K=%d N=%d lda=%d ldb=%d)", a.K, a.N, a.lda, a.ldb);
        return FVLA_ERR_ARG;
    }
    if (!aligned16(a.A) || !aligned16(a.B) || (dual && !aligned16(a.B2))) { set_error("gemm: operands must be 16-byte aligned"); return FVLA_ERR_ARG; }
    GemmPlan g = plan_gemm_mma(a.M, a.N, a.K, dual);
    a.splits = g.splits; a.k_per_split = g.k_per_split;
    if (g.splits > 1) {
        if (ws == nullptr || ws_bytes < g.ws_bytes) { set_error("gemm: workspace of %zu bytes needed, %zu given", g.ws_bytes, ws_bytes); return FVLA_ERR_WORKSPACE; }
        size_t counters = ((size_t)g.tiles_n * g.tiles_m * sizeof(int) + 255) / 256 * 256;
        a.counters = reinterpret_cast<int*>(ws);
        a.partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ws) + counters);
    }
    dim3 grid(g.tiles_n, g.tiles_m, g.splits);
    if (g.skinny) return dual ? launch_gemm_cfg<64, 64, 4, 2, 2, true>(a, grid, st)
                              : launch_gemm_cfg<64, 64, 4, 2, 2, false>(a, grid, st);
    return dual ? launch_gemm_cfg<128, 64, 3, 2, 4, true>(a, grid, st)
                : launch_gemm_cfg<128, 128, 3, 2, 4, false>(a, grid, st);
}

}  // namespace fvla
