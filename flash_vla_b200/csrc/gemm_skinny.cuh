// Weight-streaming GEMM for the action-expert decoder (M <= 64 tokens): out = x[M,K] @ W[K,N].
//
// These GEMMs are bound by the HBM read of W (5-17 MB per call, read once, always cold), so the
// kernel is built around getting every byte of W in flight at once:
//   * the problem is transposed: the 128-wide slice of N is the MMA's M (TMEM lanes), the tokens
//     are its N = 64 (TMEM columns), so no tensor-core or shared-memory work is spent on padding
//     51 rows to 128;
//   * grid = (N / 128 tiles) x (S K-splits); each CTA owns a W[KC, 128] block, asks TMA for all
//     of it at kernel start (<= 8 boxes of 64 k x 128 n, 128B-swizzled, used in place as an
//     MN-major operand) and issues KC/16 tcgen05.mma into one TMEM accumulator;
//   * the S CTAs of a K-split form a thread-block cluster. Each reads its partial accumulator
//     from TMEM and scatters it over distributed shared memory so that CTA r receives the
//     partials of its slice of tokens; after one cluster barrier CTA r sums them in rank order
//     (deterministic) and runs the fused epilogue: RMS-factor + RoPE + scatter to Q/K/V, GeGLU,
//     bias, or in-place residual add into the fp32 stream.
// The activation operand arrives by TMA as bf16 rows: either the activation itself (bf16) or the bf16
// shadow that the kernels writing the fp32 residual stream keep beside it; the per-token sum of
// squares for the RMS factor is read back from that operand tile in shared memory while the MMAs run
// and is reduced with the partials. (An fp32 activation without a shadow is still accepted: the CTA
// then converts its slice in registers.) No separate norm kernel, no global-memory scratch, no
// semaphores.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "gemm_tc5.cuh"

namespace fvla {
namespace skinny {

using tc5::mbar_init;
using tc5::mbar_expect_tx;
using tc5::mbar_wait;
using tc5::tma_load_2d;
using tc5::smem_desc;

constexpr int TN = 128;          // N columns per CTA (MMA M)
constexpr int TOK = 64;          // token slots (MMA N)
constexpr int MAX_KB = 8;        // k-blocks of 64 per CTA

enum Epi { EPI_QKV_ROPE = 0, EPI_RESIDUAL = 1, EPI_GEGLU = 2, EPI_BIAS = 3 };

struct SkinnyArgs {
    const void* x; int x_f32; int ldx;        // activations [M, K]
    const bf16* x_shadow;                     // optional bf16 copy of an fp32 x, kept current by its writers
    bf16* out_shadow;                         // optional bf16 copy of `out` to maintain (RESIDUAL / BIAS)
    int M, N, K;
    int groups;                               // independent row groups of M rows each, laid end to end (grid.z); 0 or 1 = one
    int kblocks;                              // 64-wide k-blocks per CTA (K / 64 / splits)
    int splits;                               // cluster size along K
    int need_factor;                          // compute rsqrt(mean(x^2)+1e-6) per token
    // epilogue operands
    void* out; int out_f32; int ldo;          // RESIDUAL / BIAS / GEGLU destination
    const bf16* bias; int act;
    const bf16* rope; bf16* q; bf16* k; bf16* v; int heads, head_dim;
    bf16* factor_out;                         // optional bf16 copy of the factors
    int* status;
    uint32_t spin_limit;                       // polls before a wait gives up (0 = the default limit)
    uint32_t expect_extra_bytes;               // self-test only: bytes the owners wait for that no peer sends
    FVLA_DBG_MEMBER
};

// MMA: A = W tile (MN-major, 128 n x 16 k), B = x tile (K-major, 64 tokens x 16 k), D fp32 128x64.
__host__ __device__ constexpr uint32_t skinny_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (0u << 16) | ((uint32_t)(TOK >> 3) << 17) |
           ((uint32_t)(TN >> 4) << 24);
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Shared memory map (offsets from a 1024-byte aligned base):
//   W      max(kblocks, 2) x 16 KB  [kb][atom(2)][64 k rows x 128 B]  (atom = 64 of the tile's 128 n);
//          after the MMAs it is reused as the staging area of this CTA's partial tile
//          ([token 64][n 128] fp32 + 64 partial sums of squares)
//   X      kblocks x 8 KB    [kb][64 tokens x 128 B]           (K-major, 128B swizzle)
//   RED    S x TS x 128 fp32 = 32 KB   partials received from the S ranks, [src][token][n]
//   SSQ    S x TS fp32       partial sums of squares received, [src][token]
//   ssq_local 64 x 2 fp32, barriers, tmem slot, abort flag
constexpr int THREADS = 512;

__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                 uint32_t mbar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(mbar_cluster_addr) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
skinny_gemm_kernel(const SkinnyArgs p, const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmW2,
                   const __grid_constant__ CUtensorMap tmX) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const int KB = p.kblocks, S = p.splits, TS = TOK / S;
    const uint32_t w_bytes = (KB < 2 ? 2 : KB) * 16384u + 1024u;        // + room for the staged sums of squares
    const uint32_t sW = base, sX = sW + w_bytes;
    const uint32_t off_red = w_bytes + KB * 8192u;
    float* stage = reinterpret_cast<float*>(gen);                                // aliases W
    float* red = reinterpret_cast<float*>(gen + off_red);                        // [S][TS][128]
    float* ssq_in = reinterpret_cast<float*>(gen + off_red + 32768);             // [S][TS]
    float* ssq_local = reinterpret_cast<float*>(gen + off_red + 32768 + 256);    // [64][2]
    const uint32_t off_bar = off_red + 32768 + 256 + 512;
    const uint32_t bars = base + off_bar;                                        // KB full barriers, done, incoming
    const uint32_t done_bar = bars + MAX_KB * 8, in_bar = bars + (MAX_KB + 1) * 8;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + off_bar + (MAX_KB + 2) * 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + off_bar + (MAX_KB + 2) * 8 + 8);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    FVLA_DBG_CTA(p, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x);
    FVLA_STAMP(0);
    const uint32_t rank = cluster_ctarank();                 // position along K within the cluster
    const int row0 = blockIdx.z * p.M;                       // first row of this CTA's row group in x / out
    const int tile = blockIdx.x;
    const int k0 = (int)rank * KB * 64;
    const int owners = (p.M + TS - 1) / TS;                  // ranks that own at least one real token
    const bool i_own = (int)rank < owners;

    // bf16 activations are fetched by TMA straight into the operand layout (rows past M read as
    // zero); fp32 activations are converted by the CTA further down.
    const bool x_by_tma = !p.x_f32 || p.x_shadow != nullptr;
    if (tid == 32) { tc5::prefetch_tensormap(&tmW); if (EPI == EPI_GEGLU) tc5::prefetch_tensormap(&tmW2); }
    if (tid == 64 && x_by_tma) tc5::prefetch_tensormap(&tmX);
    if (tid == 0) {
        mbar_init(done_bar, 1);
        mbar_init(in_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (i_own) mbar_expect_tx(in_bar, (uint32_t)(S - 1) * (uint32_t)TS * (512u + (p.need_factor ? 4u : 0u)) + p.expect_extra_bytes);      // S - 1 peers send
    }
    // One lane per k-block sets up that block's barrier and requests its weights: all of this
    // CTA's share of W is in flight within a few hundred cycles of kernel start.
    if (lane == 0 && warp < KB) {
        const int kb = warp;
        mbar_init(bars + kb * 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(bars + kb * 8, x_by_tma ? 16384 + 8192 : 16384);
        if (EPI == EPI_GEGLU) {
            tma_load_2d(sW + kb * 16384, &tmW, bars + kb * 8, tile * 64, k0 + kb * 64);          // gate columns
            tma_load_2d(sW + kb * 16384 + 8192, &tmW2, bars + kb * 8, tile * 64, k0 + kb * 64);  // up columns
        } else {
            tma_load_2d(sW + kb * 16384, &tmW, bars + kb * 8, tile * TN, k0 + kb * 64);
            tma_load_2d(sW + kb * 16384 + 8192, &tmW, bars + kb * 8, tile * TN + 64, k0 + kb * 64);
        }
    }
    __syncwarp();
    if (warp == 0) {
        tc5::tmem_alloc(base + off_bar + (MAX_KB + 2) * 8, 64);
        tc5::tmem_relinquish();
    }
    // Programmatic dependent launch: everything above touched only weights and this CTA's own
    // shared memory, so it may run while the previous kernel in the stream is still finishing.
    // From here on activations written by that kernel are read, so wait for it; then let the
    // next kernel in the stream start its own prologue.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (x_by_tma && lane == 0 && warp < KB)
        tma_load_2d(sX + warp * 8192, &tmX, bars + warp * 8, k0 + warp * 64, row0);
    // Tell the cluster this CTA is running (barriers initialised); peers wait for that before
    // sending anything into its shared memory.
    // (the fence after the barrier initialisation already published it cluster-wide, so a relaxed
    // arrive is enough; a releasing one would also wait for this thread's outstanding requests)
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // Epilogue operands that do not depend on the product (RoPE entries, residual values, bias) are
    // fetched now, so that their latency overlaps the weight stream instead of following the MMA.
    // Owner work items: (token of this rank's slice) x (group of 4 adjacent columns).
    constexpr int QPT = (EPI == EPI_GEGLU) ? 16 : 32;         // column quads per token
    constexpr int PRE = 4;                                    // TS * QPT <= 2048 = 4 x THREADS
    const int items = TS * QPT;
    uint4 pre[PRE];
#pragma unroll
    for (int j = 0; j < PRE; ++j) {
        pre[j] = make_uint4(0, 0, 0, 0);
        const int item = tid + j * THREADS;
        const int tl = item / QPT, c4 = (item % QPT) * 4;
        const int token = (int)rank * TS + tl;
        if (item < items && token < p.M) {
            const int n = tile * TN + c4;
            if (EPI == EPI_QKV_ROPE) {
                if (n < (p.heads + 1) * p.head_dim) {
                    const uint2 cs = __ldg(reinterpret_cast<const uint2*>(p.rope + (size_t)token * p.head_dim + (n % p.head_dim)));
                    pre[j].x = cs.x; pre[j].y = cs.y;
                }
            } else if (EPI == EPI_RESIDUAL) {
                if (p.out_f32) {
                    pre[j] = *reinterpret_cast<const uint4*>(static_cast<const float*>(p.out) + (size_t)(row0 + token) * p.ldo + n);
                } else {
                    const uint2 r = *reinterpret_cast<const uint2*>(static_cast<const bf16*>(p.out) + (size_t)(row0 + token) * p.ldo + n);
                    const float2 r0 = unpack_bf16x2(r.x), r1 = unpack_bf16x2(r.y);
                    pre[j] = make_uint4(__float_as_uint(r0.x), __float_as_uint(r0.y), __float_as_uint(r1.x), __float_as_uint(r1.y));
                }
            } else if (EPI == EPI_BIAS) {
                const uint2 bv = __ldg(reinterpret_cast<const uint2*>(p.bias + n));
                const float2 b0 = unpack_bf16x2(bv.x), b1 = unpack_bf16x2(bv.y);
                pre[j] = make_uint4(__float_as_uint(b0.x), __float_as_uint(b0.y), __float_as_uint(b1.x), __float_as_uint(b1.y));
            }
        }
    }

    FVLA_STAMP(1);
    // Activation slice -> bf16 K-major operand (manual 128B swizzle), plus partial sums of squares.
    // Each thread has four 32-byte loads in flight at a time.
    if (!x_by_tma) {
        const int chunks_per_row = KB * 8;                   // 16-byte (8 x bf16) chunks per token
        const int total = TOK * chunks_per_row;              // 512 (KB = 1) ... 4096 (KB = 8)
        for (int it0 = 0; it0 * THREADS < total; it0 += 4) {
            float4 ra[4], rb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = (it0 + u) * THREADS + tid;
                const int t = idx / chunks_per_row, c = idx % chunks_per_row;
                ra[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                rb[u] = ra[u];
                if (idx < total && t < p.M) {
                    const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.x) + (size_t)(row0 + t) * p.ldx + k0 + c * 8);
                    ra[u] = src[0];
                    rb[u] = src[1];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = (it0 + u) * THREADS + tid;
                if ((it0 + u) * THREADS < total) {           // uniform across the CTA
                    const int t = idx / chunks_per_row, c = idx % chunks_per_row;
                    const int kb = c >> 3, cc = c & 7;
                    uint4 packed = make_uint4(pack_bf16x2(ra[u].x, ra[u].y), pack_bf16x2(ra[u].z, ra[u].w),
                                              pack_bf16x2(rb[u].x, rb[u].y), pack_bf16x2(rb[u].z, rb[u].w));
                    *reinterpret_cast<uint4*>(gen + w_bytes + kb * 8192 + t * 128 + ((cc ^ (t & 7)) << 4)) = packed;
                    if (p.need_factor) {
                        float ss = ra[u].x * ra[u].x + ra[u].y * ra[u].y + ra[u].z * ra[u].z + ra[u].w * ra[u].w +
                                   rb[u].x * rb[u].x + rb[u].y * rb[u].y + rb[u].z * rb[u].z + rb[u].w * rb[u].w;
                        // chunks of one token sit in consecutive lanes: reduce over groups of min(32, chunks_per_row)
                        const int group = chunks_per_row < 32 ? chunks_per_row : 32;
                        for (int o = group >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                        if ((lane & (group - 1)) == 0) ssq_local[t * 2 + (c >> 5)] = ss;      // slot 1 only when KB = 8
                    }
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the MMA
    }
    tc5::tc_fence_before();
    __syncthreads();
    tc5::tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    FVLA_STAMP(2);

    if (tid == 0) {
        constexpr uint32_t idesc = skinny_idesc();
        bool ok = true;
        for (int kb = 0; kb < KB && ok; ++kb) {
            ok = mbar_wait(bars + kb * 8, 0, abort_flag);
            tc5::tc_fence_after();
            if (!ok) break;
#pragma unroll
            for (int k16 = 0; k16 < 4; ++k16) {
                const uint64_t adesc = smem_desc(sW + kb * 16384 + k16 * 2048, 8192, 1024);
                const uint64_t bdesc = smem_desc(sX + kb * 8192 + k16 * 32, 16, 1024);
                tc5::umma_bf16(tmem, adesc, bdesc, idesc, (kb > 0 || k16 > 0) ? 1u : 0u);
            }
        }
        tc5::umma_commit(done_bar);
    }
    __syncwarp();
    if (x_by_tma && p.need_factor) {
        // Sums of squares over this CTA's K slice, read back from the bf16 operand tile in shared
        // memory while the MMAs run (8 lanes per token, one 16-byte chunk per k-block each).
        const int t = tid >> 3, sub = tid & 7;
        float ss = 0.f;
        for (int kb = 0; kb < KB; ++kb) {
            mbar_wait(bars + kb * 8, 0, abort_flag);
            const uint4 a = *reinterpret_cast<const uint4*>(gen + w_bytes + kb * 8192 + t * 128 + sub * 16);
            const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
            ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y + f2.x * f2.x + f2.y * f2.y + f3.x * f3.x + f3.y * f3.y;
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (sub == 0) { ssq_local[t * 2] = ss; ssq_local[t * 2 + 1] = 0.f; }
    }
    const bool done = mbar_wait(done_bar, 0, abort_flag);
    tc5::tc_fence_after();
    FVLA_STAMP(3);
    __syncthreads();                                   // sums of squares are complete
    // Stage this CTA's partial tile as [token][n] fp32 over the (now idle) weight region. All 16 warps
    // take part: warp w reads TMEM lanes 32 (w & 3) .. + 32 (its n) and token columns 16 (w >> 2) .. + 16.
    {
        const int q = warp & 3, g = warp >> 2;
        float part[16];
        tc5::tmem_ld16(tmem + ((uint32_t)(q * 32) << 16) + g * 16, part);
#pragma unroll
        for (int t = 0; t < 16; ++t) stage[(g * 16 + t) * TN + q * 32 + lane] = done ? part[t] : 0.f;
    }
    if (p.need_factor && tid < TOK)
        stage[TOK * TN + tid] = tid < p.M ? ssq_local[tid * 2] + (KB == 8 ? ssq_local[tid * 2 + 1] : 0.f) : 0.f;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // staging writes -> visible to the bulk copies
    tc5::tc_fence_before();
    __syncthreads();
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // every peer has initialised its barriers
    if (tid == 0) {
        // one bulk copy per owner: its slice of tokens goes to slot [src = my rank] of its RED buffer
        for (int r = 0; r < owners; ++r) {
            if (r == (int)rank) continue;                    // the owner reads its own slice where it was staged
            bulk_copy_to_cta(map_to_cta(base + off_red + (uint32_t)(rank * TS) * 512u, (uint32_t)r),
                             base + (uint32_t)(r * TS) * 512u, (uint32_t)TS * 512u, map_to_cta(in_bar, (uint32_t)r));
            if (p.need_factor)
                bulk_copy_to_cta(map_to_cta(base + off_red + 32768 + (uint32_t)(rank * TS) * 4u, (uint32_t)r),
                                 base + (uint32_t)(TOK * TN) * 4u + (uint32_t)(r * TS) * 4u, (uint32_t)TS * 4u,
                                 map_to_cta(in_bar, (uint32_t)r));
        }
    }

    FVLA_STAMP(4);
    // Owner phase: this CTA finishes tokens [rank*TS, rank*TS + TS), summing partials in rank order.
    if (i_own) {
        mbar_wait(in_bar, 0, abort_flag, p.spin_limit ? p.spin_limit : tc5::kSpinLimit);
        FVLA_STAMP(5);
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
            const int item = tid + j * THREADS;
            const int tl = item / QPT, c4 = (item % QPT) * 4;
            const int token = (int)rank * TS + tl;
            if (item >= items || token >= p.M) continue;
            // partial of source rank s for this token: received in RED, or (own rank) still in the staging area
            auto part_row = [&](int s) { return s == (int)rank ? stage + ((int)rank * TS + tl) * TN : red + (s * TS + tl) * TN; };
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < S; ++s) {
                const float4 v = *reinterpret_cast<const float4*>(part_row(s) + c4);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            float factor = 1.f;
            if (p.need_factor) {
                float ss = 0.f;
                for (int s = 0; s < S; ++s) ss += s == (int)rank ? stage[TOK * TN + (int)rank * TS + tl] : ssq_in[s * TS + tl];
                factor = rsqrtf(ss * (1.0f / (float)p.K) + 1e-6f);
                if (p.factor_out && tile == 0 && c4 == 0) p.factor_out[token] = __float2bfloat16_rn(factor);
            }
            const int n = tile * TN + c4;
            if (EPI == EPI_QKV_ROPE) {
                float v0 = sum.x * factor, v1 = sum.y * factor, v2 = sum.z * factor, v3 = sum.w * factor;
                const int hd = p.head_dim, qd = p.heads * hd;
                bf16* dst;
                if (n < qd + hd) {
                    const float2 c0 = unpack_bf16x2(pre[j].x), c1 = unpack_bf16x2(pre[j].y);
                    const float r0 = v0 * c0.x - v1 * c0.y, r1 = v1 * c0.x + v0 * c0.y;
                    const float r2 = v2 * c1.x - v3 * c1.y, r3 = v3 * c1.x + v2 * c1.y;
                    v0 = r0; v1 = r1; v2 = r2; v3 = r3;
                    dst = n < qd ? p.q + (size_t)token * qd + n : p.k + (size_t)token * hd + (n - qd);
                } else {
                    dst = p.v + (size_t)token * hd + (n - qd - hd);
                }
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3));
            } else if (EPI == EPI_GEGLU) {
                // columns 0..63 of the tile are gate columns, 64..127 the matching up columns
                float4 up = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s = 0; s < S; ++s) {
                    const float4 v = *reinterpret_cast<const float4*>(part_row(s) + 64 + c4);
                    up.x += v.x; up.y += v.y; up.z += v.z; up.w += v.w;
                }
                const float f2 = factor;
                *reinterpret_cast<uint2*>(static_cast<bf16*>(p.out) + (size_t)(row0 + token) * p.ldo + tile * 64 + c4) =
                    make_uint2(pack_bf16x2(gelu_f(sum.x * f2) * (up.x * f2), gelu_f(sum.y * f2) * (up.y * f2)),
                               pack_bf16x2(gelu_f(sum.z * f2) * (up.z * f2), gelu_f(sum.w * f2) * (up.w * f2)));
            } else {
                float v0 = sum.x, v1 = sum.y, v2 = sum.z, v3 = sum.w;
                // pre = bias (EPI_BIAS) or residual (EPI_RESIDUAL), as four floats
                v0 += __uint_as_float(pre[j].x); v1 += __uint_as_float(pre[j].y);
                v2 += __uint_as_float(pre[j].z); v3 += __uint_as_float(pre[j].w);
                if (EPI == EPI_BIAS && p.act == 2) { v0 = silu_f(v0); v1 = silu_f(v1); v2 = silu_f(v2); v3 = silu_f(v3); }
                if (p.out_shadow)
                    *reinterpret_cast<uint2*>(p.out_shadow + (size_t)(row0 + token) * p.ldo + n) =
                        make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3));
                if (p.out_f32)
                    *reinterpret_cast<float4*>(static_cast<float*>(p.out) + (size_t)(row0 + token) * p.ldo + n) = make_float4(v0, v1, v2, v3);
                else
                    *reinterpret_cast<uint2*>(static_cast<bf16*>(p.out) + (size_t)(row0 + token) * p.ldo + n) =
                        make_uint2(pack_bf16x2(v0, v1), pack_bf16x2(v2, v3));
            }
        }
    }

    // No CTA may leave while a peer can still be reading its staging area: once every owner has
    // received all of its slices, every outgoing copy of every CTA has completed.
    FVLA_STAMP(6);
    tc5::tc_fence_before();
    // (execution barrier only: nothing read after it was written by a peer)
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
    if (warp == 0) {
        tc5::tc_fence_after();
        tc5::tmem_dealloc(tmem, 64);
    }
    FVLA_STAMP(7);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 2);
}

// ---- host side ---------------------------------------------------------------------------------
struct SkinnyPlan { int splits, kblocks, tiles; size_t smem; bool ok; };

inline SkinnyPlan plan_skinny(int M, int N, int K, bool geglu, int groups = 1) {
    SkinnyPlan pl{};
    pl.ok = false;
    const int tile_n = geglu ? 64 : TN;
    if (M <= 0 || M > TOK || N % tile_n || K % 64) return pl;
    pl.tiles = N / tile_n;
    const int kb_total = K / 64;
    PlanChoice pinned;
    if (plan_lookup(M, N, K, geglu ? PLAN_SKINNY_DUAL : PLAN_SKINNY, &pinned)) {
        // a pinned cluster size: 1, 2, 4 or 8 CTAs along K, at most 8 k-blocks each
        const int s = pinned.splits;
        if (s < 1 || s > 8 || (s & (s - 1)) || kb_total % s || kb_total / s > MAX_KB || ((kb_total / s) & (kb_total / s - 1))) return pl;
        pl.splits = s;
        pl.kblocks = kb_total / s;
        pl.smem = 1024 + (size_t)(pl.kblocks < 2 ? 2 : pl.kblocks) * 16384 + 1024 + (size_t)pl.kblocks * 8192 + 32768 + 256 + 512 +
                  (MAX_KB + 2) * 8 + 32;
        pl.ok = true;
        return pl;
    }
    // largest cluster (<= 8) that divides the k-blocks, keeps <= 8 k-blocks per CTA and stays near one wave
    int best = 0;
    for (int s = 1; s <= 8; s *= 2) {       // 8 = largest portable cluster; larger ones schedule in waves
        if (kb_total % s) continue;
        const int kb = kb_total / s;
        if (kb > MAX_KB || kb < 1 || (kb & (kb - 1))) continue;
        if (pl.tiles * s > 148 && best) break;
        best = s;
    }
    if (!best) return pl;
    if (groups > 1) {
        // Several row groups in one launch multiply the CTA count. Clusters are placed GPC by GPC: about 33
        // clusters of 4 or 15 of 8 are resident at once, so prefer the largest split whose clusters of all
        // groups are resident together (one wave) over the single-group choice.
        for (int s = best; s >= 1; s /= 2) {
            const int kb = kb_total / s;
            if (kb_total % s || kb > MAX_KB) break;
            const int resident = s >= 8 ? 15 * 8 : (s == 4 ? 33 * 4 : 148);
            if (pl.tiles * s * groups <= resident) { best = s; break; }
        }
    }
    pl.splits = best;
    pl.kblocks = kb_total / best;
    pl.smem = 1024 + (size_t)(pl.kblocks < 2 ? 2 : pl.kblocks) * 16384 + 1024 + (size_t)pl.kblocks * 8192 + 32768 + 256 + 512 +
              (MAX_KB + 2) * 8 + 32;
    pl.ok = true;
    return pl;
}

template <int EPI>
inline int launch_skinny(SkinnyArgs a, const void* W, const void* W2, int ldw, cudaStream_t st) {
    SkinnyPlan pl = plan_skinny(a.M, a.N, a.K, EPI == EPI_GEGLU, a.groups > 1 ? a.groups : 1);
    if (!pl.ok) { set_error("skinny gemm: shape %dx%dx%d not supported", a.M, a.N, a.K); return FVLA_ERR_UNSUPPORTED; }
    a.splits = pl.splits; a.kblocks = pl.kblocks;
    const int groups = a.groups > 1 ? a.groups : 1;
    if (groups > 1 && (EPI == EPI_QKV_ROPE || a.need_factor || (a.x_f32 && a.x_shadow == nullptr))) {
        set_error("skinny gemm: row groups are only built for the bias / residual forms with a bf16 operand");
        return FVLA_ERR_UNSUPPORTED;
    }
    auto kern = skinny_gemm_kernel<EPI>;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    CUtensorMap tmW, tmW2, tmX;
    int rc = tc5::make_map(&tmW, W, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)ldw, 64, 64);
    if (rc) return rc;
    rc = tc5::make_map(&tmW2, W2 ? W2 : W, (uint64_t)a.N, (uint64_t)a.K, (uint64_t)ldw, 64, 64);
    if (rc) return rc;
    if (a.x_f32 && a.x_shadow == nullptr) tmX = tmW;         // unused by the kernel in this case
    else rc = tc5::make_map(&tmX, a.x_f32 ? (const void*)a.x_shadow : a.x, (uint64_t)a.K, (uint64_t)a.M * groups, (uint64_t)a.ldx, 64, 64);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(pl.tiles, pl.splits, groups);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = pl.smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = pl.splits;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, tmW, tmW2, tmX);
    if (e != cudaSuccess) { set_error("skinny_gemm_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("skinny_gemm_kernel");
}

}  // namespace skinny
}  // namespace fvla
