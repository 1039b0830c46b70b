// Streaming-softmax attention for the three attention shapes of Pi0.
//
//   * SigLIP: per (view, head), 256 queries x 256 keys, head_dim 72 (padded to 80 in shared
//     memory), Q/K/V interleaved in one packed (tokens, 3 * 1152) buffer.
//   * Prefix encoder: multi-query; the (token, head) axes collapse to one flat query axis of
//     S * 8 rows against one K/V head of S keys, head_dim 256, unmasked.
//   * Action-expert decoder: same flat multi-query form, 408 queries x (S + 51) keys, with the
//     Pi0 mask (the state token's 8 rows see keys j <= S only) and the keys split across CTAs
//     (flash-decoding); a second kernel merges the per-split partials by log-sum-exp.
//
// One CTA = 64 query rows, 4 warps of 16 rows; K/V stream through a 2-stage cp.async ring in
// 64-key blocks; scores and probabilities never leave registers.
#pragma once

#include "common.cuh"
#include "gemm_tc5.cuh"

namespace fvla {

struct AttnArgs {
    const bf16* q; const bf16* k; const bf16* v;
    bf16* out;                 // direct mode: (nq, o_stride) rows
    float* part_o;             // split mode: (splits, nq_pad, HD) fp32, normalised per split
    float* part_lse;           // split mode: (splits, nq_pad) log2-domain log-sum-exp
    int q_stride, k_stride, v_stride, o_stride;          // row strides in elements
    long long q_bs0, q_bs1, k_bs0, k_bs1, v_bs0, v_bs1, o_bs0, o_bs1;   // batch strides
    int batch_inner;           // blockIdx.y = b0 * batch_inner + b1
    int nq, nk, hd;            // rows, keys, real head dim
    int nq_pad;
    float scale_log2;          // softmax scale * log2(e)
    int mask_rows, mask_key_le;   // rows < mask_rows only see keys j <= mask_key_le
    int splits, keys_per_split;
};

// HD: padded head dim, multiple of 16. STAGES: K/V tiles in shared memory; 2 overlaps the next
// tile's load with this tile's math inside the CTA, 1 halves the footprint so that two CTAs share an SM
// and overlap each other instead.
template <int HD, int STAGES>
__global__ void __launch_bounds__(128) attention_kernel(const AttnArgs p) {
    constexpr int BQ = 64, BKV = 64;
    constexpr int PITCH = HD * 2 + 16;          // bytes; +16 keeps ldmatrix rows on distinct banks
    constexpr int CH = HD / 8;                  // 16-byte chunks per row
    constexpr int TILE = 64 * PITCH;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sKV = sQ + TILE;             // stage s: K at sKV + s*2*TILE, V right after

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may be scheduled
    asm volatile("griddepcontrol.wait;" ::: "memory");      // no-op unless launched as a dependent
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * BQ;
    const int b0 = blockIdx.y / p.batch_inner, b1 = blockIdx.y % p.batch_inner;
    const bf16* Q = p.q + b0 * p.q_bs0 + b1 * p.q_bs1;
    const bf16* K = p.k + b0 * p.k_bs0 + b1 * p.k_bs1;
    const bf16* V = p.v + b0 * p.v_bs0 + b1 * p.v_bs1;
    const int split = blockIdx.z;
    const int key_beg = split * p.keys_per_split;
    const int key_end = min(p.nk, key_beg + p.keys_per_split);
    const int nblocks = (key_end - key_beg + BKV - 1) / BKV;
    const int hd_chunks = (p.hd + 7) / 8;       // chunks holding real data (hd % 8 == 0)

    auto load_rows = [&](uint32_t dst, const bf16* src, int stride, int row0, int row_end) {
        for (int idx = tid; idx < 64 * CH; idx += 128) {
            int r = idx / CH, c = idx % CH;
            bool ok = (row0 + r) < row_end && c < hd_chunks;
            const bf16* s = ok ? src + (size_t)(row0 + r) * stride + c * 8 : src;
            cp_async16(dst + r * PITCH + c * 16, s, ok ? 16 : 0);
        }
    };

    load_rows(sQ, Q, p.q_stride, q0, p.nq);
    if (nblocks > 0) {
        load_rows(sKV, K, p.k_stride, key_beg, key_end);
        load_rows(sKV + TILE, V, p.v_stride, key_beg, key_end);
    }
    cp_async_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int row_lo = q0 + warp * 16 + (lane >> 2);      // this thread's two rows: row_lo, row_lo + 8

    for (int jb = 0; jb < nblocks; ++jb) {
        const int stage = STAGES == 2 ? (jb & 1) : 0;
        if (STAGES == 2) {
            if (jb + 1 < nblocks) {
                const int kb = key_beg + (jb + 1) * BKV;
                load_rows(sKV + (stage ^ 1) * 2 * TILE, K, p.k_stride, kb, key_end);
                load_rows(sKV + (stage ^ 1) * 2 * TILE + TILE, V, p.v_stride, kb, key_end);
            }
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            if (jb > 0) {                    // the barrier closing the previous iteration freed the tile
                const int kb = key_beg + jb * BKV;
                load_rows(sKV, K, p.k_stride, kb, key_end);
                load_rows(sKV + TILE, V, p.v_stride, kb, key_end);
                cp_async_commit();
            }
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t sK = sKV + stage * 2 * TILE, sV = sK + TILE;

        // S = Q K^T for this warp's 16 rows x 64 keys
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t a[4];
            ldmatrix_x4(a, sQ + (warp * 16 + (lane & 15)) * PITCH + (kk * 2 + (lane >> 4)) * 16);
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
                uint32_t b[4];
                int key = nj * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(b, sK + key * PITCH + (kk * 2 + ((lane >> 3) & 1)) * 16);
                mma_bf16_16816(s[2 * nj], a, b[0], b[1]);
                mma_bf16_16816(s[2 * nj + 1], a, b[2], b[3]);
            }
        }

        // scale, mask, online softmax (log2 domain)
        const int kbase = key_beg + jb * BKV;
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int key = kbase + ni * 8 + (lane & 3) * 2 + (e & 1);
                int row = row_lo + (e >> 1) * 8;
                bool keep = key < key_end && (row >= p.mask_rows || key <= p.mask_key_le);
                float v = keep ? s[ni][e] * p.scale_log2 : -INFINITY;
                s[ni][e] = v;
                m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
            m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
        }
        float alpha[2], m_use[2], psum[2] = {0.f, 0.f};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            m_use[h] = m_new[h] == -INFINITY ? 0.f : m_new[h];       // fully masked so far
            alpha[h] = exp2f(m_run[h] - m_use[h]);                   // m_run = -inf -> 0
            m_run[h] = m_new[h];
        }
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float pv = exp2f(s[ni][e] - m_use[e >> 1]);
                s[ni][e] = pv;
                psum[e >> 1] += pv;
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            l_run[h] = l_run[h] * alpha[h] + psum[h];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
            o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dj = 0; dj < HD / 16; ++dj) {
                uint32_t b[4];
                int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(b, sV + key * PITCH + (dj * 2 + (lane >> 4)) * 16);
                mma_bf16_16816(o[2 * dj], a, b[0], b[1]);
                mma_bf16_16816(o[2 * dj + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();       // everyone is done with this stage before it is refilled
    }
    cp_async_wait<0>();

    float inv[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) inv[h] = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;

    if (p.part_o) {
        float* po = p.part_o + ((size_t)split * p.nq_pad) * HD;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            int row = row_lo + h * 8;
            if (row < p.nq) {
#pragma unroll
                for (int i = 0; i < HD / 8; ++i) {
                    int d = i * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2*>(po + (size_t)row * HD + d) =
                        make_float2(o[i][2 * h] * inv[h], o[i][2 * h + 1] * inv[h]);
                }
                if ((lane & 3) == 0)
                    p.part_lse[(size_t)split * p.nq_pad + row] =
                        l_run[h] > 0.f ? m_run[h] + log2f(l_run[h]) : -INFINITY;
            }
        }
        return;
    }
    bf16* O = p.out + b0 * p.o_bs0 + b1 * p.o_bs1;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        int row = row_lo + h * 8;
        if (row < p.nq) {
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                int d = i * 8 + (lane & 3) * 2;
                if (d < p.hd)
                    *reinterpret_cast<uint32_t*>(O + (size_t)row * p.o_stride + d) =
                        pack_bf16x2(o[i][2 * h] * inv[h], o[i][2 * h + 1] * inv[h]);
            }
        }
    }
}

// Merge flash-decoding partials: out[row] = sum_s w_s O_s / sum_s w_s, w_s = 2^(lse_s - max lse).
__global__ void __launch_bounds__(128) attention_combine_kernel(const float* __restrict__ part_o,
                                                                const float* __restrict__ part_lse,
                                                                bf16* __restrict__ out, int nq,
                                                                int nq_pad, int hd, int splits) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // no-op unless launched as a dependent
    const int row = blockIdx.x * 2 + (threadIdx.x >> 6);
    const int t = threadIdx.x & 63;
    if (row >= nq) return;
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_lse[(size_t)s * nq_pad + row]);
    float wsum = 0.f;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < splits; ++s) {
        float l = part_lse[(size_t)s * nq_pad + row];
        float w = (l == -INFINITY) ? 0.f : exp2f(l - mx);
        wsum += w;
        if (w != 0.f && t * 4 < hd) {
            float4 v = *reinterpret_cast<const float4*>(part_o + ((size_t)s * nq_pad + row) * hd + t * 4);
            acc[0] += w * v.x; acc[1] += w * v.y; acc[2] += w * v.z; acc[3] += w * v.w;
        }
    }
    if (t * 4 < hd) {
        float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
        uint2 pk = make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
        *reinterpret_cast<uint2*>(out + (size_t)row * hd + t * 4) = pk;
    }
}

template <int HD, int STAGES = 2>
inline int launch_attention(const AttnArgs& a, dim3 grid, cudaStream_t st) {
    constexpr int smem = (1 + 2 * STAGES) * 64 * (HD * 2 + 16);
    auto kern = attention_kernel<HD, STAGES>;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    cudaError_t e = launch_pdl(kern, grid, dim3(128), smem, st, a);
    if (e != cudaSuccess) { set_error("attention_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("attention_kernel");
}


// ---------------------------------------------------------------------------------------------
// Decoder attention in one launch: keys split over the CTAs of a thread-block cluster (8 for up to
// 1024 keys, one more per further 128 keys, at most 11), partial results merged through distributed
// shared memory (no partial buffers in global memory, no second kernel). Grid = (ceil(queries / 32),
// splits), cluster (1, splits), 8 warps per CTA. Warp w works on
// query rows 16 (w & 1) .. + 16 of the 32-row block, key block (w >> 1) & 1 of the CTA's <= 128 keys
// and half (w >> 2) of the head dimension: it sums Q K^T over its 128 of the 256 dimensions, swaps
// that partial 16 x 64 score tile with the warp holding the other half (both then own the full
// scores and run the same softmax) and multiplies P with its 128 columns of V. The two key blocks are
// merged in shared memory, the normalised 32 x 256 partial and its log-sum-exp are staged, and rank
// r < 8 receives rows 4r .. 4r+3 from all ranks by bulk copy, combines them with log-sum-exp weights
// in rank order and writes bf16.
// ---------------------------------------------------------------------------------------------
struct DecAttnArgs {
    const bf16* q; const bf16* k; const bf16* v; bf16* out;
    int nq, nk, keys_per_split;
    int splits;                 // cluster size: CTAs sharing the keys of one 32-row query block (8..11)
    // a batch of independent episodes (grid.z): element offsets between consecutive episodes' Q / out rows
    // and between their K / V caches; nq and nk are per episode
    long long q_episode_stride, kv_episode_stride;
    int episodes;
    float scale_log2;
    int mask_rows, mask_key_le;
    int prefix_keys;            // keys [0, prefix_keys) were not written by the preceding kernel
    int* status;
    FVLA_DBG_MEMBER
};

namespace decattn {
constexpr int HD = 256, BQ = 32, MIN_SPL = 8, MAX_SPL = 11, PITCH = HD * 2 + 16, CH = HD / 8, THREADS = 256;
constexpr int OP = HD + 8;                          // fp32 row pitch of the merge / staging buffers: rows 8 banks apart
constexpr int SLICE = 4 * OP * 4;                   // bytes of the 4 staged rows one owner receives from one rank
// K and V tiles: 128 keys x 256 dims as four 64-dim blocks of [128 rows][128 bytes] in the 128-byte swizzle a tensor
// load writes (16-byte piece c of row r at piece c ^ (r & 7): eight consecutive keys of one piece sit in eight
// different bank groups, which is what ldmatrix wants); the tiles lead the buffer so that they are 1 KB aligned.
// Q keeps the padded row pitch.
constexpr int Q_BYTES = BQ * PITCH, KV_BYTES = 128 * HD * 2, KV_BLOCK = 128 * 128;
constexpr int OFF_K = 0, OFF_V = OFF_K + KV_BYTES, OFF_Q = OFF_V + KV_BYTES;
constexpr int OFF_SX = OFF_Q + Q_BYTES;                                                  // score swap: [warp 8][32][lane 32] fp32
constexpr int OFF_BAR = OFF_SX + 8 * 32 * 32 * 4;
constexpr int OFF_RED = OFF_BAR + 64;                                                    // RED: [src spl][4 rows][OP] fp32, then LSE_IN [src spl][4] fp32
constexpr int smem_bytes(int spl) { return 1024 + OFF_RED + spl * (SLICE + 16); }      // 1 KB of slack to align the tiles
// shared-memory address of 16-byte piece `piece` (0..31) of row `row` of a K / V tile
__device__ __forceinline__ uint32_t kv_piece(uint32_t tile, int row, int piece) {
    return tile + (uint32_t)(piece >> 3) * KV_BLOCK + (uint32_t)row * 128u + (uint32_t)(((piece & 7) ^ (row & 7)) << 4);
}
static_assert(smem_bytes(MAX_SPL) <= 227 * 1024, "the largest cluster's receive buffers must fit in shared memory");
// staging areas alias K (half-merge buffer) and V (final partial) once the MMAs are done
constexpr int OFF_HALF = OFF_K;                    // [32 rows][OP] fp32 + m[32] + l[32]
constexpr int OFF_STAGE = OFF_V;                   // [32 rows][OP] fp32 + lse[32]
static_assert(BQ * OP * 4 + 256 <= KV_BYTES, "merge buffers must fit in the K / V tiles they alias");
}  // namespace decattn

__device__ __forceinline__ uint32_t dsm_map(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

__global__ void __launch_bounds__(decattn::THREADS, 1)
decoder_attention_cluster_kernel(const DecAttnArgs p, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV) {
    using namespace decattn;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
    const uint32_t sQ = sbase + OFF_Q, sK = sbase + OFF_K, sV = sbase + OFF_V;
    const uint32_t in_bar = sbase + OFF_BAR;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_BAR + 16);
    const int SPL = p.splits;
    const int OFF_LSE_IN = OFF_RED + SPL * SLICE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    FVLA_DBG_CTA(p, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x);
    FVLA_STAMP(0);
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const bf16* gq = p.q + (size_t)blockIdx.z * p.q_episode_stride;
    const bf16* gk = p.k + (size_t)blockIdx.z * p.kv_episode_stride;
    const bf16* gv = p.v + (size_t)blockIdx.z * p.kv_episode_stride;
    bf16* gout = p.out + (size_t)blockIdx.z * p.q_episode_stride;
    const int q0 = blockIdx.x * BQ;
    const int key_beg = (int)rank * p.keys_per_split;
    const int key_end = min(p.nk, key_beg + p.keys_per_split);
    const int rows_here = min(BQ, p.nq - q0);
    const int owners = (rows_here + 3) / 4;                  // at most 8: ranks beyond that only send
    const bool i_own = (int)rank < owners;

    // Prefix keys were written long before the preceding kernel: fetch them while it finishes. Rows
    // past the end (keys of the ragged last split, queries of the last block) must read as zero.
    const int pre_end = min(key_end, p.prefix_keys);
    const uint32_t pre_bar = sbase + OFF_BAR + 24;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(in_bar) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(pre_bar) : "memory");
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (i_own)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(in_bar), "r"(SPL * (SLICE + 16)) : "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pre_bar), "r"(2 * KV_BYTES) : "memory");      // whole boxes, zero fill included
    }
    // relaxed: the fence above already published the barrier to the cluster
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // The prefix K and V rows (almost all of the tile) arrive as four tensor loads per tile (64 dims x 128 keys each)
    // through maps that END at the prefix: the rows behind it, which the preceding kernel is still writing, are
    // not touched in memory and read as zero. Eight copy requests per CTA, which is what a CTA that could only
    // start after the previous kernel left its SM waits for.
    auto bounded_wait = [&](uint32_t bar) {
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(bar), "r"(0) : "memory");
            if (done) return;
            if ((i & 1023u) == 1023u && *abort_flag) return;
        }
        *abort_flag = 1;
    };
    __syncthreads();                                           // the barriers are initialised
    if (tid == 0) {
#pragma unroll
        for (int cb = 0; cb < HD / 64; ++cb) {
            tc5::tma_load_3d(sK + cb * KV_BLOCK, &tmK, pre_bar, cb * 64, key_beg, blockIdx.z);
            tc5::tma_load_3d(sV + cb * KV_BLOCK, &tmV, pre_bar, cb * 64, key_beg, blockIdx.z);
        }
    }
    // (Rows of the tile past this split's last key hold the next split's keys, or zeros past the prefix: their
    // scores are masked below and their probabilities are zero, so they need no clearing.)
    for (int idx = tid; idx < BQ * CH; idx += THREADS) {
        int r = idx / CH, c = idx % CH;
        if (q0 + r >= p.nq) *reinterpret_cast<uint4*>(smem + OFF_Q + r * PITCH + c * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    FVLA_STAMP(1);
    // What the preceding kernel wrote (Q, and the new keys in the last split) is small and is what every CTA
    // waits for next: 16-byte async copies reach shared memory sooner than a bulk copy does (about 1.0 us
    // against 1.4 us from request to data), so they keep the old path.
    {
        const int post_lo = max(key_beg, pre_end);
        for (int idx = tid; idx < BQ * CH; idx += THREADS) {
            const int r = idx / CH, c = idx % CH;
            if (q0 + r < p.nq) cp_async16(sQ + r * PITCH + c * 16, gq + (size_t)(q0 + r) * HD + c * 8, 16);
        }
        cp_async_commit();
        if (post_lo < key_end) {
            // the new keys land on rows the tensor loads zero-filled: wait for those loads first
            bounded_wait(pre_bar);
            for (int idx = tid; idx < 128 * CH; idx += THREADS) {
                const int r = idx / CH, c = idx % CH, g = key_beg + r;
                if (g >= post_lo && g < key_end) {
                    cp_async16(kv_piece(sK, r, c), gk + (size_t)g * HD + c * 8, 16);
                    cp_async16(kv_piece(sV, r, c), gv + (size_t)g * HD + c * 8, 16);
                }
            }
            cp_async_commit();
        }
        cp_async_wait<0>();
    }
    bounded_wait(pre_bar);
    __syncthreads();
    FVLA_STAMP(2);

    const int rg = warp & 1, kh = (warp >> 1) & 1, dh = warp >> 2;
    const int row_lo = q0 + rg * 16 + (lane >> 2);
    float o[HD / 16][4];                               // this warp's 128 output columns
    float m_run[2], l_run[2];
    {
        const int kv_row0 = kh * 64;                       // this warp's half of the tile's keys
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int k8 = 0; k8 < HD / 32; ++k8) {
            const int kk = dh * (HD / 32) + k8;
            uint32_t a[4];
            ldmatrix_x4(a, sQ + (rg * 16 + (lane & 15)) * PITCH + (kk * 2 + (lane >> 4)) * 16);
#pragma unroll
            for (int nj = 0; nj < 4; ++nj) {
                uint32_t b[4];
                int key = nj * 16 + (lane & 7) + (lane >> 4) * 8;
                ldmatrix_x4(b, kv_piece(sK, kv_row0 + key, kk * 2 + ((lane >> 3) & 1)));
                mma_bf16_16816(s[2 * nj], a, b[0], b[1]);
                mma_bf16_16816(s[2 * nj + 1], a, b[2], b[3]);
            }
        }
        // Swap partial scores with the warp that summed the other half of the head dimension (same rows,
        // same keys, hence the same fragment layout: element j of lane l pairs with element j of lane l).
        {
            float* sx = reinterpret_cast<float*>(smem + OFF_SX);
            float* mine = sx + warp * 1024;
            const float* theirs = sx + (warp ^ 4) * 1024;
#pragma unroll
            for (int ni = 0; ni < 8; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) mine[(ni * 4 + e) * 32 + lane] = s[ni][e];
            asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp & 3)) : "memory");
#pragma unroll
            for (int ni = 0; ni < 8; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[ni][e] += theirs[(ni * 4 + e) * 32 + lane];
        }
        const int kbase = key_beg + kh * 64;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int key = kbase + ni * 8 + (lane & 3) * 2 + (e & 1);
                int row = row_lo + (e >> 1) * 8;
                bool keep = key < key_end && (row >= p.mask_rows || key <= p.mask_key_le);
                float v = keep ? s[ni][e] * p.scale_log2 : -INFINITY;
                s[ni][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float psum[2] = {0.f, 0.f}, m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            m_use[h] = mx[h] == -INFINITY ? 0.f : mx[h];
            m_run[h] = mx[h];
        }
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float pv = exp2f(s[ni][e] - m_use[e >> 1]);
                s[ni][e] = pv;
                psum[e >> 1] += pv;
            }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 1);
            psum[h] += __shfl_xor_sync(0xffffffffu, psum[h], 2);
            l_run[h] = psum[h];
        }
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dl = 0; dl < HD / 32; ++dl) {
                const int dj = dh * (HD / 32) + dl;
                uint32_t b[4];
                int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4_trans(b, kv_piece(sV, kv_row0 + key, dj * 2 + (lane >> 4)));
                mma_bf16_16816(o[2 * dl], a, b[0], b[1]);
                mma_bf16_16816(o[2 * dl + 1], a, b[2], b[3]);
            }
        }
    }
    __syncthreads();                                   // K and V are dead from here on
    FVLA_STAMP(3);

    float* half_o = reinterpret_cast<float*>(smem + OFF_HALF);            // [32][OP]
    float* half_ml = half_o + BQ * OP;                                      // m[32], l[32]
    float* stage_o = reinterpret_cast<float*>(smem + OFF_STAGE);          // [32][OP]
    float* stage_lse = stage_o + BQ * OP;                                   // [32]
    const int r_in_blk = rg * 16 + (lane >> 2);
    const int c_base = dh * (HD / 2) + (lane & 3) * 2;                      // column of o[i][0]: c_base + 8 i
    if (kh == 1) {
#pragma unroll
        for (int i = 0; i < HD / 16; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h)
                *reinterpret_cast<float2*>(half_o + (r_in_blk + h * 8) * OP + c_base + i * 8) = make_float2(o[i][2 * h], o[i][2 * h + 1]);
        if (dh == 0 && (lane & 3) == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                half_ml[r_in_blk + h * 8] = m_run[h];
                half_ml[BQ + r_in_blk + h * 8] = l_run[h];
            }
        }
    }
    __syncthreads();
    if (kh == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = r_in_blk + h * 8;
            const float m1 = half_ml[r], l1 = half_ml[BQ + r];
            const float mn = fmaxf(m_run[h], m1);
            const float mu = mn == -INFINITY ? 0.f : mn;
            const float a0 = exp2f(m_run[h] - mu), a1 = exp2f(m1 - mu);      // exp2(-inf) = 0
            const float l = l_run[h] * a0 + l1 * a1;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
            for (int i = 0; i < HD / 16; ++i) {
                const int c = c_base + i * 8;
                const float2 o1 = *reinterpret_cast<const float2*>(half_o + r * OP + c);
                *reinterpret_cast<float2*>(stage_o + r * OP + c) =
                    make_float2((o[i][2 * h] * a0 + o1.x * a1) * inv, (o[i][2 * h + 1] * a0 + o1.y * a1) * inv);
            }
            if (dh == 0 && (lane & 3) == 0) stage_lse[r] = l > 0.f ? mn + log2f(l) : -INFINITY;
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    FVLA_STAMP(4);
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");     // peers' barriers are initialised
    if (tid == 0) {
        for (int r = 0; r < owners; ++r) {
            const uint32_t bar_r = dsm_map(in_bar, (uint32_t)r);
            asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dsm_map(sbase + OFF_RED + rank * SLICE, (uint32_t)r)),
                           "r"(sbase + OFF_STAGE + r * SLICE), "r"(SLICE), "r"(bar_r) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dsm_map(sbase + OFF_LSE_IN + rank * 16, (uint32_t)r)),
                           "r"(sbase + OFF_STAGE + BQ * OP * 4 + r * 16), "r"(16), "r"(bar_r) : "memory");
        }
    }
    if (i_own) {
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 24); ++i) {
            uint32_t done;
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                         : "=r"(done) : "r"(in_bar), "r"(0) : "memory");
            if (done) { ok = true; break; }
        }
        if (!ok) *abort_flag = 1;
        FVLA_STAMP(5);
        const float* red = reinterpret_cast<const float*>(smem + OFF_RED);
        const float* lse_in = reinterpret_cast<const float*>(smem + OFF_LSE_IN);
        const int r4 = tid >> 6, c4 = (tid & 63) * 4;
        const int row = q0 + (int)rank * 4 + r4;
        if (ok && row < p.nq) {
            float mx = -INFINITY;
            for (int s = 0; s < SPL; ++s) mx = fmaxf(mx, lse_in[s * 4 + r4]);
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            float wsum = 0.f;
#pragma unroll 4
            for (int s = 0; s < SPL; ++s) {
                const float l = lse_in[s * 4 + r4];
                const float w = l == -INFINITY ? 0.f : exp2f(l - mx);
                wsum += w;
                const float4 v0 = *reinterpret_cast<const float4*>(red + (s * 4 + r4) * OP + c4);
                acc[0] += w * v0.x; acc[1] += w * v0.y; acc[2] += w * v0.z; acc[3] += w * v0.w;
            }
            const float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
            *reinterpret_cast<uint2*>(gout + (size_t)row * HD + c4) =
                make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
        }
    }
    // outgoing copies read this CTA's staging area: stay until every owner has everything
    // (execution barrier only; nothing read after it was written by a peer)
    FVLA_STAMP(6);
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
    FVLA_STAMP(7);
    if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 3);
}

inline int launch_decoder_attention_cluster(const DecAttnArgs& a, bool pdl, cudaStream_t st) {
    auto kern = decoder_attention_cluster_kernel;
    // K / V maps that end at the prefix (rows the preceding kernel may still be writing are never fetched by them)
    CUtensorMap tmK, tmV;
    const int seqs = a.episodes > 1 ? a.episodes : 1;
    const int pre_rows = a.prefix_keys < a.nk ? a.prefix_keys : a.nk;
    if (pre_rows <= 0) { set_error("decoder attention: no prefix keys"); return FVLA_ERR_UNSUPPORTED; }
    int rc = tc5::make_map3d(&tmK, a.k, decattn::HD, (uint64_t)pre_rows, (uint64_t)seqs, decattn::HD, (uint64_t)a.kv_episode_stride, 64, 128);
    if (rc) return rc;
    rc = tc5::make_map3d(&tmV, a.v, decattn::HD, (uint64_t)pre_rows, (uint64_t)seqs, decattn::HD, (uint64_t)a.kv_episode_stride, 64, 128);
    if (rc) return rc;
    static PerDeviceFlag configured;
    if (!configured.get()) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, decattn::smem_bytes(decattn::MAX_SPL));
        if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);      // clusters of 9..11
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured.set();
    }
    cudaLaunchConfig_t cfg = {};
    if (a.splits < decattn::MIN_SPL || a.splits > decattn::MAX_SPL || a.keys_per_split > 128 || a.keys_per_split * a.splits < a.nk) {
        set_error("decoder attention: %d keys do not fit %d splits of %d", a.nk, a.splits, a.keys_per_split);
        return FVLA_ERR_UNSUPPORTED;
    }
    cfg.gridDim = dim3((a.nq + decattn::BQ - 1) / decattn::BQ, a.splits, a.episodes > 1 ? a.episodes : 1);
    cfg.blockDim = dim3(decattn::THREADS, 1, 1);
    cfg.dynamicSmemBytes = decattn::smem_bytes(a.splits);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = a.splits; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, tmK, tmV);
    if (e != cudaSuccess) { set_error("decoder_attention_cluster_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("decoder_attention_cluster_kernel");
}

}  // namespace fvla
