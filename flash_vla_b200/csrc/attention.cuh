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

template <int HD>   // padded head dim, multiple of 16
__global__ void __launch_bounds__(128) attention_kernel(const AttnArgs p) {
    constexpr int BQ = 64, BKV = 64;
    constexpr int PITCH = HD * 2 + 16;          // bytes; +16 keeps ldmatrix rows on distinct banks
    constexpr int CH = HD / 8;                  // 16-byte chunks per row
    constexpr int TILE = 64 * PITCH;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t sQ = smem_u32(smem);
    const uint32_t sKV = sQ + TILE;             // stage s: K at sKV + s*2*TILE, V right after

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
        const int stage = jb & 1;
        if (jb + 1 < nblocks) {
            const int kb = key_beg + (jb + 1) * BKV;
            load_rows(sKV + (stage ^ 1) * 2 * TILE, K, p.k_stride, kb, key_end);
            load_rows(sKV + (stage ^ 1) * 2 * TILE + TILE, V, p.v_stride, kb, key_end);
        }
        cp_async_commit();
        cp_async_wait<1>();
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

template <int HD>
inline int launch_attention(const AttnArgs& a, dim3 grid, cudaStream_t st) {
    constexpr int smem = 5 * 64 * (HD * 2 + 16);
    auto kern = attention_kernel<HD>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        configured = true;
    }
    kern<<<grid, 128, smem, st>>>(a);
    return check_launch("attention_kernel");
}

}  // namespace fvla
