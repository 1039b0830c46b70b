// Row-wise and tiny kernels: LayerNorm, RMS norm / factor, patchify, and the K = 32 / N = 32
// projections at the two ends of the action-expert decoder. All are HBM- or latency-bound.
#pragma once

#include "common.cuh"

namespace fvla {

// One warp per row. mode 0: LayerNorm(w, b), eps 1e-5, variance as E[x^2] - mean^2 (the
// reference's form, kernels/base.py:406-447). mode 1: x * rsqrt(mean(x^2) + 1e-6) (base.py:373).
// mode 2: the factor rsqrt(mean(x^2) + 1e-6), written as fp32 and/or bf16 (base.py:344), plus
// the normalised row when `out` is given.
// The input row is bf16 or fp32 (XT); outputs are always bf16.
// 8 consecutive elements of a row as floats (one 16-byte load for bf16, two for fp32).
template <typename XT>
__device__ __forceinline__ void load8(const XT* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<bf16>(const bf16* p, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(p);
    const float2 f0 = unpack_bf16x2(a.x), f1 = unpack_bf16x2(a.y), f2 = unpack_bf16x2(a.z), f3 = unpack_bf16x2(a.w);
    v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y; v[4] = f2.x; v[5] = f2.y; v[6] = f3.x; v[7] = f3.y;
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// One warp per row, K % 8 == 0 and K <= 8 * 32 * RN_MAX. The whole row is fetched in one batch of
// 16-byte loads and kept in registers, so the row is read once and normalised without a second trip.
constexpr int RN_MAX = 8;            // 16-byte chunks per lane: rows up to 2048 elements
template <typename XT>
__global__ void __launch_bounds__(128) rownorm_kernel(const XT* __restrict__ x, const bf16* __restrict__ w,
                                                      const bf16* __restrict__ b, bf16* __restrict__ out,
                                                      float* __restrict__ factor_f32,
                                                      bf16* __restrict__ factor_bf16, int M, int K, int mode) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");      // the next kernel may be scheduled
    asm volatile("griddepcontrol.wait;" ::: "memory");      // no-op unless launched as a dependent
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const XT* xr = x + (size_t)row * K;
    const int chunks = K >> 3;
    float v[RN_MAX][8];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < RN_MAX; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            load8<XT>(xr + c * 8, v[i]);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s += v[i][e]; ss += v[i][e] * v[i][e]; }
        }
    }
    s = warp_sum(s); ss = warp_sum(ss);
    if (mode == 2) {
        const float f = rsqrtf(ss / K + 1e-6f);
        if (lane == 0) {
            if (factor_f32) factor_f32[row] = f;
            if (factor_bf16) factor_bf16[row] = __float2bfloat16_rn(f);
        }
        if (out == nullptr) return;
        mode = 1;                               // also emit the normalised row
    }
    bf16* orow = out + (size_t)row * K;
    const float mean = mode == 1 ? 0.f : s / K;
    const float inv = mode == 1 ? rsqrtf(ss / K + 1e-6f) : rsqrtf(ss / K - mean * mean + 1e-5f);
#pragma unroll
    for (int i = 0; i < RN_MAX; ++i) {
        const int c = lane + 32 * i;
        if (c < chunks) {
            float y[8];
            if (mode == 1) {
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = v[i][e] * inv;
            } else {
                float wv[8], bv[8];
                load8<bf16>(w + c * 8, wv);
                load8<bf16>(b + c * 8, bv);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = (v[i][e] - mean) * inv * wv[e] + bv[e];
            }
            *reinterpret_cast<uint4*>(orow + c * 8) = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                                 pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
        }
    }
}

// Folds a LayerNorm's scale g and shift s into the linear layer that follows it, y = LN(x) W + b:
//   W'[k][n] = bf16(g[k] W[k][n]),  colsum[n] = sum_k W'[k][n],  bias'[n] = sum_k s[k] W[k][n] + b[n]
// so that y = rstd (x W' - mean colsum) + bias'. colsum is taken over the ROUNDED W', the matrix the GEMM
// multiplies by, so a constant row still maps to bias' exactly. One thread per output column; a set-up kernel.
__global__ void __launch_bounds__(128) fold_layernorm_kernel(const bf16* __restrict__ g, const bf16* __restrict__ s,
                                                             const bf16* __restrict__ W, const bf16* __restrict__ b,
                                                             bf16* __restrict__ Wf, float* __restrict__ colsum,
                                                             float* __restrict__ biasf, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float cs = 0.f, bs = 0.f;
    for (int k = 0; k < K; ++k) {
        const float wv = __bfloat162float(W[(size_t)k * N + n]);
        const bf16 f = __float2bfloat16_rn(__bfloat162float(g[k]) * wv);
        Wf[(size_t)k * N + n] = f;
        cs += __bfloat162float(f);
        bs += __bfloat162float(s[k]) * wv;
    }
    colsum[n] = cs;
    biasf[n] = bs + (b != nullptr ? __bfloat162float(b[n]) : 0.f);
}

// images (views, 224, 224, 3) -> patches (views * 256, ld) with feature order (iy, ix, c); columns
// [588, ld) are written as zero so the GEMM may read whole 16-byte chunks.
__global__ void __launch_bounds__(256) patchify_kernel(const bf16* __restrict__ img, bf16* __restrict__ out,
                                                       int views, int ld) {
    const int patch = blockIdx.x;                 // view * 256 + py * 16 + px
    const int v = patch >> 8, py = (patch >> 4) & 15, px = patch & 15;
    for (int f = threadIdx.x; f < ld; f += blockDim.x) {
        bf16 val = __float2bfloat16_rn(0.f);
        if (f < 588) {
            int iy = f / 42, rem = f % 42;        // 42 = 14 pixels x 3 channels, contiguous in the image
            val = img[(((size_t)v * 224 + py * 14 + iy) * 224 + px * 14) * 3 + rem];
        }
        out[(size_t)patch * ld + f] = val;
    }
}

// out[m, n] = act(sum_k x[m, k] W[k, n] + bias[n]) for tiny K (<= 64): the state and action
// input projections (K = 32). x may be fp32 or bf16; one thread per output element.
template <typename XT, typename OT>
__global__ void __launch_bounds__(256) small_k_proj_kernel(const XT* __restrict__ x, const bf16* __restrict__ W,
                                                           const bf16* __restrict__ bias, OT* __restrict__ out,
                                                           int M, int N, int K, int act) {
    __shared__ float xs[64];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.y;
    if (threadIdx.x < K) xs[threadIdx.x] = static_cast<float>(x[(size_t)m * K + threadIdx.x]);
    __syncthreads();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float acc = bias ? __bfloat162float(bias[n]) : 0.f;
    for (int k = 0; k < K; ++k) acc += xs[k] * __bfloat162float(W[(size_t)k * N + n]);
    if (act == 2) acc = silu_f(acc);
    out[(size_t)m * N + n] = static_cast<OT>(acc);
}

// The Euler update: out[m, :] += bias + rsqrt(mean(x[m]^2) + 1e-6) * (x[m, :] @ W), W (K, 32).
// One CTA per row; the sum of squares rides along with the dot products so x is read once.
// `out` is fp32 or bf16; when `mirror` is given the new value is also written there as bf16.
// Thread t owns k rows (t / 4) + 64 i and the 8 output columns 8 (t % 4) .. + 8: every W access is a
// 16-byte load, and a batch of eight of them (plus the matching x values) is in flight per thread.
template <typename XT, typename OT>
__global__ void __launch_bounds__(256) action_out_kernel(const XT* __restrict__ x, const bf16* __restrict__ W,
                                                         const bf16* __restrict__ bias, OT* __restrict__ out,
                                                         bf16* __restrict__ mirror, bf16* __restrict__ factor_out,
                                                         int K) {
    constexpr int N = 32;
    __shared__ float red[8][N + 1];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kg = tid >> 2, quad = tid & 3;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, ss = 0.f;
    const float prev = lane < N && warp == 0 ? static_cast<float>(out[(size_t)m * N + lane]) : 0.f;
    for (int k0 = 0; k0 < K; k0 += 512) {
        uint4 wv[8];
        float xv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = k0 + u * 64 + kg;
            wv[u] = make_uint4(0, 0, 0, 0);
            xv[u] = 0.f;
            if (k < K) {
                wv[u] = __ldg(reinterpret_cast<const uint4*>(W + (size_t)k * N + quad * 8));
                xv[u] = static_cast<float>(x[(size_t)m * K + k]);
            }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const float2 w0 = unpack_bf16x2(wv[u].x), w1 = unpack_bf16x2(wv[u].y), w2 = unpack_bf16x2(wv[u].z), w3 = unpack_bf16x2(wv[u].w);
            acc[0] += xv[u] * w0.x; acc[1] += xv[u] * w0.y; acc[2] += xv[u] * w1.x; acc[3] += xv[u] * w1.y;
            acc[4] += xv[u] * w2.x; acc[5] += xv[u] * w2.y; acc[6] += xv[u] * w3.x; acc[7] += xv[u] * w3.y;
            ss += xv[u] * xv[u];                 // the four lanes of a k group hold the same x: counted once below
        }
    }
    // lanes of a warp: 8 k groups x 4 column quads; fold the k groups
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
    }
    if (lane < 4) {
#pragma unroll
        for (int j = 0; j < 8; ++j) red[warp][lane * 8 + j] = acc[j];
        if (lane == 0) red[warp][N] = ss;
    }
    __syncthreads();
    if (warp == 0) {
        const int n = lane;
        float a = 0.f, s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { a += red[w][n]; s += red[w][N]; }
        float f = rsqrtf(s / K + 1e-6f);
        float v = prev + __bfloat162float(bias[n]) + f * a;
        out[(size_t)m * N + n] = static_cast<OT>(v);
        if (mirror) mirror[(size_t)m * N + n] = __float2bfloat16_rn(v);
        if (factor_out && lane == 0) factor_out[m] = __float2bfloat16_rn(f);
    }
}

// dst[i] = src[i] between bf16 and fp32 buffers (any of the four combinations), optionally also writing the
// value as bf16 to `shadow`. The small copies inside the decoder step (state token into the residual
// stream, the action chunk to and from its fp32 master) go through this kernel instead of a framework copy
// so that they stay inside the chain of programmatic dependent launches.
template <typename ST, typename DT>
__global__ void __launch_bounds__(256) convert_copy_kernel(const ST* __restrict__ src, DT* __restrict__ dst,
                                                           bf16* __restrict__ shadow, size_t count) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float v = static_cast<float>(src[i]);
    dst[i] = static_cast<DT>(v);
    if (shadow) shadow[i] = __float2bfloat16_rn(v);
}

// dst[i] = bf16(src[i]), four values per thread.
__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, size_t quads) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= quads) return;
    const float4 v = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<uint2*>(dst)[i] = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
}

// out[r, :] = table[ids[r], :] for bf16 rows of `dim` elements (dim % 8 == 0): the prompt embedding
// lookup. One CTA per row, 16-byte copies. An id outside [0, vocab) yields a zero row and sets the device
// status word, so a bad prompt is reported instead of reading out of bounds.
__global__ void __launch_bounds__(128) embed_rows_kernel(const bf16* __restrict__ table, const long long* __restrict__ ids,
                                                         bf16* __restrict__ out, int dim, long long vocab, int* status) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = blockIdx.x;
    const long long id = ids[r];
    const bool ok = id >= 0 && id < vocab;
    if (!ok && threadIdx.x == 0 && status) atomicExch(status, 7);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(ok ? id : 0) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * dim);
    for (int c = threadIdx.x; c < dim / 8; c += blockDim.x) dst[c] = ok ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
}

}  // namespace fvla
