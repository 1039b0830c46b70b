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
template <typename XT>
__device__ __forceinline__ float2 load_pair(const XT* row, int i);
template <>
__device__ __forceinline__ float2 load_pair<bf16>(const bf16* row, int i) {
    return unpack_bf16x2(reinterpret_cast<const uint32_t*>(row)[i]);
}
template <>
__device__ __forceinline__ float2 load_pair<float>(const float* row, int i) {
    return reinterpret_cast<const float2*>(row)[i];
}

template <typename XT>
__global__ void __launch_bounds__(128) rownorm_kernel(const XT* __restrict__ x, const bf16* __restrict__ w,
                                                      const bf16* __restrict__ b, bf16* __restrict__ out,
                                                      float* __restrict__ factor_f32,
                                                      bf16* __restrict__ factor_bf16, int M, int K, int mode) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // no-op unless launched as a dependent
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const XT* xr = x + (size_t)row * K;
    const int pairs = K >> 1;
    float s = 0.f, ss = 0.f;
    for (int i = lane; i < pairs; i += 32) {
        float2 v = load_pair<XT>(xr, i);
        s += v.x + v.y;
        ss += v.x * v.x + v.y * v.y;
    }
    s = warp_sum(s); ss = warp_sum(ss);
    if (mode == 2) {
        float f = rsqrtf(ss / K + 1e-6f);
        if (lane == 0) {
            if (factor_f32) factor_f32[row] = f;
            if (factor_bf16) factor_bf16[row] = __float2bfloat16_rn(f);
        }
        if (out == nullptr) return;
        mode = 1;                               // also emit the normalised row
    }
    uint32_t* orow = reinterpret_cast<uint32_t*>(out + (size_t)row * K);
    if (mode == 1) {
        float f = rsqrtf(ss / K + 1e-6f);
        for (int i = lane; i < pairs; i += 32) {
            float2 v = load_pair<XT>(xr, i);
            orow[i] = pack_bf16x2(v.x * f, v.y * f);
        }
        return;
    }
    const float mean = s / K;
    const float inv = rsqrtf(ss / K - mean * mean + 1e-5f);
    const uint32_t* wr = reinterpret_cast<const uint32_t*>(w);
    const uint32_t* br = reinterpret_cast<const uint32_t*>(b);
    for (int i = lane; i < pairs; i += 32) {
        float2 v = load_pair<XT>(xr, i), wv = unpack_bf16x2(wr[i]), bv = unpack_bf16x2(br[i]);
        orow[i] = pack_bf16x2((v.x - mean) * inv * wv.x + bv.x, (v.y - mean) * inv * wv.y + bv.y);
    }
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
// Each warp walks its share of K eight rows at a time so that eight loads are in flight.
template <typename XT, typename OT>
__global__ void __launch_bounds__(256) action_out_kernel(const XT* __restrict__ x, const bf16* __restrict__ W,
                                                         const bf16* __restrict__ bias, OT* __restrict__ out,
                                                         bf16* __restrict__ mirror, bf16* __restrict__ factor_out,
                                                         int K) {
    constexpr int N = 32;
    __shared__ float red[8][N + 1];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = lane;                          // each warp covers all 32 outputs for its k slice
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, ss = 0.f;
    const int per_warp = (K + 7) / 8;            // contiguous k range per warp
    const int k_begin = warp * per_warp, k_end = min(K, k_begin + per_warp);
    const float prev = static_cast<float>(out[(size_t)m * N + n]);
    for (int k0 = k_begin; k0 < k_end; k0 += 8) {
        float xv[8], wv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int k = k0 + u;
            xv[u] = k < k_end ? static_cast<float>(x[(size_t)m * K + k]) : 0.f;
            wv[u] = k < k_end ? __bfloat162float(W[(size_t)k * N + n]) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            acc[u] += xv[u] * wv[u];
            ss += xv[u] * xv[u];                 // identical in every lane of the warp
        }
    }
    red[warp][n] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    if (lane == 0) red[warp][N] = ss;
    __syncthreads();
    if (warp == 0) {
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

}  // namespace fvla
