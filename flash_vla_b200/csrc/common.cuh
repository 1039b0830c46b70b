// Shared device/host helpers for the sm_100a Pi0 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <atomic>

#include "../../include/flash_vla_b200.h"

namespace fvla {

using bf16 = __nv_bfloat16;

constexpr float kGeluC0 = 1.5957691216057308f;   // 2 * sqrt(2 / pi)
constexpr float kGeluC1 = 0.044715f;
constexpr float kLog2e = 1.4426950408889634f;

// tanh-GELU. The reference kernels write it as v * sigmoid(C0 * v * (1 + C1 v^2))
// (kernels/base.py:77-78); sigmoid(t) = (1 + tanh(t / 2)) / 2, and tanh.approx is one special-function
// instruction where exp + reciprocal are two (its 2^-11 relative error is below bf16 rounding).
__device__ __forceinline__ float gelu_f(float v) {
    float t = (0.5f * kGeluC0) * v * (1.0f + kGeluC1 * v * v), th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(t));
    const float h = 0.5f * v;
    return fmaf(h, th, h);
}
__device__ __forceinline__ float silu_f(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte async copy global -> shared; bytes beyond `src_bytes` are zero-filled.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src),
                 "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
}
__device__ __forceinline__ float round_bf16(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Host-side state that CUDA keeps per device (function attributes, SM count, symbol addresses) is
// cached per device ordinal, so that one process may drive several GPUs. Entries are atomics: two
// host threads racing on the first call both do the (idempotent) set-up, neither reads a torn value.
constexpr int kMaxDevices = 64;
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    return dev;
}
struct PerDeviceFlag {
    std::atomic<int> done[kMaxDevices];
    bool get() const { return done[current_device()].load(std::memory_order_acquire) != 0; }
    void set() { done[current_device()].store(1, std::memory_order_release); }
};

// FVLA_PDL=0 turns programmatic dependent launch off (diagnostic switch).
inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("FVLA_PDL");
        on = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// Launch `kern` as a programmatic dependent of the previous kernel in the stream: its CTAs may be
// scheduled while that kernel drains, and it must execute griddepcontrol.wait before touching
// anything the previous kernel wrote (every kernel launched through here does so first thing).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Development aid, compiled only with -DFVLA_DEBUG (the shipped library is built without it and then
// none of this exists, neither in the kernels' argument structs nor in their code): kernels record
// %globaltimer stamps, 8 per CTA, into a device buffer that the developer registered through
// fvla_debug_set_timestamps (validated there; successive launches rotate through its slots).
#ifdef FVLA_DEBUG
unsigned long long* debug_next_slot();
#define FVLA_DBG_MEMBER unsigned long long* dbg;
#define FVLA_DBG_ATTACH(args) (args).dbg = ::fvla::debug_next_slot()
#define FVLA_DBG_CTA(args, cta) unsigned long long* fvla_dbg = (args).dbg ? (args).dbg + (size_t)(cta) * 8 : nullptr
#define FVLA_STAMP_ANY(i)                                                          \
    do {                                                                           \
        if (fvla_dbg) {                                                            \
            unsigned long long t_;                                                 \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                 \
            fvla_dbg[i] = t_;                                                      \
        }                                                                          \
    } while (0)
#define FVLA_STAMP(i) do { if (threadIdx.x == 0) FVLA_STAMP_ANY(i); } while (0)
#else
#define FVLA_DBG_MEMBER
#define FVLA_DBG_ATTACH(args) ((void)0)
#define FVLA_DBG_CTA(args, cta) ((void)0)
#define FVLA_STAMP_ANY(i) ((void)0)
#define FVLA_STAMP(i) ((void)0)
#endif

// Tuned launch plans. The kernels choose tile width, K split and kernel family from cost models; a tuning
// run (the sweep harness on the Python side) may pin a measured-best choice per GEMM shape instead. A
// pinned plan that a launch cannot honour (scratch too small, an epilogue the family lacks) is an error
// for that launch, never a silent substitute, so that a sweep sees which candidates are real.
enum PlanKind { PLAN_PLAIN = 0, PLAN_ROPE = 1, PLAN_DUAL = 2, PLAN_SKINNY = 3, PLAN_SKINNY_DUAL = 4 };
enum PlanEngine { ENGINE_AUTO = 0, ENGINE_TC5_SCRATCH = 1, ENGINE_TC5_CLUSTER = 2, ENGINE_PAIR = 3, ENGINE_SKINNY = 4 };
struct PlanChoice { int engine = ENGINE_AUTO, bn = 0, splits = 0; };
bool plan_lookup(int M, int N, int K, int kind, PlanChoice* out);

// Host-side: record the message of the last failing call on this thread.
void set_error(const char* fmt, ...);
int check_launch(const char* what);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace fvla
