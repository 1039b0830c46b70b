// extern "C" surface of libfvla_b200: argument validation, kernel selection, launches.
// Nothing here allocates, frees or synchronises.
#include <atomic>
#include <mutex>
#include <vector>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "attention.cuh"
#include "attention_tc5.cuh"
#include "common.cuh"
#include "gemm_mma.cuh"
#include "gemm_tc5.cuh"
#include "gemm_skinny.cuh"
#include "gemm_tc5x2.cuh"
#include "rowops.cuh"

namespace fvla {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};

int check_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return FVLA_ERR_LAUNCH;
    }
    return FVLA_OK;
}

// ---- pinned launch plans (filled by the tuning harness or from a tuned-plan file) -----------------
struct PlanEntry { int M, N, K, kind; PlanChoice choice; };
static std::mutex g_plan_mutex;
static std::vector<PlanEntry> g_plans;
static std::atomic<int> g_plan_count{0};

bool plan_lookup(int M, int N, int K, int kind, PlanChoice* out) {
    if (g_plan_count.load(std::memory_order_acquire) == 0) return false;      // the common case: nothing pinned
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (const PlanEntry& e : g_plans)
        if (e.M == M && e.N == N && e.K == K && e.kind == kind) { *out = e.choice; return true; }
    return false;
}

static inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }
static inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
static inline const bf16* B(const void* p) { return reinterpret_cast<const bf16*>(p); }
static inline bf16* Bm(void* p) { return reinterpret_cast<bf16*>(p); }

#define FVLA_REQUIRE(cond, ...)            \
    do {                                   \
        if (!(cond)) {                     \
            set_error(__VA_ARGS__);        \
            return FVLA_ERR_ARG;           \
        }                                  \
    } while (0)

static int rownorm(const void* x, int x_is_f32, const void* w, const void* b, void* out, float* f32,
                   void* fbf, int M, int K, int mode, cudaStream_t st) {
    FVLA_REQUIRE(M > 0 && K > 0 && K % 8 == 0 && K <= 8 * 32 * RN_MAX, "rownorm: bad shape M=%d K=%d (K %% 8 == 0, K <= %d)", M, K, 8 * 32 * RN_MAX);
    cudaError_t e;
    if (x_is_f32)
        e = launch_pdl(rownorm_kernel<float>, dim3((M + 3) / 4), dim3(128), 0, st, (const float*)x, B(w), B(b), Bm(out), f32, Bm(fbf), M, K, mode);
    else
        e = launch_pdl(rownorm_kernel<bf16>, dim3((M + 3) / 4), dim3(128), 0, st, B(x), B(w), B(b), Bm(out), f32, Bm(fbf), M, K, mode);
    if (e != cudaSuccess) { set_error("rownorm_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("rownorm_kernel");
}

// Workspace layout of the GEMM-shaped ops:
//   [per-row fp32 factors | bf16 copy of the normalised rows (fp32 input only) | split-K scratch]
static size_t ws_factor_bytes(int M) { return align256((size_t)M * sizeof(float)); }
static size_t ws_xnorm_bytes(int M, int K) { return align256((size_t)M * K * sizeof(bf16)); }
static size_t op_ws_bytes(int M, int N, int K, bool dual) {
    size_t gemm = plan_gemm_mma(M, N, K, dual).ws_bytes;
    if (!dual && M > 64) {
        // the tcgen05 kernels may split K through scratch: room for the widest plan either family can be
        // given (4 splits at any tile width on the one-SM kernel, 6 on the pair kernel), so that a plan
        // pinned later never finds the scratch too small
        size_t t = 0;
        for (int bn = 64; bn <= 256; bn += 64) { size_t v = tc5::scratch_split_bytes(M, N, bn, 4); if (v > t) t = v; }
        size_t t2 = tc5x2::pair_split_bytes(M, N, 6);
        if (t2 > t) t = t2;
        if (t > gemm) gemm = t;
    }
    return ws_factor_bytes(M) + ws_xnorm_bytes(M, K) + gemm;
}
// Split-K part of an op workspace as (pointer, size); (nullptr, 0) when the caller gave none.
static void gemm_ws(void* ws, size_t ws_bytes, int M, int K, void** p, size_t* n) {
    size_t off = ws_factor_bytes(M) + ws_xnorm_bytes(M, K);
    bool has = ws != nullptr && ws_bytes >= off;
    *p = has ? (uint8_t*)ws + off : nullptr;
    *n = has ? ws_bytes - off : 0;
}

// Device status word written by kernels whose bounded waits ran out (0 = healthy).
__device__ int g_device_status;

static int* device_status_ptr() {
    static thread_local int cached_dev = -1;
    static thread_local int* cached_ptr = nullptr;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev != cached_dev) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
        cached_ptr = static_cast<int*>(ptr);
        cached_dev = dev;
    }
    return cached_ptr;
}

// FVLA_GEMM=mma forces every GEMM onto the warp-level kernel (a diagnostic switch for
// comparing the two tensor paths; the default is tcgen05 wherever the shape allows).
static bool tc5_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* v = getenv("FVLA_GEMM");
        enabled = (v != nullptr && strcmp(v, "mma") == 0) ? 0 : 1;
    }
    return enabled == 1;
}

#ifdef FVLA_DEBUG
// Development builds only: the timestamp buffer the instrumented kernels write to. It is registered
// through fvla_debug_set_timestamps (below), which checks that it is device memory of sufficient size;
// successive launches take successive 2048-entry slots, cyclically.
static unsigned long long* g_dbg_base = nullptr;
static int g_dbg_slots = 0, g_dbg_next = 0;
unsigned long long* debug_next_slot() {
    if (g_dbg_base == nullptr || g_dbg_slots < 1) return nullptr;
    unsigned long long* p = g_dbg_base + (size_t)(g_dbg_next % g_dbg_slots) * 2048;
    ++g_dbg_next;
    return p;
}
#endif

// GEMM dispatch: tcgen05 for M > 64, the warp-level kernel (with split-K) for the skinny shapes.
// FVLA_GEMM_PAIR=0 keeps the gated FFN on the one-SM kernel (diagnostic switch).
static bool pair_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("FVLA_GEMM_PAIR");
        on = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

static int launch_gemm(const GemmArgs& a, void* ws, size_t ws_bytes, cudaStream_t st) {
    PlanChoice pinned;
    if (tc5_enabled() && tc5::tc5_supports(a) &&
        plan_lookup(a.M, a.N, a.K, a.B2 != nullptr ? PLAN_DUAL : (a.rope != nullptr ? PLAN_ROPE : PLAN_PLAIN), &pinned)) {
        GemmArgs g = a;
        if (g.Kb == 0) g.Kb = g.K;
        if (a.B2 != nullptr) {          // gated FFN: the only choice is the kernel family
            if (pinned.engine == ENGINE_PAIR) return tc5x2::launch_geglu_pair(g, device_status_ptr(), st);
            return tc5::launch_gemm_tc5(g, device_status_ptr(), st, ws, ws_bytes);
        }
        if (pinned.engine == ENGINE_PAIR) return tc5x2::launch_plain_pair_pinned(g, pinned.splits, ws, ws_bytes, device_status_ptr(), st);
        return tc5::launch_gemm_tc5_pinned(g, pinned, device_status_ptr(), st, ws, ws_bytes);
    }
    if (tc5_enabled() && pair_enabled() && a.B2 != nullptr && tc5::tc5_supports(a)) {
        GemmArgs g = a;
        if (g.Kb == 0) g.Kb = g.K;
        int rc = tc5x2::launch_geglu_pair(g, device_status_ptr(), st);
        if (rc != FVLA_ERR_UNSUPPORTED) return rc;
    }
    if (tc5_enabled() && pair_enabled() && a.B2 == nullptr && a.bias == nullptr && a.act == 0 && !a.c_f32 && tc5::tc5_supports(a)) {
        // residual projections without bias: take the CTA-pair kernel when its estimate beats the one-SM plan.
        // (With a bias or GELU epilogue, i.e. at the SigLIP call sites, the pair kernel measured slower than
        // the one-SM plans at every site, 15.5 - 18.9 us against 10.9 - 17.0 us; it is reachable there
        // through a pinned plan only. The same holds for an fp32 destination, the residual projections of
        // a decoder batched over episodes: 33 - 43 us on the pair kernel against 18 - 21 us.)
        GemmArgs g = a;
        if (g.Kb == 0) g.Kb = g.K;
        tc5x2::PairPlan pp = tc5x2::plan_pair_plain(g.M, g.N, g.K, ws != nullptr);
        if (pp.ok && pp.est_us < tc5::plan_tc5(g.M, g.N, g.K, ws != nullptr && !g.c_f32).est_us) {
            int rc = tc5x2::launch_plain_pair(g, ws, ws_bytes, device_status_ptr(), st);
            if (rc != FVLA_ERR_UNSUPPORTED) return rc;
        }
    }
    if (tc5_enabled() && tc5::tc5_supports(a)) return tc5::launch_gemm_tc5(a, device_status_ptr(), st, ws, ws_bytes);
    return launch_gemm_mma(a, ws, ws_bytes, st);
}

// RMS norm + QKV projection + RoPE + scatter of the prefix encoder. fuse_norm: let the GEMM take the raw rows and
// apply the norm to its accumulators when the shape allows (x_norm is then left alone); otherwise x_norm receives
// the normalised rows from a kernel of its own.
static int encoder_qkv_rope(const void* x, const void* weight_qkv, const void* rope, void* Q, void* K, void* V, void* x_norm,
                            int M, int Kdim, int heads, int head_dim, int group_rows, int kv_group_pitch, int fuse_norm,
                            void* stream) {
    GemmArgs a;
    a.lda = Kdim; a.B = B(weight_qkv); a.ldb = (heads + 2) * head_dim;
    a.M = M; a.N = (heads + 2) * head_dim; a.K = Kdim;
    a.rope = B(rope); a.q = Bm(Q); a.k = Bm(K); a.v = Bm(V); a.heads = heads; a.head_dim = head_dim;
    a.round_first = 1;
    a.group_rows = group_rows; a.kv_group_pitch = kv_group_pitch;
    a.trigger_early = 1;      // the next kernel (prefix attention / down projection) runs one CTA per SM
    if (fuse_norm && tc5_enabled()) {
        a.A = B(x); a.norm_mode = 1;
        const int rc = tc5::launch_gemm_tc5_normed(a, device_status_ptr(), S(stream));
        if (rc != FVLA_ERR_UNSUPPORTED) return rc;
        a.norm_mode = 0;
    }
    if (x_norm == nullptr) { set_error("encoder QKV: M=%d needs the x_norm scratch", M); return FVLA_ERR_ARG; }
    int rc = rownorm(x, 0, nullptr, nullptr, x_norm, nullptr, nullptr, M, Kdim, 1, S(stream));
    if (rc) return rc;
    a.A = B(x_norm);
    return launch_gemm(a, nullptr, 0, S(stream));
}

}  // namespace fvla

using namespace fvla;

extern "C" {

const char* fvla_last_error(void) { return g_error; }
int fvla_abi_version(void) { return 4; }
unsigned long long fvla_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fvla_device_status(void* stream) {
    int* ptr = device_status_ptr();
    if (ptr == nullptr) { set_error("device_status: no CUDA device"); return FVLA_ERR_LAUNCH; }
    int value = 0;
    cudaError_t e = cudaMemcpyAsync(&value, ptr, sizeof(int), cudaMemcpyDeviceToHost, S(stream));
    if (e == cudaSuccess) e = cudaMemsetAsync(ptr, 0, sizeof(int), S(stream));      // read and clear
    if (e == cudaSuccess) e = cudaStreamSynchronize(S(stream));
    if (e != cudaSuccess) { set_error("device_status: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return value;
}

size_t fvla_gemm_workspace_bytes(int M, int N, int K, int dual) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return op_ws_bytes(M, N, K, dual != 0);
}

size_t fvla_decoder_attention_workspace_bytes(int queries, int keys) {
    if (queries <= 0 || keys <= 0) return 0;
    int splits = (keys + 127) / 128;
    size_t qpad = (size_t)(queries + 63) / 64 * 64;
    return align256(splits * qpad * sizeof(float)) + splits * qpad * 256 * sizeof(float);
}

size_t fvla_patch_embed_workspace_bytes(int views) {
    return views > 0 ? (size_t)views * 256 * 592 * sizeof(bf16) : 0;
}

int fvla_vision_patch_embed(const void* images, const void* patch_w, const void* patch_b,
                            const void* pos_emb, void* out, int views, void* ws, size_t ws_bytes,
                            void* stream) {
    FVLA_REQUIRE(views > 0, "patch_embed: views=%d", views);
    FVLA_REQUIRE(images != nullptr && patch_w != nullptr && patch_b != nullptr && pos_emb != nullptr && out != nullptr,
                 "patch_embed: null pointer");
    FVLA_REQUIRE(aligned16(images) && aligned16(patch_w) && aligned16(patch_b) && aligned16(pos_emb) && aligned16(out) &&
                 aligned16(ws), "patch_embed: every pointer must be 16-byte aligned");
    if (ws == nullptr || ws_bytes < fvla_patch_embed_workspace_bytes(views)) {
        set_error("patch_embed: workspace of %zu bytes needed", fvla_patch_embed_workspace_bytes(views));
        return FVLA_ERR_WORKSPACE;
    }
    const int M = views * 256;
    patchify_kernel<<<M, 256, 0, S(stream)>>>(B(images), Bm(ws), views, 592);
    int rc = check_launch("patchify_kernel");
    if (rc) return rc;
    GemmArgs a;
    a.A = B(ws); a.lda = 592; a.B = B(patch_w); a.ldb = 1152; a.C = out; a.ldc = 1152;
    a.bias = B(patch_b); a.R = pos_emb; a.ldr = 1152; a.res_mod = 256;
    a.M = M; a.N = 1152; a.K = 592; a.Kb = 588;
    return launch_gemm(a, nullptr, 0, S(stream));
}

// ---- patch embedding without caller-provided scratch -------------------------------------------
// The patchified image matrix normally lives in scratch the caller hands in. Some callers have
// nothing to hand in: a control loop that must not call cudaMalloc (it synchronises the device and
// its latency is unbounded), a C program with no allocator of its own, or Python code whose
// ScratchPool is already frozen and would raise on a new request. For them the matrix is kept in
// this fixed device array instead. Every GPU that loads the library holds these bytes until the
// process exits, hence the modest limit of four camera views.
#define FVLA_NOALLOC_MAX_VIEWS 4
static __device__ __align__(256) unsigned char g_patch_scratch[FVLA_NOALLOC_MAX_VIEWS * 256 * 592 * 2];

// In host code `g_patch_scratch` is only a handle for the symbol, not an address the GPU can use;
// the device address is looked up once per device (with that device current) and cached.
static void* patch_scratch_device_ptr(cudaStream_t stream) {
    static std::atomic<void*> cached[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error("patch_embed_noalloc: cannot identify the current device");
        return nullptr;
    }
    void* ptr = cached[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        // The look-up is a runtime call that must not happen inside a stream capture: refuse clearly
        // instead of letting it invalidate the caller's capture.
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
            set_error("patch_embed_noalloc: the first call on a device looks up the built-in scratch and must be made "
                      "outside stream capture");
            return nullptr;
        }
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_patch_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("patch_embed_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cached[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}

static int norm_linear(const void* x, const void* nw, const void* nb, const void* w, const void* b,
                       void* out, void* x_norm, int M, int N, int K, int act, void* stream, int trigger_early) {
    int rc = rownorm(x, 0, nw, nb, x_norm, nullptr, nullptr, M, K, 0, S(stream));
    if (rc) return rc;
    GemmArgs a;
    a.A = B(x_norm); a.lda = K; a.B = B(w); a.ldb = N; a.C = out; a.ldc = N; a.bias = B(b);
    a.act = act; a.M = M; a.N = N; a.K = K; a.trigger_early = trigger_early;
    return launch_gemm(a, nullptr, 0, S(stream));
}

int fvla_vision_patch_embed_noalloc(const void* images, const void* patch_w, const void* patch_b,
                                    const void* pos_emb, void* out, int views, void* stream) {
    FVLA_REQUIRE(views > 0, "patch_embed_noalloc: views=%d", views);
    if (views > FVLA_NOALLOC_MAX_VIEWS) {
        set_error("patch_embed_noalloc: %d views exceed the built-in scratch (at most %d views, %zu bytes); "
                  "use fvla_vision_patch_embed with caller scratch instead",
                  views, FVLA_NOALLOC_MAX_VIEWS, sizeof(g_patch_scratch));
        return FVLA_ERR_WORKSPACE;
    }
    void* scratch = patch_scratch_device_ptr(S(stream));
    if (scratch == nullptr) return FVLA_ERR_LAUNCH;
    // The patchify kernel rewrites every element it later reads, zero padding included, so the
    // previous call's contents never need clearing.
    return fvla_vision_patch_embed(images, patch_w, patch_b, pos_emb, out, views, scratch,
                                   fvla_patch_embed_workspace_bytes(views), stream);
}

int fvla_vision_norm_qkv(const void* x, const void* norm_w, const void* norm_b, const void* qkv_w,
                         const void* qkv_b, void* out, void* x_norm, int M, int N, int K, void* stream) {
    return norm_linear(x, norm_w, norm_b, qkv_w, qkv_b, out, x_norm, M, N, K, 0, stream, 0);
}

int fvla_vision_norm_ffn_up(const void* x, const void* norm_w, const void* norm_b, const void* weight,
                            const void* bias, void* out, void* x_norm, int M, int N, int K, void* stream) {
    return norm_linear(x, norm_w, norm_b, weight, bias, out, x_norm, M, N, K, 1, stream, 1);      // the down GEMM follows
}

int fvla_fold_layernorm(const void* norm_w, const void* norm_b, const void* weight, const void* bias, void* weight_folded,
                        float* colsum, float* bias_folded, int N, int K, void* stream) {
    FVLA_REQUIRE(norm_w && norm_b && weight && weight_folded && colsum && bias_folded && N > 0 && K > 0, "fold_layernorm: bad arguments");
    fold_layernorm_kernel<<<(N + 127) / 128, 128, 0, S(stream)>>>(B(norm_w), B(norm_b), B(weight), B(bias), Bm(weight_folded), colsum,
                                                                 bias_folded, N, K);
    return check_launch("fold_layernorm_kernel");
}

int fvla_fused_norm_supported(int M, int N, int K, int rope) {
    return tc5_enabled() && tc5::normed_tile_width(M, N, K, rope != 0) != 0 ? 1 : 0;
}

int fvla_vision_folded_norm_linear(const void* x, const void* weight_folded, const float* colsum, const float* bias_folded,
                                   void* out, int M, int N, int K, int act, void* stream) {
    FVLA_REQUIRE(x && weight_folded && colsum && bias_folded && out && M > 0 && N > 0 && K > 0 && (act == 0 || act == 1),
                 "vision_folded_norm_linear: bad arguments");
    GemmArgs a;
    a.A = B(x); a.lda = K; a.B = B(weight_folded); a.ldb = N; a.C = out; a.ldc = N;
    a.act = act; a.M = M; a.N = N; a.K = K; a.trigger_early = act;      // after the up projection the down GEMM follows
    a.norm_mode = 2; a.colsum = colsum; a.bias_f32 = bias_folded;
    const int rc = tc5_enabled() ? tc5::launch_gemm_tc5_normed(a, device_status_ptr(), S(stream)) : FVLA_ERR_UNSUPPORTED;
    if (rc == FVLA_ERR_UNSUPPORTED)
        set_error("vision_folded_norm_linear: M=%d N=%d K=%d is outside the fused form (see fvla_fused_norm_supported)", M, N, K);
    return rc;
}

int fvla_encoder_projector(const void* x, const void* norm_w, const void* norm_b, const void* proj_w,
                           const void* proj_b, void* out, void* x_norm, int M, int N, int K, void* stream) {
    return norm_linear(x, norm_w, norm_b, proj_w, proj_b, out, x_norm, M, N, K, 0, stream, 0);
}

int fvla_vision_attention(const void* qkv, void* out, int views, int tokens, int heads, int head_dim,
                          void* stream) {
    FVLA_REQUIRE(views > 0 && tokens > 0 && heads > 0, "vision_attention: bad shape");
    if (head_dim != 72) { set_error("vision_attention: head_dim %d not built (72 only)", head_dim); return FVLA_ERR_UNSUPPORTED; }
    const int width = heads * head_dim;
    // tcgen05 kernel for the model's shape (FVLA_ATTN=mma / FVLA_GEMM=mma keep the warp-level kernel)
    static int attn_tc5 = -1;
    if (attn_tc5 < 0) { const char* v = getenv("FVLA_ATTN"); attn_tc5 = (v != nullptr && strcmp(v, "mma") == 0) ? 0 : 1; }
    if (attn_tc5 && tc5_enabled() && tokens == attn5::vis::TOK && aligned16(qkv) && aligned16(out))
        return attn5::vis::launch_vision_attention_tc5(qkv, out, views, heads, device_status_ptr(), S(stream));
    AttnArgs a{};
    a.q = B(qkv); a.k = B(qkv) + width; a.v = B(qkv) + 2 * width; a.out = Bm(out);
    a.q_stride = a.k_stride = a.v_stride = 3 * width; a.o_stride = width;
    a.q_bs0 = a.k_bs0 = a.v_bs0 = (long long)tokens * 3 * width; a.q_bs1 = a.k_bs1 = a.v_bs1 = head_dim;
    a.o_bs0 = (long long)tokens * width; a.o_bs1 = head_dim;
    a.batch_inner = heads; a.nq = tokens; a.nk = tokens; a.hd = head_dim; a.nq_pad = tokens;
    a.scale_log2 = kLog2e / sqrtf((float)head_dim);
    a.mask_rows = 0; a.mask_key_le = 0; a.splits = 1; a.keys_per_split = tokens;
    return launch_attention<80>(a, dim3((tokens + 63) / 64, views * heads, 1), S(stream));
}

int fvla_vision_linear_bias_residual(const void* x, const void* weight, const void* bias, const void* res,
                                     void* out, int M, int N, int K, void* ws, size_t ws_bytes, void* stream) {
    GemmArgs a;
    a.A = B(x); a.lda = K; a.B = B(weight); a.ldb = N; a.C = out; a.ldc = N; a.bias = B(bias);
    a.R = res; a.ldr = N; a.M = M; a.N = N; a.K = K;
    void* gws; size_t gn;
    gemm_ws(ws, ws_bytes, M, K, &gws, &gn);
    return launch_gemm(a, gws, gn, S(stream));
}

int fvla_encoder_norm_qkv_rope(const void* x, const void* weight_qkv, const void* rope, void* Q, void* K,
                               void* V, void* x_norm, int M, int Kdim, int heads, int head_dim, int group_rows,
                               int kv_group_pitch, void* stream) {
    FVLA_REQUIRE(M > 64, "encoder_norm_qkv_rope: M=%d must exceed 64 (no split-K scratch is taken)", M);
    FVLA_REQUIRE(group_rows >= 0 && (group_rows == 0 || (M % group_rows == 0 && kv_group_pitch >= group_rows)),
                 "encoder_norm_qkv_rope: M=%d is not a whole number of sequences of %d rows (K/V pitch %d rows)", M, group_rows, kv_group_pitch);
    return encoder_qkv_rope(x, weight_qkv, rope, Q, K, V, x_norm, M, Kdim, heads, head_dim, group_rows, kv_group_pitch, 0, stream);
}

int fvla_encoder_qkv_rope_fused_norm(const void* x, const void* weight_qkv, const void* rope, void* Q, void* K,
                                     void* V, void* x_norm, int M, int Kdim, int heads, int head_dim, int group_rows,
                                     int kv_group_pitch, void* stream) {
    FVLA_REQUIRE(M > 64, "encoder_qkv_rope_fused_norm: M=%d must exceed 64 (no split-K scratch is taken)", M);
    FVLA_REQUIRE(group_rows >= 0 && (group_rows == 0 || (M % group_rows == 0 && kv_group_pitch >= group_rows)),
                 "encoder_qkv_rope_fused_norm: M=%d is not a whole number of sequences of %d rows (K/V pitch %d rows)", M, group_rows, kv_group_pitch);
    return encoder_qkv_rope(x, weight_qkv, rope, Q, K, V, x_norm, M, Kdim, heads, head_dim, group_rows, kv_group_pitch, 1, stream);
}

size_t fvla_encoder_attention_workspace_bytes(int queries, int keys) {
    if (queries <= 0 || keys <= 0) return 0;
    const size_t qpad = (size_t)(queries + 63) / 64 * 64;
    return 2 * (align256(qpad * sizeof(float)) + align256(qpad * 256 * sizeof(float)));
}

int fvla_encoder_attention(const void* Q, const void* K, const void* V, void* out, int queries, int keys,
                           int head_dim, float scale, void* ws, size_t ws_bytes, void* stream) {
    FVLA_REQUIRE(queries > 0 && keys > 0, "encoder_attention: bad shape");
    if (head_dim != 256) { set_error("encoder_attention: head_dim %d not built (256 only)", head_dim); return FVLA_ERR_UNSUPPORTED; }
    AttnArgs a{};
    a.q = B(Q); a.k = B(K); a.v = B(V); a.out = Bm(out);
    a.q_stride = a.k_stride = a.v_stride = a.o_stride = head_dim;
    a.batch_inner = 1; a.nq = queries; a.nk = keys; a.hd = head_dim; a.nq_pad = queries;
    a.scale_log2 = scale * kLog2e; a.splits = 1; a.keys_per_split = keys;
    // tcgen05 kernel (FVLA_ATTN=mma keeps the warp-level kernels: diagnostic switch)
    static int attn_tc5 = -1;
    if (attn_tc5 < 0) { const char* v = getenv("FVLA_ATTN"); attn_tc5 = (v != nullptr && strcmp(v, "mma") == 0) ? 0 : 1; }
    if (attn_tc5 && tc5_enabled() && aligned16(Q) && aligned16(K) && aligned16(V))
        return attn5::launch_attention_tc5(Q, K, V, out, queries, keys, scale * kLog2e, device_status_ptr(), S(stream));
    const int q_tiles = (queries + 63) / 64;
    // With scratch, the keys are split in two: twice the CTAs, each with a one-tile K/V buffer so that two
    // share an SM; a second kernel merges the halves. Worth it when one wave of CTAs leaves SMs idle.
    if (ws != nullptr && ws_bytes >= fvla_encoder_attention_workspace_bytes(queries, keys) && keys > 128 && q_tiles < 2 * tc5::num_sms()) {
        const size_t qpad = (size_t)q_tiles * 64;
        a.splits = 2;
        a.keys_per_split = ((keys + 1) / 2 + 63) / 64 * 64;
        a.nq_pad = (int)qpad;
        a.part_lse = (float*)ws;
        a.part_o = (float*)((uint8_t*)ws + 2 * align256(qpad * sizeof(float)));
        a.out = nullptr;
        int rc = launch_attention<256, 1>(a, dim3(q_tiles, 1, 2), S(stream));
        if (rc) return rc;
        cudaError_t e = launch_pdl(attention_combine_kernel, dim3((queries + 1) / 2), dim3(128), 0, S(stream),
                                   (const float*)a.part_o, (const float*)a.part_lse, Bm(out), queries, (int)qpad, head_dim, 2);
        if (e != cudaSuccess) { set_error("attention_combine_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        return check_launch("attention_combine_kernel");
    }
    return launch_attention<256>(a, dim3(q_tiles, 1, 1), S(stream));
}

// bf16 copy of `count` fp32 values (count % 4 == 0), for the kernels that cannot maintain a shadow of the
// fp32 residual stream in their own epilogue.
static int refresh_shadow(const void* src, void* dst, size_t count, cudaStream_t st) {
    FVLA_REQUIRE(count % 4 == 0 && aligned16(src) && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0, "shadow refresh: misaligned");
    const int blocks = (int)((count / 4 + 255) / 256);
    f32_to_bf16_kernel<<<blocks, 256, 0, st>>>(static_cast<const float*>(src), Bm(dst), count / 4);
    return check_launch("f32_to_bf16_kernel");
}

int fvla_linear_residual(const void* x, const void* weight, void* out, int out_is_f32, void* out_shadow, int M,
                         int N, int K, int group_rows, void* ws, size_t ws_bytes, void* stream) {
    FVLA_REQUIRE(group_rows >= 0 && (group_rows == 0 || M % group_rows == 0), "linear_residual: M=%d is not a whole number of groups of %d rows", M, group_rows);
    // rows as several groups of at most 64 (a batch of episodes): the decoder's cluster GEMM once per group in
    // one launch, each group streaming the weights from L2 after the first has pulled them from HBM
    const int rows = group_rows > 0 ? group_rows : M, groups = group_rows > 0 ? M / group_rows : 1;
    if (tc5_enabled() && skinny::plan_skinny(rows, N, K, false).ok && aligned16(x) && aligned16(weight)) {
        skinny::SkinnyArgs sa{};
        sa.x = x; sa.x_f32 = 0; sa.ldx = K; sa.M = rows; sa.N = N; sa.K = K; sa.groups = groups;
        sa.out = out; sa.out_f32 = out_is_f32; sa.ldo = N; sa.out_shadow = Bm(out_shadow);
        sa.status = device_status_ptr(); FVLA_DBG_ATTACH(sa);
        // With several row groups the clusters of one launch may not all be resident at once (about 15 clusters of
        // 8, 33 of 4, 74 of 2), and a second round of clusters costs as much as the first. K is then cut into 2, 4 or
        // 8 parts, one launch each, with the widest split whose clusters of all groups ARE resident together; every
        // launch after the first accumulates onto the result of the one before (the residual form does that anyway).
        auto resident = [](int splits) { return splits >= 8 ? 15 * 8 : (splits == 4 ? 33 * 4 : 148); };
        const skinny::SkinnyPlan whole = skinny::plan_skinny(rows, N, K, false, groups);
        if (groups > 1 && whole.tiles * whole.splits * groups > resident(whole.splits)) {
            for (int parts = 2; parts <= 8; parts *= 2) {
                if (K % parts || (K / parts) % 64) break;
                const skinny::SkinnyPlan part = skinny::plan_skinny(rows, N, K / parts, false, groups);
                if (!part.ok || part.tiles * part.splits * groups > resident(part.splits)) continue;
                sa.K = K / parts;
                for (int i = 0; i < parts; ++i) {
                    sa.x = B(x) + (size_t)i * (K / parts);
                    int rc = skinny::launch_skinny<skinny::EPI_RESIDUAL>(sa, B(weight) + (size_t)i * (K / parts) * N, nullptr, N, S(stream));
                    if (rc) return rc;
                }
                return FVLA_OK;
            }
            sa.K = K; sa.x = x;
        }
        return skinny::launch_skinny<skinny::EPI_RESIDUAL>(sa, weight, nullptr, N, S(stream));
    }
    FVLA_REQUIRE(out_shadow == nullptr || out_is_f32, "linear_residual: a bf16 shadow only makes sense for an fp32 `out`");
    GemmArgs a;
    a.A = B(x); a.lda = K; a.B = B(weight); a.ldb = N; a.C = out; a.ldc = N; a.c_f32 = out_is_f32;
    a.R = out; a.ldr = N; a.M = M; a.N = N; a.K = K;
    void* gws; size_t gn;
    gemm_ws(ws, ws_bytes, M, K, &gws, &gn);
    int rc = launch_gemm(a, gws, gn, S(stream));
    if (rc || out_shadow == nullptr) return rc;
    return refresh_shadow(out, out_shadow, (size_t)M * N, S(stream));      // these kernels do not write the shadow themselves
}

int fvla_encoder_norm_gated_ffn(const void* x, const void* gate_w, const void* up_w, void* out, void* x_norm,
                                int M, int N, int K, void* stream) {
    FVLA_REQUIRE(M > 64, "encoder_norm_gated_ffn: M=%d must exceed 64 (no split-K scratch is taken)", M);
    int rc = rownorm(x, 0, nullptr, nullptr, x_norm, nullptr, nullptr, M, K, 1, S(stream));
    if (rc) return rc;
    GemmArgs a;
    a.A = B(x_norm); a.lda = K; a.B = B(gate_w); a.B2 = B(up_w); a.ldb = N; a.C = out; a.ldc = N;
    a.M = M; a.N = N; a.K = K;
    a.trigger_early = 1;      // the next kernel (prefix attention / down projection) runs one CTA per SM
    return launch_gemm(a, nullptr, 0, S(stream));
}

int fvla_decoder_small_proj(const void* x, int x_is_f32, const void* weight, const void* bias, void* out,
                            int out_is_f32, void* out_shadow, int M, int N, int K, int act, void* ws,
                            size_t ws_bytes, void* stream) {
    FVLA_REQUIRE(M > 0 && N > 0 && K > 0 && (act == 0 || act == 2), "small_proj: bad arguments");
    if (K <= 64) {
        FVLA_REQUIRE(out_shadow == nullptr, "small_proj: no bf16 shadow for K <= 64");
        dim3 grid((N + 255) / 256, M);
        cudaStream_t st = S(stream);
        cudaError_t e;
        if (x_is_f32 && out_is_f32)
            e = launch_pdl(small_k_proj_kernel<float, float>, grid, dim3(256), 0, st, (const float*)x, B(weight), B(bias), (float*)out, M, N, K, act);
        else if (x_is_f32)
            e = launch_pdl(small_k_proj_kernel<float, bf16>, grid, dim3(256), 0, st, (const float*)x, B(weight), B(bias), Bm(out), M, N, K, act);
        else if (out_is_f32)
            e = launch_pdl(small_k_proj_kernel<bf16, float>, grid, dim3(256), 0, st, B(x), B(weight), B(bias), (float*)out, M, N, K, act);
        else
            e = launch_pdl(small_k_proj_kernel<bf16, bf16>, grid, dim3(256), 0, st, B(x), B(weight), B(bias), Bm(out), M, N, K, act);
        if (e != cudaSuccess) { set_error("small_k_proj_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
        return check_launch("small_k_proj_kernel");
    }
    if (tc5_enabled() && skinny::plan_skinny(M, N, K, false).ok && aligned16(x) && aligned16(weight)) {
        skinny::SkinnyArgs sa{};
        sa.x = x; sa.x_f32 = x_is_f32; sa.ldx = K; sa.M = M; sa.N = N; sa.K = K;
        sa.out = out; sa.out_f32 = out_is_f32; sa.ldo = N; sa.bias = B(bias); sa.act = act;
        sa.out_shadow = Bm(out_shadow); sa.status = device_status_ptr(); FVLA_DBG_ATTACH(sa);
        return skinny::launch_skinny<skinny::EPI_BIAS>(sa, weight, nullptr, N, S(stream));
    }
    FVLA_REQUIRE(!x_is_f32, "small_proj: fp32 input only for K <= 64");
    FVLA_REQUIRE(out_shadow == nullptr || out_is_f32, "small_proj: a bf16 shadow only makes sense for an fp32 `out`");
    GemmArgs a;
    a.A = B(x); a.lda = K; a.B = B(weight); a.ldb = N; a.C = out; a.ldc = N; a.c_f32 = out_is_f32;
    a.bias = B(bias); a.act = act; a.M = M; a.N = N; a.K = K;
    void* gws; size_t gn;
    gemm_ws(ws, ws_bytes, M, K, &gws, &gn);
    int rc = launch_gemm(a, gws, gn, S(stream));
    if (rc || out_shadow == nullptr) return rc;
    return refresh_shadow(out, out_shadow, (size_t)M * N, S(stream));
}

// Shared front half of the two decoder norm+GEMM ops: factor (and, for an fp32 residual stream,
// the bf16 normalised rows) into the workspace; fills A / row_scale of the GEMM accordingly.
static int decoder_norm_front(const void* x, int x_is_f32, void* norm_factor, int M, int N, int K, bool dual,
                              void* ws, size_t ws_bytes, const char* who, GemmArgs* a, void* stream) {
    if (ws == nullptr || ws_bytes < op_ws_bytes(M, N, K, dual)) {
        set_error("%s: workspace of %zu bytes needed", who, op_ws_bytes(M, N, K, dual));
        return FVLA_ERR_WORKSPACE;
    }
    float* factors = (float*)ws;
    bf16* xnorm = (bf16*)((uint8_t*)ws + ws_factor_bytes(M));
    int rc = rownorm(x, x_is_f32, nullptr, nullptr, x_is_f32 ? xnorm : nullptr, factors, norm_factor, M, K, 2, S(stream));
    if (rc) return rc;
    if (x_is_f32) { a->A = xnorm; a->row_scale = nullptr; }       // rows already scaled, then rounded once
    else { a->A = B(x); a->row_scale = factors; }                 // bf16 rows: scale the fp32 accumulators
    a->lda = K; a->M = M; a->N = N; a->K = K;
    return FVLA_OK;
}

int fvla_decoder_norm_qkv_rope(const void* x, int x_is_f32, const void* x_shadow, const void* weight_qkv, const void* rope, void* Q,
                               void* K, void* V, void* norm_factor, int M, int Kdim, int heads, int head_dim,
                               int group_rows, int kv_group_pitch, void* ws, size_t ws_bytes, void* stream) {
    const int N = (heads + 2) * head_dim;
    FVLA_REQUIRE(group_rows >= 0 && (group_rows == 0 || (M % group_rows == 0 && kv_group_pitch >= group_rows)),
                 "decoder_norm_qkv_rope: M=%d is not a whole number of sequences of %d rows (K/V pitch %d rows)", M, group_rows, kv_group_pitch);
    if (group_rows == 0 && tc5_enabled() && skinny::plan_skinny(M, N, Kdim, false).ok && aligned16(x) && aligned16(weight_qkv) &&
        head_dim % 2 == 0) {
        skinny::SkinnyArgs sa{};
        sa.x = x; sa.x_f32 = x_is_f32; sa.x_shadow = B(x_shadow); sa.ldx = Kdim; sa.M = M; sa.N = N; sa.K = Kdim; sa.need_factor = 1;
        sa.rope = B(rope); sa.q = Bm(Q); sa.k = Bm(K); sa.v = Bm(V); sa.heads = heads; sa.head_dim = head_dim;
        sa.factor_out = Bm(norm_factor); sa.status = device_status_ptr(); FVLA_DBG_ATTACH(sa);
        return skinny::launch_skinny<skinny::EPI_QKV_ROPE>(sa, weight_qkv, nullptr, N, S(stream));
    }
    GemmArgs a;
    int rc = decoder_norm_front(x, x_is_f32, norm_factor, M, N, Kdim, false, ws, ws_bytes, "decoder_norm_qkv_rope", &a, stream);
    if (rc) return rc;
    a.B = B(weight_qkv); a.ldb = N;
    a.rope = B(rope); a.q = Bm(Q); a.k = Bm(K); a.v = Bm(V); a.heads = heads; a.head_dim = head_dim;
    a.group_rows = group_rows; a.kv_group_pitch = kv_group_pitch;
    void* gws; size_t gn;
    gemm_ws(ws, ws_bytes, M, Kdim, &gws, &gn);
    return launch_gemm(a, gws, gn, S(stream));
}

int fvla_decoder_attention(const void* Q, const void* K, const void* V, void* out, int queries, int keys,
                           int head_dim, int heads, int encoder_seq_len, int episodes, long long q_episode_stride,
                           long long kv_episode_stride, void* ws, size_t ws_bytes, void* stream) {
    FVLA_REQUIRE(queries > 0 && keys > 0 && episodes >= 1, "decoder_attention: bad shape");
    FVLA_REQUIRE(episodes == 1 || (tc5_enabled() && q_episode_stride >= (long long)queries * head_dim &&
                                   kv_episode_stride >= (long long)keys * head_dim && q_episode_stride % 8 == 0 && kv_episode_stride % 8 == 0),
                 "decoder_attention: a batch of episodes needs the tcgen05 kernels and 16-byte aligned episode strides");
    if (head_dim != 256) { set_error("decoder_attention: head_dim %d not built (256 only)", head_dim); return FVLA_ERR_UNSUPPORTED; }
    // A batch of episodes goes to the tcgen05 flash kernel (128 flat query rows per CTA, one grid row per episode,
    // state-token mask): at one episode its 4 query tiles would occupy 8 SMs and the cluster kernel below is faster,
    // but the cluster kernel's 8-CTA clusters are resident 15 at a time, so E episodes take E / 1.15 rounds of it.
    static int batched_tc5 = -1;
    if (batched_tc5 < 0) { const char* v = getenv("FVLA_DEC_ATTN"); batched_tc5 = (v != nullptr && strcmp(v, "cluster") == 0) ? 0 : 1; }
    if (episodes > 1 && batched_tc5 && tc5_enabled() && aligned16(Q) && aligned16(K) && aligned16(V) && aligned16(out))
        return attn5::launch_attention_tc5(Q, K, V, out, queries, keys, kLog2e / sqrtf((float)head_dim), device_status_ptr(), S(stream),
                                           episodes, q_episode_stride, kv_episode_stride, heads, encoder_seq_len);
    FVLA_REQUIRE(episodes == 1 || keys <= decattn::MAX_SPL * 128, "decoder_attention: the cluster kernel takes at most %d keys", decattn::MAX_SPL * 128);
    if (ws == nullptr || ws_bytes < fvla_decoder_attention_workspace_bytes(queries, keys)) {
        set_error("decoder_attention: workspace of %zu bytes needed", fvla_decoder_attention_workspace_bytes(queries, keys));
        return FVLA_ERR_WORKSPACE;
    }
    if (tc5_enabled() && keys <= decattn::MAX_SPL * 128 && aligned16(Q) && aligned16(K) && aligned16(V)) {        // cluster kernel: 8..11 key splits of at most 128 keys
        DecAttnArgs d{};
        d.q = B(Q); d.k = B(K); d.v = B(V); d.out = Bm(out);
        d.splits = (keys + 127) / 128 < decattn::MIN_SPL ? decattn::MIN_SPL : (keys + 127) / 128;
        d.nq = queries; d.nk = keys; d.keys_per_split = ((keys + d.splits - 1) / d.splits + 7) / 8 * 8;
        d.scale_log2 = kLog2e / sqrtf((float)head_dim);
        d.mask_rows = heads; d.mask_key_le = encoder_seq_len; d.prefix_keys = encoder_seq_len;
        d.episodes = episodes; d.q_episode_stride = q_episode_stride; d.kv_episode_stride = kv_episode_stride;
        d.status = device_status_ptr(); FVLA_DBG_ATTACH(d);
        return launch_decoder_attention_cluster(d, pdl_enabled(), S(stream));
    }
    const int splits = (keys + 127) / 128;
    const int qpad = (queries + 63) / 64 * 64;
    AttnArgs a{};
    a.q = B(Q); a.k = B(K); a.v = B(V); a.out = nullptr;
    a.part_lse = (float*)ws;
    a.part_o = (float*)((uint8_t*)ws + align256((size_t)splits * qpad * sizeof(float)));
    a.q_stride = a.k_stride = a.v_stride = a.o_stride = head_dim;
    a.batch_inner = 1; a.nq = queries; a.nk = keys; a.hd = head_dim; a.nq_pad = qpad;
    a.scale_log2 = kLog2e / sqrtf((float)head_dim);
    a.mask_rows = heads; a.mask_key_le = encoder_seq_len;
    a.splits = splits; a.keys_per_split = 128;
    int rc = launch_attention<256>(a, dim3(qpad / 64, 1, splits), S(stream));
    if (rc) return rc;
    attention_combine_kernel<<<(queries + 1) / 2, 128, 0, S(stream)>>>(a.part_o, a.part_lse, Bm(out), queries, qpad, head_dim, splits);
    return check_launch("attention_combine_kernel");
}

int fvla_decoder_norm_gated_ffn(const void* x, int x_is_f32, const void* x_shadow, const void* gate_w, const void* up_w, void* out,
                                void* norm_factor, int M, int N, int K, void* ws, size_t ws_bytes, void* stream) {
    if (tc5_enabled() && skinny::plan_skinny(M, N, K, true).ok && aligned16(x) && aligned16(gate_w) && aligned16(up_w)) {
        skinny::SkinnyArgs sa{};
        sa.x = x; sa.x_f32 = x_is_f32; sa.x_shadow = B(x_shadow); sa.ldx = K; sa.M = M; sa.N = N; sa.K = K; sa.need_factor = 1;
        sa.out = out; sa.out_f32 = 0; sa.ldo = N; sa.factor_out = Bm(norm_factor); sa.status = device_status_ptr(); FVLA_DBG_ATTACH(sa);
        return skinny::launch_skinny<skinny::EPI_GEGLU>(sa, gate_w, up_w, N, S(stream));
    }
    GemmArgs a;
    int rc = decoder_norm_front(x, x_is_f32, norm_factor, M, N, K, true, ws, ws_bytes, "decoder_norm_gated_ffn", &a, stream);
    if (rc) return rc;
    a.B = B(gate_w); a.B2 = B(up_w); a.ldb = N; a.C = out; a.ldc = N;
    void* gws; size_t gn;
    gemm_ws(ws, ws_bytes, M, K, &gws, &gn);
    return launch_gemm(a, gws, gn, S(stream));
}

int fvla_decoder_action_out_proj(const void* x, int x_is_f32, const void* weight, const void* bias, void* out,
                                 int out_is_f32, void* mirror, void* norm_factor, int M, int N, int K,
                                 void* stream) {
    FVLA_REQUIRE(M > 0 && K > 0, "action_out_proj: bad shape");
    if (N != 32) { set_error("action_out_proj: N=%d not built (32 only)", N); return FVLA_ERR_UNSUPPORTED; }
    cudaStream_t st = S(stream);
    cudaError_t e;
    if (x_is_f32 && out_is_f32)
        e = launch_pdl(action_out_kernel<float, float>, dim3(M), dim3(256), 0, st, (const float*)x, B(weight), B(bias), (float*)out, Bm(mirror), Bm(norm_factor), K);
    else if (x_is_f32)
        e = launch_pdl(action_out_kernel<float, bf16>, dim3(M), dim3(256), 0, st, (const float*)x, B(weight), B(bias), Bm(out), Bm(mirror), Bm(norm_factor), K);
    else if (out_is_f32)
        e = launch_pdl(action_out_kernel<bf16, float>, dim3(M), dim3(256), 0, st, B(x), B(weight), B(bias), (float*)out, Bm(mirror), Bm(norm_factor), K);
    else
        e = launch_pdl(action_out_kernel<bf16, bf16>, dim3(M), dim3(256), 0, st, B(x), B(weight), B(bias), Bm(out), Bm(mirror), Bm(norm_factor), K);
    if (e != cudaSuccess) { set_error("action_out_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("action_out_kernel");
}

int fvla_convert_copy(const void* src, int src_is_f32, void* dst, int dst_is_f32, void* dst_shadow, size_t count, void* stream) {
    FVLA_REQUIRE(src != nullptr && dst != nullptr && count > 0 && count <= ((size_t)1 << 31), "convert_copy: null pointer or bad count");
    FVLA_REQUIRE(dst_shadow == nullptr || dst_is_f32, "convert_copy: a bf16 shadow only makes sense for an fp32 destination");
    const dim3 grid((unsigned)((count + 255) / 256)), block(256);
    cudaStream_t st = S(stream);
    cudaError_t e;
    if (src_is_f32 && dst_is_f32) e = launch_pdl(convert_copy_kernel<float, float>, grid, block, 0, st, (const float*)src, (float*)dst, Bm(dst_shadow), count);
    else if (src_is_f32) e = launch_pdl(convert_copy_kernel<float, bf16>, grid, block, 0, st, (const float*)src, Bm(dst), Bm(dst_shadow), count);
    else if (dst_is_f32) e = launch_pdl(convert_copy_kernel<bf16, float>, grid, block, 0, st, B(src), (float*)dst, Bm(dst_shadow), count);
    else e = launch_pdl(convert_copy_kernel<bf16, bf16>, grid, block, 0, st, B(src), Bm(dst), Bm(dst_shadow), count);
    if (e != cudaSuccess) { set_error("convert_copy_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("convert_copy_kernel");
}

int fvla_embed_rows(const void* table, const long long* ids, void* out, int rows, int dim, long long vocab, void* stream) {
    FVLA_REQUIRE(rows > 0 && dim > 0 && dim % 8 == 0 && vocab > 0, "embed_rows: bad shape rows=%d dim=%d (dim %% 8 == 0)", rows, dim);
    FVLA_REQUIRE(table != nullptr && ids != nullptr && out != nullptr && aligned16(table) && aligned16(out), "embed_rows: null or misaligned pointer");
    cudaError_t e = launch_pdl(embed_rows_kernel, dim3(rows), dim3(128), 0, S(stream), B(table), ids, Bm(out), dim, vocab, device_status_ptr());
    if (e != cudaSuccess) { set_error("embed_rows_kernel: %s", cudaGetErrorString(e)); return FVLA_ERR_LAUNCH; }
    return check_launch("embed_rows_kernel");
}

// ---- pinned launch plans -----------------------------------------------------------------------
int fvla_gemm_plan_set(int M, int N, int K, int kind, int engine, int bn, int splits) {
    FVLA_REQUIRE(M > 0 && N > 0 && K > 0 && kind >= PLAN_PLAIN && kind <= PLAN_SKINNY_DUAL, "gemm_plan_set: bad shape or kind");
    bool ok = false;
    switch (engine) {
        case ENGINE_TC5_SCRATCH: ok = (kind == PLAN_PLAIN && (bn == 64 || bn == 128 || bn == 192 || bn == 256) && splits >= 1 && splits <= 4) ||
                                      (kind == PLAN_DUAL && splits == 1); break;
        case ENGINE_TC5_CLUSTER: ok = kind == PLAN_PLAIN && splits >= 2 && splits <= 4; break;
        case ENGINE_PAIR: ok = (kind == PLAN_PLAIN && splits >= 1 && splits <= 6) || (kind == PLAN_DUAL && splits == 1); break;
        case ENGINE_SKINNY: ok = (kind == PLAN_SKINNY || kind == PLAN_SKINNY_DUAL) && (splits == 1 || splits == 2 || splits == 4 || splits == 8); break;
        default: ok = false;
    }
    FVLA_REQUIRE(ok, "gemm_plan_set: engine %d with tile width %d and %d splits is not a plan for kind %d", engine, bn, splits, kind);
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    for (PlanEntry& e : g_plans)
        if (e.M == M && e.N == N && e.K == K && e.kind == kind) { e.choice.engine = engine; e.choice.bn = bn; e.choice.splits = splits; return FVLA_OK; }
    PlanEntry e{M, N, K, kind, {}};
    e.choice.engine = engine; e.choice.bn = bn; e.choice.splits = splits;
    g_plans.push_back(e);
    g_plan_count.store((int)g_plans.size(), std::memory_order_release);
    return FVLA_OK;
}

int fvla_gemm_plan_clear(void) {
    std::lock_guard<std::mutex> lock(g_plan_mutex);
    g_plans.clear();
    g_plan_count.store(0, std::memory_order_release);
    return FVLA_OK;
}

int fvla_gemm_plan_count(void) { return g_plan_count.load(std::memory_order_acquire); }

// ---- failure-detection self-test ---------------------------------------------------------------
int fvla_selftest_wait_timeout(const void* x, const void* weight, void* out, int M, int N, int K,
                               unsigned spin_limit, void* stream) {
    FVLA_REQUIRE(spin_limit > 0 && spin_limit <= (1u << 16), "selftest: spin_limit must be in 1..65536");
    FVLA_REQUIRE(x != nullptr && weight != nullptr && out != nullptr && aligned16(x) && aligned16(weight) && aligned16(out),
                 "selftest: null or misaligned pointer");
    if (!skinny::plan_skinny(M, N, K, false).ok) { set_error("selftest: shape %dx%dx%d is not a cluster-GEMM shape", M, N, K); return FVLA_ERR_UNSUPPORTED; }
    skinny::SkinnyArgs sa{};
    sa.x = x; sa.x_f32 = 0; sa.ldx = K; sa.M = M; sa.N = N; sa.K = K;
    sa.out = out; sa.out_f32 = 0; sa.ldo = N;
    sa.status = device_status_ptr();
    sa.spin_limit = spin_limit;
    sa.expect_extra_bytes = 16;           // the owners' barrier expects 16 bytes that no CTA ever sends
    return skinny::launch_skinny<skinny::EPI_RESIDUAL>(sa, weight, nullptr, N, S(stream));
}

#ifdef FVLA_DEBUG
// Development builds only (not declared in the public header): register the device buffer that the
// instrumented kernels stamp; `slots` x 2048 entries of 8 bytes. NULL unregisters.
int fvla_debug_set_timestamps(void* ptr, size_t bytes, int slots) {
    if (ptr == nullptr) { g_dbg_base = nullptr; g_dbg_slots = 0; return FVLA_OK; }
    cudaPointerAttributes attr{};
    FVLA_REQUIRE(cudaPointerGetAttributes(&attr, ptr) == cudaSuccess && attr.type == cudaMemoryTypeDevice,
                 "debug timestamps: not a device pointer");
    FVLA_REQUIRE(slots >= 1 && bytes >= (size_t)slots * 2048 * sizeof(unsigned long long) && (reinterpret_cast<uintptr_t>(ptr) & 7u) == 0,
                 "debug timestamps: buffer of %d x 16384 bytes needed", slots);
    g_dbg_base = static_cast<unsigned long long*>(ptr); g_dbg_slots = slots; g_dbg_next = 0;
    return FVLA_OK;
}
#endif

}  // extern "C"
