/* C ABI of libfvla_b200: hand-written sm_100a kernels for the Pi0 forward pass.
 *
 * Entry points for every call site of the reference's operation table
 * (revollllt/flash-vla, src/flash_vla/hardware/nvidia/h100/pi0/backends/tilelang/wrappers.py
 * and fused_wrappers.py), so that a backend module exposing ALL_WRAPPERS / FUSED_WRAPPERS
 * with the reference's signatures is a thin shim over these functions.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer. Unless a parameter says otherwise, tensors are bf16,
 *     row-major and contiguous; linear weights are (in, out) with the output axis contiguous.
 *   - `stream` is a cudaStream_t. Calls only enqueue work: they never allocate, free or
 *     synchronise, so they may be issued while a CUDA graph is being captured.
 *   - `ws` / `ws_bytes` is caller-owned scratch of at least the size returned by the matching
 *     *_workspace_bytes query; it must be zero-filled once before its first use (it holds
 *     tile semaphores that reset themselves) and must not be shared by kernels that may run
 *     concurrently. Pass NULL / 0 where the query returns 0.
 *   - Return value: FVLA_OK or a negative error code; fvla_last_error() gives the text of the
 *     last failure on the calling thread. Arguments are validated before anything is launched.
 *   - Aliasing that the reference relies on is supported: a residual may be the destination
 *     (wrappers.py:176-189, :279-306, :366-392); the decoder attention may write over Q
 *     (pipeline.py:119-121).
 */
#ifndef FLASH_VLA_B200_H_
#define FLASH_VLA_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FVLA_OK 0
#define FVLA_ERR_ARG (-1)         /* bad shape, stride or alignment */
#define FVLA_ERR_WORKSPACE (-2)   /* scratch missing or too small */
#define FVLA_ERR_LAUNCH (-3)      /* the CUDA runtime rejected a launch or an attribute */
#define FVLA_ERR_UNSUPPORTED (-4) /* shape outside what the kernels implement */

const char* fvla_last_error(void);
/* ABI version of this header; bumped on any signature change. */
int fvla_abi_version(void);
/* Number of kernel launches this library has enqueued in this process so far (captured launches
 * count once, at capture time). Lets a caller report how much of a pass ran in these kernels. */
unsigned long long fvla_launch_count(void);
/* Health word of the current device: 0, or a small positive code once a kernel gave up on one of its
 * bounded waits (1..6: which kernel; its output is then invalid) or met a bad token id (7). Reading
 * clears the word. Negative: error code. This one call synchronises `stream`. */
int fvla_device_status(void* stream);
/* No counterpart in the reference (which has no device-side error reporting, only Python exceptions).
 * Failure-detection self-test: runs the decoder's cluster GEMM (out += x(M,K) @ W(K,N), all bf16, a
 * shape fvla_linear_residual serves with M <= 64) with the CTAs that finish the tiles told to wait for
 * 16 bytes that no CTA ever sends, and with that wait limited to `spin_limit` polls (1..65536). The
 * kernel must give up, release its tensor memory and return within milliseconds; fvla_device_status
 * then reports 2 and `out` is unspecified. Nothing faults and the context stays usable. */
int fvla_selftest_wait_timeout(const void* x, const void* weight, void* out, int M, int N, int K,
                               unsigned spin_limit, void* stream);

/* ---- Tuned launch plans ----------------------------------------------------------------------
 * Counterpart of the reference's per-kernel configuration sweep (benchmarks/autotune.py), whose winners the
 * reference writes into its TileLang kernel definitions. Here a measured-best launch plan can be pinned
 * per GEMM shape at run time; unpinned shapes use the library's cost models. `kind`: 0 plain (bias /
 * activation / residual epilogues), 1 QKV + RoPE, 2 gated FFN, 3 decoder cluster GEMM (M <= 64), 4 its
 * gated form. `engine`: 1 one-SM tcgen05 kernel with tile width bn (64, 128, 192, 256) and K split `splits`
 * (1..4) through caller scratch; 2 the same kernel, 128-wide tiles, K split (2..4) inside a thread-block
 * cluster; 3 the two-SM kernel, K split 1..6 through scratch (gated FFN: 1); 4 the decoder cluster GEMM
 * with `splits` (1, 2, 4, 8) CTAs along K. A launch that cannot honour its pinned plan fails with an
 * error instead of choosing another plan. Process-wide; set plans before capturing graphs and before the
 * scratch of the affected ops is first used: split-K scratch holds tile counters whose layout depends on
 * the plan, so one scratch buffer must not serve two plans. */
int fvla_gemm_plan_set(int M, int N, int K, int kind, int engine, int bn, int splits);
int fvla_gemm_plan_clear(void);
int fvla_gemm_plan_count(void);

/* Scratch needed by a GEMM-shaped op of the given logical size. `dual` = 1 for gated FFNs. */
size_t fvla_gemm_workspace_bytes(int M, int N, int K, int dual);
/* Scratch for the decoder's split-key attention with `queries` flat rows and `keys` keys. */
size_t fvla_decoder_attention_workspace_bytes(int queries, int keys);
/* Scratch for the patchified image matrix of `views` camera views. */
size_t fvla_patch_embed_workspace_bytes(int views);

/* ---- SigLIP vision tower (M = views * 256 tokens, width 1152) -------------------------- */
/* wrappers.py:252-265: patchify (views,224,224,3), (768,588) @ (588,1152) + bias + pos[row % 256]. */
int fvla_vision_patch_embed(const void* images, const void* patch_w, const void* patch_b,
                            const void* pos_emb, void* out, int views, void* ws, size_t ws_bytes,
                            void* stream);
/* No counterpart in the reference. Same result as fvla_vision_patch_embed, for callers that cannot
 * supply scratch memory: a control loop that may not call cudaMalloc (it stalls the whole device for
 * an unbounded time), a host program without an allocator, or code whose scratch pool is already
 * frozen. The patch matrix is kept in a fixed array inside the library instead (1.2 MB per GPU,
 * held until the process exits), which limits `views` to 4; more views return FVLA_ERR_WORKSPACE.
 * This function itself never allocates. The first call on each device looks up the array's device
 * address (cudaGetSymbolAddress, with that device current): make that first call before starting
 * any stream capture. All calls on a device share the one array and it keeps the last call's
 * contents; nothing in it has to start at zero, but two calls whose kernels may overlap on the GPU
 * (different streams) race on it, so keep them on one stream or order them with events. */
int fvla_vision_patch_embed_noalloc(const void* images, const void* patch_w, const void* patch_b,
                                    const void* pos_emb, void* out, int views, void* stream);
/* wrappers.py:268-276: x_norm = LayerNorm(x); out = x_norm @ W(K,N) + b. */
int fvla_vision_norm_qkv(const void* x, const void* norm_w, const void* norm_b, const void* qkv_w,
                         const void* qkv_b, void* out, void* x_norm, int M, int N, int K,
                         void* stream);
/* kernels/attention.py:20-26: packed (views,256,3,heads,head_dim) -> (views,256,heads*head_dim). */
int fvla_vision_attention(const void* qkv, void* out, int views, int tokens, int heads,
                          int head_dim, void* stream);
/* wrappers.py:279-288 and :301-306: out = x(M,K) @ W(K,N) + b + res; res may alias out.
 * `ws` (fvla_gemm_workspace_bytes(M, N, K, 0), zero-initialised once) lets the kernel split K when the
 * output has too few tiles to fill the GPU; NULL is allowed and disables the split. */
int fvla_vision_linear_bias_residual(const void* x, const void* weight, const void* bias,
                                     const void* res, void* out, int M, int N, int K, void* ws,
                                     size_t ws_bytes, void* stream);
/* wrappers.py:291-298: x_norm = LayerNorm(x); out = gelu_tanh(x_norm @ W + b). */
int fvla_vision_norm_ffn_up(const void* x, const void* norm_w, const void* norm_b,
                            const void* weight, const void* bias, void* out, void* x_norm, int M,
                            int N, int K, void* stream);
/* LayerNorm folded into the linear layer behind it (the fused table's form of wrappers.py:268-276 and :291-298;
 * no counterpart in the reference). Set-up, once per weight: fvla_fold_layernorm writes
 *   weight_folded[k][n] = bf16(norm_w[k] * weight[k][n])   (K x N bf16)
 *   colsum[n]           = sum_k weight_folded[k][n]         (N fp32)
 *   bias_folded[n]      = sum_k norm_b[k] * weight[k][n] + bias[n]   (N fp32; bias may be NULL)
 * Per call: out = act(rstd * (x @ weight_folded - mean * colsum) + bias_folded), act 0 none / 1 gelu_tanh, with
 * each row's mean and rstd (eps 1e-5) taken inside the GEMM from its operand stages; no x_norm exists. The form
 * needs every CTA to own exactly one output tile: fvla_fused_norm_supported(M, N, K, rope) says whether a shape
 * qualifies (rope 1: the QKV + RoPE epilogue below); otherwise the call returns FVLA_ERR_UNSUPPORTED and the
 * caller uses fvla_vision_norm_qkv / fvla_vision_norm_ffn_up. */
int fvla_fold_layernorm(const void* norm_w, const void* norm_b, const void* weight, const void* bias,
                        void* weight_folded, float* colsum, float* bias_folded, int N, int K, void* stream);
int fvla_fused_norm_supported(int M, int N, int K, int rope);
int fvla_vision_folded_norm_linear(const void* x, const void* weight_folded, const float* colsum,
                                   const float* bias_folded, void* out, int M, int N, int K, int act,
                                   void* stream);

/* ---- Prefix encoder (M = S tokens, width 2048) ------------------------------------------ */
/* wrappers.py:336-344: x_norm = LayerNorm(x); out = x_norm @ W + b. */
int fvla_encoder_projector(const void* x, const void* norm_w, const void* norm_b, const void* proj_w,
                           const void* proj_b, void* out, void* x_norm, int M, int N, int K,
                           void* stream);
/* wrappers.py:347-363: x_norm = rms(x); proj = bf16(x_norm @ W); RoPE on adjacent pairs of the
 * Q heads and K; scatter to Q (M, heads*hd), K (M, hd), V (M, hd). rope is (M, hd) interleaved
 * cos/sin.
 * group_rows > 0 (an extension for batches of episodes): the M rows are M / group_rows sequences laid end
 * to end; rope is then (group_rows, hd) and is indexed by the position inside the sequence, and sequence
 * g's K / V rows go to rows [g * kv_group_pitch, + group_rows) of K / V (each sequence's cache holds
 * further rows that this call leaves alone). group_rows = 0: one sequence, contiguous K / V. */
int fvla_encoder_norm_qkv_rope(const void* x, const void* weight_qkv, const void* rope, void* Q,
                               void* K, void* V, void* x_norm, int M, int Kdim, int heads,
                               int head_dim, int group_rows, int kv_group_pitch, void* stream);
/* The same op with the RMS norm folded into the GEMM (the fused table's form; no counterpart in the reference,
 * whose fused table leaves the prefix encoder alone): the GEMM reads the raw rows of x, adds up each row's sum
 * of squares from its operand stages while the tensor cores run, and scales the accumulators before rounding
 * and RoPE. x_norm is NOT written then. Shapes that give a CTA more than one tile (M beyond 768 or so) fall
 * back to the two-kernel form and do write x_norm, which may only be NULL when that cannot happen. */
int fvla_encoder_qkv_rope_fused_norm(const void* x, const void* weight_qkv, const void* rope, void* Q,
                                     void* K, void* V, void* x_norm, int M, int Kdim, int heads,
                                     int head_dim, int group_rows, int kv_group_pitch, void* stream);
/* kernels/attention.py:29-34: unmasked multi-query attention, Q flat (tokens*heads, hd). With `ws`
 * (fvla_encoder_attention_workspace_bytes; contents need no initialisation) the keys are split over
 * twice as many CTAs and a second kernel merges the halves; NULL keeps the single-kernel form. */
size_t fvla_encoder_attention_workspace_bytes(int queries, int keys);
int fvla_encoder_attention(const void* Q, const void* K, const void* V, void* out, int queries,
                           int keys, int head_dim, float scale, void* ws, size_t ws_bytes, void* stream);
/* wrappers.py:366-371, :383-392 (encoder) and :176-189 (decoder): out += x(M,K) @ W(K,N). out is
 * bf16, or an fp32 residual stream when out_is_f32 != 0. out_shadow (may be NULL; fp32 out only) is a
 * bf16 tensor of out's shape that receives the rounded new value, for a later GEMM to read: written by
 * the GEMM's own epilogue for M <= 64, by a small conversion kernel after it otherwise.
 * group_rows > 0 (an extension for batches of episodes): the M rows are M / group_rows groups of at most
 * 64 rows; the decoder's weight-streaming kernel then runs once per group inside one launch. 0: one group. */
int fvla_linear_residual(const void* x, const void* weight, void* out, int out_is_f32, void* out_shadow,
                         int M, int N, int K, int group_rows, void* ws, size_t ws_bytes, void* stream);
/* wrappers.py:374-380: x_norm = rms(x); out = gelu(x_norm @ Wg) * (x_norm @ Wu). */
int fvla_encoder_norm_gated_ffn(const void* x, const void* gate_w, const void* up_w, void* out,
                                void* x_norm, int M, int N, int K, void* stream);

/* ---- Action-expert decoder (M = chunk + 1 rows, width 1024) ------------------------------ */
/* wrappers.py:108-128: out = act(x(M,K) @ W(K,N) + b); act 0 none, 2 silu; K <= 64 uses a
 * dedicated kernel. x is bf16, or fp32 when x_is_f32 != 0 (K <= 64 only); out likewise. */
int fvla_decoder_small_proj(const void* x, int x_is_f32, const void* weight, const void* bias,
                            void* out, int out_is_f32, void* out_shadow, int M, int N, int K, int act,
                            void* ws, size_t ws_bytes, void* stream);
/* wrappers.py:131-144: factor = rsqrt(mean(x^2)+1e-6) (also stored, bf16, in norm_factor when
 * not NULL); projection scaled by it, RoPE in fp32, single rounding, scatter to Q / K / V.
 * x is the bf16 residual stream, or an fp32 one when x_is_f32 != 0; x_shadow (may be NULL) is a
 * current bf16 copy of an fp32 x, which spares the kernel the conversion.
 * group_rows > 0 (an extension for batches of episodes): the M rows are M / group_rows episodes of
 * group_rows tokens each; rope is (group_rows, hd), indexed by the token's position inside its episode,
 * and episode g's K / V rows go to rows [g * kv_group_pitch, + group_rows) of K / V (the tail of that
 * episode's cache). group_rows = 0: one episode, contiguous K / V. */
int fvla_decoder_norm_qkv_rope(const void* x, int x_is_f32, const void* x_shadow, const void* weight_qkv, const void* rope, void* Q,
                               void* K, void* V, void* norm_factor, int M, int Kdim, int heads,
                               int head_dim, int group_rows, int kv_group_pitch, void* ws, size_t ws_bytes,
                               void* stream);
/* fused_wrappers.py:88-115 (and the unfused chain wrappers.py:147-173): softmax(Q K^T / sqrt(hd))
 * V over all `keys`, with rows < heads (the state token) limited to keys j <= encoder_seq_len.
 * out may alias Q.
 * Precondition on K / V rows [0, encoder_seq_len) (the prefix cache): they must be complete before the
 * kernel that precedes this call in `stream` STARTS, not merely before it ends. The kernel fetches those
 * rows while its predecessor is still finishing (programmatic dependent launch) and only waits for the
 * predecessor before reading Q and the rows from encoder_seq_len on. A caller whose previous kernel in
 * the stream writes the prefix rows must put an event or another kernel between the two.
 * episodes > 1 (an extension): that many independent episodes in one launch; `queries` and `keys` are
 * per episode, episode e reads Q + e * q_episode_stride and K / V + e * kv_episode_stride (strides in
 * elements, multiples of 8) and writes out + e * q_episode_stride. A batch runs on the tcgen05 flash
 * kernel (one grid row per episode), which waits for its predecessor before any read. */
int fvla_decoder_attention(const void* Q, const void* K, const void* V, void* out, int queries,
                           int keys, int head_dim, int heads, int encoder_seq_len, int episodes,
                           long long q_episode_stride, long long kv_episode_stride, void* ws,
                           size_t ws_bytes, void* stream);
/* fused_wrappers.py:45-54 / wrappers.py:192-198: out = gelu(rms(x) @ Wg) * (rms(x) @ Wu). When
 * norm_factor is not NULL the bf16 factor is also stored there (the unfused side effect). */
int fvla_decoder_norm_gated_ffn(const void* x, int x_is_f32, const void* x_shadow, const void* gate_w, const void* up_w,
                                void* out, void* norm_factor, int M, int N, int K, void* ws,
                                size_t ws_bytes, void* stream);
/* fused_wrappers.py:57-67 / wrappers.py:201-208: out += b + rms(x)(M,K) @ W(K,32). x and out are
 * bf16, or fp32 when the matching flag != 0; `mirror`, if not NULL, receives the new value as bf16. */
int fvla_decoder_action_out_proj(const void* x, int x_is_f32, const void* weight, const void* bias, void* out,
                                 int out_is_f32, void* mirror, void* norm_factor, int M, int N,
                                 int K, void* stream);

/* No counterpart in the reference, where these are torch `copy_` calls inside the pipeline (pipeline.py:103,
 * engine.py:60): dst[i] = src[i] for `count` contiguous elements, each side bf16 or fp32; dst_shadow (may be
 * NULL; fp32 dst only) also receives the value as bf16. Keeps the small copies of the decoder step inside the
 * chain of programmatic dependent launches. */
int fvla_convert_copy(const void* src, int src_is_f32, void* dst, int dst_is_f32, void* dst_shadow,
                      size_t count, void* stream);

/* No counterpart in the reference, which accepts only precomputed `language_embeds` (engine.py:43, :60):
 * out[r, :] = table[ids[r], :], bf16 rows of `dim` elements (dim % 8 == 0), ids int64 on the device. An id
 * outside [0, vocab) gives a zero row and makes fvla_device_status report 7. */
int fvla_embed_rows(const void* table, const long long* ids, void* out, int rows, int dim,
                    long long vocab, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_VLA_B200_H_ */
