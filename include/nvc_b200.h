/*
 * nvc_b200.h -- C ABI of the B200-native (sm_100a) Qwen3 forward hot path that drops in
 * behind nano-vllm-candle's layer / runner API.
 *
 * The reference crate has no FFI of its own: its boundary is a set of Rust traits and
 * inherent methods that call candle tensor ops.  Each entry point
 * below names the reference interface (file:line, relative to the reference crate root)
 * whose body it replaces; INTEGRATION.md shows the Rust `extern "C"` block and the
 * candle CustomOp wrapper a maintainer would add.
 *
 * Conventions
 *   - plain C: pointers + sizes, no torch / candle types.  Every `*_d` / unqualified
 *     tensor pointer is a DEVICE pointer (CUdeviceptr cast to void*), caller-owned,
 *     row-major, contiguous unless a row stride (in ELEMENTS) is given.
 *   - `stream` is a cudaStream_t passed as void*.  Calls only ENQUEUE work on it
 *     (asynchronous w.r.t. the host) unless the name ends in `_sync` or the doc says so.
 *   - return value: NVC_OK (0) on success; negative NVC_E* for argument / shape / state
 *     errors; positive = 1000 + cudaError_t, 2000 + ncclResult_t.  Nothing aborts and
 *     nothing is swallowed (the reference's runner turns errors into EOS tokens,
 *     src/engine/llm_engine.rs:153-175; that policy stays on the Rust side).
 *   - one nvc_ctx per (process, device); a context is used from one host thread at a
 *     time (the reference is single-threaded: Rc<RefCell<..>>, src/engine/llm_engine.rs:17).
 *   - bf16 = IEEE bfloat16 bit pattern in uint16_t storage.
 *   - launch order: every kernel is launched with programmatic stream serialization (PDL) and signals its
 *     dependents at its first instruction, so a kernel of this library may START while the previous kernels of
 *     this library on the stream are still running.  It waits (griddepcontrol.wait) before reading anything
 *     those kernels produce, but reads its STATIC operands earlier: weights, norm vectors, the rope table,
 *     positions / slot_mapping / block_tables / context_lens / cu_seqlens, and - paged decode only - cache rows
 *     other than the slot of each sequence's newest token.  Static operands must therefore be complete when the
 *     call is enqueued in stream order by anything that is not a kernel of this library (memcpy, other
 *     libraries' kernels: those never signal early, so plain stream order is enough) and must never be the
 *     output of a kernel of this library in the same stream.
 *   - no CPU fallback: on a machine without a usable sm_100 device nvc_ctx_create fails.
 */
#ifndef NVC_B200_H
#define NVC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVC_ABI_VERSION 1

enum {
  NVC_OK = 0,
  NVC_EINVAL = -1,     /* bad argument (null pointer, non-positive size, misalignment) */
  NVC_ESHAPE = -2,     /* unsupported shape (e.g. head_dim != 128, K % 64 != 0)         */
  NVC_ENOTIMPL = -3,
  NVC_ESTATE = -4,     /* wrong call order / missing weights / not initialised          */
  NVC_ENOMEM = -5,     /* workspace / KV pool too small                                 */
  NVC_EDEVICE = -6,    /* no sm_100 device / driver entry point missing                 */
  NVC_ENCCL = -7,      /* NCCL library not loadable                                     */
  NVC_ENVLS = -8,      /* NVSwitch multicast not available (nvc_ctx_nvls_status says why) */
  NVC_CUDA_ERROR_BASE = 1000,
  NVC_NCCL_ERROR_BASE = 2000
};

typedef uint16_t nvc_bf16;
typedef struct nvc_ctx nvc_ctx;
typedef struct nvc_runner nvc_runner;
typedef struct nvc_engine nvc_engine;

/* ------------------------------------------------------------------ context */

int nvc_abi_version(void);
const char* nvc_status_string(int status);
/* Last error message recorded on this context (empty string if none). */
const char* nvc_last_error(const nvc_ctx* ctx);

/* Binds to CUDA device `device`; tp_rank/tp_size mirror TPConfig (src/tp.rs:3-70).
 * Fails with NVC_EDEVICE unless the device is compute capability 10.x. */
int nvc_ctx_create(int device, int tp_rank, int tp_size, nvc_ctx** out);
int nvc_ctx_destroy(nvc_ctx* ctx);
int nvc_ctx_device(const nvc_ctx* ctx);
int nvc_ctx_tp_rank(const nvc_ctx* ctx);
int nvc_ctx_tp_size(const nvc_ctx* ctx);
int nvc_ctx_num_sms(const nvc_ctx* ctx);
/* Kernels launched through this context so far (bench.py reports the per-step difference). */
uint64_t nvc_ctx_launch_count(const nvc_ctx* ctx);

/* Tensor-parallel communicator (absent in the reference: src/tp.rs has no collectives,
 * src/layers/linear.rs:184-198 does no all-reduce).  `unique_id` is the 128-byte
 * ncclUniqueId produced by nvc_nccl_unique_id on rank 0 and shipped to the other ranks
 * by the caller.  Blocking (rendezvous). */
int nvc_nccl_unique_id(void* unique_id_128B);
int nvc_ctx_init_nccl(nvc_ctx* ctx, const void* unique_id_128B);
/* In-place sum over the tp ranks of `count` bf16 / f32 elements (K9). */
int nvc_allreduce_bf16(nvc_ctx* ctx, nvc_bf16* buf, size_t count, void* stream);
int nvc_allreduce_f32(nvc_ctx* ctx, float* buf, size_t count, void* stream);
/* In-place all-gather: every rank contributes `count_per_rank` bytes at offset rank*count. */
int nvc_allgather_bytes(nvc_ctx* ctx, void* buf, size_t bytes_per_rank, void* stream);

/* Peer-memory all-reduce over NVLink / NVSwitch (one-shot, for decode-sized messages), fused with
 * the residual add + RMSNorm that follow every row-parallel linear.  Setup: every rank calls
 * nvc_ctx_p2p_export (allocates [flags | slot 0 | slot 1] and returns a 64-byte CUDA IPC handle),
 * the caller all-gathers the handles, every rank calls nvc_ctx_p2p_import with the tp_size x 64
 * bytes.  The row-parallel GEMM writes its partial [N, H] bf16 result into nvc_ctx_p2p_slot(s)
 * (alternate s between consecutive all-reduces), then
 *   nvc_p2p_allreduce_rmsnorm: sum = sum over ranks (fp32, rank order) of slot s;
 *     w != NULL: s = sum + residual_in; residual_out = s; out = bf16(rmsnorm(s) * w)  (K9 + K1)
 *     w == NULL: out = bf16(sum).
 * tp_size in {2, 4, 8}; N * H * 2 <= slot_bytes. */
int nvc_ctx_p2p_export(nvc_ctx* ctx, size_t slot_bytes, void* handle_64B);
int nvc_ctx_p2p_import(nvc_ctx* ctx, const void* handles_tp_x_64B);
int nvc_ctx_p2p_ready(const nvc_ctx* ctx);
size_t nvc_ctx_p2p_slot_bytes(const nvc_ctx* ctx);
void* nvc_ctx_p2p_slot(nvc_ctx* ctx, int slot);
int nvc_p2p_allreduce_rmsnorm(nvc_ctx* ctx, int slot, const float* residual_in, float* residual_out,
                              const nvc_bf16* w, float eps, nvc_bf16* out, int N, int H, void* stream);

/* In-switch (NVLS) all-reduce over the NVSwitch multicast object of the TP group, fused with the residual add +
 * RMSNorm that follow every row-parallel linear (same contract as nvc_p2p_allreduce_rmsnorm).
 *   nvc_ctx_nvls_init: COLLECTIVE - every rank of the group calls it with the same sizes, after
 *     nvc_ctx_init_nccl (whose unique id names the group; `group_name` may be NULL to use that name).  Allocates
 *     one buffer per rank [flags | slot | 3 LL buffers], binds it into one multicast object (cuMulticastCreate on
 *     rank 0; the POSIX descriptor travels to the peers over an abstract unix socket of the library's own) and maps
 *     it at a unicast and a multicast address.  Returns NVC_ENVLS on every rank alike when any rank cannot do its
 *     part (no multicast support, creation refused); nvc_ctx_nvls_status then says why and the caller stays on the
 *     peer-memory / NCCL path.
 *   nvc_ctx_nvls_slot: this rank's slot (device pointer, slot_bytes): where the row-parallel GEMM writes its
 *     partial [N, H] bf16 result when the two-shot kernel is to reduce it.
 *   nvc_nvls_allreduce_rmsnorm: x_partial = this rank's partial sums.  mode 0 chooses by size; 1 = LL one-shot
 *     (rank r multimem.st's its rows into every rank's LL buffer, readers spin on the data; x_partial anywhere;
 *     tp * N * H * 2 <= ll_buf_bytes); 2 = two-shot in the switch (multimem.ld_reduce of 1/tp of the slot,
 *     multimem.st of the sums in place, two flag barriers; x_partial must be nvc_ctx_nvls_slot); 3 = two-shot with
 *     the sums broadcast into an LL buffer (one barrier; N * H * 2 <= ll_buf_bytes).  Results are bit-identical on
 *     all ranks in every mode.  tp_size in {2, 4, 8}; H % 64 == 0, H <= 8192. */
int nvc_ctx_nvls_init(nvc_ctx* ctx, size_t slot_bytes, size_t ll_buf_bytes, const char* group_name);
int nvc_ctx_nvls_ready(const nvc_ctx* ctx);
const char* nvc_ctx_nvls_status(const nvc_ctx* ctx);
size_t nvc_ctx_nvls_slot_bytes(const nvc_ctx* ctx);
size_t nvc_ctx_nvls_ll_bytes(const nvc_ctx* ctx);
void* nvc_ctx_nvls_slot(nvc_ctx* ctx);
int nvc_nvls_allreduce_rmsnorm(nvc_ctx* ctx, const nvc_bf16* x_partial, const float* residual_in, float* residual_out,
                               const nvc_bf16* w, float eps, nvc_bf16* out, int N, int H, int mode, void* stream);
/* End of a TP step (vocab-parallel lm_head + per-shard argmax / sample): all-gather of the ranks' (best value,
 * token) candidates through the multicast LL buffers and merge - largest value, ties -> the larger token id
 * (llm_engine.rs:135-142 "last maximum") - in one kernel; out_tok [B] is identical on every rank.  out_val may be
 * NULL.  Replaces nvc_pack_argmax_pairs + nvc_allgather_bytes + the host-side merge. */
int nvc_nvls_argmax_merge(nvc_ctx* ctx, const float* best_val, const int32_t* best_tok, int32_t* out_tok, float* out_val,
                          int B, void* stream);

/* ------------------------------------------------------------------ kernels */

/* K0. Replaces Tensor::embedding in Qwen3Model::forward (src/models/qwen3.rs:465-468).
 * out[n, :] = table[ids[n], :].  ids must lie in [0, V) (validated by the caller on the host). */
int nvc_embed_gather(nvc_ctx* ctx, const int32_t* ids, const nvc_bf16* table, nvc_bf16* out,
                     int N, int H, int V, void* stream);

/* K1. Replaces RMSNorm::forward (src/layers/layernorm.rs:44-60), fused:
 *   s = f32(x) + residual_in (if residual_in != NULL, else s = f32(x));
 *   residual_out = s (if residual_out != NULL; may alias residual_in);
 *   out = bf16( s * rsqrt(mean(s^2) + eps) * w ).
 * x, out: bf16 [N, H]; residuals: f32 [N, H] (the reference keeps the residual stream
 * in f32, layernorm.rs:49-50); w: bf16 [H].  H % 8 == 0, H <= 16384. */
int nvc_fused_add_rmsnorm(nvc_ctx* ctx, const nvc_bf16* x, const float* residual_in,
                          float* residual_out, const nvc_bf16* w, float eps, nvc_bf16* out,
                          int N, int H, void* stream);

/* K3. Replaces candle_nn::Linear::forward inside every *ParallelLinear::forward
 * (src/layers/linear.rs:33-38,72-77,99-104,171-175,184-198) and compute_logits
 * (src/models/qwen3.rs:542-550):  C[M, Nout] = A[M, K] * W[Nout, K]^T  (W is the
 * reference's [out, in] layout), bf16 inputs, fp32 accumulation on tcgen05 / TMEM.
 * lda / ldc: row strides in elements.  K % 64 == 0, Nout % 16 == 0, lda % 8 == 0.
 * out_dtype: NVC_DT_BF16 or NVC_DT_F32. */
enum { NVC_DT_BF16 = 0, NVC_DT_F32 = 1 };
int nvc_gemm_bf16(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W, void* C, int ldc,
                  int out_dtype, int M, int Nout, int K, void* stream);

/* K3 + K6 fused.  Replaces Qwen3MLP::forward's gate_up projection and SiluAndMul
 * (src/models/qwen3.rs:323-327, src/layers/activation.rs:13-18) in one kernel:
 *   act[M, I] = silu(A Wgate^T) * (A Wup^T),  silu(x) = x / (1 + exp(-x)) on the fp32 accumulators.
 * W_gu16: bf16 [2I, K], the reference's fused [gate; up] rows (qwen3.rs:310) re-ordered in groups of
 * 16 so that both halves of a feature meet in one epilogue thread: rows [32g, 32g+16) = gate rows
 * [16g, 16g+16), rows [32g+16, 32g+32) = up rows [16g, 16g+16).  I % 16 == 0, K % 64 == 0. */
int nvc_gemm_bf16_silu_mul(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W_gu16, nvc_bf16* act,
                           int ldc, int M, int I, int K, void* stream);

/* C = act(A W^T) on the tcgen05 kernels with the activation in the epilogue; act: NVC_ACT_NONE or NVC_ACT_RELU2
 * (max(z, 0)^2 on the fp32 accumulators).  Shapes as nvc_gemm_bf16. */
int nvc_gemm_bf16_act(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W, void* C, int ldc, int out_dtype, int M,
                      int Nout, int K, int act, void* stream);

/* Grouped product on the tcgen05 kernel: the rows of A are sorted by group, every group starts at a multiple of 128 rows
 * (nvc_moe_sort_padded), W = [groups][Nout][K] and C[r] = act(A[r] . W[tile_group[r / 128]]^T); tiles whose tile_group
 * entry is negative are skipped.  M_cap (a multiple of 128) is the host's upper bound of the padded row count: the
 * launch depends on no device value and replays inside a CUDA graph.  Rows of A in a group's padding may hold anything;
 * their rows of C are written and mean nothing.  act: NVC_ACT_NONE or NVC_ACT_RELU2. */
int nvc_gemm_bf16_grouped(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W, void* C, int ldc, int out_dtype,
                          int M_cap, int Nout, int K, const int32_t* tile_group, int groups, int act, void* stream);

/* The same fused kernel with the tanh form of gelu on the gate (gated feed-forward of the Karuzen family):
 *   act[M, I] = gelu_tanh(A Wgate^T) * (A Wup^T),  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))),
 * hardware tanh on the fp32 accumulators; W_gu16 interleaved as for nvc_gemm_bf16_silu_mul. */
int nvc_gemm_bf16_gelu_mul(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W_gu16, nvc_bf16* act,
                           int ldc, int M, int I, int K, void* stream);

/* Host-side rope table: replaces RotaryEmbedding::build_cos_sin
 * (src/layers/rotary_embedding.rs:56-80), which the reference recomputes per call.
 * out: f32 [max_pos, head_dim]; row p = [cos(p*f_0..f_{hd/2-1}), sin(p*f_0..)], with
 * f_j = 1/theta^(2j/hd), all in f32 exactly as the reference (glibc powf/cosf/sinf on the
 * host, then one H2D copy).  Synchronous. */
int nvc_rope_table_init_sync(nvc_ctx* ctx, float theta, int head_dim, int max_pos, float* out);

/* K2. Replaces the split / q_norm / k_norm / RotaryEmbedding::apply block of
 * Qwen3Attention::forward (src/models/qwen3.rs:206-234, src/layers/rotary_embedding.rs:82-107)
 * and adds the KV-cache scatter (N3).  In place on qkv bf16 [N, (nh+2kv)*hd]:
 *   q_h <- rope(rmsnorm(q_h) * qw, positions[n]);  k_h <- rope(rmsnorm(k_h) * kw, positions[n]);
 *   if slot_mapping != NULL and slot_mapping[n] >= 0:
 *       k_cache[slot, h, :] = k_h;  v_cache[slot, h, :] = v_h      (bit-exact copies)
 * k_cache / v_cache: bf16 [num_slots, kv, hd] = [num_blocks, block_size, kv, hd].
 * qw == kw == NULL skips the norm (rope only = RotaryEmbedding::apply by itself).
 * hd must be 128. */
int nvc_qk_norm_rope_store(nvc_ctx* ctx, nvc_bf16* qkv, const nvc_bf16* qw, const nvc_bf16* kw,
                           float eps, const float* cos_sin, const int32_t* positions,
                           const int32_t* slot_mapping, nvc_bf16* k_cache, nvc_bf16* v_cache,
                           int N, int nh, int kv, int hd, void* stream);

/* K3 + K2: the fused QKV projection with K2 as its epilogue (Qwen3Attention::forward up to the attention call,
 * src/models/qwen3.rs:205-234).  qkv [M, (nh + 2 kv) * hd] contiguous = A W_qkv^T with q / k heads normalised and rotated
 * and the k / v rows scattered to the caches at slot_mapping[row] (may be NULL: no scatter) - exactly what nvc_gemm_bf16
 * followed by nvc_qk_norm_rope_store produce, bit for bit.  Prefill-sized M runs as ONE kernel (the pair GEMM's persistent
 * epilogue parks each head in shared memory and applies K2 there: the separate pass over the QKV buffer disappears);
 * other shapes run the two kernels. */
int nvc_qkv_proj_norm_rope(nvc_ctx* ctx, const nvc_bf16* A, int lda, const nvc_bf16* W_qkv, nvc_bf16* qkv, int M, int K,
                           const nvc_bf16* q_norm_w, const nvc_bf16* k_norm_w, float eps, const float* cos_sin,
                           const int32_t* positions, const int32_t* slot_mapping, nvc_bf16* k_cache, nvc_bf16* v_cache,
                           int nh, int kv, int hd, void* stream);

/* K2'. Stand-alone slot-mapping scatter (N3): cache[slot_mapping[n]] = {k,v}[n]; slot < 0 skips.
 * k, v: bf16 rows of kv*hd elements with row stride ld (elements).  Bit-exact. */
int nvc_store_kvcache(nvc_ctx* ctx, const nvc_bf16* k, const nvc_bf16* v, int ld,
                      nvc_bf16* k_cache, nvc_bf16* v_cache, const int32_t* slot_mapping,
                      int N, int kv, int hd, void* stream);

/* K4. Prefill: replaces the dense causal attention of Qwen3Attention::forward
 * (src/models/qwen3.rs:236-277) with varlen causal flash attention.  q: [N, nh, hd],
 * k, v: [N, kv, hd] (row strides ldq / ldk / ldv in elements, so they may point into the
 * fused qkv buffer); cu_seqlens: i32 [B+1] (device); sequence b owns rows
 * cu_seqlens[b]..cu_seqlens[b+1], positions 0..len (no cached prefix).
 * out: bf16 [N, nh*hd], head-major like the reference (:276-277).  GQA: q head h reads
 * kv head h / (nh/kv) (:236-256).  hd must be 128. */
int nvc_prefill_attn_varlen(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k, int ldk,
                            const nvc_bf16* v, int ldv, const int32_t* cu_seqlens, int B,
                            int total_tokens, int max_seqlen, int nh, int kv, int hd, float scale,
                            nvc_bf16* out, void* stream);

/* K4 (paged). The same kernel for sequences with a cached prefix (prefix caching, SURVEY.md 8f.1;
 * upstream nano-vllm passes block_table to flash_attn_varlen_func for this): q rows of sequence b
 * are the LAST q_len_b = cu_seqlens_q[b+1] - cu_seqlens_q[b] positions of a context of
 * context_lens[b] tokens whose K / V are read from the paged cache through block_tables
 * [B, bt_stride] (this step's k / v must already be stored there).  Causal: q row i sees keys
 * 0 .. context_lens[b] - q_len_b + i.  Cache rows past the context may hold anything (NaN included).
 * block_size in {16, 32, 64} or a multiple of 128. */
int nvc_prefill_attn_paged(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k_cache,
                           const nvc_bf16* v_cache, const int32_t* block_tables, int bt_stride,
                           const int32_t* context_lens, const int32_t* cu_seqlens_q, int B,
                           int total_q_tokens, int max_seqlen_q, int nh, int kv, int hd, int block_size,
                           int num_blocks, float scale, nvc_bf16* out, void* stream);

/* The same with a caller's output row stride ldo >= nh * hd (a multiple of 8; out 16-byte aligned): the heads' outputs may be the
 * left part of wider rows (a mixer that concatenates the outputs of two halves in front of one output projection). */
int nvc_prefill_attn_paged_ld(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k_cache,
                              const nvc_bf16* v_cache, const int32_t* block_tables, int bt_stride,
                              const int32_t* context_lens, const int32_t* cu_seqlens_q, int B,
                              int total_q_tokens, int max_seqlen_q, int nh, int kv, int hd, int block_size,
                              int num_blocks, float scale, nvc_bf16* out, int ldo, void* stream);

/* The same with a sink: sink (fp32 [nh], optional) adds the term exp(sink_h), as it stands, to the softmax denominator of every row
 * of head h; nothing is added to the numerator. */
int nvc_prefill_attn_paged_sink(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k_cache,
                                const nvc_bf16* v_cache, const int32_t* block_tables, int bt_stride,
                                const int32_t* context_lens, const int32_t* cu_seqlens_q, int B,
                                int total_q_tokens, int max_seqlen_q, int nh, int kv, int hd, int block_size,
                                int num_blocks, float scale, const float* sink, nvc_bf16* out, int ldo, void* stream);

/* K5. Decode: paged attention over block_tables (N2) with GQA head grouping.
 * q: [B, nh, hd] row stride ldq; caches [num_blocks, block_size, kv, hd];
 * block_tables: i32 [B, max_blocks] (-1 padded); context_lens: i32 [B] (tokens in the cache
 * INCLUDING the current one).  out: bf16 [B, nh*hd].
 * workspace: device scratch of at least nvc_paged_decode_workspace_bytes(...) bytes. */
size_t nvc_paged_decode_workspace_bytes(int B, int nh, int hd, int num_sms);
int nvc_paged_decode_attn(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k_cache,
                          const nvc_bf16* v_cache, const int32_t* block_tables, int max_blocks,
                          const int32_t* context_lens, int B, int nh, int kv, int hd, int block_size,
                          float scale, nvc_bf16* out, void* workspace, size_t workspace_bytes,
                          void* stream);

/* K5, allocation-free variant.  No counterpart in the reference: added at the request of the run's operators for
 * callers that cannot call cudaMalloc (CUDA graph capture, tight serving loops, harnesses that forbid it).  Same
 * kernels and results as nvc_paged_decode_attn; the KV-split partials go to a static device array inside the
 * library (nvc_paged_decode_static_scratch_bytes() = 4 MiB per GPU, held until exit) instead of a caller workspace.
 * Returns NVC_ENOMEM (nothing launched, message in nvc_last_error) when the shape's partials exceed that array -
 * the library's own split choice needs at most ~2.5 MB.  Calls no cudaMalloc / cudaFree.  All calls on a device
 * share the array: calls that overlap on the GPU (different streams) race; nothing in it has to be cleared between
 * calls (every partial read is written by the same call). */
size_t nvc_paged_decode_static_scratch_bytes(void);
int nvc_paged_decode_attn_static(nvc_ctx* ctx, const nvc_bf16* q, int ldq, const nvc_bf16* k_cache,
                                 const nvc_bf16* v_cache, const int32_t* block_tables, int max_blocks,
                                 const int32_t* context_lens, int B, int nh, int kv, int hd, int block_size,
                                 float scale, nvc_bf16* out, void* stream);

/* K6. Replaces SiluAndMul::forward (src/layers/activation.rs:13-18):
 * out[n, i] = silu(x[n, i]) * x[n, I + i]. */
int nvc_silu_and_mul(nvc_ctx* ctx, const nvc_bf16* x, nvc_bf16* out, int N, int I, void* stream);

/* K7. Row gather: out[b, :] = x[rows[b], :] (last token of each sequence before the final
 * norm / lm_head; the reference computes logits for all positions, src/models/qwen3.rs:548). */
int nvc_gather_rows(nvc_ctx* ctx, const nvc_bf16* x, const float* residual, const int32_t* rows,
                    nvc_bf16* x_out, float* residual_out, int B, int H, void* stream);

/* ---- mechanisms of the models with an fp32 residual stream (Karuzen).  `dtype` arguments are NVC_DT_BF16 (serving:
 * bf16 storage, fp32 arithmetic) or NVC_DT_F32 (exact mode: fp32 storage, plain IEEE products and sums); strides are in
 * elements; buffers may be wider than the logical row (padding columns are never written). ---- */
enum { NVC_ACT_NONE = 0, NVC_ACT_RELU2 = 1, NVC_ACT_GELU_TANH_MUL = 2 };   /* 3, 4: NVC_ACT_GELU_TANH, NVC_ACT_GLU_CLAMP below */

/* out[n, :H] = f32(table[ids[n], :H]). */
int nvc_embed_gather_f32(nvc_ctx* ctx, const int32_t* ids, const void* table, int table_dtype, int ldt, float* out, int ldo,
                         int N, int H, void* stream);
/* Dynamic Tanh norm fused with the residual accumulation (all sums fp32):
 *   s = res_in[r] + a0[r] + a1[r] + a2[r]   (each operand optional, fp32 [*, ld]);  res_out[r] = s (optional, may alias);
 *   out[i, j] = tanh(alpha * s_j) * w_j + b_j,  j < H     (w == NULL: accumulate only, out must be NULL).
 * rows == NULL: r = i; else r = rows[i] (gathers N rows; res_out must be NULL).  w, b: fp32 [H]; alpha: fp32 scalar in
 * device memory. */
int nvc_dyt_norm(nvc_ctx* ctx, const float* res_in, const float* a0, const float* a1, const float* a2, float* res_out, int ld,
                 const float* w, const float* b, const float* alpha, void* out, int out_dtype, int ldo, const int32_t* rows,
                 int N, int H, void* stream);
/* The two latents of latent attention from one fused down-projection row in[n] (fp32):
 *   out0[n, :n0]               = rmsnorm(in[n, :n0]) * w0          (query latent)
 *   cache[slot_mapping[n], :n1] = rmsnorm(in[n, off1 : off1 + n1]) * w1   (key / value latent; slot < 0 skips)
 * rmsnorm(x) = x / sqrt(mean(x^2) + eps) over the logical width.  cache may be NULL. */
int nvc_latent_norm_store(nvc_ctx* ctx, const float* in, int ldi, int n0, int off1, int n1, const float* w0, const float* w1,
                          float eps, void* out0, int ld0, void* cache, int ldc, const int32_t* slot_mapping, int dtype, int N,
                          void* stream);
/* kind NVC_ACT_GELU_TANH_MUL: out[n, j] = gelu_tanh(in[n, j]) * in[n, Fp + j];  NVC_ACT_RELU2: out[n, j] = max(in[n, j], 0)^2;
 * j < F.  in and out may alias for NVC_ACT_RELU2. */
int nvc_act_mul(nvc_ctx* ctx, const void* in, int ldi, void* out, int ldo, int dtype, int N, int F, int Fp, int kind, void* stream);
/* C[b] = act(A[b] . W[b]^T), any sizes (fp32 operands: FMA pipe, plain IEEE; bf16 operands with 16-byte-aligned rows - lda,
 * ldw, sa, sw, K multiples of 8 - tensor pipe with fp32 accumulators, other bf16 shapes: FMA pipe): A [M, K] (+ b * sa), W [N, K] (+ b * sw), C [M, N] (+ b * sc),
 * b < batch.  in_dtype: A and W; out_dtype: C (fp32 operands give fp32).  act: NVC_ACT_NONE or NVC_ACT_RELU2. */
int nvc_linear(nvc_ctx* ctx, const void* A, int lda, int64_t sa, const void* W, int ldw, int64_t sw, void* C, int ldc, int64_t sc,
               int in_dtype, int out_dtype, int M, int N, int K, int batch, int act, void* stream);
/* Grouped form: rows [offsets[g], offsets[g + 1]) of C are act(A[a_rows[r]] . (W + g * sw)^T); offsets: int32 [groups + 1] in
 * DEVICE memory, offsets[groups] <= max_rows; a_rows may be NULL (identity). */
int nvc_linear_grouped(nvc_ctx* ctx, const void* A, int lda, const int32_t* a_rows, const void* W, int ldw, int64_t sw, void* C,
                       int ldc, const int32_t* offsets, int groups, int max_rows, int in_dtype, int out_dtype, int N, int K, int act,
                       void* stream);
/* Router of a mixture of experts, one token per warp, fp32: z = W_router h; s = sigmoid(z); the `top` experts with the
 * largest s + correction (ties -> lower index) are chosen; topk_w = s_chosen / (sum of the chosen s + 1e-20) * scale.
 * gate[n] = sigmoid(w_shared_gate . h[n]) when w_shared_gate != NULL.  experts <= 256. */
int nvc_moe_route(nvc_ctx* ctx, const void* h, int h_dtype, int ldh, const float* w_router, const float* correction,
                  const float* w_shared_gate, int E, int top, float scale, int32_t* topk_idx, float* topk_w, float* gate, int N,
                  int H, void* stream);
/* The same choice from router logits that a matrix product has already taken (z fp32 [N, ldz], the weights of the router
 * as rows of one matrix); gate[n] = sigmoid(z[n, gate_col]) when gate_col >= 0. */
int nvc_moe_route_logits(nvc_ctx* ctx, const float* z, int ldz, const float* correction, int E, int top, float scale, int gate_col,
                         int32_t* topk_idx, float* topk_w, float* gate, int N, void* stream);
/* Stable counting sort of the N * top (token, choice) pairs by expert: offsets [E + 1], src_rows [N * top] (token of the
 * pair at each sorted position), pos [N * top] (sorted position of pair n * top + t). */
int nvc_moe_sort(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int32_t* offsets, int32_t* src_rows, int32_t* pos,
                 void* stream);
/* The same sort with every expert's group starting at a multiple of `align` rows (the layout of nvc_gemm_bf16_grouped,
 * align = 128): offsets[e] are the padded starts (offsets[E] = padded row count), src_rows has -1 in the padding rows,
 * pos points into the padded layout, and tile_group [tiles_cap] (optional) names the expert of every `align`-row tile, -1
 * behind the last group.  tiles_cap * align >= N * top + E * (align - 1); src_rows needs tiles_cap * align entries. */
int nvc_moe_sort_padded(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int align, int32_t* offsets, int32_t* src_rows,
                        int32_t* pos, int32_t* tile_group, int tiles_cap, void* stream);
/* out[r, :width] = in[src_rows[r], :width] for r < min(rows_cap, *num_rows) (num_rows: a count in device memory), zeros
 * where src_rows[r] < 0.  bf16 rows, width and strides multiples of 8. */
int nvc_gather_rows_bf16(nvc_ctx* ctx, const nvc_bf16* in, int ld_in, const int32_t* src_rows, const int32_t* num_rows, nvc_bf16* out,
                         int ld_out, int rows_cap, int width, void* stream);
/* out[n, :H] = sum_t topk_w[n, t] * y[pos[n * top + t], :H] + gate[n] * shared[n, :H]   (fp32; shared / gate optional). */
int nvc_moe_combine(nvc_ctx* ctx, const void* y, int y_dtype, int ldy, const int32_t* pos, const float* topk_w, int top,
                    const void* shared, int shared_dtype, int lds, const float* gate, float* out, int ldo, int N, int H,
                    void* stream);
/* Latent attention over a paged cache of shared latent rows (absorbed multi-head latent attention, no positional part):
 *   out[i, h, :D] = sum_{j <= pos_i} softmax_j(scale * q[i, h, :D] . c_j) * c_j,   c_j = cache[slot of token j, :D].
 * q / out: [rows, heads, head_stride] with row strides ldq / ldo; sequence b owns rows cu_seqlens[b] .. cu_seqlens[b + 1]
 * (cu_seqlens == NULL: one row per sequence), which are the LAST positions of its context_lens[b] tokens; the slot of token
 * j is block_tables[b, j / block_size] * block_size + j % block_size.  D <= 512.  bf16 rows with head_stride 64 or 128 run
 * on the tensor pipe and read head_stride numbers per row: columns [D, head_stride) of q and of the cache rows must be zero.
 * workspace (optional, device memory): lets a decode launch (max_qlen == 1) of a small batch split every sequence's keys
 * over up to 8 CTAs; B * ceil(heads / 16) * 16 * splits * (2 + head_stride) floats are used, fewer splits if it is smaller. */
int nvc_latent_attn_paged(nvc_ctx* ctx, const void* q, int ldq, const void* cache, int ldc, const int32_t* block_tables,
                          int bt_stride, const int32_t* context_lens, const int32_t* cu_seqlens, int B, int max_qlen, int heads,
                          int D, int head_stride, int block_size, float scale, void* out, int ldo, int dtype, void* workspace,
                          size_t workspace_bytes, void* stream);

/* ---- mechanisms of the models with RMS norms on an fp32 residual stream, windowed / sink attention and retention (Ranilix) ---- */
/* out[n, :H] = f32(table[ids[n], :H]) * scale. */
int nvc_embed_gather_scaled_f32(nvc_ctx* ctx, const int32_t* ids, const void* table, int table_dtype, int ldt, float scale, float* out,
                                int ldo, int N, int H, void* stream);
/* RMS norms fused with the residual accumulation (all sums fp32), up to two norms of the same sum:
 *   s = res_in[r] + a0[r] + a1[r]   (each operand optional, fp32 [*, ld]);  res_out[r] = s (optional, may alias);
 *   out0[i, :H] = s / sqrt(mean(s^2) + eps) * w0,  out1[i, :H] = ... * w1   (w0 == NULL: accumulate only; w1 optional).
 * rows == NULL: r = i; else r = rows[i] (gathers N rows; res_out must be NULL).  Both outputs have the row stride ldo. */
int nvc_rms_norm_pair(nvc_ctx* ctx, const float* res_in, const float* a0, const float* a1, float* res_out, int ld, const float* w0,
                      void* out0, const float* w1, void* out1, int out_dtype, int ldo, float eps, const int32_t* rows, int N, int H,
                      void* stream);
/* Output stage of a mixer, per (row, head) of vdim numbers: y = o (norm == 0) or o / sqrt(mean(o^2) + eps) (norm != 0, no
 * weight); out = y * act(gate) * out_scale with act = sigmoid or z sigmoid(z); gate == NULL: no gate.  o, gate: fp32. */
enum { NVC_GATE_SIGMOID = 0, NVC_GATE_SILU = 1 };
int nvc_head_gate(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, void* out, int ldout, int out_dtype, int heads,
                  int vdim, int norm, float eps, int act, float out_scale, int N, void* stream);
/* (cos, sin) of position * base^(-2 i / dims), i < dims / 2, for positions below max_pos: out fp32 [max_pos, dims / 2, 2] in
 * device memory, angles taken in double precision on the host.  Synchronous. */
int nvc_rotary_table_init_sync(nvc_ctx* ctx, float base, int dims, int max_pos, float* out);
/* Everything between a fused q / k / v projection (fp32 rows `in`) and the attention or recurrence behind it, in one pass:
 * bias; per-head RMS norm of q and k (weights of `dim` numbers shared by the heads); rotary positions on the first rot_dims
 * numbers of every q / k head - pairs (2i, 2i + 1), or (i, i + rot_dims / 2) when rot_half - with (cos, sin) from rot_table at
 * positions[n]; k *= k_scale; value blending (NVC_BLEND_PROVIDE: v_first[n] = v, NVC_BLEND_MIX: v <- (1 - *lambda) v +
 * *lambda v_first[n]); v *= v_scale; q goes to q_out[n], k and v to row slot_mapping[n] of k_out / v_out (a paged cache; a negative slot
 * skips the token) or to row n when slot_mapping == NULL. */
enum { NVC_BLEND_NONE = 0, NVC_BLEND_PROVIDE = 1, NVC_BLEND_MIX = 2 };
typedef struct nvc_qkv_prep {
  const float* in; int ldi;
  const float* bias;                      /* indexed like a row of `in`; NULL: none */
  int q_off, k_off, v_off;                /* first column of q / k / v in a row */
  int q_heads, kv_heads, dim, vdim;
  const float* q_norm; const float* k_norm; float eps;   /* both or neither */
  int rot_dims, rot_half; const float* rot_table; const int32_t* positions;
  float k_scale;
  int blend; const float* lambda; float* v_first; int ldvf;
  void* q_out; int ldq;
  void* k_out; void* v_out; int ldk, ldv;
  const int32_t* slot_mapping;
  int q_dtype, kv_dtype;
  float v_scale;                          /* v *= v_scale on the way out (after blending); a mixer's constant weight can ride here */
  int unit_norm;                          /* q and k heads are divided by their root mean square (eps inside the root) without a weight;
                                           * q_norm and k_norm must be NULL */
  int act;                                /* NVC_PREP_ACT_SILU: q, k and v go through z sigmoid(z) right after the bias */
} nvc_qkv_prep;
enum { NVC_PREP_ACT_NONE = 0, NVC_PREP_ACT_SILU = 1 };
int nvc_qkv_prep_run(nvc_ctx* ctx, const nvc_qkv_prep* p, int N, void* stream);
/* Grouped-query softmax attention over a paged cache with separate key and value widths:
 *   out[i, h, :vdim] = out_scale * gate_i,h * sum_j p_j v_j,   p_j = exp(s_j) / (sum_j' exp(s_j') + exp(sink_h)),
 *   s_j = scale * q[i, h] . k[j, h / (heads / kv_heads)],  j over max(0, pos_i - window + 1) .. pos_i  (window == 0: from 0).
 * sink (fp32 [heads]) and gate (fp32 [rows, ldg], through a sigmoid) are optional.  Rows, block tables and context lengths
 * as in nvc_latent_attn_paged (cu_seqlens == NULL: one row per sequence); rows = total query rows, max_qlen the longest
 * portion.  dim, vdim <= 512.  bf16 storage with dim and vdim multiples of 16 up to 256 runs on the tensor pipe, everything
 * else on the FMA pipe. */
typedef struct nvc_attn_spec {
  int heads, kv_heads, dim, vdim;
  float scale;
  int window;
  const float* sink;
  const float* gate; int ldg;
  float out_scale;
  float softcap;             /* > 0: s_j <- softcap * tanh(s_j / softcap) */
  int chunk;                 /* > 0 (window must be 0): j over pos_i - pos_i % chunk .. pos_i - the keys of the row's own chunk */
  int gate_per_head;         /* the gate is fp32 [rows, ldg] with ONE number per head (column h) instead of one per output number */
} nvc_attn_spec;
int nvc_attn_paged_wide(nvc_ctx* ctx, const void* q, int ldq, const void* k_cache, int ldk, const void* v_cache, int ldv,
                        const int32_t* block_tables, int bt_stride, const int32_t* context_lens, const int32_t* cu_seqlens, int B,
                        int rows, int max_qlen, int block_size, const nvc_attn_spec* spec, void* out, int ldo, int dtype, void* stream);
/* Retention: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head over the new tokens of every sequence (rows
 * cu_seqlens[b] .. cu_seqlens[b + 1], or row b when cu_seqlens == NULL).  state: fp32 [slots, heads, dim, vdim]; sequence b
 * uses slot state_slots[b], starts from zeros when positions[first row] == 0 and leaves its last state in the slot.
 * q, k, v, o: fp32 rows.  max_qlen: the longest portion; above 4 tokens the recurrence runs 32 tokens at a time (the same
 * sums regrouped, fp32 FMA), else token by token. */
int nvc_retention_scan(nvc_ctx* ctx, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, float* o, int ldo,
                       float* state, const int32_t* state_slots, const int32_t* cu_seqlens, const int32_t* positions,
                       const float* decay, int B, int max_qlen, int heads, int dim, int vdim, void* stream);

/* ---- mechanisms of the models with sandwich norms, rotary latent attention, the gated delta rule and softmax-routed experts
 * (Fefozen) ---- */
/* Norms in front of and behind a sublayer on an fp32 residual stream, in one pass over the row (all sums fp32):
 *   s = res_in[r] + y[r] / sqrt(mean(y[r]^2) + eps) * (wy + weight_offset)      (y == NULL: s = res_in[r]);
 *   res_out[r] = s (optional, may alias res_in);   out[i, :H] = s / sqrt(mean(s^2) + eps) * (w + weight_offset)   (w == NULL: none).
 * y is the sublayer's output (fp32 [*, ld]), wy the weight of the norm behind it, w the weight of the norm in front of the next
 * sublayer; weight_offset = 1 for weights stored around zero.  rows as in nvc_rms_norm_pair (gathers; res_out must be NULL). */
int nvc_rms_norm_sandwich(nvc_ctx* ctx, const float* res_in, const float* y, const float* wy, float* res_out, int ld, const float* w,
                          void* out, int out_dtype, int ldo, float eps, float weight_offset, const int32_t* rows, int N, int H,
                          void* stream);
/* nvc_latent_norm_store for latent attention with a rotated key part that all heads share: the cache row of a token is
 *   [ rmsnorm(in[n, off1 : off1 + n1]) * w1 | rot(in[n, off1 + n1 : off1 + n1 + rot_dim]) ]
 * where rot turns the first rot_dims numbers of the part by the angles of positions[n] ((cos, sin) table of
 * nvc_rotary_table_init_sync; pairs (2i, 2i + 1), or (i, i + rot_dims / 2) when rot_half) and leaves the rest.  cache == NULL:
 * only the query latent (a layer that reads another layer's rows). */
int nvc_latent_norm_store_rot(nvc_ctx* ctx, const float* in, int ldi, int n0, int off1, int n1, const float* w0, const float* w1,
                              float eps, void* out0, int ld0, void* cache, int ldc, const int32_t* slot_mapping, int rot_dim,
                              int rot_dims, int rot_half, const float* rot_table, const int32_t* positions, int dtype, int N,
                              void* stream);
/* Heads of a query projection laid out [heads][dim | rot_dim] (fp32 rows `in`): the unrotated part of head h goes to
 * out_a[n, h * hs_a : + dim], the rotated part (first rot_dims numbers turned as above) to out_b[n, h * hs_b + off_b : + rot_dim]. */
int nvc_head_split_rot(nvc_ctx* ctx, const float* in, int ldi, int heads, int dim, int rot_dim, int rot_dims, int rot_half,
                       const float* rot_table, const int32_t* positions, void* out_a, int ld_a, int hs_a, void* out_b, int ld_b,
                       int hs_b, int off_b, int dtype, int N, void* stream);
/* nvc_head_gate with a weight of vdim numbers shared by the heads on the normed output (NULL: none). */
int nvc_head_gate_w(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, const float* weight, void* out, int ldout,
                    int out_dtype, int heads, int vdim, int norm, float eps, int act, float out_scale, int N, void* stream);
/* nvc_act_mul with parameters.  NVC_ACT_GELU_TANH: out = gelu_tanh(in[n, j]).  NVC_ACT_GLU_CLAMP: g = min(in[n, j], p0),
 * u = clamp(in[n, Fp + j], -p0, p0), out = g * sigmoid(p1 * g) * (u + 1). */
enum { NVC_ACT_GELU_TANH = 3, NVC_ACT_GLU_CLAMP = 4 };
int nvc_act_mul_p(nvc_ctx* ctx, const void* in, int ldi, void* out, int ldo, int dtype, int N, int F, int Fp, int kind, float p0, float p1,
                  void* stream);
/* nvc_moe_route_logits with a choice of score function and weights: score NVC_ROUTE_SIGMOID or NVC_ROUTE_SOFTMAX (over all E
 * columns); normalize != 0: topk_w = s_chosen / (sum of the chosen s + 1e-20) * scale, else topk_w = s_chosen * scale. */
enum { NVC_ROUTE_SIGMOID = 0, NVC_ROUTE_SOFTMAX = 1 };
int nvc_moe_route_logits_ex(nvc_ctx* ctx, const float* z, int ldz, const float* correction, int E, int top, float scale, int gate_col,
                            int score, int normalize, int32_t* topk_idx, float* topk_w, float* gate, int N, void* stream);
/* nvc_moe_sort_padded for a router whose experts from E_real on have no product (identity experts): their tiles get
 * tile_group -1. */
int nvc_moe_sort_padded_ex(nvc_ctx* ctx, const int32_t* topk_idx, int N, int top, int E, int E_real, int align, int32_t* offsets,
                           int32_t* src_rows, int32_t* pos, int32_t* tile_group, int tiles_cap, void* stream);
/* nvc_moe_combine where the experts from E_real on are identity experts: a pair (n, t) with topk_idx[n, t] >= E_real contributes
 * topk_w[n, t] * x[n, :H] instead of a row of y. */
int nvc_moe_combine_identity(nvc_ctx* ctx, const void* y, int y_dtype, int ldy, const int32_t* pos, const float* topk_w,
                             const int32_t* topk_idx, int top, int E_real, const void* x, int x_dtype, int ldx, float* out, int ldo,
                             int N, int H, void* stream);
/* Gated delta rule, the part between the fused projection and the recurrence, over the new tokens of every sequence:
 *   q, k, v channels: causal convolution over time per channel (conv_w [taps, C], tap-major, last row = the current token; the taps - 1
 *   inputs in front of a portion come from conv_state [slots, taps - 1, C], zeros when the portion starts at position 0), silu;
 *   q and k heads: x / sqrt(sum(x^2) + unit_eps), q times q_scale;   beta = sigmoid(in[b_off + h]);
 *   decay = exp(-exp(A_log[h]) * softplus(in[a_off + h] + dt_bias[h])).
 * Channel order of conv_w and conv_state: q (kv_heads * dim), k (kv_heads * dim), v (heads * vdim).  Outputs are fp32 rows;
 * gb_out [N, 2 * heads] = (log decay, beta) per head.  The conv state is NOT advanced here (nvc_delta_rule_scan does it). */
typedef struct nvc_delta_prep {
  const float* in; int ldi;
  int q_off, k_off, v_off, b_off, a_off;
  int heads, kv_heads, dim, vdim, taps;
  const float* conv_w;
  float* conv_state;
  const int32_t* state_slots; const int32_t* cu_seqlens; const int32_t* positions;
  const float* A_log; const float* dt_bias;
  float unit_eps, q_scale;
  float* q_out; float* k_out; float* v_out; int ldq, ldk, ldv;
  float* gb_out;
  int B;
} nvc_delta_prep;
int nvc_delta_prep_run(nvc_ctx* ctx, const nvc_delta_prep* p, int N, int max_qlen, void* stream);   /* max_qlen: the longest portion (a bound will do) */
/* The recurrence, per (sequence, head) with state S [dim, vdim] fp32 in state [slots, heads, dim, vdim]:
 *   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q        (head h reads q / k head h / (heads / kv_heads))
 * token by token over rows cu_seqlens[b] .. cu_seqlens[b + 1] (row b when cu_seqlens == NULL); a sequence starts from zeros when
 * positions[first row] == 0; portions of 8 tokens and more (max_qlen) run 32 tokens at a time (the same sums regrouped, fp32 FMA).
 * Also advances the convolution state of nvc_delta_prep_run (p->in still holds the step's rows). */
int nvc_delta_rule_scan(nvc_ctx* ctx, const nvc_delta_prep* p, float* o, int ldo, float* state, int max_qlen, void* stream);

/* ---- mechanisms of the models with chunked capped attention beside a selective state space layer, lightning attention, a looped
 * block with an input projection and input-weighted experts (Batatar) ---- */
/* Residual accumulation with up to two branch outputs, each plain or RMS-normed with a weight first, and the norm in front of the
 * next sublayer, in one pass over the row (all sums fp32):
 *   f(y, w) = y (w == NULL) or y / sqrt(mean(y^2) + eps) * w;
 *   s = res_in[r] + bias + c0 f(y0[r], w0) + c1 f(y1[r], w1)      (res_in, bias [H], y0, y1 optional);  res_out[r] = s (optional);
 *   out[i, :H] = s / sqrt(mean(s^2) + eps) * w  (w != NULL)  or  s  (w == NULL, out != NULL: the sum in the storage format).
 * rows as in nvc_rms_norm_pair (gathers; res_out must be NULL). */
int nvc_rms_norm_blend(nvc_ctx* ctx, const float* res_in, const float* bias, const float* y0, const float* w0, float c0, const float* y1,
                       const float* w1, float c1, float* res_out, int ld, const float* w, void* out, int out_dtype, int ldo, float eps,
                       const int32_t* rows, int N, int H, void* stream);
/* Output stage of a mixer whose norm spans groups of columns: per row, `groups` equal parts of gsize numbers;
 *   gate_first != 0:  y = o * act(gate);  out = y / sqrt(mean_group(y^2) + eps) * weight
 *   gate_first == 0:  out = o / sqrt(mean_group(o^2) + eps) * weight * act(gate)
 * weight: fp32 [groups * gsize] (NULL: none); gate fp32 [N, ldg] (NULL: none); act: NVC_GATE_SIGMOID or NVC_GATE_SILU. */
int nvc_group_norm_gate(nvc_ctx* ctx, const float* o, int ldo, const float* gate, int ldg, const float* weight, void* out, int ldout,
                        int out_dtype, int groups, int gsize, int gate_first, float eps, int act, int N, void* stream);
/* Linear recurrence with a decaying matrix state per (sequence, head), S [dim, vdim] fp32 in state [slots, heads, dim, vdim]:
 *   S_t = d_t S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t + skip_w[h] skip_t
 * d_t = decay[h] (a constant per head) or exp(log_decay[t, h]) (per token and head, log_decay <= 0); head h reads q / k head
 * h / (heads / qk_heads); skip optional.  Rows, slots, start from zeros and max_qlen as in nvc_retention_scan (which is this with
 * decay, qk_heads = heads and no skip). */
typedef struct nvc_decay_scan_args {
  const float* q; const float* k; const float* v; int ldq, ldk, ldv;
  float* o; int ldo;
  float* state; const int32_t* state_slots; const int32_t* cu_seqlens; const int32_t* positions;
  const float* decay;
  const float* log_decay; int ldl;
  const float* skip; const float* skip_w; int lds;
  int heads, qk_heads, dim, vdim;
} nvc_decay_scan_args;
int nvc_decay_scan(nvc_ctx* ctx, const nvc_decay_scan_args* p, int B, int max_qlen, void* stream);
/* Selective state space layer, the part between the fused projection and the recurrence, over the new tokens of every sequence.
 * A projection row holds the convolution channels [x: heads * vdim | B: groups * state | C: groups * state] from column xbc_off and
 * one step size per head from column dt_off.  Channels: causal convolution over time (conv_w [taps, C] tap-major, last row = the
 * current token; bias conv_b; the taps - 1 inputs in front of a portion come from conv_state [slots, taps - 1, C], zeros when the
 * portion starts at position 0), silu.  dt = softplus(in[dt_off + h] + dt_bias[h]).  Outputs (fp32 rows): x, v = dt x, B, C and
 * log_decay[n, h] = -exp(A_log[h]) dt.  nvc_ssd_conv_advance then moves every sequence's convolution state past the step's rows. */
typedef struct nvc_ssd_prep {
  const float* in; int ldi;
  int xbc_off, dt_off;
  int heads, vdim, groups, state, taps;
  const float* conv_w; const float* conv_b;
  float* conv_state;
  const int32_t* state_slots; const int32_t* cu_seqlens; const int32_t* positions;
  const float* A_log; const float* dt_bias;
  float* x_out; float* v_out; int ldx;
  float* b_out; float* c_out; int ldbc;
  float* log_decay; int ldl;
  int B;
} nvc_ssd_prep;
int nvc_ssd_prep_run(nvc_ctx* ctx, const nvc_ssd_prep* p, int N, void* stream);
int nvc_ssd_conv_advance(nvc_ctx* ctx, const nvc_ssd_prep* p, void* stream);
/* Experts whose router weight multiplies their INPUT: out[pos[n * top + t], :H] = topk_w[n, t] * h[n, :H] in the storage format
 * (the product in fp32, rounded once); pos from nvc_moe_sort or nvc_moe_sort_padded. */
int nvc_moe_scatter_scaled(nvc_ctx* ctx, const void* h, int dtype, int ldh, const int32_t* pos, const float* topk_w, int top, void* out,
                           int ldo, int N, int H, void* stream);
/* NVC_ACT_SILU_MUL for nvc_act_mul_p: out[n, j] = silu(in[n, j]) * in[n, Fp + j]. */
enum { NVC_ACT_SILU_MUL = 5 };

/* K8. Replaces Qwen3ModelRunner::argmax (src/engine/llm_engine.rs:135-142) on device:
 * idx[b] = LAST index of the maximum of logits[b, :] (Iterator::max_by tie rule);
 * val[b] = that maximum.  idx is offset by `index_offset` (TP vocab shard). */
int nvc_argmax_last(nvc_ctx* ctx, const float* logits, int ld, int32_t* idx, float* val,
                    int B, int V, int index_offset, void* stream);

/* K8s. Replaces Qwen3ModelRunner::sample_token (src/engine/llm_engine.rs:97-133) on device.  The
 * reference draws from softmax((l - max) / max(T, 1e-6)) with an unseeded rand::rng() (:128); this is
 * the Gumbel-max form of the same categorical distribution with counter-based, reproducible noise:
 *   idx[b] = argmax_i( logits[b, i] / max(T_b, 1e-6) + g ),  g = -log(-log(u)),
 *   u = (2 * (x >> 9) + 1) * 2^-24 (exact in fp32, never 0 or 1),  x = word (gi % 4) of Philox4x32-10(key = seed,
 *   counter = (gi / 4, streams[b] lo, streams[b] hi, 0)),  gi = index_offset + i  (global vocab index),
 * ties -> last index.  val[b] = the winning perturbed score, so tensor-parallel vocab shards merge
 * like the greedy (max, idx) pairs.  temperatures: f32 [B]; streams: u64 [B] (one value per
 * (sequence, step)); V, ld, index_offset multiples of 4. */
int nvc_sample_gumbel(nvc_ctx* ctx, const float* logits, int ld, const float* temperatures,
                      const uint64_t* streams, uint64_t seed, int32_t* idx, float* val, int B, int V,
                      int index_offset, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NVC_B200_H */
