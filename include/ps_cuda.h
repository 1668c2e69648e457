/* include/ps_cuda.h — C ABI of the B200-native CUDA backend for PowerServe's decode / prefill hot path.
 *
 * This is the drop-in boundary: one shared library (libps_cuda.so), plain pointers and sizes only, no C++ or torch
 * types.  A PowerServe maintainer binds it from a `CUDABackend` class that mirrors `powerserve::ggml::GGMLBackend`
 * (/root/reference/src/backend/ggml/ggml.hpp:186-250) — see INTEGRATION.md for the stub — exactly the way the QNN
 * backend is bound today (src/backend/platform.hpp:31-33, src/executor/executor.cpp:142-165).
 *
 * Conventions
 *   - ggml dimension order everywhere: ne0 is the contiguous dim; a weight W is {K, N} = N rows of K quantised
 *     elements; activations are {dim, bs} fp32 (src/core/tensor.hpp:27-31, src/graph/graph.cpp:64-76).
 *   - every call enqueues on the context's stream and returns an int status: 0 = ok, otherwise an error whose text
 *     `ps_cuda_last_error` returns.  The C++ side converts non-zero into POWERSERVE_ABORT to keep the reference's
 *     error convention (src/core/logger.hpp:56-82).
 *   - results are BIT-IDENTICAL to the reference's x86 AVX2+FMA build.
 *   - there is NO CPU fallback: without a CUDA device every entry point fails (PS_CUDA_ERR_NO_DEVICE).
 */
#ifndef PS_CUDA_H
#define PS_CUDA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PS_CUDA_ABI_VERSION 1

/* ggml type ids as stored in GGUF (libs/ggml/include/ggml.h:386-401) */
enum ps_cuda_type { PS_TYPE_F32 = 0, PS_TYPE_Q4_0 = 2, PS_TYPE_Q8_0 = 8, PS_TYPE_Q4_K = 12, PS_TYPE_Q6_K = 14, PS_TYPE_I32 = 26, PS_TYPE_BF16 = 30 };

enum ps_cuda_status {
    PS_CUDA_OK = 0,
    PS_CUDA_ERR_NO_DEVICE = 1,
    PS_CUDA_ERR_CUDA = 2,
    PS_CUDA_ERR_INVALID = 3,
    PS_CUDA_ERR_UNSUPPORTED = 4,
    PS_CUDA_ERR_OOM = 5,
    PS_CUDA_ERR_KV_FULL = 6
};

typedef struct ps_cuda_ctx ps_cuda_ctx;

/* Mirrors ModelConfig::LLMConfig + RopeConfig (src/core/config.hpp:86-109) — the fields the hot path reads. */
typedef struct {
    int32_t dim, ffn_dim, n_layers, n_heads, n_kv_heads, head_size, vocab_size;
    int32_t n_ctx;          /* KV slots to allocate (cap of model.json's n_ctx) */
    float   norm_eps;
    int32_t rope_n_dims;    /* == head_size (asserted by NormAttention::build, norm_attention.cpp:38) */
    int32_t rope_type;      /* mode & 2 -> NEOX pairs, else adjacent pairs (ggml.c:15440) */
    float   rope_freq_base, rope_freq_scale, rope_attn_factor;
    int32_t qkv_bias;       /* Qwen2 (src/model/qwen2/qwen2_model.cpp:89) */
    int32_t max_batch;      /* largest bs a forward() will see (prefill chunk / verify width); workspace is sized once */
    int32_t tp_rank, tp_size; /* tensor-parallel position of this context (1 = single GPU) */
} ps_cuda_model_desc;

typedef struct { const void *host; int32_t type; int32_t _pad; } ps_cuda_tensor; /* host pointer into GGUF memory */

/* Same names as LayerWeights / Weight (src/model/common/weights.hpp:24-74). */
typedef struct {
    ps_cuda_tensor attn_norm, ffn_norm, attn_q, attn_k, attn_v, attn_output, ffn_gate, ffn_up, ffn_down;
    ps_cuda_tensor attn_q_bias, attn_k_bias, attn_v_bias;
} ps_cuda_layer_weights;

typedef struct {
    ps_cuda_tensor token_embd, output_norm, output; /* output.host == token_embd.host when tied (weights.hpp:67) */
    const ps_cuda_layer_weights *layers;            /* n_layers entries */
} ps_cuda_model_weights;

/* ---------------------------------------------------------------------------------------------- lifecycle
 * replaces Platform::init_ggml_backend / destroy_ggml_backend (src/backend/platform.cpp:19-25) */
int  ps_cuda_abi_version(void);
int  ps_cuda_device_count(void);
int  ps_cuda_create(ps_cuda_ctx **out, int device, const ps_cuda_model_desc *desc);
void ps_cuda_destroy(ps_cuda_ctx *ctx);
const char *ps_cuda_last_error(const ps_cuda_ctx *ctx); /* ctx may be NULL: error of a failed create */
int  ps_cuda_sync(ps_cuda_ctx *ctx);
void *ps_cuda_stream(ps_cuda_ctx *ctx);                 /* the cudaStream_t every call enqueues on */

/* ---------------------------------------------------------------------------------------------- memory
 * CUDABuffer backing for graph intermediates (replaces CPUBuffer::create_buffer, src/backend/cpu_buffer.hpp:41-51)
 * and the weight registry: graph leaves arrive as CPUBuffer views of GGUF memory (weights.hpp:45-52), so weights are
 * uploaded once and looked up by host pointer. */
int   ps_cuda_malloc(ps_cuda_ctx *ctx, size_t bytes, void **dev);
int   ps_cuda_free(ps_cuda_ctx *ctx, void *dev);
int   ps_cuda_memcpy_h2d(ps_cuda_ctx *ctx, void *dev, const void *host, size_t bytes);
int   ps_cuda_memcpy_d2h(ps_cuda_ctx *ctx, void *host, const void *dev, size_t bytes);  /* synchronises */
int   ps_cuda_register_weight(ps_cuda_ctx *ctx, const void *host, int type, int64_t ne0, int64_t ne1, void **dev);
void *ps_cuda_lookup_weight(ps_cuda_ctx *ctx, const void *host);
int   ps_cuda_unregister_weight(ps_cuda_ctx *ctx, const void *host); /* frees the device copy (model unload) */

/* ---------------------------------------------------------------------------------------------- operator table
 * One entry per GGMLBackend method on the hot path (ggml.hpp:216-244); all pointers are DEVICE pointers except
 * `tokens` / `pos`, which are host arrays like the reference's std::vector<int> arguments. */
int ps_cuda_get_embedding(ps_cuda_ctx *ctx, float *dst, const void *w, int wtype, int64_t dim, const int32_t *tokens, int64_t bs);
int ps_cuda_rmsnorm(ps_cuda_ctx *ctx, float *dst, const float *x, const float *w, int64_t dim, int64_t bs, float eps);
int ps_cuda_matmul(ps_cuda_ctx *ctx, float *dst, const void *w, int wtype, int64_t K, int64_t N, const float *x, int64_t bs);
int ps_cuda_rope(ps_cuda_ctx *ctx, float *dst, const float *src, int64_t head_size, int64_t n_heads, int64_t bs, const int32_t *pos);
/* RoPE frequency factors (rope_freqs.weight of Llama-3.1 / 3.2 GGUFs; ggml_rope_cache_init, ggml.c:15342-15356: theta / ff).
 * The reference never passes them (ggml_wrapper.cpp:104-106), so the default - and parity - is WITHOUT;
 * factors == NULL restores that.  n must be rope_n_dims / 2.  Rebuilds the context's cos / sin table. */
int ps_cuda_set_rope_freq_factors(ps_cuda_ctx *ctx, const float *factors, int n);
int ps_cuda_add(ps_cuda_ctx *ctx, float *dst, const float *a, const float *b, int64_t n, int64_t nb); /* b row-broadcast */
int ps_cuda_silu_hadamard(ps_cuda_ctx *ctx, float *dst, const float *gate, const float *up, int64_t n);
int ps_cuda_get_mask(ps_cuda_ctx *ctx, float *mask, int64_t n_kv, int64_t bs, const int32_t *pos);
int ps_cuda_softmax_ext(ps_cuda_ctx *ctx, float *dst, const float *x, const float *mask, int64_t ne0, int64_t ne1, int64_t ne2, float scale);
/* the two fp32 attention matmuls over the reference's cache layout: K {kv_dim, n_kv} rows, V transposed
 * {n_ctx, kv_dim} (norm_attention.cpp:82-147); q is the rope output {head_size, n_heads, bs}. */
int ps_cuda_attn_scores(ps_cuda_ctx *ctx, float *kq, const float *k_cache, const float *q, int64_t head_size, int64_t n_heads,
                        int64_t n_kv_heads, int64_t n_kv, int64_t bs);
int ps_cuda_attn_pv(ps_cuda_ctx *ctx, float *out, const float *v_cache_t, const float *p, int64_t head_size, int64_t n_heads,
                    int64_t n_kv_heads, int64_t n_kv, int64_t n_ctx, int64_t bs);
/* strided fp32 copy (GGMLBackend::copy / cont -> powerserve_compute_forward_dup): 2-D, byte strides */
int ps_cuda_copy_2d(ps_cuda_ctx *ctx, void *dst, int64_t dst_stride0, int64_t dst_stride1, const void *src,
                    int64_t src_stride0, int64_t src_stride1, int64_t ne0, int64_t ne1);

/* the same for views of up to four dims whose shapes may differ (GGMLBackend::cont of a permuted view, copy into a
 * cache view; ggml_wrapper.cpp:135-161 -> powerserve_compute_forward_dup, ggml.c:9519-9558): element t of the source in
 * its row-major order lands on element t of the destination; shapes in elements, strides in bytes */
int ps_cuda_copy_4d(ps_cuda_ctx *ctx, void *dst, const int64_t dst_ne[4], const int64_t dst_nb[4], const void *src,
                    const int64_t src_ne[4], const int64_t src_nb[4]);
/* GGMLBackend::matmul with an FP32 src0 (ggml_wrapper.cpp:20-40 -> vec_dot_f32; the attention products over strided
 * cache views, norm_attention.cpp:117-147): dst {ne01, ne11, ne12} contiguous; src0 {ne00, ne01, ne02}, src1 {ne00, ne11,
 * ne12}, ne12 % ne02 == 0 (GQA broadcast, ggml.c:13365); innermost dims contiguous, nb* in bytes */
int ps_cuda_matmul_f32(ps_cuda_ctx *ctx, float *dst, const void *src0, int64_t ne00, int64_t ne01, int64_t ne02, int64_t nb01,
                       int64_t nb02, const void *src1, int64_t ne11, int64_t ne12, int64_t nb11, int64_t nb12);
/* GGMLBackend::softmax (ggml_wrapper.cpp:57-69 -> powerserve_compute_forward_soft_max, ggml.c:15060-15089): scale 1, no mask */
int ps_cuda_softmax(ps_cuda_ctx *ctx, float *dst, const float *x, int64_t ne0, int64_t n_rows);

/* ---------------------------------------------------------------------------------------------- KV cache
 * Device implementation of the position bookkeeping of KVCacheInterface (src/core/kv_cache.hpp:97-163) that
 * Platform::get/reset_kv_position (src/backend/platform.cpp:34-50) and LlamaModel::forward (:84-86,109) use. */
int     ps_cuda_kv_position(ps_cuda_ctx *ctx);
int     ps_cuda_kv_reset(ps_cuda_ctx *ctx);                    /* truncate_tokens(0) */
int     ps_cuda_kv_truncate(ps_cuda_ctx *ctx, int n_tokens);   /* truncate_tokens(n) */
int     ps_cuda_kv_rollback(ps_cuda_ctx *ctx, int n_tokens);   /* rollback_tokens(n) */
int     ps_cuda_kv_advance(ps_cuda_ctx *ctx, int n_tokens);    /* advance_tokens(n) */
/* slot operations of KVCacheInterface used by the speculative path (src/core/kv_cache.hpp:120-143, 188-231;
 * src/speculative/token_tree.cpp:195-212, 295-315): cache SLOTS are decoupled from token positions and carry a mask bit
 * (advance unmasks, rollback masks); `copy` takes a token of the LAST ps_cuda_forward_tree batch. */
int     ps_cuda_kv_copy_slot(ps_cuda_ctx *ctx, int dst_cache_index, int src_token_index);   /* copy(dst, src) */
int     ps_cuda_kv_move_slot(ps_cuda_ctx *ctx, int dst_cache_index, int src_cache_index);   /* move(dst, src) */
int     ps_cuda_kv_mask_slot(ps_cuda_ctx *ctx, int cache_index);                            /* mask(idx), idx < position */
int     ps_cuda_kv_unmask_slot(ps_cuda_ctx *ctx, int cache_index);                          /* unmask(idx) */
float  *ps_cuda_kv_k(ps_cuda_ctx *ctx, int layer);             /* device ptr, [n_ctx][kv_dim] */
float  *ps_cuda_kv_v(ps_cuda_ctx *ctx, int layer);             /* device ptr, [kv_dim][n_ctx] (transposed) */

/* ---------------------------------------------------------------------------------------------- whole-model path
 * The QNN precedent (`g.qnn_forward`, llama_model.cpp:66-77): one graph op that runs the whole forward pass inside
 * the backend.  bind uploads every weight; forward == LlamaModel::forward / Qwen2Model::forward (llama_model.cpp:
 * 52-117): tokens/pos are HOST arrays, logits_host (may be NULL when lm_head == 0) receives [bs][vocab] fp32 and the
 * call returns after the copy has landed; the KV position advances by bs. */
int ps_cuda_bind_model(ps_cuda_ctx *ctx, const ps_cuda_model_weights *w);
int ps_cuda_forward(ps_cuda_ctx *ctx, const int32_t *tokens, const int32_t *pos, int bs, int lm_head, float *logits_host);
/* The same forward as the speculative path calls it (src/speculative/spec_model.hpp:96-103, token_tree.cpp:131-133): arbitrary
 * token positions, `tree_mask` = bs x bs bytes, row i = the batch tokens token i attends to (TokenTree::attention_mask; NULL =
 * causal), attention over the unmasked cache slots below the current position; the batch's K / V rows are appended at cache
 * slots position .. position + bs - 1 and the position advances by bs (CausalLM::Batch::save_kv + advance, causal_models.cpp:
 * 353-359) - callers roll back and `copy` the accepted tokens, as TokenTree::verify does.  bs <= min(max_batch, 32).
 * lm_head = 1: logits_host receives [bs][vocab] fp32; lm_head = 2: the greedy pick is made on the device (first maximum per row,
 * llama_model.cpp:124-128 with top_k = 1) and logits_host receives bs int32 token ids instead. */
int ps_cuda_forward_tree(ps_cuda_ctx *ctx, const int32_t *tokens, const int32_t *pos, int bs, const uint8_t *tree_mask, int lm_head,
                         float *logits_host);
/* ---------------------------------------------------------------------------------------------- sessions
 * Server-side batching (app/server/server_handler.hpp:512-720): the reference serves one generation
 * per model at a time because the KV position is shared state (server_handler.hpp:224-240).  A context can hold several
 * independent KV sets over one set of weights.  Session 0 is the context's own cache.  ps_cuda_session_select makes a
 * session the target of every single-sequence call (forward / forward_tree / decode_greedy / kv_*), so prefill and KV
 * bookkeeping work per session unchanged; ps_cuda_forward_sessions advances n DISTINCT sessions by one token each in one
 * forward pass: one weight stream for the n columns, attention per column over its own cache and position.  logits_host
 * ([n][vocab], may be NULL) and greedy_ids ([n], may be NULL: arg-max on the device) are in batch order.  Each column's
 * result is bit-identical to decoding that session alone with batch 1. */
int ps_cuda_session_create(ps_cuda_ctx *ctx, int *session_id);
int ps_cuda_session_destroy(ps_cuda_ctx *ctx, int session_id);   /* not the selected one */
int ps_cuda_session_select(ps_cuda_ctx *ctx, int session_id);
int ps_cuda_session_current(ps_cuda_ctx *ctx);
int ps_cuda_session_position(ps_cuda_ctx *ctx, int session_id);  /* -1: unknown session */
int ps_cuda_forward_sessions(ps_cuda_ctx *ctx, const int32_t *session_ids, const int32_t *tokens, int n, int lm_head,
                             float *logits_host, int32_t *greedy_ids);

/* Model::decode with top_k = 1 (llama_model.cpp:119-132): forward + arg-max on the device; only the token id comes
 * back.  `n_steps` > 1 keeps feeding the produced id back in without a host round trip (ids_host gets n_steps ids). */
int ps_cuda_decode_greedy(ps_cuda_ctx *ctx, int32_t first_token, int n_steps, int32_t *ids_host);
/* device-side logits of the last forward ([bs][vocab]) for callers that sample on the GPU */
const float *ps_cuda_logits_dev(ps_cuda_ctx *ctx);
/* Device-side sampling: ps_cuda_forward / ps_cuda_forward_sessions accept logits_host == NULL with
 * lm_head = 1 - the logits stay on the device - and ps_cuda_sample_topk returns what ProbArray holds after
 * TopKSampler::apply (src/sampler/sampler.cpp:39-56, prob_array.hpp:43-49): the k <= 64 largest logits of row `row` of the
 * last forward pass, descending (equal logits by ascending token id), with their token ids.  2 k words cross PCIe instead of
 * the vocabulary's logits; the rest of the sampler chain (temperature, soft-max, top-p, stochastic pick) runs on k entries. */
int ps_cuda_sample_topk(ps_cuda_ctx *ctx, int row, int k, float *logits_out, int32_t *tokens_out);

/* ---------------------------------------------------------------------------------------------- tensor parallelism
 * One process per GPU.  A context created with desc.tp_size = N > 1 owns rows [rank * rows / N, (rank + 1) * rows / N) of
 * EVERY matrix (bind_model slices the host tensors itself) and only its own kv heads of the cache; the sharded outputs
 * of the fused decode step are exchanged with NCCL all-gathers on the context stream (4 per layer + 1 or 2 per token),
 * so every dot product keeps its full K and the results stay bit-identical to one GPU.  The host side moves the
 * 128-byte NCCL id from rank 0 to the other ranks (any transport: torch.distributed, MPI, a file). */
int ps_cuda_tp_unique_id(void *out128);                        /* rank 0: ncclGetUniqueId */
int ps_cuda_tp_init(ps_cuda_ctx *ctx, const void *id128);      /* every rank, after create, before the first forward */
/* Fused compute + all-gather over NVLink peer memory (optional, on top of tp_init): every rank exports the CUDA-IPC
 * handle of its exchange heap (64 bytes), the host gathers the N handles in rank order and every rank imports them.
 * From then on the producing kernels store their output rows straight into every rank's copy of the gathered vector
 * and publish an epoch flag; the consuming kernels wait on the flags (bounded spin; counter "tp_error").  Option
 * "tp_p2p" = 0 switches back to NCCL all-gathers (same results; tests compare the two).  The four per-layer exchanges
 * carry their flag in band (64-bit {value, epoch} peer stores, polled by the consumer: no fences); option "tp_ll" = 0
 * makes them use the fence + epoch-flag protocol as well. */
int ps_cuda_tp_export(ps_cuda_ctx *ctx, void *handle64);
int ps_cuda_tp_import(ps_cuda_ctx *ctx, const void *handles, int n);

/* ---------------------------------------------------------------------------------------------- layer-list models
 * Models that a configuration file describes layer by layer (config.json + model.safetensors, weights in bfloat16)
 * instead of the fixed llama / qwen2 stack above.  A layer is a token mixer plus an optional feed-forward.
 *   block_kind PS_BLOCK_PARALLEL: both read ONE norm's output, x <- x + (mixer(N(x)) + ff(N(x)));
 *   block_kind PS_BLOCK_SEQUENTIAL: x <- x + P1(mixer(N1(x))), then x <- x + P2(ff(N2(x))); P1 / P2 are norms of the
 *   sublayer's OUTPUT when post_norm = 1, the identity otherwise.
 * Every mechanism is a parameter set of its own, so that another design can combine them differently:
 *   attention  - grouped-query, separate query/key and value head sizes, projection biases, no rotation;
 *                qk_norm = 1: every head's q and k are divided by their root mean square (no weight, eps = norm_eps);
 *                score = q.k * score_scale [* head_temp[h]] [+ rel[bucket(i - j)][h]] [- r1[h] ln(1 + r2[h] (i - j))]
 *                [mixed over heads by head_mix]; window > 0: query i sees the keys i - window < j <= i only;
 *                soft-max with an optional sink (one more term in the denominator that carries no value: exp(0) for
 *                sink = PS_SINK_ZERO, exp(sink[h]) for PS_SINK_LEARNED);
 *                bucket(n) = n below rel_buckets / 2, then logarithmic up to rel_max_dist (last bucket beyond);
 *                v_mix: PS_VMIX_SOURCE keeps the layer's value rows of the tokens in flight, PS_VMIX_BLEND replaces
 *                v by (1 - vmix) v + vmix v_source before it is cached (same value width in both layers).
 *   latent attention - queries through a normed latent (c_q = N(W_dq h; dq_norm), q = W_uq c_q, per head qk_dim plain
 *                + rot_dim rotated dims); W_dkv h gives kv_rank latent dims (normed with dkv_norm: the latent c) and
 *                rot_dim dims of ONE rotated key part shared by all heads; per head k = W_uk c, v = W_uv c;
 *                score = (q_plain . k + q_rot . k_rot) * score_scale, causal or windowed, sink as above.  The cache
 *                holds c and the rotated key part only: the executor folds W_uk into the query and applies W_uv to
 *                the weighted sum of latents.
 *   rotation   - the first rope_dims dims of a rotated vector, pairs (i, i + rope_dims / 2), angle pos * f_i with
 *                f_i = rope_base^(-2 i / rope_dims); rope_factor > 0 adds YaRN: f_i <- f_i / factor * ramp_i +
 *                f_i (1 - ramp_i) with the ramp between the dims whose wavelength fits rope_original positions
 *                rope_fast and rope_slow times, and cos / sin scaled by 0.1 ln(factor) + 1.
 *                chunk > 0: query i sees key j <= i only when floor(i / chunk) = floor(j / chunk) (chunks counted from position 0);
 *                conv_taps > 0: a causal convolution over time on every channel of q, k and v directly after the projection
 *                (y_t = sum_j w[c][j] u_(t - taps + 1 + j), zeros before position 0); the last conv_taps - 1 projected rows are
 *                part of the sequence's state; qk_norm = PS_QKNORM_WHOLE: q (all heads at once) and k are RMS-normed as ONE
 *                vector each with the weights q_norm / k_norm.
 *   retention  - PS_MIXER_RETENTION: per head S_t = decay[h] S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, no soft-max; q and k
 *                rotated (rotation below, rope_dims of qk_dim), k times qk_dim^(-1/2); every head's o divided by its root mean
 *                square, the concatenation times silu(W_g h), then the output projection.  State: S per head, qk_dim x v_dim, fp32.
 *   mamba2     - PS_MIXER_MAMBA2: W_in h = [z | x | B | C | dt] (inner = n_heads * v_dim, B and C of ssm_groups * ssm_state);
 *                x|B|C through a causal convolution of conv_taps taps with bias and silu; dt = softplus(dt + dt_bias);
 *                S_t = exp(-exp(A_log[h]) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D[h] x_t; y silu(z) is RMS-normed in
 *                gate_norm_groups equal parts times mix_norm, then the output projection.  State: S per head, ssm_state x v_dim, fp32,
 *                and the last conv_taps - 1 inputs of the convolution.
 *   recurrent state lives where a cache set keeps an attention layer's K rows (first buffer) and V^T rows (second buffer);
 *                a sequence at position 0 starts from zero state whatever the buffers hold; ps_cuda_kv_rollback to a
 *                position other than 0 is refused for models with such layers.
 *   dense ff   - PS_MLP_DENSE: one gated feed-forward of expert_ff rows with the expert's activation below.
 *   routed ff  - n_experts gated experts, the top_k largest router scores choose; router_act 1 = sigmoid scores;
 *                route_on_input = 1: the score multiplies the expert's INPUT; route_renorm = 1: the chosen scores are
 *                divided by their sum (+ route_renorm_eps); router_act 2 = soft-max over all experts; route_groups > 1:
 *                the experts form that many equal groups of neighbours, a group is worth its best score and only the
 *                route_keep best groups can be chosen from.  Expert: g = min(Wg z, act_limit), u = clamp(Wu z, +-act_limit),
 *                y = g * sigmoid(act_alpha * g) * (u + up_shift), out = Wd y; act_kind PS_ACT_GELU_TANH: y = gelu_tanh(Wg z) * (Wu z).
 *                shared_ff > 0: one more expert of that many rows runs for every token and is added, times
 *                sigmoid(shared_sg . z) when shared_gate = 1.
 *   raw_input  - sequential blocks: the sublayers read the residual stream itself (no norm on the way in).
 *   values from keys - v_is_k = 1: there is no W_v; a position's value row is its projected key row as it leaves the projection
 *                (before any q / k norm); v_dim = qk_dim.
 *   pooled window - pool > 0 (with window > 0): beside the window's tokens a query at position i sees one key and value for every block
 *                of `pool` positions that lies wholly before its window (block b = positions b pool .. b pool + pool - 1, seen when
 *                b pool + pool - 1 <= i - window): the means of the block's cached key rows and value rows.  Tokens that have left the
 *                window and whose block is not complete yet are not seen.  Tokens and blocks share one soft-max; a block's score
 *                carries no distance term.  The cache set keeps the means behind the layer's K rows and V^T rows.
 *   linear distance bias - lin_bias = 1: score -= lin[h] * (i - j).
 *   output gate - out_gate = 1: the concatenated heads are multiplied by sigmoid(W_g h) (tensor g, [H * v_dim][dim]) before the
 *                output projection; W_g reads the mixer's input.
 *   side mixer - side_kind = PS_MIXER_MINGRU: a gated recurrence beside the attention, reading the same input: z = sigmoid(W_z h + b_z),
 *                u = W_x h + b_x, candidate c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0), S_t = (1 - z) S_(t-1) + z c element by
 *                element over side_width channels (fp32, zero at position 0), output W_so (S_t silu(W_sg h)).  The layer's mixer
 *                output is mix_scale * attention + side_scale * side (one product over the concatenated inputs).
 *   interleaved rotation - rope_interleaved = 1: the rotation pairs dims (2i, 2i + 1) instead of (i, i + rope_dims / 2).
 *   ungated ff - mlp_ungated = 1 (PS_MLP_DENSE): out = W_down act(W_up h), act the one-argument form of act_kind; PS_ACT_XIELU with the
 *                two numbers p, q of tensor act: z > 0: softplus(p) z^2 + z / 2; z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2.
 *   layer runs - the descriptor's layer list is the list of layer RUNS: share_weights = j + 1 makes a run use the weights of run j
 *                (same sizes; its own cache and state), so a group of layers can be passed through several times.  pass_embed = 1
 *                adds the embedding output (the residual stream as it was before the first run) to the stream before the run,
 *                pass_step = r + 1 adds row r of the model's pass_steps table [n_pass_steps][dim].
 *   norm       - RMS norm with eps inside the root; norm_kind = PS_NORM_LAYER: the mean is taken off first and the divisor is
 *                sqrt(variance + eps) (a weight, no bias); norm_unit_offset = 1: the stored weight is around zero (1 + w);
 *                norm_groups > 1: the vector is cut into that many equal parts, each divided by its own root mean square;
 *                norm_scalar = 1: every norm's weight is a single number for all coordinates.
 * The context made by ps_cuda_create_arch is an ordinary ps_cuda_ctx: ps_cuda_forward, ps_cuda_decode_greedy,
 * ps_cuda_sample_topk, ps_cuda_logits_dev, the ps_cuda_kv_* position calls and the ps_cuda_session_* calls work on it
 * as on a llama context (the per-layer cache rows have the layer's own widths; V is kept transposed like there).  The
 * llama-only entry points (operator table on the context's workspace, forward_tree, forward_sessions, slot operations,
 * tensor parallelism) return PS_CUDA_ERR_UNSUPPORTED.
 * compute = PS_COMPUTE_BF16: matrix products take bfloat16 operands and accumulate in fp32; the residual stream, norms,
 * attention scores / weights, routers and the cache stay fp32.  PS_COMPUTE_F32: every product in true fp32 (FMA). */
enum ps_cuda_compute { PS_COMPUTE_BF16 = 0, PS_COMPUTE_F32 = 1 };
enum ps_cuda_mixer_kind { PS_MIXER_ATTENTION = 1, PS_MIXER_LATENT = 2, PS_MIXER_RETENTION = 3, PS_MIXER_MAMBA2 = 4, PS_MIXER_MINGRU = 5 /* side mixer only */ };
enum ps_cuda_mlp_kind { PS_MLP_NONE = 0, PS_MLP_ROUTED = 1, PS_MLP_DENSE = 2 };
enum ps_cuda_block_kind { PS_BLOCK_PARALLEL = 0, PS_BLOCK_SEQUENTIAL = 1 };
enum ps_cuda_sink_kind { PS_SINK_NONE = 0, PS_SINK_ZERO = 1, PS_SINK_LEARNED = 2 };
enum ps_cuda_vmix_kind { PS_VMIX_NONE = 0, PS_VMIX_SOURCE = 1, PS_VMIX_BLEND = 2 };
enum ps_cuda_qknorm_kind { PS_QKNORM_NONE = 0, PS_QKNORM_HEAD = 1, PS_QKNORM_WHOLE = 2 };
enum ps_cuda_act_kind { PS_ACT_SWISH = 0, PS_ACT_GELU_TANH = 1, PS_ACT_XIELU = 2 };
enum ps_cuda_norm_kind { PS_NORM_RMS = 0, PS_NORM_LAYER = 1 };
enum ps_cuda_router_act { PS_ROUTER_SIGMOID = 1, PS_ROUTER_SOFTMAX = 2 };

typedef struct {
    int32_t mixer_kind;
    int32_t n_heads, n_kv_heads, qk_dim, v_dim;
    float   score_scale;
    int32_t proj_bias;                  /* q, k, v and output projections carry biases */
    int32_t head_temp;                  /* per-head score multiplier */
    int32_t rel_buckets; float rel_max_dist; /* rows of the distance-bias table (0 = none) and the distance of its last bucket */
    int32_t head_mix;                   /* [H][H] mixing of the heads' scores before the soft-max */
    int32_t sink;                       /* enum ps_cuda_sink_kind: one more term in the soft-max denominator */
    int32_t mlp_kind;
    int32_t n_experts, top_k, expert_ff;
    int32_t router_act;                 /* enum ps_cuda_router_act */
    int32_t route_on_input, route_renorm;
    float   act_limit, act_alpha, up_shift;
    int32_t block_kind;                 /* enum ps_cuda_block_kind */
    int32_t post_norm;                  /* sequential blocks: every sublayer's output is normed before the residual add */
    int32_t qk_norm;                    /* enum ps_cuda_qknorm_kind */
    int32_t window;                     /* > 0: keys further back than window - 1 positions are not seen */
    int32_t log_bias;                   /* score -= r1[h] * ln(1 + r2[h] * distance) */
    int32_t v_mix;                      /* enum ps_cuda_vmix_kind */
    int32_t q_rank, kv_rank, rot_dim;   /* latent attention */
    int32_t rope_dims, rope_original;   /* rotation: rotated dims; YaRN's original context */
    float   rope_base, rope_factor, rope_fast, rope_slow; /* rope_factor = 0: plain rotation */
    int32_t raw_input;                  /* sequential blocks: no norm on a sublayer's input */
    int32_t chunk;                      /* > 0: attention inside chunks of this many positions only */
    int32_t conv_taps;                  /* short causal convolution: on q, k, v (attention), on x|B|C (mamba2); 0 = none */
    int32_t ssm_state, ssm_groups;      /* mamba2: state size N, groups of heads that share B and C */
    int32_t gate_norm_groups;           /* mamba2: parts of the gated output that are normed separately */
    int32_t act_kind;                   /* enum ps_cuda_act_kind */
    int32_t route_groups, route_keep;   /* group-limited routing (route_groups <= 1: every expert can be chosen) */
    float   route_renorm_eps;           /* added to the sum of the chosen scores before the division */
    int32_t shared_ff, shared_gate;     /* rows of the shared expert (0 = none); 1 = its output is scaled by sigmoid(shared_sg . z) */
    int32_t v_is_k;                     /* the value rows are the projected key rows (no W_v) */
    int32_t pool;                       /* > 0: mean key / value per block of this many positions wholly before the window */
    int32_t lin_bias;                   /* score -= lin[h] * distance */
    int32_t out_gate;                   /* heads' outputs times sigmoid(W_g h) before the output projection */
    int32_t side_kind, side_width;      /* a second mixer beside the attention (0 = none, PS_MIXER_MINGRU) and its channels */
    float   mix_scale, side_scale;      /* mixer output = mix_scale * attention + side_scale * side (used when side_kind != 0) */
    int32_t rope_interleaved;           /* rotation pairs (2i, 2i + 1) */
    int32_t mlp_ungated;                /* dense feed-forward without a gate: down(act(up h)) */
    int32_t share_weights;              /* j + 1: this run uses the weights of run j */
    int32_t pass_embed, pass_step;      /* before the run: add the embedding output; add row pass_step - 1 of pass_steps */
} ps_cuda_layer_desc;

typedef struct {
    int32_t dim, vocab_size, n_layers;
    int32_t n_ctx, max_batch;
    float   norm_eps, embed_scale;
    int32_t norm_unit_offset;
    int32_t compute;                    /* enum ps_cuda_compute */
    const ps_cuda_layer_desc *layers;   /* n_layers entries */
    int32_t norm_groups;                /* 0 or 1: one group */
    int32_t norm_scalar;                /* the norms' weights are single numbers */
    int32_t norm_kind;                  /* enum ps_cuda_norm_kind: the block norms and the final norm */
    int32_t n_pass_steps;               /* rows of the pass_steps table */
} ps_cuda_arch_desc;

/* matrices [out][in] in bfloat16; vectors and the small tables in bfloat16 or fp32 */
typedef struct {
    ps_cuda_tensor norm, q, q_bias, k, k_bias, v, v_bias, o, o_bias, rel, head_mix, head_temp, router;
    const ps_cuda_tensor *gate, *up, *down; /* n_experts entries each, one for a dense feed-forward (NULL without a feed-forward) */
    /* sequential blocks: norm of the mixer's output, norm before the feed-forward, norm of its output */
    ps_cuda_tensor norm_mix_out, norm_ff, norm_ff_out;
    ps_cuda_tensor r1, r2, sink, vmix;  /* [H], [H], [H], scalar */
    ps_cuda_tensor dq, dq_norm, uq, dkv, dkv_norm, uk, uv; /* latent attention */
    ps_cuda_tensor q_norm, k_norm, q_conv, k_conv, v_conv; /* whole-projection norms [H * qk_dim], [G * qk_dim]; convolutions [channels][taps] */
    ps_cuda_tensor g, decay;            /* retention: gate projection [H * v_dim][dim]; decays [H] */
    ps_cuda_tensor w_in, conv_w, conv_b, dt_bias, a_log, d_skip, mix_norm; /* mamba2 */
    ps_cuda_tensor shared_gate, shared_up, shared_down, shared_sg; /* shared expert */
    ps_cuda_tensor lin, act;            /* linear distance-bias slopes [H]; the activation's numbers [2] */
    ps_cuda_tensor side_z, side_z_bias, side_x, side_x_bias, side_g, side_o; /* side mixer: [W][dim], [W], [W][dim], [W], [W][dim], [dim][W] */
} ps_cuda_arch_layer_weights;

typedef struct {
    ps_cuda_tensor embed, final_norm, head;
    const ps_cuda_arch_layer_weights *layers; /* one entry per run; the entries of runs that share another run's weights are not read */
    ps_cuda_tensor pass_steps;          /* [n_pass_steps][dim] */
} ps_cuda_arch_weights;

int ps_cuda_create_arch(ps_cuda_ctx **out, int device, const ps_cuda_arch_desc *desc);
int ps_cuda_bind_arch(ps_cuda_ctx *ctx, const ps_cuda_arch_weights *w);
/* debug / bring-up: the residual stream after layer `layer` of the last forward ([bs][dim] fp32; option "arch_taps" = 1
 * makes forward keep them) */
int ps_cuda_arch_tap(ps_cuda_ctx *ctx, int layer, float *host, int bs);

/* execution switches (0/1): "graph" = replay the decode step as a captured CUDA graph, "fused" = fused decode
 * kernels instead of one kernel per table op, "pdl" = programmatic dependent launch between the fused kernels.  All
 * produce bit-identical results; they exist so tests can prove it.  "ktime" = 1 runs the fused step un-graphed with
 * CUDA events around every mat-vec launch (bench.py's roofline leg); "trace" = 1 records a per-kernel device timeline;
 * "cta_trace" = k (with "trace") adds a per-CTA stream trace of one mat-vec launch site (1 Wdown, 2 gate|up, 3 QKV, 4 Wo,
 * 5 lm_head; trace slots 256..); "rw_kb" = n caps the blocks per TMA ring stage of the mat-vec (tuning; default 16).
 * Kernel choice for batches (prefill chunks, verify batches; every choice computes the same bits): "attn_tile" = 0 runs
 * the first-generation batch attention kernels instead of the register-tiled ones; "tc_min" = n is the narrowest batch that takes
 * the tcgen05 GEMM (default 6; narrower ones walk with the multi-column row-walker); "scores_batch_min" (default 2) and
 * "pv_batch_min" (default 3) are the narrowest batches for the query-blocked scores / P.V kernels. */
int ps_cuda_set_option(ps_cuda_ctx *ctx, const char *name, int value);
/* counters: "kernel_launches" (kernels enqueued since create), "graph_replays", "h2d_bytes", "d2h_bytes",
 * "last_device_ns" (CUDA-event time, on the context stream, of the last forward / decode_greedy call),
 * "matvec_kernel_ns" / "matvec_kernel_launches" (option "ktime": summed event time / count of the mat-vec launches of
 * the last decode_greedy call), "tp_allgathers" (NCCL all-gathers enqueued since create) */
int64_t ps_cuda_get_counter(ps_cuda_ctx *ctx, const char *name);

/* debug: with option "trace" = 1 every kernel of the fused decode step records globaltimer stamps into its slot
 * (8 x int64 per launch: first start, last end, first dependency-resolved, slowest prologue, 3 prologue probes, spare;
 * at most 512 launches); read the first n_launches slots back here.  Not used in production. */
int ps_cuda_read_trace(ps_cuda_ctx *ctx, long long *host, int n_launches);

/* host-side restatement of glibc expf used by the device code; exported so CPU-only tests can pin it against libm */
float ps_cuda_host_expf_ref(float x);
float ps_cuda_host_v_expf(float x);
/* host-side distance bucket of a layer-list attention's bias table (rows, rel_max_dist): the table the device reads is built
 * from this function, so CPU-only tests can pin it */
int ps_cuda_host_rel_bucket(int distance, int rows, float max_dist);
/* host-side rotation frequencies of a layer-list attention (freq[dims / 2]; factor > 0: YaRN); returns the factor on
 * cos / sin.  The table the device reads holds the same values before their rounding to float32, so CPU-only tests can pin it */
float ps_cuda_host_rope_freq(int dims, float base, float factor, int original, float fast, float slow, float *freq);

#ifdef __cplusplus
}
#endif
#endif /* PS_CUDA_H */
