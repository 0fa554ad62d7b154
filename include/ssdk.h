/*
 * ssdk.h — C-ABI of libssdk.so, the sm_100a speculative-decoding hot path.
 *
 * The reference (tanishqkumar/ssd) has no native code and no FFI: its hot path is
 * Python/torch calling cuBLAS, torch.compile(Triton), FlashAttention-3, FlashInfer
 * and NCCL.  Every entry point below therefore replaces a *Python* interface of the
 * reference; the file:line each one replaces is cited on the declaration
 * (paths relative to the reference root).  INTEGRATION.md shows the ctypes stub a
 * reference maintainer would add to bind them.
 *
 * Conventions
 *  - plain C types only: raw device/host pointers, sizes, `void* stream`
 *    (a cudaStream_t); no torch types.
 *  - every function returns 0 on success, <0 on error; ssdk_last_error() returns a
 *    thread-local, NUL-terminated description of the last failure.
 *  - the caller (PyTorch on the host side) owns all device memory: weights,
 *    KV cache, workspace, logits.  The library owns only its plan objects, CUDA
 *    graphs, TMA descriptors and a few KB of pinned staging for step I/O.
 *  - not thread-safe per handle; one handle per rank process; all work is enqueued
 *    on the caller's stream.
 *  - bf16 storage everywhere unless stated; fp32 accumulation and statistics.
 */
#ifndef SSDK_H_
#define SSDK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSDK_ABI_VERSION 1

typedef struct ssdk_engine* ssdk_handle;

/* which model of the pair an argument refers to */
enum { SSDK_TARGET = 0, SSDK_DRAFT = 1 };

/* weight kinds for ssdk_bind_weight (shapes are per tensor-parallel rank) */
enum {
  SSDK_W_EMBED      = 0,  /* [vocab/tp, hidden]            layers/embed_head.py:33-47 */
  SSDK_W_LM_HEAD    = 1,  /* [vocab/tp, hidden]            layers/embed_head.py:78-116 */
  SSDK_W_FINAL_NORM = 2,  /* [hidden]                      models/llama3.py:246,266 */
  SSDK_W_INPUT_NORM = 3,  /* [hidden]           per layer  models/llama3.py:182 */
  SSDK_W_QKV        = 4,  /* [(H+2KV)*hd/tp, hidden]       layers/linear.py:125-162 (q|k|v packed) */
  SSDK_W_Q_NORM     = 5,  /* [hd]  (Qwen3 only)            models/qwen3.py:87-88 */
  SSDK_W_K_NORM     = 6,  /* [hd]  (Qwen3 only) */
  SSDK_W_O          = 7,  /* [hidden, H*hd/tp]             layers/linear.py:165-199 */
  SSDK_W_POST_NORM  = 8,  /* [hidden]                      models/llama3.py:183 */
  SSDK_W_GATE_UP    = 9,  /* [2*ffn/tp, hidden] gate|up    layers/linear.py:101-122 */
  SSDK_W_DOWN       = 10, /* [hidden, ffn/tp]              layers/linear.py:165-199 */
  SSDK_W_ROPE_TABLE = 11, /* fp32 [max_pos, hd] cos|sin    layers/rotary_embedding.py:30-37 */
  SSDK_W_KIND_COUNT = 12
};

/* Mirrors the HF config fields the reference reads (models/llama3.py:157-183,
 * models/qwen3.py:163-193) after tensor-parallel division. */
typedef struct ssdk_model_cfg {
  int32_t hidden;        /* d */
  int32_t layers;        /* L */
  int32_t heads;         /* total query heads H */
  int32_t kv_heads;      /* total KV heads */
  int32_t head_dim;      /* hd */
  int32_t ffn;           /* total intermediate size */
  int32_t vocab;         /* total vocab V */
  int32_t qk_norm;       /* 1 = per-head RMSNorm on q,k before RoPE (Qwen3) */
  float   rms_eps;
  int32_t max_pos;       /* rows in the RoPE table that will be bound */
  int32_t tp_size;       /* 1 for the draft (replica on one GPU) */
  int32_t tp_rank;
} ssdk_model_cfg;

typedef struct ssdk_runtime_cfg {
  int32_t spec_k;             /* K (speculate_k); 0 = autoregressive only */
  int32_t max_batch;          /* max sequences per step (b); max_batch*(K+1) <= 64 */
  int32_t block_size;         /* KV page size (kvcache_block_size, 256 in bench.py:40) */
  int32_t max_blocks_per_seq; /* ceil(max_model_len / block_size) */
  int32_t use_graph;          /* 1 = capture the spec step into one CUDA graph */
  int32_t use_pdl;            /* 1 = programmatic dependent launch between kernels */
  int32_t jit_speculate;      /* verify(): ratio acceptance on every temp>0 row (utils/verify.py:59-62) */
  int32_t reserved;
} ssdk_runtime_cfg;

/* ---- lifetime ------------------------------------------------------------- */
int  ssdk_abi_version(void);
const char* ssdk_last_error(void);

/* Replaces ModelRunner.__init__ / setup_and_warmup_model_and_cudagraphs
 * (engine/model_runner.py:39-157, 186-260) for both models of the pair.
 * `draft` may be NULL (autoregressive engine). */
int ssdk_create(const ssdk_model_cfg* target, const ssdk_model_cfg* draft,
                const ssdk_runtime_cfg* rt, ssdk_handle* out);
int ssdk_destroy(ssdk_handle h);

/* Replaces utils/loader.py:186-218 + the per-parameter weight_loader callbacks:
 * the host side shards/packs exactly as the reference does and hands over the
 * resulting device tensor.  `layer` is ignored for non-per-layer kinds. */
int ssdk_bind_weight(ssdk_handle h, int which, int kind, int layer,
                     const void* dev_ptr, int64_t rows, int64_t cols);

/* Replaces ModelRunner.allocate_kv_cache (engine/model_runner.py:446-503):
 * one tensor [2, L, num_blocks, block_size, kv_heads/tp, hd] (bf16);
 * k = base, v = base + L*num_blocks*block_size*kv_heads/tp*hd elements. */
int ssdk_bind_kv_cache(ssdk_handle h, int which, void* kv_base, int64_t num_blocks);

/* Scratch owned by the caller (activations, split-K partials, attention partials,
 * logits_q/logits_p, token buffers). */
int64_t ssdk_workspace_bytes(ssdk_handle h);
int ssdk_bind_workspace(ssdk_handle h, void* dev_ptr, int64_t bytes);

/* Optional tensor-parallel plumbing (target only): a ncclComm_t created by the
 * host side over the TP ranks (replaces dist.new_group, engine/model_runner.py:100-107),
 * and the per-rank peer pointers of a symmetric buffer for the fused
 * GEMM + one-shot all-reduce (replaces dist.all_reduce, layers/linear.py:195-199). */
int ssdk_set_nccl_comm(ssdk_handle h, void* nccl_comm);
int64_t ssdk_symm_bytes(ssdk_handle h);
int ssdk_bind_symm(ssdk_handle h, void* const* peer_ptrs, int n_peers);

/* Finalise: builds TMA descriptors for every bound weight and (if use_graph)
 * captures the step graphs (replaces capture_cudagraph / capture_verify_cudagraph,
 * engine/helpers/cudagraph_helpers.py:440-633). */
int ssdk_finalize(ssdk_handle h, void* stream);

/* ---- the hot path ---------------------------------------------------------- */

/* One synchronous speculative-decoding step for `batch` sequences:
 *   K+1 draft forwards (speculator_sync.py:25-69) -> one (K+1)-token target
 *   forward (verifier.py:54-106) -> accept/reject + recovery (utils/verify.py:5-181),
 * enqueued as ONE call with no host control flow per token.
 *  in : ctx_len[b]      tokens already in both KV caches (= seq.num_cached_tokens,
 *                       engine/step.py:101) — the recovery token sits at this position
 *       recovery[b]     seq.recovery_token_id (speculator_sync.py:38-45)
 *       block_tables_*  [batch, max_blocks_per_seq] int32, -1 padded
 *                       (helpers/runner_helpers.py:110-121), covering ctx_len+K+1 slots
 *       temp_t/temp_q   per-sequence temperatures (verifier.py:83-90)
 *       seed, step_id   Philox key / counter for temp>0 (replaces torch's global RNG)
 *  out: out_tokens[b*(K+1) + j]  = [recovery, draft_1..draft_K]   (speculations)
 *       out_n_accept[b]          = number of accepted draft tokens (0..K)
 *       out_recovery[b]          = next recovery token
 * Host pointers; the call blocks until the results are on the host. */
int ssdk_spec_step(ssdk_handle h, int batch,
                   const int32_t* ctx_len, const int64_t* recovery,
                   const int32_t* block_tables_target, const int32_t* block_tables_draft,
                   const float* temp_t, const float* temp_q,
                   uint64_t seed, uint64_t step_id,
                   int64_t* out_tokens, int32_t* out_n_accept, int64_t* out_recovery,
                   void* stream);

/* Device-resident variant for measurement: same work, inputs already staged on the
 * device by a previous ssdk_spec_step_stage(); nothing crosses PCIe. */
int ssdk_spec_step_stage(ssdk_handle h, int batch,
                         const int32_t* ctx_len, const int64_t* recovery,
                         const int32_t* block_tables_target, const int32_t* block_tables_draft,
                         const float* temp_t, const float* temp_q,
                         uint64_t seed, uint64_t step_id, void* stream);
int ssdk_spec_step_resident(ssdk_handle h, int batch, void* stream);
int ssdk_spec_step_fetch(ssdk_handle h, int batch, int64_t* out_tokens,
                         int32_t* out_n_accept, int64_t* out_recovery, void* stream);
/* Resident mode: copy the tokens sequence `seq` has emitted since ssdk_spec_step_stage (each step's recovery token +
 * accepted draft tokens, i.e. what Scheduler.postprocess_speculate appends, engine/scheduler.py:285-327) into
 * out_tokens[0 .. cap).  Returns the number of tokens copied (>= 0) or < 0 on error.  The device keeps at most
 * 16384 tokens per sequence. */
int ssdk_spec_step_log(ssdk_handle h, int seq, int64_t* out_tokens, int cap, void* stream);

/* Generic multi-token forward + sample of the last position of every sequence.
 * Replaces ModelRunner.run for prefill chunks (q_len<=64 per call, causal over the
 * paged cache; engine/model_runner.py:634-680 with is_prefill) and for
 * single-token autoregressive decode (q_len=1; engine/step.py:36-47).
 *   ids[b*q_len + j] tokens, written to positions ctx_len[b]+j.
 *   want_sample: 1 = run lm_head on the last row of each sequence and sample with
 *   temps[b] (layers/sampler.py:14-36) into out_tokens[b].
 * Blocks until out_tokens is on the host when want_sample != 0. */
int ssdk_forward_tokens(ssdk_handle h, int which, int batch, int q_len,
                        const int64_t* ids, const int32_t* ctx_len,
                        const int32_t* block_tables, int want_sample,
                        const float* temps, uint64_t seed, uint64_t step_id,
                        int64_t* out_tokens, void* stream);

/* Debug/parity taps: device pointers to the logits of the last spec step
 * (bf16 [batch, K+1, V] and [batch, K, V]) and of the last ssdk_forward_tokens
 * (bf16 [batch, V]).  Valid until the next call. */
const void* ssdk_logits_p(ssdk_handle h);
const void* ssdk_logits_q(ssdk_handle h);
const void* ssdk_logits_last(ssdk_handle h);
/* Debug timeline: CTA 0 of every kernel appends (kernel id, %globaltimer ns) to dev_buf (uint64 [cap][2]) right
 * after its grid dependency resolves; replaces the reference's SSD_PROFILE perf_counter prints (engine/step.py:92-161).
 * dev_buf = NULL turns tracing off. */
int ssdk_debug_trace(void* dev_buf, int cap);
/* number of kernels this library launched (or replayed inside graphs) so far */
int64_t ssdk_launch_count(ssdk_handle h);

/* ---- stand-alone ops (parity tests call these through the same C-ABI) ------ */

/* y[M,N] = x[M,K] · w[N,K]^T  (bf16 in, fp32 accumulate in TMEM, bf16 out),
 * M <= 64: weight-streaming tcgen05 GEMM with TMA-fed 128B-swizzled smem tiles.
 * Replaces F.linear at layers/linear.py:98,196 and embed_head.py:95,111.
 * split_k = 0 lets the library choose; `partials` (fp32 [split_k, M, N]) is only
 * needed when split_k != 1.  When split_k > 1 the result is left in `partials`
 * AND reduced+rounded into y. */
int ssdk_gemm_small_m(const void* x, const void* w, void* y, float* partials,
                      int M, int N, int K, int ldy, int split_k, void* stream);

/* h[M,ffn] = silu(x·Wg^T) * (x·Wu^T) with gate|up packed [2*ffn, K]
 * (layers/linear.py:101-122 + layers/activation.py:11-14), fused epilogue. */
int ssdk_gemm_gate_up_silu(const void* x, const void* w_gate_up, void* h,
                           int M, int ffn, int K, void* stream);

/* RMSDNorm (layers/layernorm.py:53-98), compiled single-rounding semantics:
 * r = x (+ residual); residual_out = bf16(r); y = bf16(r * rsqrt(mean r^2 + eps) * w).
 * residual_in may be NULL (first layer: y = norm(x), residual_out = x). */
int ssdk_rmsnorm(const void* x, const void* residual_in, const void* w, float eps,
                 void* y, void* residual_out, int M, int d, void* stream);

/* Optional per-head RMSNorm (RMSHeadNorm, layers/layernorm.py:5-50) + NeoX RoPE
 * (layers/rotary_embedding.py:6-60) on q,k, then KV-cache scatter
 * (store_kvcache, layers/attention.py:10-41).  qkv [M, (H+2KV)*hd] packed;
 * positions int64 [M]; slot_mapping int32 [M] (-1 = skip);
 * q_out [M, H*hd]; caches viewed as [num_slots, KV*hd]. */
int ssdk_rope_store_kv(const void* qkv, const int64_t* positions, const int32_t* slot_mapping,
                       const float* rope_table, const void* q_norm_w, const void* k_norm_w,
                       float norm_eps, void* q_out, void* k_cache, void* v_cache,
                       int M, int heads, int kv_heads, int head_dim, void* stream);

/* silu(x[:, :ffn]) * x[:, ffn:]  (layers/activation.py:11-14). */
int ssdk_silu_mul(const void* gate_up, void* out, int M, int ffn, void* stream);

/* Paged attention for decode (q_len=1) and verify/prefill-chunk (q_len>1):
 * replaces flash_attn_with_kvcache at layers/attention.py:107-111,128-131.
 * q [batch*q_len, H, hd]; caches [num_blocks, block_size, KV, hd];
 * context_lens[b] INCLUDES the q_len new tokens; causal, bottom-right aligned.
 * `scratch` fp32, at least ssdk_paged_attn_scratch_bytes(...) bytes. */
int64_t ssdk_paged_attn_scratch_bytes(int batch, int q_len, int heads, int head_dim, int max_ctx);
int ssdk_paged_attn(const void* q, const void* k_cache, const void* v_cache,
                    const int32_t* block_tables, const int32_t* context_lens,
                    void* out, void* scratch,
                    int batch, int q_len, int heads, int kv_heads, int head_dim,
                    int block_size, int max_blocks_per_seq, float scale, void* stream);

/* Sampler.forward (layers/sampler.py:14-36): greedy where temp==0, else
 * argmax(softmax(l/T) / Exp(1)) with Philox(seed, step_id) exponentials.
 * logits bf16 [B, V] with row stride ld (elements); out int64 [B]. */
int ssdk_sample(const void* logits, int64_t ld, const float* temps, int B, int V,
                uint64_t seed, uint64_t step_id, int64_t* out_tokens, void* stream);

/* verify() (utils/verify.py:5-181), one fused kernel.
 * logits_p bf16 [B,K+1,V], logits_q bf16 [B,K,V], speculations int64 [B,K+1],
 * temps_* fp32 [B].  ratio_rows semantics follow jit_speculate / cache_hits
 * (cache_hits may be NULL).  Outputs on the device: n_accept int32 [B],
 * recovery int64 [B].  `scratch` >= ssdk_verify_scratch_bytes(B,K) bytes. */
int64_t ssdk_verify_scratch_bytes(int B, int K);
int ssdk_verify(const void* logits_p, const void* logits_q, const int64_t* speculations,
                const float* temps_t, const float* temps_q, const int32_t* cache_hits,
                int jit_speculate, int B, int K, int V, uint64_t seed, uint64_t step_id,
                int32_t* n_accept, int64_t* recovery, void* scratch, void* stream);


/* ---- layered ("hybrid") models ---------------------------------------------------
 * A second model family beside the dense Llama / Qwen3 decoders above: a program of layers, each one token mixer
 * (a recurrent layer, latent attention, or grouped-query attention beside a delta rule) and an optional feed-forward.
 * Block kinds (SSDK_BLOCK_*): mixer and mixture of experts read the SAME normed input and join the residual
 * stream through per-channel layer scales (parallel pre-norm); each sublayer reads the residual stream itself and
 * its OUTPUT is normed before it is added (serial post-norm); or mixer and feed-forward read the same residual row
 * through a norm weight of their own and are added unscaled (parallel, two norms); or both read one plain norm's rows, each
 * through a short input convolution of its own, and are gated per channel before they are added (parallel, one norm).  The reference has no such model; these entry
 * points follow the conventions of the ones above (caller-owned device memory, int return codes).
 * Storage type T of weights / activations / latent cache: bf16 (fp32 accumulation; residual stream, norms, routers,
 * attention scores, gates and recurrent state in fp32) or fp32 throughout (no TF32). */
enum { SSDK_DT_F32 = 0, SSDK_DT_BF16 = 1 };
enum { SSDK_MIX_WKV = 0, SSDK_MIX_MLSTM = 1, SSDK_MIX_LATENT_ATTN = 2,
       SSDK_MIX_RGLRU = 3,        /* gated diagonal linear recurrence behind a short convolution, times a gelu branch */
       SSDK_MIX_SELECTIVE = 4,    /* selective scan (input-dependent step, B, C) behind a short convolution, silu gate */
       SSDK_MIX_ATTN_DELTA = 5,   /* grouped-query sink attention and a gated delta rule side by side on the same input */
       SSDK_MIX_ATTENTION = 6 };  /* grouped-query attention alone: biased q | k | v projections behind a short convolution,
                                   * rotate-half rotation of the first rot_dims entries, optional sliding window, learned sink */
enum { SSDK_MLP_NONE = 0, SSDK_MLP_MOE = 1, SSDK_MLP_GLU = 2, /* dense: down(gelu_tanh(gate h) * (up h)) */
       SSDK_MLP_FFN = 3 };        /* dense, not gated: down(act(up h + b_up)) + b_down, act = ff_act */
/* activations of the feed-forward kernels; CLAMPED is the limited GLU g sigmoid(1.702 g) (u + 1) */
enum { SSDK_ACT_CLAMPED = 0, SSDK_ACT_SILU = 1, SSDK_ACT_GELU_TANH = 2, SSDK_ACT_RELU2 = 3, /* relu(z)^2 */
       SSDK_ACT_POLYNORM = 4 };   /* k1 u1 + k2 u2 + k3 u3 + k0 with u_p = z^p / rms(z^p) over the row; SSDK_HT_FFN_ACT holds k1, k2, k3, k0 */
/* how a layer joins the residual stream */
enum { SSDK_BLOCK_PARALLEL_PRENORM = 0,  /* x += ls1 * mixer(h) + ls2 * ff(h), h = norm(x) */
       SSDK_BLOCK_SERIAL_POSTNORM = 1,   /* x += m * norm1(mixer(x)); x += m * norm2(ff(x)): the sublayers read x itself */
       SSDK_BLOCK_PARALLEL_TWO_NORMS = 2, /* x += mixer(norm1(x)) + ff(norm2(x)): one statistic, two weights, no layer scales */
       SSDK_BLOCK_PARALLEL_ONE_NORM = 3 }; /* h = norm(x); x += g1 * mixer(h + conv1(h)) + g2 * ff(h + conv2(h)): plain norm weight; the
                                            * input convolutions (canon_taps > 0) and the gates g = sigmoid(W_g h + b) (gated_residual) are optional */

/* tensors of a hybrid model (ssdk_hyb_bind); [out, in] row-major, storage type T */
enum {
  SSDK_HT_EMBED = 0,     /* [vocab, width]                       layer = -1 */
  SSDK_HT_HEAD,          /* [vocab, width] */
  SSDK_HT_FINAL_NORM,    /* [width] unit-offset weight */
  SSDK_HT_NORM,          /* [width] unit-offset weight of the block's single norm */
  SSDK_HT_LS_MIX,        /* [width] layer scale of the mixer branch */
  SSDK_HT_LS_MLP,        /* [width] layer scale of the feed-forward branch */
  /* wkv */
  SSDK_HT_WKV_MU,        /* [5, width] token-shift coefficients, order r k v g w */
  SSDK_HT_WKV_R, SSDK_HT_WKV_K, SSDK_HT_WKV_V, SSDK_HT_WKV_G,   /* [H*D, width] */
  SSDK_HT_WKV_W1,        /* [decay_rank, width] */
  SSDK_HT_WKV_W2,        /* [H*D, decay_rank] */
  SSDK_HT_WKV_W0,        /* [H*D] */
  SSDK_HT_WKV_U,         /* [H, D] */
  /* mlstm */
  SSDK_HT_MLSTM_IN,      /* [2 H D + 2 H V + 2 H, width]: q | k | v | g | i | f rows packed by the loader */
  SSDK_HT_MLSTM_IB, SSDK_HT_MLSTM_FB,   /* [H] */
  /* latent attention */
  SSDK_HT_LAT_DOWN,      /* [q_rank + kv_rank + rot_dim, width]: dq | dkv rows packed by the loader */
  SSDK_HT_LAT_QNORM,     /* [q_rank] */
  SSDK_HT_LAT_KVNORM,    /* [kv_rank] */
  SSDK_HT_LAT_UQ,        /* [H (D + R), q_rank] */
  SSDK_HT_LAT_UKT,       /* [H, kv_rank, D]: per head W_uk^T (transposed by the loader) */
  SSDK_HT_LAT_UV,        /* [H V, kv_rank] */
  SSDK_HT_LAT_SINK,      /* [H] */
  /* every mixer */
  SSDK_HT_MIX_NORM,      /* [H V] channel weight after the per-head unit RMS (wkv, mlstm) */
  SSDK_HT_MIX_OUT,       /* [width, H V] */
  /* mixture of experts */
  SSDK_HT_ROUTER,        /* [E + identity, width] */
  SSDK_HT_EXPERT_IN,     /* [E, 2 ff, width]: per expert gate rows then up rows */
  SSDK_HT_EXPERT_OUT,    /* [E, width, ff] */
  SSDK_HT_SHARED_IN,     /* [2 sff (+ 1), width]: gate | up (| shared-gate row when shared_gate) */
  SSDK_HT_SHARED_OUT,    /* [width, sff] */
  /* serial post-norm blocks */
  SSDK_HT_NORM2,         /* [width] norm on the feed-forward's output (serial blocks) or input (two-norm blocks) */
  SSDK_HT_GLU_IN,        /* [2 ff, width]: gate rows then up rows */
  SSDK_HT_GLU_OUT,       /* [width, ff] */
  /* short convolutions of the recurrent mixers */
  SSDK_HT_CONV_W,        /* [channels, taps], the last column multiplies the current token */
  SSDK_HT_CONV_B,        /* [channels] or unbound */
  /* rglru */
  SSDK_HT_RGLRU_IN,      /* [2 R, width]: y-branch rows then x-branch rows */
  SSDK_HT_RGLRU_IN_B,    /* [2 R] their biases */
  SSDK_HT_RGLRU_GATE,    /* [blocks, 2 bs, bs]: per block the recurrence-gate rows then the input-gate rows */
  SSDK_HT_RGLRU_GATE_B,  /* [blocks, 2 bs] */
  SSDK_HT_RGLRU_LAM,     /* [R] */
  /* selective scan */
  SSDK_HT_SEL_IN,        /* [2 inner, width]: x rows then z rows */
  SSDK_HT_SEL_X,         /* [dt_rank + 2 state, inner] */
  SSDK_HT_SEL_DT,        /* [inner, dt_rank] */
  SSDK_HT_SEL_DT_B,      /* [inner] */
  SSDK_HT_SEL_ALOG,      /* [inner, state] */
  SSDK_HT_SEL_D,         /* [inner] */
  /* attention + delta rule pair: ONE stacked input projection,
   * rows: attn q [H D] | k [G D] | v [G V] | gate [H V] | delta q [Gd Dd] | k [Gd Dd] | v [Hd Vd] | gate [Hd Vd] | beta [Hd] | a [Hd] */
  SSDK_HT_PAIR_IN,
  SSDK_HT_ATTN_OUT,      /* [width, H V] */
  SSDK_HT_DELTA_ALOG,    /* [Hd] */
  SSDK_HT_DELTA_DT_B,    /* [Hd] */
  /* latent attention with full-rank queries (q_rank = 0): ONE stacked input projection,
   * rows: q [H (D + R)] | dkv [kv_rank + rot_dim] (absent when kv_from >= 0) | output gate [H V] (when out_gate) */
  SSDK_HT_LAT_IN,
  /* dense feed-forward without a gate (SSDK_MLP_FFN) */
  SSDK_HT_FFN_IN,        /* [ff, width] */
  SSDK_HT_FFN_IN_B,      /* [ff] */
  SSDK_HT_FFN_OUT,       /* [width, ff] */
  SSDK_HT_FFN_OUT_B,     /* [width] */
  SSDK_HT_ROUTER_BIAS,   /* [E + identity] added to the scores for the CHOICE of experts only (route_bias) */
  /* grouped-query attention alone (SSDK_MIX_ATTENTION): ONE stacked input projection q [H D] | k [G D] | v [G V], its bias,
   * the per-channel taps of the convolution that follows it (SSDK_HT_CONV_W, same row order) and one sink logit per head */
  SSDK_HT_ATTN_IN,       /* [H D + G D + G V, width] */
  SSDK_HT_ATTN_IN_B,     /* [H D + G D + G V] or unbound */
  SSDK_HT_ATTN_SINK,     /* [H] (learned_sink) */
  SSDK_HT_FFN_ACT,       /* [4] coefficients k1, k2, k3, k0 of SSDK_ACT_POLYNORM */
  /* SSDK_BLOCK_PARALLEL_ONE_NORM */
  SSDK_HT_CANON_W,       /* [2, width, canon_taps]: taps of the mixer's input convolution, then of the feed-forward's */
  SSDK_HT_RES_GATE,      /* [2 width, width]: rows of the mixer's residual gate, then of the feed-forward's */
  SSDK_HT_RES_GATE_B,    /* [2 width] */
  SSDK_HT_COUNT
};

typedef struct ssdk_hyb_layer_cfg {
  int32_t mixer;        /* SSDK_MIX_* */
  int32_t heads, dim, vdim;          /* per head: key (unrotated query/key for latent attention) and value size */
  int32_t rot_dim, rot_dims;         /* latent attention: rotated part per head; how many of them RoPE turns */
  int32_t kv_rank, q_rank;           /* latent sizes */
  int32_t decay_rank;                /* wkv: rows of the decay bottleneck */
  float   rot_base, attn_scale, gate_cap;
  int32_t mlp;          /* SSDK_MLP_* */
  int32_t experts, top, groups, keep;
  int32_t ff, shared_ff;             /* shared_ff = 0: no shared expert */
  float   route_scale, limit, shared_limit;
  /* grouped-query attention (SSDK_MIX_ATTN_DELTA uses heads / dim / vdim / rot_dims / rot_base / attn_scale above) */
  int32_t kv_heads;                  /* key/value heads; query head h reads head h / (heads / kv_heads) */
  int32_t qk_norm;                   /* 1: q and k divided by their RMS over dim after the rotation */
  float   sink;                      /* constant added to the softmax denominator (0: plain softmax; 1: a sink of score 0) */
  float   yarn_factor;               /* 0: no frequency scaling; else YaRN with the three values below */
  float   yarn_original, yarn_fast, yarn_slow;
  /* short convolution (rglru, selective scan, delta rule) */
  int32_t conv;                      /* taps */
  /* rglru: `inner` channels in `blocks` gate blocks; selective scan: inner x state, dt_rank */
  int32_t inner, blocks, state, dt_rank;
  float   decay_mult;                /* rglru: log a = -decay_mult * r * softplus(lam) */
  /* gated delta rule of SSDK_MIX_ATTN_DELTA */
  int32_t d_heads, d_kv_heads, d_dim, d_vdim;
  float   left_scale, right_scale;   /* result = left_scale * attention + right_scale * delta rule */
  /* latent attention variants (q_rank = 0: the queries come straight from the input, SSDK_HT_LAT_IN) */
  int32_t rot_interleaved;           /* 0: entry i turns with i + rot_dims/2; 1: entry 2i turns with 2i + 1 */
  int32_t kv_from;                   /* -1: the layer fills a pool of its own; j: it reads the pool of latent layer j < i */
  int32_t out_gate;                  /* 1: the concatenated heads are multiplied by sigmoid(W_g h) before the output projection */
  int32_t learned_sink;              /* 1: SSDK_HT_LAT_SINK joins the softmax denominator; 0: plain softmax */
  /* router variants */
  int32_t identity;                  /* the last `identity` router outputs are experts that return their input */
  int32_t route_softmax;             /* scores: 0 sigmoid, 1 softmax over all router outputs */
  int32_t route_bias;                /* 1: SSDK_HT_ROUTER_BIAS is added to the scores for the choice (not for the weights) */
  int32_t group_best;                /* a group's score: the sum of its `group_best` best choice scores (1 or 2) */
  int32_t route_renorm;              /* 1: the chosen scores are divided by their sum */
  int32_t expert_act, shared_gate;   /* SSDK_ACT_CLAMPED | SSDK_ACT_SILU; 1: the shared expert is scaled by sigmoid of its gate row */
  int32_t ff_act;                    /* SSDK_MLP_FFN: SSDK_ACT_* */
  int32_t window;                    /* attention (latent or grouped-query): a query at position p reads the keys at p - window + 1 .. p; 0: all of 0 .. p */
  int32_t rot_half;                  /* SSDK_MIX_ATTENTION: 1 = entry i turns with i + rot_dims/2, 0 = entry 2i with 2i + 1 */
  int32_t expert_glu;                /* 1: experts are down(act(gate h) * (up h)), SSDK_HT_EXPERT_IN / SHARED_IN hold gate | up rows;
                                      * 0: down(act(up h)), they hold the up rows only */
  int32_t route_top_softmax;         /* 1: the choice is made on the raw logits and the weights are the softmax over the chosen logits */
} ssdk_hyb_layer_cfg;

typedef struct ssdk_hyb_cfg {
  int32_t width, vocab, n_layers, dtype;
  float   eps;
  int32_t max_tokens;        /* rows per forward call */
  int32_t max_seqs;          /* sequences per forward call */
  int32_t max_logit_rows;    /* rows whose logits one call can return */
  int32_t block_size, max_blocks_per_seq;
  int32_t block;             /* SSDK_BLOCK_* */
  float   norm_offset;       /* a norm scales by norm_offset + w: 1 for unit-offset weights, 0 for plain ones */
  float   embed_scale;       /* x = embed[token] * embed_scale */
  float   residual_mult;     /* m of SSDK_BLOCK_SERIAL_POSTNORM */
  int32_t canon_taps;        /* SSDK_BLOCK_PARALLEL_ONE_NORM: taps of the sublayers' input convolutions (0: none) */
  int32_t gated_residual;    /* SSDK_BLOCK_PARALLEL_ONE_NORM: 1 = each sublayer's result is multiplied by sigmoid(W_g h + b) */
} ssdk_hyb_cfg;

typedef struct ssdk_hyb_engine* ssdk_hyb_handle;

int ssdk_hyb_create(const ssdk_hyb_cfg* cfg, const ssdk_hyb_layer_cfg* layers, ssdk_hyb_handle* out);
int ssdk_hyb_destroy(ssdk_hyb_handle h);
int ssdk_hyb_bind(ssdk_hyb_handle h, int layer, int tensor, const void* dev_ptr, int64_t rows, int64_t cols);
/* caller-owned pools: paged cache (per latent-attention layer [num_blocks, block_size, kv_rank + rot_dim] T, per
 * grouped-query attention layer (SSDK_MIX_ATTN_DELTA, SSDK_MIX_ATTENTION) [num_blocks, block_size, G (D + V)] T: keys of all heads, then values; layers back to back), recurrent state (fp32, n_slots slots), workspace */
int64_t ssdk_hyb_cache_bytes(ssdk_hyb_handle h, int64_t num_blocks);
int64_t ssdk_hyb_state_bytes(ssdk_hyb_handle h, int64_t n_slots);
int64_t ssdk_hyb_workspace_bytes(ssdk_hyb_handle h);
int ssdk_hyb_bind_pools(ssdk_hyb_handle h, void* cache, int64_t num_blocks, void* state, int64_t n_slots,
                        void* workspace, int64_t workspace_bytes);
/* One forward over a ragged batch: sequence s brings rows cu[s] .. cu[s+1]-1 (tokens ids[...]) that continue it at
 * position pos0[s]; its recurrent state lives in slot[s] (read only if pos0[s] > 0) and its latent rows in the pages
 * tables[s, :] (-1 padded).  Logits (fp32, [n_want, vocab]) of the rows want_rows[] are copied to logits_host if it
 * is not NULL; if temps is not NULL the same rows are sampled (Sampler semantics of ssdk_sample) into out_tokens.
 * residual_host, if not NULL, receives the fp32 residual stream after every layer, [n_layers, M, width] (debug tap).
 * All pointers are host pointers; the call blocks until the results are on the host. */
int ssdk_hyb_forward(ssdk_hyb_handle h, int n_seqs, int n_tokens, const int32_t* ids, const int32_t* cu,
                     const int32_t* pos0, const int32_t* slot, const int32_t* tables,
                     int n_want, const int32_t* want_rows, float* logits_host,
                     const float* temps, uint64_t seed, uint64_t step_id, int64_t* out_tokens,
                     float* residual_host, void* stream);
int64_t ssdk_hyb_launch_count(ssdk_hyb_handle h);

#ifdef __cplusplus
}
#endif
#endif /* SSDK_H_ */
