/*
 * tgis_engine.h — C ABI of libtgis_engine.so, the B200-native continuous-batching engine that replaces the
 * vLLM AsyncLLMEngine behind the TGIS gRPC adapter's generation path.
 *
 * Drop-in boundary.  The reference has no FFI; its seam is the `EngineClient` object that
 * `TextGenerationService` holds.  Each entry point below cites the reference call site it serves
 * (paths relative to /root/reference/src/vllm_tgis_adapter):
 *
 *   tgis_engine_create / _load_weight / _start   <- __main__.py:48   `build_async_engine_client(args)`
 *   tgis_engine_add_request                      <- grpc/grpc_server.py:205-225 `_make_generator` -> engine.generate(
 *                                                   prompt=TokensPrompt(prompt_token_ids=...), sampling_params=...,
 *                                                   request_id=...)
 *   tgis_engine_poll                             <- the AsyncGenerator[RequestOutput] consumed at
 *                                                   grpc_server.py:281 (Generate) and :367 (GenerateStream)
 *   tgis_engine_abort                            <- grpc_server.py:292, :388  `await self.engine.abort(request_id)`
 *   tgis_engine_set_mask_provider                <- grpc_server.py:581-586 `structured_outputs=get_structured_output_params(
 *                                                   decoding)` (tgis_utils/structured_outputs.py:14-38): the engine asks the
 *                                                   host's grammar matcher for each guided request's allowed-token bitmask
 *                                                   before it samples, and the sampling kernel applies it
 *   tgis_engine_load_adapter_weight / _clear_adapter <- grpc/adapters.py:139-155 `load_lora_adapter(LoadLoRAAdapterRequest)`
 *   tgis_engine_status                           <- grpc_server.py:117 `engine.errored and not engine.is_running`,
 *                                                   __main__.py:71
 *   tgis_engine_max_model_len                    <- grpc_server.py:196-199 `engine.vllm_config.model_config`
 *   tgis_engine_shutdown / _destroy              <- __main__.py:48 (exit of the `async with`)
 *
 * Conventions: plain pointers and sizes only (no torch types).  Every function returns 0 on success, <0 on error;
 * tgis_last_error() returns a thread-local message valid until the next call on the same thread.  The caller owns
 * input buffers until the call returns (the engine copies).  One dedicated engine thread per process runs the step
 * loop (scheduler + kernel launches); all entry points are thread-safe enqueue/dequeue operations.
 * There is NO CPU fallback: tgis_engine_create fails if no sm_100 device is present.
 */
#ifndef TGIS_ENGINE_H_
#define TGIS_ENGINE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TGIS_ABI_VERSION 11
#define TGIS_MAX_REQUEST_ID 96
#define TGIS_MAX_TOPN 12 /* reference forces max_logprobs >= 11: tgis_utils/args.py:214-216 */
#define TGIS_MAX_STOP_TOKEN_IDS 8

typedef struct tgis_engine tgis_engine;

/* Architectures (tgis_config.arch).  The reference names a model by --model-name (tgis_utils/args.py:104,185-186) and lets
 * vLLM pick the architecture from the checkpoint's config.json; the host-side loader does the same and passes it here.
 *   LLAMA: RMSNorm, neox RoPE, GQA, SwiGLU, no biases (BASELINE configs[1..4])
 *   OPT:   learned positions (offset 2), LayerNorm with bias, biased q/k/v/out/fc1/fc2, ReLU, tied lm_head,
 *          do_layer_norm_before = true, word_embed_proj_dim == hidden -- facebook/opt-125m, the reference's own test
 *          model (/root/reference/tests/conftest.py:79-91 (no --model: vLLM's default, facebook/opt-125m) and tests/test_hub.py:17; BASELINE configs[0]).  64-dim heads (head_dim = 64) run on the
 *          128-dim attention tiles: the engine zero-pads every head's q/k/v rows and out_proj columns at load time, which
 *          leaves every dot product unchanged.  Single GPU, no LoRA slots. */
#define TGIS_ARCH_LLAMA 0
#define TGIS_ARCH_OPT 1
/*   PONENEX: a stack of per-layer described blocks (tgis_model_spec / tgis_layer_spec below) on an fp32 residual stream:
 *          pre- and post-normed sublayers scaled by a residual multiplier, a latent-attention mixer (low-rank query and
 *          key/value latents, one shared rotary key part, sliding window, sigmoid output gate per head) and an optional
 *          mixture-of-experts feed-forward (biased top-k router, softmax over the chosen logits, gated shared expert).
 *          Created with tgis_engine_create_spec; bf16 or fp32 operands.  Single GPU, no LoRA slots. */
#define TGIS_ARCH_PONENEX 2

/*   FALERAX: a layer list as well (tgis_engine_create_spec), fp32 residual stream, sublayers that read the stream itself
 *          and are normed on their OUTPUT only (x += rmsnorm(sublayer(x)) * w, TGIS_STYLE_POST_NORM), logits from the
 *          embedding table (TGIS_STYLE_TIED_HEAD).  Mixers: softcapped grouped-query attention beside a gated matrix
 *          memory (TGIS_MIXER_PARALLEL), selective scan (TGIS_MIXER_SELECTIVE_SCAN), decayed outer-product memory with
 *          token shift (TGIS_MIXER_WKV); dense GeGLU feed-forward.  The recurrent mixers keep fp32 state per sequence slot.
 *          bf16 or fp32 operands.  Single GPU, no LoRA slots. */
#define TGIS_ARCH_FALERAX 3

/*   REVEPEL: a layer list as well (tgis_engine_create_spec), fp32 residual stream.  A layer has ONE norm; its mixer and its
 *          feed-forward both read that norm's output and are added to the stream together, each multiplied by a sigmoid
 *          gate computed from the same normed row (TGIS_STYLE_PARALLEL_GATED); the mixer reads the normed row blended with
 *          the previous token's (token shift; the previous normed row is part of the sequence slot's state).  Mixers:
 *          sliding-window attention with sigmoid weights, rotary positions with YaRN scaling and optionally another
 *          layer's keys and values (TGIS_MIXER_SIGMOID_ATTENTION), state-space duality scan (TGIS_MIXER_SSD), gated delta rule
 *          with a decay per key channel (TGIS_MIXER_CHANNEL_DELTA); mixture-of-experts feed-forward with a sigmoid router,
 *          squared-ReLU experts whose INPUT is weighted, and a shared expert (TGIS_MLP_MOE_SIGMOID).  Logits times
 *          logit_scale.  bf16 or fp32 operands.  Single GPU, no LoRA slots. */
#define TGIS_ARCH_REVEPEL 4

/*   SIKAZEN: a layer list as well (tgis_engine_create_spec), fp32 residual stream.  A layer has two norms that carry ONE number
 *          each; its mixer and its feed-forward read the same stream and are added together (TGIS_STYLE_PARALLEL_PAIR):
 *          x += mixer(rms(x) g1) + ff(rms(x) g2); then a per-layer token input is added: x += rms(P (gelu(G x) * e)) * w with e
 *          the layer's slice of the token's row of a side table.  A span of layers may run several passes in a row on the same
 *          weights (loop_start / loop_stop / loop_times), every pass with cache rows and state of its own; the embedding
 *          output is added to the stream before every pass but the first.  Mixers: grouped-query attention over a sliding
 *          window plus pooled blocks of what left it (TGIS_MIXER_POOLED_ATTENTION), latent attention with interleaved rotary
 *          pairs, no window, no output gate and a sink in the softmax (TGIS_MIXER_LATENT_ATTENTION + TGIS_LAYER_* flags),
 *          HGRN2 (TGIS_MIXER_HGRN); dense SwiGLU feed-forward (TGIS_MLP_DENSE_SILU).  bf16 or fp32 operands.  Single GPU,
 *          no LoRA slots. */
#define TGIS_ARCH_SIKAZEN 5

/* Model + runtime configuration (bf16 decoder-only transformer; see TGIS_ARCH_*). */
typedef struct tgis_config {
  int32_t abi_version; /* must be TGIS_ABI_VERSION */
  int32_t n_layers;
  int32_t hidden;
  int32_t n_q_heads;
  int32_t n_kv_heads;
  int32_t head_dim; /* 128; OPT: 64 or 128 */
  int32_t ffn;
  int32_t vocab;
  float rope_theta;
  float rms_eps;              /* RMSNorm epsilon; OPT: the LayerNorm epsilon */
  int32_t max_model_len;      /* reference: --max-sequence-length / --max-model-len (tgis_utils/args.py:187-192) */
  int32_t max_num_seqs;       /* concurrent sequences in the running batch */
  int32_t max_batched_tokens; /* token budget of one step (prefill chunk size) */
  int64_t kv_cache_bytes;     /* 0 = size from gpu_mem_fraction */
  float gpu_mem_fraction;     /* fraction of free HBM the KV cache may take when kv_cache_bytes == 0 */
  int32_t device;             /* CUDA device ordinal */
  int32_t tp_size;            /* tensor-parallel world (1 = single GPU); heads, ffn and vocab must divide */
  int32_t tp_rank;
  int32_t use_cuda_graphs;    /* capture decode steps into CUDA graphs */
  int32_t debug_gemm_ref;     /* debug only: route GEMMs through the SIMT cross-check kernel */
  uint64_t seed;              /* engine RNG for unseeded sampling requests */
  /* tensor parallelism (tp_size > 1): one process per GPU on one node.  Column-parallel q/k/v/gate/up, row-parallel
   * o/down with an NCCL all-reduce, vocab-parallel lm_head with an all-gather; rank 0 schedules and samples, the
   * other ranks run tgis_engine_worker_run().  nccl_id comes from tgis_nccl_unique_id() on rank 0 (distributed by
   * the host, e.g. torch.distributed); shm_name names the POSIX shm segment that carries the per-step plan. */
  uint8_t nccl_id[128];
  char shm_name[64];
  /* LoRA adapters (reference: grpc/adapters.py:63-163 -> lora_request; vLLM --enable-lora / --max-loras / --max-lora-rank):
   * max_loras > 0 reserves that many adapter slots of rank capacity max_lora_rank (multiple of 8, <= 64) over the seven
   * projections of every layer.  Single GPU only (tp_size == 1). */
  int32_t max_loras;
  int32_t max_lora_rank;
  int32_t arch;               /* TGIS_ARCH_LLAMA / TGIS_ARCH_OPT */
  int32_t reserved0;
} tgis_config;

/* Per-layer geometry for architectures whose layers are listed one by one (TGIS_ARCH_PONENEX); tgis_config carries hidden,
 * vocab, max_model_len and the runtime limits, its head / ffn / rope fields are unused. */
#define TGIS_MIXER_LATENT_ATTENTION 1
#define TGIS_MIXER_PARALLEL 2        /* softcapped attention and a gated matrix memory on the same input, averaged */
#define TGIS_MIXER_SELECTIVE_SCAN 3  /* short causal convolution + input-dependent state-space scan */
#define TGIS_MIXER_WKV 4             /* token shift + per-channel decayed outer-product memory with a current-token bonus */
#define TGIS_MIXER_SIGMOID_ATTENTION 5 /* grouped-query attention, rotary positions, window, weight = sigmoid(score + bias_h) */
#define TGIS_MIXER_SSD 6             /* short convolution + per-head scalar-decay state-space scan, gated group norm */
#define TGIS_MIXER_CHANNEL_DELTA 7   /* short convolutions + delta-rule memory whose key channels decay one by one */
#define TGIS_MIXER_POOLED_ATTENTION 8 /* grouped-query softmax attention: rotary positions, unit-norm queries and keys, a window
                                       * of tokens and one mean key / value for every block of `pool` tokens behind it */
#define TGIS_MIXER_HGRN 9            /* outer-product memory that writes with the complement of its forget gate (bounded below per channel) */
#define TGIS_MLP_NONE 0
#define TGIS_MLP_MOE 1
#define TGIS_MLP_DENSE_GELU 2        /* down(gelu_tanh(gate h) * (up h)), width `ff` */
#define TGIS_MLP_MOE_SIGMOID 3       /* experts down(relu(up (s h))^2) weighted on their input by s = sigmoid(router logit), the
                                      * `top` largest, their scores used as they are; shared expert of width shared_ff added (0: none) */
#define TGIS_MLP_DENSE_SILU 4        /* down(silu(gate h) * (up h)), width `ff` */
/* tgis_layer_spec.flags */
#define TGIS_LAYER_ROT_INTERLEAVED 1 /* rotary pairs are (2i, 2i + 1) instead of (i, i + rot_dims / 2) */
#define TGIS_LAYER_SINK 2            /* the softmax denominator of head h also holds exp(sink_h): "l<i>.mix.sink" */
#define TGIS_LAYER_NO_OUT_GATE 4     /* latent attention without the sigmoid output gate (no "l<i>.mix.g") */
#define TGIS_LAYER_QKV_BIAS 8        /* "l<i>.mix.q.b|k.b|v.b" are added to the projections */
#define TGIS_LAYER_UNIT_QK 16        /* queries and keys are divided by their root mean square per head after the rotation */
typedef struct tgis_layer_spec {
  int32_t mixer;        /* TGIS_MIXER_* */
  int32_t heads, dim, rot_dim, vdim, kv_rank, q_rank; /* per head: dim unrotated + rot_dim rotated query/key dims, vdim values */
  int32_t window;       /* position i sees j with 0 <= i - j < window; <= 0: all earlier positions */
  int32_t rot_dims;     /* the first rot_dims of the rot_dim dims are rotated (pairs i, i + rot_dims / 2) */
  float rot_base;
  float scale;          /* softmax scale */
  int32_t mlp;          /* TGIS_MLP_* */
  int32_t experts, top, expert_ff;
  int32_t shared_ff;    /* 0: no shared expert */
  int32_t ff;           /* TGIS_MLP_DENSE_GELU */
  /* TGIS_MIXER_PARALLEL, attention side: heads query heads of `dim`, kv_heads key/value heads (values of `vdim`), `scale`;
   * score <- softcap * tanh(score / softcap) (softcap <= 0: none); the query is multiplied by
   * 1 + qt_coef * ln(floor((pos + 1) / qt_every) + 1) (qt_every <= 0: no temperature) */
  int32_t kv_heads;
  float softcap, qt_coef;
  int32_t qt_every;
  /* ... matrix-memory side: mm_heads heads, keys / queries of mm_dim, values of mm_vdim, log gates capped at gate_cap */
  int32_t mm_heads, mm_dim, mm_vdim;
  float gate_cap;
  /* TGIS_MIXER_SELECTIVE_SCAN: `inner` channels with `state` entries each, step-size rank, convolution taps */
  int32_t inner, state, dt_rank, conv;
  /* TGIS_MIXER_WKV: heads x dim (keys and values alike); rank of the decay's low-rank map */
  int32_t decay_rank;
  int32_t reserved;
  /* TGIS_MIXER_SIGMOID_ATTENTION: heads / kv_heads / dim / vdim / window / rot_dims / rot_base / scale as above; rotary
   * frequencies under YaRN scaling (yarn_factor <= 0: plain): f_i <- f_i / factor * r_i + f_i * (1 - r_i) with r_i the linear
   * ramp between the dimensions that make yarn_fast and yarn_slow turns over yarn_original positions, cos and sin times
   * 0.1 ln(factor) + 1.  kv_from > 0: no key / value projections, the layer reads the cache rows of layer kv_from - 1 (an
   * earlier attention layer with projections of its own and the same kv_heads / dim / vdim / rotation) */
  int32_t kv_from;
  float yarn_factor, yarn_original, yarn_fast, yarn_slow;
  /* TGIS_MIXER_SSD: heads x vdim channels, `state` entries per channel, `groups` B / C groups, `conv` taps, the gated output
   * normed in norm_groups parts.  TGIS_MIXER_CHANNEL_DELTA: heads (values, vdim) / kv_heads (queries and keys, dim), `conv`
   * taps, decay_rank and gate_rank: inner sizes of the two low-rank maps (decay logits, output gate) */
  int32_t groups, norm_groups, gate_rank;
  /* TGIS_MIXER_POOLED_ATTENTION: heads / kv_heads / dim / vdim / window / rot_dims / rot_base / scale as above; `pool`: tokens per
   * pooled block (<= 0: a plain sliding window); rot_linear > 0: every rotary frequency is divided by it (also read by
   * TGIS_MIXER_LATENT_ATTENTION).  TGIS_MIXER_HGRN: heads x dim query / gate channels, heads x vdim values.  flags: TGIS_LAYER_* */
  int32_t pool;
  float rot_linear;
  int32_t flags;
  int32_t reserved2;
} tgis_layer_spec;
#define TGIS_STYLE_POST_NORM 1 /* x += rmsnorm(sublayer(x)) * w with a plain weight; unset: pre- and post-norm, weights stored
                                * as deviations from one */
#define TGIS_STYLE_TIED_HEAD 2 /* logits = embedding table x (no "head" tensor) */
#define TGIS_STYLE_PARALLEL_GATED 4 /* one norm per layer; x += sigmoid(R1 n + b1) * mixer(shift(n)) + sigmoid(R2 n + b2) * ff(n) */
#define TGIS_STYLE_PARALLEL_PAIR 8  /* two norms of ONE number each; x += mixer(rms(x) g1) + ff(rms(x) g2), then the per-layer token
                                     * input (side_dim > 0): x += rms(side.proj (gelu_tanh(side.gate x) * e)) * side.norm */
#define TGIS_DTYPE_BF16 0 /* bf16 operands, fp32 accumulation; norms, softmax, routers and the residual sum in fp32 */
#define TGIS_DTYPE_F32 1  /* everything in true fp32 (no TF32) */
typedef struct tgis_model_spec {
  int32_t n_layers;
  int32_t dtype;        /* TGIS_DTYPE_* */
  float embed_scale;    /* x = embed[token] * embed_scale */
  float residual_mult;  /* x += residual_mult * post_norm(sublayer(pre_norm(x))) */
  float norm_eps;
  int32_t style;        /* TGIS_STYLE_* bits */
  const tgis_layer_spec* layers; /* [n_layers] */
  float logit_scale;    /* logits = head x * logit_scale (0 is read as 1) */
  int32_t side_dim;     /* TGIS_STYLE_PARALLEL_PAIR: columns of the side table "side.embed" [vocab, n_layers * side_dim] that layer i
                           reads at [i * side_dim, (i + 1) * side_dim); 0: no per-layer token input */
  /* layers [loop_start, loop_stop) run loop_times passes in a row on the same weights, every pass with cache rows and state of
   * its own; before every pass but the first the embedding output is added to the stream.  loop_times <= 1: no loop */
  int32_t loop_start, loop_stop, loop_times;
  int32_t reserved;
} tgis_model_spec;

/* What the adapter's proto->SamplingParams mapping (grpc_server.py:508-628) hands to the engine. */
typedef struct tgis_sampling_params {
  int32_t greedy;             /* method == GREEDY or temperature == 0.0 (grpc_server.py:593-596) */
  float temperature;          /* used when !greedy */
  int32_t top_k;              /* <= 0: disabled (grpc_server.py:600) */
  float top_p;                /* >= 1: disabled (grpc_server.py:601) */
  float typical_p;            /* in (0,1): TypicalLogitsWarper mass; the caller passes 0 for method GREEDY (:562-565) */
  float repetition_penalty;   /* 1.0: disabled (:614) */
  int32_t has_length_penalty; /* DecodingParameters.length_penalty set (:567-578) */
  uint32_t lp_start_index;
  float lp_decay_factor;
  int32_t eos_token_id;       /* tokenizer.eos_token_id */
  int32_t min_tokens;         /* (:530) */
  int32_t max_tokens;         /* effective per-request maximum (:787-798) */
  int32_t num_logprobs;       /* vLLM `logprobs`: 0 = none, n>=1 = sampled-token logprob+rank and n top entries */
  int32_t prompt_logprobs;    /* 0 = none; k>=1: per prompt position logprob + rank of the prompt token and k top entries */
  int32_t has_seed;
  uint64_t seed;
  int32_t n_stop_token_ids;
  int32_t stop_token_ids[TGIS_MAX_STOP_TOKEN_IDS];
  int32_t guided;             /* DecodingParameters.guided / format set (structured_outputs.py:14-38): every sampled token
                                 is restricted to the bitmask the mask provider returns for this request */
  int32_t lora_slot;          /* 0: base model; s in 1..max_loras: the adapter loaded into slot s (lora_request, :205-225) */
} tgis_sampling_params;

/* Guided decoding.  The grammar state machine lives with the host (the reference hands a StructuredOutputsParams to vLLM,
 * whose scheduler fills one token bitmask per guided request per step: vllm v1/structured_output/__init__.py:204-300
 * `grammar_bitmask`, and the model runner masks the logits before the sampler: v1/structured_output/utils.py
 * `apply_grammar_bitmask`).  Here the engine thread calls the provider right before a step that samples for a guided
 * request: new_tokens[0..n_new) are the tokens generated since the previous call for this request (0 on the first call,
 * normally 1 afterwards; in order, each reported exactly once -- a preempted and recomputed sequence reports nothing
 * twice); the provider advances its matcher over them and writes the next step's bitmask: bit (i & 31) of word (i >> 5)
 * set = token i allowed (xgrammar's int32 token-bitmask layout), n_words = ceil(vocab / 32), bits >= vocab ignored.
 * allow_bits points into pinned host memory owned by the engine and is valid only during the call.
 * Return 0: bitmask written; 1: no constraint for this step; < 0: failure -- the request is finished with TGIS_FINISH_ABORT.
 * The sampling kernel turns the raw logit of every cleared bit into -inf before log-softmax, processors and selection. */
typedef int (*tgis_mask_fn)(void* user, const char* request_id, const int32_t* new_tokens, int32_t n_new,
                            uint32_t* allow_bits, int32_t n_words);

enum tgis_finish_reason {
  TGIS_FINISH_NONE = 0,
  TGIS_FINISH_LENGTH = 1,     /* vLLM finish_reason "length" */
  TGIS_FINISH_STOP_EOS = 2,   /* "stop", stop_reason None     */
  TGIS_FINISH_STOP_TOKEN = 3, /* "stop", stop_reason = int    */
  TGIS_FINISH_ABORT = 4,      /* "abort"                      */
  TGIS_FINISH_ERROR = 5
};

/* One record per request per engine step that produced a token or a terminal event
 * (the fields RequestOutput/CompletionOutput/Logprob expose at grpc_server.py:430-493, 701-756). */
typedef struct tgis_step_output {
  char request_id[TGIS_MAX_REQUEST_ID];
  int32_t n_new_tokens;   /* 0 or 1 */
  int32_t token_id;
  float logprob;          /* raw log-softmax of token_id (valid when num_logprobs > 0) */
  int32_t rank;           /* 1-based rank on the raw log-softmax */
  int32_t n_topn;
  int32_t topn_ids[TGIS_MAX_TOPN];
  float topn_logprobs[TGIS_MAX_TOPN];
  int32_t finish_reason;  /* enum tgis_finish_reason */
  int32_t stop_token_id;  /* valid for TGIS_FINISH_STOP_TOKEN */
  int32_t n_prompt_tokens;
  int32_t n_output_tokens; /* cumulative */
  double ts_arrival, ts_first_scheduled, ts_first_token, ts_last_token; /* CLOCK_MONOTONIC seconds */
  int32_t prompt_pos;     /* -1: generation record; >= 1: prompt-logprob record for prompt token `prompt_pos`
                             (token_id / logprob / rank / topn describe that prompt token given its prefix; emitted
                             before the request's first generated token; vllm prompt_logprobs semantics) */
  int32_t reserved;
} tgis_step_output;

typedef struct tgis_status {
  int32_t errored;     /* sticky after a fatal CUDA error */
  int32_t is_running;  /* step loop alive */
  int32_t n_running, n_waiting;
  int32_t free_blocks, total_blocks;
  int64_t steps;             /* engine steps executed */
  int64_t tokens_generated;
  int64_t kernel_launches;   /* kernels launched by this library since start */
  double gpu_busy_ms;        /* CUDA-event time of all steps (H2D of metadata .. D2H of results, on the engine stream) */
  double gpu_decode_ms;      /* ... of the pure-decode steps (every sequence advances by exactly one token) */
  double gpu_mixed_ms;       /* ... of the steps that carried prefill work */
  int64_t decode_steps;
  int64_t decode_tokens;     /* tokens sampled in pure-decode steps */
  int64_t h2d_bytes;         /* per-step metadata shipped host->device, cumulative */
  int64_t d2h_bytes;         /* per-step result records read back, cumulative */
  double gemm_ms;            /* with profiling on: summed CUDA-event time of every tcgen05 GEMM launch */
  double gemm_bytes;         /* ... and their algorithmic bytes (weights + activations in + result out) */
  int64_t gemm_calls;
  int64_t graph_launches;    /* decode steps replayed from a captured CUDA graph */
  double exchange_ms;        /* with profiling on, tensor parallelism: summed CUDA-event time of every row-parallel
                                exchange (fused push all-reduce + residual + RMSNorm kernel, or ncclAllReduce) */
  int64_t exchange_calls;
  int64_t preemptions;       /* sequences evicted from the KV cache and queued for recomputation (vLLM V1 policy) */
} tgis_status;

const char* tgis_last_error(void);
int tgis_abi_version(void);

int tgis_engine_create(const tgis_config* cfg, tgis_engine** out);
/* Layer-list architectures.  cfg->arch == TGIS_ARCH_PONENEX; parameter names: "embed", "head", "final.norm", "l<i>.norm1|norm1b|norm2|norm2b",
 * "l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o", "l<i>.mlp.router|router.b|e<j>.gate|e<j>.up|e<j>.down|shared.gate|
 * shared.up|shared.down|shared.sg" (bf16 [out, in]; the engine widens them for TGIS_DTYPE_F32). */
int tgis_engine_create_spec(const tgis_config* cfg, const tgis_model_spec* spec, tgis_engine** out);
/* cfg->arch == TGIS_ARCH_FALERAX; parameter names: "embed", "final.norm", "l<i>.norm1|norm2", "l<i>.mlp.gate|up|down",
 * TGIS_MIXER_PARALLEL "l<i>.mix.left.q|k|v|g|o|q.norm|k.norm|out", "l<i>.mix.right.q|k|v|g|o|norm|i|i.b|f|f.b|out";
 * TGIS_MIXER_SELECTIVE_SCAN "l<i>.mix.in|conv|conv.b|x|dt|dt.b|A_log|D|o"; TGIS_MIXER_WKV "l<i>.mix.mu.r|mu.k|mu.v|mu.g|mu.w|
 * r|k|v|g|w1|w2|w0|u|norm|o". */
/* cfg->arch == TGIS_ARCH_REVEPEL; parameter names: "embed", "head", "final.norm", "l<i>.norm1|shift|rg1|rg1.b|rg2|rg2.b",
 * "l<i>.mlp.router|e<j>.up|e<j>.down|shared.up|shared.down"; TGIS_MIXER_SIGMOID_ATTENTION "l<i>.mix.q|k|v|pb|o" (k, v absent
 * with kv_from); TGIS_MIXER_SSD "l<i>.mix.in|conv|conv.b|dt_bias|A_log|D|norm|o"; TGIS_MIXER_CHANNEL_DELTA "l<i>.mix.q|q.conv|k|
 * k.conv|v|v.conv|b|A_log|norm|a1|a2|dt_bias|g1|g2|o". */
/* cfg->arch == TGIS_ARCH_SIKAZEN; parameter names: "embed", "side.embed", "head", "final.norm" (one number), "l<i>.norm1|norm2" (one
 * number each), "l<i>.mlp.gate|up|down", "l<i>.side.gate|proj|norm"; TGIS_MIXER_POOLED_ATTENTION "l<i>.mix.q|q.b|k|k.b|v|v.b|o";
 * TGIS_MIXER_LATENT_ATTENTION "l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|o"; TGIS_MIXER_HGRN "l<i>.mix.q|f|f.b|lower|v|norm|o". */
/* name: HF Llama parameter name ("model.layers.3.self_attn.q_proj.weight", "lm_head.weight", ...) or
 * "tgis.rope_cos_sin" ([max_model_len,128] bf16 = cos|sin); arch OPT: HF OPT parameter names
 * ("model.decoder.layers.3.self_attn.q_proj.bias", "model.decoder.embed_positions.weight" with >= max_model_len + 2 rows,
 * ...; a 1-D tensor is passed as rows = n, cols = 1).  ptr may be host or device memory (cudaMemcpyDefault);
 * dtype 0 = bf16.  rows/cols describe the full (unsharded) tensor. */
int tgis_engine_load_weight(tgis_engine* e, const char* name, const void* ptr, int64_t rows, int64_t cols, int32_t dtype);
int tgis_engine_start(tgis_engine* e);
int tgis_engine_add_request(tgis_engine* e, const char* request_id, const int32_t* prompt_ids, int32_t n_prompt,
                            const tgis_sampling_params* params);
int tgis_engine_abort(tgis_engine* e, const char* request_id);
/* LoRA adapter slots.  name: "layers.<i>.<module>.lora_A" ([r, in] bf16) or "...lora_B" ([out, r] bf16, alpha / r already
 * folded in by the host: vllm lora_weights.py `optimize`), module in q_proj k_proj v_proj o_proj gate_proj up_proj down_proj;
 * r <= max_lora_rank (the slot is zero padded).  ptr may be host or device memory.  A slot must not be cleared or rewritten
 * while a queued or running request names it (checked).  tgis_engine_clear_adapter zeroes every tensor of the slot. */
int tgis_engine_load_adapter_weight(tgis_engine* e, int32_t slot, const char* name, const void* ptr, int64_t rows,
                                    int64_t cols);
int tgis_engine_clear_adapter(tgis_engine* e, int32_t slot);
/* fn == NULL removes the provider; requests with params->guided != 0 are rejected while none is installed */
int tgis_engine_set_mask_provider(tgis_engine* e, tgis_mask_fn fn, void* user);
/* Blocks up to timeout_ms for at least one record; returns the number written to out[0..cap) (>= 0) or <0 on error. */
int tgis_engine_poll(tgis_engine* e, tgis_step_output* out, int32_t cap, int32_t timeout_ms);
int tgis_engine_status(tgis_engine* e, tgis_status* out);
/* tensor-parallel plumbing (reference seam: tgis_utils/args.py:201-213 --num-gpus/--num-shard -> tensor_parallel_size) */
int tgis_nccl_unique_id(uint8_t out[128]);
/* ranks > 0: blocks, executing rank 0's step plans on this rank's shard, until rank 0 shuts down; 0 on clean exit */
int tgis_engine_worker_run(tgis_engine* e);
/* on != 0: bracket every GEMM launch with CUDA events (costs a little host time; used by bench.py's roofline leg);
 * on == 2: only in pure-decode steps */
int tgis_engine_set_profiling(tgis_engine* e, int32_t on);
int tgis_engine_max_model_len(tgis_engine* e);
int tgis_engine_shutdown(tgis_engine* e);
void tgis_engine_destroy(tgis_engine* e);

/* Trace replay: feed GIVEN tokens through the engine's own step function (scheduler slots, block manager, the same kernels
 * and batch layout as generation), sampling nothing.  One call = one step = one batch: entry i brings the next n_tokens of
 * request request_id (admitted at its first entry: a sequence slot and cache blocks are taken from the engine's pools;
 * a request may be left out of a step and go on later) and asks for the logits after its tokens want[0..n_want) (indices
 * into this entry's tokens).  logits_out: fp32 [sum n_want, vocab] in entry / want order.  end_ids: requests that are
 * finished after this step; their slot and blocks go back to the pools.  Not to be mixed with add_request traffic. */
typedef struct tgis_trace_entry {
  const char* request_id;
  const int32_t* tokens;
  int32_t n_tokens;
  int32_t n_want;
  const int32_t* want;
} tgis_trace_entry;
int tgis_engine_trace_step(tgis_engine* e, const tgis_trace_entry* entries, int32_t n_entries, const char* const* end_ids,
                           int32_t n_end, float* logits_out);

/* Synchronous driver used by bench.py / tests: run the step loop on the calling thread until every queued request has
 * finished (no engine thread needed).  Returns the number of steps, <0 on error.  Step wall/GPU times accumulate in
 * tgis_status. */
int tgis_engine_run_until_idle(tgis_engine* e);

#ifdef __cplusplus
}
#endif
#endif /* TGIS_ENGINE_H_ */
