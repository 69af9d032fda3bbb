// Internal launcher declarations for the sm_100a kernels of the TGIS decode/prefill hot path.
// (Internal C++ header; the drop-in C ABI is include/tgis_engine.h.)
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tgis {

// ---- gemm_tcgen05.cu --------------------------------------------------------------------------------------------
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems,
                      uint32_t box_rows, uint32_t box_cols);
int gemm_pick_bt(int T);
int gemm_nw(int T);  // weight tiles (128 rows each) per unit sharing one activation tile: 2 for decode-shaped launches
size_t gemm_workspace_bytes(int num_sms);
int gemm_timeline_read(unsigned long long* out64);  // debug builds (-DTGIS_GEMM_TIMELINE) only
// -DTGIS_STEP_TIMELINE builds: point every translation unit's kernels at the timeline buffer (ptx.cuh); else -2
int gemm_set_step_timeline(unsigned long long* buf);
int elementwise_set_step_timeline(unsigned long long* buf);
int attention_set_step_timeline(unsigned long long* buf);
int sampler_set_step_timeline(unsigned long long* buf);
// Decode-shaped successor of a GEMM launch: lets the running kernel pull the first `kb_prefetch` weight boxes of every
// CTA of the NEXT GEMM into L2 while its own tail drains (kb_prefetch == 0: off).
struct GemmNext {
  int n_tiles, KB, grid, kb_prefetch;
};
int gemm_grid_size(int T, int N, int K, int num_sms);
int gemm_even_split(int T, int N, int K, int num_sms);  // every tile cut over this many consecutive CTAs, or 0
GemmNext gemm_next_desc(int T_next, int N_next, int K_next, int num_sms, int kb_prefetch);
// Y: bf16 [T, ldy] (out_f32 = 0), fp32 [T, ldy] (out_f32 = 1, lm_head logits), or out_f32 = 2: fused SwiGLU — W rows are
// interleaved (gate_j, up_j) pairs and Y is bf16 [T, ldy >= N/2] = bf16(bf16(silu(gate)) * up); out_f32 = 3: the same with
// the tanh form of gelu on the gate, evaluated on the fp32 accumulators (GeGLU)
// Optional fused epilogue of the qkv projection (cluster mode only, gemm_cluster_split() > 0): RoPE on the q / k heads
// and scatter of k / v into the paged cache, replacing rope_kvwrite_kernel.  N must be (n_q + 2 n_kv) * 128.
struct GemmRope {
  const int32_t* positions;     // [T]; nullptr = no fusion
  const int32_t* slot_mapping;  // [T], < 0: do not cache
  const __nv_bfloat16* cos_sin; // [max_pos][128]: cos (64) | sin (64)
  __nv_bfloat16* k_cache;       // this layer's caches
  __nv_bfloat16* v_cache;
  int32_t n_q, n_kv;
};
// Optional fusion of the layer stack's  residual add + RMSNorm  (vllm layernorm.py fused_add_rms_norm; same rounding
// points as add_rmsnorm_launch) into the two GEMMs either side of it, decode-shaped launches only (one token tile,
// T <= 64):
//  * producer (o / down projection, cluster mode required): the split-tile reduction does not write Y; it computes
//    h = bf16(bf16(acc) + residual), stores h back to `residual` [T, N] and the tile's sum of h^2 to
//    sumsq_out[t * (N / 128) + tile]  (N % 128 == 0);
//  * consumer (qkv / gate_up projection): the activation operand is not loaded by TMA; two extra warps build
//    bf16(bf16(h * rstd) * w_norm) straight into the swizzled shared-memory stage, rstd[t] from the n_parts partial sums
//    added in tile order (deterministic).  K % 64 == 0.
struct GemmNorm {
  __nv_bfloat16* residual;       // producer: in/out [T, N]; nullptr = off
  float* sumsq_out;              // producer: [T][N / 128]
  const __nv_bfloat16* h;        // consumer: [T, K]; nullptr = off
  const float* sumsq_in;         // consumer: [T][n_parts]
  const __nv_bfloat16* w_norm;   // consumer: [K]
  int32_t n_parts;
  float eps;
};
constexpr int GEMM_NORM_MAX_T = 64;
constexpr int GEMM_NORM_MAX_PARTS = 64;  // hidden <= 8192
int gemm_cluster_split(int T, int N, int K, int num_sms);
cudaError_t gemm_bf16_launch(const CUtensorMap& wmap, const CUtensorMap& xmap, void* Y, int ldy, int T, int N, int K,
                             float* ws, int* counters, int num_sms, cudaStream_t stream, int out_f32 = 0,
                             const CUtensorMap* next_wmap = nullptr, const GemmNext* next = nullptr,
                             const GemmRope* rope = nullptr, const GemmNorm* norm = nullptr);

// ---- gemm_ref.cu (debug cross-check only; never on the product path) ---------------------------------------------
cudaError_t gemm_bf16_ref_launch(const __nv_bfloat16* X, int ldx, const __nv_bfloat16* W, void* Y, int ldy, int T,
                                 int N, int K, cudaStream_t stream, int out_f32 = 0);

// ---- elementwise.cu ----------------------------------------------------------------------------------------------
cudaError_t stl_marker_launch(int kid, cudaStream_t stream);  // -DTGIS_STEP_TIMELINE builds only (else a no-op)
cudaError_t embed_gather_launch(const int32_t* token_ids, const __nv_bfloat16* table, __nv_bfloat16* out, int T,
                                int hidden, int vocab, cudaStream_t stream);
// out = rmsnorm(x) * w                                   (first layer: residual := x is done by the caller)
cudaError_t rmsnorm_launch(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, int T, int hidden,
                           float eps, cudaStream_t stream);
// residual = bf16(x + residual); out = rmsnorm(residual) * w     (vllm: layernorm.py fused_add_rms_norm)
cudaError_t add_rmsnorm_launch(const __nv_bfloat16* x, __nv_bfloat16* residual, const __nv_bfloat16* w,
                               __nv_bfloat16* out, int T, int hidden, float eps, cudaStream_t stream);
// Tensor parallelism, decode-shaped steps: one-shot all-reduce of the row-parallel GEMM partials over NVLink peer memory
// fused with the residual add + RMSNorm (elementwise.cu).  own: this rank's partial [T, hidden]; recv[q]: rank q's receive
// area for this exchange parity, mapped into this process (recv[own rank] = local): [8 source ranks][AR_MAX_ROWS rows]
// [hidden / 8 vectors][2 lines of 16 bytes = {data, epoch, data, epoch}].
constexpr int AR_MAX_ROWS = 256;
inline size_t ar_recv_bytes(int hidden) { return (size_t)8 * AR_MAX_ROWS * (hidden / 8) * 2 * 16; }
struct ArPeers {
  const __nv_bfloat16* own;
  uint4* recv[8];
};
// The exchange's epoch is *epoch_base + epoch_idx (epoch_base: device memory written by the step's metadata copy).
cudaError_t ar_add_rmsnorm_launch(const ArPeers& peers, int tp, int rank, const uint32_t* epoch_base, uint32_t epoch_idx,
                                  __nv_bfloat16* residual, const __nv_bfloat16* w, __nv_bfloat16* out, int T, int hidden,
                                  float eps, cudaStream_t stream);
// Two-shot variant (reduce-scatter by row owner t mod tp, all-gather of the bf16 reduced rows; elementwise.cu) for
// exchanges whose one-shot egress would be large.  area[q]: rank q's two-shot area for this exchange parity, mapped here.
inline size_t ar2_area_bytes(int hidden) { return (size_t)9 * AR_MAX_ROWS * hidden * 2 + (size_t)9 * AR_MAX_ROWS * 4; }
struct Ar2Peers {
  const __nv_bfloat16* own;
  uint8_t* area[8];
};
cudaError_t ar2_add_rmsnorm_launch(const Ar2Peers& peers, int tp, int rank, const uint32_t* epoch_base, uint32_t epoch_idx,
                                   __nv_bfloat16* residual, const __nv_bfloat16* w, __nv_bfloat16* out, int T, int hidden,
                                   float eps, cudaStream_t stream);
// Vocab-parallel lm_head without NCCL: ranks > 0 push their shard into rank 0's logits buffer (peer memory) and raise a
// flag there; rank 0 waits for the flags (elementwise.cu).  Sizes in bytes (multiples of 16).
cudaError_t logits_push_launch(const void* shard, void* dst_peer0, int R, int Vl_bytes, int V_bytes, int col_bytes,
                               uint32_t* remote_flag, int* local_counter, const uint32_t* epoch_base, uint32_t epoch_idx,
                               cudaStream_t stream);
cudaError_t logits_wait_launch(const uint32_t* flags, int tp, const uint32_t* epoch_base, uint32_t epoch_idx,
                               cudaStream_t stream);
// act[t, i] = bf16(silu(gate_up[t, i])) * gate_up[t, F + i]
cudaError_t silu_mul_launch(const __nv_bfloat16* gate_up, __nv_bfloat16* act, int T, int ffn, cudaStream_t stream);
// ---- multi-adapter LoRA (lora.cu): y[t, col0 + n] += bf16(B_s[n, :] . bf16(A_s x[t])), s = tok_slot[t] (0 = no adapter)
struct LoraModule {
  const __nv_bfloat16* A;  // [slots][Rm][K]  (slot s >= 1 lives at index s - 1), zero padded to Rm rows
  const __nv_bfloat16* B;  // [slots][N][Rm]  (alpha / r already folded in), zero padded to Rm columns
  int K, N, Rm;            // Rm: rank capacity of the module (multiple of 8, <= 128)
  int col0;                // first output column of the module in y (multiple of 8)
  int v_off;               // offset of the module's rank vector inside a token's row of the shrink buffer
};
constexpr int LORA_GROUP_MAX = 3;  // modules that read the same x (q, k, v)
struct LoraGroup {
  LoraModule mod[LORA_GROUP_MAX];
  int n_mods;
  int v_ld;                // floats per token in the shrink buffer
};
cudaError_t lora_shrink_launch(const __nv_bfloat16* x, int ldx, const int32_t* tok_slot, const LoraGroup& g, float* v, int T,
                               cudaStream_t stream);
cudaError_t lora_expand_launch(const float* v, const int32_t* tok_slot, const LoraGroup& g, __nv_bfloat16* y, int ldy, int T,
                               cudaStream_t stream);
// act[t, j] = bf16(silu(gate_up[t, 2j])) * gate_up[t, 2j + 1]  (the interleaved gate_up layout the fused GEMM epilogue reads)
cudaError_t silu_mul_interleaved_launch(const __nv_bfloat16* gate_up, __nv_bfloat16* act, int T, int ffn,
                                        cudaStream_t stream);
// ---- opt.cu (OPT layer stack: learned positions, biased projections, ReLU, LayerNorm) ------------------------------
// out[t] = bf16(tok_table[tok[t]] + pos_table[pos[t] + offset])
cudaError_t opt_embed_launch(const int32_t* token_ids, const int32_t* positions, const __nv_bfloat16* tok_table,
                             const __nv_bfloat16* pos_table, __nv_bfloat16* out, int T, int hidden, int vocab,
                             int n_pos_rows, int offset, cudaStream_t stream);
// acc != nullptr: residual = bf16(residual + bf16(acc + acc_bias)) first (acc: fp32 GEMM accumulators [T, hidden]);
// out = LayerNorm(residual) * w + b
cudaError_t opt_layernorm_launch(const float* acc, const __nv_bfloat16* acc_bias, __nv_bfloat16* residual,
                                 const __nv_bfloat16* w, const __nv_bfloat16* b, __nv_bfloat16* out, int T, int hidden,
                                 float eps, cudaStream_t stream);
// out[t, n] = bf16(act(acc[t, n] + bias[n])), act = ReLU or identity
cudaError_t opt_bias_act_launch(const float* acc, int ld_acc, const __nv_bfloat16* bias, __nv_bfloat16* out, int ld_out,
                                int T, int N, int relu, int num_sms, cudaStream_t stream);
// qkv epilogue: q_out[t, head, :] = bf16(acc + bias) for the q heads; k / v heads go straight into the paged cache
// (slot_mapping[t] < 0: not cached).  acc fp32 [T, (n_q + 2 n_kv) * 128], q_out bf16 with the same row stride.
cudaError_t opt_qkv_bias_kvwrite_launch(const float* acc, const __nv_bfloat16* bias, __nv_bfloat16* q_out,
                                        const int32_t* slot_mapping, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, int T,
                                        int n_q, int n_kv, cudaStream_t stream);
// gather rows: out[r, :] = x[rows[r], :]
cudaError_t gather_rows_launch(const __nv_bfloat16* x, const int32_t* rows, __nv_bfloat16* out, int R, int hidden,
                               cudaStream_t stream);

// Paged KV cache layout (per layer), chosen for the decode kernel's TMA bulk loads:
//   K: [num_blocks][n_kv][HEAD_DIM/8][BLOCK][8] bf16  (8-dim chunk major: lanes=tokens read conflict-free 16 B)
//   V: [num_blocks][n_kv][BLOCK][16 chunks ^ (tok&7)][8] bf16  (row-major with the 16-B chunk index XOR-swizzled)
// one (block, kv_head) K or V tile is a contiguous BLOCK*HEAD_DIM*2 bytes.
constexpr int KV_BLOCK = 32;
constexpr int HEAD_DIM = 128;

// neox RoPE on q,k in-place inside qkv[T, (nq+2nkv)*128] and scatter of k,v into the paged cache.
// cos_sin: [max_pos][128] bf16 = cos(64) | sin(64)   (vllm: rotary_embedding/base.py cache.to(dtype))
cudaError_t rope_kvwrite_launch(__nv_bfloat16* qkv, const int32_t* positions, const int32_t* slot_mapping,
                                const __nv_bfloat16* cos_sin, __nv_bfloat16* k_cache, __nv_bfloat16* v_cache, int T,
                                int n_q, int n_kv, cudaStream_t stream);

// ---- attention.cu ------------------------------------------------------------------------------------------------
struct AttnSeq {        // one entry per sequence scheduled this step (device array)
  int32_t q_start;      // first row of this sequence's queries in the flat token batch
  int32_t q_len;        // number of query tokens this step (1 = decode)
  int32_t kv_len;       // context length INCLUDING this step's tokens
  int32_t block_row;    // row in the block table
};
// Decode (q_len == 1): split-KV over chunks of DECODE_SPLIT tokens; the host lists the (sequence, split) entries of
// the step, the kernel crosses them with the kv heads.  items[0].q_row = number of entries, entries follow from [1].
constexpr int DECODE_SPLIT = 128;
struct DecItem {       // 32 bytes
  int32_t q_row;       // row of the sequence's token in qkv / out            ([0]: number of entries)
  int32_t kv_len;      // of the whole sequence
  int32_t seq_split;   // seq | split << 16; seq = index among this step's decode sequences (partial buffers)
  int32_t reserved;
  int32_t blocks[DECODE_SPLIT / KV_BLOCK];  // physical KV blocks of the split (resolved on the host: no table walk)
};
static_assert(DECODE_SPLIT / KV_BLOCK == 4 && sizeof(DecItem) == 32, "DecItem is read as two int4");
// Entries are listed longest first (all full splits, then the partial tails by decreasing length): the kernel deals
// them to its warps round-robin, so the order is the load balance.  Ties keep (sequence, split) order: deterministic.
inline int decode_items_build(DecItem* items, const AttnSeq* seqs, const int32_t* seq_ids, int n_seqs,
                              const int32_t* block_table, int bt_stride) {
  constexpr int BPS = DECODE_SPLIT / KV_BLOCK;
  int n = 0;
  auto emit = [&](int i, const AttnSeq& sq, int sp) {
    const int n_blocks = (sq.kv_len + KV_BLOCK - 1) / KV_BLOCK;
    const int32_t* row = block_table + (size_t)sq.block_row * bt_stride;
    DecItem& it = items[++n];
    it = DecItem{sq.q_start, sq.kv_len, i | (sp << 16), 0, {0, 0, 0, 0}};
    for (int j = 0; j < BPS; ++j) it.blocks[j] = sp * BPS + j < n_blocks ? row[sp * BPS + j] : 0;
  };
  for (int i = 0; i < n_seqs; ++i) {  // full splits
    const AttnSeq& sq = seqs[seq_ids ? seq_ids[i] : i];
    for (int sp = 0; sp < sq.kv_len / DECODE_SPLIT; ++sp) emit(i, sq, sp);
  }
  for (int nb = BPS; nb >= 1; --nb) {  // tails: 4, 3, 2, 1 blocks (a tail of exactly DECODE_SPLIT tokens was a full split)
    for (int i = 0; i < n_seqs; ++i) {
      const AttnSeq& sq = seqs[seq_ids ? seq_ids[i] : i];
      const int rem = sq.kv_len % DECODE_SPLIT;
      if (rem > 0 && (rem + KV_BLOCK - 1) / KV_BLOCK == nb) emit(i, sq, sq.kv_len / DECODE_SPLIT);
    }
  }
  items[0] = DecItem{n, 0, 0, 0, {0, 0, 0, 0}};
  return n;
}
// Streaming kernel + (max_splits > 1) the split-merge kernel.  seqs / seq_ids / n_seqs: this step's decode sequences in
// the order decode_items_build numbered them.
cudaError_t attn_decode_launch(const __nv_bfloat16* qkv, int qkv_ld, const __nv_bfloat16* k_cache,
                               const __nv_bfloat16* v_cache, const DecItem* items, int max_entries,
                               const AttnSeq* seqs, const int32_t* seq_ids, int n_seqs, int max_splits, float* part_o,
                               float* part_ml, __nv_bfloat16* out, int out_ld, int n_q, int n_kv, float scale,
                               int num_sms, cudaStream_t stream, int* arrive = nullptr);
// arrive: [n_seqs * n_kv] ints, zero before the first launch (re-armed by the kernel): with it, the split merge runs inside
// the streaming kernel (last-arriving warp per (sequence, kv head)) and attn_merge_kernel is not launched.
// Prefill / chunked prefill (q_len >= 1), causal over the paged cache.
cudaError_t attn_prefill_launch(const __nv_bfloat16* qkv, int qkv_ld, const __nv_bfloat16* k_cache,
                                const __nv_bfloat16* v_cache, const AttnSeq* seqs, const int32_t* tile_seq,
                                const int32_t* tile_q0, int n_tiles, const int32_t* block_table, int bt_stride,
                                __nv_bfloat16* out, int out_ld, int n_q, int n_kv, float scale, cudaStream_t stream);

// ---- element types of the kernels that run more than one (gemm_any.cu, attention_latent.cu, moe.cu, the fp32-residual norms)
constexpr int DT_F32 = 0, DT_BF16 = 1;
inline size_t dt_size(int dt) { return dt == DT_BF16 ? 2 : 4; }

// ---- gemm_any.cu: Y = X W^T for any shape, bf16 or fp32 operands, dense / batched / grouped (see the file's header) -----
constexpr int GEMM_ANY_PLAIN = 0;     // Y[row, n] = acc
constexpr int GEMM_ANY_SWIGLU = 1;    // W rows interleaved (gate_j, up_j): Y[row, j] = silu(acc[2j]) * acc[2j + 1], N = 2 ff
constexpr int GEMM_ANY_ROWSCALE = 2;  // Y[row, n] = acc * row_scale[row * scale_ld + batch index]
constexpr int GEMM_ANY_GEGLU = 3;     // as SWIGLU with the tanh form of gelu on the gate
constexpr int GEMM_ANY_TANH = 4;      // Y[row, n] = tanh(acc)
constexpr int GEMM_ANY_RELU2 = 5;     // Y[row, n] = max(acc * s, 0)^2, s = row_scale[gather ? gather[row] : row] (row_scale == nullptr: 1):
                                      // a squared-ReLU layer whose INPUT row was multiplied by s
struct GemmAny {
  const void* X; const void* W; void* Y;
  int x_dtype, w_dtype, y_dtype;   // DT_*
  int T, N, K;                     // rows of X (grouped: total rows over all segments), rows of W, reduction length
  int ldx, ldw, ldy;               // leading dimensions in elements
  int batch;                       // > 1: blockIdx.z problems, operands x_bs / w_bs / y_bs elements apart
  long long x_bs, w_bs, y_bs;
  const int* seg_off;              // grouped: [n_groups + 1] row offsets on the device (nullptr: dense)
  int n_groups;
  long long w_gs;                  // elements between the weight matrices of consecutive groups
  const int* gather;               // grouped: X row of position p = gather[p] / gather_div (nullptr: p itself)
  int gather_div;
  int mode;                        // GEMM_ANY_*
  const float* row_scale; int scale_ld;
};
cudaError_t gemm_any_launch(const GemmAny& a, cudaStream_t stream);

// ---- norms over an fp32 residual stream (elementwise.cu) ------------------------------------------------------------
// out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * (w_off + w)      x fp32 [T, ldx], n columns normed; out: DT_* [T, ldo]
cudaError_t rmsnorm_f32_launch(const float* x, int ldx, const float* w, float w_off, void* out, int out_dtype, int ldo, int T,
                               int n, float eps, cudaStream_t stream);
// resid[t] = table[tok[t]] * scale   (fp32 residual stream from a bf16 / fp32 embedding table)
cudaError_t embed_scale_f32_launch(const int32_t* token_ids, const void* table, int table_dtype, float scale, float* resid,
                                   int T, int hidden, int vocab, cudaStream_t stream);
// One sublayer's tail on an fp32 residual stream, row per CTA:
//   y[t]      = y_main[t]                                               (y_main != nullptr), or the mixture
//             = sum_k mix_w[t, k] * y_rows[inv[t * top + k]] + side_gate[t] * y_side[t]     (terms with null pointers drop out)
//   resid[t] += mult * rmsnorm(y[t]) * (w_off + w_post)
//   out[t]    = rmsnorm(resid[t]) * (w_off + w_pre)                      (w_pre != nullptr: the next sublayer's input)
//             = (rmsnorm(y_main[t]) * w_main + rmsnorm(y_pair[t]) * w_pair) / 2             (y_pair != nullptr: two mixers
//                                                                                            side by side, plain weights)
//   cast_out != 0 (and w_pre == nullptr): out[t] = resid[t] in the operand type -- the next sublayer reads the stream itself
//   extra != nullptr: resid[t] += extra[t] after the update;  w_pre2 / out2: out2[t] = rmsnorm(resid[t]) * (w_off + w_pre2)
struct ResidTail {
  const float* y_main;
  const float* y_rows; const int32_t* inv; const float* mix_w; int top;
  const float* y_side; const float* side_gate;
  const float* w_post; const float* w_pre;
  float* resid; void* out; int out_dtype;
  float mult, w_off, eps;
  const float* y_pair; const float* w_main; const float* w_pair;
  int cast_out;
  const float* extra;                 // optional fp32 [T, hidden]: added to resid after the sublayer's update, before the pre-norm
  const float* w_pre2; void* out2;    // optional second pre-norm of the same rows with another weight (two sublayers side by side)
};
cudaError_t resid_tail_launch(const ResidTail& a, int T, int hidden, cudaStream_t stream);
// Tail of a layer whose mixer and feed-forward run side by side on ONE normed input and are gated per channel, row per CTA:
//   resid[t] += sigmoid(gl[t, :hidden] + b1) * y_mix[t] + sigmoid(gl[t, hidden : 2 hidden] + b2) * (sum_k y_rows[inv[t * top + k]] + y_side[t])
//   n = rmsnorm(resid[t]) * w_next * out_scale -> n_f32[t] (fp32, optional) and out[t] (operand type): the next layer's normed input
//   (the feed-forward terms with null pointers drop out; gl == nullptr: both gates are one)
// and, for the last row of every portion, prev_state[slot] = n_cur[t]: the token shift's state of THIS layer.
struct GatedTail {
  const float* y_mix;
  const float* gl; int ldg; const float *b1, *b2;
  const float* y_rows; const int32_t* inv; int top;
  const float* y_side;
  float* resid;
  const float* w_next; float eps, out_scale;
  float* n_f32; void* out; int out_dtype;
  const float* n_cur; float* prev_state; const int32_t* tok_slot;
  const float* w_next2; void* out2;   // optional: the same normed rows under a second weight (operand type)
  void* resid_out;                    // optional: the updated stream itself in the operand type
  const float* extra;                 // optional fp32 [T, hidden]: added to the stream together with the update
};
cudaError_t gated_tail_launch(const GatedTail& a, int T, int hidden, cudaStream_t stream);
// out[t, j] = gelu_tanh(z[t, j]) * table[tok[t], col0 + j]   j < n: a gate on per-token side rows (z fp32 [T, ldz], table DT_*
// [vocab, ld_table], out DT_* [T, n])
cudaError_t gelu_gate_rows_launch(const float* z, int ldz, const int32_t* token_ids, const void* table, int table_dtype,
                                  int ld_table, int col0, int n, void* out, int out_dtype, int T, cudaStream_t stream);
// rows of any DT_* matrix: out[r, :] = x[rows[r], :]
cudaError_t gather_rows_any_launch(const void* x, const int32_t* rows, void* out, int R, int hidden, int dtype,
                                   cudaStream_t stream);
// dst[r * rs + c * cs] = src[r, c]   (bf16 checkpoint tensor -> DT_* arena slice; transposes and row interleaves at load time)
cudaError_t weight_place_launch(const __nv_bfloat16* src, int rows, int cols, void* dst, int dst_dtype, long long rs,
                                long long cs, cudaStream_t stream);

// ---- attention_latent.cu: attention over a cached low-rank latent (one shared key/value row per token) ---------------
// A token's cache row is [c (kv_rank) | k_rot (rot_dim)]; with the per-head up-projections folded into the query and
// the output ("absorbed" form) every head scores and sums the SAME rows:
//   score_h(i, j) = scale * (q_abs_h(i) . c(j) + q_rot_h(i) . k_rot(j)),  q_abs_h = W_uk,h^T q_nope_h
//   o_h(i)        = W_uv,h sum_j p_h(i, j) c(j)
// Visibility: causal, and with window > 0 only the last `window` positions (0 <= i - j < window).
struct LatentGeom {
  int heads, dim, rot_dim, vdim, kv_rank, q_rank, window;
  int rot_dims;      // the first rot_dims of the rot_dim rotated dims turn ("rotate half": i pairs with i + rot_dims / 2)
  float scale;
  int interleaved;   // != 0: the rotated entries pair as (2i, 2i + 1) instead of (i, i + rot_dims / 2)
  const float* sink; // fp32 [heads] or nullptr: the softmax denominator of head h also holds exp(sink[h]): a term of the
                     // normaliser alone -- nothing is summed for it and the score scale does not apply to it
  __host__ __device__ int row() const { return kv_rank + rot_dim; }   // cache row / absorbed query length
};
// y [T, ldy] fp32 = the fused down-projection [q latent (q_rank) | kv latent (kv_rank) | k_rot (rot_dim) | gate (heads)]:
//   cq[t]    = rmsnorm(q latent) * w_q            -> DT_* [T, q_rank]
//   cache[slot[t]] = [rmsnorm(kv latent) * w_kv | rotary(k_rot, pos[t])]   (slot < 0: not cached)
//   gate[t]  = sigmoid(gate logits)               -> fp32 [T, heads]       (heads_gate == 0: no gate columns)
// cos_sin: fp32 [max_pos][rot_dims] = cos (rot_dims / 2) | sin (rot_dims / 2)
cudaError_t latent_prep_launch(const float* y, int ldy, const LatentGeom& g, const float* w_q, const float* w_kv, float eps,
                               const int32_t* positions, const int32_t* slot_mapping, const float* cos_sin, void* cq,
                               void* cache, int dtype, float* gate, int T, cudaStream_t stream);
// q [T, heads * (dim + rot_dim)] DT_* -> q_abs[t, h, kv_rank ..] = rotary(q_rot_h, pos[t])   (the first kv_rank entries of
// every head are written by the absorbing batched product)
cudaError_t latent_q_rope_launch(const void* q, int q_dtype, const LatentGeom& g, const int32_t* positions,
                                 const float* cos_sin, float* q_abs, int T, cudaStream_t stream);
struct LatentTile {  // one CTA's queries: tokens [q0, q0 + nq) of the step's sequence `seq` (device array)
  int32_t seq, q0, nq, pad;
};
constexpr int LATENT_PAIRS = 16;  // (token, head) pairs per CTA
inline int latent_tile_tokens(int heads) { return heads >= LATENT_PAIRS ? 1 : LATENT_PAIRS / heads; }
// q_abs fp32 [T, heads, row()], cache DT_* [num_blocks][KV_BLOCK][row()], o_lat DT_* [T, heads, kv_rank]
// split_ws (optional, fp32): with it, steps of few tiles cut every tile's keys into fixed splits of LATENT_SPLIT_BLOCKS cache
// blocks that run as CTAs of their own and are merged by a second kernel; max_kv_len: the longest sequence of the step
constexpr int LATENT_SPLIT_BLOCKS = 4;
cudaError_t latent_attn_launch(const float* q_abs, const void* cache, int dtype, const AttnSeq* seqs,
                               const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                               void* o_lat, int o_dtype, const LatentGeom& g, cudaStream_t stream, float* split_ws = nullptr,
                               size_t split_ws_floats = 0, int max_kv_len = 0, int num_sms = 148, int* n_launched = nullptr);

// ---- attention_capped.cu: grouped-query attention with normed queries / keys and a soft cap on the scores ------------
// No rotation: positions enter through the causal mask and a query temperature.  Per head: q <- rmsnorm(q) * w_q *
// (1 + qt_coef * ln(floor((pos + 1) / qt_every) + 1)), k <- rmsnorm(k) * w_k (one weight of `dim` entries for all heads);
// score = scale * q . k, then softcap * tanh(score / softcap) (softcap <= 0: none); softmax over the keys j <= i; query head h
// reads key/value head h / (heads / kv_heads); the heads' outputs are multiplied by sigmoid(gate logits).
struct CapAttnGeom {
  int heads, kv_heads, dim, vdim;
  float scale, softcap, qt_coef;
  int qt_every;      // <= 0: no query temperature
};
constexpr int CAPATTN_TILE = 16;      // query tokens per CTA
constexpr int CAPATTN_MAX_VDIM = 512; // value columns per head the kernel's accumulators cover
// y fp32 [T, ldy] holds q at column q_off (heads * dim), k at k_off (kv_heads * dim), v at v_off (kv_heads * vdim):
//   q_out DT_* [T, heads * dim]; cache rows K [num_blocks][KV_BLOCK][kv_heads * dim], V [..][kv_heads * vdim] at slot[t]
cudaError_t capattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const CapAttnGeom& g,
                                const float* w_q, const float* w_k, float eps, const int32_t* positions,
                                const int32_t* slot_mapping, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                cudaStream_t stream);
// out DT_* [T, heads * vdim] = softmax(.) V * sigmoid(gate[t * gate_ld + h * vdim + c])   (gate == nullptr: no gate)
cudaError_t capattn_launch(const void* q, const void* k_cache, const void* v_cache, int dtype, const AttnSeq* seqs,
                           const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                           const float* gate, int gate_ld, void* out, int out_dtype, const CapAttnGeom& g,
                           cudaStream_t stream);

// ---- attention_sigmoid.cu: grouped-query attention with rotary positions, a window, and sigmoid weights -------------------
// weight(i, j) = sigmoid(scale * q_h(i) . k_g(j) + head_bias[h]) for 0 <= i - j < window (window <= 0: every earlier position),
// o_h(i) = sum_j weight(i, j) v_g(j): nothing is normalised over the keys.  Query head h reads key/value head h / (heads / kv_heads).
struct SigAttnGeom {
  int heads, kv_heads, dim, vdim, window;
  int rot_dims;      // the first rot_dims entries of every query / key head turn ("rotate half": i pairs with i + rot_dims / 2)
  float scale;
};
constexpr int SIGATTN_TILE = 16;      // query tokens per CTA
constexpr int SIGATTN_MAX_VDIM = 512; // value columns per head the FMA kernel's accumulators cover
// y fp32 [T, ldy] holds q at column q_off (heads * dim), k at k_off (kv_heads * dim), v at v_off (kv_heads * vdim); k_off < 0:
// the layer reads another layer's cache rows and only q is produced.  cos_sin fp32 [max_pos][rot_dims] = cos | sin (the
// host folds any frequency scaling and magnitude in).  q_out DT_* [T, heads * dim]; cache rows as in attention_capped.cu.
cudaError_t sigattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const SigAttnGeom& g,
                                const float* cos_sin, const int32_t* positions, const int32_t* slot_mapping, void* q_out,
                                void* k_cache, void* v_cache, int dtype, int T, cudaStream_t stream);
// out DT_* [T, heads * vdim]; head_bias fp32 [heads] (nullptr: zeros)
cudaError_t sigattn_launch(const void* q, const void* k_cache, const void* v_cache, int dtype, const AttnSeq* seqs,
                           const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                           const float* head_bias, void* out, int out_dtype, const SigAttnGeom& g, cudaStream_t stream);

// ---- attention_pooled.cu: grouped-query softmax attention over a sliding window plus pooled blocks of what left it -----
// Per head: rotary turn of the first rot_dims entries of every query and key ("rotate half": i pairs with i + rot_dims / 2),
// then (unit_norm != 0) q and k divided by their root mean square over dim; score = scale * q . k.  Query i sees the tokens j
// with 0 <= i - j < window one by one and, with pool > 0, every block b of `pool` consecutive positions that ends at or
// before i - window (b * pool + pool - 1 <= i - window) through ONE key and ONE value: the means of the block's cached
// keys and of its values.  Tokens behind the window whose block is not complete by then are not seen.  The softmax runs
// over window tokens and visible blocks together.  window <= 0: every earlier position, no blocks.  Query head h reads key/value head h / (heads / kv_heads).
struct PoolAttnGeom {
  int heads, kv_heads, dim, vdim, window, pool;
  int rot_dims;
  float scale;
  int unit_norm;
  __host__ __device__ int rows_per_page() const { return pool > 0 ? (KV_BLOCK + pool - 1) / pool : 0; }   // pooled rows a cache page owns
};
constexpr int POOLATTN_TILE = 16;      // query tokens per CTA
constexpr int POOLATTN_MAX_VDIM = 512; // value columns per head the FMA kernel's accumulators cover
// y fp32 [T, ldy] holds q at column q_off (heads * dim), k at k_off (kv_heads * dim), v at v_off (kv_heads * vdim); bias fp32
// (q | k | v, in that order, or nullptr) is added first.  cos_sin fp32 [max_pos][rot_dims] = cos | sin.  q_out DT_* [T, heads * dim];
// cache rows K [num_blocks][KV_BLOCK][kv_heads * dim], V [..][kv_heads * vdim] at slot[t].
cudaError_t poolattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const float* bias,
                                 const PoolAttnGeom& g, const float* cos_sin, float eps, const int32_t* positions,
                                 const int32_t* slot_mapping, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                 cudaStream_t stream);
// The blocks that this step's tokens complete: pooled row b = mean over the block's rows as the cache holds them (fp32 sum
// in position order).  Block b of a sequence lives in the page of its FIRST token, page p = b * pool / KV_BLOCK, at index
// b - ceil(p * KV_BLOCK / pool): pk [num_blocks][rows_per_page()][kv_heads * dim], pv [..][kv_heads * vdim], DT_*.
cudaError_t poolattn_pool_launch(const void* k_cache, const void* v_cache, void* pk, void* pv, int dtype,
                                 const AttnSeq* seqs, int n_seqs, const int32_t* block_table, int bt_stride,
                                 const PoolAttnGeom& g, int max_q_len, cudaStream_t stream);
// out DT_* [T, heads * vdim]
cudaError_t poolattn_launch(const void* q, const void* k_cache, const void* v_cache, const void* pk, const void* pv, int dtype,
                            const AttnSeq* seqs, const LatentTile* tiles, int n_tiles, const int32_t* block_table,
                            int bt_stride, void* out, int out_dtype, const PoolAttnGeom& g, cudaStream_t stream);

// ---- recurrent.cu: mixers that carry a state from token to token ----------------------------------------------------
// Every sequence owns one state slot per layer (the engine's sequence slot).  A kernel reads the slot's state for the first
// token of a portion unless that token's position is 0 (then the state is zero: a slot needs no clearing when it is handed
// to a new sequence), walks the portion's tokens in order and leaves the state after the last one.  tok_slot[t] is the
// slot of token t; consecutive tokens of one slot are consecutive positions of one sequence.
// out[s][t] = x[t] + (prev(t) - x[t]) * mu[s]    s < n_mix; prev(t) = x[t - 1], the slot's saved row, or zeros at position 0
cudaError_t token_shift_mix_launch(const float* x, int width, const float* mu, int n_mix, const int32_t* positions,
                                   const int32_t* tok_slot, const float* prev_state, void* out, int out_dtype,
                                   long long out_bs, int T, cudaStream_t stream);
// out[t, c] = silu(b[c] + sum_j w[c, taps - 1 - j] * x(t - j, c)),  x = xz[:, :inner]; tokens before the portion come from
// conv_state [slots][taps - 1][inner] (entry e: position first - (taps - 1) + e), positions < 0 are zeros
cudaError_t short_conv_silu_launch(const float* xz, int ld, int inner, const float* w, const float* b, int taps,
                                   const int32_t* positions, const int32_t* tok_slot, const float* conv_state,
                                   float* out_f32, void* out_op, int out_dtype, int T, cudaStream_t stream);
// Selective scan, one thread per channel:  dt = softplus(dt_raw + dt_b);  S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x_c B_n;
// y_c = S[c] . C + D_c x_c;  out = y * silu(z)   (A = -exp(A_log)).  Also moves the convolution's tail forward.
struct SelScan {
  const float* x;        // fp32 [T, inner] after convolution and silu
  const float* xz; int ld_xz;   // in-projection [T, 2 inner]: the convolution's inputs and z
  const float* proj; int ld_proj; int dt_rank;  // [dt (dt_rank) | B (state) | C (state)]
  const float* dt_raw;   // fp32 [T, inner]
  const float *dt_b, *A_log, *D;
  float* S;              // [slots][inner][state]
  float* conv_state;     // [slots][taps - 1][inner]
  void* out; int out_dtype;
  int inner, state, taps;
};
constexpr int SELSCAN_MAX_STATE = 128;
cudaError_t selective_scan_launch(const SelScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                                  cudaStream_t stream);
// Outer-product memories, per head a matrix S [dim, vdim] (fp32), the CTAs of one head split the value columns:
//   OUTER_SCAN_DECAY:  o = (S + diag(u) k v^T)^T q;  S <- diag(w) S + k v^T,  w = exp(-exp(decay_raw + w0))
//   OUTER_SCAN_GATED:  i = cap tanh((ig + b_i) / cap), f = logsigmoid(cap tanh((fg + b_f) / cap)), m' = max(f + m, i),
//                      S <- e^(f + m - m') S + e^(i - m') k v^T, n likewise with k;  o = S^T q / (max(|n . q|, e^-m') + 1e-6)
//   OUTER_SCAN_SSD:    dt = softplus(step_raw + step_b), S <- exp(-exp(A_log_h) dt) S + dt k v^T;  o = S^T q + D_h v
//                      (one decay per head and token; the query reads the state after the token's update; q / k heads may be
//                      shared by groups of heads: qk_heads)
//   OUTER_SCAN_HGRN:   f = l + (1 - l) sigmoid(decay_raw + w0), l = u (a lower bound per head and key channel);
//                      S <- diag(f) S + (1 - f) v^T;  o = S^T silu(q)   (no key: what the gate forgets is what it writes; the
//                      query reads the state after the token's update)
constexpr int OUTER_SCAN_DECAY = 0, OUTER_SCAN_GATED = 1, OUTER_SCAN_SSD = 2, OUTER_SCAN_HGRN = 3;
constexpr int OUTER_SCAN_MAX_DIM = 256;
struct OuterScan {
  int mode;
  const float *q, *k, *v; int ldq, ldk, ldv;   // fp32 [T, heads * dim] / [T, heads * vdim]
  float q_scale;
  const float* decay_raw; int ldd; const float* w0; const float* u;   // DECAY: [T, heads * dim], [heads * dim], [heads * dim]
  const float *ig, *fg; int ldg; const float *ig_b, *fg_b; float gate_cap;  // GATED: [T, heads], biases [heads]
  float *S, *n, *m;      // state [slots][heads][dim][vdim], [slots][heads][dim], [slots][heads]
  float* out; int ldo;   // fp32 [T, heads * vdim]
  int heads, dim, vdim;
  const float* x; float* x_last; int width;   // optional: x_last[slot] = x[last row of the portion] (the token shift's state)
  int qk_heads;                                // q / k heads (head h reads h / (heads / qk_heads)); 0: one per head
  const float* step_raw; int lds; const float *step_b, *A_log, *D;   // SSD: [T, heads], [heads], [heads], [heads]
};
cudaError_t outer_scan_launch(const OuterScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                              cudaStream_t stream);
// out[t, h, :] = rmsnorm(o[t, h, :]) * w[h, :] * act(gate[t, h, :])    act: 0 sigmoid, 1 silu, 2 none (gate may be nullptr)
// gate_first != 0: out[t, h, :] = rmsnorm(o[t, h, :] * act(gate[t, h, :])) * w[h, :]   (the gate enters the norm)
cudaError_t head_norm_gate_launch(const float* o, int ldo, int heads, int vdim, const float* w, const float* gate,
                                  int ldg, int act, float eps, void* out, int out_dtype, int T, cudaStream_t stream,
                                  int gate_first = 0);
// The short convolution's state after a step: conv_state[slot][e][c] = input at position end - (taps - 1) + e, taken from the
// step's rows x [T, ld] (channels c < n) or, for positions before the portion, from the old state.  Runs after the
// convolution that read the old state.
cudaError_t conv_state_save_launch(const float* x, int ld, int n, int taps, const AttnSeq* seqs, int n_seqs,
                                   const int32_t* tok_slot, float* conv_state, cudaStream_t stream);
// Gated delta rule with one decay per key channel, per head a matrix S [dim, vdim] (fp32):
//   q <- q / sqrt(sum q^2 + 1e-6) * dim^-1/2,  k <- k / sqrt(sum k^2 + 1e-6)   (per q / k head; head h reads h / (heads / qk_heads))
//   g = exp(-exp(A_log_h) * softplus(decay_raw + decay_b))   [dim];   beta = sigmoid(beta_raw)
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
struct DeltaScan {
  const float *q, *k, *v; int ldq, ldk, ldv;   // fp32 [T, qk_heads * dim] / [T, heads * vdim]
  const float* decay_raw; int ldd; const float* decay_b; const float* A_log;   // [T, heads * dim], [heads * dim], [heads]
  const float* beta_raw; int ldb;              // [T, heads]
  float* S;                                    // [slots][heads][dim][vdim]
  float* out; int ldo;                         // fp32 [T, heads * vdim]
  int heads, qk_heads, dim, vdim;
};
constexpr int DELTA_SCAN_MAX_DIM = 256;
cudaError_t delta_scan_launch(const DeltaScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                              cudaStream_t stream);
// out[i] = x[i] in the operand type
cudaError_t convert_f32_launch(const float* x, void* out, int out_dtype, size_t n, cudaStream_t stream);

// ---- moe.cu: top-k router and the bookkeeping of the grouped expert products ----------------------------------------
// logits fp32 [T, ld] (columns [0, E): experts; column E, when side_gate != nullptr: the shared expert's gate logit):
//   ids[t, k], w[t, k] = the `top` largest of logits + bias and the softmax over just those;  side_gate[t] = sigmoid(.)
// weight_mode MOE_W_SIGMOID: w[t, k] = sigmoid(logit) of each chosen expert, used as it is
constexpr int MOE_W_SOFTMAX = 0, MOE_W_SIGMOID = 1;
cudaError_t moe_route_launch(const float* logits, int ld, const float* bias, int E, int top, int32_t* ids, float* w,
                             float* side_gate, int T, cudaStream_t stream, int weight_mode = MOE_W_SOFTMAX);
// seg_off[E + 1]: rows per expert, prefix-summed; order[p] = t * top + k of the p-th row; inv[t * top + k] = p
cudaError_t moe_align_launch(const int32_t* ids, int T, int top, int E, int32_t* seg_off, int32_t* order, int32_t* inv,
                             cudaStream_t stream);

// ---- sampler.cu --------------------------------------------------------------------------------------------------
constexpr int MAX_TOPN = 12;  // reference forces max_logprobs >= 11 (tgis_utils/args.py:214-216)
struct SampleRow {            // per sampled row parameters (device array, 64 B)
  int32_t flags;              // bit0 greedy, bit1 want_logprobs, bit2 typical, bit3 len_penalty, bit4 seeded
  int32_t n_topn;             // number of top-n entries to return (0..MAX_TOPN)
  float temperature;
  int32_t top_k;              // <=0: off
  float top_p;                // >=1: off
  float typical_p;
  float rep_penalty;          // 1.0: off
  float len_decay_factor;     // decay ** max(0, n_out - start)  precomputed on host in double, cast to fp32
  int32_t eos_id;
  int32_t n_out;              // tokens generated so far
  int32_t min_tokens;
  int32_t seq_slot;           // row of the seen-token bitmap
  uint32_t seed_lo, seed_hi;  // philox key
  uint32_t step;              // philox counter offset
  int32_t logits_row;         // row in the logits matrix
};
struct SampleOut {            // per row result (pinned host readable)
  int32_t token;
  float logprob;
  int32_t rank;
  int32_t n_topn;
  int32_t topn_ids[MAX_TOPN];
  float topn_lps[MAX_TOPN];
};
constexpr int SAMPLE_GREEDY = 1, SAMPLE_LOGPROBS = 2, SAMPLE_TYPICAL = 4, SAMPLE_LENPEN = 8, SAMPLE_SEEDED = 16;
constexpr int SAMPLE_MASKED = 64;  // guided decoding: row seq_slot of the allow bitmap holds this step's allowed-token bits
constexpr int SAMPLE_FORCED = 32;  // token = seed_lo is given (prompt logprobs): report its logprob / rank / top-n only
// logits: [rows, ld] bf16 (logits_bf16 = 1: the lm_head GEMM's model-dtype output, what vLLM's sampler sees after its
// fp32 cast) or fp32 (kernel-level golden tests).  any_complex: some row needs selection passes (sampling rows: typical-p /
// top-k / top-p / race) -> 8 CTAs per row; otherwise the cluster size shrinks with the row count (sampler_cluster_size).
cudaError_t sampler_launch(const void* logits, int logits_bf16, int ld, int vocab, const SampleRow* rows, int n_rows,
                           const uint32_t* seen_bitmap, int bitmap_words, float* scratch, SampleOut* out,
                           cudaStream_t stream, int any_complex = 1, int num_sms = 148,
                           const uint32_t* allow_bitmap = nullptr /* [slots][bitmap_words], rows flagged SAMPLE_MASKED */);
int sampler_cluster_size(int n_rows, int any_complex, int num_sms);
// seen-token bitmap maintenance
cudaError_t bitmap_clear_launch(uint32_t* bitmap, int bitmap_words, int slot, cudaStream_t stream);
cudaError_t bitmap_set_launch(uint32_t* bitmap, int bitmap_words, const int32_t* slots, const int32_t* tokens, int n,
                              cudaStream_t stream);
size_t sampler_scratch_floats(int vocab);

}  // namespace tgis
