// libtgis_engine.so — continuous-batching engine + C ABI (include/tgis_engine.h).
//
// This is the B200-native replacement for what sits behind `self.engine.generate(...)`
// (/root/reference/src/vllm_tgis_adapter/grpc/grpc_server.py:222): vLLM's EngineCore busy loop, scheduler,
// KV block manager, GPUModelRunner and Sampler (SURVEY.md §2.2 K1-K15, §3.2 "THE HOT LOOP").
//
//   host side (this file, C++): request queues, paged-KV block allocator, continuous-batching scheduler with chunked
//       prefill + recompute preemption, stop checks (vllm v1/core/sched/utils.py:94-130), output ring.
//   device side: one flat token batch per step -> Llama layer stack built from the sm_100a kernels in this directory.
//       All per-step metadata is packed into ONE pinned staging buffer and shipped with ONE H2D copy; results come
//       back with ONE D2H copy of SampleOut records.
#include <algorithm>
#include <set>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <random>
#include <stdexcept>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include <dlfcn.h>
#include <errno.h>
#include <signal.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <nccl.h>
#include <sys/mman.h>
#include <unistd.h>

#include "../../include/tgis_engine.h"
#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace {

thread_local std::string g_last_error;
int fail(const std::string& msg, int code = -1) {
  g_last_error = msg;
  return code;
}
double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

struct CudaError : std::runtime_error {
  using std::runtime_error::runtime_error;
};
// NCCL is resolved at run time (dlopen) and only when tp_size > 1: a hard link-time dependency would pin whichever
// libnccl.so.2 the loader finds first and can break a later `import torch` (torch 2.11 needs 2.28 symbols) when this
// library is loaded before torch.  dlopen by SONAME returns torch's already-loaded copy when there is one.
struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};
NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    auto sym = [&](const char* n) { return dlsym(h, n); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.AllReduce && api.AllGather && api.CommDestroy && api.GetErrorString;
  });
  if (!api.ok) throw CudaError("libnccl.so.2 could not be loaded (needed for tp_size > 1)");
  return api;
}
#define NK(expr)                                                                                        \
  do {                                                                                                  \
    ncclResult_t _r = (expr);                                                                           \
    if (_r != ncclSuccess)                                                                              \
      throw CudaError(std::string(#expr) + " failed: " + nccl().GetErrorString(_r));                       \
  } while (0)
#define CK(expr)                                                                                        \
  do {                                                                                                  \
    cudaError_t _e = (expr);                                                                            \
    if (_e != cudaSuccess)                                                                              \
      throw CudaError(std::string(#expr) + " failed: " + cudaGetErrorString(_e) + " (" __FILE__ ":" +   \
                      std::to_string(__LINE__) + ")");                                                  \
  } while (0)

using bf16 = __nv_bfloat16;
using namespace tgis;

struct Request {
  std::string id;
  std::vector<int32_t> tokens;  // prompt + generated
  int n_prompt = 0;
  int n_computed = 0;  // tokens whose K/V are in the cache
  tgis_sampling_params sp{};
  int slot = -1;
  std::vector<int32_t> blocks;
  bool aborted = false;
  uint64_t seed = 0;
  int guided_fed = 0;  // generated tokens already reported to the mask provider (guided decoding)
  double ts_arrival = 0, ts_first_sched = 0, ts_first_token = 0, ts_last_token = 0;
  int n_out() const { return (int)tokens.size() - n_prompt; }
};

struct Sched {  // one scheduled sequence of the current step
  Request* r;
  int q_len;
  bool sample;
};

template <class T>
struct DevBuf {
  T* p = nullptr;
  size_t n = 0;
  void alloc(size_t count) {
    n = count;
    CK(cudaMalloc(&p, std::max<size_t>(count, 1) * sizeof(T)));
  }
  void zero() { CK(cudaMemset(p, 0, n * sizeof(T))); }
  ~DevBuf() {
    if (p) cudaFree(p);
  }
};

struct LayerW {
  bf16 *wqkv, *wo, *wgu, *wd, *ln1, *ln2;
  // OPT only (tgis_config.arch == TGIS_ARCH_OPT): wgu holds fc1 [ffn, hidden] (not interleaved), wd holds fc2; biases of
  // the four projections (q/k/v concatenated, head-padded like wqkv) and of the two LayerNorms
  bf16 *b_qkv = nullptr, *b_o = nullptr, *b_fc1 = nullptr, *b_fc2 = nullptr, *ln1_b = nullptr, *ln2_b = nullptr;
  CUtensorMap m_qkv, m_o, m_gu, m_d;
};

// Tensor-parallel step plan, shared by POSIX shm between the ranks of one node: rank 0 (scheduler) publishes the
// packed staging buffer + launch header of every step; workers spin on `seq`, copy, acknowledge and launch the same
// kernel sequence on their shard.  (The data path itself only exchanges through NCCL.)
struct StepHeader {
  int32_t T, n_dec, n_tiles, R, max_dec_kv, S;
  int32_t graphable;     // replay (or capture) the CUDA graph keyed by (S, KV splits, samp_complex) instead of launching
  int32_t samp_complex;  // bit 0: some sampled row needs selection passes (sampling): decides the sampler's cluster
                         // size; bit 1: some row carries a guided-decoding bitmask (the masked sampler instantiation);
                         // bit 2: some token carries a LoRA adapter (unfused projections + lora.cu kernels)
  uint64_t copy_bytes;
  int32_t kind;          // 0: engine step; 1: prompt-logprob pass over R rows of the step just executed (T = its tokens,
  int32_t need_norm;     //    need_norm: the final RMSNorm has not run yet)
  int32_t lg_idx;        // index of this plan's logits gather inside the step (epoch = staged base + lg_idx)
  int32_t pad;
};
struct ShmCtl {
  std::atomic<uint64_t> seq;
  std::atomic<uint32_t> shutdown;
  uint32_t pad;
  std::atomic<uint64_t> ack[16];
  std::atomic<int32_t> pid[16];      // liveness: every rank publishes its process id
  std::atomic<int32_t> failed[16];   // a worker that hit an error says so before it leaves
  StepHeader hdr;
  // followed by stage bytes (256-B aligned)
};
static_assert(sizeof(ShmCtl) <= 1024, "ShmCtl must fit below SHM_STAGE_OFF");
constexpr size_t SHM_STAGE_OFF = 1024;

// gathered: [tp][R][Vl] -> out: [R][tp*Vl], elements of `esz` bytes moved as 16-byte vectors (Vl * esz % 16 == 0)
__global__ void gather_relayout_kernel(const uint4* __restrict__ gathered, uint4* __restrict__ out, int R, int Vl16,
                                       int tp) {
  griddep_launch();
  griddep_wait();
  const size_t total = (size_t)tp * R * Vl16;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int rk = (int)(i / ((size_t)R * Vl16));
    const size_t rem = i % ((size_t)R * Vl16);
    const int r = (int)(rem / Vl16), v = (int)(rem % Vl16);
    out[(size_t)r * tp * Vl16 + (size_t)rk * Vl16 + v] = gathered[i];
  }
}

constexpr int N_BT = 5;
const int BT_VALUES[N_BT] = {16, 32, 64, 128, 256};
int bt_index(int T) {
  int bt = gemm_pick_bt(T);
  for (int i = 0; i < N_BT; ++i)
    if (BT_VALUES[i] == bt) return i;
  return N_BT - 1;
}

}  // namespace

struct tgis_engine {
  tgis_config cfg{};
  int num_sms = 148;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int q_dim = 0, qkv_dim = 0, bt_stride = 0, max_splits_cap = 0, bitmap_words = 0;
  // tensor parallelism: local (per-rank) head / ffn / vocab-shard sizes
  int tp = 1, rank = 0, nq = 0, nkv = 0, Fl = 0, Vl = 0;
  ncclComm_t comm = nullptr;
  ShmCtl* shm = nullptr;
  size_t shm_bytes = 0;
  bool shm_owner = false;
  std::string shm_name;
  uint64_t plan_seq = 0;
  double tp_timeout_s = 120.0;  // TGIS_TP_TIMEOUT_S: a worker that takes no plan for this long is declared hung
  DevBuf<uint8_t> logits_shard, logits_gather;  // [R, V/tp] and [tp][R, V/tp] in the logits dtype
  int T_max = 0, S_max = 0, tiles_max = 0;

  // weights
  DevBuf<bf16> w_arena;
  bf16 *embed = nullptr, *lm_head = nullptr, *final_norm = nullptr, *cos_sin = nullptr;
  bool lm_head_loaded = false, cos_sin_loaded = false;
  // OPT (opt.cu): learned positions [max_model_len + 2, hidden], final LayerNorm bias; model head dim (64 or 128: every
  // head is zero-padded to the 128-dim attention tiles at load time); fp32 GEMM accumulators of the biased projections
  bool opt = false;
  bf16 *pos_embed = nullptr, *final_norm_b = nullptr;
  int pos_rows = 0, model_head_dim = HEAD_DIM;
  float attn_scale = 0.f;
  DevBuf<float> y32;
  std::set<std::string> opt_loaded;  // tensor names seen by load_weight_opt (completeness check at start)
  std::vector<LayerW> layers;
  CUtensorMap m_lm{};
  // ---- layer-list architectures (TGIS_ARCH_PONENEX, TGIS_ARCH_FALERAX): per-layer geometry, weights, caches and the fp32-residual buffers
  bool pnx_on = false;
  tgis_model_spec pnx_spec{};
  std::vector<tgis_layer_spec> pnx_layer_specs;
  struct PnxLayer {
    tgis_layer_spec sp{};
    LatentGeom g{};
    void *w_down = nullptr, *w_uq = nullptr, *w_ukT = nullptr, *w_uv = nullptr, *w_o = nullptr;   // operand type
    float *norm1 = nullptr, *norm1b = nullptr, *norm2 = nullptr, *norm2b = nullptr, *qnorm = nullptr, *kvnorm = nullptr;
    const float* cos_sin = nullptr;  // [max_model_len][rot_dims]
    void* cache = nullptr;           // [num_blocks][KV_BLOCK][kv_rank + rot_dim], operand type
    void *w_router = nullptr, *w_gu_e = nullptr, *w_d_e = nullptr, *w_gu_s = nullptr, *w_d_s = nullptr;
    float* router_b = nullptr;
    int n_down() const { return sp.q_rank + sp.kv_rank + sp.rot_dim + (out_gate ? sp.heads : 0); }
    // ---- mixers with state slots and the dense feed-forward (TGIS_ARCH_FALERAX)
    void* w_in = nullptr;             // every projection that reads the mixer input, stacked ([in_cols, width], operand type)
    int in_cols = 0;                  // ... rounded up to a multiple of 8 (zero rows)
    // TGIS_MIXER_PARALLEL: columns of the stacked projection, the attention's paged caches, both sides' small weights
    CapAttnGeom ca{};
    int c_q = 0, c_k = 0, c_v = 0, c_g = 0, c_mq = 0, c_mk = 0, c_mv = 0, c_mg = 0, c_mi = 0, c_mf = 0;
    void *k_cache = nullptr, *v_cache = nullptr;   // [num_blocks][KV_BLOCK][kv_heads * dim | vdim], operand type
    void* w_o2 = nullptr;                          // the matrix memory's output projection
    float *qk_norm = nullptr, *mm_norm = nullptr, *mm_bias = nullptr, *out_l = nullptr, *out_r = nullptr;
    float *st_S = nullptr, *st_n = nullptr, *st_m = nullptr;   // per sequence slot: matrix, normaliser, running maximum
    // TGIS_MIXER_SELECTIVE_SCAN
    void *w_x = nullptr, *w_dt = nullptr;
    float *conv_w = nullptr, *conv_b = nullptr, *dt_b = nullptr, *A_log = nullptr, *Dv = nullptr, *st_conv = nullptr;
    // TGIS_MIXER_WKV (w_in: r | k | v | g, each reading its own mix)
    void *w_w1 = nullptr, *w_w2 = nullptr;
    float *mu = nullptr, *w0 = nullptr, *u = nullptr, *st_prev = nullptr;
    // TGIS_MLP_DENSE_GELU: gate / up rows interleaved, down
    void *w_gu = nullptr, *w_d = nullptr;
    // ---- layers of the parallel gated style (TGIS_ARCH_REVEPEL): one norm, token shift, per-channel gates on both sublayers
    void* w_gates = nullptr;          // [gates_cols, width]: mixer gate | feed-forward gate | router rows (operand type)
    int gates_cols = 0;               // 2 width + experts, rounded up to a multiple of 8 (zero rows)
    float *gate_b = nullptr, *shift = nullptr;   // [2 width] gate biases; [width] token-shift blend (st_prev: the previous normed row)
    // TGIS_MIXER_SIGMOID_ATTENTION (w_in: q | k | v, or q alone when the layer reads another layer's cache rows)
    SigAttnGeom sa{};
    float* head_bias = nullptr;
    int kv_src = -1;                  // layer whose k_cache / v_cache this layer reads (-1: its own)
    // TGIS_MIXER_SSD (w_in as stored: z | x | B | C | dt) and TGIS_MIXER_CHANNEL_DELTA (w_in: q | k | v | beta | decay rank | gate rank)
    int conv_ch = 0, c_b = 0, c_a1 = 0, c_g1 = 0;
    void* w_g2 = nullptr;             // channel delta: output-gate up-projection (w_w2: the decay's)
    // ---- layers of the parallel pair style (TGIS_ARCH_SIKAZEN): two one-number norms (kept as rows of `width` equal entries),
    // mixer and dense feed-forward side by side, then the per-layer token input
    PoolAttnGeom pa{};                // TGIS_MIXER_POOLED_ATTENTION (w_in: q | k | v; k_cache / v_cache as above)
    void *pk_cache = nullptr, *pv_cache = nullptr;   // pooled rows [num_blocks][rows_per_page][kv_heads * dim | vdim], operand type
    float *in_bias = nullptr, *sink = nullptr;       // [in_cols] projection biases; [heads] softmax sinks
    bool out_gate = true;             // latent attention: sigmoid output gate per head (its logits ride in w_down)
    void *w_sg = nullptr, *w_sp = nullptr;           // token input: gate [side_dim, width], projection [width, side_dim]
    float* side_norm = nullptr;
    int weights_of = -1;              // the layer of the checkpoint whose weights this run uses
    bool add_x0 = false;              // the embedding output is added to the stream right before this run
    int c_f = 0;                      // TGIS_MIXER_HGRN (w_in: q | f | v): column of the gate logits
  };
  std::vector<PnxLayer> pair_runs;    // parallel pair style: one entry per layer RUN (a looped span repeats), weights shared
  bool pair_style = false;            // TGIS_STYLE_PARALLEL_PAIR
  void *pnx_side = nullptr, *pnx_hB = nullptr;       // side table [vocab, n_layers * side_dim]; norm2's rows (operand type)
  float* pnx_x0 = nullptr;                           // the embedding output, kept for the passes of a loop
  int step_max_q = 0;                                // longest portion of the step
  // the feed-forward of a parallel pair layer reads the same stream as the mixer: its two products run on a second stream
  // beside the mixer's kernels (fork after the tail that leaves both normed inputs, join before the tail that adds both
  // outputs), with a product workspace of their own.  TGIS_PAIR_OVERLAP=0: one stream
  cudaStream_t stream2 = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  DevBuf<float> gemm_ws2;
  DevBuf<int> gemm_counters2;
  bool pair_overlap = true, on_side_stream = false;
  size_t off_ltiles16 = 0;                           // query tiles of POOLATTN_TILE tokens (the latent attention's are smaller)
  int step_n_ltiles16 = 0;
  std::vector<PnxLayer> pnx_layers;
  std::vector<void*> pnx_allocs;                     // everything pnx_alloc handed out
  std::vector<std::pair<std::vector<float>, float*>> pnx_rope_tables;  // (base, dims, scaling) -> table
  std::set<std::string> pnx_loaded;
  size_t pnx_expected_tensors = 0;
  int pnx_dt = DT_BF16;                              // operand type of weights / matrix-product inputs / cache rows
  void *pnx_embed = nullptr, *pnx_head = nullptr, *pnx_hA = nullptr, *pnx_cq = nullptr, *pnx_oA = nullptr, *pnx_actS = nullptr,
       *pnx_actE = nullptr, *pnx_last = nullptr;
  void *pnx_q = nullptr, *pnx_olat = nullptr;  // operand type: they feed the per-head products
  bool post_norm = false, tied_head = false;   // TGIS_STYLE_*
  float *flx_f1 = nullptr, *flx_f2 = nullptr, *flx_f3 = nullptr;   // fp32 scratch of the recurrent mixers
  bool gated_style = false;                                        // TGIS_STYLE_PARALLEL_GATED
  float* rvp_n[2] = {nullptr, nullptr};                            // fp32 normed rows of the current / the next layer
  void *flx_op2 = nullptr, *flx_mix = nullptr;                     // operand-type scratch: gated memory output, token-shift mixes
  float *pnx_final_norm = nullptr, *pnx_resid = nullptr, *pnx_y1 = nullptr, *pnx_gate = nullptr,
        *pnx_qabs = nullptr, *pnx_o = nullptr, *pnx_rl = nullptr, *pnx_mixw = nullptr, *pnx_sgate = nullptr,
        *pnx_yS = nullptr, *pnx_yE = nullptr;
  int32_t *pnx_ids = nullptr, *pnx_segoff = nullptr, *pnx_order = nullptr, *pnx_inv = nullptr;
  int pnx_tile_tokens = 1, step_n_ltiles = 0, step_max_kv = 0;
  float* pnx_attn_ws = nullptr;                      // split partials of decode-shaped attention launches
  size_t pnx_attn_ws_floats = 0;
  size_t off_ltiles = 0;
  int logit_rows_cap = 0;                            // rows of the logits buffer (>= max_num_seqs)
  int logits_ld = 0;                                 // its row length: the vocabulary rounded up to the sampler's 8-column
                                                     // vectors; the padding columns hold -inf for good
  std::string pnx_dump_path;                         // TGIS_DUMP_RESID: append the residual stream after every layer (debug)
  // kv cache
  DevBuf<bf16> k_cache, v_cache;
  size_t kv_layer_elems = 0;
  int num_blocks = 0;
  std::vector<int32_t> free_blocks;
  // activations
  DevBuf<bf16> resid, xn, qkv, attn_out, tmp, act, last_hidden;
  // lm_head output [rows, V].  bf16 = the model dtype, rounded once from the fp32 accumulator exactly where vLLM's
  // lm_head rounds (vllm model_executor/layers/logits_processor.py:89-104 -> F.linear in bf16; the sampler then casts to
  // fp32, v1/sample/sampler.py:91): exact ties between bf16 logits, and the ranks / lowest-id argmax they cause, are
  // reproduced.  TGIS_LOGITS_FP32=1 keeps the raw fp32 accumulator (round 1's behaviour; an experiment switch).
  DevBuf<uint8_t> logits;
  bool logits_bf16 = true;
  size_t lsz = 2;  // bytes per logit
  CUtensorMap xm_xn[N_BT], xm_attn[N_BT], xm_act[N_BT], xm_last[N_BT], xm_resid[N_BT];
  DevBuf<float> gemm_ws, part_o, part_ml, samp_scratch;
  DevBuf<int> gemm_counters, attn_arrive;
  DevBuf<float> norm_ssq;  // [2][GEMM_NORM_MAX_T][hidden / 128] partial sums of h^2 (fused residual RMSNorm)
  DevBuf<uint32_t> seen_bitmap;
  // guided decoding: allowed-token bits of the step, one row per sequence slot (same geometry as seen_bitmap); the
  // provider writes the pinned host row, the row is copied in front of the step, the sampler reads it for SAMPLE_MASKED rows
  DevBuf<uint32_t> allow_bitmap;
  uint32_t* h_allow = nullptr;
  tgis_mask_fn mask_fn = nullptr;
  void* mask_user = nullptr;
  long long guided_rows = 0;
  // LoRA adapters (lora.cu): per layer and module  A [slots][Rm][K], B [slots][N][Rm] bf16, zero padded to the rank capacity;
  // gate_proj / up_proj form ONE module of capacity 2R over the interleaved gate_up projection
  int max_loras = 0, lora_R = 0;
  struct LoraLayerW {
    bf16 *A_q, *B_q, *A_k, *B_k, *A_v, *B_v, *A_o, *B_o, *A_gu, *B_gu, *A_d, *B_d;
  };
  DevBuf<bf16> lora_arena;
  size_t lora_slot_elems = 0;  // (unused by the kernels; bookkeeping for clear)
  std::vector<LoraLayerW> lora_layers;
  DevBuf<float> lora_v;   // [T][3R] fp32 shrink sums
  DevBuf<bf16> gu_buf;    // [T][2F] raw (interleaved) gate_up output of steps that carry adapter tokens
  long long lora_steps = 0;
  DevBuf<SampleOut> d_samp_out;
  SampleOut* h_samp_out = nullptr;
  SampleOut* h_plp_out = nullptr;  // prompt-logprob pass results (kept apart from the step's sampled rows)
  float* h_trace_logits = nullptr; // pinned landing area of the trace replay's logits (logit_rows_cap rows)
  // staging
  uint8_t* h_stage = nullptr;
  DevBuf<uint8_t> d_stage;
  size_t off_tok = 0, off_pos = 0, off_slotmap = 0, off_tokslot = 0, off_seqs = 0, off_decids = 0, off_tileseq = 0,
         off_tileq0 = 0, off_samplesrc = 0, off_rows = 0, off_epoch = 0, off_bt = 0, off_toklora = 0, stage_bytes = 0;

  // host state
  std::mutex mu;
  std::condition_variable cv_in, cv_out;
  std::deque<std::unique_ptr<Request>> incoming;
  std::vector<std::string> abort_ids;
  std::deque<std::unique_ptr<Request>> waiting;
  std::vector<std::unique_ptr<Request>> running;
  std::deque<tgis_step_output> outputs;
  std::vector<int> free_slots;
  std::thread th;
  std::atomic<bool> stop_flag{false}, thread_alive{false}, errored{false};
  std::string error_msg;
  bool started = false, ready = false;
  std::mt19937_64 rng;
  // stats
  std::atomic<long long> n_steps{0}, n_tokens{0}, n_launches{0}, n_preempt{0};
  // scheduler-state snapshot for tgis_engine_status (the queues themselves belong to the engine thread)
  std::atomic<int> snap_running{0}, snap_waiting{0}, snap_free_blocks{0};
  void snapshot() {
    snap_running = (int)running.size();
    snap_waiting = (int)waiting.size();
    snap_free_blocks = (int)free_blocks.size();
  }
  double gpu_ms = 0, gpu_ms_decode = 0, gpu_ms_mixed = 0;
  long long decode_steps = 0, decode_tokens = 0, h2d_bytes = 0, d2h_bytes = 0;
  // optional per-GEMM timing (tgis_engine_set_profiling): CUDA events around every GEMM launch of a step
  bool profiling = false;
  bool prof_decode_only = false, step_is_decode = false;
  bool fuse_rope = true;
  int rope_fuse_max_t = 32;
  int rope_fuse_cluster_max_t = 256;
  // residual add + RMSNorm folded into the o / down projections' cluster reduction and the gate_up / qkv projections'
  // operand staging (GemmNorm, gemm_tcgen05.cu): tp == 1, steps of at most GEMM_NORM_MAX_T tokens.  TGIS_FUSE_NORM=0: off
  bool fuse_norm = false;
  // tensor parallelism, decode-shaped steps: one-shot all-reduce + residual + RMSNorm over NVLink peer memory
  // (ar_add_rmsnorm_kernel) instead of ncclAllReduce + rmsnorm kernel.  TGIS_TP_FUSED_AR=0: NCCL baseline.
  bool tp_fused_ar = true;
  int tp_exchange_force = -1;                 // TGIS_TP_EXCHANGE
  size_t tp_oneshot_max_bytes = 2u << 20;     // TGIS_TP_ONESHOT_MAX_KB
  bool tp_graphs = true;  // TGIS_TP_GRAPHS=0: tensor-parallel decode steps are launched kernel by kernel (round 1)
  static constexpr int AR_MAX_T = AR_MAX_ROWS;
  uint8_t* ar_mem = nullptr;        // [2 parities] receive areas (ar_recv_bytes each), then the two local partial buffers
  uint8_t* ar_peer[8] = {};         // the same allocation of every rank, mapped here (cudaIpc)
  uint32_t ar_epoch[2] = {0, 0};     // rank 0: epoch of the last exchange of each parity (staged per step: off_epoch)
  uint32_t step_ar_idx[2] = {0, 0};  // exchanges of each parity enqueued so far in the step being built
  uint32_t lg_epoch = 0;             // rank 0: epoch of the last logits gather (staged per step: off_epoch[2])
  int lg_idx_step = 0;               // rank 0: gathers issued for the current step (the step's own, then prompt-logprob passes)
  size_t lg_off = 0;                 // inside ar_mem: [S_max, V] logits receive buffer (rank 0's is the one used), then flags
  int l2_prefetch_kb = 0;   // (off: measured no gain, costs DRAM traffic in the issuing kernel) k-blocks (16 KiB each) per CTA of the NEXT GEMM pulled into L2 by the current one
  std::vector<cudaEvent_t> prof_events;
  size_t prof_used = 0;
  std::vector<double> prof_bytes;  // algorithmic bytes of the GEMM between events 2i and 2i+1 (< 0: an exchange)
  double gemm_ms = 0, gemm_bytes = 0, exchange_ms = 0;
  long long gemm_calls = 0, exchange_calls = 0;
  // event pair around an exchange (profiling only)
  cudaEvent_t prof_begin_exchange() {
    if (!(profiling && (!prof_decode_only || step_is_decode))) return nullptr;
    while (prof_events.size() < prof_used + 2) {
      cudaEvent_t ev;
      CK(cudaEventCreate(&ev));
      prof_events.push_back(ev);
    }
    cudaEvent_t e1 = prof_events[prof_used + 1];
    CK(cudaEventRecord(prof_events[prof_used], stream));
    prof_used += 2;
    prof_bytes.push_back(-1.0);
    return e1;
  }
  // CUDA graphs of pure-decode steps, keyed by (batch size, number of KV splits)
  std::unordered_map<uint64_t, cudaGraphExec_t> graphs;
  std::unordered_map<uint64_t, long long> graph_nodes;
  long long n_graph_launches = 0;
  // Experiment switches for the step-to-step turnaround (scripts/step_timeline.py measured ~1 ms between the end of one
  // graph replay and the first kernel of the next, against ~26 us when the same step is launched kernel by kernel):
  bool sync_spin = true;              // TGIS_SYNC_SPIN: wait for the step by polling its end event instead of
                                      // cudaStreamSynchronize (no blocking-wait wake-up latency)
  bool graph_copy_outside = true;     // TGIS_GRAPH_COPY_OUTSIDE: metadata H2D / result D2H as plain stream copies
                                      // around the graph launch instead of memcpy nodes inside the graph
  bool capturing = false;
  bool attn_inkernel_merge = false;   // TGIS_ATTN_INKERNEL_MERGE (read by attention.cu as well): launch accounting only
  int debug_step_sleep_us = 0;        // TGIS_STEP_SLEEP_US (experiment)
  bool debug_launch = false;          // TGIS_DEBUG_LAUNCH=1: host time spent inside cudaGraphLaunch, printed at destroy
  double graph_launch_host_s = 0;
  // TGIS_DEBUG_LAUNCH: host-side phase times of the last steps: [sched+build, launch, wait, post] in microseconds
  struct HostPhase {
    float sched, launch, wait, post;
  };
  std::vector<HostPhase> host_phases;
  double t_step_begin = 0, t_after_wait = 0;

  ~tgis_engine() {
    if (debug_launch && n_graph_launches > 0)
      fprintf(stderr, "[tgis] rank %d: %lld graph launches, %.1f us host time per cudaGraphLaunch\n", rank,
              n_graph_launches, 1e6 * graph_launch_host_s / (double)n_graph_launches);
    if (debug_launch && !host_phases.empty()) {
      const size_t n = host_phases.size(), lo = n > 48 ? n - 48 : 0;
      fprintf(stderr, "[tgis] host phases of the last %zu steps (us): sched+build / launch / wait / post\n", n - lo);
      for (size_t i = lo; i < n; ++i)
        fprintf(stderr, "  %5.0f %5.0f %6.0f %5.0f\n", host_phases[i].sched, host_phases[i].launch, host_phases[i].wait,
                host_phases[i].post);
    }
    for (void* q : pnx_allocs) cudaFree(q);
    if (stream2) cudaStreamSynchronize(stream2);
    if (ev_fork) cudaEventDestroy(ev_fork);
    if (ev_join) cudaEventDestroy(ev_join);
    if (stream2) cudaStreamDestroy(stream2);
    if (h_stage) cudaFreeHost(h_stage);
    if (h_samp_out) cudaFreeHost(h_samp_out);
    if (h_allow) cudaFreeHost(h_allow);
    if (h_plp_out) cudaFreeHost(h_plp_out);
    if (h_trace_logits) cudaFreeHost(h_trace_logits);
    if (shm) {
      if (rank == 0) shm->shutdown.store(1, std::memory_order_release);
      munmap(shm, shm_bytes);
      if (shm_owner) shm_unlink(shm_name.c_str());
    }
    for (int r = 0; r < 8; ++r)
      if (ar_peer[r] && ar_peer[r] != ar_mem) cudaIpcCloseMemHandle(ar_peer[r]);
    if (ar_mem) cudaFree(ar_mem);
    // captured graphs hold NCCL work of `comm` (the logits all-gather of tensor-parallel decode steps): they must be gone
    // before the communicator is destroyed, or ncclCommDestroy waits for them forever
    for (auto& kv : graphs) cudaGraphExecDestroy(kv.second);
    graphs.clear();
    if (stream) cudaStreamSynchronize(stream);
    if (comm) nccl().CommDestroy(comm);
    for (cudaEvent_t ev : prof_events) cudaEventDestroy(ev);
    if (ev0) cudaEventDestroy(ev0);
    if (ev1) cudaEventDestroy(ev1);
    if (stream) cudaStreamDestroy(stream);
  }

  // ------------------------------------------------------------------------------------------------ setup
  void init() {
    const tgis_config& c = cfg;
    CK(cudaSetDevice(c.device));
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, c.device));
    if (prop.major != 10) throw CudaError("tgis_engine requires an sm_100 (B200) device; found sm_" +
                                          std::to_string(prop.major) + std::to_string(prop.minor));
    num_sms = prop.multiProcessorCount;
    CK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    CK(cudaEventCreate(&ev0));
    CK(cudaEventCreate(&ev1));
    tp = c.tp_size > 1 ? c.tp_size : 1;
    rank = tp > 1 ? c.tp_rank : 0;
    nq = c.n_q_heads / tp;
    nkv = c.n_kv_heads / tp;
    Fl = c.ffn / tp;
    Vl = c.vocab / tp;
    opt = c.arch == TGIS_ARCH_OPT;
    pnx_on = c.arch == TGIS_ARCH_PONENEX || c.arch == TGIS_ARCH_FALERAX || c.arch == TGIS_ARCH_REVEPEL || c.arch == TGIS_ARCH_SIKAZEN;  // the layer-list architectures
    if (pnx_on) logits_bf16 = false;  // fp32 logits straight from the accumulators
    model_head_dim = opt ? c.head_dim : HEAD_DIM;
    attn_scale = 1.0f / std::sqrt((float)model_head_dim);  // zero-padded head dims add nothing to q . k
    pos_rows = opt ? c.max_model_len + 2 : 0;
    q_dim = nq * HEAD_DIM;
    qkv_dim = (nq + 2 * nkv) * HEAD_DIM;
    bt_stride = (c.max_model_len + KV_BLOCK - 1) / KV_BLOCK;
    max_splits_cap = (c.max_model_len + DECODE_SPLIT - 1) / DECODE_SPLIT;
    bitmap_words = (c.vocab + 31) / 32;
    T_max = c.max_batched_tokens;
    S_max = c.max_num_seqs;
    // TMA boxes are up to 256 rows tall: keep every activation tensor at least that tall
    const size_t T_alloc = std::max(T_max, 256), S_alloc = std::max(S_max, 256);
    tiles_max = T_max / 16 + S_max + 1;
    rng.seed(c.seed ? c.seed : 0x5DEECE66Dull);
    if (const char* e = getenv("TGIS_L2_PREFETCH_KB")) l2_prefetch_kb = atoi(e);
    if (const char* e = getenv("TGIS_FUSE_ROPE")) fuse_rope = atoi(e) != 0;
    if (const char* e = getenv("TGIS_FUSE_ROPE_MAX_T")) rope_fuse_max_t = atoi(e);
    if (const char* e = getenv("TGIS_FUSE_ROPE_CLUSTER_MAX_T")) rope_fuse_cluster_max_t = atoi(e);
    if (const char* e = getenv("TGIS_FUSE_NORM")) fuse_norm = atoi(e) != 0;
    if (const char* e = getenv("TGIS_TP_FUSED_AR")) tp_fused_ar = atoi(e) != 0;
    if (const char* e = getenv("TGIS_LOGITS_FP32")) logits_bf16 = atoi(e) == 0;
    if (const char* e = getenv("TGIS_TP_TIMEOUT_S")) tp_timeout_s = atof(e);
    if (const char* e = getenv("TGIS_DEBUG_LAUNCH")) debug_launch = atoi(e) != 0;
    if (const char* e = getenv("TGIS_SYNC_SPIN")) sync_spin = atoi(e) != 0;
    if (const char* e = getenv("TGIS_ATTN_INKERNEL_MERGE")) attn_inkernel_merge = atoi(e) != 0;
    if (const char* e = getenv("TGIS_STEP_SLEEP_US")) debug_step_sleep_us = atoi(e);
    if (const char* e = getenv("TGIS_GRAPH_COPY_OUTSIDE")) graph_copy_outside = atoi(e) != 0;
    if (const char* e = getenv("TGIS_TP_GRAPHS")) tp_graphs = atoi(e) != 0;
    if (const char* e = getenv("TGIS_TP_ONESHOT_MAX_KB")) tp_oneshot_max_bytes = (size_t)atol(e) << 10;
    if (const char* e = getenv("TGIS_TP_EXCHANGE")) {
      const std::string v = e;
      tp_exchange_force = v == "nccl" ? 0 : v == "oneshot" ? 1 : v == "twoshot" ? 2 : -1;
    }
    if (pnx_on) logits_bf16 = false;
    lsz = logits_bf16 ? 2 : 4;
    logit_rows_cap = std::max(S_max, 64);
    logits_ld = pnx_on ? (c.vocab + 7) / 8 * 8 : c.vocab;

    const size_t H = c.hidden, F = Fl, V = c.vocab, L = c.n_layers;  // F: this rank's ffn shard
    if (!pnx_on) {
    // ---- weights: one arena
    const size_t per_layer = (size_t)qkv_dim * H + H * q_dim + 2 * F * H + H * F + 2 * H;
    const size_t opt_extra = opt ? (size_t)pos_rows * H + H + L * ((size_t)qkv_dim + 4 * H + F) + 64 * (6 * L + 4) : 0;
    const size_t total = V * H /*embed*/ + V * H /*lm_head*/ + H /*norm*/ + (size_t)c.max_model_len * HEAD_DIM +
                         L * per_layer + 64 * (6 * L + 8) + opt_extra;
    w_arena.alloc(total);
    if (opt) w_arena.zero();  // the padded head dims of q/k/v rows, out_proj columns and their biases stay zero
    bf16* p = w_arena.p;
    auto take = [&](size_t n) {
      bf16* r = p;
      p += (n + 63) / 64 * 64;  // 128-B aligned slices (TMA needs 16 B)
      return r;
    };
    embed = take(V * H);
    lm_head = take(V * H);
    final_norm = take(H);
    cos_sin = take((size_t)c.max_model_len * HEAD_DIM);
    layers.resize(L);
    for (auto& l : layers) {
      l.wqkv = take((size_t)qkv_dim * H);
      l.wo = take(H * q_dim);
      l.wgu = take(2 * F * H);
      l.wd = take(H * F);
      l.ln1 = take(H);
      l.ln2 = take(H);
      if (opt) {
        l.b_qkv = take(qkv_dim);
        l.b_o = take(H);
        l.b_fc1 = take(F);
        l.b_fc2 = take(H);
        l.ln1_b = take(H);
        l.ln2_b = take(H);
      }
    }
    if (opt) {
      pos_embed = take((size_t)pos_rows * H);
      final_norm_b = take(H);
      // no rotary embedding: cos_sin stays unused (zeroed with the arena)
    } else {
      default_rope_table();
    }

    // ---- activations
    resid.alloc(T_alloc * H);
    xn.alloc(T_alloc * H);
    qkv.alloc(T_alloc * qkv_dim);
    attn_out.alloc(T_alloc * q_dim);
    tmp.alloc(T_alloc * H);
    act.alloc(T_alloc * F);
    if (opt) y32.alloc(T_alloc * std::max<size_t>({(size_t)qkv_dim, F, H}));
    if (c.max_loras > 0) {
      max_loras = c.max_loras;
      lora_R = c.max_lora_rank;
      const size_t R = lora_R, Sl = max_loras, kvd = (size_t)nkv * HEAD_DIM;
      const size_t per_layer = Sl * (R * H + q_dim * R + 2 * (R * H + kvd * R) + R * q_dim + H * R + 2 * R * H +
                                     (size_t)2 * F * 2 * R + R * F + H * R);
      lora_arena.alloc(per_layer * L);
      lora_arena.zero();
      lora_layers.resize(L);
      bf16* p = lora_arena.p;
      auto take = [&](size_t n) {
        bf16* r = p;
        p += n;
        return r;
      };
      for (auto& ll : lora_layers) {
        ll.A_q = take(Sl * R * H);      ll.B_q = take(Sl * q_dim * R);
        ll.A_k = take(Sl * R * H);      ll.B_k = take(Sl * kvd * R);
        ll.A_v = take(Sl * R * H);      ll.B_v = take(Sl * kvd * R);
        ll.A_o = take(Sl * R * q_dim);  ll.B_o = take(Sl * H * R);
        ll.A_gu = take(Sl * 2 * R * H); ll.B_gu = take(Sl * (size_t)2 * F * 2 * R);
        ll.A_d = take(Sl * R * F);      ll.B_d = take(Sl * H * R);
      }
      lora_v.alloc(T_alloc * 3 * R);
      gu_buf.alloc(T_alloc * (size_t)2 * F);
    }
    }  // !pnx_on
    last_hidden.alloc(S_alloc * H);
    logits.alloc((size_t)logit_rows_cap * logits_ld * lsz);
    if (logits_ld != c.vocab) {  // (fp32 logits) columns [vocab, logits_ld): never written again, never chosen
      std::vector<float> fill((size_t)logit_rows_cap * logits_ld, 0.f);
      for (int r = 0; r < logit_rows_cap; ++r)
        for (int j = c.vocab; j < logits_ld; ++j) fill[(size_t)r * logits_ld + j] = -INFINITY;
      CK(cudaMemcpy(logits.p, fill.data(), fill.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    if (tp > 1) {
      logits_shard.alloc((size_t)S_max * Vl * lsz);
      logits_gather.alloc((size_t)tp * S_max * Vl * lsz);
    }
    if (!pnx_on) { xn.zero(); attn_out.zero(); act.zero(); }
    last_hidden.zero();
    gemm_ws.alloc(gemm_workspace_bytes(num_sms) / sizeof(float));
    gemm_counters.alloc(1 << 16);
    gemm_counters.zero();
    attn_arrive.alloc((size_t)S_max * std::max(nkv, 1));
    attn_arrive.zero();
    norm_ssq.alloc((size_t)2 * GEMM_NORM_MAX_T * (c.hidden / 128 + 1));
    const int G = c.n_q_heads / std::max(c.n_kv_heads, 1);
    part_o.alloc((size_t)S_max * nkv * max_splits_cap * G * HEAD_DIM);
    part_ml.alloc((size_t)S_max * nkv * max_splits_cap * G * 2);
    samp_scratch.alloc((size_t)logit_rows_cap * logits_ld);
    seen_bitmap.alloc((size_t)S_max * bitmap_words);
    seen_bitmap.zero();
    if (rank == 0) {  // only the sampling rank needs the masks
      allow_bitmap.alloc((size_t)S_max * bitmap_words);
      CK(cudaHostAlloc(&h_allow, sizeof(uint32_t) * (size_t)S_max * bitmap_words, cudaHostAllocDefault));
    }
    d_samp_out.alloc(S_max);
    CK(cudaHostAlloc(&h_samp_out, sizeof(SampleOut) * S_max, cudaHostAllocDefault));
    CK(cudaHostAlloc(&h_plp_out, sizeof(SampleOut) * S_max, cudaHostAllocDefault));
    CK(cudaHostAlloc(&h_trace_logits, (size_t)logit_rows_cap * logits_ld * sizeof(float), cudaHostAllocDefault));

    // ---- staging layout
    size_t o = 0;
    auto place = [&](size_t bytes) {
      size_t r = o;
      o += (bytes + 255) / 256 * 256;
      return r;
    };
    off_tok = place(4 * (size_t)T_max);
    off_pos = place(4 * (size_t)T_max);
    off_slotmap = place(4 * (size_t)T_max);
    off_tokslot = place(4 * (size_t)T_max);
    off_toklora = place(4 * (size_t)T_max);  // adapter slot of every token (0: base model)
    off_seqs = place(sizeof(AttnSeq) * (size_t)S_max);
    off_decids = place(4 * (size_t)S_max);
    off_tileseq = place(4 * (size_t)tiles_max);
    off_tileq0 = place(4 * (size_t)tiles_max);
    off_samplesrc = place(4 * (size_t)std::max(S_max, logit_rows_cap));
    off_rows = place(sizeof(SampleRow) * (size_t)S_max);
    off_epoch = place(4 * sizeof(uint32_t));  // tensor parallelism: exchange epochs before this step ([0], [1]: per
                                               // parity) and the logits-gather epoch ([2])
    off_ltiles = place(sizeof(LatentTile) * (size_t)(T_max + S_max));  // attention query tiles of the layer-list architectures
    off_ltiles16 = place(sizeof(LatentTile) * (size_t)(T_max / POOLATTN_TILE + S_max + 1));
    off_bt = place(4 * (size_t)S_max * bt_stride);
    // decode work items follow the USED part of the block table (items_off(S)); room for the worst case
    place(sizeof(DecItem) * (1 + (size_t)S_max * max_splits_cap));
    stage_bytes = o;
    CK(cudaHostAlloc(&h_stage, stage_bytes, cudaHostAllocDefault));
    memset(h_stage, 0, stage_bytes);
    d_stage.alloc(stage_bytes);
    d_stage.zero();

    if (pnx_on) {
      init_pnx();
      free_slots.resize(S_max);
      for (int i = 0; i < S_max; ++i) free_slots[i] = S_max - 1 - i;
      snapshot();
      CK(cudaDeviceSynchronize());
      ready = true;
      return;
    }
    // ---- tensor maps (weights: box 128 rows x 64 k; activations: box BT rows x 64 k)
    auto wmap = [&](CUtensorMap* m, const bf16* w, size_t rows, size_t cols) {
      if (make_tmap_bf16_2d(m, w, rows, cols, cols, 128, 64) != 0) throw CudaError("cuTensorMapEncodeTiled(weight) failed");
    };
    for (auto& l : layers) {
      wmap(&l.m_qkv, l.wqkv, qkv_dim, H);
      wmap(&l.m_o, l.wo, H, q_dim);
      wmap(&l.m_gu, l.wgu, opt ? F : 2 * F, H);  // OPT: fc1
      wmap(&l.m_d, l.wd, H, F);
    }
    wmap(&m_lm, lm_head, Vl, H);  // this rank's vocab shard (== V when tp == 1)
    for (int i = 0; i < N_BT; ++i) {
      const int bt = BT_VALUES[i];
      auto xmap = [&](CUtensorMap* m, const bf16* x, size_t rows, size_t cols) {
        if (make_tmap_bf16_2d(m, x, rows, cols, cols, bt, 64) != 0)
          throw CudaError("cuTensorMapEncodeTiled(activation) failed");
      };
      xmap(&xm_xn[i], xn.p, T_alloc, H);
      xmap(&xm_resid[i], resid.p, T_alloc, H);  // fused-norm consumers read the residual stream
      xmap(&xm_attn[i], attn_out.p, T_alloc, q_dim);
      xmap(&xm_act[i], act.p, T_alloc, F);
      xmap(&xm_last[i], last_hidden.p, S_alloc, H);
    }

    // ---- KV cache
    const size_t block_elems = (size_t)nkv * KV_BLOCK * HEAD_DIM;  // per layer, per K or V (this rank's kv heads)
    size_t kv_bytes = c.kv_cache_bytes;
    if (kv_bytes == 0) {
      size_t free_b = 0, total_b = 0;
      CK(cudaMemGetInfo(&free_b, &total_b));
      const float frac = c.gpu_mem_fraction > 0 ? c.gpu_mem_fraction : 0.85f;
      kv_bytes = (size_t)(free_b * (double)frac);
    }
    const size_t bytes_per_block = 2 * L * block_elems * sizeof(bf16);
    size_t nb = kv_bytes / bytes_per_block;
    const size_t nb_cap = (size_t)S_max * bt_stride + 1;  // more can never be used
    nb = std::min(nb, nb_cap);
    if (nb < (size_t)bt_stride) throw CudaError("KV cache too small for one max_model_len sequence");
    num_blocks = (int)nb;
    kv_layer_elems = nb * block_elems;
    k_cache.alloc(L * kv_layer_elems);
    v_cache.alloc(L * kv_layer_elems);
    k_cache.zero();  // finite garbage invariant: masked slots must never hold NaN/Inf (see attention.cu)
    v_cache.zero();
    free_blocks.resize(num_blocks);
    for (int i = 0; i < num_blocks; ++i) free_blocks[i] = num_blocks - 1 - i;
    free_slots.resize(S_max);
    for (int i = 0; i < S_max; ++i) free_slots[i] = S_max - 1 - i;
    snapshot();
    CK(cudaStreamSynchronize(stream));
    CK(cudaDeviceSynchronize());
    if (tp > 1) init_tp();
    ready = true;
  }

  void init_tp() {
    ncclUniqueId id;
    static_assert(sizeof(id.internal) == 128, "nccl id size");
    memcpy(id.internal, cfg.nccl_id, 128);
    NK(nccl().CommInitRank(&comm, tp, id, rank));
    shm_name = cfg.shm_name[0] ? std::string(cfg.shm_name) : std::string("/tgis_tp_plan");
    shm_bytes = SHM_STAGE_OFF + stage_bytes;
    int fd = -1;
    if (rank == 0) {
      shm_unlink(shm_name.c_str());
      fd = shm_open(shm_name.c_str(), O_CREAT | O_RDWR, 0600);
      if (fd < 0 || ftruncate(fd, (off_t)shm_bytes) != 0) throw CudaError("shm_open/ftruncate failed for " + shm_name);
      shm_owner = true;
    } else {
      for (int i = 0; i < 6000 && fd < 0; ++i) {
        fd = shm_open(shm_name.c_str(), O_RDWR, 0600);
        if (fd >= 0) {
          struct stat st;
          if (fstat(fd, &st) != 0 || (size_t)st.st_size < shm_bytes) { close(fd); fd = -1; }
        }
        if (fd < 0) usleep(10000);
      }
      if (fd < 0) throw CudaError("worker could not open the TP plan shm " + shm_name);
    }
    void* m = mmap(nullptr, shm_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (m == MAP_FAILED) throw CudaError("mmap of TP plan failed");
    shm = reinterpret_cast<ShmCtl*>(m);
    if (rank == 0) {
      shm->seq.store(0);
      shm->shutdown.store(0);
      for (auto& a : shm->ack) a.store(0);
      for (auto& a : shm->pid) a.store(0);
      for (auto& a : shm->failed) a.store(0);
      shm->pid[0].store((int32_t)getpid(), std::memory_order_release);
    }
    // first collective doubles as a start-up barrier (and creates NCCL's channels outside the timed path)
    NK(nccl().AllReduce(tmp.p, tmp.p, 1024, ncclBfloat16, ncclSum, comm, stream));
    CK(cudaStreamSynchronize(stream));
    if (tp_fused_ar && tp <= 8) init_fused_ar();
    else tp_fused_ar = false;
  }

  size_t ar_buf_bytes() const { return (size_t)AR_MAX_T * cfg.hidden * sizeof(bf16); }
  size_t lg_logits_bytes() const { return ((size_t)S_max * cfg.vocab * lsz + 255) / 256 * 256; }
  // rank 0's full-vocabulary logits: inside the peer-mapped allocation when the ranks can reach each other's memory
  uint8_t* logits_ptr() { return (tp > 1 && tp_fused_ar && ar_mem) ? ar_mem + lg_off : logits.p; }
  size_t ar2_area_stride() const { return (ar2_area_bytes(cfg.hidden) + 255) / 256 * 256; }
  size_t ar2_area_off(int parity) const { return 2 * ar_recv_bytes(cfg.hidden) + 2 * ar_buf_bytes() + parity * ar2_area_stride(); }
  // How the row-parallel partials of a T-token step are exchanged (TGIS_TP_EXCHANGE=auto|oneshot|twoshot|nccl):
  //   0 ncclAllReduce + add_rmsnorm kernel (prefill-sized steps, or the peer mappings are unavailable)
  //   1 one-shot push ("LL" lines; one NVLink traversal) while a rank's egress 2 (tp-1) T H 2 B stays small
  //   2 two-shot (reduce-scatter by row owner + all-gather of the reduced rows)
  int exchange_mode(int T) const {
    if (tp <= 1 || !tp_fused_ar || T > AR_MAX_T) return 0;
    if (tp_exchange_force >= 0) return tp_exchange_force;
    const size_t oneshot_egress = (size_t)2 * (tp - 1) * T * cfg.hidden * 2;
    return oneshot_egress <= tp_oneshot_max_bytes ? 1 : 2;
  }
  bf16* ar_buf(int parity) { return reinterpret_cast<bf16*>(ar_mem + 2 * ar_recv_bytes(cfg.hidden) + parity * ar_buf_bytes()); }

  // Every rank allocates its exchange buffer, the cudaIpc handles travel by ncclAllGather, every rank maps the others.
  // All ranks must take the same decision: the per-rank success bits are summed with an all-reduce.
  void init_fused_ar() {
    lg_off = 2 * ar_recv_bytes(cfg.hidden) + 2 * ar_buf_bytes() + 2 * ar2_area_stride();
    const size_t bytes = lg_off + lg_logits_bytes() + 256;
    int ok = 1;
    cudaIpcMemHandle_t mine;
    if (cudaMalloc(&ar_mem, bytes) != cudaSuccess || cudaMemset(ar_mem, 0, bytes) != cudaSuccess ||
        cudaIpcGetMemHandle(&mine, ar_mem) != cudaSuccess) {
      ok = 0;
      memset(&mine, 0, sizeof(mine));
      cudaGetLastError();
    }
    DevBuf<uint8_t> hbuf;
    hbuf.alloc(sizeof(cudaIpcMemHandle_t) * 8);
    CK(cudaMemcpy(hbuf.p + rank * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice));
    NK(nccl().AllGather(hbuf.p + rank * sizeof(mine), hbuf.p, sizeof(mine), ncclInt8, comm, stream));
    CK(cudaStreamSynchronize(stream));
    cudaIpcMemHandle_t all[8];
    CK(cudaMemcpy(all, hbuf.p, sizeof(mine) * tp, cudaMemcpyDeviceToHost));
    for (int r = 0; r < tp && ok; ++r) {
      if (r == rank) {
        ar_peer[r] = ar_mem;
      } else if (cudaIpcOpenMemHandle(reinterpret_cast<void**>(&ar_peer[r]), all[r], cudaIpcMemLazyEnablePeerAccess) !=
                 cudaSuccess) {
        ar_peer[r] = nullptr;
        ok = 0;
        cudaGetLastError();
      }
    }
    DevBuf<float> vote;
    vote.alloc(1);
    const float mine_ok = (float)ok;
    CK(cudaMemcpy(vote.p, &mine_ok, sizeof(float), cudaMemcpyHostToDevice));
    NK(nccl().AllReduce(vote.p, vote.p, 1, ncclFloat, ncclSum, comm, stream));
    CK(cudaStreamSynchronize(stream));
    float total = 0.f;
    CK(cudaMemcpy(&total, vote.p, sizeof(float), cudaMemcpyDeviceToHost));
    tp_fused_ar = ((int)(total + 0.5f) == tp);
  }

  // exchange #parity of a layer (0: after o-proj, 1: after down-proj) + residual add + RMSNorm with weight w
  void fused_ar_norm(int parity, const bf16* w, int T) {
    cudaEvent_t pe = prof_begin_exchange();
    if (exchange_mode(T) == 2) {
      Ar2Peers P;
      memset(&P, 0, sizeof(P));
      P.own = ar_buf(parity);
      for (int r = 0; r < tp; ++r) P.area[r] = ar_peer[r] + ar2_area_off(parity);
      CK(ar2_add_rmsnorm_launch(P, tp, rank, ds<uint32_t>(off_epoch) + parity, ++step_ar_idx[parity], resid.p, w, xn.p, T,
                                cfg.hidden, cfg.rms_eps, stream));
    } else {
      ArPeers P;
      memset(&P, 0, sizeof(P));
      P.own = ar_buf(parity);
      for (int r = 0; r < tp; ++r) P.recv[r] = reinterpret_cast<uint4*>(ar_peer[r] + parity * ar_recv_bytes(cfg.hidden));
      CK(ar_add_rmsnorm_launch(P, tp, rank, ds<uint32_t>(off_epoch) + parity, ++step_ar_idx[parity], resid.p, w, xn.p, T,
                               cfg.hidden, cfg.rms_eps, stream));
    }
    if (pe) CK(cudaEventRecord(pe, stream));
    ++n_launches;
  }

  static bool pid_alive(int pid) { return pid > 0 && (kill(pid, 0) == 0 || errno == EPERM); }

  // rank 0: wait until every worker has taken the previous plan, then publish this one.  The wait is a spin (the
  // common case is microseconds) with a liveness check: a worker that died or reported a failure turns into an
  // exception here -> fail_all -> errored, instead of rank 0 spinning forever behind a healthy-looking /health.
  void publish_plan(const StepHeader& h) {
    for (int r = 1; r < tp; ++r) {
      double t_check = 0;
      const double t_start = now_s();
      while (shm->ack[r].load(std::memory_order_acquire) != plan_seq) {
        if (stop_flag) return;
        const double t = now_s();
        if (t - t_start > 0.002 && t - t_check > 0.05) {
          t_check = t;
          if (shm->failed[r].load(std::memory_order_acquire))
            throw CudaError("tensor-parallel worker rank " + std::to_string(r) + " reported a failure");
          const int pid = shm->pid[r].load(std::memory_order_acquire);
          if (pid > 0 && !pid_alive(pid))
            throw CudaError("tensor-parallel worker rank " + std::to_string(r) + " (pid " + std::to_string(pid) + ") died");
          if (t - t_start > tp_timeout_s)
            throw CudaError("tensor-parallel worker rank " + std::to_string(r) + " did not take a step plan for " +
                            std::to_string((int)tp_timeout_s) + " s");
        }
      }
    }
    memcpy(reinterpret_cast<uint8_t*>(shm) + SHM_STAGE_OFF, h_stage, h.copy_bytes);
    shm->hdr = h;
    shm->seq.store(++plan_seq, std::memory_order_release);
  }

  // worker ranks: follow rank 0's step plans until shutdown (or until rank 0 disappears)
  int worker_loop() {
    CK(cudaSetDevice(cfg.device));
    shm->pid[rank].store((int32_t)getpid(), std::memory_order_release);
    uint64_t seen = 0;
    try {
      for (;;) {
        uint64_t s;
        double t_check = now_s();
        while ((s = shm->seq.load(std::memory_order_acquire)) == seen) {
          if (shm->shutdown.load(std::memory_order_acquire)) return 0;
          const double t = now_s();
          if (t - t_check > 0.5) {
            t_check = t;
            const int pid0 = shm->pid[0].load(std::memory_order_acquire);
            if (pid0 > 0 && !pid_alive(pid0)) return fail("rank 0 (pid " + std::to_string(pid0) + ") is gone", -2);
          }
        }
        const StepHeader h = shm->hdr;
        memcpy(h_stage, reinterpret_cast<uint8_t*>(shm) + SHM_STAGE_OFF, h.copy_bytes);
        seen = s;
        shm->ack[rank].store(s, std::memory_order_release);
        exec_step(h);
        CK(cudaStreamSynchronize(stream));
        ++n_steps;
      }
    } catch (...) {
      shm->failed[rank].store(1, std::memory_order_release);
      throw;
    }
  }

  void default_rope_table() {
    // HF LlamaRotaryEmbedding: inv_freq fp32, freqs = pos * inv_freq (fp32), cos/sin fp32 -> model dtype.
    const int half = HEAD_DIM / 2;
    std::vector<bf16> tab((size_t)cfg.max_model_len * HEAD_DIM);
    for (int pos = 0; pos < cfg.max_model_len; ++pos)
      for (int i = 0; i < half; ++i) {
        const float inv = (float)(1.0 / std::pow((double)cfg.rope_theta, (double)(2 * i) / HEAD_DIM));
        const float f = (float)pos * inv;
        tab[(size_t)pos * HEAD_DIM + i] = __float2bfloat16_rn((float)std::cos((double)f));
        tab[(size_t)pos * HEAD_DIM + half + i] = __float2bfloat16_rn((float)std::sin((double)f));
      }
    CK(cudaMemcpy(cos_sin, tab.data(), tab.size() * sizeof(bf16), cudaMemcpyHostToDevice));
  }

  // Copies the FULL (unsharded) tensor's shard for this rank into the arena: row blocks for column-parallel layers
  // (q/k/v/gate/up, lm_head), column blocks for row-parallel layers (o, down), everything else replicated.
  // OPT checkpoints (HF names, "model.decoder." or "decoder." prefix).  Single GPU: every tensor is kept whole.  q/k/v rows,
  // out_proj columns and the q/k/v biases are spread head by head over 128-dim head slots (the upper 128 - head_dim dims of
  // every slot stay zero: the arena was zeroed), so the attention kernels and the paged cache keep their one geometry.
  int load_weight_opt(const std::string& full_name, const void* ptr, int64_t rows, int64_t cols) {
    const tgis_config& c = cfg;
    const int64_t H = c.hidden, F = c.ffn, V = c.vocab, hd = model_head_dim, nh = c.n_q_heads;
    std::string name = full_name;
    if (name.rfind("model.", 0) == 0) name = name.substr(6);
    auto shape_err = [&]() {
      return fail("shape mismatch for " + full_name + ": got " + std::to_string(rows) + "x" + std::to_string(cols));
    };
    auto copy = [&](bf16* dst, int64_t n) -> int {
      if (rows * cols != n) return shape_err();
      const cudaError_t e = cudaMemcpy(dst, ptr, (size_t)n * sizeof(bf16), cudaMemcpyDefault);
      return e == cudaSuccess ? 0 : fail(std::string("cudaMemcpy(weight) failed: ") + cudaGetErrorString(e));
    };
    // n_rows source rows of `w` elements each -> destination rows `dpitch` elements apart
    auto copy2d = [&](bf16* dst, int64_t dpitch, int64_t w, int64_t n_rows) -> int {
      if (rows * cols != w * n_rows) return shape_err();
      const cudaError_t e = cudaMemcpy2D(dst, (size_t)dpitch * sizeof(bf16), ptr, (size_t)w * sizeof(bf16),
                                         (size_t)w * sizeof(bf16), (size_t)n_rows, cudaMemcpyDefault);
      return e == cudaSuccess ? 0 : fail(std::string("cudaMemcpy2D(weight) failed: ") + cudaGetErrorString(e));
    };
    if (name == "lm_head.weight") { lm_head_loaded = true; return copy(lm_head, V * H); }
    if (name.rfind("decoder.", 0) != 0) return fail("unknown weight " + full_name);
    name = name.substr(8);
    opt_loaded.insert(name);  // (a failed copy fails the load as a whole)
    if (name == "embed_tokens.weight") return copy(embed, V * H);
    if (name == "embed_positions.weight") {
      // the checkpoint's table covers max_position_embeddings + 2 rows; the engine keeps what max_model_len can reach
      if (cols != H || rows < pos_rows) return shape_err();
      const cudaError_t e = cudaMemcpy(pos_embed, ptr, (size_t)pos_rows * H * sizeof(bf16), cudaMemcpyDefault);
      return e == cudaSuccess ? 0 : fail(std::string("cudaMemcpy(weight) failed: ") + cudaGetErrorString(e));
    }
    if (name == "final_layer_norm.weight") return copy(final_norm, H);
    if (name == "final_layer_norm.bias") return copy(final_norm_b, H);
    if (name.rfind("layers.", 0) != 0) return fail("unknown weight " + full_name);
    const size_t dot = name.find('.', 7);
    if (dot == std::string::npos) return fail("bad weight name " + full_name);
    const int li = atoi(name.substr(7, dot - 7).c_str());
    if (li < 0 || li >= c.n_layers) return fail("layer index out of range in " + full_name);
    LayerW& l = layers[li];
    const std::string sub = name.substr(dot + 1);
    const int64_t slot_w = (int64_t)HEAD_DIM * H;  // elements of one padded head's rows in wqkv
    for (int j = 0; j < 3; ++j) {
      static const char* const qkv_names[3] = {"q_proj", "k_proj", "v_proj"};
      const std::string base = std::string("self_attn.") + qkv_names[j];
      // head h's hd rows of [H] -> rows [h * 128, h * 128 + hd) of the projection's block
      if (sub == base + ".weight") return copy2d(l.wqkv + (size_t)j * nh * slot_w, slot_w, hd * H, nh);
      if (sub == base + ".bias") return copy2d(l.b_qkv + (size_t)j * nh * HEAD_DIM, HEAD_DIM, hd, nh);
    }
    // out_proj [H, nh * hd]: (row, head) pairs are the source rows of hd elements, 128 apart in wo [H, nh * 128]
    if (sub == "self_attn.out_proj.weight") return copy2d(l.wo, HEAD_DIM, hd, H * nh);
    if (sub == "self_attn.out_proj.bias") return copy(l.b_o, H);
    if (sub == "self_attn_layer_norm.weight") return copy(l.ln1, H);
    if (sub == "self_attn_layer_norm.bias") return copy(l.ln1_b, H);
    if (sub == "fc1.weight") return copy(l.wgu, F * H);
    if (sub == "fc1.bias") return copy(l.b_fc1, F);
    if (sub == "fc2.weight") return copy(l.wd, H * F);
    if (sub == "fc2.bias") return copy(l.b_fc2, H);
    if (sub == "final_layer_norm.weight") return copy(l.ln2, H);
    if (sub == "final_layer_norm.bias") return copy(l.ln2_b, H);
    return fail("unknown layer weight " + full_name);
  }

  int load_weight(const std::string& name, const void* ptr, int64_t rows, int64_t cols) {
    if (opt) return load_weight_opt(name, ptr, rows, cols);
    if (pnx_on) return pnx_load_weight(name, ptr, rows, cols);
    const tgis_config& c = cfg;
    const int64_t H = c.hidden, F = c.ffn, V = c.vocab;
    const uint8_t* src = static_cast<const uint8_t*>(ptr);
    bf16* dst = nullptr;
    int64_t er = 0, ec = 0;             // expected full shape
    int64_t r0 = 0, nr = 0, c0 = 0, nc = 0;  // shard = rows [r0, r0+nr) x cols [c0, c0+nc)
    int interleave = 0;                      // destination row stride 2 (gate/up pairs)
    auto rows_shard = [&](bf16* d, int64_t full_rows, int64_t full_cols, int64_t per_rank) {
      dst = d; er = full_rows; ec = full_cols; r0 = rank * per_rank; nr = per_rank; c0 = 0; nc = full_cols;
    };
    auto cols_shard = [&](bf16* d, int64_t full_rows, int64_t full_cols, int64_t per_rank) {
      dst = d; er = full_rows; ec = full_cols; r0 = 0; nr = full_rows; c0 = rank * per_rank; nc = per_rank;
    };
    auto full = [&](bf16* d, int64_t full_rows, int64_t full_cols) {
      dst = d; er = full_rows; ec = full_cols; r0 = 0; nr = full_rows; c0 = 0; nc = full_cols;
    };
    if (name == "model.embed_tokens.weight") full(embed, V, H);
    else if (name == "lm_head.weight") { rows_shard(lm_head, V, H, Vl); lm_head_loaded = true; }
    else if (name == "model.norm.weight") full(final_norm, H, 1);
    else if (name == "tgis.rope_cos_sin") { full(cos_sin, c.max_model_len, HEAD_DIM); cos_sin_loaded = true; }
    else if (name.rfind("model.layers.", 0) == 0) {
      const size_t dot = name.find('.', 13);
      if (dot == std::string::npos) return fail("bad weight name " + name);
      const int li = atoi(name.substr(13, dot - 13).c_str());
      if (li < 0 || li >= c.n_layers) return fail("layer index out of range in " + name);
      LayerW& l = layers[li];
      const std::string sub = name.substr(dot + 1);
      const int64_t kvd = (int64_t)nkv * HEAD_DIM;  // local
      if (sub == "self_attn.q_proj.weight") rows_shard(l.wqkv, (int64_t)c.n_q_heads * HEAD_DIM, H, q_dim);
      else if (sub == "self_attn.k_proj.weight") rows_shard(l.wqkv + (size_t)q_dim * H, (int64_t)c.n_kv_heads * HEAD_DIM, H, kvd);
      else if (sub == "self_attn.v_proj.weight") rows_shard(l.wqkv + (size_t)(q_dim + kvd) * H, (int64_t)c.n_kv_heads * HEAD_DIM, H, kvd);
      else if (sub == "self_attn.o_proj.weight") cols_shard(l.wo, H, (int64_t)c.n_q_heads * HEAD_DIM, q_dim);
      // gate / up rows are INTERLEAVED in wgu (row 2j = gate_j, row 2j+1 = up_j) so the GEMM epilogue can fuse SwiGLU
      else if (sub == "mlp.gate_proj.weight") { rows_shard(l.wgu, F, H, Fl); interleave = 1; }
      else if (sub == "mlp.up_proj.weight") { rows_shard(l.wgu + H, F, H, Fl); interleave = 1; }
      else if (sub == "mlp.down_proj.weight") cols_shard(l.wd, H, F, Fl);
      else if (sub == "input_layernorm.weight") full(l.ln1, H, 1);
      else if (sub == "post_attention_layernorm.weight") full(l.ln2, H, 1);
      else return fail("unknown layer weight " + name);
    } else {
      return fail("unknown weight " + name);
    }
    if (rows * cols != er * ec) return fail("shape mismatch for " + name + ": got " + std::to_string(rows) + "x" +
                                            std::to_string(cols) + " expected " + std::to_string(er) + "x" + std::to_string(ec));
    cudaError_t e;
    if (interleave) {
      e = cudaMemcpy2D(dst, (size_t)2 * ec * sizeof(bf16), src + (size_t)r0 * ec * sizeof(bf16), (size_t)ec * sizeof(bf16),
                       (size_t)ec * sizeof(bf16), (size_t)nr, cudaMemcpyDefault);
    } else if (nc == ec) {
      e = cudaMemcpy(dst, src + (size_t)r0 * ec * sizeof(bf16), (size_t)(nr * ec) * sizeof(bf16), cudaMemcpyDefault);
    } else {
      e = cudaMemcpy2D(dst, (size_t)nc * sizeof(bf16), src + (size_t)c0 * sizeof(bf16), (size_t)ec * sizeof(bf16),
                       (size_t)nc * sizeof(bf16), (size_t)nr, cudaMemcpyDefault);
    }
    if (e != cudaSuccess) return fail(std::string("cudaMemcpy(weight) failed: ") + cudaGetErrorString(e));
    return 0;
  }

  // ---- LoRA adapter slots (host threads other than the engine thread call these: legacy-stream copies into tensors no
  // running step reads -- the host pins a slot while a request names it, engine/lora.py LoRAManager)
  int lora_slot_check(int32_t slot) const {
    if (max_loras == 0) return fail("the engine was created without LoRA slots (max_loras = 0)");
    if (slot < 1 || slot > max_loras) return fail("adapter slot out of range");
    return 0;
  }
  template <class Fn>
  void lora_for_each(int32_t slot, Fn fn) {
    const size_t R = lora_R, H = cfg.hidden, F = Fl, kvd = (size_t)nkv * HEAD_DIM, s = (size_t)(slot - 1);
    for (auto& ll : lora_layers) {
      fn(ll.A_q + s * R * H, R * H);              fn(ll.B_q + s * q_dim * R, (size_t)q_dim * R);
      fn(ll.A_k + s * R * H, R * H);              fn(ll.B_k + s * kvd * R, kvd * R);
      fn(ll.A_v + s * R * H, R * H);              fn(ll.B_v + s * kvd * R, kvd * R);
      fn(ll.A_o + s * R * q_dim, R * q_dim);      fn(ll.B_o + s * H * R, H * R);
      fn(ll.A_gu + s * 2 * R * H, 2 * R * H);     fn(ll.B_gu + s * 2 * F * 2 * R, 2 * F * 2 * R);
      fn(ll.A_d + s * R * F, R * F);              fn(ll.B_d + s * H * R, H * R);
    }
  }
  int clear_adapter(int32_t slot) {
    if (int rc = lora_slot_check(slot)) return rc;
    CK(cudaSetDevice(cfg.device));
    lora_for_each(slot, [&](bf16* p, size_t n) { CK(cudaMemset(p, 0, n * sizeof(bf16))); });
    CK(cudaStreamSynchronize(cudaStreamLegacy));
    return 0;
  }
  int load_adapter_weight(int32_t slot, const std::string& name, const void* ptr, int64_t rows, int64_t cols) {
    if (int rc = lora_slot_check(slot)) return rc;
    if (name.rfind("layers.", 0) != 0) return fail("bad adapter weight name " + name);
    const size_t dot = name.find('.', 7);
    if (dot == std::string::npos) return fail("bad adapter weight name " + name);
    const int li = atoi(name.substr(7, dot - 7).c_str());
    if (li < 0 || li >= cfg.n_layers) return fail("layer index out of range in " + name);
    const std::string rest = name.substr(dot + 1);
    const size_t dot2 = rest.find('.');
    if (dot2 == std::string::npos) return fail("bad adapter weight name " + name);
    const std::string mod = rest.substr(0, dot2), which = rest.substr(dot2 + 1);
    if (which != "lora_A" && which != "lora_B") return fail("bad adapter weight name " + name);
    const bool isA = which == "lora_A";
    const int64_t R = lora_R, H = cfg.hidden, F = Fl, kvd = (int64_t)nkv * HEAD_DIM, s = slot - 1;
    LoraLayerW& ll = lora_layers[li];
    bf16* dst = nullptr;
    int64_t fin = 0, fout = 0, cap = R;   // module geometry; cap: rank capacity of the stored tensor (row length of B)
    int64_t b_row_stride = 0;             // B: destination elements between consecutive source rows
    if (mod == "q_proj") { fin = H; fout = q_dim; dst = isA ? ll.A_q + s * R * H : ll.B_q + s * q_dim * R; }
    else if (mod == "k_proj") { fin = H; fout = kvd; dst = isA ? ll.A_k + s * R * H : ll.B_k + s * kvd * R; }
    else if (mod == "v_proj") { fin = H; fout = kvd; dst = isA ? ll.A_v + s * R * H : ll.B_v + s * kvd * R; }
    else if (mod == "o_proj") { fin = q_dim; fout = H; dst = isA ? ll.A_o + s * R * q_dim : ll.B_o + s * H * R; }
    else if (mod == "down_proj") { fin = F; fout = H; dst = isA ? ll.A_d + s * R * F : ll.B_d + s * H * R; }
    else if (mod == "gate_proj" || mod == "up_proj") {
      // one module of capacity 2R over the interleaved projection: A rows [0, R) gate / [R, 2R) up; B row 2j = gate_j
      // (columns [0, R)), row 2j + 1 = up_j (columns [R, 2R))
      const bool up = mod == "up_proj";
      fin = H; fout = F; cap = 2 * R;
      if (isA) dst = ll.A_gu + s * 2 * R * H + (up ? R * H : 0);
      else { dst = ll.B_gu + s * 2 * F * 2 * R + (up ? 2 * R + R : 0); b_row_stride = 2 * cap; }
    } else return fail("unsupported LoRA module " + mod);
    const int64_t r = isA ? rows : cols;
    if (r < 1 || r > R) return fail("adapter rank " + std::to_string(r) + " exceeds max_lora_rank " + std::to_string(R));
    if (isA ? cols != fin : rows != fout)
      return fail("shape mismatch for " + name + ": got " + std::to_string(rows) + "x" + std::to_string(cols));
    CK(cudaSetDevice(cfg.device));
    if (isA) {
      CK(cudaMemcpy(dst, ptr, (size_t)(rows * cols) * sizeof(bf16), cudaMemcpyDefault));
    } else {
      if (b_row_stride == 0) b_row_stride = cap;
      CK(cudaMemcpy2D(dst, (size_t)b_row_stride * sizeof(bf16), ptr, (size_t)cols * sizeof(bf16), (size_t)cols * sizeof(bf16),
                      (size_t)rows, cudaMemcpyDefault));
    }
    CK(cudaStreamSynchronize(cudaStreamLegacy));
    return 0;
  }

  void finalize_weights() {
    if (pnx_on) {  // a checkpoint with a tensor missing must not come up on zeros
      if (pnx_loaded.size() != pnx_expected_tensors)
        throw CudaError("checkpoint incomplete: " + std::to_string(pnx_loaded.size()) + " of " +
                        std::to_string(pnx_expected_tensors) + " tensors loaded");
      return;
    }
    if (opt) {
      // an OPT checkpoint with a tensor missing must not come up healthy on zeros (the reference's engine fails the load)
      const size_t expected = 4 + (size_t)16 * cfg.n_layers;
      if (opt_loaded.size() < expected)
        throw CudaError("OPT checkpoint incomplete: " + std::to_string(opt_loaded.size()) + " of " + std::to_string(expected) +
                        " tensors loaded (embed_tokens, embed_positions, final_layer_norm.{weight,bias} and 16 per layer)");
    }
    if (!lm_head_loaded)  // tie_word_embeddings
      CK(cudaMemcpy(lm_head, embed + (size_t)rank * Vl * cfg.hidden, (size_t)Vl * cfg.hidden * sizeof(bf16),
                    cudaMemcpyDeviceToDevice));
  }

  // ------------------------------------------------------------------------------------------------ layer-list models
  // TGIS_ARCH_PONENEX / TGIS_ARCH_FALERAX.  Scheduler, sequence slots, block manager, step metadata, lm_head rows, sampler and CUDA-graph
  // replay are the engine's; what differs is the layer stack (pnx_forward) and the per-layer cache of latent rows, which
  // is paged with the same block ids as every other model's KV cache.
  template <class T>
  T* pnx_alloc(size_t count, bool zero = false) {
    void* q = nullptr;
    CK(cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T)));
    if (zero) CK(cudaMemset(q, 0, std::max<size_t>(count, 1) * sizeof(T)));
    pnx_allocs.push_back(q);
    return reinterpret_cast<T*>(q);
  }
  void* pnx_alloc_dt(size_t count, bool zero = false) {
    return pnx_alloc<uint8_t>(count * dt_size(pnx_dt), zero);
  }
  // cos | sin of p * f_i, f_i = base^(-2i / dims), i < dims / 2, evaluated in double and stored fp32: [max_model_len][dims].
  // YaRN scaling (factor > 0): with dim(t) = dims ln(original / (2 pi t)) / (2 ln base) the dimension whose wave makes t turns
  // over `original` positions, lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dims - 1) and the ramp
  // r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1):  f_i <- f_i / factor * r_i + f_i (1 - r_i), cos and sin times 0.1 ln(factor) + 1.
  // linear > 0: every frequency is divided by it (linear position scaling).
  const float* pnx_rope_table(float base, int dims, float factor = 0.f, float original = 0.f, float fast = 0.f, float slow = 0.f,
                              float linear = 1.f) {
    const std::vector<float> key = {base, (float)dims, factor, original, fast, slow, linear};
    for (auto& kv : pnx_rope_tables)
      if (kv.first == key) return kv.second;
    const int half = dims / 2;
    std::vector<double> freq(std::max(half, 1));
    double mag = 1.0;
    for (int i = 0; i < half; ++i) freq[i] = std::pow((double)base, -2.0 * i / dims) / (linear > 0.f ? (double)linear : 1.0);
    if (factor > 0.f) {
      const double pi = 3.14159265358979323846;
      auto turn_dim = [&](double turns) { return dims * std::log((double)original / (2.0 * pi * turns)) / (2.0 * std::log((double)base)); };
      const double lo = std::max(std::floor(turn_dim(fast)), 0.0), hi = std::min(std::ceil(turn_dim(slow)), (double)dims - 1.0);
      for (int i = 0; i < half; ++i) {
        const double r = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
        freq[i] = freq[i] / (double)factor * r + freq[i] * (1.0 - r);
      }
      mag = 0.1 * std::log((double)factor) + 1.0;
    }
    std::vector<float> tab((size_t)cfg.max_model_len * std::max(dims, 1));
    for (int pos = 0; pos < cfg.max_model_len; ++pos)
      for (int i = 0; i < half; ++i) {
        const double a = (double)pos * freq[i];
        tab[(size_t)pos * dims + i] = (float)(std::cos(a) * mag);
        tab[(size_t)pos * dims + half + i] = (float)(std::sin(a) * mag);
      }
    float* d = pnx_alloc<float>(tab.size());
    CK(cudaMemcpy(d, tab.data(), tab.size() * sizeof(float), cudaMemcpyHostToDevice));
    pnx_rope_tables.push_back({key, d});
    return d;
  }

  void init_pnx() {
    const tgis_config& c = cfg;
    const size_t W = c.hidden, V = c.vocab, T = std::max(T_max, 256);
    pnx_rows_alloc = T;
    pnx_dt = pnx_spec.dtype == TGIS_DTYPE_F32 ? DT_F32 : DT_BF16;
    if (const char* e = getenv("TGIS_PNX_TC")) pnx_tc = atoi(e) != 0;
    if (const char* e = getenv("TGIS_DUMP_RESID")) pnx_dump_path = e;
    post_norm = (pnx_spec.style & TGIS_STYLE_POST_NORM) != 0;
    tied_head = (pnx_spec.style & TGIS_STYLE_TIED_HEAD) != 0;
    gated_style = (pnx_spec.style & TGIS_STYLE_PARALLEL_GATED) != 0;
    pair_style = (pnx_spec.style & TGIS_STYLE_PARALLEL_PAIR) != 0;
    pnx_embed = pnx_alloc_dt(V * W);
    pnx_head = tied_head ? pnx_embed : pnx_alloc_dt(V * W);
    pnx_final_norm = pnx_alloc<float>(W);
    pnx_expected_tensors = tied_head ? 2 : 3;
    size_t m_f1 = 1, m_f2 = 1, m_f3 = 1, m_mix = 1;
    size_t m_down = 1, m_qr = 1, m_q = 1, m_qabs = 1, m_olat = 1, m_ov = 1, m_heads = 1, m_E = 1, m_top = 1, m_ff = 1, m_ffs = 1;
    size_t cache_row_bytes = 0;
    pnx_tile_tokens = LATENT_PAIRS;
    pnx_layers.resize(pnx_layer_specs.size());
    for (size_t i = 0; i < pnx_layers.size(); ++i) {
      PnxLayer& l = pnx_layers[i];
      const tgis_layer_spec& s = pnx_layer_specs[i];
      l.sp = s;
      if (pair_style) {   // weights only: cache rows and state belong to the layer RUNS (pair_runs, below)
        const size_t sd = pnx_spec.side_dim;
        l.weights_of = (int)i;
        l.norm1 = pnx_alloc<float>(W);
        pnx_expected_tensors += 1;
        if (s.mlp == TGIS_MLP_DENSE_SILU) {
          l.norm2 = pnx_alloc<float>(W);
          l.w_gu = pnx_alloc_dt((size_t)2 * s.ff * W);
          l.w_d = pnx_alloc_dt(W * s.ff);
          pnx_expected_tensors += 4;  // norm2, mlp.gate, mlp.up, mlp.down
          m_ffs = std::max<size_t>(m_ffs, s.ff);
        }
        if (sd > 0) {
          l.w_sg = pnx_alloc_dt(sd * W);
          l.w_sp = pnx_alloc_dt(W * sd);
          l.side_norm = pnx_alloc<float>(W);
          pnx_expected_tensors += 3;  // side.gate, side.proj, side.norm
          m_E = std::max(m_E, sd); m_qr = std::max(m_qr, sd);
        }
        m_mix = std::max(m_mix, W);
        const float lin = s.rot_linear > 0.f ? s.rot_linear : 1.f;
        if (s.mixer == TGIS_MIXER_POOLED_ATTENTION) {
          const int H = s.heads, G = s.kv_heads;
          l.pa = PoolAttnGeom{H, G, s.dim, s.vdim, s.window, s.window > 0 ? s.pool : 0, s.rot_dims, s.scale,
                              (s.flags & TGIS_LAYER_UNIT_QK) != 0 ? 1 : 0};
          l.c_q = 0; l.c_k = H * s.dim; l.c_v = l.c_k + G * s.dim;
          l.in_cols = (l.c_v + G * s.vdim + 7) / 8 * 8;
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_o = pnx_alloc_dt(W * H * s.vdim);
          if ((s.flags & TGIS_LAYER_QKV_BIAS) != 0) {
            l.in_bias = pnx_alloc<float>(l.in_cols, true);
            pnx_expected_tensors += 3;  // q.b, k.b, v.b
          }
          l.cos_sin = s.rot_dims > 0 ? pnx_rope_table(s.rot_base, s.rot_dims, 0.f, 0.f, 0.f, 0.f, lin) : nullptr;
          pnx_expected_tensors += 4;  // q, k, v, o
          m_q = std::max<size_t>(m_q, (size_t)H * s.dim);
          m_ov = std::max<size_t>(m_ov, (size_t)H * s.vdim);
          m_down = std::max<size_t>(m_down, l.in_cols);
        } else if (s.mixer == TGIS_MIXER_HGRN) {
          const size_t H = s.heads, hd = H * s.dim, hv = H * s.vdim;
          l.c_q = 0; l.c_f = (int)hd; l.c_v = (int)(2 * hd);
          l.in_cols = (int)((2 * hd + hv + 7) / 8 * 8);
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_o = pnx_alloc_dt(W * hv);
          l.w0 = pnx_alloc<float>(hd);        // the gate's bias
          l.u = pnx_alloc<float>(hd);         // its lower bound
          l.mm_norm = pnx_alloc<float>(hv);   // the per-head weight, repeated for every head
          pnx_expected_tensors += 7;  // q, f, f.b, lower, v, norm, o
          m_f1 = std::max(m_f1, hv);
          m_down = std::max<size_t>(m_down, l.in_cols);
        } else {  // TGIS_MIXER_LATENT_ATTENTION
          l.out_gate = (s.flags & TGIS_LAYER_NO_OUT_GATE) == 0;
          l.g = LatentGeom{s.heads, s.dim, s.rot_dim, s.vdim, s.kv_rank, s.q_rank, s.window, s.rot_dims, s.scale,
                           (s.flags & TGIS_LAYER_ROT_INTERLEAVED) != 0 ? 1 : 0, nullptr};
          const size_t hd = (size_t)s.dim + s.rot_dim, row = (size_t)s.kv_rank + s.rot_dim;
          l.w_down = pnx_alloc_dt((size_t)l.n_down() * W);
          l.w_uq = pnx_alloc_dt((size_t)s.heads * hd * s.q_rank);
          l.w_ukT = pnx_alloc_dt((size_t)s.heads * s.kv_rank * s.dim);
          l.w_uv = pnx_alloc_dt((size_t)s.heads * s.vdim * s.kv_rank);
          l.w_o = pnx_alloc_dt(W * s.heads * s.vdim);
          l.qnorm = pnx_alloc<float>(s.q_rank);
          l.kvnorm = pnx_alloc<float>(s.kv_rank);
          if ((s.flags & TGIS_LAYER_SINK) != 0) {
            l.sink = pnx_alloc<float>(s.heads);
            l.g.sink = l.sink;
            pnx_expected_tensors += 1;
          }
          l.cos_sin = pnx_rope_table(s.rot_base, s.rot_dims, 0.f, 0.f, 0.f, 0.f, lin);
          pnx_expected_tensors += 8 + (l.out_gate ? 1 : 0);  // dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o (+ g)
          m_down = std::max<size_t>(m_down, l.n_down()); m_qr = std::max<size_t>(m_qr, s.q_rank);
          m_q = std::max(m_q, s.heads * hd); m_qabs = std::max(m_qabs, s.heads * row);
          m_olat = std::max(m_olat, (size_t)s.heads * s.kv_rank); m_ov = std::max(m_ov, (size_t)s.heads * s.vdim);
          m_heads = std::max<size_t>(m_heads, s.heads);
          pnx_tile_tokens = std::min(pnx_tile_tokens, latent_tile_tokens(s.heads));
        }
        continue;
      }
      if (gated_style) {
        const size_t slots = S_max, E = s.mlp == TGIS_MLP_MOE_SIGMOID ? s.experts : 0;
        l.norm1 = pnx_alloc<float>(W);
        l.shift = pnx_alloc<float>(W);
        l.gate_b = pnx_alloc<float>(2 * W, true);
        l.gates_cols = (int)((2 * W + E + 7) / 8 * 8);
        l.w_gates = pnx_alloc_dt((size_t)l.gates_cols * W, true);
        l.st_prev = pnx_alloc<float>(slots * W, true);
        pnx_expected_tensors += 4;  // norm1, shift, rg1, rg1.b
        if (E > 0) {
          const size_t ff = s.expert_ff, ffs = s.shared_ff;
          l.w_gu_e = pnx_alloc_dt(E * ff * W);     // up-projections, one [ff, width] matrix per expert
          l.w_d_e = pnx_alloc_dt(E * W * ff);
          pnx_expected_tensors += 3 + 2 * E;  // rg2, rg2.b, router, e<j>.{up, down}
          if (ffs > 0) {
            l.w_gu_s = pnx_alloc_dt(ffs * W);
            l.w_d_s = pnx_alloc_dt(W * ffs);
            pnx_expected_tensors += 2;  // shared.{up, down}
          }
          m_top = std::max<size_t>(m_top, s.top); m_ff = std::max(m_ff, ff); m_ffs = std::max(m_ffs, ffs);
        }
        m_E = std::max<size_t>(m_E, l.gates_cols);
        m_mix = std::max(m_mix, W);
        if (s.mixer == TGIS_MIXER_SIGMOID_ATTENTION) {
          const int H = s.heads, G = s.kv_heads;
          l.sa = SigAttnGeom{H, G, s.dim, s.vdim, s.window, s.rot_dims, s.scale};
          l.kv_src = s.kv_from > 0 ? s.kv_from - 1 : -1;
          l.c_q = 0; l.c_k = H * s.dim; l.c_v = l.c_k + G * s.dim;
          l.in_cols = ((l.kv_src >= 0 ? H * s.dim : l.c_v + G * s.vdim) + 7) / 8 * 8;
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_o = pnx_alloc_dt(W * H * s.vdim);
          l.head_bias = pnx_alloc<float>(H);
          l.cos_sin = s.rot_dims > 0 ? pnx_rope_table(s.rot_base, s.rot_dims, s.yarn_factor, s.yarn_original, s.yarn_fast, s.yarn_slow) : nullptr;
          pnx_expected_tensors += l.kv_src >= 0 ? 3 : 5;  // q, pb, o (+ k, v)
          m_q = std::max<size_t>(m_q, (size_t)H * s.dim);
          m_ov = std::max<size_t>(m_ov, (size_t)H * s.vdim);
          if (l.kv_src < 0) cache_row_bytes += (size_t)G * (s.dim + s.vdim) * dt_size(pnx_dt);
          pnx_tile_tokens = std::min(pnx_tile_tokens, SIGATTN_TILE);
        } else if (s.mixer == TGIS_MIXER_SSD) {
          const size_t inner = (size_t)s.heads * s.vdim, GN = (size_t)s.groups * s.state;
          l.conv_ch = (int)(inner + 2 * GN);
          l.in_cols = (int)((2 * inner + 2 * GN + s.heads + 7) / 8 * 8);
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_o = pnx_alloc_dt(W * inner);
          l.conv_w = pnx_alloc<float>((size_t)l.conv_ch * s.conv);
          l.conv_b = pnx_alloc<float>(l.conv_ch);
          l.dt_b = pnx_alloc<float>(s.heads);
          l.A_log = pnx_alloc<float>(s.heads);
          l.Dv = pnx_alloc<float>(s.heads);
          l.mm_norm = pnx_alloc<float>(inner);
          l.st_S = pnx_alloc<float>(slots * inner * s.state, true);
          l.st_conv = pnx_alloc<float>(slots * std::max(s.conv - 1, 1) * l.conv_ch, true);
          pnx_expected_tensors += 8;  // in, conv, conv.b, dt_bias, A_log, D, norm, o
          m_f1 = std::max<size_t>(m_f1, l.conv_ch); m_f2 = std::max(m_f2, inner);
        } else {  // TGIS_MIXER_CHANNEL_DELTA
          const size_t H = s.heads, G = s.kv_heads, qk = G * s.dim, hv = H * s.vdim, hd = H * s.dim;
          l.conv_ch = (int)(2 * qk + hv);
          l.c_q = 0; l.c_k = (int)qk; l.c_v = (int)(2 * qk); l.c_b = l.conv_ch; l.c_a1 = l.c_b + (int)H; l.c_g1 = l.c_a1 + s.decay_rank;
          l.in_cols = (l.c_g1 + s.gate_rank + 7) / 8 * 8;
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_w2 = pnx_alloc_dt(hd * s.decay_rank);
          l.w_g2 = pnx_alloc_dt(hv * s.gate_rank);
          l.w_o = pnx_alloc_dt(W * hv);
          l.conv_w = pnx_alloc<float>((size_t)l.conv_ch * s.conv);
          l.dt_b = pnx_alloc<float>(hd);
          l.A_log = pnx_alloc<float>(H);
          l.mm_norm = pnx_alloc<float>(hv);   // the per-head weight, repeated for every head
          l.st_S = pnx_alloc<float>(slots * hd * s.vdim, true);
          l.st_conv = pnx_alloc<float>(slots * std::max(s.conv - 1, 1) * l.conv_ch, true);
          pnx_expected_tensors += 15;  // q, q.conv, k, k.conv, v, v.conv, b, A_log, norm, a1, a2, dt_bias, g1, g2, o
          m_f1 = std::max<size_t>(m_f1, l.conv_ch); m_f2 = std::max(m_f2, hv); m_f3 = std::max(m_f3, hd + hv);
        }
        m_down = std::max<size_t>(m_down, l.in_cols);
        continue;
      }
      if (s.mlp == TGIS_MLP_DENSE_GELU) {
        l.norm2 = pnx_alloc<float>(W);
        l.w_gu = pnx_alloc_dt((size_t)2 * s.ff * W);
        l.w_d = pnx_alloc_dt(W * s.ff);
        pnx_expected_tensors += 4;  // norm2, mlp.gate, mlp.up, mlp.down
        m_ffs = std::max<size_t>(m_ffs, s.ff);
      }
      if (s.mixer != TGIS_MIXER_LATENT_ATTENTION) {
        l.norm1 = pnx_alloc<float>(W);
        pnx_expected_tensors += 1;
        const size_t slots = S_max;
        if (s.mixer == TGIS_MIXER_PARALLEL) {
          l.ca = CapAttnGeom{s.heads, s.kv_heads, s.dim, s.vdim, s.scale, s.softcap, s.qt_coef, s.qt_every};
          const int H = s.heads, G = s.kv_heads, mH = s.mm_heads;
          int col = 0;
          auto colsz = [&](int n) { const int r = col; col += n; return r; };
          l.c_q = colsz(H * s.dim); l.c_k = colsz(G * s.dim); l.c_v = colsz(G * s.vdim); l.c_g = colsz(H * s.vdim);
          l.c_mq = colsz(mH * s.mm_dim); l.c_mk = colsz(mH * s.mm_dim); l.c_mv = colsz(mH * s.mm_vdim);
          l.c_mg = colsz(mH * s.mm_vdim); l.c_mi = colsz(mH); l.c_mf = colsz(mH);
          l.in_cols = (col + 7) / 8 * 8;
          l.w_in = pnx_alloc_dt((size_t)l.in_cols * W, true);
          l.w_o = pnx_alloc_dt(W * H * s.vdim);
          l.w_o2 = pnx_alloc_dt(W * mH * s.mm_vdim);
          l.qk_norm = pnx_alloc<float>((size_t)2 * s.dim);
          l.mm_norm = pnx_alloc<float>((size_t)mH * s.mm_vdim);
          l.mm_bias = pnx_alloc<float>((size_t)2 * mH);
          l.out_l = pnx_alloc<float>(W);
          l.out_r = pnx_alloc<float>(W);
          l.st_S = pnx_alloc<float>(slots * mH * s.mm_dim * s.mm_vdim, true);
          l.st_n = pnx_alloc<float>(slots * mH * s.mm_dim, true);
          l.st_m = pnx_alloc<float>(slots * mH, true);
          pnx_expected_tensors += 19;  // left.{q,k,v,g,o,q.norm,k.norm,out}, right.{q,k,v,g,o,norm,i,i.b,f,f.b,out}
          m_q = std::max<size_t>(m_q, (size_t)H * s.dim);
          m_ov = std::max<size_t>(m_ov, (size_t)H * s.vdim);
          m_f1 = std::max<size_t>(m_f1, (size_t)mH * s.mm_vdim);
          cache_row_bytes += (size_t)G * (s.dim + s.vdim) * dt_size(pnx_dt);
          pnx_tile_tokens = std::min(pnx_tile_tokens, CAPATTN_TILE);
        } else if (s.mixer == TGIS_MIXER_SELECTIVE_SCAN) {
          const size_t I = s.inner, N = s.state, R = s.dt_rank;
          l.in_cols = (int)(2 * I);
          l.w_in = pnx_alloc_dt(2 * I * W);
          l.w_x = pnx_alloc_dt((R + 2 * N) * I);
          l.w_dt = pnx_alloc_dt(I * R);
          l.w_o = pnx_alloc_dt(W * I);
          l.conv_w = pnx_alloc<float>(I * s.conv);
          l.conv_b = pnx_alloc<float>(I);
          l.dt_b = pnx_alloc<float>(I);
          l.A_log = pnx_alloc<float>(I * N);
          l.Dv = pnx_alloc<float>(I);
          l.st_S = pnx_alloc<float>(slots * I * N, true);
          l.st_conv = pnx_alloc<float>(slots * std::max(s.conv - 1, 1) * I, true);
          pnx_expected_tensors += 9;  // in, conv, conv.b, x, dt, dt.b, A_log, D, o
          m_ov = std::max(m_ov, I);
          m_f1 = std::max(m_f1, I); m_f2 = std::max(m_f2, R + 2 * N); m_f3 = std::max(m_f3, I);
        } else {  // TGIS_MIXER_WKV
          const size_t A_ = (size_t)s.heads * s.dim, R = s.decay_rank;
          l.in_cols = (int)(4 * A_);
          l.w_in = pnx_alloc_dt(4 * A_ * W);
          l.w_w1 = pnx_alloc_dt(R * W);
          l.w_w2 = pnx_alloc_dt(A_ * R);
          l.w_o = pnx_alloc_dt(W * A_);
          l.mu = pnx_alloc<float>(5 * W);
          l.w0 = pnx_alloc<float>(A_);
          l.u = pnx_alloc<float>(A_);
          l.mm_norm = pnx_alloc<float>(A_);
          l.st_S = pnx_alloc<float>(slots * A_ * s.dim, true);
          l.st_prev = pnx_alloc<float>(slots * W, true);
          pnx_expected_tensors += 15;  // mu.{r,k,v,g,w}, r, k, v, g, w1, w2, w0, u, norm, o
          m_qr = std::max(m_qr, R);
          m_f1 = std::max(m_f1, A_); m_f2 = std::max(m_f2, A_); m_mix = std::max(m_mix, 5 * W);
        }
        m_down = std::max<size_t>(m_down, l.in_cols);
        continue;
      }
      l.g = LatentGeom{s.heads, s.dim, s.rot_dim, s.vdim, s.kv_rank, s.q_rank, s.window, s.rot_dims, s.scale};
      const size_t hd = (size_t)s.dim + s.rot_dim, row = (size_t)s.kv_rank + s.rot_dim;
      l.w_down = pnx_alloc_dt((size_t)l.n_down() * W);
      l.w_uq = pnx_alloc_dt((size_t)s.heads * hd * s.q_rank);
      l.w_ukT = pnx_alloc_dt((size_t)s.heads * s.kv_rank * s.dim);
      l.w_uv = pnx_alloc_dt((size_t)s.heads * s.vdim * s.kv_rank);
      l.w_o = pnx_alloc_dt(W * s.heads * s.vdim);
      l.norm1 = pnx_alloc<float>(W);
      l.norm1b = pnx_alloc<float>(W);
      l.qnorm = pnx_alloc<float>(s.q_rank);
      l.kvnorm = pnx_alloc<float>(s.kv_rank);
      l.cos_sin = pnx_rope_table(s.rot_base, s.rot_dims);
      pnx_expected_tensors += 11;  // norm1, norm1b, dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o
      if (s.mlp == TGIS_MLP_MOE) {
        const size_t E = s.experts, ff = s.expert_ff, ffs = s.shared_ff;
        l.norm2 = pnx_alloc<float>(W);
        l.norm2b = pnx_alloc<float>(W);
        l.w_router = pnx_alloc_dt((E + (ffs > 0 ? 1 : 0)) * W);
        l.router_b = pnx_alloc<float>(E);
        l.w_gu_e = pnx_alloc_dt(E * 2 * ff * W);
        l.w_d_e = pnx_alloc_dt(E * W * ff);
        pnx_expected_tensors += 4 + 3 * E;  // norm2, norm2b, router, router.b, e<j>.{gate, up, down}
        if (ffs > 0) {
          l.w_gu_s = pnx_alloc_dt(2 * ffs * W);
          l.w_d_s = pnx_alloc_dt(W * ffs);
          pnx_expected_tensors += 4;  // shared.{gate, up, down, sg}
        }
        m_E = std::max(m_E, E + 1); m_top = std::max<size_t>(m_top, s.top); m_ff = std::max(m_ff, ff); m_ffs = std::max(m_ffs, ffs);
      }
      m_down = std::max<size_t>(m_down, l.n_down()); m_qr = std::max<size_t>(m_qr, s.q_rank);
      m_q = std::max(m_q, s.heads * hd); m_qabs = std::max(m_qabs, s.heads * row);
      m_olat = std::max(m_olat, (size_t)s.heads * s.kv_rank); m_ov = std::max(m_ov, (size_t)s.heads * s.vdim);
      m_heads = std::max<size_t>(m_heads, s.heads);
      cache_row_bytes += row * dt_size(pnx_dt);
      pnx_tile_tokens = std::min(pnx_tile_tokens, latent_tile_tokens(s.heads));
    }
    if (pair_style) {
      // the layer runs: layers [loop_start, loop_stop) repeat loop_times passes in a row; every run owns cache rows and state
      const int L = (int)pnx_layers.size(), a = pnx_spec.loop_start, b = pnx_spec.loop_stop;
      const int passes = (pnx_spec.loop_times > 1 && b > a) ? pnx_spec.loop_times : 1;
      auto push = [&](int li, bool add) {
        pair_runs.push_back(pnx_layers[li]);
        pair_runs.back().add_x0 = add;
      };
      for (int li = 0; li < (passes > 1 ? a : L); ++li) push(li, false);
      if (passes > 1) {
        for (int p = 0; p < passes; ++p)
          for (int li = a; li < b; ++li) push(li, p > 0 && li == a);
        for (int li = b; li < L; ++li) push(li, false);
        pnx_x0 = pnx_alloc<float>(T * W);
      }
      for (PnxLayer& r : pair_runs) {
        const tgis_layer_spec& s = r.sp;
        if (s.mixer == TGIS_MIXER_POOLED_ATTENTION)
          cache_row_bytes += (size_t)s.kv_heads * (s.dim + s.vdim) * dt_size(pnx_dt);   // (+ the pooled rows: counted per block below)
        else if (s.mixer == TGIS_MIXER_LATENT_ATTENTION)
          cache_row_bytes += (size_t)r.g.row() * dt_size(pnx_dt);
        else
          r.st_S = pnx_alloc<float>((size_t)S_max * s.heads * s.dim * s.vdim, true);
      }
      if (pnx_spec.side_dim > 0) {
        pnx_side = pnx_alloc_dt(V * pnx_layers.size() * pnx_spec.side_dim);
        pnx_expected_tensors += 1;
      }
      pnx_hB = pnx_alloc_dt(T * W, true);
      if (const char* e = getenv("TGIS_PAIR_OVERLAP")) pair_overlap = atoi(e) != 0;
      if (pair_overlap) {
        CK(cudaStreamCreateWithFlags(&stream2, cudaStreamNonBlocking));
        CK(cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming));
        CK(cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming));
        gemm_ws2.alloc(gemm_workspace_bytes(num_sms) / sizeof(float));
        gemm_counters2.alloc(1 << 16);
        gemm_counters2.zero();
      }
    }
    // activations
    pnx_resid = pnx_alloc<float>(T * W);
    pnx_hA = pnx_alloc_dt(T * W, true);
    pnx_y1 = pnx_alloc<float>(T * m_down);
    pnx_cq = pnx_alloc_dt(T * m_qr, true);
    pnx_gate = pnx_alloc<float>(T * m_heads);
    pnx_q = pnx_alloc_dt(T * m_q, true);
    pnx_qabs = pnx_alloc<float>(T * m_qabs);
    pnx_olat = pnx_alloc_dt(T * m_olat, true);
    pnx_oA = pnx_alloc_dt(T * m_ov, true);
    pnx_o = pnx_alloc<float>(T * W);
    pnx_rl = pnx_alloc<float>(T * m_E);
    pnx_mixw = pnx_alloc<float>(T * m_top);
    pnx_sgate = pnx_alloc<float>(T);
    pnx_ids = pnx_alloc<int32_t>(T * m_top);
    pnx_order = pnx_alloc<int32_t>(T * m_top);
    pnx_inv = pnx_alloc<int32_t>(T * m_top);
    pnx_segoff = pnx_alloc<int32_t>(m_E + 1);
    pnx_actS = pnx_alloc_dt(T * m_ffs, true);
    pnx_yS = pnx_alloc<float>(T * W);
    pnx_actE = pnx_alloc_dt(T * m_top * m_ff, true);
    pnx_yE = pnx_alloc<float>(T * m_top * W);
    pnx_last = pnx_alloc_dt(std::max<size_t>(logit_rows_cap, T) * W, true);
    flx_f1 = pnx_alloc<float>(T * m_f1);
    flx_f2 = pnx_alloc<float>(T * m_f2);
    flx_f3 = pnx_alloc<float>(T * m_f3);
    flx_op2 = pnx_alloc_dt(T * std::max(m_f1, m_f2), true);
    flx_mix = pnx_alloc_dt(T * m_mix, true);
    if (gated_style) {
      rvp_n[0] = pnx_alloc<float>(T * W);
      rvp_n[1] = pnx_alloc<float>(T * W);
    }
    if (pnx_dt == DT_BF16) {
      pnx_attn_ws_floats = (size_t)8 << 20;  // 32 MB
      pnx_attn_ws = pnx_alloc<float>(pnx_attn_ws_floats);
    }
    // paged cache of latent rows: the block ids of the engine's block manager index every layer's cache
    size_t kv_bytes = c.kv_cache_bytes;
    if (kv_bytes == 0) {
      size_t free_b = 0, total_b = 0;
      CK(cudaMemGetInfo(&free_b, &total_b));
      kv_bytes = (size_t)(free_b * (double)(c.gpu_mem_fraction > 0 ? c.gpu_mem_fraction : 0.85f));
    }
    size_t bytes_per_block = (size_t)KV_BLOCK * cache_row_bytes;
    for (PnxLayer& r : pair_runs)   // pooled rows of the windowed attention runs
      if (r.sp.mixer == TGIS_MIXER_POOLED_ATTENTION)
        bytes_per_block += (size_t)r.pa.rows_per_page() * r.pa.kv_heads * (r.pa.dim + r.pa.vdim) * dt_size(pnx_dt);
    size_t nb = std::min(kv_bytes / std::max<size_t>(bytes_per_block, 1), (size_t)S_max * bt_stride + 1);
    if (nb < 1) throw CudaError("cache too small for one block");
    num_blocks = (int)nb;
    for (PnxLayer& l : pnx_layers) {  // finite everywhere
      if (pair_style) break;   // (the layer runs own the caches)
      if (l.sp.mixer == TGIS_MIXER_LATENT_ATTENTION) l.cache = pnx_alloc_dt(nb * KV_BLOCK * l.g.row(), true);
      if (l.sp.mixer == TGIS_MIXER_PARALLEL) {
        l.k_cache = pnx_alloc_dt(nb * KV_BLOCK * l.ca.kv_heads * l.ca.dim, true);
        l.v_cache = pnx_alloc_dt(nb * KV_BLOCK * l.ca.kv_heads * l.ca.vdim, true);
      }
      if (l.sp.mixer == TGIS_MIXER_SIGMOID_ATTENTION) {
        if (l.kv_src >= 0) {   // the rows another (earlier) layer writes
          l.k_cache = pnx_layers[l.kv_src].k_cache;
          l.v_cache = pnx_layers[l.kv_src].v_cache;
        } else {
          l.k_cache = pnx_alloc_dt(nb * KV_BLOCK * l.sa.kv_heads * l.sa.dim, true);
          l.v_cache = pnx_alloc_dt(nb * KV_BLOCK * l.sa.kv_heads * l.sa.vdim, true);
        }
      }
    }
    for (PnxLayer& r : pair_runs) {
      if (r.sp.mixer == TGIS_MIXER_LATENT_ATTENTION) r.cache = pnx_alloc_dt(nb * KV_BLOCK * r.g.row(), true);
      if (r.sp.mixer == TGIS_MIXER_POOLED_ATTENTION) {
        r.k_cache = pnx_alloc_dt(nb * KV_BLOCK * r.pa.kv_heads * r.pa.dim, true);
        r.v_cache = pnx_alloc_dt(nb * KV_BLOCK * r.pa.kv_heads * r.pa.vdim, true);
        if (r.pa.pool > 0) {
          r.pk_cache = pnx_alloc_dt(nb * r.pa.rows_per_page() * r.pa.kv_heads * r.pa.dim, true);
          r.pv_cache = pnx_alloc_dt(nb * r.pa.rows_per_page() * r.pa.kv_heads * r.pa.vdim, true);
        }
      }
    }
    free_blocks.resize(num_blocks);
    for (int i = 0; i < num_blocks; ++i) free_blocks[i] = num_blocks - 1 - i;
  }

  int pnx_load_weight(const std::string& name, const void* ptr, int64_t rows, int64_t cols) {
    const int64_t W = cfg.hidden, V = cfg.vocab;
    const int64_t n = rows * cols;
    // the checkpoint tensor (bf16, host or device) -> device scratch -> its place in the operand type
    bf16* tmp_src = nullptr;
    if (cudaMalloc(&tmp_src, (size_t)std::max<int64_t>(n, 1) * sizeof(bf16)) != cudaSuccess) return fail("cudaMalloc(scratch) failed");
    struct Guard { bf16* p; ~Guard() { cudaFree(p); } } guard{tmp_src};
    if (cudaMemcpy(tmp_src, ptr, (size_t)n * sizeof(bf16), cudaMemcpyDefault) != cudaSuccess) return fail("cudaMemcpy(weight) failed");
    auto bad_shape = [&]() { return fail("shape mismatch for " + name + ": got " + std::to_string(rows) + "x" + std::to_string(cols)); };
    // src viewed as [r, cc] -> dst[r * rs + c * cs]
    auto place = [&](void* dst, int dt, int64_t r, int64_t cc, int64_t rs, int64_t cs) -> int {
      if (r * cc != n) return bad_shape();
      const cudaError_t e = weight_place_launch(tmp_src, (int)r, (int)cc, dst, dt, rs, cs, 0);
      if (e != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return fail("weight placement failed for " + name);
      pnx_loaded.insert(name);
      return 0;
    };
    auto at = [&](void* base, size_t elem_off) { return reinterpret_cast<uint8_t*>(base) + elem_off * dt_size(pnx_dt); };
    auto mat = [&](void* dst, int64_t r, int64_t cc) { return place(dst, pnx_dt, r, cc, cc, 1); };
    auto vec = [&](float* dst, int64_t len) { return place(dst, DT_F32, len, 1, 1, 1); };
    // a norm that carries ONE number: kept as a row of `len` equal entries
    auto one = [&](float* dst, int64_t len) -> int {
      if (n != 1) return bad_shape();
      uint16_t bits = 0;
      if (cudaMemcpy(&bits, tmp_src, sizeof(bits), cudaMemcpyDeviceToHost) != cudaSuccess) return fail("weight placement failed for " + name);
      const uint32_t wide = (uint32_t)bits << 16;   // bf16 -> fp32
      float v;
      memcpy(&v, &wide, sizeof(v));
      const std::vector<float> row((size_t)len, v);
      if (cudaMemcpy(dst, row.data(), row.size() * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
        return fail("weight placement failed for " + name);
      pnx_loaded.insert(name);
      return 0;
    };
    // [heads * dim, kv_rank] -> per head the transpose [kv_rank, dim]: the matrix that folds a key up-projection into the query
    auto place_ukT = [&](void* dst, int heads, int dim, int kv_rank) -> int {
      if (n != (int64_t)heads * dim * kv_rank) return bad_shape();
      for (int h = 0; h < heads; ++h) {
        const cudaError_t e = weight_place_launch(tmp_src + (size_t)h * dim * kv_rank, dim, kv_rank,
                                                  at(dst, (size_t)h * kv_rank * dim), pnx_dt, 1, dim, 0);
        if (e != cudaSuccess) return fail("weight placement failed for " + name);
      }
      if (cudaDeviceSynchronize() != cudaSuccess) return fail("weight placement failed for " + name);
      pnx_loaded.insert(name);
      return 0;
    };
    // one weight of `len` entries for all heads: kept once per head
    auto per_head = [&](float* dst, int heads, int len) -> int {
      if (n != len) return bad_shape();
      for (int h = 0; h < heads; ++h)
        if (weight_place_launch(tmp_src, len, 1, dst + (size_t)h * len, DT_F32, 1, 1, 0) != cudaSuccess)
          return fail("weight placement failed for " + name);
      if (cudaDeviceSynchronize() != cudaSuccess) return fail("weight placement failed for " + name);
      pnx_loaded.insert(name);
      return 0;
    };
    if (name == "embed") return mat(pnx_embed, V, W);
    if (name == "head" && !tied_head) return mat(pnx_head, V, W);
    if (name == "final.norm") return pair_style ? one(pnx_final_norm, W) : vec(pnx_final_norm, W);
    if (name == "side.embed" && pnx_side != nullptr) return mat(pnx_side, V, (int64_t)pnx_layers.size() * pnx_spec.side_dim);
    if (name.size() < 3 || name[0] != 'l') return fail("unknown weight " + name);
    const size_t dot = name.find('.');
    if (dot == std::string::npos) return fail("unknown weight " + name);
    const int li = atoi(name.substr(1, dot - 1).c_str());
    if (li < 0 || li >= (int)pnx_layers.size()) return fail("layer index out of range in " + name);
    PnxLayer& l = pnx_layers[li];
    const tgis_layer_spec& s = l.sp;
    const std::string sub = name.substr(dot + 1);
    if (pair_style) {
      auto in_rows = [&](int col, int64_t r) { return mat(at(l.w_in, (size_t)col * W), r, W); };
      const int64_t sd = pnx_spec.side_dim;
      if (sub == "norm1") return one(l.norm1, W);
      if (s.mlp == TGIS_MLP_DENSE_SILU) {
        // gate / up rows interleave (row 2j = gate_j, row 2j + 1 = up_j): one product, the gated activation in its epilogue
        if (sub == "norm2") return one(l.norm2, W);
        if (sub == "mlp.gate") return place(l.w_gu, pnx_dt, s.ff, W, 2 * W, 1);
        if (sub == "mlp.up") return place(at(l.w_gu, (size_t)W), pnx_dt, s.ff, W, 2 * W, 1);
        if (sub == "mlp.down") return mat(l.w_d, W, s.ff);
      }
      if (sd > 0) {
        if (sub == "side.gate") return mat(l.w_sg, sd, W);
        if (sub == "side.proj") return mat(l.w_sp, W, sd);
        if (sub == "side.norm") return vec(l.side_norm, W);
      }
      if (s.mixer == TGIS_MIXER_POOLED_ATTENTION) {
        const int64_t H = s.heads, G = s.kv_heads;
        if (sub == "mix.q") return in_rows(l.c_q, H * s.dim);
        if (sub == "mix.k") return in_rows(l.c_k, G * s.dim);
        if (sub == "mix.v") return in_rows(l.c_v, G * s.vdim);
        if (l.in_bias != nullptr) {
          if (sub == "mix.q.b") return vec(l.in_bias + l.c_q, H * s.dim);
          if (sub == "mix.k.b") return vec(l.in_bias + l.c_k, G * s.dim);
          if (sub == "mix.v.b") return vec(l.in_bias + l.c_v, G * s.vdim);
        }
        if (sub == "mix.o") return mat(l.w_o, W, H * s.vdim);
      } else if (s.mixer == TGIS_MIXER_HGRN) {
        const int64_t hd = (int64_t)s.heads * s.dim, hv = (int64_t)s.heads * s.vdim;
        if (sub == "mix.q") return in_rows(l.c_q, hd);
        if (sub == "mix.f") return in_rows(l.c_f, hd);
        if (sub == "mix.v") return in_rows(l.c_v, hv);
        if (sub == "mix.f.b") return vec(l.w0, hd);
        if (sub == "mix.lower") return vec(l.u, hd);
        if (sub == "mix.norm") return per_head(l.mm_norm, s.heads, s.vdim);
        if (sub == "mix.o") return mat(l.w_o, W, hv);
      } else {
        const int64_t hd = s.dim + s.rot_dim;
        if (sub == "mix.dq") return mat(l.w_down, s.q_rank, W);
        if (sub == "mix.dkv") return mat(at(l.w_down, (size_t)s.q_rank * W), s.kv_rank + s.rot_dim, W);
        if (sub == "mix.g" && l.out_gate) return mat(at(l.w_down, (size_t)(s.q_rank + s.kv_rank + s.rot_dim) * W), s.heads, W);
        if (sub == "mix.dq.norm") return vec(l.qnorm, s.q_rank);
        if (sub == "mix.dkv.norm") return vec(l.kvnorm, s.kv_rank);
        if (sub == "mix.uq") return mat(l.w_uq, s.heads * hd, s.q_rank);
        if (sub == "mix.uk") return place_ukT(l.w_ukT, s.heads, s.dim, s.kv_rank);
        if (sub == "mix.uv") return mat(l.w_uv, (int64_t)s.heads * s.vdim, s.kv_rank);
        if (sub == "mix.sink" && l.sink != nullptr) return vec(l.sink, s.heads);
        if (sub == "mix.o") return mat(l.w_o, W, (int64_t)s.heads * s.vdim);
      }
      return fail("unknown layer weight " + name);
    }
    if (sub == "norm1") return vec(l.norm1, W);
    if (s.mlp == TGIS_MLP_DENSE_GELU) {
      // gate / up rows interleave (row 2j = gate_j, row 2j + 1 = up_j): one product, the gated activation in its epilogue
      if (sub == "norm2") return vec(l.norm2, W);
      if (sub == "mlp.gate") return place(l.w_gu, pnx_dt, s.ff, W, 2 * W, 1);
      if (sub == "mlp.up") return place(at(l.w_gu, (size_t)W), pnx_dt, s.ff, W, 2 * W, 1);
      if (sub == "mlp.down") return mat(l.w_d, W, s.ff);
    }
    auto in_rows = [&](int col, int64_t r) { return mat(at(l.w_in, (size_t)col * W), r, W); };
    if (gated_style) {
      const bool moe = s.mlp == TGIS_MLP_MOE_SIGMOID;
      if (sub == "shift") return vec(l.shift, W);
      if (sub == "rg1") return mat(l.w_gates, W, W);
      if (sub == "rg1.b") return vec(l.gate_b, W);
      if (sub == "rg2" || sub == "rg2.b") {
        if (!moe) return rows * cols == (sub == "rg2" ? W * W : W) ? 0 : bad_shape();   // a gate with nothing to gate: not kept
        return sub == "rg2" ? mat(at(l.w_gates, (size_t)W * W), W, W) : vec(l.gate_b + W, W);
      }
      if (moe) {
        const int64_t E = s.experts, ff = s.expert_ff, ffs = s.shared_ff;
        if (sub == "mlp.router") return mat(at(l.w_gates, (size_t)2 * W * W), E, W);
        if (ffs > 0 && sub == "mlp.shared.up") return mat(l.w_gu_s, ffs, W);
        if (ffs > 0 && sub == "mlp.shared.down") return mat(l.w_d_s, W, ffs);
        if (sub.rfind("mlp.e", 0) == 0) {
          const size_t d2 = sub.find('.', 5);
          if (d2 == std::string::npos) return fail("unknown layer weight " + name);
          const int ei = atoi(sub.substr(5, d2 - 5).c_str());
          if (ei < 0 || ei >= E) return fail("expert index out of range in " + name);
          const std::string which = sub.substr(d2 + 1);
          if (which == "up") return mat(at(l.w_gu_e, (size_t)ei * ff * W), ff, W);
          if (which == "down") return mat(at(l.w_d_e, (size_t)ei * W * ff), W, ff);
        }
      }
      if (s.mixer == TGIS_MIXER_SIGMOID_ATTENTION) {
        const int64_t H = s.heads, G = s.kv_heads;
        if (sub == "mix.q") return in_rows(l.c_q, H * s.dim);
        if (sub == "mix.k" && l.kv_src < 0) return in_rows(l.c_k, G * s.dim);
        if (sub == "mix.v" && l.kv_src < 0) return in_rows(l.c_v, G * s.vdim);
        if (sub == "mix.pb") return vec(l.head_bias, H);
        if (sub == "mix.o") return mat(l.w_o, W, H * s.vdim);
      } else if (s.mixer == TGIS_MIXER_SSD) {
        const int64_t inner = (int64_t)s.heads * s.vdim, GN = (int64_t)s.groups * s.state;
        if (sub == "mix.in") return mat(l.w_in, 2 * inner + 2 * GN + s.heads, W);
        if (sub == "mix.conv") return place(l.conv_w, DT_F32, l.conv_ch, s.conv, s.conv, 1);
        if (sub == "mix.conv.b") return vec(l.conv_b, l.conv_ch);
        if (sub == "mix.dt_bias") return vec(l.dt_b, s.heads);
        if (sub == "mix.A_log") return vec(l.A_log, s.heads);
        if (sub == "mix.D") return vec(l.Dv, s.heads);
        if (sub == "mix.norm") return vec(l.mm_norm, inner);
        if (sub == "mix.o") return mat(l.w_o, W, inner);
      } else {  // TGIS_MIXER_CHANNEL_DELTA
        const int64_t H = s.heads, qk = (int64_t)s.kv_heads * s.dim, hv = H * s.vdim, hd = H * s.dim;
        if (sub == "mix.q") return in_rows(l.c_q, qk);
        if (sub == "mix.k") return in_rows(l.c_k, qk);
        if (sub == "mix.v") return in_rows(l.c_v, hv);
        if (sub == "mix.b") return in_rows(l.c_b, H);
        if (sub == "mix.a1") return in_rows(l.c_a1, s.decay_rank);
        if (sub == "mix.g1") return in_rows(l.c_g1, s.gate_rank);
        if (sub == "mix.q.conv") return place(l.conv_w + (size_t)l.c_q * s.conv, DT_F32, qk, s.conv, s.conv, 1);
        if (sub == "mix.k.conv") return place(l.conv_w + (size_t)l.c_k * s.conv, DT_F32, qk, s.conv, s.conv, 1);
        if (sub == "mix.v.conv") return place(l.conv_w + (size_t)l.c_v * s.conv, DT_F32, hv, s.conv, s.conv, 1);
        if (sub == "mix.a2") return mat(l.w_w2, hd, s.decay_rank);
        if (sub == "mix.g2") return mat(l.w_g2, hv, s.gate_rank);
        if (sub == "mix.dt_bias") return vec(l.dt_b, hd);
        if (sub == "mix.A_log") return vec(l.A_log, H);
        if (sub == "mix.o") return mat(l.w_o, W, hv);
        if (sub == "mix.norm") {   // one weight of vdim entries for all heads: kept once per head
          if (n != s.vdim) return bad_shape();
          for (int h = 0; h < H; ++h)
            if (weight_place_launch(tmp_src, s.vdim, 1, l.mm_norm + (size_t)h * s.vdim, DT_F32, 1, 1, 0) != cudaSuccess)
              return fail("weight placement failed for " + name);
          if (cudaDeviceSynchronize() != cudaSuccess) return fail("weight placement failed for " + name);
          pnx_loaded.insert(name);
          return 0;
        }
      }
      return fail("unknown layer weight " + name);
    }
    if (s.mixer == TGIS_MIXER_PARALLEL) {
      const int64_t H = s.heads, G = s.kv_heads, mH = s.mm_heads;
      if (sub == "mix.left.q") return in_rows(l.c_q, H * s.dim);
      if (sub == "mix.left.k") return in_rows(l.c_k, G * s.dim);
      if (sub == "mix.left.v") return in_rows(l.c_v, G * s.vdim);
      if (sub == "mix.left.g") return in_rows(l.c_g, H * s.vdim);
      if (sub == "mix.left.o") return mat(l.w_o, W, H * s.vdim);
      if (sub == "mix.left.q.norm") return vec(l.qk_norm, s.dim);
      if (sub == "mix.left.k.norm") return vec(l.qk_norm + s.dim, s.dim);
      if (sub == "mix.left.out") return vec(l.out_l, W);
      if (sub == "mix.right.q") return in_rows(l.c_mq, mH * s.mm_dim);
      if (sub == "mix.right.k") return in_rows(l.c_mk, mH * s.mm_dim);
      if (sub == "mix.right.v") return in_rows(l.c_mv, mH * s.mm_vdim);
      if (sub == "mix.right.g") return in_rows(l.c_mg, mH * s.mm_vdim);
      if (sub == "mix.right.i") return in_rows(l.c_mi, mH);
      if (sub == "mix.right.f") return in_rows(l.c_mf, mH);
      if (sub == "mix.right.i.b") return vec(l.mm_bias, mH);
      if (sub == "mix.right.f.b") return vec(l.mm_bias + mH, mH);
      if (sub == "mix.right.o") return mat(l.w_o2, W, mH * s.mm_vdim);
      if (sub == "mix.right.norm") return vec(l.mm_norm, mH * s.mm_vdim);
      if (sub == "mix.right.out") return vec(l.out_r, W);
      return fail("unknown layer weight " + name);
    }
    if (s.mixer == TGIS_MIXER_SELECTIVE_SCAN) {
      const int64_t I = s.inner, N = s.state, R = s.dt_rank;
      if (sub == "mix.in") return mat(l.w_in, 2 * I, W);
      if (sub == "mix.conv") return place(l.conv_w, DT_F32, I, s.conv, s.conv, 1);
      if (sub == "mix.conv.b") return vec(l.conv_b, I);
      if (sub == "mix.x") return mat(l.w_x, R + 2 * N, I);
      if (sub == "mix.dt") return mat(l.w_dt, I, R);
      if (sub == "mix.dt.b") return vec(l.dt_b, I);
      if (sub == "mix.A_log") return place(l.A_log, DT_F32, I, N, N, 1);
      if (sub == "mix.D") return vec(l.Dv, I);
      if (sub == "mix.o") return mat(l.w_o, W, I);
      return fail("unknown layer weight " + name);
    }
    if (s.mixer == TGIS_MIXER_WKV) {
      const int64_t A_ = (int64_t)s.heads * s.dim, R = s.decay_rank;
      static const char* const kMix[5] = {"r", "k", "v", "g", "w"};
      for (int j = 0; j < 5; ++j) {
        if (sub == std::string("mix.mu.") + kMix[j]) return vec(l.mu + (size_t)j * W, W);
        if (j < 4 && sub == std::string("mix.") + kMix[j]) return in_rows((int)(j * A_), A_);
      }
      if (sub == "mix.w1") return mat(l.w_w1, R, W);
      if (sub == "mix.w2") return mat(l.w_w2, A_, R);
      if (sub == "mix.w0") return vec(l.w0, A_);
      if (sub == "mix.u") return vec(l.u, A_);
      if (sub == "mix.norm") return vec(l.mm_norm, A_);
      if (sub == "mix.o") return mat(l.w_o, W, A_);
      return fail("unknown layer weight " + name);
    }
    const int64_t hd = s.dim + s.rot_dim;
    if (sub == "norm1b") return vec(l.norm1b, W);
    if (sub == "mix.dq") return mat(l.w_down, s.q_rank, W);
    if (sub == "mix.dkv") return mat(at(l.w_down, (size_t)s.q_rank * W), s.kv_rank + s.rot_dim, W);
    if (sub == "mix.g") return mat(at(l.w_down, (size_t)(s.q_rank + s.kv_rank + s.rot_dim) * W), s.heads, W);
    if (sub == "mix.dq.norm") return vec(l.qnorm, s.q_rank);
    if (sub == "mix.dkv.norm") return vec(l.kvnorm, s.kv_rank);
    if (sub == "mix.uq") return mat(l.w_uq, s.heads * hd, s.q_rank);
    if (sub == "mix.uk") {
      // [heads * dim, kv_rank] -> per head the transpose [kv_rank, dim]: the matrix that folds W_uk into the query
      if (n != (int64_t)s.heads * s.dim * s.kv_rank) return bad_shape();
      for (int h = 0; h < s.heads; ++h) {
        const cudaError_t e = weight_place_launch(tmp_src + (size_t)h * s.dim * s.kv_rank, s.dim, s.kv_rank,
                                                  at(l.w_ukT, (size_t)h * s.kv_rank * s.dim), pnx_dt, 1, s.dim, 0);
        if (e != cudaSuccess) return fail("weight placement failed for " + name);
      }
      if (cudaDeviceSynchronize() != cudaSuccess) return fail("weight placement failed for " + name);
      pnx_loaded.insert(name);
      return 0;
    }
    if (sub == "mix.uv") return mat(l.w_uv, (int64_t)s.heads * s.vdim, s.kv_rank);
    if (sub == "mix.o") return mat(l.w_o, W, (int64_t)s.heads * s.vdim);
    if (s.mlp != TGIS_MLP_MOE) return fail("unknown layer weight " + name);
    const int64_t E = s.experts, ff = s.expert_ff, ffs = s.shared_ff;
    if (sub == "norm2") return vec(l.norm2, W);
    if (sub == "norm2b") return vec(l.norm2b, W);
    if (sub == "mlp.router") return mat(l.w_router, E, W);
    if (sub == "mlp.router.b") return vec(l.router_b, E);
    if (ffs > 0) {
      if (sub == "mlp.shared.sg") return mat(at(l.w_router, (size_t)E * W), 1, W);
      // gate / up rows interleave (row 2j = gate_j, row 2j + 1 = up_j) so that one product's epilogue applies SwiGLU
      if (sub == "mlp.shared.gate") return place(l.w_gu_s, pnx_dt, ffs, W, 2 * W, 1);
      if (sub == "mlp.shared.up") return place(at(l.w_gu_s, (size_t)W), pnx_dt, ffs, W, 2 * W, 1);
      if (sub == "mlp.shared.down") return mat(l.w_d_s, W, ffs);
    }
    if (sub.rfind("mlp.e", 0) == 0) {
      const size_t d2 = sub.find('.', 5);
      if (d2 == std::string::npos) return fail("unknown layer weight " + name);
      const int ei = atoi(sub.substr(5, d2 - 5).c_str());
      if (ei < 0 || ei >= E) return fail("expert index out of range in " + name);
      const std::string which = sub.substr(d2 + 1);
      if (which == "gate") return place(at(l.w_gu_e, (size_t)ei * 2 * ff * W), pnx_dt, ff, W, 2 * W, 1);
      if (which == "up") return place(at(l.w_gu_e, (size_t)ei * 2 * ff * W + W), pnx_dt, ff, W, 2 * W, 1);
      if (which == "down") return mat(at(l.w_d_e, (size_t)ei * W * ff), W, ff);
    }
    return fail("unknown layer weight " + name);
  }

  // Dense Y = X W^T.  bf16 operands in the tcgen05 kernel's layout (whole 64-element k-blocks, at least four of them -- the
  // range its stream-K schedules are tested in --, at least one full weight tile)
  // go to that kernel -- fp32 accumulators out, or SwiGLU fused over interleaved gate / up rows --, everything else to the
  // general kernel.  Tensor maps are made on first use and kept (one per weight; one per activation buffer, width and
  // token-tile height).  TGIS_PNX_TC=0: general kernel only.
  std::unordered_map<const void*, CUtensorMap> pnx_wmaps;
  std::unordered_map<uint64_t, CUtensorMap> pnx_xmaps;
  bool pnx_tc = true;
  size_t pnx_rows_alloc = 0;  // rows of every activation buffer (>= 256: a TMA box never leaves the allocation)
  bool pnx_gemm_tc(const void* X, const void* Wt, void* Y, int ldy, int T, int N, int K, int out_mode) {
    auto wit = pnx_wmaps.find(Wt);
    if (wit == pnx_wmaps.end()) {
      CUtensorMap m;
      if (make_tmap_bf16_2d(&m, Wt, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128, 64) != 0) return false;
      wit = pnx_wmaps.emplace(Wt, m).first;
    }
    const int bi = bt_index(T);
    const uint64_t xkey = (reinterpret_cast<uint64_t>(X) << 3) ^ ((uint64_t)K << 44) ^ (uint64_t)bi;
    auto xit = pnx_xmaps.find(xkey);
    if (xit == pnx_xmaps.end()) {
      CUtensorMap m;
      if (make_tmap_bf16_2d(&m, X, (uint64_t)pnx_rows_alloc, (uint64_t)K, (uint64_t)K, BT_VALUES[bi], 64) != 0) return false;
      xit = pnx_xmaps.emplace(xkey, m).first;
    }
    CK(gemm_bf16_launch(wit->second, xit->second, Y, ldy, T, N, K, on_side_stream ? gemm_ws2.p : gemm_ws.p,
                        on_side_stream ? gemm_counters2.p : gemm_counters.p, num_sms, on_side_stream ? stream2 : stream, out_mode));
    ++n_launches;
    return true;
  }
  void pnx_gemm(const void* X, int x_dt, int ldx, const void* Wt, void* Y, int y_dt, int ldy, int T, int N, int K,
                int mode = GEMM_ANY_PLAIN, bool x_tma_ok = true) {
    if (pnx_tc && x_tma_ok && pnx_dt == DT_BF16 && x_dt == DT_BF16 && ldx == K && K % 64 == 0 && K >= 256 && N % 8 == 0 &&
        N >= 128 && !cfg.debug_gemm_ref && (reinterpret_cast<uintptr_t>(Y) & 15) == 0 && (reinterpret_cast<uintptr_t>(X) & 15) == 0) {
      const int out_mode = mode == GEMM_ANY_SWIGLU && y_dt == DT_BF16 ? 2 : mode == GEMM_ANY_GEGLU && y_dt == DT_BF16 ? 3
                           : mode == GEMM_ANY_RELU2 && y_dt == DT_BF16 ? 4
                           : mode == GEMM_ANY_PLAIN ? (y_dt == DT_F32 ? 1 : 0) : -1;
      if (out_mode >= 0 && pnx_gemm_tc(X, Wt, Y, ldy, T, N, K, out_mode)) return;
    }
    GemmAny a{};
    a.X = X; a.W = Wt; a.Y = Y;
    a.x_dtype = x_dt; a.w_dtype = pnx_dt; a.y_dtype = y_dt;
    a.T = T; a.N = N; a.K = K; a.ldx = ldx; a.ldw = K; a.ldy = ldy;
    a.batch = 1; a.mode = mode;
    CK(gemm_any_launch(a, on_side_stream ? stream2 : stream));
    ++n_launches;
  }

  void pnx_dump_resid(int T) {
    if (pnx_dump_path.empty() || capturing) return;
    CK(cudaStreamSynchronize(stream));
    std::vector<float> hbuf((size_t)T * cfg.hidden);
    CK(cudaMemcpy(hbuf.data(), pnx_resid, hbuf.size() * sizeof(float), cudaMemcpyDeviceToHost));
    if (FILE* f = fopen(pnx_dump_path.c_str(), "ab")) {
      fwrite(hbuf.data(), sizeof(float), hbuf.size(), f);
      fclose(f);
    }
  }

  // One layer of a post-norm stack (TGIS_STYLE_POST_NORM): x += rmsnorm(mixer(x)) * norm1, x += rmsnorm(ff(x)) * norm2.
  // pnx_hA holds the stream in the operand type on entry and on exit (after the last layer: the final norm's output).
  // T tokens of S sequences, any mix of whole prompts, portions and single tokens.
  void stream_layer(int li, int T, int S) {
    PnxLayer& l = pnx_layers[li];
    const tgis_layer_spec& s = l.sp;
    const int W = cfg.hidden, A = pnx_dt;
    const float eps = pnx_spec.norm_eps;
    const int32_t* d_pos = ds<int32_t>(off_pos);
    const int32_t* d_slot = ds<int32_t>(off_slotmap);
    const int32_t* d_tokslot = ds<int32_t>(off_tokslot);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const bool has_ff = s.mlp == TGIS_MLP_DENSE_GELU;
    const bool last = li + 1 == (int)pnx_layers.size();
    ResidTail rt{};
    rt.resid = pnx_resid; rt.out = pnx_hA; rt.out_dtype = A; rt.mult = 1.f; rt.w_off = 0.f; rt.eps = eps;
    rt.w_post = l.norm1;
    rt.w_pre = (last && !has_ff) ? pnx_final_norm : nullptr;
    rt.cast_out = 1;
    if (s.mixer == TGIS_MIXER_PARALLEL) {
      const int H = s.heads, mH = s.mm_heads, ld = l.in_cols;
      // every projection of both sides in one product: [q | k | v | gate | q' | k' | v' | gate' | i | f]
      pnx_gemm(pnx_hA, A, W, l.w_in, pnx_y1, DT_F32, ld, T, ld, W);
      CK(capattn_prep_launch(pnx_y1, ld, l.c_q, l.c_k, l.c_v, l.ca, l.qk_norm, l.qk_norm + s.dim, eps, d_pos, d_slot, pnx_q,
                             l.k_cache, l.v_cache, A, T, stream));
      CK(capattn_launch(pnx_q, l.k_cache, l.v_cache, A, d_seqs, ds<LatentTile>(off_ltiles), step_n_ltiles, ds<int32_t>(off_bt),
                        bt_stride, pnx_y1 + l.c_g, ld, pnx_oA, A, l.ca, stream));
      pnx_gemm(pnx_oA, A, H * s.vdim, l.w_o, pnx_o, DT_F32, W, T, W, H * s.vdim);
      OuterScan os{};
      os.mode = OUTER_SCAN_GATED;
      os.q = pnx_y1 + l.c_mq; os.k = pnx_y1 + l.c_mk; os.v = pnx_y1 + l.c_mv; os.ldq = os.ldk = os.ldv = ld;
      os.q_scale = 1.f / std::sqrt((float)s.mm_dim);
      os.ig = pnx_y1 + l.c_mi; os.fg = pnx_y1 + l.c_mf; os.ldg = ld; os.ig_b = l.mm_bias; os.fg_b = l.mm_bias + mH;
      os.gate_cap = s.gate_cap;
      os.S = l.st_S; os.n = l.st_n; os.m = l.st_m;
      os.out = flx_f1; os.ldo = mH * s.mm_vdim;
      os.heads = mH; os.dim = s.mm_dim; os.vdim = s.mm_vdim;
      CK(outer_scan_launch(os, d_seqs, S, d_tokslot, stream));
      CK(head_norm_gate_launch(flx_f1, mH * s.mm_vdim, mH, s.mm_vdim, l.mm_norm, pnx_y1 + l.c_mg, ld, /*sigmoid*/ 0, eps, flx_op2,
                               A, T, stream));
      n_launches += 4;
      pnx_gemm(flx_op2, A, mH * s.mm_vdim, l.w_o2, pnx_yS, DT_F32, W, T, W, mH * s.mm_vdim);
      rt.y_main = pnx_o; rt.y_pair = pnx_yS; rt.w_main = l.out_l; rt.w_pair = l.out_r;
    } else if (s.mixer == TGIS_MIXER_SELECTIVE_SCAN) {
      const int I = s.inner, N = s.state, R = s.dt_rank;
      pnx_gemm(pnx_hA, A, W, l.w_in, pnx_y1, DT_F32, 2 * I, T, 2 * I, W);
      CK(short_conv_silu_launch(pnx_y1, 2 * I, I, l.conv_w, l.conv_b, s.conv, d_pos, d_tokslot, l.st_conv, flx_f1,
                                A == DT_F32 ? nullptr : pnx_oA, A, T, stream));
      const void* xc = A == DT_F32 ? (const void*)flx_f1 : (const void*)pnx_oA;
      pnx_gemm(xc, A, I, l.w_x, flx_f2, DT_F32, R + 2 * N, T, R + 2 * N, I);
      pnx_gemm(flx_f2, DT_F32, R + 2 * N, l.w_dt, flx_f3, DT_F32, I, T, I, R);
      SelScan sc{};
      sc.x = flx_f1; sc.xz = pnx_y1; sc.ld_xz = 2 * I; sc.proj = flx_f2; sc.ld_proj = R + 2 * N; sc.dt_rank = R;
      sc.dt_raw = flx_f3; sc.dt_b = l.dt_b; sc.A_log = l.A_log; sc.D = l.Dv; sc.S = l.st_S; sc.conv_state = l.st_conv;
      sc.out = flx_op2; sc.out_dtype = A; sc.inner = I; sc.state = N; sc.taps = s.conv;
      CK(selective_scan_launch(sc, d_seqs, S, d_tokslot, stream));
      n_launches += 2;
      pnx_gemm(flx_op2, A, I, l.w_o, pnx_o, DT_F32, W, T, W, I);
      rt.y_main = pnx_o;
    } else {  // TGIS_MIXER_WKV
      const int H = s.heads, D = s.dim, Ad = H * D, R = s.decay_rank;
      const long long bs = (long long)pnx_rows_alloc * W;   // one mix buffer
      auto mix = [&](int j) { return reinterpret_cast<uint8_t*>(flx_mix) + (size_t)j * bs * dt_size(A); };
      CK(token_shift_mix_launch(pnx_resid, W, l.mu, 5, d_pos, d_tokslot, l.st_prev, flx_mix, A, bs, T, stream));
      for (int j = 0; j < 4; ++j)  // r | k | v | gate logits, each from its own mix
        pnx_gemm(mix(j), A, W, reinterpret_cast<uint8_t*>(l.w_in) + (size_t)j * Ad * W * dt_size(A), pnx_y1 + (size_t)j * Ad, DT_F32,
                 4 * Ad, T, Ad, W);
      pnx_gemm(mix(4), A, W, l.w_w1, pnx_cq, A, R, T, R, W, GEMM_ANY_TANH);
      pnx_gemm(pnx_cq, A, R, l.w_w2, flx_f2, DT_F32, Ad, T, Ad, R);
      OuterScan os{};
      os.mode = OUTER_SCAN_DECAY;
      os.q = pnx_y1; os.k = pnx_y1 + Ad; os.v = pnx_y1 + 2 * Ad; os.ldq = os.ldk = os.ldv = 4 * Ad;
      os.q_scale = 1.f;
      os.decay_raw = flx_f2; os.ldd = Ad; os.w0 = l.w0; os.u = l.u;
      os.S = l.st_S;
      os.out = flx_f1; os.ldo = Ad;
      os.heads = H; os.dim = D; os.vdim = D;
      os.x = pnx_resid; os.x_last = l.st_prev; os.width = W;
      CK(outer_scan_launch(os, d_seqs, S, d_tokslot, stream));
      CK(head_norm_gate_launch(flx_f1, Ad, H, D, l.mm_norm, pnx_y1 + 3 * Ad, 4 * Ad, /*silu*/ 1, eps, flx_op2, A, T, stream));
      n_launches += 3;
      pnx_gemm(flx_op2, A, Ad, l.w_o, pnx_o, DT_F32, W, T, W, Ad);
      rt.y_main = pnx_o;
    }
    CK(resid_tail_launch(rt, T, W, stream));
    ++n_launches;
    if (has_ff) {
      pnx_gemm(pnx_hA, A, W, l.w_gu, pnx_actS, A, s.ff, T, 2 * s.ff, W, GEMM_ANY_GEGLU);
      pnx_gemm(pnx_actS, A, s.ff, l.w_d, pnx_o, DT_F32, W, T, W, s.ff);
      ResidTail r2{};
      r2.resid = pnx_resid; r2.out = pnx_hA; r2.out_dtype = A; r2.mult = 1.f; r2.w_off = 0.f; r2.eps = eps;
      r2.y_main = pnx_o; r2.w_post = l.norm2; r2.w_pre = last ? pnx_final_norm : nullptr; r2.cast_out = 1;
      CK(resid_tail_launch(r2, T, W, stream));
      ++n_launches;
    }
    pnx_dump_resid(T);
  }

  // One layer of the parallel gated style (TGIS_STYLE_PARALLEL_GATED).  On entry rvp_n[li & 1] holds the layer's normed rows
  // n = rmsnorm(x) * norm1 in fp32 and pnx_hA the same in the operand type; the mixer reads n blended with the previous
  // token's n (token shift), the feed-forward, both gates and the router read n itself:
  //   x += sigmoid(R1 n + b1) * mixer(shift(n)) + sigmoid(R2 n + b2) * ff(n)
  // and the tail leaves the NEXT layer's normed rows (after the last layer: the final norm times the logit scale) behind.
  void gated_layer(int li, int T, int S) {
    PnxLayer& l = pnx_layers[li];
    const tgis_layer_spec& s = l.sp;
    const int W = cfg.hidden, A = pnx_dt;
    const float eps = pnx_spec.norm_eps;
    const int32_t* d_pos = ds<int32_t>(off_pos);
    const int32_t* d_slot = ds<int32_t>(off_slotmap);
    const int32_t* d_tokslot = ds<int32_t>(off_tokslot);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const bool last = li + 1 == (int)pnx_layers.size();
    const bool moe = s.mlp == TGIS_MLP_MOE_SIGMOID;
    float* n32 = rvp_n[li & 1];
    const int gc = l.gates_cols;
    // ---- what the mixer reads, and everything else that reads n: gate logits of both sublayers and the router logits
    CK(token_shift_mix_launch(n32, W, l.shift, 1, d_pos, d_tokslot, l.st_prev, flx_mix, A, 0, T, stream));
    ++n_launches;
    pnx_gemm(pnx_hA, A, W, l.w_gates, pnx_rl, DT_F32, gc, T, gc, W);
    const int ld = l.in_cols;
    pnx_gemm(flx_mix, A, W, l.w_in, pnx_y1, DT_F32, ld, T, ld, W);
    if (s.mixer == TGIS_MIXER_SIGMOID_ATTENTION) {
      const int H = s.heads;
      CK(sigattn_prep_launch(pnx_y1, ld, l.c_q, l.kv_src >= 0 ? -1 : l.c_k, l.c_v, l.sa, l.cos_sin, d_pos, d_slot, pnx_q, l.k_cache,
                             l.v_cache, A, T, stream));
      CK(sigattn_launch(pnx_q, l.k_cache, l.v_cache, A, d_seqs, ds<LatentTile>(off_ltiles), step_n_ltiles, ds<int32_t>(off_bt),
                        bt_stride, l.head_bias, pnx_oA, A, l.sa, stream));
      n_launches += 2;
      pnx_gemm(pnx_oA, A, H * s.vdim, l.w_o, pnx_o, DT_F32, W, T, W, H * s.vdim);
    } else if (s.mixer == TGIS_MIXER_SSD) {
      const int inner = s.heads * s.vdim, GN = s.groups * s.state, C = l.conv_ch;
      CK(short_conv_silu_launch(pnx_y1 + inner, ld, C, l.conv_w, l.conv_b, s.conv, d_pos, d_tokslot, l.st_conv, flx_f1, nullptr, A, T, stream));
      CK(conv_state_save_launch(pnx_y1 + inner, ld, C, s.conv, d_seqs, S, d_tokslot, l.st_conv, stream));
      OuterScan os{};
      os.mode = OUTER_SCAN_SSD;
      os.v = flx_f1; os.k = flx_f1 + inner; os.q = flx_f1 + inner + GN; os.ldq = os.ldk = os.ldv = C;
      os.q_scale = 1.f;
      os.step_raw = pnx_y1 + 2 * inner + 2 * GN; os.lds = ld; os.step_b = l.dt_b; os.A_log = l.A_log; os.D = l.Dv;
      os.S = l.st_S;
      os.out = flx_f2; os.ldo = inner;
      os.heads = s.heads; os.qk_heads = s.groups; os.dim = s.state; os.vdim = s.vdim;
      CK(outer_scan_launch(os, d_seqs, S, d_tokslot, stream));
      CK(head_norm_gate_launch(flx_f2, inner, s.norm_groups, inner / s.norm_groups, l.mm_norm, pnx_y1, ld, /*silu*/ 1, eps, flx_op2, A,
                               T, stream, /*gate_first=*/1));
      n_launches += s.conv > 1 ? 4 : 3;
      pnx_gemm(flx_op2, A, inner, l.w_o, pnx_o, DT_F32, W, T, W, inner);
    } else {  // TGIS_MIXER_CHANNEL_DELTA
      const int H = s.heads, qk = s.kv_heads * s.dim, hv = H * s.vdim, hd = H * s.dim, C = l.conv_ch, ld3 = hd + hv;
      CK(short_conv_silu_launch(pnx_y1, ld, C, l.conv_w, nullptr, s.conv, d_pos, d_tokslot, l.st_conv, flx_f1, nullptr, A, T, stream));
      CK(conv_state_save_launch(pnx_y1, ld, C, s.conv, d_seqs, S, d_tokslot, l.st_conv, stream));
      // the two low-rank maps: decay logits [heads x dim] and output-gate logits [heads x vdim], side by side in one buffer
      pnx_gemm(pnx_y1 + l.c_a1, DT_F32, ld, l.w_w2, flx_f3, DT_F32, ld3, T, hd, s.decay_rank);
      pnx_gemm(pnx_y1 + l.c_g1, DT_F32, ld, l.w_g2, flx_f3 + hd, DT_F32, ld3, T, hv, s.gate_rank);
      DeltaScan dsn{};
      dsn.q = flx_f1 + l.c_q; dsn.k = flx_f1 + l.c_k; dsn.v = flx_f1 + l.c_v; dsn.ldq = dsn.ldk = dsn.ldv = C;
      dsn.decay_raw = flx_f3; dsn.ldd = ld3; dsn.decay_b = l.dt_b; dsn.A_log = l.A_log;
      dsn.beta_raw = pnx_y1 + l.c_b; dsn.ldb = ld;
      dsn.S = l.st_S;
      dsn.out = flx_f2; dsn.ldo = hv;
      dsn.heads = H; dsn.qk_heads = s.kv_heads; dsn.dim = s.dim; dsn.vdim = s.vdim;
      (void)qk;
      CK(delta_scan_launch(dsn, d_seqs, S, d_tokslot, stream));
      CK(head_norm_gate_launch(flx_f2, hv, H, s.vdim, l.mm_norm, flx_f3 + hd, ld3, /*sigmoid*/ 0, eps, flx_op2, A, T, stream));
      n_launches += s.conv > 1 ? 4 : 3;
      pnx_gemm(flx_op2, A, hv, l.w_o, pnx_o, DT_F32, W, T, W, hv);
    }
    GatedTail gt{};
    gt.y_mix = pnx_o;
    gt.gl = pnx_rl; gt.ldg = gc; gt.b1 = l.gate_b; gt.b2 = l.gate_b + W;
    if (moe) {
      const int E = s.experts, top = s.top, ff = s.expert_ff, ffs = s.shared_ff;
      CK(moe_route_launch(pnx_rl + 2 * W, gc, nullptr, E, top, pnx_ids, pnx_mixw, nullptr, T, stream, MOE_W_SIGMOID));
      CK(moe_align_launch(pnx_ids, T, top, E, pnx_segoff, pnx_order, pnx_inv, stream));
      n_launches += 2;
      if (ffs > 0) {
        pnx_gemm(pnx_hA, A, W, l.w_gu_s, pnx_actS, A, ffs, T, ffs, W, GEMM_ANY_RELU2);
        pnx_gemm(pnx_actS, A, ffs, l.w_d_s, pnx_yS, DT_F32, W, T, W, ffs);
        gt.y_side = pnx_yS;
      }
      {  // routed experts: one row segment per expert; the router's weight scales a row's INPUT, i.e. the sum before the activation
        GemmAny a{};
        a.X = pnx_hA; a.W = l.w_gu_e; a.Y = pnx_actE;
        a.x_dtype = A; a.w_dtype = A; a.y_dtype = A;
        a.T = T * top; a.N = ff; a.K = W; a.ldx = W; a.ldw = W; a.ldy = ff;
        a.batch = 1; a.seg_off = pnx_segoff; a.n_groups = E; a.w_gs = (long long)ff * W;
        a.gather = pnx_order; a.gather_div = top; a.mode = GEMM_ANY_RELU2; a.row_scale = pnx_mixw;
        CK(gemm_any_launch(a, stream));
        GemmAny b{};
        b.X = pnx_actE; b.W = l.w_d_e; b.Y = pnx_yE;
        b.x_dtype = A; b.w_dtype = A; b.y_dtype = DT_F32;
        b.T = T * top; b.N = W; b.K = ff; b.ldx = ff; b.ldw = ff; b.ldy = W;
        b.batch = 1; b.seg_off = pnx_segoff; b.n_groups = E; b.w_gs = (long long)W * ff;
        CK(gemm_any_launch(b, stream));
        n_launches += 2;
      }
      gt.y_rows = pnx_yE; gt.inv = pnx_inv; gt.top = top;
    }
    gt.resid = pnx_resid;
    gt.w_next = last ? pnx_final_norm : pnx_layers[li + 1].norm1;
    gt.eps = eps;
    gt.out_scale = last && pnx_spec.logit_scale != 0.f ? pnx_spec.logit_scale : 1.f;
    gt.n_f32 = last ? nullptr : rvp_n[(li + 1) & 1];
    gt.out = pnx_hA; gt.out_dtype = A;
    gt.n_cur = n32; gt.prev_state = l.st_prev; gt.tok_slot = d_tokslot;
    CK(gated_tail_launch(gt, T, W, stream));
    ++n_launches;
    pnx_dump_resid(T);
  }

  // One layer run of the parallel pair style (TGIS_STYLE_PARALLEL_PAIR).  On entry pnx_hA holds rms(x) * g1 and pnx_hB rms(x) * g2
  // (operand type; hB only when the layer has a feed-forward):
  //   x += mixer(hA) + ff(hB);   x += rms(P (gelu_tanh(G x) * e)) * w   (the per-layer token input; e: the layer's slice of the
  //   token's row of the side table);   x += x0 if the NEXT run opens a pass of a loop
  // and the tail leaves the next run's two normed inputs (after the last run: the final norm) behind.
  void pair_layer(int ri, int T, int S) {
    PnxLayer& l = pair_runs[ri];
    const tgis_layer_spec& s = l.sp;
    const int W = cfg.hidden, A = pnx_dt;
    const float eps = pnx_spec.norm_eps;
    const int32_t* d_tok = ds<int32_t>(off_tok);
    const int32_t* d_pos = ds<int32_t>(off_pos);
    const int32_t* d_slot = ds<int32_t>(off_slotmap);
    const int32_t* d_tokslot = ds<int32_t>(off_tokslot);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const int32_t* d_bt = ds<int32_t>(off_bt);
    const bool last = ri + 1 == (int)pair_runs.size();
    const PnxLayer* nx = last ? nullptr : &pair_runs[ri + 1];
    // ---- feed-forward on the second norm's rows -> pnx_yS, beside the mixer
    const bool has_ff = s.mlp == TGIS_MLP_DENSE_SILU;
    auto feed_forward = [&]() {
      pnx_gemm(pnx_hB, A, W, l.w_gu, pnx_actS, A, s.ff, T, 2 * s.ff, W, GEMM_ANY_SWIGLU);
      pnx_gemm(pnx_actS, A, s.ff, l.w_d, pnx_yS, DT_F32, W, T, W, s.ff);
    };
    const bool forked = has_ff && stream2 != nullptr;
    if (forked) {
      CK(cudaEventRecord(ev_fork, stream));
      CK(cudaStreamWaitEvent(stream2, ev_fork, 0));
      on_side_stream = true;
      feed_forward();
      on_side_stream = false;
      CK(cudaEventRecord(ev_join, stream2));
    }
    // ---- mixer -> pnx_o [T, width] fp32
    if (s.mixer == TGIS_MIXER_POOLED_ATTENTION) {
      const int H = s.heads, ld = l.in_cols;
      pnx_gemm(pnx_hA, A, W, l.w_in, pnx_y1, DT_F32, ld, T, ld, W);
      CK(poolattn_prep_launch(pnx_y1, ld, l.c_q, l.c_k, l.c_v, l.in_bias, l.pa, l.cos_sin, eps, d_pos, d_slot, pnx_q, l.k_cache,
                              l.v_cache, A, T, stream));
      CK(poolattn_pool_launch(l.k_cache, l.v_cache, l.pk_cache, l.pv_cache, A, d_seqs, S, d_bt, bt_stride, l.pa, step_max_q, stream));
      CK(poolattn_launch(pnx_q, l.k_cache, l.v_cache, l.pk_cache, l.pv_cache, A, d_seqs, ds<LatentTile>(off_ltiles16), step_n_ltiles16,
                         d_bt, bt_stride, pnx_oA, A, l.pa, stream));
      n_launches += l.pa.pool > 0 ? 3 : 2;
      pnx_gemm(pnx_oA, A, H * s.vdim, l.w_o, pnx_o, DT_F32, W, T, W, H * s.vdim);
    } else if (s.mixer == TGIS_MIXER_HGRN) {
      const int H = s.heads, hd = H * s.dim, hv = H * s.vdim, ld = l.in_cols;
      pnx_gemm(pnx_hA, A, W, l.w_in, pnx_y1, DT_F32, ld, T, ld, W);
      OuterScan os{};
      os.mode = OUTER_SCAN_HGRN;
      os.q = pnx_y1 + l.c_q; os.k = nullptr; os.v = pnx_y1 + l.c_v; os.ldq = os.ldk = os.ldv = ld;
      os.q_scale = 1.f;
      os.decay_raw = pnx_y1 + l.c_f; os.ldd = ld; os.w0 = l.w0; os.u = l.u;
      os.S = l.st_S;
      os.out = flx_f1; os.ldo = hv;
      os.heads = H; os.dim = s.dim; os.vdim = s.vdim;
      (void)hd;
      CK(outer_scan_launch(os, d_seqs, S, d_tokslot, stream));
      CK(head_norm_gate_launch(flx_f1, hv, H, s.vdim, l.mm_norm, nullptr, 0, /*no gate*/ 2, eps, flx_op2, A, T, stream));
      n_launches += 2;
      pnx_gemm(flx_op2, A, hv, l.w_o, pnx_o, DT_F32, W, T, W, hv);
    } else {  // TGIS_MIXER_LATENT_ATTENTION
      const LatentGeom& g = l.g;
      const int H = s.heads, hd = s.dim + s.rot_dim, D = g.row();
      pnx_gemm(pnx_hA, A, W, l.w_down, pnx_y1, DT_F32, l.n_down(), T, l.n_down(), W);
      CK(latent_prep_launch(pnx_y1, l.n_down(), g, l.qnorm, l.kvnorm, eps, d_pos, d_slot, l.cos_sin, pnx_cq, l.cache, A,
                            l.out_gate ? pnx_gate : nullptr, T, stream));
      pnx_gemm(pnx_cq, A, s.q_rank, l.w_uq, pnx_q, A, H * hd, T, H * hd, s.q_rank);
      CK(latent_q_rope_launch(pnx_q, A, g, d_pos, l.cos_sin, pnx_qabs, T, stream));
      {  // q_abs_h = W_uk,h^T q_plain_h  (one problem per head)
        GemmAny a{};
        a.X = pnx_q; a.W = l.w_ukT; a.Y = pnx_qabs;
        a.x_dtype = A; a.w_dtype = A; a.y_dtype = DT_F32;
        a.T = T; a.N = s.kv_rank; a.K = s.dim; a.ldx = H * hd; a.ldw = s.dim; a.ldy = H * D;
        a.batch = H; a.x_bs = hd; a.w_bs = (long long)s.kv_rank * s.dim; a.y_bs = D;
        CK(gemm_any_launch(a, stream));
      }
      int attn_launches = 0;
      CK(latent_attn_launch(pnx_qabs, l.cache, A, d_seqs, ds<LatentTile>(off_ltiles), step_n_ltiles, d_bt, bt_stride, pnx_olat, A, g,
                            stream, pnx_attn_ws, pnx_attn_ws_floats, step_max_kv, num_sms, &attn_launches));
      n_launches += attn_launches - 1;
      {  // o_h = W_uv,h o_lat_h  (times the head's gate where the layer has one)
        GemmAny a{};
        a.X = pnx_olat; a.W = l.w_uv; a.Y = pnx_oA;
        a.x_dtype = A; a.w_dtype = A; a.y_dtype = A;
        a.T = T; a.N = s.vdim; a.K = s.kv_rank; a.ldx = H * s.kv_rank; a.ldw = s.kv_rank; a.ldy = H * s.vdim;
        a.batch = H; a.x_bs = s.kv_rank; a.w_bs = (long long)s.vdim * s.kv_rank; a.y_bs = s.vdim;
        if (l.out_gate) { a.mode = GEMM_ANY_ROWSCALE; a.row_scale = pnx_gate; a.scale_ld = H; }
        CK(gemm_any_launch(a, stream));
      }
      n_launches += 5;
      pnx_gemm(pnx_oA, A, H * s.vdim, l.w_o, pnx_o, DT_F32, W, T, W, H * s.vdim);
    }
    if (forked) CK(cudaStreamWaitEvent(stream, ev_join, 0));
    else if (has_ff) feed_forward();
    const float* w_a = last ? pnx_final_norm : nx->norm1;
    const float* w_b = (!last && nx->sp.mlp == TGIS_MLP_DENSE_SILU) ? nx->norm2 : nullptr;
    const float* extra = (!last && nx->add_x0) ? pnx_x0 : nullptr;
    const int sd = pnx_spec.side_dim;
    GatedTail gt{};
    gt.y_mix = pnx_o; gt.y_side = has_ff ? pnx_yS : nullptr;
    gt.resid = pnx_resid; gt.eps = eps; gt.out_scale = 1.f; gt.out_dtype = A;
    if (sd > 0) {
      gt.resid_out = flx_mix;   // the token input's gate reads the stream itself
    } else {
      gt.extra = extra;
      gt.w_next = w_a; gt.out = pnx_hA; gt.w_next2 = w_b; gt.out2 = pnx_hB;
    }
    CK(gated_tail_launch(gt, T, W, stream));
    ++n_launches;
    if (sd > 0) {
      pnx_gemm(flx_mix, A, W, l.w_sg, pnx_rl, DT_F32, sd, T, sd, W);
      CK(gelu_gate_rows_launch(pnx_rl, sd, d_tok, pnx_side, A, (int)pnx_layers.size() * sd, l.weights_of * sd, sd, pnx_cq, A, T, stream));
      pnx_gemm(pnx_cq, A, sd, l.w_sp, pnx_yE, DT_F32, W, T, W, sd);
      ResidTail rt{};
      rt.y_main = pnx_yE; rt.w_post = l.side_norm; rt.w_off = 0.f; rt.mult = 1.f; rt.eps = eps;
      rt.resid = pnx_resid; rt.extra = extra;
      rt.w_pre = w_a; rt.out = pnx_hA; rt.out_dtype = A; rt.w_pre2 = w_b; rt.out2 = pnx_hB;
      CK(resid_tail_launch(rt, T, W, stream));
      n_launches += 2;
    }
    pnx_dump_resid(T);
  }

  // embeddings + layer stack + final norm -> pnx_hA [T, hidden] (operand type), fp32 residual stream in pnx_resid
  void pnx_forward(int T, int S) {
    const int W = cfg.hidden, A = pnx_dt;
    const float eps = pnx_spec.norm_eps, mult = pnx_spec.residual_mult;
    const int32_t* d_tok = ds<int32_t>(off_tok);
    const int32_t* d_pos = ds<int32_t>(off_pos);
    const int32_t* d_slot = ds<int32_t>(off_slotmap);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const int32_t* d_bt = ds<int32_t>(off_bt);
    const LatentTile* d_tiles = ds<LatentTile>(off_ltiles);
    CK(embed_scale_f32_launch(d_tok, pnx_embed, A, pnx_spec.embed_scale, pnx_resid, T, W, cfg.vocab, stream));
    if (pair_style) {
      const PnxLayer& f = pair_runs[0];
      if (pnx_x0 != nullptr) CK(cudaMemcpyAsync(pnx_x0, pnx_resid, (size_t)T * W * sizeof(float), cudaMemcpyDeviceToDevice, stream));
      CK(rmsnorm_f32_launch(pnx_resid, W, f.norm1, 0.f, pnx_hA, A, W, T, W, eps, stream));
      if (f.sp.mlp == TGIS_MLP_DENSE_SILU) CK(rmsnorm_f32_launch(pnx_resid, W, f.norm2, 0.f, pnx_hB, A, W, T, W, eps, stream));
      n_launches += 3;
      for (int ri = 0; ri < (int)pair_runs.size(); ++ri) pair_layer(ri, T, S);
      return;
    }
    if (gated_style) {
      CK(rmsnorm_f32_launch(pnx_resid, W, pnx_layers[0].norm1, 0.f, rvp_n[0], DT_F32, W, T, W, eps, stream));
      CK(convert_f32_launch(rvp_n[0], pnx_hA, A, (size_t)T * W, stream));
      n_launches += 3;
      for (int li = 0; li < (int)pnx_layers.size(); ++li) gated_layer(li, T, S);
      return;
    }
    if (post_norm) CK(convert_f32_launch(pnx_resid, pnx_hA, A, (size_t)T * W, stream));
    else CK(rmsnorm_f32_launch(pnx_resid, W, pnx_layers[0].norm1, 1.f, pnx_hA, A, W, T, W, eps, stream));
    n_launches += 2;
    const int L = (int)pnx_layers.size();
    for (int li = 0; li < L; ++li) {
      if (post_norm) {
        stream_layer(li, T, S);
        continue;
      }
      PnxLayer& l = pnx_layers[li];
      const tgis_layer_spec& s = l.sp;
      const LatentGeom& g = l.g;
      const int H = s.heads, hd = s.dim + s.rot_dim, D = g.row();
      const float* next_pre = li + 1 < L ? pnx_layers[li + 1].norm1 : pnx_final_norm;
      // ---- mixer: fused down-projections [q latent | kv latent | rotary key | gate logits]
      pnx_gemm(pnx_hA, A, W, l.w_down, pnx_y1, DT_F32, l.n_down(), T, l.n_down(), W);
      CK(latent_prep_launch(pnx_y1, l.n_down(), g, l.qnorm, l.kvnorm, eps, d_pos, d_slot, l.cos_sin, pnx_cq, l.cache, A,
                            pnx_gate, T, stream));
      pnx_gemm(pnx_cq, A, s.q_rank, l.w_uq, pnx_q, A, H * hd, T, H * hd, s.q_rank);
      CK(latent_q_rope_launch(pnx_q, A, g, d_pos, l.cos_sin, pnx_qabs, T, stream));
      {  // q_abs_h = W_uk,h^T q_nope_h  (one problem per head)
        GemmAny a{};
        a.X = pnx_q; a.W = l.w_ukT; a.Y = pnx_qabs;
        a.x_dtype = A; a.w_dtype = A; a.y_dtype = DT_F32;
        a.T = T; a.N = s.kv_rank; a.K = s.dim; a.ldx = H * hd; a.ldw = s.dim; a.ldy = H * D;
        a.batch = H; a.x_bs = hd; a.w_bs = (long long)s.kv_rank * s.dim; a.y_bs = D;
        CK(gemm_any_launch(a, stream));
      }
      int attn_launches = 0;
      CK(latent_attn_launch(pnx_qabs, l.cache, A, d_seqs, d_tiles, step_n_ltiles, d_bt, bt_stride, pnx_olat, A, g, stream,
                            pnx_attn_ws, pnx_attn_ws_floats, step_max_kv, num_sms, &attn_launches));
      n_launches += attn_launches - 1;  // (one attention launch is part of the count below)
      {  // o_h = gate_h * W_uv,h o_lat_h
        GemmAny a{};
        a.X = pnx_olat; a.W = l.w_uv; a.Y = pnx_oA;
        a.x_dtype = A; a.w_dtype = A; a.y_dtype = A;
        a.T = T; a.N = s.vdim; a.K = s.kv_rank; a.ldx = H * s.kv_rank; a.ldw = s.kv_rank; a.ldy = H * s.vdim;
        a.batch = H; a.x_bs = s.kv_rank; a.w_bs = (long long)s.vdim * s.kv_rank; a.y_bs = s.vdim;
        a.mode = GEMM_ANY_ROWSCALE; a.row_scale = pnx_gate; a.scale_ld = H;
        CK(gemm_any_launch(a, stream));
      }
      n_launches += 5;
      pnx_gemm(pnx_oA, A, H * s.vdim, l.w_o, pnx_o, DT_F32, W, T, W, H * s.vdim);
      const bool moe = s.mlp == TGIS_MLP_MOE;
      {
        ResidTail rt{};
        rt.y_main = pnx_o; rt.w_post = l.norm1b; rt.w_pre = moe ? l.norm2 : next_pre;
        rt.resid = pnx_resid; rt.out = pnx_hA; rt.out_dtype = A; rt.mult = mult; rt.w_off = 1.f; rt.eps = eps;
        CK(resid_tail_launch(rt, T, W, stream));
        ++n_launches;
      }
      if (moe) {
        const int E = s.experts, top = s.top, ff = s.expert_ff, ffs = s.shared_ff;
        const int n_rl = E + (ffs > 0 ? 1 : 0);
        pnx_gemm(pnx_hA, A, W, l.w_router, pnx_rl, DT_F32, n_rl, T, n_rl, W);
        CK(moe_route_launch(pnx_rl, n_rl, l.router_b, E, top, pnx_ids, pnx_mixw, ffs > 0 ? pnx_sgate : nullptr, T, stream));
        CK(moe_align_launch(pnx_ids, T, top, E, pnx_segoff, pnx_order, pnx_inv, stream));
        n_launches += 2;
        if (ffs > 0) {
          pnx_gemm(pnx_hA, A, W, l.w_gu_s, pnx_actS, A, ffs, T, 2 * ffs, W, GEMM_ANY_SWIGLU);
          pnx_gemm(pnx_actS, A, ffs, l.w_d_s, pnx_yS, DT_F32, W, T, W, ffs);
        }
        {  // routed experts: one row segment per expert
          GemmAny a{};
          a.X = pnx_hA; a.W = l.w_gu_e; a.Y = pnx_actE;
          a.x_dtype = A; a.w_dtype = A; a.y_dtype = A;
          a.T = T * top; a.N = 2 * ff; a.K = W; a.ldx = W; a.ldw = W; a.ldy = ff;
          a.batch = 1; a.seg_off = pnx_segoff; a.n_groups = E; a.w_gs = (long long)2 * ff * W;
          a.gather = pnx_order; a.gather_div = top; a.mode = GEMM_ANY_SWIGLU;
          CK(gemm_any_launch(a, stream));
          GemmAny b{};
          b.X = pnx_actE; b.W = l.w_d_e; b.Y = pnx_yE;
          b.x_dtype = A; b.w_dtype = A; b.y_dtype = DT_F32;
          b.T = T * top; b.N = W; b.K = ff; b.ldx = ff; b.ldw = ff; b.ldy = W;
          b.batch = 1; b.seg_off = pnx_segoff; b.n_groups = E; b.w_gs = (long long)W * ff;
          CK(gemm_any_launch(b, stream));
          n_launches += 2;
        }
        ResidTail rt{};
        rt.y_rows = pnx_yE; rt.inv = pnx_inv; rt.mix_w = pnx_mixw; rt.top = top;
        rt.y_side = ffs > 0 ? pnx_yS : nullptr; rt.side_gate = ffs > 0 ? pnx_sgate : nullptr;
        rt.w_post = l.norm2b; rt.w_pre = next_pre;
        rt.resid = pnx_resid; rt.out = pnx_hA; rt.out_dtype = A; rt.mult = mult; rt.w_off = 1.f; rt.eps = eps;
        CK(resid_tail_launch(rt, T, W, stream));
        ++n_launches;
      }
      pnx_dump_resid(T);
    }
  }

  // ------------------------------------------------------------------------------------------------ device step
  // next_wm / nT,nN,nK describe the GEMM that follows this one in the layer stack: its first weight boxes are
  // prefetched into L2 by this launch's producer warp (gemm_tcgen05.cu)
  void gemm(const CUtensorMap* xmaps, const CUtensorMap& wm, const bf16* X, const bf16* W, void* Y, int T, int N, int K,
            int out_f32 = 0, const CUtensorMap* next_wm = nullptr, int nT = 0, int nN = 0, int nK = 0, int ldy = 0,
            const GemmRope* rope = nullptr, const GemmNorm* norm = nullptr) {
    if (ldy == 0) ldy = N;
    cudaEvent_t pe0 = nullptr, pe1 = nullptr;
    if (profiling && (!prof_decode_only || step_is_decode)) {
      while (prof_events.size() < prof_used + 2) {
        cudaEvent_t ev;
        CK(cudaEventCreate(&ev));
        prof_events.push_back(ev);
      }
      pe0 = prof_events[prof_used];
      pe1 = prof_events[prof_used + 1];
      prof_used += 2;
      // algorithmic bytes: weights once + activations in + result out
      prof_bytes.push_back((double)N * K * 2 + (double)T * K * 2 + (double)T * N * (out_f32 == 1 ? 4 : out_f32 == 2 ? 1 : 2));
      CK(cudaEventRecord(pe0, stream));
    }
    if (cfg.debug_gemm_ref) {
      CK(gemm_bf16_ref_launch(X, K, W, Y, ldy, T, N, K, stream, out_f32));
    } else {
      GemmNext nx{};
      if (next_wm && l2_prefetch_kb > 0) nx = gemm_next_desc(nT, nN, nK, num_sms, l2_prefetch_kb);
      CK(gemm_bf16_launch(wm, xmaps[bt_index(T)], Y, ldy, T, N, K, gemm_ws.p, gemm_counters.p, num_sms, stream, out_f32,
                          nx.kb_prefetch > 0 ? next_wm : nullptr, nx.kb_prefetch > 0 ? &nx : nullptr, rope, norm));
    }
    if (pe1) CK(cudaEventRecord(pe1, stream));
    ++n_launches;
  }

  template <class T>
  T* hs(size_t off) { return reinterpret_cast<T*>(h_stage + off); }
  template <class T>
  T* ds(size_t off) { return reinterpret_cast<T*>(d_stage.p + off); }

  void all_reduce_tmp(int T) {
    if (tp > 1) {
      cudaEvent_t pe = prof_begin_exchange();
      NK(nccl().AllReduce(tmp.p, tmp.p, (size_t)T * cfg.hidden, ncclBfloat16, ncclSum, comm, stream));
      if (pe) CK(cudaEventRecord(pe, stream));
    }
  }

  // Enqueue one step on `stream`: H2D metadata, layer stack, lm_head + sampler, D2H results.  Reads every per-step
  // quantity from the device staging buffer, so the same sequence can be captured once into a CUDA graph and replayed.
  size_t items_off(int S) const { return (off_bt + sizeof(int32_t) * (size_t)S * bt_stride + 255) / 256 * 256; }

  void launch_step(size_t copy_bytes, int T, int n_dec, int n_tiles, int R, int max_dec_kv, int S, int samp_complex) {
    const tgis_config& c = cfg;
    const int H = c.hidden, F = Fl, V = c.vocab;  // F: local ffn shard
    const bool copies_here = !(capturing && graph_copy_outside);
    CK(stl_marker_launch(20, stream));  // timeline builds: step begin (before the metadata copy)
    if (copies_here) CK(cudaMemcpyAsync(d_stage.p, h_stage, copy_bytes, cudaMemcpyHostToDevice, stream));
    CK(stl_marker_launch(21, stream));  // metadata landed
    step_is_decode = (n_tiles == 0);
    step_ar_idx[0] = step_ar_idx[1] = 0;

    const int32_t* d_tok = ds<int32_t>(off_tok);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const int32_t* d_bt = ds<int32_t>(off_bt);
    const float scale = attn_scale;

    if (rank == 0) {
      CK(bitmap_set_launch(seen_bitmap.p, bitmap_words, ds<int32_t>(off_tokslot), d_tok, T, stream));
      ++n_launches;
    }
    if (opt) {
      opt_layers(T, n_dec, n_tiles, max_dec_kv, S, R);  // embeddings + layer stack + final LayerNorm -> xn
    } else if (pnx_on) {
      pnx_forward(T, S);  // embeddings + layer stack + final norm -> pnx_hA
    } else {
      CK(embed_gather_launch(d_tok, embed, resid.p, T, H, V, stream));
      ++n_launches;
    }
    const bool ar_fused = exchange_mode(T) != 0;
    // RoPE + KV-cache scatter fused into the qkv GEMM's split-tile reduction (decode-shaped steps where every weight
    // tile is split over several CTAs; TGIS_FUSE_ROPE=0: off)
    // (measured: -2 % per step at 32 tokens, but +2...5 % at 64...256 -- the last-arriving CTA's serial tail grows with
    // T while the stand-alone kernel spreads over all SMs -- hence the token limit)
    // ... unless the qkv launch reduces its split tiles on chip (cluster mode): then the epilogue is spread over the
    // cluster's CTAs by token and the fusion pays up to 256 tokens (TGIS_FUSE_ROPE_CLUSTER_MAX_T)
    const int qkv_cluster = (cfg.debug_gemm_ref || pnx_on) ? 0 : gemm_cluster_split(T, qkv_dim, H, num_sms);
    // LoRA steps: the adapter deltas are added to the RAW projections (before RoPE, before SwiGLU, before the residual
    // add), so the fused epilogues are switched off for the step and the deltas land between the GEMM and its consumer
    const bool lora = (samp_complex & 4) != 0 && max_loras > 0;
    const int32_t* d_toklora = ds<int32_t>(off_toklora);
    const int LR = lora_R, kvd = nkv * HEAD_DIM;
    auto lora_apply = [&](const LoraGroup& g, const bf16* x, int ldx, bf16* y, int ldy) {
      CK(lora_shrink_launch(x, ldx, d_toklora, g, lora_v.p, T, stream));
      CK(lora_expand_launch(lora_v.p, d_toklora, g, y, ldy, T, stream));
      n_launches += 2;
    };
    if (lora) ++lora_steps;
    const bool rope_fused = !pnx_on && !lora && fuse_rope && !cfg.debug_gemm_ref && gemm_even_split(T, qkv_dim, H, num_sms) >= 2 &&
                            T <= (qkv_cluster > 0 ? std::max(rope_fuse_max_t, rope_fuse_cluster_max_t) : rope_fuse_max_t);
    // residual add + RMSNorm inside the GEMMs either side of it (single GPU, small steps, both row-"producers" reduced
    // on chip): o-proj -> [post-attention norm] -> gate_up and down-proj -> [next layer's input norm] -> qkv
    const bool norm_fused = !pnx_on && !lora && fuse_norm && tp == 1 && !cfg.debug_gemm_ref && T <= GEMM_NORM_MAX_T && H % 128 == 0 && H / 128 <= GEMM_NORM_MAX_PARTS &&
                            gemm_cluster_split(T, H, q_dim, num_sms) > 0 && gemm_cluster_split(T, H, F, num_sms) > 0;
    const int n_parts = H / 128;
    float* ssq_attn = norm_ssq.p;                                      // written by o-proj, read by gate_up
    float* ssq_mlp = norm_ssq.p + (size_t)GEMM_NORM_MAX_T * n_parts;   // written by down-proj, read by the next qkv
    const GemmNorm prod_attn{resid.p, ssq_attn, nullptr, nullptr, nullptr, 0, 0.f};
    const GemmNorm prod_mlp{resid.p, ssq_mlp, nullptr, nullptr, nullptr, 0, 0.f};
    for (int li = 0; li < ((opt || pnx_on) ? 0 : c.n_layers); ++li) {  // Llama stack (OPT: opt_layers() above)
      LayerW& l = layers[li];
      const GemmNorm cons_qkv{nullptr, nullptr, resid.p, ssq_mlp, l.ln1, n_parts, c.rms_eps};
      const GemmNorm cons_gu{nullptr, nullptr, resid.p, ssq_attn, l.ln2, n_parts, c.rms_eps};
      const bool qkv_norm_in = norm_fused && li > 0;
      {
        if (li == 0) {
          CK(rmsnorm_launch(resid.p, l.ln1, xn.p, T, H, c.rms_eps, stream));
          ++n_launches;
        } else if (qkv_norm_in) {
          // the previous layer's down-proj left h in resid and sum(h^2) in ssq_mlp; the qkv GEMM normalises on the fly
        } else if (ar_fused) {
          fused_ar_norm(1, l.ln1, T);  // previous layer's down-proj partials
        } else {
          CK(add_rmsnorm_launch(tmp.p, resid.p, l.ln1, xn.p, T, H, c.rms_eps, stream));
          ++n_launches;
        }
        const GemmRope rp{ds<int32_t>(off_pos), ds<int32_t>(off_slotmap), cos_sin,
                          k_cache.p + (size_t)li * kv_layer_elems, v_cache.p + (size_t)li * kv_layer_elems, nq, nkv};
        gemm(qkv_norm_in ? xm_resid : xm_xn, l.m_qkv, xn.p, l.wqkv, qkv.p, T, qkv_dim, H, 0, &l.m_o, T, H, q_dim, 0,
             rope_fused ? &rp : nullptr, qkv_norm_in ? &cons_qkv : nullptr);
        if (lora) {
          const LoraLayerW& ll = lora_layers[li];
          LoraGroup g{};
          g.n_mods = 3;
          g.v_ld = 3 * LR;
          g.mod[0] = LoraModule{ll.A_q, ll.B_q, H, q_dim, LR, 0, 0};
          g.mod[1] = LoraModule{ll.A_k, ll.B_k, H, kvd, LR, q_dim, LR};
          g.mod[2] = LoraModule{ll.A_v, ll.B_v, H, kvd, LR, q_dim + kvd, 2 * LR};
          lora_apply(g, xn.p, H, qkv.p, qkv_dim);
        }
      }
      bf16* kc = k_cache.p + (size_t)li * kv_layer_elems;
      bf16* vc = v_cache.p + (size_t)li * kv_layer_elems;
      if (!rope_fused) {
        CK(rope_kvwrite_launch(qkv.p, ds<int32_t>(off_pos), ds<int32_t>(off_slotmap), cos_sin, kc, vc, T, nq, nkv,
                               stream));
        ++n_launches;
      }
      if (n_dec > 0) {
        const int max_splits = (max_dec_kv + DECODE_SPLIT - 1) / DECODE_SPLIT;
        CK(attn_decode_launch(qkv.p, qkv_dim, kc, vc, ds<DecItem>(items_off(S)), n_dec * max_splits, d_seqs,
                              ds<int32_t>(off_decids), n_dec, max_splits, part_o.p, part_ml.p, attn_out.p, q_dim, nq,
                              nkv, scale, num_sms, stream, attn_arrive.p));
        n_launches += (max_splits > 1 && !attn_inkernel_merge) ? 2 : 1;
      }
      if (n_tiles > 0) {
        CK(attn_prefill_launch(qkv.p, qkv_dim, kc, vc, d_seqs, ds<int32_t>(off_tileseq), ds<int32_t>(off_tileq0),
                               n_tiles, d_bt, bt_stride, attn_out.p, q_dim, nq, nkv, scale, stream));
        ++n_launches;
      }
      gemm(xm_attn, l.m_o, attn_out.p, l.wo, ar_fused ? ar_buf(0) : tmp.p, T, H, q_dim, 0, &l.m_gu, T, 2 * F, H, 0, nullptr,
           norm_fused ? &prod_attn : nullptr);
      if (lora) {
        LoraGroup g{};
        g.n_mods = 1;
        g.v_ld = 3 * LR;
        g.mod[0] = LoraModule{lora_layers[li].A_o, lora_layers[li].B_o, q_dim, H, LR, 0, 0};
        lora_apply(g, attn_out.p, q_dim, tmp.p, H);
      }
      if (norm_fused) {
      } else if (ar_fused) {
        fused_ar_norm(0, l.ln2, T);
      } else {
        all_reduce_tmp(T);  // row-parallel partial sums (tp > 1)
        CK(add_rmsnorm_launch(tmp.p, resid.p, l.ln2, xn.p, T, H, c.rms_eps, stream));
        ++n_launches;
      }
      // gate_up GEMM with SwiGLU fused into its epilogue: writes act[T, F] directly (no gate_up round trip)
      if (lora) {
        // raw interleaved gate_up -> + adapter deltas (gate and up as one module of capacity 2R) -> SwiGLU
        gemm(xm_xn, l.m_gu, xn.p, l.wgu, gu_buf.p, T, 2 * F, H, /*out_mode=*/0, &l.m_d, T, H, F, /*ldy=*/2 * F);
        LoraGroup g{};
        g.n_mods = 1;
        g.v_ld = 3 * LR;
        g.mod[0] = LoraModule{lora_layers[li].A_gu, lora_layers[li].B_gu, H, 2 * F, 2 * LR, 0, 0};
        lora_apply(g, xn.p, H, gu_buf.p, 2 * F);
        CK(silu_mul_interleaved_launch(gu_buf.p, act.p, T, F, stream));
        ++n_launches;
      } else
      gemm(norm_fused ? xm_resid : xm_xn, l.m_gu, xn.p, l.wgu, act.p, T, 2 * F, H, /*out_mode=*/2, &l.m_d, T, H, F,
           /*ldy=*/F, nullptr, norm_fused ? &cons_gu : nullptr);
      bf16* down_out = ar_fused ? ar_buf(1) : tmp.p;
      if (li + 1 < c.n_layers)
        gemm(xm_act, l.m_d, act.p, l.wd, down_out, T, H, F, 0, &layers[li + 1].m_qkv, T, qkv_dim, H, 0, nullptr,
             norm_fused ? &prod_mlp : nullptr);
      else gemm(xm_act, l.m_d, act.p, l.wd, down_out, T, H, F, 0, R > 0 ? &m_lm : nullptr, R, Vl, H);
      if (lora) {
        LoraGroup g{};
        g.n_mods = 1;
        g.v_ld = 3 * LR;
        g.mod[0] = LoraModule{lora_layers[li].A_d, lora_layers[li].B_d, F, H, LR, 0, 0};
        lora_apply(g, act.p, F, down_out, H);
      }
      if (!ar_fused) all_reduce_tmp(T);
    }
    // The last down-proj exchange is run even when no row is sampled this step (R == 0): it is what guarantees that
    // every rank has finished READING this step's buffers before a faster rank overwrites them in the next step.
    if (ar_fused) fused_ar_norm(1, final_norm, T);
    if (R > 0) {
      if (ar_fused || opt || pnx_on) {
      } else {
        CK(add_rmsnorm_launch(tmp.p, resid.p, final_norm, xn.p, T, H, c.rms_eps, stream));
        ++n_launches;
      }
      gather_final_rows(R);
      lm_head_logits(R, 1);
      if (rank == 0) {
        CK(sampler_launch(logits_ptr(), logits_bf16 ? 1 : 0, logits_ld, logits_ld, ds<SampleRow>(off_rows), R, seen_bitmap.p, bitmap_words,
                          samp_scratch.p, d_samp_out.p, stream, samp_complex & 1, num_sms,
                          (samp_complex & 2) ? allow_bitmap.p : nullptr));
        ++n_launches;
        if (copies_here)
          CK(cudaMemcpyAsync(h_samp_out, d_samp_out.p, sizeof(SampleOut) * R, cudaMemcpyDeviceToHost, stream));
      }
    }
    CK(stl_marker_launch(22, stream));  // timeline builds: step end (after the result copy)
  }

  // OPT layer stack (vllm model_executor/models/opt.py:170-197, do_layer_norm_before): the tcgen05 GEMMs write their fp32
  // accumulators (out mode 1) and the kernels of opt.cu add the bias before the single rounding to bf16; the paged
  // attention kernels run unchanged on zero-padded 128-dim heads with the model's softmax scale.  Per layer:
  //   LN1 [+ previous fc2 bias/residual] -> qkv GEMM -> bias + KV scatter -> attention -> out_proj GEMM ->
  //   LN2 + out_proj bias/residual -> fc1 GEMM -> bias + ReLU -> fc2 GEMM;  final LayerNorm after the last layer.
  void opt_layers(int T, int n_dec, int n_tiles, int max_dec_kv, int S, int R) {
    const tgis_config& c = cfg;
    const int H = c.hidden, F = Fl, V = c.vocab;
    const int32_t* d_tok = ds<int32_t>(off_tok);
    const int32_t* d_pos = ds<int32_t>(off_pos);
    const AttnSeq* d_seqs = ds<AttnSeq>(off_seqs);
    const int32_t* d_bt = ds<int32_t>(off_bt);
    CK(opt_embed_launch(d_tok, d_pos, embed, pos_embed, resid.p, T, H, V, pos_rows, /*offset=*/2, stream));
    ++n_launches;
    for (int li = 0; li < c.n_layers; ++li) {
      LayerW& l = layers[li];
      // h += fc2 of the previous layer (its fp32 accumulators are still in y32), then LN1
      CK(opt_layernorm_launch(li == 0 ? nullptr : y32.p, li == 0 ? nullptr : layers[li - 1].b_fc2, resid.p, l.ln1, l.ln1_b,
                              xn.p, T, H, c.rms_eps, stream));
      gemm(xm_xn, l.m_qkv, xn.p, l.wqkv, y32.p, T, qkv_dim, H, /*out_f32=*/1, &l.m_o, T, H, q_dim);
      bf16* kc = k_cache.p + (size_t)li * kv_layer_elems;
      bf16* vc = v_cache.p + (size_t)li * kv_layer_elems;
      // bias + rounding; q -> qkv buffer, k / v -> paged cache (no rotary embedding in between)
      CK(opt_qkv_bias_kvwrite_launch(y32.p, l.b_qkv, qkv.p, ds<int32_t>(off_slotmap), kc, vc, T, nq, nkv, stream));
      n_launches += 2;
      if (n_dec > 0) {
        const int max_splits = (max_dec_kv + DECODE_SPLIT - 1) / DECODE_SPLIT;
        CK(attn_decode_launch(qkv.p, qkv_dim, kc, vc, ds<DecItem>(items_off(S)), n_dec * max_splits, d_seqs,
                              ds<int32_t>(off_decids), n_dec, max_splits, part_o.p, part_ml.p, attn_out.p, q_dim, nq,
                              nkv, attn_scale, num_sms, stream, attn_arrive.p));
        n_launches += (max_splits > 1 && !attn_inkernel_merge) ? 2 : 1;
      }
      if (n_tiles > 0) {
        CK(attn_prefill_launch(qkv.p, qkv_dim, kc, vc, d_seqs, ds<int32_t>(off_tileseq), ds<int32_t>(off_tileq0),
                               n_tiles, d_bt, bt_stride, attn_out.p, q_dim, nq, nkv, attn_scale, stream));
        ++n_launches;
      }
      gemm(xm_attn, l.m_o, attn_out.p, l.wo, y32.p, T, H, q_dim, /*out_f32=*/1, &l.m_gu, T, F, H);
      CK(opt_layernorm_launch(y32.p, l.b_o, resid.p, l.ln2, l.ln2_b, xn.p, T, H, c.rms_eps, stream));
      gemm(xm_xn, l.m_gu, xn.p, l.wgu, y32.p, T, F, H, /*out_f32=*/1, &l.m_d, T, H, F);
      CK(opt_bias_act_launch(y32.p, F, l.b_fc1, act.p, F, T, F, /*relu=*/1, num_sms, stream));
      // (the successor's first weight boxes are pulled into L2 by this launch's producer warp, as on the Llama path)
      if (li + 1 < c.n_layers) gemm(xm_act, l.m_d, act.p, l.wd, y32.p, T, H, F, /*out_f32=*/1, &layers[li + 1].m_qkv, T, qkv_dim, H);
      else gemm(xm_act, l.m_d, act.p, l.wd, y32.p, T, H, F, /*out_f32=*/1, R > 0 ? &m_lm : nullptr, R, Vl, H);
      n_launches += 2;
    }
    // always run (even when no row is sampled this step): a prompt-logprob pass may read xn afterwards
    CK(opt_layernorm_launch(y32.p, layers[c.n_layers - 1].b_fc2, resid.p, final_norm, final_norm_b, xn.p, T, H, c.rms_eps,
                            stream));
    ++n_launches;
  }

  // Prompt-logprob pass (vllm prompt_logprobs; grpc_server.py:609-611): lm_head + FORCED sampler rows over m prompt
  // positions of the step that has just run (row indices and SampleRows staged at off_samplesrc / off_rows).  Under tensor
  // parallelism every rank runs its vocabulary shard of the lm_head and the all-gather; rank 0 samples.
  // lm_head over `rows` rows of last_hidden -> the full [rows, V] logits on rank 0 (logits_ptr()).  Tensor parallel: every
  // rank computes its vocabulary shard; with peer mappings the shards are pushed into rank 0's buffer (logits_push_kernel,
  // no NCCL in the step), otherwise ncclAllGather + re-layout.
  // rows listed at off_samplesrc of the final-normed hidden states -> the lm_head's input rows
  void gather_final_rows(int m) {
    if (pnx_on) CK(gather_rows_any_launch(pnx_hA, ds<int32_t>(off_samplesrc), pnx_last, m, cfg.hidden, pnx_dt, stream));
    else CK(gather_rows_launch(xn.p, ds<int32_t>(off_samplesrc), last_hidden.p, m, cfg.hidden, stream));
    ++n_launches;
  }

  void lm_head_logits(int rows, int lg_idx) {
    const tgis_config& c = cfg;
    const int H = c.hidden, V = c.vocab;
    const int lm_mode = logits_bf16 ? 0 : 1;
    if (pnx_on) {
      pnx_gemm(pnx_last, pnx_dt, H, pnx_head, logits.p, DT_F32, logits_ld, rows, V, H);
    } else if (tp == 1) {
      gemm(xm_last, m_lm, last_hidden.p, lm_head, logits.p, rows, V, H, lm_mode);
    } else if (tp_fused_ar) {
      uint32_t* flags0 = reinterpret_cast<uint32_t*>(ar_peer[0] + lg_off + lg_logits_bytes());  // in rank 0's memory
      if (rank == 0) {
        gemm(xm_last, m_lm, last_hidden.p, lm_head, logits_ptr(), rows, Vl, H, lm_mode, nullptr, 0, 0, 0, /*ldy=*/V);
        CK(logits_wait_launch(flags0, tp, ds<uint32_t>(off_epoch) + 2, (uint32_t)lg_idx, stream));
      } else {
        gemm(xm_last, m_lm, last_hidden.p, lm_head, logits_shard.p, rows, Vl, H, lm_mode);
        int* counter = reinterpret_cast<int*>(ar_mem + lg_off + lg_logits_bytes() + 128);  // local
        CK(logits_push_launch(logits_shard.p, ar_peer[0] + lg_off, rows, (int)(Vl * lsz), (int)((size_t)V * lsz),
                              (int)((size_t)rank * Vl * lsz), flags0 + rank, counter, ds<uint32_t>(off_epoch) + 2,
                              (uint32_t)lg_idx, stream));
      }
      ++n_launches;
    } else {
      gemm(xm_last, m_lm, last_hidden.p, lm_head, logits_shard.p, rows, Vl, H, lm_mode);
      NK(nccl().AllGather(logits_shard.p, logits_gather.p, (size_t)rows * Vl * lsz, ncclInt8, comm, stream));
      if (rank == 0) {
        CK(launch_k(gather_relayout_kernel, dim3(148 * 4), dim3(256), 0, stream, (const uint4*)logits_gather.p,
                    (uint4*)logits.p, rows, (int)(Vl * lsz / 16), tp));
        ++n_launches;
      }
    }
  }

  void plp_pass(int m, int need_norm, int T, size_t copy_bytes, int lg_idx) {
    const tgis_config& c = cfg;
    const int H = c.hidden, V = c.vocab;
    CK(cudaMemcpyAsync(d_stage.p, h_stage, copy_bytes, cudaMemcpyHostToDevice, stream));
    if (need_norm && !opt && !pnx_on) {  // no sampled row in the step -> its final norm has not run yet (OPT: always run)
      CK(add_rmsnorm_launch(tmp.p, resid.p, final_norm, xn.p, T, H, c.rms_eps, stream));
      ++n_launches;
    }
    gather_final_rows(m);
    lm_head_logits(m, lg_idx);
    if (rank == 0) {
      CK(sampler_launch(logits_ptr(), logits_bf16 ? 1 : 0, logits_ld, logits_ld, ds<SampleRow>(off_rows), m, seen_bitmap.p, bitmap_words,
                        samp_scratch.p, d_samp_out.p, stream, /*any_complex=*/0, num_sms));
      ++n_launches;
      CK(cudaMemcpyAsync(h_plp_out, d_samp_out.p, sizeof(SampleOut) * m, cudaMemcpyDeviceToHost, stream));
    }
  }

  // Wait until everything up to ev1 (the step's last operation on the stream) has executed.
  void wait_step_end() {
    if (!sync_spin) {
      CK(cudaStreamSynchronize(stream));
      return;
    }
    for (;;) {
      const cudaError_t q = cudaEventQuery(ev1);
      if (q == cudaSuccess) return;
      if (q != cudaErrorNotReady) CK(q);
      if (stop_flag) {  // shutting down: do not spin on a possibly wedged device
        CK(cudaStreamSynchronize(stream));
        return;
      }
#if defined(__x86_64__)
      __builtin_ia32_pause();
#endif
    }
  }

  // Enqueue the step described by `h` (metadata already in h_stage): a CUDA-graph replay for pure-decode steps -- one
  // graph per (batch size, KV splits), captured on first use; every per-step quantity is read from the staged device
  // buffer, so the captured launch sequence is step-independent -- or the plain launch sequence otherwise.  Rank 0
  // and the tensor-parallel workers run the same function on the same header.
  void exec_step(const StepHeader& h) {
    if (h.kind == 1) {
      plp_pass(h.R, h.need_norm, h.T, h.copy_bytes, h.lg_idx);
      return;
    }
    if (!h.graphable) {
      launch_step(h.copy_bytes, h.T, h.n_dec, h.n_tiles, h.R, h.max_dec_kv, h.S, h.samp_complex);
      return;
    }
    const int max_splits = (h.max_dec_kv + DECODE_SPLIT - 1) / DECODE_SPLIT;
    const uint64_t key = ((uint64_t)(h.samp_complex & 7) << 40) | ((uint64_t)h.S << 16) | (uint64_t)max_splits;
    auto it = graphs.find(key);
    if (it == graphs.end()) {
      if (graphs.size() >= 64) {
        for (auto& kv : graphs) cudaGraphExecDestroy(kv.second);
        graphs.clear();
      }
      const long long launches_before = n_launches;
      cudaGraph_t g = nullptr;
      CK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
      capturing = true;
      try {
        launch_step(h.copy_bytes, h.T, h.n_dec, h.n_tiles, h.R, h.max_dec_kv, h.S, h.samp_complex);
      } catch (...) {
        capturing = false;
        cudaStreamEndCapture(stream, &g);
        if (g) cudaGraphDestroy(g);
        throw;
      }
      capturing = false;
      CK(cudaStreamEndCapture(stream, &g));
      cudaGraphExec_t ge = nullptr;
      CK(cudaGraphInstantiate(&ge, g, 0));
      CK(cudaGraphDestroy(g));
      graph_nodes[key] = n_launches - launches_before;
      n_launches = launches_before;
      it = graphs.emplace(key, ge).first;
    }
    const double t_gl = debug_launch ? now_s() : 0.0;
    if (graph_copy_outside) CK(cudaMemcpyAsync(d_stage.p, h_stage, h.copy_bytes, cudaMemcpyHostToDevice, stream));
    CK(cudaGraphLaunch(it->second, stream));
    if (graph_copy_outside && rank == 0 && h.R > 0)
      CK(cudaMemcpyAsync(h_samp_out, d_samp_out.p, sizeof(SampleOut) * h.R, cudaMemcpyDeviceToHost, stream));
    if (debug_launch) graph_launch_host_s += now_s() - t_gl;
    n_launches += graph_nodes[key];
    ++n_graph_launches;
  }

  // returns number of sampled rows
  int run_batch(std::vector<Sched>& batch) {
    const tgis_config& c = cfg;
    const int H = c.hidden, V = c.vocab;
    int T = 0, n_dec = 0, n_tiles = 0, R = 0, max_dec_kv = 0, samp_complex = 0;
    struct PromptRow {
      int row, target, pos;
      Request* r;
    };
    std::vector<PromptRow> prompt_rows;
    int32_t* tok = hs<int32_t>(off_tok);
    int32_t* pos = hs<int32_t>(off_pos);
    int32_t* slotmap = hs<int32_t>(off_slotmap);
    int32_t* tokslot = hs<int32_t>(off_tokslot);
    int32_t* toklora = hs<int32_t>(off_toklora);
    AttnSeq* seqs = hs<AttnSeq>(off_seqs);
    int32_t* decids = hs<int32_t>(off_decids);
    int32_t* tileseq = hs<int32_t>(off_tileseq);
    int32_t* tileq0 = hs<int32_t>(off_tileq0);
    int32_t* samplesrc = hs<int32_t>(off_samplesrc);
    SampleRow* rows = hs<SampleRow>(off_rows);
    int32_t* bt = hs<int32_t>(off_bt);
    const int S = (int)batch.size();
    step_n_ltiles = 0;
    step_n_ltiles16 = 0;
    step_max_q = 0;
    step_max_kv = 0;
    for (int s = 0; s < S; ++s) {
      Request& r = *batch[s].r;
      const int q_len = batch[s].q_len;
      const int kv_len = r.n_computed + q_len;
      step_max_kv = std::max(step_max_kv, kv_len);
      seqs[s] = AttnSeq{T, q_len, kv_len, s};
      memcpy(bt + (size_t)s * bt_stride, r.blocks.data(), sizeof(int32_t) * r.blocks.size());
      for (int j = 0; j < q_len; ++j) {
        const int p = r.n_computed + j;
        tok[T + j] = r.tokens[p];
        pos[T + j] = p;
        slotmap[T + j] = r.blocks[p / KV_BLOCK] * KV_BLOCK + p % KV_BLOCK;
        tokslot[T + j] = r.slot;
        toklora[T + j] = r.sp.lora_slot;
      }
      if (r.sp.lora_slot > 0) samp_complex |= 4;  // step flag: some token carries a LoRA adapter
      if (r.sp.prompt_logprobs > 0 && r.n_computed < r.n_prompt - 1) {
        // prompt logprobs (vllm gpu_model_runner.py:3638): position p predicts prompt token p+1
        for (int j = 0; j < q_len; ++j) {
          const int p = r.n_computed + j;
          if (p + 1 < r.n_prompt) prompt_rows.push_back(PromptRow{T + j, r.tokens[p + 1], p + 1, &r});
        }
      }
      if (pnx_on) {  // latent-attention query tiles: prompts, portions and single tokens alike
        LatentTile* lt = hs<LatentTile>(off_ltiles);
        for (int q0 = 0; q0 < q_len; q0 += pnx_tile_tokens)
          lt[step_n_ltiles++] = LatentTile{s, q0, std::min(pnx_tile_tokens, q_len - q0), 0};
        if (pair_style) {
          LatentTile* lt16 = hs<LatentTile>(off_ltiles16);
          for (int q0 = 0; q0 < q_len; q0 += POOLATTN_TILE)
            lt16[step_n_ltiles16++] = LatentTile{s, q0, std::min(POOLATTN_TILE, q_len - q0), 0};
          step_max_q = std::max(step_max_q, q_len);
        }
      }
      if (q_len == 1) {
        decids[n_dec++] = s;
        max_dec_kv = std::max(max_dec_kv, kv_len);
      } else {
        for (int q0 = 0; q0 < q_len; q0 += 16) {
          tileseq[n_tiles] = s;
          tileq0[n_tiles++] = q0;
        }
      }
      if (batch[s].sample) {
        const tgis_sampling_params& sp = r.sp;
        SampleRow& row = rows[R];
        memset(&row, 0, sizeof(row));
        const int n_out = r.n_out();
        row.flags = (sp.greedy ? SAMPLE_GREEDY : 0) | (sp.num_logprobs > 0 ? SAMPLE_LOGPROBS : 0) |
                    ((sp.typical_p > 0.f && sp.typical_p < 1.f) ? SAMPLE_TYPICAL : 0);
        if (!(row.flags & SAMPLE_GREEDY) || (row.flags & SAMPLE_TYPICAL)) samp_complex |= 1;
        row.n_topn = std::min<int>(sp.num_logprobs > 0 ? sp.num_logprobs : 0, MAX_TOPN);
        row.temperature = sp.greedy ? 1.f : sp.temperature;
        row.top_k = sp.greedy ? 0 : sp.top_k;
        row.top_p = sp.greedy ? 1.f : ((sp.top_p > 0.f && sp.top_p < 1.f) ? sp.top_p : 1.f);
        row.typical_p = sp.typical_p;
        row.rep_penalty = sp.repetition_penalty > 0.f ? sp.repetition_penalty : 1.f;
        row.len_decay_factor = 0.f;
        if (sp.has_length_penalty) {
          // reference: tgis_utils/logits_processors.py:38-46  p_factor = pow(penalty, max(0, n_out - start)) (python
          // double); logit + |logit| * (p_factor - 1) with the scalar cast to fp32
          const int past = std::max(0, n_out - (int)sp.lp_start_index);
          const double pf = std::pow((double)sp.lp_decay_factor, (double)past);
          if (pf != 1.0) {
            row.flags |= SAMPLE_LENPEN;
            row.len_decay_factor = (float)(pf - 1.0);
          }
        }
        row.eos_id = sp.eos_token_id;
        row.n_out = n_out;
        row.min_tokens = sp.min_tokens;
        row.seq_slot = r.slot;
        row.seed_lo = (uint32_t)r.seed;
        row.seed_hi = (uint32_t)(r.seed >> 32);
        row.step = (uint32_t)n_out;
        row.logits_row = R;
        if (sp.guided) {
          // guided decoding: report the tokens generated since the last call, get this step's allowed-token bits
          // (vllm v1/structured_output/__init__.py:204-300 grammar_bitmask) and ship them ahead of the step
          tgis_mask_fn fn;
          void* user;
          {
            std::lock_guard<std::mutex> lk(mu);
            fn = mask_fn;
            user = mask_user;
          }
          int rc = -1;
          uint32_t* hm = h_allow + (size_t)r.slot * bitmap_words;
          if (fn != nullptr)
            rc = fn(user, r.id.c_str(), r.tokens.data() + r.n_prompt + r.guided_fed, n_out - r.guided_fed, hm, bitmap_words);
          r.guided_fed = n_out;
          if (rc == 0) {
            row.flags |= SAMPLE_MASKED;
            samp_complex |= 2;
            CK(cudaMemcpyAsync(allow_bitmap.p + (size_t)r.slot * bitmap_words, hm, sizeof(uint32_t) * bitmap_words,
                               cudaMemcpyHostToDevice, stream));
            h2d_bytes += (long long)sizeof(uint32_t) * bitmap_words;
            ++guided_rows;
          } else if (rc < 0) {
            r.aborted = true;  // the provider failed: the request ends with TGIS_FINISH_ABORT at the next step
          }
        }
        samplesrc[R] = T + q_len - 1;
        ++R;
      }
      T += q_len;
    }
    // ---- ship metadata + run the layer stack (one CUDA graph launch for a pure-decode step when enabled)
    // decode work items: (sequence, DECODE_SPLIT-token split) entries; the copy covers the worst case for this
    // (S, max_splits) so that its size is a function of the CUDA-graph key
    const int max_splits_step = (max_dec_kv + DECODE_SPLIT - 1) / DECODE_SPLIT;
    decode_items_build(hs<DecItem>(items_off(S)), seqs, decids, n_dec, bt, bt_stride);
    const size_t copy_bytes = items_off(S) + sizeof(DecItem) * (1 + (size_t)n_dec * max_splits_step);
    const double t_ev0 = debug_launch ? now_s() : 0.0;
    CK(cudaEventRecord(ev0, stream));
    const bool graphable = cfg.use_cuda_graphs && (tp == 1 || tp_graphs) && !profiling && n_tiles == 0 && n_dec == S && R == S;
    StepHeader hdr{T, n_dec, n_tiles, R, max_dec_kv, S, graphable ? 1 : 0, samp_complex, (uint64_t)copy_bytes, 0, 0, 1, 0};
    if (tp > 1) {
      // exchange epochs of this step = staged base + index inside the step (ar_add_rmsnorm_kernel)
      uint32_t* eb = hs<uint32_t>(off_epoch);
      eb[0] = ar_epoch[0];
      eb[1] = ar_epoch[1];
      lg_epoch += (uint32_t)lg_idx_step;  // gathers of the previous step (its own and its prompt-logprob passes)
      eb[2] = lg_epoch;
      lg_idx_step = (R > 0) ? 1 : 0;
      if (exchange_mode(T) != 0) {
        ar_epoch[0] += (uint32_t)cfg.n_layers;
        ar_epoch[1] += (uint32_t)cfg.n_layers;
      }
      publish_plan(hdr);
    }
    exec_step(hdr);
    CK(cudaEventRecord(ev1, stream));
    const double t_launched = debug_launch ? now_s() : 0.0;
    wait_step_end();
    if (debug_launch) {
      t_after_wait = now_s();
      host_phases.push_back(HostPhase{(float)(1e6 * (t_ev0 - t_step_begin)), (float)(1e6 * (t_launched - t_ev0)),
                                      (float)(1e6 * (t_after_wait - t_launched)), 0.f});
    }
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, ev0, ev1));
    gpu_ms += ms;
    h2d_bytes += (long long)copy_bytes;
    d2h_bytes += (long long)sizeof(SampleOut) * R;
    if (n_tiles == 0) {  // pure decode step
      gpu_ms_decode += ms;
      ++decode_steps;
      decode_tokens += R;
    } else {
      gpu_ms_mixed += ms;
    }
    if (profiling) {
      for (size_t i = 0; i + 1 < prof_used; i += 2) {
        float gm = 0.f;
        CK(cudaEventElapsedTime(&gm, prof_events[i], prof_events[i + 1]));
        if (prof_bytes[i / 2] < 0) {
          exchange_ms += gm;
          ++exchange_calls;
        } else {
          gemm_ms += gm;
          gemm_bytes += prof_bytes[i / 2];
          ++gemm_calls;
        }
      }
      prof_used = 0;
      prof_bytes.clear();
    }
    // ---- prompt logprobs: lm_head + forced-token sampler rows over the prompt positions of this step, S_max rows at a
    // time (512x the decode logits work per prompt: rare, so it stays a simple separate pass on the same stream)
    if (!prompt_rows.empty()) {
      const bool fused_exchange = exchange_mode(T) != 0;   // then the final norm always ran
      int need_norm = (R == 0 && !fused_exchange) ? 1 : 0;
      const size_t plp_bytes = off_rows + sizeof(SampleRow) * (size_t)S_max;  // the staged regions up to the sample rows
      for (size_t off = 0; off < prompt_rows.size(); off += (size_t)S_max) {
        const int m = (int)std::min<size_t>(S_max, prompt_rows.size() - off);
        for (int i = 0; i < m; ++i) {
          const PromptRow& pr = prompt_rows[off + i];
          samplesrc[i] = pr.row;
          SampleRow& row = rows[i];
          memset(&row, 0, sizeof(row));
          row.flags = SAMPLE_FORCED | SAMPLE_LOGPROBS;
          row.n_topn = std::min<int>(pr.r->sp.prompt_logprobs, MAX_TOPN);
          row.temperature = 1.f;
          row.top_p = 1.f;
          row.rep_penalty = 1.f;
          row.eos_id = -1;
          row.seq_slot = -1;
          row.seed_lo = (uint32_t)pr.target;
          row.logits_row = i;
        }
        StepHeader ph{T, 0, 0, m, 0, 0, 0, 0, (uint64_t)plp_bytes, 1, need_norm, ++lg_idx_step, 0};
        if (tp > 1) publish_plan(ph);
        exec_step(ph);
        need_norm = 0;
        CK(cudaStreamSynchronize(stream));
        for (int i = 0; i < m; ++i) emit_prompt(*prompt_rows[off + i].r, prompt_rows[off + i].pos, h_plp_out[i]);
      }
    }
    return R;
  }

  // ------------------------------------------------------------------------------------------------ scheduler
  void free_request(Request& r) {
    for (int b : r.blocks) free_blocks.push_back(b);
    r.blocks.clear();
    if (r.slot >= 0) free_slots.push_back(r.slot);
    r.slot = -1;
  }
  bool ensure_blocks(Request& r, int n_tokens) {
    const int need = (n_tokens + KV_BLOCK - 1) / KV_BLOCK;
    while ((int)r.blocks.size() < need) {
      if (free_blocks.empty()) return false;
      r.blocks.push_back(free_blocks.back());
      free_blocks.pop_back();
    }
    return true;
  }
  void emit_prompt(const Request& r, int pos, const SampleOut& so) {
    tgis_step_output o;
    memset(&o, 0, sizeof(o));
    snprintf(o.request_id, sizeof(o.request_id), "%s", r.id.c_str());
    o.prompt_pos = pos;
    o.token_id = so.token;
    o.logprob = so.logprob;
    o.rank = so.rank;
    o.n_topn = so.n_topn;
    for (int i = 0; i < o.n_topn; ++i) {
      o.topn_ids[i] = so.topn_ids[i];
      o.topn_logprobs[i] = so.topn_lps[i];
    }
    o.n_prompt_tokens = r.n_prompt;
    o.ts_arrival = r.ts_arrival;
    std::lock_guard<std::mutex> lk(mu);
    outputs.push_back(o);
    cv_out.notify_all();
  }

  void emit(const Request& r, bool new_token, const SampleOut* so, int finish, int stop_tok) {
    tgis_step_output o;
    memset(&o, 0, sizeof(o));
    snprintf(o.request_id, sizeof(o.request_id), "%s", r.id.c_str());
    o.prompt_pos = -1;
    o.n_new_tokens = new_token ? 1 : 0;
    if (new_token && so) {
      o.token_id = so->token;
      o.logprob = so->logprob;
      o.rank = so->rank;
      o.n_topn = r.sp.num_logprobs > 0 ? so->n_topn : 0;
      for (int i = 0; i < o.n_topn; ++i) {
        o.topn_ids[i] = so->topn_ids[i];
        o.topn_logprobs[i] = so->topn_lps[i];
      }
    }
    o.finish_reason = finish;
    o.stop_token_id = stop_tok;
    o.n_prompt_tokens = r.n_prompt;
    o.n_output_tokens = r.n_out();
    o.ts_arrival = r.ts_arrival;
    o.ts_first_scheduled = r.ts_first_sched;
    o.ts_first_token = r.ts_first_token;
    o.ts_last_token = r.ts_last_token;
    std::lock_guard<std::mutex> lk(mu);
    outputs.push_back(o);
    cv_out.notify_all();
  }

  // ------------------------------------------------------------------------------------------------ trace replay
  // lm_head over the listed rows of the step that has just run -> fp32 logits on the host, logit_rows_cap rows at a time
  void logits_of_rows(const std::vector<int>& rows, int T, float* out) {
    const int V = cfg.vocab;
    bool need_norm = !opt && !pnx_on;  // the Llama stack leaves its last residual add + final norm to the sampling tail
    for (size_t off = 0; off < rows.size(); off += (size_t)logit_rows_cap) {
      const int m = (int)std::min<size_t>(logit_rows_cap, rows.size() - off);
      int32_t* src = hs<int32_t>(off_samplesrc);
      for (int i = 0; i < m; ++i) src[i] = rows[off + i];
      CK(cudaMemcpyAsync(d_stage.p + off_samplesrc, h_stage + off_samplesrc, sizeof(int32_t) * m, cudaMemcpyHostToDevice,
                         stream));
      if (need_norm) {
        CK(add_rmsnorm_launch(tmp.p, resid.p, final_norm, xn.p, T, cfg.hidden, cfg.rms_eps, stream));
        ++n_launches;
        need_norm = false;
      }
      gather_final_rows(m);
      lm_head_logits(m, 1);
      CK(cudaMemcpyAsync(h_trace_logits, logits.p, (size_t)m * logits_ld * lsz, cudaMemcpyDeviceToHost, stream));
      CK(cudaStreamSynchronize(stream));
      d2h_bytes += (long long)m * logits_ld * lsz;
      float* dst = out + off * V;
      if (logits_bf16) {
        const bf16* hb = reinterpret_cast<const bf16*>(h_trace_logits);
        for (size_t i = 0; i < (size_t)m * V; ++i) dst[i] = __bfloat162float(hb[i]);  // (logits_ld == V)
      } else {
        for (int r = 0; r < m; ++r)
          memcpy(dst + (size_t)r * V, h_trace_logits + (size_t)r * logits_ld, (size_t)V * sizeof(float));
      }
    }
  }

  int trace_step(const tgis_trace_entry* entries, int n_entries, const char* const* end_ids, int n_end, float* logits_out) {
    if (tp > 1) throw CudaError("trace replay runs on a single GPU");
    if (n_entries > S_max) throw CudaError("more entries than sequence slots in one step");
    std::vector<Request*> req(n_entries, nullptr);
    int T = 0;
    for (int i = 0; i < n_entries; ++i) {
      const tgis_trace_entry& en = entries[i];
      if (!en.request_id || !en.tokens || en.n_tokens < 1) throw CudaError("bad trace entry");
      for (int j = 0; j < i; ++j)
        if (strcmp(entries[j].request_id, en.request_id) == 0) throw CudaError("a request appears twice in one step");
      for (auto& r : running)
        if (r->id == en.request_id) req[i] = r.get();
      if (!req[i]) {  // admitted at its first entry
        if (free_slots.empty() || (int)running.size() >= S_max) throw CudaError("no free sequence slot for " + std::string(en.request_id));
        auto r = std::make_unique<Request>();
        r->id = en.request_id;
        r->slot = free_slots.back();
        free_slots.pop_back();
        r->ts_arrival = now_s();
        req[i] = r.get();
        running.push_back(std::move(r));
      }
      Request& r = *req[i];
      for (int j = 0; j < en.n_tokens; ++j) {
        if (en.tokens[j] < 0 || en.tokens[j] >= cfg.vocab) throw CudaError("token id out of range");
        r.tokens.push_back(en.tokens[j]);
      }
      r.n_prompt = (int)r.tokens.size();
      if ((int)r.tokens.size() > cfg.max_model_len) throw CudaError("request longer than max_model_len");
      if (!ensure_blocks(r, (int)r.tokens.size())) throw CudaError("cache pool exhausted");
      for (int j = 0; j < en.n_want; ++j)
        if (en.want[j] < 0 || en.want[j] >= en.n_tokens) throw CudaError("wanted position outside the entry");
      T += en.n_tokens;
    }
    if (T > T_max) throw CudaError("step exceeds max_batched_tokens");
    // the step order of step(): single tokens first, then the portions
    std::vector<int> order;
    for (int pass = 0; pass < 2; ++pass)
      for (int i = 0; i < n_entries; ++i)
        if ((entries[i].n_tokens == 1) == (pass == 0)) order.push_back(i);
    std::vector<Sched> batch;
    std::vector<int> row0(n_entries, 0);
    int at = 0;
    for (int i : order) {
      batch.push_back(Sched{req[i], entries[i].n_tokens, false});
      row0[i] = at;
      at += entries[i].n_tokens;
    }
    if (!batch.empty()) {
      run_batch(batch);
      ++n_steps;
      for (Sched& s : batch) s.r->n_computed += s.q_len;
      std::vector<int> rows;
      for (int i = 0; i < n_entries; ++i)
        for (int j = 0; j < entries[i].n_want; ++j) rows.push_back(row0[i] + entries[i].want[j]);
      if (!rows.empty()) {
        if (!logits_out) throw CudaError("logits wanted but no output buffer");
        logits_of_rows(rows, T, logits_out);
      }
    }
    for (int k = 0; k < n_end; ++k)
      for (size_t i = 0; i < running.size(); ++i)
        if (running[i]->id == end_ids[k]) {
          free_request(*running[i]);
          running.erase(running.begin() + i);
          break;
        }
    snapshot();
    return 0;
  }

  // one engine step; returns false when there was nothing to do
  bool step() {
    if (debug_step_sleep_us > 0) usleep(debug_step_sleep_us);  // experiment: GPU idle time between steps
    if (debug_launch) t_step_begin = now_s();
    // ---- intake
    {
      std::lock_guard<std::mutex> lk(mu);
      while (!incoming.empty()) {
        waiting.push_back(std::move(incoming.front()));
        incoming.pop_front();
      }
      for (const std::string& id : abort_ids) {
        for (auto& r : running)
          if (r->id == id) r->aborted = true;
        for (auto& r : waiting)
          if (r->id == id) r->aborted = true;
      }
      abort_ids.clear();
    }
    for (size_t i = 0; i < running.size();) {
      if (running[i]->aborted) {
        emit(*running[i], false, nullptr, TGIS_FINISH_ABORT, -1);
        free_request(*running[i]);
        running.erase(running.begin() + i);
      } else ++i;
    }
    for (size_t i = 0; i < waiting.size();) {
      if (waiting[i]->aborted) {
        emit(*waiting[i], false, nullptr, TGIS_FINISH_ABORT, -1);
        waiting.erase(waiting.begin() + i);
      } else ++i;
    }
    if (running.empty() && waiting.empty()) {
      snapshot();
      return false;
    }

    // ---- schedule
    std::vector<Sched> dec, pre;
    int budget = T_max;
    for (size_t i = 0; i < running.size(); ++i) {
      Request& r = *running[i];
      int remaining = (int)r.tokens.size() - r.n_computed;
      if (budget <= 0) break;
      int q = std::min(remaining, budget);
      bool ok = ensure_blocks(r, r.n_computed + q);
      while (!ok && running.size() > i + 1) {  // preempt from the back (recompute later)
        std::unique_ptr<Request> victim = std::move(running.back());
        running.pop_back();
        free_request(*victim);
        victim->n_computed = 0;
        ++n_preempt;
        waiting.push_front(std::move(victim));
        ok = ensure_blocks(r, r.n_computed + q);
      }
      if (!ok) {  // r itself is the last one: preempt it
        std::unique_ptr<Request> victim = std::move(running.back());
        running.pop_back();
        free_request(*victim);
        victim->n_computed = 0;
        ++n_preempt;
        waiting.push_front(std::move(victim));
        break;
      }
      budget -= q;
      Sched s{&r, q, r.n_computed + q == (int)r.tokens.size()};
      (q == 1 ? dec : pre).push_back(s);
    }
    const double t_now = now_s();
    while (!waiting.empty() && budget > 0 && (int)running.size() < S_max && !free_slots.empty()) {
      Request& r = *waiting.front();
      const int remaining = (int)r.tokens.size() - r.n_computed;
      const int q = std::min(remaining, budget);
      // admit only if the whole sequence so far fits (keeps chunked prefill from dead-locking the cache)
      if ((int)free_blocks.size() < ((int)r.tokens.size() + KV_BLOCK) / KV_BLOCK) break;
      r.slot = free_slots.back();
      free_slots.pop_back();
      ensure_blocks(r, r.n_computed + q);
      CK(bitmap_clear_launch(seen_bitmap.p, bitmap_words, r.slot, stream));
      ++n_launches;
      if (r.ts_first_sched == 0) r.ts_first_sched = t_now;
      budget -= q;
      Sched s{&r, q, r.n_computed + q == (int)r.tokens.size()};
      (q == 1 ? dec : pre).push_back(s);
      running.push_back(std::move(waiting.front()));
      waiting.pop_front();
    }
    std::vector<Sched> batch;
    batch.reserve(dec.size() + pre.size());
    batch.insert(batch.end(), dec.begin(), dec.end());
    batch.insert(batch.end(), pre.begin(), pre.end());
    if (batch.empty()) {
      if (!waiting.empty() && running.empty())
        throw CudaError("request does not fit in the KV cache (" + std::to_string(num_blocks) + " blocks)");
      snapshot();
      return false;
    }

    // LoRA: sequences that share an adapter sit next to each other in the step, so that lora.cu's 8-token tiles are
    // same-adapter tiles (A / B rows read once per tile) instead of falling back to one pass per token.  Every kernel's
    // result for a token is independent of its neighbours, and post-processing below walks the same order.
    if (max_loras > 0) {
      bool any_lora = false;
      for (const Sched& s : batch) any_lora |= s.r->sp.lora_slot > 0;
      if (any_lora)
        std::stable_sort(batch.begin(), batch.end(),
                         [](const Sched& a, const Sched& b) { return a.r->sp.lora_slot < b.r->sp.lora_slot; });
    }

    // ---- run
    run_batch(batch);
    ++n_steps;

    // ---- post-process (vllm v1/core/sched/utils.py:94-130 check_stop)
    const double t_done = now_s();
    int R = 0;
    std::vector<Request*> finished;
    for (Sched& s : batch) {
      Request& r = *s.r;
      r.n_computed += s.q_len;
      if (!s.sample) continue;
      const SampleOut& so = h_samp_out[R++];
      r.tokens.push_back(so.token);
      ++n_tokens;
      if (r.ts_first_token == 0) r.ts_first_token = t_done;
      r.ts_last_token = t_done;
      int finish = TGIS_FINISH_NONE, stop_tok = -1;
      const int n_out = r.n_out();
      if (n_out >= r.sp.min_tokens) {
        if (so.token == r.sp.eos_token_id) finish = TGIS_FINISH_STOP_EOS;
        else {
          for (int k = 0; k < r.sp.n_stop_token_ids; ++k)
            if (r.sp.stop_token_ids[k] == so.token) {
              finish = TGIS_FINISH_STOP_TOKEN;
              stop_tok = so.token;
            }
        }
        if (finish == TGIS_FINISH_NONE && ((int)r.tokens.size() >= cfg.max_model_len || n_out >= r.sp.max_tokens))
          finish = TGIS_FINISH_LENGTH;
      }
      // Safety net outside the min_tokens guard (vLLM's check_stop returns early there; its SamplingParams validation
      // is what keeps min_tokens <= max_tokens -- add_request enforces the same, so this never changes a result): a
      // sequence must never outgrow its block-table row / the RoPE table.
      if (finish == TGIS_FINISH_NONE && (int)r.tokens.size() >= cfg.max_model_len) finish = TGIS_FINISH_LENGTH;
      emit(r, true, &so, finish, stop_tok);
      if (finish != TGIS_FINISH_NONE) finished.push_back(&r);
    }
    for (Request* f : finished) {
      for (size_t i = 0; i < running.size(); ++i)
        if (running[i].get() == f) {
          free_request(*running[i]);
          running.erase(running.begin() + i);
          break;
        }
    }
    snapshot();
    if (debug_launch && !host_phases.empty()) host_phases.back().post = (float)(1e6 * (now_s() - t_after_wait));
    return true;
  }

  void fail_all(const std::string& msg) {
    error_msg = msg;
    errored = true;
    std::vector<std::unique_ptr<Request>> all;
    {
      std::lock_guard<std::mutex> lk(mu);
      for (auto& r : incoming) all.push_back(std::move(r));
      incoming.clear();
    }
    for (auto& r : waiting) all.push_back(std::move(r));
    waiting.clear();
    for (auto& r : running) all.push_back(std::move(r));
    running.clear();
    for (auto& r : all) emit(*r, false, nullptr, TGIS_FINISH_ERROR, -1);
    snapshot();
  }

  void loop() {
    thread_alive = true;
    cudaSetDevice(cfg.device);
    while (!stop_flag) {
      bool did = false;
      try {
        did = step();
      } catch (const std::exception& e) {
        fail_all(e.what());
        break;
      }
      if (!did) {
        std::unique_lock<std::mutex> lk(mu);
        cv_in.wait_for(lk, std::chrono::milliseconds(50),
                       [&] { return stop_flag || !incoming.empty() || !abort_ids.empty(); });
      }
    }
    thread_alive = false;
    cv_out.notify_all();
  }
};

// ==================================================================================================== C ABI
extern "C" {

const char* tgis_last_error(void) { return g_last_error.c_str(); }
static_assert(offsetof(tgis_sampling_params, lora_slot) == 112, "ctypes mirror: engine/_lib.py TgisSamplingParams");
static_assert(sizeof(tgis_sampling_params) == 120, "ctypes mirror: engine/_lib.py TgisSamplingParams");
static_assert(sizeof(tgis_config) == 304, "ctypes mirror: engine/_lib.py TgisConfig");
int tgis_abi_version(void) { return TGIS_ABI_VERSION; }

int tgis_engine_create(const tgis_config* cfg, tgis_engine** out) {
  if (!cfg || !out) return fail("null argument");
  if (cfg->abi_version != TGIS_ABI_VERSION) return fail("ABI version mismatch");
  if (cfg->arch == TGIS_ARCH_PONENEX || cfg->arch == TGIS_ARCH_FALERAX || cfg->arch == TGIS_ARCH_REVEPEL || cfg->arch == TGIS_ARCH_SIKAZEN)
    return fail("this architecture is described layer by layer: use tgis_engine_create_spec");
  if (cfg->arch != TGIS_ARCH_LLAMA && cfg->arch != TGIS_ARCH_OPT) return fail("unknown arch");
  if (cfg->arch == TGIS_ARCH_OPT) {
    if (cfg->head_dim != 64 && cfg->head_dim != HEAD_DIM) return fail("OPT: head_dim must be 64 or 128");
    if (cfg->n_q_heads != cfg->n_kv_heads) return fail("OPT: n_kv_heads must equal n_q_heads (multi-head attention)");
    if (cfg->hidden != cfg->n_q_heads * cfg->head_dim) return fail("OPT: hidden must be n_q_heads * head_dim");
    if (cfg->tp_size > 1) return fail("OPT runs on a single GPU only (tp_size must be 1)");
    if (cfg->max_loras > 0) return fail("OPT: LoRA adapter slots are not supported (max_loras must be 0)");
  } else if (cfg->head_dim != HEAD_DIM) {
    return fail("head_dim must be 128");
  }
  if (cfg->n_kv_heads <= 0 || cfg->n_q_heads % cfg->n_kv_heads != 0) return fail("n_q_heads must be a multiple of n_kv_heads");
  const int G = cfg->n_q_heads / cfg->n_kv_heads;
  if (!(G == 1 || G == 2 || G == 3 || G == 4 || G == 8)) return fail("GQA group size must be 1, 2, 3, 4 or 8");
  if (cfg->hidden % 64 || cfg->ffn % 64 || cfg->vocab % 8) return fail("hidden/ffn must be multiples of 64, vocab of 8");
  if (cfg->hidden > 8192) return fail("hidden > 8192 unsupported");
  const int tpv = cfg->tp_size > 1 ? cfg->tp_size : 1;
  if (tpv > 16 || cfg->tp_rank < 0 || cfg->tp_rank >= tpv) return fail("bad tp_size / tp_rank");
  if (cfg->n_kv_heads % tpv || cfg->ffn % (64 * tpv) || cfg->vocab % (8 * tpv))
    return fail("n_kv_heads, ffn/64 and vocab/8 must be divisible by tp_size");
  if (cfg->max_batched_tokens < 16 || cfg->max_num_seqs < 1 || cfg->max_model_len < 2) return fail("bad limits");
  if (cfg->max_loras < 0 || cfg->max_loras > 64) return fail("max_loras must be in [0, 64]");
  if (cfg->max_loras > 0) {
    if (tpv > 1) return fail("LoRA adapters are supported on a single GPU only (tp_size must be 1)");
    if (cfg->max_lora_rank < 8 || cfg->max_lora_rank > 64 || cfg->max_lora_rank % 8)
      return fail("max_lora_rank must be a multiple of 8 in [8, 64]");
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail("no CUDA device: the TGIS engine has no CPU fallback");
  auto* e = new tgis_engine();
  e->cfg = *cfg;
  try {
    e->init();
  } catch (const std::exception& ex) {
    std::string m = ex.what();
    delete e;
    return fail(m);
  }
  *out = e;
  return 0;
}

int tgis_engine_create_spec(const tgis_config* cfg, const tgis_model_spec* spec, tgis_engine** out) {
  if (!cfg || !spec || !out || !spec->layers) return fail("null argument");
  if (cfg->abi_version != TGIS_ABI_VERSION) return fail("ABI version mismatch");
  if (cfg->arch != TGIS_ARCH_PONENEX && cfg->arch != TGIS_ARCH_FALERAX && cfg->arch != TGIS_ARCH_REVEPEL && cfg->arch != TGIS_ARCH_SIKAZEN)
    return fail("tgis_engine_create_spec: arch must be a layer-list architecture");
  if (spec->n_layers < 1 || spec->n_layers > 4096) return fail("bad n_layers");
  if (spec->dtype != TGIS_DTYPE_BF16 && spec->dtype != TGIS_DTYPE_F32) return fail("dtype must be bf16 or fp32");
  if (cfg->hidden < 1 || cfg->hidden > 12288 || cfg->vocab < 1) return fail("bad hidden / vocab");
  if (cfg->tp_size > 1) return fail("this architecture runs on a single GPU only (tp_size must be 1)");
  if (cfg->max_loras > 0) return fail("LoRA adapter slots are not supported for this architecture");
  if (cfg->max_batched_tokens < 1 || cfg->max_num_seqs < 1 || cfg->max_model_len < 2) return fail("bad limits");
  for (int i = 0; i < spec->n_layers; ++i) {
    const tgis_layer_spec& s = spec->layers[i];
    const std::string at = " (layer " + std::to_string(i) + ")";
    const bool post = (spec->style & TGIS_STYLE_POST_NORM) != 0;
    if ((spec->style & TGIS_STYLE_PARALLEL_PAIR) != 0) {
      if (spec->style != TGIS_STYLE_PARALLEL_PAIR) return fail("the parallel pair style has its own norm placement and an untied head");
      if (spec->side_dim < 0 || spec->side_dim > 4096) return fail("bad width of the per-layer token input");
      if (spec->loop_times > 1 && (spec->loop_start < 0 || spec->loop_stop > spec->n_layers || spec->loop_start >= spec->loop_stop))
        return fail("the looped span must lie inside the layer list");
      if (spec->loop_times > 64) return fail("more than 64 passes of a loop");
      if (s.mlp != TGIS_MLP_NONE && s.mlp != TGIS_MLP_DENSE_SILU) return fail("unknown feed-forward kind" + at);
      if (s.mlp == TGIS_MLP_DENSE_SILU && s.ff < 1) return fail("bad feed-forward width" + at);
      if (s.rot_dims > 0 && !(s.rot_base > 0.f)) return fail("bad rotary base" + at);
      if (s.mixer == TGIS_MIXER_POOLED_ATTENTION) {
        if (s.heads < 1 || s.kv_heads < 1 || s.heads % s.kv_heads != 0 || s.dim < 1 || s.vdim < 1 || s.vdim > POOLATTN_MAX_VDIM ||
            s.dim > 512)
          return fail("bad attention sizes" + at);
        if (s.rot_dims < 0 || s.rot_dims > s.dim || (s.rot_dims & 1)) return fail("rot.dims must be even and <= dim" + at);
        if (s.pool > 0 && s.window <= 0) return fail("pooled blocks need a window" + at);
      } else if (s.mixer == TGIS_MIXER_HGRN) {
        if (s.heads < 1 || s.dim < 1 || s.dim > OUTER_SCAN_MAX_DIM || s.vdim < 1) return fail("bad hgrn sizes" + at);
      } else if (s.mixer == TGIS_MIXER_LATENT_ATTENTION) {
        if (s.heads < 1 || s.dim < 1 || s.rot_dim < 0 || s.vdim < 1 || s.kv_rank < 1 || s.q_rank < 1) return fail("bad mixer sizes" + at);
        if (s.kv_rank > 512) return fail("kv_rank > 512 unsupported" + at);
        if (s.rot_dims < 0 || s.rot_dims > s.rot_dim || (s.rot_dims & 1)) return fail("rot.dims must be even and <= rot_dim" + at);
      } else {
        return fail("unknown mixer type" + at);
      }
      continue;
    }
    if ((spec->style & TGIS_STYLE_PARALLEL_GATED) != 0) {
      if (post || (spec->style & TGIS_STYLE_TIED_HEAD) != 0) return fail("the parallel gated style has its own norm placement and an untied head");
      if (s.mlp != TGIS_MLP_NONE && s.mlp != TGIS_MLP_MOE_SIGMOID) return fail("unknown feed-forward kind" + at);
      if (s.mlp == TGIS_MLP_MOE_SIGMOID && (s.experts < 1 || s.top < 1 || s.top > s.experts || s.top > 32 || s.expert_ff < 1 ||
                                            s.shared_ff < 0 || s.experts > 2048))
        return fail("bad mixture-of-experts sizes" + at);
      if (s.mixer == TGIS_MIXER_SIGMOID_ATTENTION) {
        if (s.heads < 1 || s.kv_heads < 1 || s.heads % s.kv_heads != 0 || s.dim < 1 || s.vdim < 1 || s.vdim > SIGATTN_MAX_VDIM ||
            s.dim > 512)
          return fail("bad attention sizes" + at);
        if (s.rot_dims < 0 || s.rot_dims > s.dim || (s.rot_dims & 1)) return fail("rot.dims must be even and <= dim" + at);
        if (s.rot_dims > 0 && !(s.rot_base > 0.f)) return fail("bad rotary base" + at);
        if (s.yarn_factor > 0.f && !(s.yarn_original > 0.f && s.yarn_fast > 0.f && s.yarn_slow > 0.f && s.rot_base > 1.f))
          return fail("bad rotary scaling" + at);
        if (s.kv_from > 0) {
          if (s.kv_from - 1 >= i) return fail("kv_from must name an earlier layer" + at);
          const tgis_layer_spec& o = spec->layers[s.kv_from - 1];
          if (o.mixer != TGIS_MIXER_SIGMOID_ATTENTION || o.kv_from > 0 || o.kv_heads != s.kv_heads || o.dim != s.dim || o.vdim != s.vdim)
            return fail("kv_from must name an attention layer with keys and values of its own and the same sizes" + at);
        }
      } else if (s.mixer == TGIS_MIXER_SSD) {
        if (s.heads < 1 || s.vdim < 1 || s.state < 1 || s.state > OUTER_SCAN_MAX_DIM || s.groups < 1 || s.heads % s.groups != 0 ||
            s.conv < 1 || s.conv > 64 || s.norm_groups < 1 || (s.heads * s.vdim) % s.norm_groups != 0)
          return fail("bad state-space sizes" + at);
      } else if (s.mixer == TGIS_MIXER_CHANNEL_DELTA) {
        if (s.heads < 1 || s.kv_heads < 1 || s.heads % s.kv_heads != 0 || s.dim < 1 || s.dim > DELTA_SCAN_MAX_DIM || s.vdim < 1 ||
            s.conv < 1 || s.conv > 64 || s.decay_rank < 1 || s.gate_rank < 1)
          return fail("bad delta-rule sizes" + at);
      } else {
        return fail("unknown mixer type" + at);
      }
      continue;
    }
    if (post != (s.mixer != TGIS_MIXER_LATENT_ATTENTION)) return fail("this mixer does not run in this norm style" + at);
    if (post) {
      if (s.mlp != TGIS_MLP_NONE && s.mlp != TGIS_MLP_DENSE_GELU) return fail("unknown feed-forward kind" + at);
      if (s.mlp == TGIS_MLP_DENSE_GELU && s.ff < 1) return fail("bad feed-forward width" + at);
      if (s.mixer == TGIS_MIXER_PARALLEL) {
        if (s.heads < 1 || s.kv_heads < 1 || s.heads % s.kv_heads != 0 || s.dim < 1 || s.vdim < 1 || s.vdim > CAPATTN_MAX_VDIM ||
            s.dim > 512)
          return fail("bad attention sizes" + at);
        if (s.mm_heads < 1 || s.mm_dim < 1 || s.mm_dim > OUTER_SCAN_MAX_DIM || s.mm_vdim < 1 || !(s.gate_cap > 0.f))
          return fail("bad matrix-memory sizes" + at);
      } else if (s.mixer == TGIS_MIXER_SELECTIVE_SCAN) {
        if (s.inner < 1 || s.state < 1 || s.state > SELSCAN_MAX_STATE || s.dt_rank < 1 || s.conv < 1 || s.conv > 64)
          return fail("bad selective-scan sizes" + at);
      } else if (s.mixer == TGIS_MIXER_WKV) {
        if (s.heads < 1 || s.dim < 1 || s.dim > OUTER_SCAN_MAX_DIM || s.decay_rank < 1) return fail("bad wkv sizes" + at);
      } else {
        return fail("unknown mixer type" + at);
      }
      continue;
    }
    if (s.heads < 1 || s.dim < 1 || s.rot_dim < 0 || s.vdim < 1 || s.kv_rank < 1 || s.q_rank < 1) return fail("bad mixer sizes" + at);
    if (s.kv_rank > 512) return fail("kv_rank > 512 unsupported" + at);
    if (s.rot_dims < 0 || s.rot_dims > s.rot_dim || (s.rot_dims & 1)) return fail("rot.dims must be even and <= rot_dim" + at);
    if (s.mlp != TGIS_MLP_NONE && s.mlp != TGIS_MLP_MOE) return fail("unknown feed-forward kind" + at);
    if (s.mlp == TGIS_MLP_MOE && (s.experts < 1 || s.top < 1 || s.top > s.experts || s.top > 32 || s.expert_ff < 1 ||
                                  s.shared_ff < 0 || s.experts > 2048))
      return fail("bad mixture-of-experts sizes" + at);
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail("no CUDA device: the TGIS engine has no CPU fallback");
  auto* e = new tgis_engine();
  e->cfg = *cfg;
  e->cfg.n_layers = spec->n_layers;
  e->cfg.n_q_heads = e->cfg.n_kv_heads = 1;  // (unused by this architecture; kept sane for the shared set-up code)
  e->cfg.head_dim = HEAD_DIM;
  e->cfg.ffn = 64;
  e->cfg.tp_size = 1;
  e->cfg.tp_rank = 0;
  e->pnx_spec = *spec;
  e->pnx_layer_specs.assign(spec->layers, spec->layers + spec->n_layers);
  e->pnx_spec.layers = nullptr;
  try {
    e->init();
  } catch (const std::exception& ex) {
    std::string m = ex.what();
    delete e;
    return fail(m);
  }
  *out = e;
  return 0;
}

int tgis_engine_load_weight(tgis_engine* e, const char* name, const void* ptr, int64_t rows, int64_t cols, int32_t dtype) {
  if (!e || !name || !ptr) return fail("null argument");
  if (dtype != 0) return fail("only bf16 (dtype 0) weights are supported");
  if (e->started) return fail("engine already started");
  return e->load_weight(name, ptr, rows, cols);
}

int tgis_engine_start(tgis_engine* e) {
  if (!e) return fail("null engine");
  if (e->started) return 0;
  try {
    e->finalize_weights();
  } catch (const std::exception& ex) {
    return fail(ex.what());
  }
  e->started = true;
  e->th = std::thread([e] { e->loop(); });
  return 0;
}

static int engine_prepare_sync(tgis_engine* e) {
  if (e->th.joinable()) return fail("run_until_idle cannot be mixed with the engine thread");
  if (!e->started) {
    try {
      e->finalize_weights();
    } catch (const std::exception& ex) {
      return fail(ex.what());
    }
    e->started = true;
  }
  return 0;
}

int tgis_engine_run_until_idle(tgis_engine* e) {
  if (!e) return fail("null engine");
  if (engine_prepare_sync(e) != 0) return -1;
  int steps = 0;
  try {
    while (e->step()) ++steps;
  } catch (const std::exception& ex) {
    e->fail_all(ex.what());
    return fail(ex.what());
  }
  return steps;
}

int tgis_engine_trace_step(tgis_engine* e, const tgis_trace_entry* entries, int32_t n_entries, const char* const* end_ids,
                           int32_t n_end, float* logits_out) {
  if (!e || (n_entries > 0 && !entries) || (n_end > 0 && !end_ids) || n_entries < 0 || n_end < 0) return fail("bad argument");
  if (engine_prepare_sync(e) != 0) return -1;
  try {
    return e->trace_step(entries, n_entries, end_ids, n_end, logits_out);
  } catch (const std::exception& ex) {
    e->fail_all(ex.what());
    return fail(ex.what());
  }
}

int tgis_engine_add_request(tgis_engine* e, const char* request_id, const int32_t* prompt_ids, int32_t n_prompt,
                            const tgis_sampling_params* params) {
  if (!e || !request_id || !prompt_ids || !params) return fail("null argument");
  if (e->errored) return fail("engine errored: " + e->error_msg);
  if (n_prompt < 1) return fail("empty prompt");
  if (n_prompt >= e->cfg.max_model_len) return fail("prompt longer than max_model_len");
  if (strlen(request_id) >= TGIS_MAX_REQUEST_ID) return fail("request id too long");
  if (params->max_tokens < 1) return fail("max_tokens must be >= 1");
  // vllm sampling_params.py _verify_args: min_tokens <= max_tokens; validation.py:64-77: prompt + min_tokens must fit
  if (params->min_tokens < 0) return fail("min_tokens must be >= 0");
  if (params->min_tokens > params->max_tokens) return fail("min_tokens must be less than or equal to max_tokens");
  if ((long long)n_prompt + params->min_tokens > e->cfg.max_model_len)
    return fail("prompt length + min_tokens exceeds max_model_len");
  if (params->n_stop_token_ids > TGIS_MAX_STOP_TOKEN_IDS || params->n_stop_token_ids < 0) return fail("too many stop token ids");
  if (!params->greedy && !(params->temperature > 0.f)) return fail("temperature must be > 0 when sampling");
  if (params->num_logprobs > TGIS_MAX_TOPN || params->prompt_logprobs > TGIS_MAX_TOPN) return fail("num_logprobs too large");
  for (int i = 0; i < n_prompt; ++i)
    if (prompt_ids[i] < 0 || prompt_ids[i] >= e->cfg.vocab) return fail("prompt token id out of range");
  if (params->lora_slot < 0 || params->lora_slot > e->max_loras)
    return fail("lora_slot out of range (the engine was created with max_loras = " + std::to_string(e->max_loras) + ")");
  if (params->guided) {
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->mask_fn == nullptr) return fail("guided decoding requested but no mask provider is installed");
  }
  auto r = std::make_unique<Request>();
  r->id = request_id;
  r->tokens.assign(prompt_ids, prompt_ids + n_prompt);
  r->n_prompt = n_prompt;
  r->sp = *params;
  r->ts_arrival = now_s();
  {
    std::lock_guard<std::mutex> lk(e->mu);
    r->seed = params->has_seed ? params->seed : e->rng();
    e->incoming.push_back(std::move(r));
  }
  e->cv_in.notify_all();
  return 0;
}

int tgis_engine_abort(tgis_engine* e, const char* request_id) {
  if (!e || !request_id) return fail("null argument");
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->abort_ids.emplace_back(request_id);
  }
  e->cv_in.notify_all();
  return 0;
}

int tgis_engine_load_adapter_weight(tgis_engine* e, int32_t slot, const char* name, const void* ptr, int64_t rows,
                                    int64_t cols) {
  if (!e || !name || !ptr) return fail("null argument");
  try {
    return e->load_adapter_weight(slot, name, ptr, rows, cols);
  } catch (const std::exception& ex) {
    return fail(ex.what());
  }
}

int tgis_engine_clear_adapter(tgis_engine* e, int32_t slot) {
  if (!e) return fail("null argument");
  try {
    return e->clear_adapter(slot);
  } catch (const std::exception& ex) {
    return fail(ex.what());
  }
}

int tgis_engine_set_mask_provider(tgis_engine* e, tgis_mask_fn fn, void* user) {
  if (!e) return fail("null argument");
  std::lock_guard<std::mutex> lk(e->mu);
  e->mask_fn = fn;
  e->mask_user = user;
  return 0;
}

int tgis_engine_poll(tgis_engine* e, tgis_step_output* out, int32_t cap, int32_t timeout_ms) {
  if (!e || !out || cap <= 0) return fail("bad argument");
  std::unique_lock<std::mutex> lk(e->mu);
  if (e->outputs.empty() && timeout_ms > 0)
    e->cv_out.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !e->outputs.empty() || e->stop_flag.load(); });
  int n = 0;
  while (n < cap && !e->outputs.empty()) {
    out[n++] = e->outputs.front();
    e->outputs.pop_front();
  }
  return n;
}

int tgis_engine_status(tgis_engine* e, tgis_status* out) {
  if (!e || !out) return fail("null argument");
  memset(out, 0, sizeof(*out));
  std::lock_guard<std::mutex> lk(e->mu);
  out->errored = e->errored ? 1 : 0;
  out->is_running = (e->thread_alive || (e->started && !e->th.joinable() && !e->errored)) ? 1 : 0;
  out->n_running = e->snap_running;
  out->n_waiting = e->snap_waiting + (int)e->incoming.size();
  out->free_blocks = e->snap_free_blocks;
  out->total_blocks = e->num_blocks;
  out->steps = e->n_steps;
  out->tokens_generated = e->n_tokens;
  out->kernel_launches = e->n_launches;
  out->gpu_busy_ms = e->gpu_ms;
  out->gpu_decode_ms = e->gpu_ms_decode;
  out->gpu_mixed_ms = e->gpu_ms_mixed;
  out->decode_steps = e->decode_steps;
  out->decode_tokens = e->decode_tokens;
  out->h2d_bytes = e->h2d_bytes;
  out->d2h_bytes = e->d2h_bytes;
  out->gemm_ms = e->gemm_ms;
  out->gemm_bytes = e->gemm_bytes;
  out->gemm_calls = e->gemm_calls;
  out->graph_launches = e->n_graph_launches;
  out->exchange_ms = e->exchange_ms;
  out->exchange_calls = e->exchange_calls;
  out->preemptions = e->n_preempt;
  if (e->errored) g_last_error = e->error_msg;
  return 0;
}

int tgis_nccl_unique_id(uint8_t out[128]) {
  ncclUniqueId id;
  try {
    if (nccl().GetUniqueId(&id) != ncclSuccess) return fail("ncclGetUniqueId failed");
  } catch (const std::exception& ex) {
    return fail(ex.what());
  }
  memcpy(out, id.internal, 128);
  return 0;
}

int tgis_engine_worker_run(tgis_engine* e) {
  if (!e) return fail("null engine");
  if (e->tp <= 1 || e->rank == 0) return fail("worker_run is for tensor-parallel ranks > 0");
  try {
    e->finalize_weights();
    e->started = true;
    return e->worker_loop();
  } catch (const std::exception& ex) {
    e->error_msg = ex.what();
    e->errored = true;
    return fail(ex.what());
  }
}

int tgis_engine_set_profiling(tgis_engine* e, int32_t on) {
  if (!e) return fail("null engine");
  e->profiling = on != 0;
  e->prof_decode_only = on == 2;  // 2: time only the GEMMs of pure-decode steps (the HBM-bound regime)
  return 0;
}

int tgis_engine_max_model_len(tgis_engine* e) { return e ? e->cfg.max_model_len : fail("null engine"); }

int tgis_engine_shutdown(tgis_engine* e) {
  if (!e) return fail("null engine");
  e->stop_flag = true;
  if (e->shm && e->rank == 0) e->shm->shutdown.store(1, std::memory_order_release);
  e->cv_in.notify_all();
  if (e->th.joinable()) e->th.join();
  e->cv_out.notify_all();
  return 0;
}

void tgis_engine_destroy(tgis_engine* e) {
  if (!e) return;
  tgis_engine_shutdown(e);
  cudaSetDevice(e->cfg.device);
  delete e;
}

}  // extern "C"
