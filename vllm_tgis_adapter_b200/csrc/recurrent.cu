// Mixers that carry a state from token to token: the token shift and decayed outer-product memory of RWKV-style time
// mixing, the gated matrix memory of xLSTM (mLSTM), the short convolution and selective scan of Mamba, and the per-head
// norm + gate that follows the two memories.
//
// State lives in fp32, one slot per sequence and layer (the engine's sequence slot).  A kernel reads the slot's state
// for the first token of a portion unless that token sits at position 0 -- then the state is zero, so a slot needs no
// clearing when it passes to another sequence --, walks the portion's tokens in ascending order and leaves the state
// behind the last one.  The arithmetic of a token therefore depends on the tokens before it only, never on how the
// sequence was cut into steps, on the other sequences of the batch or on the slot.  Everything that enters a recurrence
// (decays, gates, step sizes, normalisers) is evaluated in fp32 with expf / tanhf / log1pf, no fast-math forms.
//
// The scans are sequential over tokens and parallel over what is independent: channels (selective scan), heads and
// value columns (outer-product memories).  A state update is done by the thread that owns the entry, in the launch that
// is the LAST reader of the old state in its layer, so no launch reads a state another CTA of the same launch rewrites.
#include <cstdint>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

__device__ __forceinline__ void st_op(void* out, int dt, size_t i, float v) {
  if (dt == DT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[i] = v;
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoid_f(float z) { return z >= 0.f ? -log1pf(expf(-z)) : z - log1pf(expf(z)); }
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------------ token shift
__global__ void __launch_bounds__(128)
token_shift_mix_kernel(const float* __restrict__ x, int width, const float* __restrict__ mu, int n_mix,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ tok_slot,
                       const float* __restrict__ prev_state, void* __restrict__ out, int out_dtype, long long out_bs) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const int slot = tok_slot[t];
  const float* prev = nullptr;   // nullptr: zeros
  if (positions[t] > 0) prev = (t > 0 && tok_slot[t - 1] == slot) ? x + (size_t)(t - 1) * width : prev_state + (size_t)slot * width;
  const float* xr = x + (size_t)t * width;
  for (int i = threadIdx.x; i < width; i += 128) {
    const float h = xr[i], d = (prev ? prev[i] : 0.f) - h;
    for (int s = 0; s < n_mix; ++s) st_op(out, out_dtype, (size_t)s * out_bs + (size_t)t * width + i, fmaf(d, mu[(size_t)s * width + i], h));
  }
}

// ------------------------------------------------------------------------------------------------ short convolution
// VEC channels per thread (VEC = 4: 16-byte loads and stores; needs ld, inner and every base pointer aligned to four floats)
template <int VEC>
__global__ void __launch_bounds__(128)
short_conv_silu_kernel(const float* __restrict__ xz, int ld, int inner, const float* __restrict__ w,
                       const float* __restrict__ b, int taps, const int32_t* __restrict__ positions,
                       const int32_t* __restrict__ tok_slot, const float* __restrict__ conv_state,
                       float* __restrict__ out_f32, void* __restrict__ out_op, int out_dtype) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, c = (blockIdx.y * 128 + threadIdx.x) * VEC;
  if (c >= inner) return;
  const int slot = tok_slot[t], p = positions[t];
  int nb = 0;  // predecessors of this token inside the batch (as far as the taps reach)
  while (nb < taps - 1 && t - nb - 1 >= 0 && tok_slot[t - nb - 1] == slot) ++nb;
  float acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = b != nullptr ? b[c + e] : 0.f;
  for (int j = taps - 1; j >= 0; --j) {   // oldest input first
    if (p - j < 0) continue;
    const float* src = j <= nb ? xz + (size_t)(t - j) * ld + c
                               : conv_state + ((size_t)slot * (taps - 1) + (taps - 1 - j + nb)) * inner + c;
    float v[VEC];
    if (VEC == 4) {
      const float4 q = *reinterpret_cast<const float4*>(src);
      v[0] = q.x; v[1 % VEC] = q.y; v[2 % VEC] = q.z; v[3 % VEC] = q.w;
    } else {
      v[0] = *src;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = fmaf(w[(size_t)(c + e) * taps + (taps - 1 - j)], v[e], acc[e]);
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = silu_f(acc[e]);
  if (out_f32) {
    if (VEC == 4) *reinterpret_cast<float4*>(out_f32 + (size_t)t * inner + c) = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
    else out_f32[(size_t)t * inner + c] = acc[0];
  }
  if (out_op) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) st_op(out_op, out_dtype, (size_t)t * inner + c + e, acc[e]);
  }
}

// ------------------------------------------------------------------------------------------------ selective scan
constexpr int SCAN_THREADS = 64, SCAN_CHUNK = 8, SCAN_REG_STATE = 16, SCAN_LPC = 4, SCAN_RPL = SCAN_REG_STATE / SCAN_LPC;
// REG (state <= SCAN_REG_STATE): SCAN_LPC lanes share a channel, lane `sub` keeps states sub, sub + 4, ... and their decay rates in
// registers and the lanes' partial outputs meet through two shuffles; otherwise one thread per channel, state in shared memory.
// A chunk's B / C rows are staged in shared memory and its per-channel scalars (step size, input, gate) are fetched ahead
// of the chunk's arithmetic, so the token loop waits for memory once per chunk, not once per token.
template <bool REG>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(SelScan a, const AttnSeq* __restrict__ seqs, const int32_t* __restrict__ tok_slot) {
  extern __shared__ float scan_smem[];
  const int N = a.state;
  float* BC = scan_smem;                                         // [SCAN_CHUNK][2 N]
  float* Ss = BC + (size_t)SCAN_CHUNK * 2 * N;                   // !REG: [N][SCAN_THREADS]
  float* As = Ss + (REG ? 0 : (size_t)N * SCAN_THREADS);         // !REG: [N][SCAN_THREADS]
  griddep_launch();
  griddep_wait();
  const AttnSeq sq = seqs[blockIdx.x];
  const int tid = threadIdx.x;
  const int sub = REG ? tid % SCAN_LPC : 0;
  const int c = REG ? blockIdx.y * (SCAN_THREADS / SCAN_LPC) + tid / SCAN_LPC : blockIdx.y * SCAN_THREADS + tid;
  const bool live = c < a.inner;
  const int slot = tok_slot[sq.q_start];
  const int first = sq.kv_len - sq.q_len;   // position of the portion's first token
  float* Sg = a.S + ((size_t)slot * a.inner + (live ? c : 0)) * N;
  float Sr[SCAN_RPL], Ar[SCAN_RPL];
  if (REG) {
#pragma unroll
    for (int j = 0; j < SCAN_RPL; ++j) {
      const int n = sub + j * SCAN_LPC;
      Sr[j] = (live && first > 0 && n < N) ? Sg[n] : 0.f;
      Ar[j] = (live && n < N) ? -expf(a.A_log[(size_t)c * N + n]) : 0.f;
    }
  } else {
    for (int n = 0; n < N; ++n) {
      Ss[n * SCAN_THREADS + tid] = (live && first > 0) ? Sg[n] : 0.f;
      As[n * SCAN_THREADS + tid] = live ? -expf(a.A_log[(size_t)c * N + n]) : 0.f;
    }
  }
  const float dtb = live ? a.dt_b[c] : 0.f, Dc = live ? a.D[c] : 0.f;
  for (int t0 = 0; t0 < sq.q_len; t0 += SCAN_CHUNK) {
    const int nt = min(SCAN_CHUNK, sq.q_len - t0);
    __syncthreads();
    for (int i = tid; i < nt * 2 * N; i += SCAN_THREADS) {
      const int tt = i / (2 * N), j = i % (2 * N);
      BC[i] = a.proj[(size_t)(sq.q_start + t0 + tt) * a.ld_proj + a.dt_rank + j];
    }
    float dtv[SCAN_CHUNK], xv[SCAN_CHUNK], zv[SCAN_CHUNK];
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
      const size_t row = (size_t)(sq.q_start + t0 + tt);
      const bool ok = live && tt < nt;
      dtv[tt] = ok ? a.dt_raw[row * a.inner + c] : 0.f;
      xv[tt] = ok ? a.x[row * a.inner + c] : 0.f;
      zv[tt] = ok ? a.xz[row * a.ld_xz + a.inner + c] : 0.f;
    }
    __syncthreads();
    if (!REG && !live) continue;   // (REG: every lane takes part in the shuffles)
#pragma unroll
    for (int tt = 0; tt < SCAN_CHUNK; ++tt) {
      if (tt < nt) {
        const size_t row = (size_t)(sq.q_start + t0 + tt);
        const float dt = softplus_f(dtv[tt] + dtb);
        const float dx = dt * xv[tt];
        const float* Bt = BC + (size_t)tt * 2 * N;
        float y = 0.f;
        if (REG) {
#pragma unroll
          for (int j = 0; j < SCAN_RPL; ++j) {
            const int n = sub + j * SCAN_LPC;
            if (n < N) {
              Sr[j] = fmaf(expf(dt * Ar[j]), Sr[j], dx * Bt[n]);
              y = fmaf(Sr[j], Bt[N + n], y);
            }
          }
          y += __shfl_xor_sync(0xffffffffu, y, 1);
          y += __shfl_xor_sync(0xffffffffu, y, 2);
          if (!live || sub != 0) continue;
        } else {
          for (int n = 0; n < N; ++n) {
            const float sv = fmaf(expf(dt * As[n * SCAN_THREADS + tid]), Ss[n * SCAN_THREADS + tid], dx * Bt[n]);
            Ss[n * SCAN_THREADS + tid] = sv;
            y = fmaf(sv, Bt[N + n], y);
          }
        }
        y = fmaf(Dc, xv[tt], y);
        st_op(a.out, a.out_dtype, row * a.inner + c, y * silu_f(zv[tt]));
      }
    }
  }
  if (!live) return;
  if (REG) {
#pragma unroll
    for (int j = 0; j < SCAN_RPL; ++j)
      if (sub + j * SCAN_LPC < N) Sg[sub + j * SCAN_LPC] = Sr[j];
    if (sub != 0) return;
  } else {
    for (int n = 0; n < N; ++n) Sg[n] = Ss[n * SCAN_THREADS + tid];
  }
  // the convolution's tail: inputs of the last taps - 1 positions (entry e: position end - (taps - 1) + e)
  const int K1 = a.taps - 1;
  float* cs = a.conv_state + (size_t)slot * K1 * a.inner + c;
  for (int e = 0; e < K1; ++e) {   // ascending: entry e + q_len is read before it could be rewritten
    const int pp = sq.kv_len - K1 + e;
    float v = 0.f;
    if (pp >= first) v = a.xz[(size_t)(sq.q_start + pp - first) * a.ld_xz + c];
    else if (pp >= 0) v = cs[(size_t)(e + sq.q_len) * a.inner];
    cs[(size_t)e * a.inner] = v;
  }
}

// ------------------------------------------------------------------------------------------------ outer-product memories
// grid (sequences, heads, ceil(vdim / 32)); 256 threads = 8 row groups (warps) x 32 value columns (lanes).  Thread (g, c)
// keeps rows g, g + 8, ... of column c in registers.  The tokens' q / k / decay vectors, value columns and gates are staged
// in shared memory OS_CHUNK tokens at a time (one wait for memory per chunk).  The recurrence itself is private to a thread (its
// rows of S, and redundantly the running maximum and its rows of n); only a token's OUTPUT sums over the row groups.  So a thread
// runs through the chunk's tokens without any barrier, leaving its partial sums per token in shared memory, and after ONE barrier
// warp w sums and writes the outputs of the chunk's token w.
constexpr int OS_GROUPS = 8, OS_COLS = 32, OS_THREADS = OS_GROUPS * OS_COLS, OS_CHUNK = 16;
template <int RPT, int MODE>
__global__ void __launch_bounds__(OS_THREADS)
outer_scan_kernel(OuterScan a, const AttnSeq* __restrict__ seqs, const int32_t* __restrict__ tok_slot) {
  extern __shared__ float os_smem[];
  const int D = a.dim;
  float* vec = os_smem;                                  // [OS_CHUNK][3][D]: q | k | w
  float* vcol = vec + (size_t)OS_CHUNK * 3 * D;          // [OS_CHUNK][OS_COLS]
  __shared__ float part[OS_CHUNK][OS_GROUPS][OS_COLS + 1];
  __shared__ float part_n[OS_CHUNK][OS_GROUPS];
  __shared__ float gates[OS_CHUNK][2];                   // GATED: capped log input gate, log forget gate
  __shared__ float floor_m[OS_CHUNK];                    // GATED: e^(-m) after each token
  static_assert(OS_CHUNK % OS_GROUPS == 0, "warp w writes the outputs of the chunk's tokens w, w + OS_GROUPS, ...");
  griddep_launch();
  griddep_wait();
  const AttnSeq sq = seqs[blockIdx.x];
  const int h = blockIdx.y, tid = threadIdx.x, g = tid >> 5, lane = tid & 31;
  const int hq = a.qk_heads > 0 ? h / (a.heads / a.qk_heads) : h;   // the q / k head this head reads
  const int c0 = blockIdx.z * OS_COLS, c = c0 + lane;
  const bool col_ok = c < a.vdim;
  const int slot = tok_slot[sq.q_start];
  const bool fresh = sq.kv_len - sq.q_len == 0;
  float S[RPT];
  float* Sg = a.S + (((size_t)slot * a.heads + h) * D) * a.vdim + (col_ok ? c : 0);
#pragma unroll
  for (int j = 0; j < RPT; ++j) {
    const int i = g + j * OS_GROUPS;
    S[j] = (!fresh && col_ok && i < D) ? Sg[(size_t)i * a.vdim] : 0.f;
  }
  float u_r[RPT];   // DECAY: the bonus u of this thread's rows; GATED: the normaliser n of its rows (the same in every lane)
  float m_run = 0.f;
  const float ssd_rate = MODE == OUTER_SCAN_SSD ? -expf(a.A_log[h]) : 0.f, ssd_skip = MODE == OUTER_SCAN_SSD ? a.D[h] : 0.f;
  if (MODE == OUTER_SCAN_SSD || MODE == OUTER_SCAN_HGRN) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) u_r[j] = 0.f;
  } else if (MODE == OUTER_SCAN_DECAY) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int i = g + j * OS_GROUPS;
      u_r[j] = i < D ? a.u[(size_t)h * D + i] : 0.f;
    }
  } else {
    const float* ng = a.n + ((size_t)slot * a.heads + h) * D;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int i = g + j * OS_GROUPS;
      u_r[j] = (!fresh && i < D) ? ng[i] : 0.f;
    }
    m_run = fresh ? 0.f : a.m[(size_t)slot * a.heads + h];
  }
  // A chunk's raw values travel global memory -> registers -> shared memory: thread (tt = tid / 16, l = tid % 16) stages entries
  // l, l + 16, ... of token tt's vectors and two of its value columns, all loads of a chunk are issued back to back, and the
  // loads of chunk n + 1 are issued before the token loop of chunk n.
  constexpr int EPT = RPT / 2, TPT = OS_THREADS / OS_CHUNK;
  static_assert(TPT == 16 && OS_CHUNK * OS_COLS == 2 * OS_THREADS, "staging map");
  const int st_tt = tid / TPT, st_l = tid % TPT;
  float pq[EPT], pk[EPT], pd[EPT], pv[2], pg0 = 0.f, pg1 = 0.f;
  auto fetch = [&](int t0) {
    const int nt = min(OS_CHUNK, sq.q_len - t0);
    const bool tok = st_tt < nt;
    const size_t row = (size_t)(sq.q_start + t0 + (tok ? st_tt : 0));
    const float* qr = a.q + row * a.ldq + (size_t)hq * D;
    const float* kr = MODE == OUTER_SCAN_HGRN ? nullptr : a.k + row * a.ldk + (size_t)hq * D;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int i = st_l + e * TPT;
      const bool in = tok && i < D;
      pq[e] = in ? qr[i] : 0.f;
      pk[e] = in ? (MODE == OUTER_SCAN_HGRN ? a.u[(size_t)h * D + i] : kr[i]) : 0.f;   // HGRN: the gate's lower bound
      if (MODE == OUTER_SCAN_DECAY || MODE == OUTER_SCAN_HGRN)
        pd[e] = in ? a.decay_raw[row * a.ldd + (size_t)h * D + i] + a.w0[(size_t)h * D + i] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = c0 + 2 * st_l + e;
      pv[e] = (tok && col < a.vdim) ? a.v[row * a.ldv + (size_t)h * a.vdim + col] : 0.f;
    }
    if (tid < nt) {
      const size_t grow = (size_t)(sq.q_start + t0 + tid);
      if (MODE == OUTER_SCAN_GATED) { pg0 = a.ig[grow * a.ldg + h]; pg1 = a.fg[grow * a.ldg + h]; }
      if (MODE == OUTER_SCAN_SSD) pg0 = a.step_raw[grow * a.lds + h];
    }
  };
  fetch(0);
  for (int t0 = 0; t0 < sq.q_len; t0 += OS_CHUNK) {
    const int nt = min(OS_CHUNK, sq.q_len - t0);
    __syncthreads();   // the previous chunk's vectors and partial sums are consumed
    if (st_tt < nt) {
      float* v3 = vec + (size_t)st_tt * 3 * D;
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int i = st_l + e * TPT;
        if (i < D) {
          if (MODE == OUTER_SCAN_HGRN) {   // q = silu(.), f = l + (1 - l) sigmoid(.), and what is written: 1 - f
            v3[i] = silu_f(pq[e]) * a.q_scale;
            v3[D + i] = (1.f - pk[e]) * sigmoid_f(-pd[e]);                 // 1 - f without the cancellation near f = 1
            v3[2 * D + i] = pk[e] + (1.f - pk[e]) * sigmoid_f(pd[e]);
          } else {
            v3[i] = pq[e] * a.q_scale;
            v3[D + i] = pk[e];
            if (MODE == OUTER_SCAN_DECAY) v3[2 * D + i] = expf(-expf(pd[e]));
          }
        }
      }
    }
    vcol[st_tt * OS_COLS + 2 * st_l] = pv[0];
    vcol[st_tt * OS_COLS + 2 * st_l + 1] = pv[1];
    if (MODE == OUTER_SCAN_GATED && tid < nt) {
      gates[tid][0] = a.gate_cap * tanhf((pg0 + a.ig_b[h]) / a.gate_cap);
      gates[tid][1] = logsigmoid_f(a.gate_cap * tanhf((pg1 + a.fg_b[h]) / a.gate_cap));
    }
    if (MODE == OUTER_SCAN_SSD && tid < nt) {   // the token's step size and the decay it gives
      const float dt = softplus_f(pg0 + a.step_b[h]);
      gates[tid][0] = expf(ssd_rate * dt);
      gates[tid][1] = dt;
    }
    __syncthreads();
    if (t0 + OS_CHUNK < sq.q_len) fetch(t0 + OS_CHUNK);   // lands while this chunk's tokens are worked through
    for (int tt = 0; tt < nt; ++tt) {
      const float* v3 = vec + (size_t)tt * 3 * D;
      const float vc = vcol[tt * OS_COLS + lane];
      float o = 0.f, nq = 0.f;
      if (MODE == OUTER_SCAN_DECAY) {
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int i = g + j * OS_GROUPS;
          if (i < D) {
            const float kv = v3[D + i] * vc;
            o = fmaf(v3[i], fmaf(u_r[j], kv, S[j]), o);
            S[j] = fmaf(v3[2 * D + i], S[j], kv);
          }
        }
      } else if (MODE == OUTER_SCAN_HGRN) {
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int i = g + j * OS_GROUPS;
          if (i < D) {
            S[j] = fmaf(v3[2 * D + i], S[j], v3[D + i] * vc);
            o = fmaf(v3[i], S[j], o);
          }
        }
      } else if (MODE == OUTER_SCAN_SSD) {
        const float da = gates[tt][0], dv = gates[tt][1] * vc;
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int i = g + j * OS_GROUPS;
          if (i < D) {
            S[j] = fmaf(da, S[j], v3[D + i] * dv);
            o = fmaf(v3[i], S[j], o);
          }
        }
      } else {
        const float ig = gates[tt][0], fg = gates[tt][1];
        const float m_new = fmaxf(fg + m_run, ig);
        const float da = expf(fg + m_run - m_new), db = expf(ig - m_new);
        m_run = m_new;
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int i = g + j * OS_GROUPS;
          if (i < D) {
            const float kk = v3[D + i], qq = v3[i];
            S[j] = fmaf(da, S[j], db * kk * vc);
            o = fmaf(qq, S[j], o);
            u_r[j] = fmaf(da, u_r[j], db * kk);
            nq = fmaf(u_r[j], qq, nq);
          }
        }
        if (lane == 0) part_n[tt][g] = nq;
        if (tid == 0) floor_m[tt] = expf(-m_run);
      }
      part[tt][g][lane] = o;
    }
    __syncthreads();   // the chunk's partial sums are complete
    for (int tt = g; tt < nt; tt += OS_GROUPS) {   // this warp's tokens of the chunk
      float sum = 0.f;
#pragma unroll
      for (int r = 0; r < OS_GROUPS; ++r) sum += part[tt][r][lane];
      if (MODE == OUTER_SCAN_GATED) {
        float d = 0.f;
#pragma unroll
        for (int r = 0; r < OS_GROUPS; ++r) d += part_n[tt][r];
        sum = sum / (fmaxf(fabsf(d), floor_m[tt]) + 1e-6f);
      }
      if (MODE == OUTER_SCAN_SSD) sum = fmaf(ssd_skip, vcol[tt * OS_COLS + lane], sum);
      if (col_ok) a.out[(size_t)(sq.q_start + t0 + tt) * a.ldo + (size_t)h * a.vdim + c] = sum;
    }
  }
  // ---- leave the state behind the portion's last token
  if (col_ok) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int i = g + j * OS_GROUPS;
      if (i < D) Sg[(size_t)i * a.vdim] = S[j];
    }
  }
  if (blockIdx.z == 0) {
    if (MODE == OUTER_SCAN_GATED) {
      float* ng = a.n + ((size_t)slot * a.heads + h) * D;
      if (lane == 0) {
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int i = g + j * OS_GROUPS;
          if (i < D) ng[i] = u_r[j];
        }
      }
      if (tid == 0) a.m[(size_t)slot * a.heads + h] = m_run;
    }
    if (a.x_last != nullptr && h == 0) {
      const float* src = a.x + (size_t)(sq.q_start + sq.q_len - 1) * a.width;
      for (int i = tid; i < a.width; i += OS_THREADS) a.x_last[(size_t)slot * a.width + i] = src[i];
    }
  }
}

// ------------------------------------------------------------------------------------------------ convolution state
// grid (sequences, ceil(n / 128)): one thread per channel moves the tail of its convolution forward
__global__ void __launch_bounds__(128)
conv_state_save_kernel(const float* __restrict__ x, int ld, int n, int taps, const AttnSeq* __restrict__ seqs,
                       const int32_t* __restrict__ tok_slot, float* __restrict__ conv_state) {
  griddep_launch();
  griddep_wait();
  const AttnSeq sq = seqs[blockIdx.x];
  const int c = blockIdx.y * 128 + threadIdx.x;
  if (c >= n) return;
  const int K1 = taps - 1, first = sq.kv_len - sq.q_len, slot = tok_slot[sq.q_start];
  float* cs = conv_state + (size_t)slot * K1 * n + c;
  for (int e = 0; e < K1; ++e) {   // ascending: entry e + q_len is read before it could be rewritten
    const int pp = sq.kv_len - K1 + e;
    float v = 0.f;
    if (pp >= first) v = x[(size_t)(sq.q_start + pp - first) * ld + c];
    else if (pp >= 0) v = cs[(size_t)(e + sq.q_len) * n];
    cs[(size_t)e * n] = v;
  }
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// grid (sequences, heads, ceil(vdim / 32)); 256 threads = 32 value columns x DS_LPC lanes.  A column of S is independent of
// the others (its write u_c needs only its own S[:, c] . k), so DS_LPC neighbouring lanes share one column, lane `sub` keeping
// rows 32 jj + 4 sub + (0..3) in registers; the two sums over the rows that a token needs -- (g S)[:, c] . k for the write and
// (g S)[:, c] . q for the read-out, which with the write becomes o_c = (g S)[:, c] . q + u_c (k . q) -- meet through one round of
// shuffles.  Normalised q / k, the decays and the per-token scalars are staged in shared memory DS_CHUNK tokens at a time (rows
// padded to a multiple of four with zeros, so a lane fetches its four rows of each vector with one 16-byte load); the token
// loop itself runs without a barrier.
constexpr int DS_LPC = 8, DS_COLS = 32, DS_THREADS = DS_LPC * DS_COLS, DS_CHUNK = 16;
template <int RPT>
__global__ void __launch_bounds__(DS_THREADS)
delta_scan_kernel(DeltaScan a, const AttnSeq* __restrict__ seqs, const int32_t* __restrict__ tok_slot) {
  extern __shared__ __align__(16) float ds_smem[];
  static_assert(RPT % 4 == 0, "a lane owns whole groups of four rows");
  const int D = a.dim, Dp = (D + 3) & ~3;
  float* vec = ds_smem;                                  // [DS_CHUNK][3][Dp]: q | k | decay
  float* vcol = vec + (size_t)DS_CHUNK * 3 * Dp;         // [DS_CHUNK][DS_COLS]
  __shared__ float beta_s[DS_CHUNK], kq_s[DS_CHUNK];
  griddep_launch();
  griddep_wait();
  const AttnSeq sq = seqs[blockIdx.x];
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane & (DS_LPC - 1);
  const int hq = h / (a.heads / a.qk_heads);
  const int cl = warp * (32 / DS_LPC) + lane / DS_LPC;   // column inside the CTA's 32
  const int c = blockIdx.z * DS_COLS + cl;
  const bool col_ok = c < a.vdim;
  const int slot = tok_slot[sq.q_start];
  const bool fresh = sq.kv_len - sq.q_len == 0;
  float S[RPT];
  float* Sg = a.S + (((size_t)slot * a.heads + h) * D) * a.vdim + (col_ok ? c : 0);
#pragma unroll
  for (int j = 0; j < RPT; ++j) {
    const int i = (j >> 2) * 32 + sub * 4 + (j & 3);
    S[j] = (!fresh && col_ok && i < D) ? Sg[(size_t)i * a.vdim] : 0.f;
  }
  const float rate = -expf(a.A_log[h]), q_mult = 1.f / sqrtf((float)D);
  // A chunk's raw values travel global memory -> registers -> shared memory: all loads of a chunk are issued back to back
  // (one round trip to memory, not one per element), and the loads of chunk n + 1 are issued before the token loop of chunk n.
  // thread (tt = tid / 16, l = tid % 16) stages entries l, l + 16, ... of token tt's vectors, and two of the chunk's values
  constexpr int EPT = RPT / 2;   // 8 RPT rows at most, 16 threads per token
  constexpr int TPT = DS_THREADS / DS_CHUNK;
  static_assert(TPT == 16 && DS_CHUNK * DS_COLS == 2 * DS_THREADS, "staging map");
  const int st_tt = tid / TPT, st_l = tid % TPT;
  float pq[EPT], pk[EPT], pd[EPT], pv[2], pb = 0.f;
  auto fetch = [&](int t0) {
    const int nt = min(DS_CHUNK, sq.q_len - t0);
    const bool tok = st_tt < nt;
    const size_t row = (size_t)(sq.q_start + t0 + (tok ? st_tt : 0));
    const float* qr = a.q + row * a.ldq + (size_t)hq * D;
    const float* kr_ = a.k + row * a.ldk + (size_t)hq * D;
    const float* dr = a.decay_raw + row * a.ldd + (size_t)h * D;
    const float* db = a.decay_b + (size_t)h * D;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
      const int i = st_l + e * TPT;
      const bool in = tok && i < D;
      pq[e] = in ? qr[i] : 0.f;
      pk[e] = in ? kr_[i] : 0.f;
      pd[e] = in ? dr[i] + db[i] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {   // value columns: token tt, columns 2 l + e
      const int col = blockIdx.z * DS_COLS + 2 * st_l + e;
      pv[e] = (tok && col < a.vdim) ? a.v[row * a.ldv + (size_t)h * a.vdim + col] : 0.f;
    }
    pb = tid < nt ? a.beta_raw[(size_t)(sq.q_start + t0 + tid) * a.ldb + h] : 0.f;
  };
  fetch(0);
  for (int t0 = 0; t0 < sq.q_len; t0 += DS_CHUNK) {
    const int nt = min(DS_CHUNK, sq.q_len - t0);
    __syncthreads();   // the previous chunk's vectors are consumed
    if (st_tt < nt) {
      float* v3 = vec + (size_t)st_tt * 3 * Dp;
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        const int i = st_l + e * TPT;
        if (i < Dp) {
          v3[i] = pq[e];
          v3[Dp + i] = pk[e];
          v3[2 * Dp + i] = i < D ? expf(rate * softplus_f(pd[e])) : 0.f;
        }
      }
    }
    vcol[st_tt * DS_COLS + 2 * st_l] = pv[0];
    vcol[st_tt * DS_COLS + 2 * st_l + 1] = pv[1];
    if (tid < nt) beta_s[tid] = sigmoid_f(pb);
    __syncthreads();
    if (t0 + DS_CHUNK < sq.q_len) fetch(t0 + DS_CHUNK);   // lands while this chunk's tokens are worked through
    for (int tt = warp; tt < nt; tt += DS_THREADS / 32) {   // unit vectors, and k . q of the unit vectors
      float* v3 = vec + (size_t)tt * 3 * Dp;
      float sq2 = 0.f, sk2 = 0.f, skq = 0.f;
      for (int i = lane; i < D; i += 32) {
        const float qv = v3[i], kv = v3[Dp + i];
        sq2 = fmaf(qv, qv, sq2); sk2 = fmaf(kv, kv, sk2); skq = fmaf(qv, kv, skq);
      }
      sq2 = warp_sum_f(sq2); sk2 = warp_sum_f(sk2); skq = warp_sum_f(skq);
      const float rq = q_mult / sqrtf(sq2 + 1e-6f), rk = 1.f / sqrtf(sk2 + 1e-6f);
      for (int i = lane; i < D; i += 32) { v3[i] *= rq; v3[Dp + i] *= rk; }
      if (lane == 0) kq_s[tt] = skq * rq * rk;
    }
    __syncthreads();
    const float* v3 = vec;
    for (int tt = 0; tt < nt; ++tt, v3 += 3 * Dp) {
      float kr[RPT];
      float sk = 0.f, sqv = 0.f;
#pragma unroll
      for (int jj = 0; jj < RPT / 4; ++jj) {
        const int i0 = jj * 32 + sub * 4;
        if (i0 < Dp) {
          const float4 q4 = *reinterpret_cast<const float4*>(v3 + i0);
          const float4 k4 = *reinterpret_cast<const float4*>(v3 + Dp + i0);
          const float4 g4 = *reinterpret_cast<const float4*>(v3 + 2 * Dp + i0);
          const float qa[4] = {q4.x, q4.y, q4.z, q4.w}, ka[4] = {k4.x, k4.y, k4.z, k4.w}, ga[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = jj * 4 + e;
            S[j] *= ga[e];
            sk = fmaf(S[j], ka[e], sk);
            sqv = fmaf(S[j], qa[e], sqv);
            kr[j] = ka[e];
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) kr[jj * 4 + e] = 0.f;
        }
      }
#pragma unroll
      for (int o = DS_LPC / 2; o > 0; o >>= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sqv += __shfl_xor_sync(0xffffffffu, sqv, o);
      }
      const float u = beta_s[tt] * (vcol[tt * DS_COLS + cl] - sk);
#pragma unroll
      for (int j = 0; j < RPT; ++j) S[j] = fmaf(kr[j], u, S[j]);
      if (sub == 0 && col_ok) a.out[(size_t)(sq.q_start + t0 + tt) * a.ldo + (size_t)h * a.vdim + c] = fmaf(u, kq_s[tt], sqv);
    }
  }
  if (col_ok) {
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int i = (j >> 2) * 32 + sub * 4 + (j & 3);
      if (i < D) Sg[(size_t)i * a.vdim] = S[j];
    }
  }
}

// ------------------------------------------------------------------------------------------------ head norm + gate
// grid (T, ceil(heads / 4)), 128 threads: one warp per (token, head)
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int ldo, int heads, int vdim, const float* __restrict__ w,
                      const float* __restrict__ gate, int ldg, int act, float eps, void* __restrict__ out, int out_dtype,
                      int out_ld, int gate_first) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, h = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (h >= heads) return;
  const float* orow = o + (size_t)t * ldo + (size_t)h * vdim;
  float ss = 0.f;
  if (gate_first) {   // the gated values are what is normed
    const float* grow = gate + (size_t)t * ldg + (size_t)h * vdim;
    for (int i = lane; i < vdim; i += 32) {
      const float v = orow[i] * (act == 1 ? silu_f(grow[i]) : sigmoid_f(grow[i]));
      ss = fmaf(v, v, ss);
    }
    const float rs = 1.f / sqrtf(warp_sum_f(ss) / (float)vdim + eps);
    for (int i = lane; i < vdim; i += 32) {
      const float v = orow[i] * (act == 1 ? silu_f(grow[i]) : sigmoid_f(grow[i]));
      st_op(out, out_dtype, (size_t)t * out_ld + (size_t)h * vdim + i, v * rs * w[(size_t)h * vdim + i]);
    }
    return;
  }
  for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
  const float rs = 1.f / sqrtf(warp_sum_f(ss) / (float)vdim + eps);
  for (int i = lane; i < vdim; i += 32) {
    float gv = 1.f;
    if (act != 2) {
      const float gl = gate[(size_t)t * ldg + (size_t)h * vdim + i];
      gv = act == 1 ? silu_f(gl) : sigmoid_f(gl);
    }
    st_op(out, out_dtype, (size_t)t * out_ld + (size_t)h * vdim + i, orow[i] * rs * w[(size_t)h * vdim + i] * gv);
  }
}

// wide groups (a whole row normed as one or a few groups): grid (T, heads), 256 threads, one CTA per (token, group)
__global__ void __launch_bounds__(256)
head_norm_gate_wide_kernel(const float* __restrict__ o, int ldo, int heads, int vdim, const float* __restrict__ w,
                           const float* __restrict__ gate, int ldg, int act, float eps, void* __restrict__ out, int out_dtype,
                           int out_ld, int gate_first) {
  __shared__ float red[8];
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const float* orow = o + (size_t)t * ldo + (size_t)h * vdim;
  const float* grow = gate + (size_t)t * ldg + (size_t)h * vdim;
  float ss = 0.f;
  for (int i = tid; i < vdim; i += 256) {
    float v = orow[i];
    if (gate_first && act != 2) v *= act == 1 ? silu_f(grow[i]) : sigmoid_f(grow[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum_f(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int r = 0; r < 8; ++r) tot += red[r];   // the same order in every thread
  const float rs = 1.f / sqrtf(tot / (float)vdim + eps);
  for (int i = tid; i < vdim; i += 256) {
    const float gv = act == 2 ? 1.f : act == 1 ? silu_f(grow[i]) : sigmoid_f(grow[i]);
    st_op(out, out_dtype, (size_t)t * out_ld + (size_t)h * vdim + i, orow[i] * gv * rs * w[(size_t)h * vdim + i]);
  }
}

__global__ void convert_f32_kernel(const float* __restrict__ x, void* __restrict__ out, int out_dtype, size_t n) {
  griddep_launch();
  griddep_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    st_op(out, out_dtype, i, x[i]);
}

}  // namespace

cudaError_t token_shift_mix_launch(const float* x, int width, const float* mu, int n_mix, const int32_t* positions,
                                   const int32_t* tok_slot, const float* prev_state, void* out, int out_dtype,
                                   long long out_bs, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  return launch_k(token_shift_mix_kernel, dim3(T), dim3(128), 0, stream, x, width, mu, n_mix, positions, tok_slot, prev_state,
                  out, out_dtype, out_bs);
}

cudaError_t short_conv_silu_launch(const float* xz, int ld, int inner, const float* w, const float* b, int taps,
                                   const int32_t* positions, const int32_t* tok_slot, const float* conv_state,
                                   float* out_f32, void* out_op, int out_dtype, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (taps < 1) return cudaErrorInvalidValue;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (ld % 4 == 0 && inner % 4 == 0 && al16(xz) && al16(conv_state) && al16(out_f32))
    return launch_k(short_conv_silu_kernel<4>, dim3(T, (inner / 4 + 127) / 128), dim3(128), 0, stream, xz, ld, inner, w, b, taps,
                    positions, tok_slot, conv_state, out_f32, out_op, out_dtype);
  return launch_k(short_conv_silu_kernel<1>, dim3(T, (inner + 127) / 128), dim3(128), 0, stream, xz, ld, inner, w, b, taps,
                  positions, tok_slot, conv_state, out_f32, out_op, out_dtype);
}

cudaError_t selective_scan_launch(const SelScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                                  cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  if (a.state < 1 || a.state > SELSCAN_MAX_STATE || a.taps < 1) return cudaErrorInvalidValue;
  const size_t bc = (size_t)SCAN_CHUNK * 2 * a.state * sizeof(float);
  if (a.state <= SCAN_REG_STATE) {
    constexpr int per_cta = SCAN_THREADS / SCAN_LPC;
    return launch_k(selective_scan_kernel<true>, dim3(n_seqs, (a.inner + per_cta - 1) / per_cta), dim3(SCAN_THREADS), bc, stream, a,
                    seqs, tok_slot);
  }
  const dim3 grid(n_seqs, (a.inner + SCAN_THREADS - 1) / SCAN_THREADS);
  const size_t smem = bc + (size_t)2 * a.state * SCAN_THREADS * sizeof(float);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    const cudaError_t e = cudaFuncSetAttribute(selective_scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    smem_set = smem;
  }
  return launch_k(selective_scan_kernel<false>, grid, dim3(SCAN_THREADS), smem, stream, a, seqs, tok_slot);
}

template <int MODE>
static cudaError_t outer_scan_mode(const OuterScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                                   cudaStream_t stream) {
  const dim3 grid(n_seqs, a.heads, (a.vdim + OS_COLS - 1) / OS_COLS);
  const size_t smem = ((size_t)OS_CHUNK * 3 * a.dim + OS_CHUNK * OS_COLS) * sizeof(float);   // <= 50 KB (+ 18 KB static)
  if (a.dim <= 8 * OS_GROUPS) return launch_k(outer_scan_kernel<8, MODE>, grid, dim3(OS_THREADS), smem, stream, a, seqs, tok_slot);
  if (a.dim <= 16 * OS_GROUPS) return launch_k(outer_scan_kernel<16, MODE>, grid, dim3(OS_THREADS), smem, stream, a, seqs, tok_slot);
  static bool attr_set = false;   // keys of more than 128 entries: the staged chunk passes the default 48 KB of shared memory
  if (!attr_set) {
    const cudaError_t e = cudaFuncSetAttribute(outer_scan_kernel<32, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  return launch_k(outer_scan_kernel<32, MODE>, grid, dim3(OS_THREADS), smem, stream, a, seqs, tok_slot);
}
cudaError_t outer_scan_launch(const OuterScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                              cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  if (a.dim < 1 || a.dim > OUTER_SCAN_MAX_DIM || a.heads < 1 || a.heads > 65535 || a.vdim < 1) return cudaErrorInvalidValue;
  if (a.qk_heads > 0 && a.heads % a.qk_heads != 0) return cudaErrorInvalidValue;
  if (a.mode == OUTER_SCAN_SSD) {
    if (a.step_raw == nullptr || a.step_b == nullptr || a.A_log == nullptr || a.D == nullptr) return cudaErrorInvalidValue;
    return outer_scan_mode<OUTER_SCAN_SSD>(a, seqs, n_seqs, tok_slot, stream);
  }
  if (a.mode == OUTER_SCAN_HGRN) {
    if (a.decay_raw == nullptr || a.w0 == nullptr || a.u == nullptr) return cudaErrorInvalidValue;
    return outer_scan_mode<OUTER_SCAN_HGRN>(a, seqs, n_seqs, tok_slot, stream);
  }
  return a.mode == OUTER_SCAN_GATED ? outer_scan_mode<OUTER_SCAN_GATED>(a, seqs, n_seqs, tok_slot, stream)
                                    : outer_scan_mode<OUTER_SCAN_DECAY>(a, seqs, n_seqs, tok_slot, stream);
}

cudaError_t head_norm_gate_launch(const float* o, int ldo, int heads, int vdim, const float* w, const float* gate,
                                  int ldg, int act, float eps, void* out, int out_dtype, int T, cudaStream_t stream,
                                  int gate_first) {
  if (T <= 0) return cudaSuccess;
  if (act == 2) gate_first = 0;
  else if (gate == nullptr) return cudaErrorInvalidValue;
  if (vdim >= 1024 && heads <= 65535)
    return launch_k(head_norm_gate_wide_kernel, dim3(T, heads), dim3(256), 0, stream, o, ldo, heads, vdim, w, gate, ldg, act, eps, out,
                    out_dtype, heads * vdim, gate_first);
  return launch_k(head_norm_gate_kernel, dim3(T, (heads + 3) / 4), dim3(128), 0, stream, o, ldo, heads, vdim, w, gate, ldg, act,
                  eps, out, out_dtype, heads * vdim, gate_first);
}

cudaError_t conv_state_save_launch(const float* x, int ld, int n, int taps, const AttnSeq* seqs, int n_seqs,
                                   const int32_t* tok_slot, float* conv_state, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return cudaSuccess;
  return launch_k(conv_state_save_kernel, dim3(n_seqs, (n + 127) / 128), dim3(128), 0, stream, x, ld, n, taps, seqs, tok_slot,
                  conv_state);
}

template <int RPT>
static cudaError_t delta_scan_rpt(const DeltaScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot, cudaStream_t stream) {
  const dim3 grid(n_seqs, a.heads, (a.vdim + DS_COLS - 1) / DS_COLS);
  const size_t smem = ((size_t)DS_CHUNK * 3 * ((a.dim + 3) & ~3) + DS_CHUNK * DS_COLS) * sizeof(float);
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      const cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
  }
  return launch_k(delta_scan_kernel<RPT>, grid, dim3(DS_THREADS), smem, stream, a, seqs, tok_slot);
}
cudaError_t delta_scan_launch(const DeltaScan& a, const AttnSeq* seqs, int n_seqs, const int32_t* tok_slot,
                              cudaStream_t stream) {
  if (n_seqs <= 0) return cudaSuccess;
  if (a.dim < 1 || a.dim > DELTA_SCAN_MAX_DIM || a.heads < 1 || a.heads > 65535 || a.vdim < 1 || a.qk_heads < 1 ||
      a.heads % a.qk_heads != 0)
    return cudaErrorInvalidValue;
  if (a.dim <= 32) return delta_scan_rpt<4>(a, seqs, n_seqs, tok_slot, stream);
  if (a.dim <= 8 * DS_LPC) return delta_scan_rpt<8>(a, seqs, n_seqs, tok_slot, stream);
  if (a.dim <= 16 * DS_LPC) return delta_scan_rpt<16>(a, seqs, n_seqs, tok_slot, stream);
  return delta_scan_rpt<32>(a, seqs, n_seqs, tok_slot, stream);
}

cudaError_t convert_f32_launch(const float* x, void* out, int out_dtype, size_t n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 8);
  return launch_k(convert_f32_kernel, dim3(blocks), dim3(256), 0, stream, x, out, out_dtype, n);
}

}  // namespace tgis
