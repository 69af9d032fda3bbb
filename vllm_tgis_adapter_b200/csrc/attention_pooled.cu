// Grouped-query softmax attention over a sliding window of tokens plus pooled blocks of the tokens that left it
// (kernels.h: PoolAttnGeom).  A query at position i sees
//   * the tokens j with 0 <= i - j < window, each with its own key and value, and
//   * every block b of `pool` consecutive positions with b * pool + pool - 1 <= i - window through ONE key and ONE value: the
//     means of the block's cached keys (after rotation and norm) and values,
// all under one softmax.  Tokens behind the window whose block is still incomplete at i - window are not seen at all.
//
//   poolattn_prep_kernel   per token and head: bias, rotary turn (fp32 table), unit RMS norm of queries and keys, cache write
//   poolattn_pool_kernel   the blocks that this step's tokens complete: mean of the block's cache rows -> the pooled cache
//   poolattn_mma_kernel    bf16 rows whose sizes fit the MMA tiles: both products on mma.sync with fp32 accumulators
//   poolattn_kernel        any sizes and fp32 rows (FMA pipe)
//
// The attention kernels take one CTA per (tile of POOLATTN_TILE query tokens of one sequence, query head) and walk "chunks" of
// 32 keys in a fixed order: first the pooled rows 0..31, 32..63, ... that the tile's last query sees, then the sequence's
// 32-token cache blocks from the first one the tile's window touches.  Scores, the running softmax (maximum, sum) and the
// accumulators are fp32; a key that a query does not see weighs exactly zero.  So a query row's arithmetic depends on its own
// position and on the 32-row grids of its sequence only: not on the tile it shares with other queries, on how the prompt was cut,
// on the other sequences of the step, or on which physical pages hold the rows.
//
// Pooled rows live in a cache of their own that is paged by the SAME block ids: block b belongs to the page of its first
// token, p = b * pool / KV_BLOCK, at index b - ceil(p * KV_BLOCK / pool); a page owns ceil(KV_BLOCK / pool) of them.
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

template <class T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// pooled blocks a query at position `pos` sees
__device__ __forceinline__ int pooled_visible(int pos, int window, int pool) {
  const int e = pos - window + 1;   // positions [0, e) lie behind the window
  return (window > 0 && pool > 0 && e > 0) ? e / pool : 0;
}
// row of pooled block b inside the pooled cache (page table bt of the sequence)
__device__ __forceinline__ size_t pooled_row(int b, int pool, int rpp, const int32_t* bt) {
  const int page = (int)(((long long)b * pool) / KV_BLOCK);
  const int first = (page * KV_BLOCK + pool - 1) / pool;   // first block whose first token lies in the page
  return (size_t)bt[page] * rpp + (b - first);
}

// ---------------------------------------------------------------------------------------------------------------- prep
// grid (T, ceil((heads + 2 kv_heads) / 4)), 128 threads: one warp per (token, query head | key head | value head)
constexpr int PREP_WARPS = 4, PREP_MAX_DIM = 512;
template <class CT, int PREP_MAX>   // dim <= 32 * PREP_MAX
__global__ void __launch_bounds__(PREP_WARPS * 32)
poolattn_prep_kernel(const float* __restrict__ y, int ldy, int q_off, int k_off, int v_off, const float* __restrict__ bias,
                     PoolAttnGeom g, const float* __restrict__ cos_sin, float eps, const int32_t* __restrict__ positions,
                     const int32_t* __restrict__ slot_mapping, CT* __restrict__ q_out, CT* __restrict__ k_cache,
                     CT* __restrict__ v_cache) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x, hh = blockIdx.y * PREP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (hh >= g.heads + 2 * g.kv_heads) return;
  const int slot = slot_mapping[t];
  const int nq = g.heads * g.dim, nk = g.kv_heads * g.dim;
  if (hh < g.heads + g.kv_heads) {
    const bool is_q = hh < g.heads;
    const int h = is_q ? hh : hh - g.heads;
    if (!is_q && slot < 0) return;
    const float* src = y + (size_t)t * ldy + (is_q ? q_off : k_off) + (size_t)h * g.dim;
    const float* b = bias != nullptr ? bias + (is_q ? 0 : nq) + (size_t)h * g.dim : nullptr;
    const float* cs = cos_sin != nullptr ? cos_sin + (size_t)positions[t] * g.rot_dims : nullptr;
    const int half = g.rot_dims / 2;
    float val[PREP_MAX];
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < PREP_MAX; ++e) {
      const int i = lane + 32 * e;
      float v = 0.f;
      if (i < g.dim) {
        v = src[i] + (b ? b[i] : 0.f);
        if (i < g.rot_dims) {
          const int j = i < half ? i + half : i - half, f = i < half ? i : i - half;
          const float w = src[j] + (b ? b[j] : 0.f);
          v = i < half ? v * cs[f] - w * cs[half + f] : v * cs[f] + w * cs[half + f];
        }
      }
      val[e] = v;
      ss = fmaf(v, v, ss);
    }
    const float rs = g.unit_norm ? 1.f / sqrtf(warp_sum_f(ss) / (float)g.dim + eps) : 1.f;
    CT* dst = is_q ? q_out + ((size_t)t * g.heads + h) * g.dim : k_cache + ((size_t)slot * g.kv_heads + h) * g.dim;
#pragma unroll
    for (int e = 0; e < PREP_MAX; ++e) {
      const int i = lane + 32 * e;
      if (i < g.dim) stf(dst + i, val[e] * rs);
    }
  } else if (slot >= 0) {
    const int h = hh - g.heads - g.kv_heads;
    const float* src = y + (size_t)t * ldy + v_off + (size_t)h * g.vdim;
    const float* b = bias != nullptr ? bias + nq + nk + (size_t)h * g.vdim : nullptr;
    CT* dst = v_cache + ((size_t)slot * g.kv_heads + h) * g.vdim;
    for (int i = lane; i < g.vdim; i += 32) stf(dst + i, src[i] + (b ? b[i] : 0.f));
  }
}

// ---------------------------------------------------------------------------------------------------------------- pool
// grid (sequences, blocks per sequence in strides of gridDim.y), 128 threads over the columns of a K | V row
template <class CT>
__global__ void __launch_bounds__(128)
poolattn_pool_kernel(const CT* __restrict__ k_cache, const CT* __restrict__ v_cache, CT* __restrict__ pk, CT* __restrict__ pv,
                     const AttnSeq* __restrict__ seqs, const int32_t* __restrict__ block_table, int bt_stride, PoolAttnGeom g) {
  griddep_launch();
  griddep_wait();
  const AttnSeq sq = seqs[blockIdx.x];
  const int P = g.pool, first = sq.kv_len - sq.q_len;
  const int b_lo = first / P, b_hi = sq.kv_len / P;   // blocks whose last position is one of this step's tokens
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  const int nk = g.kv_heads * g.dim, nv = g.kv_heads * g.vdim, rpp = g.rows_per_page();
  const float inv = 1.f / (float)P;
  for (int b = b_lo + blockIdx.y; b < b_hi; b += gridDim.y) {
    const size_t dst = pooled_row(b, P, rpp, bt);
    if (sizeof(CT) == 2 && nk % 8 == 0 && nv % 8 == 0) {   // bf16 rows of whole 16-byte groups: eight columns per thread
      for (int c8 = threadIdx.x; c8 < (nk + nv) / 8; c8 += blockDim.x) {
        const bool is_k = c8 < nk / 8;
        const int col = is_k ? c8 * 8 : c8 * 8 - nk;
        float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int r = 0; r < P; ++r) {   // position order
          const int pos = b * P + r;
          const size_t row = (size_t)bt[pos / KV_BLOCK] * KV_BLOCK + pos % KV_BLOCK;
          const uint4 v = *reinterpret_cast<const uint4*>(is_k ? reinterpret_cast<const __nv_bfloat16*>(k_cache) + row * nk + col
                                                               : reinterpret_cast<const __nv_bfloat16*>(v_cache) + row * nv + col);
          const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s8[2 * e] += __bfloat162float(v2[e].x);
            s8[2 * e + 1] += __bfloat162float(v2[e].y);
          }
        }
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(s8[2 * e] * inv, s8[2 * e + 1] * inv);
        *reinterpret_cast<uint4*>(is_k ? reinterpret_cast<__nv_bfloat16*>(pk) + dst * nk + col
                                       : reinterpret_cast<__nv_bfloat16*>(pv) + dst * nv + col) = o;
      }
      continue;
    }
    for (int c = threadIdx.x; c < nk + nv; c += blockDim.x) {
      float s = 0.f;
#pragma unroll 4
      for (int r = 0; r < P; ++r) {   // position order
        const int pos = b * P + r;
        const size_t row = (size_t)bt[pos / KV_BLOCK] * KV_BLOCK + pos % KV_BLOCK;
        s += c < nk ? ldf(k_cache + row * nk + c) : ldf(v_cache + row * nv + (c - nk));
      }
      if (c < nk) stf(pk + dst * nk + c, s * inv);
      else stf(pv + dst * nv + (c - nk), s * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------- FMA kernel
constexpr int PA_THREADS = 128, PA_QT = POOLATTN_TILE, PA_CC = POOLATTN_MAX_VDIM / PA_THREADS;
static_assert(PA_QT == 16 && PA_THREADS == 128, "score mapping: 4 warps x 4 queries x 32 keys");

template <class CT, class OT>
__global__ void __launch_bounds__(PA_THREADS)
poolattn_kernel(const CT* __restrict__ q, const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
                const CT* __restrict__ pk, const CT* __restrict__ pv, const AttnSeq* __restrict__ seqs,
                const LatentTile* __restrict__ tiles, const int32_t* __restrict__ block_table, int bt_stride,
                OT* __restrict__ out, PoolAttnGeom g) {
  extern __shared__ __align__(16) float pa_smem[];
  const int d = g.dim, dv = g.vdim, ldk = d + 1;
  float* Qs = pa_smem;                        // [PA_QT][d]      scaled queries
  float* Ks = Qs + PA_QT * d;                 // [KV_BLOCK][d+1]
  float* Vs = Ks + KV_BLOCK * ldk;            // [KV_BLOCK][dv]
  float* Ps = Vs + KV_BLOCK * dv;             // [PA_QT][KV_BLOCK]
  float* alpha = Ps + PA_QT * KV_BLOCK;       // [PA_QT]
  float* lsum = alpha + PA_QT;                // [PA_QT]
  __shared__ long long rowoff[KV_BLOCK];      // cache row of every key of the chunk (-1: none)
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int h = blockIdx.y, kvh = h / (g.heads / g.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = sq.q_start + tl.q0;             // first query row of the tile in the flat batch
  const int pos0 = sq.kv_len - sq.q_len + tl.q0;   // its position
  const int nq = tl.nq, pos_last = pos0 + nq - 1;
  for (int i = tid; i < PA_QT * d; i += PA_THREADS) {
    const int qi = i / d, kk = i % d;
    Qs[i] = qi < nq ? ldf(q + ((size_t)(row0 + qi) * g.heads + h) * d + kk) * g.scale : 0.f;
  }
  float acc[PA_QT][PA_CC];
#pragma unroll
  for (int qi = 0; qi < PA_QT; ++qi)
#pragma unroll
    for (int cc = 0; cc < PA_CC; ++cc) acc[qi][cc] = 0.f;
  float m_run[4], l_run[4];   // this warp's four query rows (valid in every lane)
  int n_vis[4];               // pooled blocks each of them sees
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m_run[i] = -INFINITY;
    l_run[i] = 0.f;
    n_vis[i] = pooled_visible(pos0 + warp * 4 + i, g.window, g.pool);
  }
  const int n_pooled = pooled_visible(pos_last, g.window, g.pool);
  const int n_pc = (n_pooled + KV_BLOCK - 1) / KV_BLOCK;
  const int kmin = g.window > 0 ? max(0, pos0 - g.window + 1) : 0;
  const int blk0 = kmin / KV_BLOCK, blk1 = pos_last / KV_BLOCK;
  const int n_chunks = n_pc + blk1 - blk0 + 1;
  const int rpp = g.rows_per_page();
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  for (int c = 0; c < n_chunks; ++c) {
    const bool pooled = c < n_pc;
    __syncthreads();   // the previous chunk's Ks / Vs / Ps / rowoff are consumed (first pass: Qs complete)
    if (tid < KV_BLOCK) {
      long long r;
      if (pooled) {
        const int b = c * KV_BLOCK + tid;
        r = b < n_pooled ? (long long)pooled_row(b, g.pool, rpp, bt) : -1;
      } else {
        r = (long long)bt[blk0 + c - n_pc] * KV_BLOCK + tid;
      }
      rowoff[tid] = r;
    }
    __syncthreads();
    const CT* kb = pooled ? pk : k_cache;
    const CT* vb = pooled ? pv : v_cache;
    for (int i = tid; i < KV_BLOCK * d; i += PA_THREADS) {
      const int j = i / d, kk = i % d;
      const long long r = rowoff[j];
      Ks[j * ldk + kk] = r >= 0 ? ldf(kb + ((size_t)r * g.kv_heads + kvh) * d + kk) : 0.f;
    }
    for (int i = tid; i < KV_BLOCK * dv; i += PA_THREADS) {
      const int j = i / dv, cc = i % dv;
      const long long r = rowoff[j];
      Vs[i] = r >= 0 ? ldf(vb + ((size_t)r * g.kv_heads + kvh) * dv + cc) : 0.f;
    }
    __syncthreads();
    // ---- scores: lane = key, this warp's four queries
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * ldk;
    const float* qr = Qs + warp * 4 * d;
    for (int kk = 0; kk < d; ++kk) {
      const float kv = kr[kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(qr[i * d + kk], kv, s[i]);
    }
    const int kidx = (pooled ? c : blk0 + c - n_pc) * KV_BLOCK + lane;   // pooled block number, or token position
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = warp * 4 + i, pi = pos0 + qi;
      const bool ok = qi < nq && (pooled ? kidx < n_vis[i] : (kidx <= pi && (g.window <= 0 || pi - kidx < g.window)));
      const float sc = ok ? s[i] : -INFINITY;
      const float m_new = fmaxf(m_run[i], warp_max_f(sc));
      const float p = ok ? expf(sc - m_new) : 0.f;
      const float al = m_new == -INFINITY ? 1.f : expf(m_run[i] - m_new);   // (-inf: nothing seen yet, nothing to scale)
      l_run[i] = fmaf(l_run[i], al, warp_sum_f(p));
      m_run[i] = m_new;
      Ps[qi * KV_BLOCK + lane] = p;
      if (lane == 0) alpha[qi] = al;
    }
    __syncthreads();
    // ---- weighted sum of the values: thread = value column(s), all queries of the tile
#pragma unroll
    for (int cc = 0; cc < PA_CC; ++cc) {
      const int col = tid + cc * PA_THREADS;
      if (col < dv) {
#pragma unroll
        for (int qi = 0; qi < PA_QT; ++qi)
          if (qi < nq) acc[qi][cc] *= alpha[qi];
        for (int j = 0; j < KV_BLOCK; ++j) {
          const float vv = Vs[j * dv + col];
#pragma unroll
          for (int qi = 0; qi < PA_QT; ++qi)
            if (qi < nq) acc[qi][cc] = fmaf(Ps[qi * KV_BLOCK + j], vv, acc[qi][cc]);
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) lsum[warp * 4 + i] = l_run[i];
  }
  __syncthreads();
#pragma unroll
  for (int cc = 0; cc < PA_CC; ++cc) {
    const int col = tid + cc * PA_THREADS;
    if (col < dv) {
#pragma unroll
      for (int qi = 0; qi < PA_QT; ++qi)
        if (qi < nq) stf(out + ((size_t)(row0 + qi) * g.heads + h) * dv + col, acc[qi][cc] / lsum[qi]);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------- tensor cores
// bf16 queries and cache rows, dim a multiple of 16 (<= 16 MMA_KS), vdim a multiple of 8 (<= 32 MMA_NT per warp).  Both products
// on mma.sync m16n8k16 with fp32 accumulators: the tile's 16 queries are the M rows; for the scores each of the four warps owns
// 8 of a chunk's 32 keys (the query's A fragments stay in registers for the whole walk, key rows are B fragments as they lie;
// the chunk after the current one lands in a second buffer through cp.async meanwhile), for the weighted sum each warp owns
// every fourth group of 8 value columns (value rows through ldmatrix.trans).  Scale, mask and the running softmax are fp32 on
// the accumulator fragments; the weights are rounded to bf16 once and the SAME rounded numbers are summed for the normaliser.
// Pooled chunks and token chunks differ only in where a row comes from and in which queries see it.
constexpr int MMA_KS = 8, MMA_NT = 8, PA_NST = 4;
__device__ __forceinline__ void pa_ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pa_ldsm_x2(uint32_t (&r)[2], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void pa_ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void pa_cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void pa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(PA_THREADS)
poolattn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const __nv_bfloat16* __restrict__ pk,
                    const __nv_bfloat16* __restrict__ pv, const AttnSeq* __restrict__ seqs, const LatentTile* __restrict__ tiles,
                    const int32_t* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ out, PoolAttnGeom g, int gs) {
  // gs: query heads per tile.  1: the 16 rows are 16 tokens of head blockIdx.y; grid (tiles, heads).  heads / kv_heads (2, 4, 8 or
  // 16): the rows are (token, head of key/value head blockIdx.y) pairs, 16 / gs tokens x gs heads, so a chunk's rows are fetched
  // once for the whole group and a decoded token fills gs rows instead of one; grid (tiles, kv_heads, gs), CTA z takes the
  // tile's tokens [z * 16 / gs, (z + 1) * 16 / gs) and leaves at once when the tile has none there.
  using bf = __nv_bfloat16;
  extern __shared__ __align__(16) uint8_t pam_smem[];
  const int d = g.dim, dv = g.vdim, LDK = d + 8, LDV = dv + 8, LDP = KV_BLOCK + 8;
  bf* Qs = reinterpret_cast<bf*>(pam_smem);            // [16][LDK]
  bf* Ks2 = Qs + PA_QT * LDK;                          // [PA_NST][32][LDK]   a ring of chunks: one in use, the next ones landing
  bf* Vs2 = Ks2 + PA_NST * KV_BLOCK * LDK;             // [PA_NST][32][LDV]
  bf* Ps = Vs2 + PA_NST * KV_BLOCK * LDV;              // [16][LDP]
  float* smax = reinterpret_cast<float*>(Ps + PA_QT * LDP);   // [4][16]; reused for the final row sums
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int kvh = gs > 1 ? blockIdx.y : blockIdx.y / (g.heads / g.kv_heads);
  const int h_base = gs > 1 ? kvh * gs : blockIdx.y;     // head of row r: h_base + r % gs
  const int tpt = PA_QT / gs;                             // tokens of this CTA's rows; token of row r: r / gs
  const int tok0 = gs > 1 ? blockIdx.z * tpt : 0;
  if (tok0 >= tl.nq) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t2 = (lane & 3) * 2;
  const int row0 = sq.q_start + tl.q0 + tok0, pos0 = sq.kv_len - sq.q_len + tl.q0 + tok0, nq = min(tpt, tl.nq - tok0);
  const int pos_last = pos0 + nq - 1;
  const int dch = d / 8, vch = dv / 8;   // 16-byte chunks per row
  for (int i = tid; i < PA_QT * dch; i += PA_THREADS) {
    const int r = i / dch, ch = i % dch, tq = r / gs;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tq < nq) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + tq) * g.heads + h_base + r % gs) * d + ch * 8);
    *reinterpret_cast<uint4*>(Qs + r * LDK + ch * 8) = v;
  }
  __syncthreads();
  const int nks = d / 16;
  uint32_t qa[MMA_KS][4];
#pragma unroll
  for (int ks = 0; ks < MMA_KS; ++ks)
    if (ks < nks) pa_ldsm_x4(qa[ks], Qs + (size_t)(lane & 15) * LDK + ks * 16 + (lane >> 4) * 8);
  float acc[MMA_NT][4];
#pragma unroll
  for (int j = 0; j < MMA_NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};   // rows gq and gq + 8
  const int tqr[2] = {gq / gs, (gq + 8) / gs};   // tokens of this thread's two rows
  const int n_vis[2] = {pooled_visible(pos0 + tqr[0], g.window, g.pool), pooled_visible(pos0 + tqr[1], g.window, g.pool)};
  const int n_pooled = pooled_visible(pos_last, g.window, g.pool);
  const int n_pc = (n_pooled + KV_BLOCK - 1) / KV_BLOCK;
  const int kmin = g.window > 0 ? max(0, pos0 - g.window + 1) : 0;
  const int blk0 = kmin / KV_BLOCK, blk1 = pos_last / KV_BLOCK;
  const int n_chunks = n_pc + blk1 - blk0 + 1;
  const int rpp = g.rows_per_page();
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  // chunk c's K and V rows -> stage c % PA_NST of the ring, as 16-byte asynchronous copies: four threads share a row, every
  // call is one commit group (an empty one past the last chunk, so that the group count tells which chunk has landed); pooled
  // rows that do not exist yet are zeros
  const int fj = tid >> 2, fl = tid & 3;
  auto fetch = [&](int c) {
    if (c < n_chunks) {
      const bool pooled = c < n_pc;
      long long r;
      if (pooled) {
        const int b = c * KV_BLOCK + fj;
        r = b < n_pooled ? (long long)pooled_row(b, g.pool, rpp, bt) : -1;
      } else {
        r = (long long)bt[blk0 + c - n_pc] * KV_BLOCK + fj;
      }
      bf* Kd = Ks2 + ((size_t)(c % PA_NST) * KV_BLOCK + fj) * LDK;
      bf* Vd = Vs2 + ((size_t)(c % PA_NST) * KV_BLOCK + fj) * LDV;
      if (r < 0) {
        for (int ch = fl; ch < dch; ch += 4) *reinterpret_cast<uint4*>(Kd + ch * 8) = make_uint4(0, 0, 0, 0);
        for (int ch = fl; ch < vch; ch += 4) *reinterpret_cast<uint4*>(Vd + ch * 8) = make_uint4(0, 0, 0, 0);
      } else {
        const bf* ks = (pooled ? pk : k_cache) + ((size_t)r * g.kv_heads + kvh) * d;
        const bf* vs = (pooled ? pv : v_cache) + ((size_t)r * g.kv_heads + kvh) * dv;
        for (int ch = fl; ch < dch; ch += 4) pa_cp_async16(Kd + ch * 8, ks + ch * 8);
        for (int ch = fl; ch < vch; ch += 4) pa_cp_async16(Vd + ch * 8, vs + ch * 8);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
#pragma unroll
  for (int c = 0; c < PA_NST - 1; ++c) fetch(c);
  for (int c = 0; c < n_chunks; ++c) {
    const bool pooled = c < n_pc;
    // the stage that chunk c + PA_NST - 1 goes to was last read in the previous pass, which ended with a barrier
    fetch(c + PA_NST - 1);
    asm volatile("cp.async.wait_group %0;\n" ::"n"(PA_NST - 1) : "memory");
    __syncthreads();   // every thread's copies of chunk c have landed
    const bf* Ks = Ks2 + (size_t)(c % PA_NST) * KV_BLOCK * LDK;
    const bf* Vs = Vs2 + (size_t)(c % PA_NST) * KV_BLOCK * LDV;
    // ---- scores of this warp's 8 keys
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < MMA_KS; ++ks)
      if (ks < nks) {
        uint32_t kb2[2];
        pa_ldsm_x2(kb2, Ks + (size_t)(warp * 8 + (lane & 7)) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
        pa_mma(sc, qa[ks], kb2[0], kb2[1]);
      }
    bool ok[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1, pi = pos0 + tqr[r];
      const int kidx = (pooled ? c : blk0 + c - n_pc) * KV_BLOCK + warp * 8 + t2 + (e & 1);   // pooled block number, or token position
      ok[e] = tqr[r] < nq && (pooled ? kidx < n_vis[r] : (kidx <= pi && (g.window <= 0 || pi - kidx < g.window)));
      sc[e] = ok[e] ? sc[e] * g.scale : -INFINITY;
    }
    float mx[2] = {fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3])};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    if ((lane & 3) == 0) {
      smax[warp * PA_QT + gq] = mx[0];
      smax[warp * PA_QT + gq + 8] = mx[1];
    }
    __syncthreads();
    float al[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int qi = gq + r * 8;
      const float bm = fmaxf(fmaxf(smax[qi], smax[PA_QT + qi]), fmaxf(smax[2 * PA_QT + qi], smax[3 * PA_QT + qi]));
      const float m_new = fmaxf(m_run[r], bm);
      al[r] = m_new == -INFINITY ? 1.f : expf(m_run[r] - m_new);
      const bf p0 = __float2bfloat16_rn(ok[2 * r] ? expf(sc[2 * r] - m_new) : 0.f);
      const bf p1 = __float2bfloat16_rn(ok[2 * r + 1] ? expf(sc[2 * r + 1] - m_new) : 0.f);
      l_part[r] = fmaf(l_part[r], al[r], __bfloat162float(p0) + __bfloat162float(p1));
      m_run[r] = m_new;
      __nv_bfloat162 pp;
      pp.x = p0; pp.y = p1;
      *reinterpret_cast<__nv_bfloat162*>(Ps + qi * LDP + warp * 8 + t2) = pp;
    }
    __syncthreads();
    // ---- weighted sum of the values: this warp's groups of 8 columns
    uint32_t a0[4], a1[4];
    pa_ldsm_x4(a0, Ps + (size_t)(lane & 15) * LDP + (lane >> 4) * 8);
    pa_ldsm_x4(a1, Ps + (size_t)(lane & 15) * LDP + 16 + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n0 = (warp + 4 * j) * 8;
      if (n0 < dv) {
        acc[j][0] *= al[0]; acc[j][1] *= al[0]; acc[j][2] *= al[1]; acc[j][3] *= al[1];
        uint32_t vb2[4];
        pa_ldsm_x4_trans(vb2, Vs + (size_t)lane * LDV + n0);
        pa_mma(acc[j], a0, vb2[0], vb2[1]);
        pa_mma(acc[j], a1, vb2[2], vb2[3]);
      }
    }
    __syncthreads();   // this pass's buffers, maxima and weights are consumed
  }
  // ---- row sums: over the quad, then over the warps
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 1);
    l_part[r] += __shfl_xor_sync(0xffffffffu, l_part[r], 2);
  }
  __syncthreads();
  if ((lane & 3) == 0) {
    smax[warp * PA_QT + gq] = l_part[0];
    smax[warp * PA_QT + gq + 8] = l_part[1];
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = gq + r * 8;
    if (tqr[r] >= nq) continue;
    const float inv_l = 1.f / (smax[qi] + smax[PA_QT + qi] + smax[2 * PA_QT + qi] + smax[3 * PA_QT + qi]);
    const size_t row = (size_t)(row0 + tqr[r]);
    const int h = h_base + qi % gs;
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n = (warp + 4 * j) * 8 + t2;
      if (n < dv) {
        __nv_bfloat162 pp;
        pp.x = __float2bfloat16_rn(acc[j][2 * r] * inv_l); pp.y = __float2bfloat16_rn(acc[j][2 * r + 1] * inv_l);
        *reinterpret_cast<__nv_bfloat162*>(out + (row * g.heads + h) * dv + n) = pp;
      }
    }
  }
}

bool mma_eligible(const PoolAttnGeom& g, const void* q, const void* k, const void* v, const void* pk, const void* pv, const void* out) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TGIS_POOLATTN_MMA");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return on && g.dim % 16 == 0 && g.dim <= 16 * MMA_KS && g.vdim % 8 == 0 && g.vdim <= 32 * MMA_NT && al16(q) && al16(k) && al16(v) &&
         al16(pk) && al16(pv) && al16(out);
}

template <class CT>
cudaError_t launch_fma(const void* q, const void* k_cache, const void* v_cache, const void* pk, const void* pv,
                       const AttnSeq* seqs, const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                       void* out, const PoolAttnGeom& g, cudaStream_t stream) {
  const size_t smem = ((size_t)PA_QT * g.dim + (size_t)KV_BLOCK * (g.dim + 1) + (size_t)KV_BLOCK * g.vdim + PA_QT * KV_BLOCK +
                       2 * PA_QT) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  static size_t attr_bytes = 0;   // per instantiation
  if (smem > 48 * 1024 && smem > attr_bytes) {
    const cudaError_t e = cudaFuncSetAttribute(poolattn_kernel<CT, CT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes = smem;
  }
  return launch_k(poolattn_kernel<CT, CT>, dim3(n_tiles, g.heads), dim3(PA_THREADS), smem, stream,
                  reinterpret_cast<const CT*>(q), reinterpret_cast<const CT*>(k_cache), reinterpret_cast<const CT*>(v_cache),
                  reinterpret_cast<const CT*>(pk), reinterpret_cast<const CT*>(pv), seqs, tiles, block_table, bt_stride,
                  reinterpret_cast<CT*>(out), g);
}

bool geom_ok(const PoolAttnGeom& g) {
  return g.heads >= 1 && g.kv_heads >= 1 && g.heads % g.kv_heads == 0 && g.heads <= 65535 && g.dim >= 1 && g.vdim >= 1 &&
         g.dim <= PREP_MAX_DIM && g.vdim <= POOLATTN_MAX_VDIM && g.rot_dims >= 0 && g.rot_dims <= g.dim && (g.rot_dims & 1) == 0;
}

}  // namespace

cudaError_t poolattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const float* bias,
                                 const PoolAttnGeom& g, const float* cos_sin, float eps, const int32_t* positions,
                                 const int32_t* slot_mapping, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                 cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (!geom_ok(g) || (g.rot_dims > 0 && cos_sin == nullptr)) return cudaErrorInvalidValue;
  const dim3 grid(T, (g.heads + 2 * g.kv_heads + PREP_WARPS - 1) / PREP_WARPS);
  using bf = __nv_bfloat16;
  const bool small = g.dim <= 128;   // four entries per lane
  if (dtype == DT_BF16)
    return launch_k(small ? poolattn_prep_kernel<bf, 4> : poolattn_prep_kernel<bf, PREP_MAX_DIM / 32>, grid, dim3(PREP_WARPS * 32), 0,
                    stream, y, ldy, q_off, k_off, v_off, bias, g, cos_sin, eps, positions, slot_mapping, reinterpret_cast<bf*>(q_out),
                    reinterpret_cast<bf*>(k_cache), reinterpret_cast<bf*>(v_cache));
  return launch_k(small ? poolattn_prep_kernel<float, 4> : poolattn_prep_kernel<float, PREP_MAX_DIM / 32>, grid, dim3(PREP_WARPS * 32),
                  0, stream, y, ldy, q_off, k_off, v_off, bias, g, cos_sin, eps, positions, slot_mapping,
                  reinterpret_cast<float*>(q_out), reinterpret_cast<float*>(k_cache), reinterpret_cast<float*>(v_cache));
}

cudaError_t poolattn_pool_launch(const void* k_cache, const void* v_cache, void* pk, void* pv, int dtype,
                                 const AttnSeq* seqs, int n_seqs, const int32_t* block_table, int bt_stride,
                                 const PoolAttnGeom& g, int max_q_len, cudaStream_t stream) {
  if (n_seqs <= 0 || g.pool <= 0 || g.window <= 0) return cudaSuccess;
  if (!geom_ok(g)) return cudaErrorInvalidValue;
  const dim3 grid(n_seqs, std::min(max_q_len / g.pool + 1, 4096));
  if (dtype == DT_BF16)
    return launch_k(poolattn_pool_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream,
                    reinterpret_cast<const __nv_bfloat16*>(k_cache), reinterpret_cast<const __nv_bfloat16*>(v_cache),
                    reinterpret_cast<__nv_bfloat16*>(pk), reinterpret_cast<__nv_bfloat16*>(pv), seqs, block_table, bt_stride, g);
  return launch_k(poolattn_pool_kernel<float>, grid, dim3(128), 0, stream, reinterpret_cast<const float*>(k_cache),
                  reinterpret_cast<const float*>(v_cache), reinterpret_cast<float*>(pk), reinterpret_cast<float*>(pv), seqs,
                  block_table, bt_stride, g);
}

cudaError_t poolattn_launch(const void* q, const void* k_cache, const void* v_cache, const void* pk, const void* pv, int dtype,
                            const AttnSeq* seqs, const LatentTile* tiles, int n_tiles, const int32_t* block_table,
                            int bt_stride, void* out, int out_dtype, const PoolAttnGeom& g, cudaStream_t stream) {
  if (n_tiles <= 0) return cudaSuccess;
  if (!geom_ok(g) || out_dtype != dtype) return cudaErrorInvalidValue;
  if (dtype == DT_BF16 && mma_eligible(g, q, k_cache, v_cache, pk, pv, out)) {
    using bf = __nv_bfloat16;
    const size_t smem = ((size_t)(PA_QT + PA_NST * KV_BLOCK) * (g.dim + 8) + (size_t)PA_NST * KV_BLOCK * (g.vdim + 8) + PA_QT * (KV_BLOCK + 8)) * sizeof(bf) +
                        4 * PA_QT * sizeof(float);   // <= 108 KB
    static bool attr_set = false;
    if (!attr_set) {
      const cudaError_t e = cudaFuncSetAttribute(poolattn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    static int group_on = -1;
    if (group_on < 0) {
      const char* e = getenv("TGIS_POOLATTN_GROUP");
      group_on = (e && e[0] == '0') ? 0 : 1;
    }
    const int per_kv = g.heads / g.kv_heads;
    const int gs = (group_on && per_kv >= 2 && per_kv <= PA_QT && PA_QT % per_kv == 0) ? per_kv : 1;
    const dim3 grid = gs > 1 ? dim3(n_tiles, g.kv_heads, gs) : dim3(n_tiles, g.heads, 1);
    return launch_k(poolattn_mma_kernel, grid, dim3(PA_THREADS), smem, stream, reinterpret_cast<const bf*>(q),
                    reinterpret_cast<const bf*>(k_cache), reinterpret_cast<const bf*>(v_cache), reinterpret_cast<const bf*>(pk),
                    reinterpret_cast<const bf*>(pv), seqs, tiles, block_table, bt_stride, reinterpret_cast<bf*>(out), g, gs);
  }
  if (dtype == DT_BF16)
    return launch_fma<__nv_bfloat16>(q, k_cache, v_cache, pk, pv, seqs, tiles, n_tiles, block_table, bt_stride, out, g, stream);
  return launch_fma<float>(q, k_cache, v_cache, pk, pv, seqs, tiles, n_tiles, block_table, bt_stride, out, g, stream);
}

}  // namespace tgis
