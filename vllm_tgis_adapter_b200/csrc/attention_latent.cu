// Attention over a cached low-rank latent (kernels.h, LatentGeom): every token leaves ONE cache row
// [c (kv_rank) | k_rot (rot_dim)]; the per-head key and value up-projections are folded into the query and the output,
// so all heads of a token score against -- and sum over -- the same rows of the paged cache:
//   s_h(i, j) = scale * q_abs_h(i) . row(j),        o_lat_h(i) = sum_j softmax_j(s_h(i, .)) c(j)
// with j causal and, for window > 0, inside the last `window` positions.  Softmax, its running maximum / sum and the
// output accumulators are fp32; cache rows are read in their storage type and widened.
//
// latent_attn_kernel serves prompts, prompt portions and single decoded tokens alike: a CTA owns up to LATENT_PAIRS
// (token, head) pairs of one sequence, walks the cache blocks its queries can see (block table; blocks wholly outside
// the window are never touched), stages each 32-row block in shared memory once and lets every warp run two pairs
// against it: lane = key for the scores, lane = latent dimension (strided by 32) for the weighted sum.  A query's
// arithmetic depends only on its own position and on the block grid of its sequence, not on the tile or step it came in.
#include <algorithm>
#include <cfloat>
#include <cstdint>
#include <cstdlib>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

constexpr int LAT_THREADS = 256;
constexpr int LAT_WARPS = LAT_THREADS / 32;
static_assert(LATENT_PAIRS == 2 * LAT_WARPS, "two pairs per warp");

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
template <int THREADS>
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  v = warp_sum_f(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < THREADS / 32) ? red[l] : 0.f;
  t = warp_sum_f(t);
  __syncthreads();
  return t;
}
__device__ __forceinline__ void st_any(void* out, int dt, size_t i, float v) {
  if (dt == DT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(out)[i] = v;
}
template <class T>
__device__ __forceinline__ float widen(T v);
template <>
__device__ __forceinline__ float widen<float>(float v) { return v; }
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// "rotate half" over the first rot_dims entries of a rot_dim-long vector: entry i pairs with i + rot_dims / 2
// (interleaved: entry 2i pairs with 2i + 1; the table stays cos (rot_dims / 2) | sin (rot_dims / 2))
__device__ __forceinline__ float rotary_entry(const float* v, int j, int rot_dims, const float* cs, int interleaved = 0) {
  const int half = rot_dims / 2;
  if (j >= rot_dims) return v[j];
  if (interleaved) {
    const int f = j >> 1;
    return (j & 1) ? v[j] * cs[f] + v[j - 1] * cs[half + f] : v[j] * cs[f] - v[j + 1] * cs[half + f];
  }
  if (j < half) return v[j] * cs[j] - v[j + half] * cs[half + j];
  return v[j] * cs[j - half] + v[j - half] * cs[j];  // cs[j] with j >= half is sin(j - half)
}

constexpr int PREP_THREADS = 256;
__global__ void __launch_bounds__(PREP_THREADS)
latent_prep_kernel(const float* __restrict__ y, int ldy, LatentGeom g, const float* __restrict__ w_q,
                   const float* __restrict__ w_kv, float eps, const int32_t* __restrict__ positions,
                   const int32_t* __restrict__ slot_mapping, const float* __restrict__ cos_sin, void* __restrict__ cq,
                   void* __restrict__ cache, int dtype, float* __restrict__ gate) {
  __shared__ float red[PREP_THREADS / 32];
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const float* row = y + (size_t)t * ldy;
  const float* yq = row;
  const float* ykv = row + g.q_rank;
  const float* ykr = ykv + g.kv_rank;
  const float* yg = ykr + g.rot_dim;
  float ss = 0.f;
  for (int i = threadIdx.x; i < g.q_rank; i += PREP_THREADS) ss += yq[i] * yq[i];
  const float rs_q = 1.f / sqrtf(block_sum_f<PREP_THREADS>(ss, red) / (float)g.q_rank + eps);
  ss = 0.f;
  for (int i = threadIdx.x; i < g.kv_rank; i += PREP_THREADS) ss += ykv[i] * ykv[i];
  const float rs_kv = 1.f / sqrtf(block_sum_f<PREP_THREADS>(ss, red) / (float)g.kv_rank + eps);
  for (int i = threadIdx.x; i < g.q_rank; i += PREP_THREADS) st_any(cq, dtype, (size_t)t * g.q_rank + i, yq[i] * rs_q * w_q[i]);
  if (gate != nullptr)
    for (int h = threadIdx.x; h < g.heads; h += PREP_THREADS) gate[(size_t)t * g.heads + h] = 1.f / (1.f + expf(-yg[h]));
  const int slot = slot_mapping[t];
  if (slot < 0) return;
  const size_t crow = (size_t)slot * g.row();
  for (int i = threadIdx.x; i < g.kv_rank; i += PREP_THREADS) st_any(cache, dtype, crow + i, ykv[i] * rs_kv * w_kv[i]);
  const float* cs = cos_sin + (size_t)positions[t] * g.rot_dims;
  for (int j = threadIdx.x; j < g.rot_dim; j += PREP_THREADS)
    st_any(cache, dtype, crow + g.kv_rank + j, rotary_entry(ykr, j, g.rot_dims, cs, g.interleaved));
}

template <class QT>
__global__ void latent_q_rope_kernel(const QT* __restrict__ q, LatentGeom g, const int32_t* __restrict__ positions,
                                     const float* __restrict__ cos_sin, float* __restrict__ q_abs) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x;
  const float* cs = cos_sin + (size_t)positions[t] * g.rot_dims;
  const int hd = g.dim + g.rot_dim, D = g.row(), half = g.rot_dims / 2;
  for (int e = threadIdx.x; e < g.heads * g.rot_dim; e += blockDim.x) {
    const int h = e / g.rot_dim, j = e % g.rot_dim;
    const QT* v = q + ((size_t)t * g.heads + h) * hd + g.dim;
    float r;  // "rotate half" over the first rot_dims entries (rotary_entry, on the stored type)
    if (j >= g.rot_dims) r = widen<QT>(v[j]);
    else if (g.interleaved) {
      const int f = j >> 1;
      r = (j & 1) ? widen<QT>(v[j]) * cs[f] + widen<QT>(v[j - 1]) * cs[half + f] : widen<QT>(v[j]) * cs[f] - widen<QT>(v[j + 1]) * cs[half + f];
    } else if (j < half) r = widen<QT>(v[j]) * cs[j] - widen<QT>(v[j + half]) * cs[half + j];
    else r = widen<QT>(v[j]) * cs[j - half] + widen<QT>(v[j - half]) * cs[j];
    q_abs[((size_t)t * g.heads + h) * D + g.kv_rank + j] = r;
  }
}

// NACC * 32 >= kv_rank.  Dynamic shared memory: Ks [KV_BLOCK][ldk] + Qs [LATENT_PAIRS][D] floats.
template <class CT, int NACC>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_kernel(const float* __restrict__ q_abs, const CT* __restrict__ cache, const AttnSeq* __restrict__ seqs,
                   const LatentTile* __restrict__ tiles, const int32_t* __restrict__ block_table, int bt_stride,
                   void* __restrict__ o_lat, int o_dtype, LatentGeom g) {
  extern __shared__ __align__(16) float smem_f[];
  griddep_launch();
  griddep_wait();
  const int D = g.row(), R = g.kv_rank;
  const int ldk = D | 1;  // odd row stride: lanes (= keys) hit 32 different banks in the score loop
  float* Ks = smem_f;
  float* Qs = smem_f + (size_t)KV_BLOCK * ldk;
  const LatentTile tile = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tile.seq];
  const int h0 = blockIdx.y * LATENT_PAIRS;
  const int nh = min(g.heads - h0, LATENT_PAIRS);
  const int npairs = tile.nq * nh;  // <= LATENT_PAIRS by construction of the tiles
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos0 = sq.kv_len - sq.q_len + tile.q0;  // position of the tile's first query
  const int row0 = sq.q_start + tile.q0;            // its row in the step's flat token batch
  for (int e = threadIdx.x; e < npairs * D; e += LAT_THREADS) {
    const int p = e / D, d = e % D;
    const int tq = p / nh, h = h0 + p % nh;
    Qs[(size_t)p * D + d] = q_abs[((size_t)(row0 + tq) * g.heads + h) * D + d] * g.scale;
  }
  // this warp's two pairs
  int pp[2], posq[2];
  bool on[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    pp[u] = warp + u * LAT_WARPS;
    on[u] = pp[u] < npairs;
    posq[u] = on[u] ? pos0 + pp[u] / nh : -1;
  }
  float m[2] = {-FLT_MAX, -FLT_MAX}, l[2] = {0.f, 0.f};
  float acc[2][NACC];
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[u][i] = 0.f;

  const int pos_last = pos0 + tile.nq - 1;
  const int kmin = g.window > 0 ? max(0, pos0 - g.window + 1) : 0;
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  for (int blk = kmin / KV_BLOCK; blk <= pos_last / KV_BLOCK; ++blk) {
    __syncthreads();  // the previous block's rows (and, first time round, Qs) are settled
    const CT* src = cache + (size_t)bt[blk] * KV_BLOCK * D;
    for (int e = threadIdx.x; e < KV_BLOCK * D; e += LAT_THREADS) Ks[(size_t)(e / D) * ldk + e % D] = widen<CT>(src[e]);
    __syncthreads();
    const int kp = blk * KV_BLOCK + lane;  // this lane's key position
    float s[2] = {0.f, 0.f};
    const float* krow = Ks + (size_t)lane * ldk;
    const float* q0p = Qs + (size_t)(on[0] ? pp[0] : 0) * D;
    const float* q1p = Qs + (size_t)(on[1] ? pp[1] : 0) * D;
    for (int d = 0; d < D; ++d) {
      const float kv = krow[d];
      s[0] = fmaf(q0p[d], kv, s[0]);
      s[1] = fmaf(q1p[d], kv, s[1]);
    }
    float p[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool vis = on[u] && kp <= posq[u] && (g.window <= 0 || posq[u] - kp < g.window);
      const float sv = vis ? s[u] : -FLT_MAX;
      const float m_new = fmaxf(m[u], warp_max_f(sv));
      // nothing visible so far (m_new still the sentinel): all weights 0, state unchanged
      const float corr = m_new == -FLT_MAX ? 1.f : expf(m[u] - m_new);
      p[u] = vis ? expf(sv - m_new) : 0.f;
      l[u] = l[u] * corr + warp_sum_f(p[u]);
      m[u] = m_new;
#pragma unroll
      for (int i = 0; i < NACC; ++i) acc[u][i] *= corr;
    }
    for (int j = 0; j < KV_BLOCK; ++j) {
      const float p0 = __shfl_sync(0xffffffffu, p[0], j), p1 = __shfl_sync(0xffffffffu, p[1], j);
      if (p0 == 0.f && p1 == 0.f) continue;  // warp-uniform
      const float* cj = Ks + (size_t)j * ldk;
#pragma unroll
      for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < R) {
          const float cv = cj[d];
          acc[0][i] = fmaf(p0, cv, acc[0][i]);
          acc[1][i] = fmaf(p1, cv, acc[1][i]);
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (!on[u]) continue;
    const int tq = pp[u] / nh, h = h0 + pp[u] % nh;
    const size_t o = ((size_t)(row0 + tq) * g.heads + h) * R;
    // the sink joins the denominator only: exp(sink - m) beside the keys' exp(s - m) (a causal row always sees itself: m is finite)
    const float inv = 1.f / (l[u] + (g.sink != nullptr ? expf(g.sink[h] - m[u]) : 0.f));
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int d = lane + 32 * i;
      if (d < R) st_any(o_lat, o_dtype, o + d, acc[u][i] * inv);
    }
  }
}

// ---- tensor-core variant (bf16 cache rows of a multiple of 8 entries) ------------------------------------------------
// Same work split as latent_attn_kernel (a CTA = up to 16 (token, head) pairs of one sequence against the 32-row cache
// blocks they can see), with the two products on mma.sync m16n8k16: the 16 pairs are the M rows of both.
//   scores  S [16 x 32] = Q [16 x D] K^T: the row length D is cut in two halves over the warps (warps 0-3 / 4-7), each warp
//           takes 8 keys; the two fp32 partial tiles meet in shared memory
//   softmax fp32, one warp per two rows, lane = key (as in the FMA kernel): running maximum and sum, P rounded to bf16
//   output  O [16 x kv_rank] += P [16 x 32] C [32 x kv_rank]: warp w owns the 8-column tiles w, w + 8, ... (fp32 accumulators
//           in registers for the whole walk), C read straight from the staged rows with ldmatrix.trans
// Cache blocks arrive by cp.async, double-buffered: block i + 1 lands while block i is being used.  Q is scaled and rounded
// to bf16 once.  A query's arithmetic still depends only on its own position and its sequence's block grid.
__device__ __forceinline__ void lat_cp_async_16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void lat_ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lat_ldsm_x2(uint32_t (&r)[2], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(s));
}
__device__ __forceinline__ void lat_ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void lat_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
inline __host__ __device__ int lat_ldq(int D) { return (D + 15) / 16 * 16 + 8; }  // padded row length (bf16 elements)
inline size_t lat_mma_smem(int D) {
  return (size_t)(LATENT_PAIRS + 2 * KV_BLOCK) * lat_ldq(D) * 2 + (size_t)2 * LATENT_PAIRS * 33 * 4 + LATENT_PAIRS * 40 * 2 +
         2 * LATENT_PAIRS * 4;
}

template <int NT>  // NT * 64 >= kv_rank
__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_mma_kernel(const float* __restrict__ q_abs, const __nv_bfloat16* __restrict__ cache,
                       const AttnSeq* __restrict__ seqs, const LatentTile* __restrict__ tiles,
                       const int32_t* __restrict__ block_table, int bt_stride, void* __restrict__ o_lat, int o_dtype,
                       LatentGeom g, float* __restrict__ part, int n_splits) {
  using bf = __nv_bfloat16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = g.row(), R = g.kv_rank, LDQ = lat_ldq(D);
  bf* Qs = reinterpret_cast<bf*>(smem_raw);                       // [16][LDQ]
  bf* Ks = Qs + (size_t)LATENT_PAIRS * LDQ;                       // [2][32][LDQ]
  float* Sp = reinterpret_cast<float*>(Ks + (size_t)2 * KV_BLOCK * LDQ);  // [2][16][33]
  bf* Ps = reinterpret_cast<bf*>(Sp + 2 * LATENT_PAIRS * 33);     // [16][40]
  float* corr_s = reinterpret_cast<float*>(Ps + LATENT_PAIRS * 40);  // [16]
  float* l_s = corr_s + LATENT_PAIRS;                             // [16]
  griddep_launch();
  griddep_wait();
  const LatentTile tile = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tile.seq];
  const int h0 = blockIdx.y * LATENT_PAIRS;
  const int nh = min(g.heads - h0, LATENT_PAIRS);
  const int npairs = tile.nq * nh;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pos0 = sq.kv_len - sq.q_len + tile.q0;
  const int row0 = sq.q_start + tile.q0;
  // zero once what no copy fills, then fill Q
  {  // all of Q (unused pair rows, k padding); of the two K buffers only the columns behind D (the copies fill the rest)
    uint32_t* z = reinterpret_cast<uint32_t*>(smem_raw);
    for (int i = tid; i < LATENT_PAIRS * LDQ / 2; i += LAT_THREADS) z[i] = 0u;
    const int pad = LDQ - D;
    for (int i = tid; i < 2 * KV_BLOCK * pad; i += LAT_THREADS) Ks[(size_t)(i / pad) * LDQ + D + i % pad] = __float2bfloat16_rn(0.f);
  }
  __syncthreads();
  for (int e = tid; e < npairs * D; e += LAT_THREADS) {
    const int p = e / D, d = e - p * D;
    const int tq = p / nh, h = h0 + p - tq * nh;
    Qs[(size_t)p * LDQ + d] = __float2bfloat16_rn(q_abs[((size_t)(row0 + tq) * g.heads + h) * D + d] * g.scale);
  }
  const int pos_last = pos0 + tile.nq - 1;
  const int kmin = g.window > 0 ? max(0, pos0 - g.window + 1) : 0;
  int blk0 = kmin / KV_BLOCK, blk1 = pos_last / KV_BLOCK;
  // split launches (n_splits > 1, decode-shaped steps): CTA z takes the blocks of ONE fixed split -- LATENT_SPLIT_BLOCKS
  // consecutive blocks, boundaries at multiples of it in the sequence's own block numbering -- and leaves an unnormalised
  // partial (acc, m, l) per pair for latent_attn_merge_kernel
  float* my_part = nullptr;
  if (n_splits > 1) {
    my_part = part + ((((size_t)blockIdx.x * gridDim.y + blockIdx.y) * n_splits + blockIdx.z) * LATENT_PAIRS) * (R + 2);
    const int s_abs = blk0 / LATENT_SPLIT_BLOCKS + blockIdx.z;
    blk0 = max(blk0, s_abs * LATENT_SPLIT_BLOCKS);
    blk1 = min(blk1, s_abs * LATENT_SPLIT_BLOCKS + LATENT_SPLIT_BLOCKS - 1);
    if (blk0 > blk1) {  // nothing in this split (CTA-uniform): an empty partial
      if (tid < npairs) {
        my_part[(size_t)tid * (R + 2) + R] = -FLT_MAX;
        my_part[(size_t)tid * (R + 2) + R + 1] = 0.f;
      }
      return;
    }
  }
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  const int chunks_per_row = D / 8;
  auto load_block = [&](int blk, int st) {
    const bf* src = cache + (size_t)bt[blk] * KV_BLOCK * D;
    bf* dst = Ks + (size_t)st * KV_BLOCK * LDQ;
    for (int c = tid; c < KV_BLOCK * chunks_per_row; c += LAT_THREADS) {
      const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
      lat_cp_async_16(dst + (size_t)r * LDQ + cc * 8, src + (size_t)r * D + cc * 8);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  // softmax rows of this warp (two pairs), as in the FMA kernel
  int prow[2], posq[2];
  bool on[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    prow[u] = warp + u * LAT_WARPS;
    on[u] = prow[u] < npairs;
    posq[u] = on[u] ? pos0 + prow[u] / nh : -1;
  }
  float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.f, 0.f};
  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
  const int KS = (D + 15) / 16, half = warp >> 2, ntk = warp & 3;
  const int ks_lo = half == 0 ? 0 : KS / 2, ks_hi = half == 0 ? KS / 2 : KS;
  const int gq = lane >> 2, t2 = (lane & 3) * 2;

  load_block(blk0, 0);
  for (int blk = blk0; blk <= blk1; ++blk) {
    const int st = (blk - blk0) & 1;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();  // block `blk` has landed for everyone; everyone is done with the other buffer, P, S and corr
    if (blk < blk1) load_block(blk + 1, st ^ 1);
    const bf* Kb = Ks + (size_t)st * KV_BLOCK * LDQ;
    {  // ---- scores: this warp's 8 keys over its half of the row length
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      for (int ks = ks_lo; ks < ks_hi; ++ks) {
        uint32_t a[4], b[2];
        lat_ldsm_x4(a, Qs + (size_t)(lane & 15) * LDQ + ks * 16 + (lane >> 4) * 8);
        lat_ldsm_x2(b, Kb + (size_t)(ntk * 8 + (lane & 7)) * LDQ + ks * 16 + ((lane >> 3) & 1) * 8);
        lat_mma(c, a, b[0], b[1]);
      }
      float* sp = Sp + (size_t)half * LATENT_PAIRS * 33;
      sp[gq * 33 + ntk * 8 + t2] = c[0];
      sp[gq * 33 + ntk * 8 + t2 + 1] = c[1];
      sp[(gq + 8) * 33 + ntk * 8 + t2] = c[2];
      sp[(gq + 8) * 33 + ntk * 8 + t2 + 1] = c[3];
    }
    __syncthreads();
    {  // ---- softmax: rows warp and warp + 8, lane = key
      const int kp = blk * KV_BLOCK + lane;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = prow[u];
        const bool vis = on[u] && kp <= posq[u] && (g.window <= 0 || posq[u] - kp < g.window);
        const float sv = vis ? Sp[r * 33 + lane] + Sp[(LATENT_PAIRS + r) * 33 + lane] : -FLT_MAX;
        const float m_new = fmaxf(m_run[u], warp_max_f(sv));
        const float corr = m_new == -FLT_MAX ? 1.f : expf(m_run[u] - m_new);
        const float p = vis ? expf(sv - m_new) : 0.f;
        l_run[u] = l_run[u] * corr + warp_sum_f(p);
        m_run[u] = m_new;
        Ps[r * 40 + lane] = __float2bfloat16_rn(p);
        if (lane == 0) corr_s[r] = corr;
      }
    }
    __syncthreads();
    {  // ---- output: rescale, then O += P C over this warp's column tiles
      const float c_lo = corr_s[gq], c_hi = corr_s[gq + 8];
      uint32_t a0[4], a1[4];
      lat_ldsm_x4(a0, Ps + (size_t)(lane & 15) * 40 + (lane >> 4) * 8);
      lat_ldsm_x4(a1, Ps + (size_t)(lane & 15) * 40 + 16 + (lane >> 4) * 8);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int n0 = (warp + LAT_WARPS * j) * 8;
        if (n0 < R) {
          acc[j][0] *= c_lo; acc[j][1] *= c_lo; acc[j][2] *= c_hi; acc[j][3] *= c_hi;
          uint32_t b[4];
          lat_ldsm_x4_trans(b, Kb + (size_t)lane * LDQ + n0);
          lat_mma(acc[j], a0, b[0], b[1]);
          lat_mma(acc[j], a1, b[2], b[3]);
        }
      }
    }
  }
  if (my_part != nullptr) {
    if (lane == 0)
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if (on[u]) {
          my_part[(size_t)prow[u] * (R + 2) + R] = m_run[u];
          my_part[(size_t)prow[u] * (R + 2) + R + 1] = l_run[u];
        }
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int p = gq + hf * 8;
      if (p >= npairs) continue;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        const int n = (warp + LAT_WARPS * j) * 8 + t2;
        if (n < R) {
          my_part[(size_t)p * (R + 2) + n] = acc[j][hf * 2];
          my_part[(size_t)p * (R + 2) + n + 1] = acc[j][hf * 2 + 1];
        }
      }
    }
    return;
  }
  if (lane == 0) {
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (on[u]) l_s[prow[u]] = l_run[u] + (g.sink != nullptr ? expf(g.sink[h0 + prow[u] % nh] - m_run[u]) : 0.f);
  }
  __syncthreads();
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int p = gq + hf * 8;
    if (p >= npairs) continue;
    const int tq = p / nh, h = h0 + p - tq * nh;
    const size_t o = ((size_t)(row0 + tq) * g.heads + h) * R;
    const float inv = 1.f / l_s[p];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int n = (warp + LAT_WARPS * j) * 8 + t2;
      if (n < R) {
        st_any(o_lat, o_dtype, o + n, acc[j][hf * 2] * inv);
        st_any(o_lat, o_dtype, o + n + 1, acc[j][hf * 2 + 1] * inv);
      }
    }
  }
}

// o_lat[pair] = sum_z e^(m_z - M) acc_z / sum_z e^(m_z - M) l_z over the splits in ascending order, M = max_z m_z.
// One CTA per (tile, head group, pair); the split weights are worked out once in shared memory.
constexpr int LATENT_MAX_SPLITS = 64;
__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_merge_kernel(const float* __restrict__ part, int n_splits, const AttnSeq* __restrict__ seqs,
                         const LatentTile* __restrict__ tiles, void* __restrict__ o_lat, int o_dtype, LatentGeom g) {
  __shared__ float w_s[LATENT_MAX_SPLITS];
  __shared__ float inv_s;
  griddep_launch();
  griddep_wait();
  const int R = g.kv_rank;
  const LatentTile tile = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tile.seq];
  const int h0 = blockIdx.y * LATENT_PAIRS;
  const int nh = min(g.heads - h0, LATENT_PAIRS);
  const int p = blockIdx.z;
  if (p >= tile.nq * nh) return;
  const float* base = part + (((size_t)blockIdx.x * gridDim.y + blockIdx.y) * n_splits * LATENT_PAIRS + p) * (R + 2);
  const size_t zs = (size_t)LATENT_PAIRS * (R + 2);  // floats between consecutive splits of one pair
  if (threadIdx.x < 32) {  // one warp: lane z, z + 32 (n_splits <= 64)
    float m[2], l[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int z = threadIdx.x + 32 * u;
      l[u] = z < n_splits ? base[z * zs + R + 1] : 0.f;
      m[u] = l[u] > 0.f ? base[z * zs + R] : -FLT_MAX;
    }
    const float M = warp_max_f(fmaxf(m[0], m[1]));
    float den = 0.f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const float w = l[u] > 0.f ? expf(m[u] - M) : 0.f;
      if (threadIdx.x + 32 * u < n_splits) w_s[threadIdx.x + 32 * u] = w;
      den += w * l[u];
    }
    den = warp_sum_f(den);
    if (g.sink != nullptr) den += expf(g.sink[h0 + p % nh] - M);
    if (threadIdx.x == 0) inv_s = 1.f / den;
  }
  __syncthreads();
  const int tq = p / nh, h = h0 + p - tq * nh;
  const size_t o = ((size_t)(sq.q_start + tile.q0 + tq) * g.heads + h) * R;
  for (int d = threadIdx.x; d < R; d += LAT_THREADS) {
    float num = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      const float w = w_s[z];
      if (w > 0.f) num = fmaf(w, base[z * zs + d], num);
    }
    st_any(o_lat, o_dtype, o + d, num * inv_s);
  }
}

template <int NT>
cudaError_t launch_attn_mma(const float* q_abs, const void* cache, const AttnSeq* seqs, const LatentTile* tiles, int n_tiles,
                            const int32_t* block_table, int bt_stride, void* o_lat, int o_dtype, const LatentGeom& g,
                            cudaStream_t stream, float* part = nullptr, int n_splits = 1) {
  const size_t smem = lat_mma_smem(g.row());
  static size_t attr_bytes = 0;
  if (smem > 48 * 1024 && smem > attr_bytes) {
    const cudaError_t e = cudaFuncSetAttribute(latent_attn_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes = smem;
  }
  const dim3 grid(n_tiles, (g.heads + LATENT_PAIRS - 1) / LATENT_PAIRS, n_splits);
  const cudaError_t e = launch_k(latent_attn_mma_kernel<NT>, grid, dim3(LAT_THREADS), smem, stream, q_abs,
                                 reinterpret_cast<const __nv_bfloat16*>(cache), seqs, tiles, block_table, bt_stride, o_lat,
                                 o_dtype, g, part, n_splits);
  if (e != cudaSuccess || n_splits <= 1) return e;
  return launch_k(latent_attn_merge_kernel, dim3(grid.x, grid.y, LATENT_PAIRS), dim3(LAT_THREADS), 0, stream,
                  (const float*)part, n_splits, seqs, tiles, o_lat, o_dtype, g);
}

bool latent_mma_eligible(const void* cache, int dtype, const LatentGeom& g) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TGIS_LATENT_ATTN_MMA");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on && dtype == DT_BF16 && g.row() % 8 == 0 && g.kv_rank % 8 == 0 && g.kv_rank <= 512 &&
         (reinterpret_cast<uintptr_t>(cache) & 15) == 0 && lat_mma_smem(g.row()) <= 200 * 1024;
}

template <class CT, int NACC>
cudaError_t launch_attn(const float* q_abs, const void* cache, const AttnSeq* seqs, const LatentTile* tiles, int n_tiles,
                        const int32_t* block_table, int bt_stride, void* o_lat, int o_dtype, const LatentGeom& g,
                        cudaStream_t stream) {
  const int D = g.row();
  const size_t smem = ((size_t)KV_BLOCK * (D | 1) + (size_t)LATENT_PAIRS * D) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  static size_t attr_bytes = 0;  // per instantiation
  if (smem > 48 * 1024 && smem > attr_bytes) {
    const cudaError_t e = cudaFuncSetAttribute(latent_attn_kernel<CT, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem);
    if (e != cudaSuccess) return e;
    attr_bytes = smem;
  }
  const dim3 grid(n_tiles, (g.heads + LATENT_PAIRS - 1) / LATENT_PAIRS);
  return launch_k(latent_attn_kernel<CT, NACC>, grid, dim3(LAT_THREADS), smem, stream, q_abs,
                  reinterpret_cast<const CT*>(cache), seqs, tiles, block_table, bt_stride, o_lat, o_dtype, g);
}

template <class CT>
cudaError_t launch_attn_ct(const float* q_abs, const void* cache, const AttnSeq* seqs, const LatentTile* tiles, int n_tiles,
                           const int32_t* block_table, int bt_stride, void* o_lat, int o_dtype, const LatentGeom& g,
                           cudaStream_t stream) {
  if (g.kv_rank <= 128) return launch_attn<CT, 4>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream);
  if (g.kv_rank <= 256) return launch_attn<CT, 8>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream);
  if (g.kv_rank <= 512) return launch_attn<CT, 16>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream);
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t latent_prep_launch(const float* y, int ldy, const LatentGeom& g, const float* w_q, const float* w_kv, float eps,
                               const int32_t* positions, const int32_t* slot_mapping, const float* cos_sin, void* cq,
                               void* cache, int dtype, float* gate, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (g.rot_dims > g.rot_dim || (g.rot_dims & 1)) return cudaErrorInvalidValue;
  return launch_k(latent_prep_kernel, dim3(T), dim3(PREP_THREADS), 0, stream, y, ldy, g, w_q, w_kv, eps, positions,
                  slot_mapping, cos_sin, cq, cache, dtype, gate);
}

cudaError_t latent_q_rope_launch(const void* q, int q_dtype, const LatentGeom& g, const int32_t* positions,
                                 const float* cos_sin, float* q_abs, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (q_dtype == DT_BF16)
    return launch_k(latent_q_rope_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream,
                    reinterpret_cast<const __nv_bfloat16*>(q), g, positions, cos_sin, q_abs);
  return launch_k(latent_q_rope_kernel<float>, dim3(T), dim3(128), 0, stream, reinterpret_cast<const float*>(q), g, positions,
                  cos_sin, q_abs);
}

cudaError_t latent_attn_launch(const float* q_abs, const void* cache, int dtype, const AttnSeq* seqs,
                               const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                               void* o_lat, int o_dtype, const LatentGeom& g, cudaStream_t stream, float* split_ws,
                               size_t split_ws_floats, int max_kv_len, int num_sms, int* n_launched) {
  if (n_launched) *n_launched = n_tiles > 0 ? 1 : 0;
  if (n_tiles <= 0) return cudaSuccess;
  if (latent_mma_eligible(cache, dtype, g)) {
    // Steps with too few tiles to fill the GPU (decode-shaped): every tile's key range is cut into fixed splits that run as
    // CTAs of their own.  The split count is a function of the longest sequence rounded up to whole splits (and of the
    // window), so a captured launch stays valid for every step of its CUDA-graph key.
    int n_splits = 1;
    const int hg = (g.heads + LATENT_PAIRS - 1) / LATENT_PAIRS;
    static int split_on = -1;
    if (split_on < 0) {
      const char* e = getenv("TGIS_LATENT_ATTN_SPLIT");
      split_on = (e && e[0] == '0') ? 0 : 1;
    }
    if (split_on && split_ws != nullptr && n_tiles * hg < num_sms) {
      const int split_keys = LATENT_SPLIT_BLOCKS * KV_BLOCK;
      int span = (max_kv_len + split_keys - 1) / split_keys * split_keys;
      if (g.window > 0) span = std::min(span, (g.window + LATENT_PAIRS + split_keys - 1) / split_keys * split_keys);
      const int z = span / split_keys + 1;
      if (z > 2 && z <= LATENT_MAX_SPLITS && (size_t)n_tiles * hg * z * LATENT_PAIRS * (g.kv_rank + 2) <= split_ws_floats)
        n_splits = z;
    }
    if (n_launched && n_splits > 1) *n_launched = 2;  // + the merge kernel
    if (g.kv_rank <= 128) return launch_attn_mma<2>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream, split_ws, n_splits);
    if (g.kv_rank <= 256) return launch_attn_mma<4>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream, split_ws, n_splits);
    return launch_attn_mma<8>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream, split_ws, n_splits);
  }
  if (dtype == DT_BF16)
    return launch_attn_ct<__nv_bfloat16>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream);
  return launch_attn_ct<float>(q_abs, cache, seqs, tiles, n_tiles, block_table, bt_stride, o_lat, o_dtype, g, stream);
}

}  // namespace tgis
