// Grouped-query attention over a paged cache whose weights are NOT a softmax: a visible key weighs
// sigmoid(scale * q . k + bias_h), every key by itself, nothing is normalised over the keys (kernels.h: SigAttnGeom).
// Queries and keys carry rotary positions on their first rot_dims entries (pairs i, i + rot_dims / 2; the table holds
// cos | sin per position, frequencies and magnitude already scaled by the host), visibility is causal within a window.
//
//   sigattn_prep_kernel   per token: rotation of every query and key head (fp32), cache write of the rotated keys and the values;
//                         a layer that reads another layer's cache rows passes no keys / values and only its queries are made
//   sigattn_mma_kernel    bf16 rows whose sizes fit the MMA tiles: both products on mma.sync m16n8k16, fp32 accumulators
//   sigattn_kernel        fp32 or bf16 rows of any size on the FMA pipe
//
// One CTA per (tile of SIGATTN_TILE query tokens of one sequence, query head).  The sequence's cache blocks are walked in
// ascending order from the first block the tile's window touches; a key outside a query's window weighs exactly zero, so
// a query row's sum depends on its own position and on the 32-token block grid of its sequence only: not on the tile it
// shares with other queries, on the other sequences of the step, or on which physical blocks hold the keys.
// Cache rows: K [num_blocks][KV_BLOCK][kv_heads * dim], V [..][kv_heads * vdim] in the operand type; block ids are the engine's.
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
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// grid (T, ceil((heads + 2 kv_heads) / 4)), 128 threads: one warp per (token, query head | key head | value head)
constexpr int PREP_WARPS = 4;
template <class CT>
__global__ void __launch_bounds__(PREP_WARPS * 32)
sigattn_prep_kernel(const float* __restrict__ y, int ldy, int q_off, int k_off, int v_off, SigAttnGeom g,
                    const float* __restrict__ cos_sin, const int32_t* __restrict__ positions,
                    const int32_t* __restrict__ slot_mapping, CT* __restrict__ q_out, CT* __restrict__ k_cache,
                    CT* __restrict__ v_cache) {
  griddep_launch();
  griddep_wait();
  const bool own_kv = k_off >= 0;
  const int t = blockIdx.x, hh = blockIdx.y * PREP_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (hh >= g.heads + (own_kv ? 2 * g.kv_heads : 0)) return;
  const int slot = slot_mapping[t];
  if (hh < g.heads + g.kv_heads) {
    const bool is_q = hh < g.heads;
    const int h = is_q ? hh : hh - g.heads;
    if (!is_q && slot < 0) return;
    const float* src = y + (size_t)t * ldy + (is_q ? q_off : k_off) + (size_t)h * g.dim;
    CT* dst = is_q ? q_out + ((size_t)t * g.heads + h) * g.dim : k_cache + ((size_t)slot * g.kv_heads + h) * g.dim;
    const int half = g.rot_dims / 2;
    const float* cs = cos_sin + (size_t)positions[t] * g.rot_dims;
    for (int i = lane; i < half; i += 32) {
      const float u = src[i], v = src[i + half], c = cs[i], s = cs[half + i];
      stf(dst + i, u * c - v * s);
      stf(dst + i + half, v * c + u * s);
    }
    for (int i = g.rot_dims + lane; i < g.dim; i += 32) stf(dst + i, src[i]);
  } else if (slot >= 0) {
    const int h = hh - g.heads - g.kv_heads;
    const float* src = y + (size_t)t * ldy + v_off + (size_t)h * g.vdim;
    CT* dst = v_cache + ((size_t)slot * g.kv_heads + h) * g.vdim;
    for (int i = lane; i < g.vdim; i += 32) stf(dst + i, src[i]);
  }
}

constexpr int SA_THREADS = 128, SA_QT = SIGATTN_TILE, SA_CC = SIGATTN_MAX_VDIM / SA_THREADS;
static_assert(SA_QT == 16 && SA_THREADS == 128, "score mapping: 4 warps x 4 queries x 32 keys");

// first cache block that holds a key some query of a tile starting at position pos0 sees
__device__ __forceinline__ int first_block(int pos0, int window) {
  return window > 0 ? max(pos0 - window + 1, 0) / KV_BLOCK : 0;
}

template <class CT, class OT>
__global__ void __launch_bounds__(SA_THREADS)
sigattn_kernel(const CT* __restrict__ q, const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
               const AttnSeq* __restrict__ seqs, const LatentTile* __restrict__ tiles,
               const int32_t* __restrict__ block_table, int bt_stride, const float* __restrict__ head_bias,
               OT* __restrict__ out, SigAttnGeom g) {
  extern __shared__ __align__(16) float sa_smem[];
  const int d = g.dim, dv = g.vdim, ldk = d + 1;
  float* Qs = sa_smem;                        // [SA_QT][d]      scaled queries
  float* Ks = Qs + SA_QT * d;                 // [KV_BLOCK][d+1]
  float* Vs = Ks + KV_BLOCK * ldk;            // [KV_BLOCK][dv]
  float* Ps = Vs + KV_BLOCK * dv;             // [SA_QT][KV_BLOCK]
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int h = blockIdx.y, kvh = h / (g.heads / g.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = sq.q_start + tl.q0;             // first query row of the tile in the flat batch
  const int pos0 = sq.kv_len - sq.q_len + tl.q0;   // its position
  const int nq = tl.nq;
  const float hb = head_bias != nullptr ? head_bias[h] : 0.f;
  for (int i = tid; i < SA_QT * d; i += SA_THREADS) {
    const int qi = i / d, kk = i % d;
    Qs[i] = qi < nq ? ldf(q + ((size_t)(row0 + qi) * g.heads + h) * d + kk) * g.scale : 0.f;
  }
  float acc[SA_QT][SA_CC];
#pragma unroll
  for (int qi = 0; qi < SA_QT; ++qi)
#pragma unroll
    for (int cc = 0; cc < SA_CC; ++cc) acc[qi][cc] = 0.f;
  const int n_blocks = (pos0 + nq - 1) / KV_BLOCK + 1;   // blocks up to the last query's own
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  for (int b = first_block(pos0, g.window); b < n_blocks; ++b) {
    const size_t blk = (size_t)bt[b];
    __syncthreads();   // the previous block's Ks / Vs / Ps are consumed (first pass: Qs complete)
    for (int i = tid; i < KV_BLOCK * d; i += SA_THREADS) {
      const int j = i / d, kk = i % d;
      Ks[j * ldk + kk] = ldf(k_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * d + kk);
    }
    for (int i = tid; i < KV_BLOCK * dv; i += SA_THREADS) {
      const int j = i / dv, cc = i % dv;
      Vs[i] = ldf(v_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * dv + cc);
    }
    __syncthreads();
    // ---- weights: lane = key, this warp's four queries
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * ldk;
    const float* qr = Qs + warp * 4 * d;
    for (int kk = 0; kk < d; ++kk) {
      const float kv = kr[kk];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(qr[i * d + kk], kv, s[i]);
    }
    const int kpos = b * KV_BLOCK + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = warp * 4 + i, dist = pos0 + qi - kpos;
      const bool ok = qi < nq && dist >= 0 && (g.window <= 0 || dist < g.window);
      Ps[qi * KV_BLOCK + lane] = ok ? sigmoid_f(s[i] + hb) : 0.f;
    }
    __syncthreads();
    // ---- weighted sum of the values: thread = value column(s), all queries of the tile
#pragma unroll
    for (int cc = 0; cc < SA_CC; ++cc) {
      const int c = tid + cc * SA_THREADS;
      if (c < dv) {
        for (int j = 0; j < KV_BLOCK; ++j) {
          const float vv = Vs[j * dv + c];
#pragma unroll
          for (int qi = 0; qi < SA_QT; ++qi)
            if (qi < nq) acc[qi][cc] = fmaf(Ps[qi * KV_BLOCK + j], vv, acc[qi][cc]);
        }
      }
    }
  }
#pragma unroll
  for (int cc = 0; cc < SA_CC; ++cc) {
    const int c = tid + cc * SA_THREADS;
    if (c < dv) {
#pragma unroll
      for (int qi = 0; qi < SA_QT; ++qi)
        if (qi < nq) stf(out + ((size_t)(row0 + qi) * g.heads + h) * dv + c, acc[qi][cc]);
    }
  }
}

// ---- tensor-core variant: bf16 queries and cache rows, dim a multiple of 16 (<= 16 MMA_KS), vdim a multiple of 8 (<= 32 MMA_NT).
// The tile's 16 queries are the M rows of both products.  For the weights each of the four warps owns 8 of a block's 32
// keys (the query's A fragments stay in registers for the whole walk; the block after the current one lands in a second
// buffer through cp.async meanwhile); scale, bias, sigmoid and mask are fp32 on the accumulator fragments, the weights
// are rounded to bf16 once for the second product, where each warp owns every fourth group of 8 value columns.  With no
// running maximum or normaliser to agree on, a block costs two barriers.
constexpr int MMA_KS = 8, MMA_NT = 8;
__device__ __forceinline__ void sa_ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sa_ldsm_x2(uint32_t (&r)[2], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void sa_ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void sa_cp_async16(void* smem, const void* gmem) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(gmem) : "memory");
}
__device__ __forceinline__ void sa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(SA_THREADS)
sigattn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                   const __nv_bfloat16* __restrict__ v_cache, const AttnSeq* __restrict__ seqs,
                   const LatentTile* __restrict__ tiles, const int32_t* __restrict__ block_table, int bt_stride,
                   const float* __restrict__ head_bias, __nv_bfloat16* __restrict__ out, SigAttnGeom g) {
  using bf = __nv_bfloat16;
  extern __shared__ __align__(16) uint8_t sam_smem[];
  const int d = g.dim, dv = g.vdim, LDK = d + 8, LDV = dv + 8, LDP = KV_BLOCK + 8;
  bf* Qs = reinterpret_cast<bf*>(sam_smem);            // [16][LDK]
  bf* Ks2 = Qs + SA_QT * LDK;                          // [2][32][LDK]   two blocks: one in use, the next one landing
  bf* Vs2 = Ks2 + 2 * KV_BLOCK * LDK;                  // [2][32][LDV]
  bf* Ps = Vs2 + 2 * KV_BLOCK * LDV;                   // [16][LDP]
  griddep_launch();
  griddep_wait();
  const LatentTile tl = tiles[blockIdx.x];
  const AttnSeq sq = seqs[tl.seq];
  const int h = blockIdx.y, kvh = h / (g.heads / g.kv_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t2 = (lane & 3) * 2;
  const int row0 = sq.q_start + tl.q0, pos0 = sq.kv_len - sq.q_len + tl.q0, nq = tl.nq;
  const int dch = d / 8, vch = dv / 8;   // 16-byte chunks per row
  const float hb = head_bias != nullptr ? head_bias[h] : 0.f;
  for (int i = tid; i < SA_QT * dch; i += SA_THREADS) {
    const int qi = i / dch, ch = i % dch;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qi < nq) v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + qi) * g.heads + h) * d + ch * 8);
    *reinterpret_cast<uint4*>(Qs + qi * LDK + ch * 8) = v;
  }
  __syncthreads();
  const int nks = d / 16;
  uint32_t qa[MMA_KS][4];
#pragma unroll
  for (int ks = 0; ks < MMA_KS; ++ks)
    if (ks < nks) sa_ldsm_x4(qa[ks], Qs + (size_t)(lane & 15) * LDK + ks * 16 + (lane >> 4) * 8);
  float acc[MMA_NT][4];
#pragma unroll
  for (int j = 0; j < MMA_NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
  const int b_lo = first_block(pos0, g.window), n_blocks = (pos0 + nq - 1) / KV_BLOCK + 1;
  const int32_t* bt = block_table + (size_t)sq.block_row * bt_stride;
  // block b's K and V rows -> buffer (b - b_lo) & 1, as 16-byte asynchronous copies (one commit group per block)
  auto fetch = [&](int b) {
    const size_t blk = (size_t)bt[b];
    bf* Kd = Ks2 + (size_t)((b - b_lo) & 1) * KV_BLOCK * LDK;
    bf* Vd = Vs2 + (size_t)((b - b_lo) & 1) * KV_BLOCK * LDV;
    for (int i = tid; i < KV_BLOCK * dch; i += SA_THREADS) {
      const int j = i / dch, ch = i % dch;
      sa_cp_async16(Kd + j * LDK + ch * 8, k_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * d + ch * 8);
    }
    for (int i = tid; i < KV_BLOCK * vch; i += SA_THREADS) {
      const int j = i / vch, ch = i % vch;
      sa_cp_async16(Vd + j * LDV + ch * 8, v_cache + ((blk * KV_BLOCK + j) * g.kv_heads + kvh) * dv + ch * 8);
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
  };
  fetch(b_lo);
  for (int b = b_lo; b < n_blocks; ++b) {
    // the other buffer was last read in the previous pass, which ended with a barrier
    if (b + 1 < n_blocks) {
      fetch(b + 1);
      asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    __syncthreads();   // every thread's copies of block b have landed
    const bf* Ks = Ks2 + (size_t)((b - b_lo) & 1) * KV_BLOCK * LDK;
    const bf* Vs = Vs2 + (size_t)((b - b_lo) & 1) * KV_BLOCK * LDV;
    // ---- weights of this warp's 8 keys
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int ks = 0; ks < MMA_KS; ++ks)
      if (ks < nks) {
        uint32_t kb[2];
        sa_ldsm_x2(kb, Ks + (size_t)(warp * 8 + (lane & 7)) * LDK + ks * 16 + ((lane >> 3) & 1) * 8);
        sa_mma(c, qa[ks], kb[0], kb[1]);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int qi = gq + r * 8;
      float p[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int dist = pos0 + qi - (b * KV_BLOCK + warp * 8 + t2 + e);
        const bool ok = qi < nq && dist >= 0 && (g.window <= 0 || dist < g.window);
        p[e] = ok ? sigmoid_f(fmaf(c[2 * r + e], g.scale, hb)) : 0.f;
      }
      *reinterpret_cast<__nv_bfloat162*>(Ps + qi * LDP + warp * 8 + t2) = __floats2bfloat162_rn(p[0], p[1]);
    }
    __syncthreads();
    // ---- weighted sum of the values: this warp's groups of 8 columns
    uint32_t a0[4], a1[4];
    sa_ldsm_x4(a0, Ps + (size_t)(lane & 15) * LDP + (lane >> 4) * 8);
    sa_ldsm_x4(a1, Ps + (size_t)(lane & 15) * LDP + 16 + (lane >> 4) * 8);
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n0 = (warp + 4 * j) * 8;
      if (n0 < dv) {
        uint32_t vb[4];
        sa_ldsm_x4_trans(vb, Vs + (size_t)lane * LDV + n0);
        sa_mma(acc[j], a0, vb[0], vb[1]);
        sa_mma(acc[j], a1, vb[2], vb[3]);
      }
    }
    __syncthreads();   // this pass's buffers and weights are consumed
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int qi = gq + r * 8;
    if (qi >= nq) continue;
    const size_t row = (size_t)(row0 + qi);
#pragma unroll
    for (int j = 0; j < MMA_NT; ++j) {
      const int n = (warp + 4 * j) * 8 + t2;
      if (n < dv)
        *reinterpret_cast<__nv_bfloat162*>(out + (row * g.heads + h) * dv + n) = __floats2bfloat162_rn(acc[j][2 * r], acc[j][2 * r + 1]);
    }
  }
}

bool sigattn_mma_eligible(const SigAttnGeom& g, const void* q, const void* k_cache, const void* v_cache, const void* out) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TGIS_SIGATTN_MMA");   // 0: the FMA kernel for every shape (A/B and the tests)
    on = (e && e[0] == '0') ? 0 : 1;
  }
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return on == 1 && g.dim % 16 == 0 && g.dim <= 16 * MMA_KS && g.vdim % 8 == 0 && g.vdim <= 32 * MMA_NT && al16(q) &&
         al16(k_cache) && al16(v_cache) && al16(out);
}

size_t sigattn_smem(const SigAttnGeom& g) {
  return ((size_t)SA_QT * g.dim + (size_t)KV_BLOCK * (g.dim + 1) + (size_t)KV_BLOCK * g.vdim + SA_QT * KV_BLOCK) * sizeof(float);
}

template <class CT, class OT>
cudaError_t sigattn_launch_t(const void* q, const void* k_cache, const void* v_cache, const AttnSeq* seqs,
                             const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                             const float* head_bias, void* out, const SigAttnGeom& g, cudaStream_t stream) {
  const size_t smem = sigattn_smem(g);
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    const cudaError_t e = cudaFuncSetAttribute(sigattn_kernel<CT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    smem_set = smem;
  }
  return launch_k(sigattn_kernel<CT, OT>, dim3(n_tiles, g.heads), dim3(SA_THREADS), smem, stream,
                  reinterpret_cast<const CT*>(q), reinterpret_cast<const CT*>(k_cache), reinterpret_cast<const CT*>(v_cache),
                  seqs, tiles, block_table, bt_stride, head_bias, reinterpret_cast<OT*>(out), g);
}

}  // namespace

cudaError_t sigattn_prep_launch(const float* y, int ldy, int q_off, int k_off, int v_off, const SigAttnGeom& g,
                                const float* cos_sin, const int32_t* positions, const int32_t* slot_mapping, void* q_out,
                                void* k_cache, void* v_cache, int dtype, int T, cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if (g.rot_dims < 0 || g.rot_dims > g.dim || (g.rot_dims & 1) || (g.rot_dims > 0 && cos_sin == nullptr)) return cudaErrorInvalidValue;
  const int n = g.heads + (k_off >= 0 ? 2 * g.kv_heads : 0);
  const dim3 grid(T, (n + PREP_WARPS - 1) / PREP_WARPS);
  if (dtype == DT_BF16)
    return launch_k(sigattn_prep_kernel<__nv_bfloat16>, grid, dim3(PREP_WARPS * 32), 0, stream, y, ldy, q_off, k_off, v_off, g,
                    cos_sin, positions, slot_mapping, reinterpret_cast<__nv_bfloat16*>(q_out),
                    reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache));
  return launch_k(sigattn_prep_kernel<float>, grid, dim3(PREP_WARPS * 32), 0, stream, y, ldy, q_off, k_off, v_off, g, cos_sin,
                  positions, slot_mapping, reinterpret_cast<float*>(q_out), reinterpret_cast<float*>(k_cache),
                  reinterpret_cast<float*>(v_cache));
}

cudaError_t sigattn_launch(const void* q, const void* k_cache, const void* v_cache, int dtype, const AttnSeq* seqs,
                           const LatentTile* tiles, int n_tiles, const int32_t* block_table, int bt_stride,
                           const float* head_bias, void* out, int out_dtype, const SigAttnGeom& g, cudaStream_t stream) {
  if (n_tiles <= 0) return cudaSuccess;
  if (g.heads < 1 || g.kv_heads < 1 || g.heads % g.kv_heads != 0 || g.heads > 65535 || g.dim < 1 || g.vdim < 1 ||
      g.vdim > SIGATTN_MAX_VDIM || sigattn_smem(g) > 200 * 1024 || out_dtype != dtype)
    return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  if (dtype == DT_BF16 && sigattn_mma_eligible(g, q, k_cache, v_cache, out)) {
    const size_t smem = ((size_t)(SA_QT + 2 * KV_BLOCK) * (g.dim + 8) + (size_t)2 * KV_BLOCK * (g.vdim + 8) + SA_QT * (KV_BLOCK + 8)) * sizeof(bf);
    static bool attr_set = false;
    if (!attr_set) {
      const cudaError_t e = cudaFuncSetAttribute(sigattn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    return launch_k(sigattn_mma_kernel, dim3(n_tiles, g.heads), dim3(SA_THREADS), smem, stream, reinterpret_cast<const bf*>(q),
                    reinterpret_cast<const bf*>(k_cache), reinterpret_cast<const bf*>(v_cache), seqs, tiles, block_table, bt_stride,
                    head_bias, reinterpret_cast<bf*>(out), g);
  }
  if (dtype == DT_BF16)
    return sigattn_launch_t<bf, bf>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, head_bias, out, g, stream);
  return sigattn_launch_t<float, float>(q, k_cache, v_cache, seqs, tiles, n_tiles, block_table, bt_stride, head_bias, out, g, stream);
}

}  // namespace tgis
