// General matrix product  Y = X W^T  for the shapes the tcgen05 kernel does not take: any T / N / K and leading
// dimensions, bf16 or fp32 operands (fp32 accumulation in both cases; fp32 operands are multiplied in true fp32, no TF32),
// three launch geometries
//   dense    one problem,
//   batched  blockIdx.z walks equal problems whose operands lie a fixed stride apart (one problem per attention head),
//   grouped  the rows are cut into segments (seg_off, on the device) and segment g multiplies with weight matrix g
//            (one segment per expert of a mixture-of-experts layer); rows of X may be gathered through an index list,
// and six epilogues (plain store, SwiGLU or GeGLU over interleaved gate/up rows, per-(row, batch) scale, tanh, squared ReLU of
// the row-scaled sum).
//
// Every output element is the sum over k = 0 .. K-1 in ascending order inside one thread, so a row's result depends
// neither on the other rows of the launch nor on where in a segment it landed.
//
// Three kernels: a handful of outputs over long rows (router and gate projections of a decode step) take one warp per
// output (gemm_any_rowdot_kernel); bf16 operands whose rows start on 16-byte boundaries run on the tensor cores
// (gemm_any_mma_kernel);
// everything else -- fp32 operands, odd leading dimensions -- runs on the FMA pipe (a [16 TM x 64] tile per 256-thread CTA,
// TM x 4 outputs per thread, k-blocks of 16 staged through shared memory).  Dense launches that fit the tcgen05 kernel's
// operand layout are routed there by the engine.
#include <cstdint>
#include <cstdlib>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

constexpr int ANY_THREADS = 256;
constexpr int ANY_BN = 64;
constexpr int ANY_BK = 16;

template <class T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st_from_float(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_from_float(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
// act(gate) * up: silu (GEMM_ANY_SWIGLU) or the tanh form of gelu (GEMM_ANY_GEGLU)
__device__ __forceinline__ float glu_pair(int mode, float g, float u) {
  if (mode == GEMM_ANY_SWIGLU) return g / (1.f + expf(-g)) * u;
  return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
}

// max(acc * s, 0)^2 with s the scale of the row's INPUT (GEMM_ANY_RELU2)
__device__ __forceinline__ float relu2_scaled(float acc, float s) {
  const float z = fmaxf(acc * s, 0.f);
  return z * z;
}
__device__ __forceinline__ float relu2_row_scale(const GemmAny& a, int dst) {
  return a.row_scale == nullptr ? 1.f : a.row_scale[a.gather != nullptr ? a.gather[dst] : dst];
}

template <class XT, class WT, class OT, int TM>
__global__ void __launch_bounds__(ANY_THREADS) gemm_any_kernel(GemmAny a) {
  constexpr int BM = 16 * TM;
  __shared__ __align__(16) float Xs[ANY_BK][BM + 4];
  __shared__ __align__(16) float Ws[ANY_BK][ANY_BN + 4];
  __shared__ int row_src[BM], row_dst[BM];
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x;
  // ---- which rows
  int row0, row_end, group = 0;
  if (a.seg_off != nullptr) {
    int t = blockIdx.y;
    for (; group < a.n_groups; ++group) {
      const int cnt = a.seg_off[group + 1] - a.seg_off[group];
      const int nt = (cnt + BM - 1) / BM;
      if (t < nt) break;
      t -= nt;
    }
    if (group >= a.n_groups) return;
    row0 = a.seg_off[group] + t * BM;
    row_end = a.seg_off[group + 1];
  } else {
    row0 = blockIdx.y * BM;
    row_end = a.T;
  }
  if (tid < BM) {
    const int r = row0 + tid;
    int src = -1;
    if (r < row_end) src = a.gather != nullptr ? a.gather[r] / a.gather_div : r;
    row_src[tid] = src;
    row_dst[tid] = r < row_end ? r : -1;
  }
  __syncthreads();
  const int z = blockIdx.z;
  const XT* X = reinterpret_cast<const XT*>(a.X) + (size_t)z * a.x_bs;
  const WT* W = reinterpret_cast<const WT*>(a.W) + (size_t)z * a.w_bs + (size_t)group * a.w_gs;
  OT* Y = reinterpret_cast<OT*>(a.Y) + (size_t)z * a.y_bs;
  const int n0 = blockIdx.x * ANY_BN;
  const int ty = tid / 16, tx = tid % 16;
  float acc[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < a.K; k0 += ANY_BK) {
    // stage the two operand tiles (k fastest in memory; transposed into [k][row] so the FMA loop reads rows of 4)
    for (int e = tid; e < BM * ANY_BK; e += ANY_THREADS) {
      const int r = e / ANY_BK, k = e % ANY_BK;
      const int src = row_src[r];
      float v = 0.f;
      if (src >= 0 && k0 + k < a.K) v = ld_as_float(X + (size_t)src * a.ldx + k0 + k);
      Xs[k][r] = v;
    }
    for (int e = tid; e < ANY_BN * ANY_BK; e += ANY_THREADS) {
      const int n = e / ANY_BK, k = e % ANY_BK;
      float v = 0.f;
      if (n0 + n < a.N && k0 + k < a.K) v = ld_as_float(W + (size_t)(n0 + n) * a.ldw + k0 + k);
      Ws[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < ANY_BK; ++k) {
      float xa[TM];
#pragma unroll
      for (int i = 0; i < TM; ++i) xa[i] = Xs[k][ty * TM + i];
      const float4 wb = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        acc[i][0] = fmaf(xa[i], wb.x, acc[i][0]);
        acc[i][1] = fmaf(xa[i], wb.y, acc[i][1]);
        acc[i][2] = fmaf(xa[i], wb.z, acc[i][2]);
        acc[i][3] = fmaf(xa[i], wb.w, acc[i][3]);
      }
    }
    __syncthreads();
  }
  // ---- epilogue
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int dst = row_dst[ty * TM + i];
    if (dst < 0) continue;
    const int n = n0 + tx * 4;
    if (a.mode == GEMM_ANY_SWIGLU || a.mode == GEMM_ANY_GEGLU) {
      // columns (2j, 2j + 1) = (gate_j, up_j): out[j] = act(gate) * up
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        if (n + j + 1 < a.N) st_from_float(Y + (size_t)dst * a.ldy + (n + j) / 2, glu_pair(a.mode, acc[i][j], acc[i][j + 1]));
      }
    } else if (a.mode == GEMM_ANY_RELU2) {
      const float s = relu2_row_scale(a, dst);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < a.N) st_from_float(Y + (size_t)dst * a.ldy + n + j, relu2_scaled(acc[i][j], s));
    } else {
      const float s = a.mode == GEMM_ANY_ROWSCALE ? a.row_scale[(size_t)dst * a.scale_ld + z] : 1.f;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n + j < a.N) st_from_float(Y + (size_t)dst * a.ldy + n + j, a.mode == GEMM_ANY_TANH ? tanhf(acc[i][j]) : acc[i][j] * s);
    }
  }
}

// ---- tensor-core variant (bf16 operands, 16-byte aligned rows): mma.sync m16n8k16, fp32 accumulators ---------------
// CTA tile 64 or 128 rows x 128 weight rows, k-blocks of 32 in a three-stage cp.async ring (out-of-range rows and the k tail
// are zero-filled by the copy), 8 warps as 2 x 4; operands reach the registers through ldmatrix from rows
// padded to 80 bytes (conflict-free).  Same geometries and epilogues as the FMA kernel; the k order inside an output
// element is fixed (ascending k-blocks, the MMA's own order inside), so a row's result does not depend on its neighbours.
constexpr int MMA_BN = 128, MMA_BK = 32, MMA_LD = MMA_BK + 8;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// MI = 16-row MMA tiles per warp along M: CTA tile (32 MI) rows x 128 weight rows (MI = 2: 64 rows, MI = 4: 128 rows).
// Dynamic shared memory: MMA_STAGES x (32 MI + 128) rows of MMA_LD bf16.
constexpr int MMA_STAGES = 3;
template <int MI>
constexpr size_t mma_smem_bytes() { return (size_t)MMA_STAGES * (32 * MI + MMA_BN) * MMA_LD * 2; }

template <class OT, int MI>
__global__ void __launch_bounds__(ANY_THREADS) gemm_any_mma_kernel(GemmAny a) {
  using bf = __nv_bfloat16;
  constexpr int BM = 32 * MI;
  extern __shared__ __align__(16) unsigned char mma_smem[];
  bf* Xs = reinterpret_cast<bf*>(mma_smem);                 // [stage][BM][MMA_LD]
  bf* Ws = Xs + (size_t)MMA_STAGES * BM * MMA_LD;           // [stage][MMA_BN][MMA_LD]
  __shared__ int row_src[BM], row_dst[BM];
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int row0, row_end, group = 0;
  if (a.seg_off != nullptr) {
    int t = blockIdx.y;
    for (; group < a.n_groups; ++group) {
      const int cnt = a.seg_off[group + 1] - a.seg_off[group];
      const int nt = (cnt + BM - 1) / BM;
      if (t < nt) break;
      t -= nt;
    }
    if (group >= a.n_groups) return;
    row0 = a.seg_off[group] + t * BM;
    row_end = a.seg_off[group + 1];
  } else {
    row0 = blockIdx.y * BM;
    row_end = a.T;
  }
  if (tid < BM) {
    const int r = row0 + tid;
    row_src[tid] = r < row_end ? (a.gather != nullptr ? a.gather[r] / a.gather_div : r) : -1;
    row_dst[tid] = r < row_end ? r : -1;
  }
  __syncthreads();
  const int z = blockIdx.z;
  const bf* X = reinterpret_cast<const bf*>(a.X) + (size_t)z * a.x_bs;
  const bf* W = reinterpret_cast<const bf*>(a.W) + (size_t)z * a.w_bs + (size_t)group * a.w_gs;
  OT* Y = reinterpret_cast<OT*>(a.Y) + (size_t)z * a.y_bs;
  const int n0 = blockIdx.x * MMA_BN;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps, warp tile (16 MI) x 32

  auto stage_load = [&](int st, int k0) {
    bf* xs = Xs + (size_t)st * BM * MMA_LD;
    bf* ws = Ws + (size_t)st * MMA_BN * MMA_LD;
#pragma unroll
    for (int i = 0; i < BM / 64; ++i) {  // X: BM rows x 4 chunks of 8 elements
      const int id = tid + i * ANY_THREADS;
      const int r = id >> 2, c = id & 3;
      const int src = row_src[r];
      const bool ok = src >= 0 && k0 + c * 8 < a.K;
      cp_async_16(xs + (size_t)r * MMA_LD + c * 8, ok ? X + (size_t)src * a.ldx + k0 + c * 8 : X, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // W: 128 rows x 4 chunks
      const int id = tid + i * ANY_THREADS;
      const int n = id >> 2, c = id & 3;
      const bool ok = n0 + n < a.N && k0 + c * 8 < a.K;
      cp_async_16(ws + (size_t)n * MMA_LD + c * 8, ok ? W + (size_t)(n0 + n) * a.ldw + k0 + c * 8 : W, ok);
    }
  };

  float acc[MI][4][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

  const int KB = (a.K + MMA_BK - 1) / MMA_BK;
#pragma unroll
  for (int s = 0; s < MMA_STAGES - 1; ++s) {  // prologue (one commit group per stage, empty ones included)
    if (s < KB) stage_load(s, s * MMA_BK);
    cp_async_commit();
  }
  for (int kb = 0; kb < KB; ++kb) {
    cp_async_wait<MMA_STAGES - 2>();  // k-block kb has landed (for this thread's copies)
    __syncthreads();                  // ... for everyone's; and everyone is done with the stage refilled below
    if (kb + MMA_STAGES - 1 < KB) stage_load((kb + MMA_STAGES - 1) % MMA_STAGES, (kb + MMA_STAGES - 1) * MMA_BK);
    cp_async_commit();
    const bf* xs = Xs + (size_t)(kb % MMA_STAGES) * BM * MMA_LD;
    const bf* ws = Ws + (size_t)(kb % MMA_STAGES) * MMA_BN * MMA_LD;
#pragma unroll
    for (int ks = 0; ks < MMA_BK / 16; ++ks) {
      uint32_t af[MI][4], bfr[2][4];
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
        ldsm_x4(af[mi], xs + (size_t)(wm * 16 * MI + mi * 16 + (lane & 15)) * MMA_LD + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nj = 0; nj < 2; ++nj)
        ldsm_x4(bfr[nj], ws + (size_t)(wn * 32 + nj * 16 + (lane >> 4) * 8 + (lane & 7)) * MMA_LD + ks * 16 + ((lane >> 3) & 1) * 8);
#pragma unroll
      for (int mi = 0; mi < MI; ++mi)
#pragma unroll
        for (int ni = 0; ni < 4; ++ni) mma_bf16_16816(acc[mi][ni], af[mi], bfr[ni >> 1][(ni & 1) * 2], bfr[ni >> 1][(ni & 1) * 2 + 1]);
    }
  }
  // ---- epilogue: a thread holds columns (2t, 2t + 1) of rows g and g + 8 of every 16 x 8 block
  const int g = lane >> 2, t2 = (lane & 3) * 2;
#pragma unroll
  for (int mi = 0; mi < MI; ++mi)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int dst = row_dst[wm * 16 * MI + mi * 16 + g + half * 8];
      if (dst < 0) continue;
      const float s = a.mode == GEMM_ANY_ROWSCALE ? a.row_scale[(size_t)dst * a.scale_ld + z]
                      : a.mode == GEMM_ANY_RELU2  ? relu2_row_scale(a, dst) : 1.f;
#pragma unroll
      for (int ni = 0; ni < 4; ++ni) {
        const int n = n0 + wn * 32 + ni * 8 + t2;
        const float v0 = acc[mi][ni][half * 2], v1 = acc[mi][ni][half * 2 + 1];
        if (a.mode == GEMM_ANY_SWIGLU || a.mode == GEMM_ANY_GEGLU) {
          if (n + 1 < a.N) st_from_float(Y + (size_t)dst * a.ldy + n / 2, glu_pair(a.mode, v0, v1));
        } else if (a.mode == GEMM_ANY_TANH) {
          if (n < a.N) st_from_float(Y + (size_t)dst * a.ldy + n, tanhf(v0));
          if (n + 1 < a.N) st_from_float(Y + (size_t)dst * a.ldy + n + 1, tanhf(v1));
        } else if (a.mode == GEMM_ANY_RELU2) {
          if (n < a.N) st_from_float(Y + (size_t)dst * a.ldy + n, relu2_scaled(v0, s));
          if (n + 1 < a.N) st_from_float(Y + (size_t)dst * a.ldy + n + 1, relu2_scaled(v1, s));
        } else {
          if (n < a.N) st_from_float(Y + (size_t)dst * a.ldy + n, v0 * s);
          if (n + 1 < a.N) st_from_float(Y + (size_t)dst * a.ldy + n + 1, v1 * s);
        }
      }
    }
}

template <class OT, int MI>
cudaError_t launch_mma_mi(const GemmAny& a, cudaStream_t stream) {
  constexpr int BM = 32 * MI;
  static bool attr_set = false;
  if (!attr_set) {
    const cudaError_t e = cudaFuncSetAttribute(gemm_any_mma_kernel<OT, MI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)mma_smem_bytes<MI>());
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int row_tiles = a.seg_off != nullptr ? (a.T + BM - 1) / BM + a.n_groups : (a.T + BM - 1) / BM;
  const dim3 grid((a.N + MMA_BN - 1) / MMA_BN, row_tiles, a.batch > 0 ? a.batch : 1);
  if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
  return launch_k(gemm_any_mma_kernel<OT, MI>, grid, dim3(ANY_THREADS), mma_smem_bytes<MI>(), stream, a);
}

template <class OT>
cudaError_t launch_mma(const GemmAny& a, cudaStream_t stream) {
  // 128-row tiles once the problems (or the average expert segment) are tall enough to fill them
  const int rows = a.seg_off != nullptr ? (a.T + a.n_groups - 1) / (a.n_groups > 0 ? a.n_groups : 1) : a.T;
  return rows > 96 ? launch_mma_mi<OT, 4>(a, stream) : launch_mma_mi<OT, 2>(a, stream);
}

bool mma_eligible(const GemmAny& a) {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("TGIS_GEMM_ANY_MMA");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return on && a.x_dtype == DT_BF16 && a.w_dtype == DT_BF16 && a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 &&
         a.x_bs % 8 == 0 && a.w_bs % 8 == 0 && a.w_gs % 8 == 0 && al16(a.X) && al16(a.W);
}

// ---- few outputs, long rows (a router or gate projection in a decode step): one warp per output element -------------
// lanes stride the reduction (coalesced), fixed shuffle tree at the end; any alignment, any operand types.
template <class XT, class WT, bool VEC8>
__global__ void __launch_bounds__(ANY_THREADS) gemm_any_rowdot_kernel(GemmAny a) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const long long out = (long long)blockIdx.x * (ANY_THREADS / 32) + (threadIdx.x >> 5);
  if (out >= (long long)a.T * a.N) return;
  const int t = (int)(out / a.N), n = (int)(out % a.N);
  const XT* x = reinterpret_cast<const XT*>(a.X) + (size_t)t * a.ldx;
  const WT* w = reinterpret_cast<const WT*>(a.W) + (size_t)n * a.ldw;
  float acc = 0.f;
  if (VEC8) {  // bf16 rows on 16-byte boundaries, K % 8 == 0: 8 elements per load, several loads in flight
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
#pragma unroll 8
    for (int c = lane; c < a.K / 8; c += 32) {
      const uint4 xv = x4[c], wv = w4[c];
      const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 xf = __bfloat1622float2(xp[e]), wf = __bfloat1622float2(wp[e]);
        acc = fmaf(xf.x, wf.x, acc);
        acc = fmaf(xf.y, wf.y, acc);
      }
    }
  } else {
#pragma unroll 4
    for (int k = lane; k < a.K; k += 32) acc = fmaf(ld_as_float(x + k), ld_as_float(w + k), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) reinterpret_cast<float*>(a.Y)[(size_t)t * a.ldy + n] = acc;
}
bool rowdot_eligible(const GemmAny& a) {
  return a.seg_off == nullptr && a.batch <= 1 && a.mode == GEMM_ANY_PLAIN && a.y_dtype == DT_F32 && a.N < 128 &&
         (long long)a.T * a.N <= 8192 && a.K >= 256 && !(a.x_dtype == DT_BF16 && a.w_dtype == DT_F32);
}
template <class XT, class WT, bool VEC8 = false>
cudaError_t launch_rowdot(const GemmAny& a, cudaStream_t stream) {
  const long long outs = (long long)a.T * a.N;
  return launch_k(gemm_any_rowdot_kernel<XT, WT, VEC8>, dim3((unsigned)((outs + ANY_THREADS / 32 - 1) / (ANY_THREADS / 32))),
                  dim3(ANY_THREADS), 0, stream, a);
}

template <class XT, class WT, class OT>
cudaError_t launch_tm(const GemmAny& a, cudaStream_t stream) {
  // rows per tile: 16 for skinny problems (decode steps, small expert segments), 64 otherwise
  const int rows = a.seg_off != nullptr ? (a.T + a.n_groups - 1) / (a.n_groups > 0 ? a.n_groups : 1) : a.T;
  const bool small = rows <= 24;
  const int BM = small ? 16 : 64;
  const int row_tiles = a.seg_off != nullptr ? (a.T + BM - 1) / BM + a.n_groups : (a.T + BM - 1) / BM;
  const dim3 grid((a.N + ANY_BN - 1) / ANY_BN, row_tiles, a.batch > 0 ? a.batch : 1);
  if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
  if (small) return launch_k(gemm_any_kernel<XT, WT, OT, 1>, grid, dim3(ANY_THREADS), 0, stream, a);
  return launch_k(gemm_any_kernel<XT, WT, OT, 4>, grid, dim3(ANY_THREADS), 0, stream, a);
}

}  // namespace

cudaError_t gemm_any_launch(const GemmAny& a, cudaStream_t stream) {
  if (a.T <= 0 || a.N <= 0) return cudaSuccess;
  if (a.K <= 0 || ((a.mode == GEMM_ANY_SWIGLU || a.mode == GEMM_ANY_GEGLU) && (a.N & 1))) return cudaErrorInvalidValue;
  if (a.mode == GEMM_ANY_ROWSCALE && a.row_scale == nullptr) return cudaErrorInvalidValue;
  if (a.gather != nullptr && a.gather_div <= 0) return cudaErrorInvalidValue;
  using bf = __nv_bfloat16;
  if (rowdot_eligible(a)) {
    if (a.x_dtype == DT_BF16) {
      const bool vec = a.K % 8 == 0 && a.ldx % 8 == 0 && a.ldw % 8 == 0 && (reinterpret_cast<uintptr_t>(a.X) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(a.W) & 15) == 0;
      return vec ? launch_rowdot<bf, bf, true>(a, stream) : launch_rowdot<bf, bf>(a, stream);
    }
    return a.w_dtype == DT_BF16 ? launch_rowdot<float, bf>(a, stream) : launch_rowdot<float, float>(a, stream);
  }
  if (mma_eligible(a)) return a.y_dtype == DT_BF16 ? launch_mma<bf>(a, stream) : launch_mma<float>(a, stream);
  const int key = a.x_dtype * 4 + a.w_dtype * 2 + a.y_dtype;  // DT_F32 = 0, DT_BF16 = 1
  switch (key) {
    case 0: return launch_tm<float, float, float>(a, stream);
    case 2: return launch_tm<float, bf, float>(a, stream);
    case 3: return launch_tm<float, bf, bf>(a, stream);
    case 6: return launch_tm<bf, bf, float>(a, stream);
    case 7: return launch_tm<bf, bf, bf>(a, stream);
    default: return cudaErrorInvalidValue;  // (fp32 weights under bf16 activations are not a combination any model uses)
  }
}

}  // namespace tgis
