// Mixture-of-experts bookkeeping: the top-k router and the row lists that turn "token t uses experts ids[t, :]" into
// one contiguous row segment per expert, which the grouped product of gemm_any.cu walks.  The expert products themselves
// are matrix products (gemm_any.cu); the weighted sum of their outputs is part of the sublayer's tail (resid_tail_kernel).
//
// Router arithmetic is fp32 throughout: logits + bias, selection, and the weights of the selected experts: the softmax over
// the selected logits only (MOE_W_SOFTMAX) or each one's own sigmoid (MOE_W_SIGMOID; the order of sigmoid scores is the order
// of the logits).
#include <cfloat>

#include "kernels.h"
#include "launch.cuh"
#include "ptx.cuh"

namespace tgis {
namespace {

constexpr int ROUTE_WARPS = 4;

// one warp per token; dynamic shared memory: ROUTE_WARPS x E floats
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int E, int top,
                 int32_t* __restrict__ ids, float* __restrict__ w, float* __restrict__ side_gate, int T, int weight_mode) {
  extern __shared__ float sm[];
  griddep_launch();
  griddep_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* z = sm + (size_t)warp * E;
  const float* row = logits + (size_t)t * ld;
  for (int e = lane; e < E; e += 32) z[e] = row[e] + (bias ? bias[e] : 0.f);
  if (side_gate != nullptr && lane == 0) side_gate[t] = 1.f / (1.f + expf(-row[E]));
  __syncwarp();
  float my_val = -FLT_MAX;  // lane k keeps the k-th selected logit
  for (int k = 0; k < top; ++k) {
    float best = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == (k & 31)) my_val = best;
    if (lane == 0) {
      ids[(size_t)t * top + k] = bi;
      z[bi] = -FLT_MAX;
    }
    __syncwarp();
  }
  if (weight_mode == MOE_W_SIGMOID) {   // every chosen expert weighs its own sigmoid score; nothing is renormalised
    if (lane < top) w[(size_t)t * top + lane] = 1.f / (1.f + expf(-my_val));
    return;
  }
  // softmax over the selected logits (the first selected one is the largest)
  const float m = __shfl_sync(0xffffffffu, my_val, 0);
  float e = lane < top ? expf(my_val - m) : 0.f;
  float sum = e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane < top) w[(size_t)t * top + lane] = e / sum;
}

// single CTA; dynamic shared memory: 2 E ints
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int32_t* __restrict__ ids, int n, int E, int32_t* __restrict__ seg_off, int32_t* __restrict__ order,
                 int32_t* __restrict__ inv) {
  extern __shared__ int sm_i[];
  int* cnt = sm_i;
  int* cur = sm_i + E;
  griddep_launch();
  griddep_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      seg_off[e] = run;
      cur[e] = run;
      run += cnt[e];
    }
    seg_off[E] = run;
  }
  __syncthreads();
  // the place of a row inside its segment does not enter any result (every row of a grouped product is computed alone)
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cur[ids[i]], 1);
    order[p] = i;
    inv[i] = p;
  }
}

}  // namespace

cudaError_t moe_route_launch(const float* logits, int ld, const float* bias, int E, int top, int32_t* ids, float* w,
                             float* side_gate, int T, cudaStream_t stream, int weight_mode) {
  if (T <= 0) return cudaSuccess;
  if (top < 1 || top > 32 || top > E || (size_t)ROUTE_WARPS * E * 4 > 48 * 1024) return cudaErrorInvalidValue;
  return launch_k(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32),
                  (size_t)ROUTE_WARPS * E * sizeof(float), stream, logits, ld, bias, E, top, ids, w, side_gate, T, weight_mode);
}

cudaError_t moe_align_launch(const int32_t* ids, int T, int top, int E, int32_t* seg_off, int32_t* order, int32_t* inv,
                             cudaStream_t stream) {
  if (T <= 0) return cudaSuccess;
  if ((size_t)2 * E * 4 > 48 * 1024) return cudaErrorInvalidValue;
  return launch_k(moe_align_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, ids, T * top, E, seg_off, order,
                  inv);
}

}  // namespace tgis
