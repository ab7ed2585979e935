// Mixture of experts: the router and the weighting of the experts' activations.
//
// moe_route, one warp per token: logits z = W_router h in float (h in the activation type,
// the router's rows in float), the `top` largest chosen (the lower index wins a tie), their
// weights the softmax over the chosen logits alone.  It leaves a dense row of weights
// `route_w [T, E (+1)]` (zero for an expert not chosen) beside the chosen ids and weights;
// with a shared expert that has a gate of its own, row E of the router matrix is that gate's
// weight vector and column E receives sigmoid(w_sg . h).
//
// moe_act: for experts whose gate and up projections are stacked into one product
// `gu [T, 2F]` (gate rows of all experts, then up rows; F = E ff + ff_shared), the
// activations of every expert scaled by the token's weight for that expert,
//   act[t, c] = silu(gu[t, c]) * gu[t, F + c] * route_w[t, expert(c)],
// so that one product with the stacked down projections gives the weighted sum.
#include <float.h>

#include "common.cuh"

template <typename A>
__global__ void moe_route_kernel(const A* __restrict__ h, long long stride,
                                 const float* __restrict__ w, int T, int width, int E, int top,
                                 int shared_gate, float* __restrict__ route_w,
                                 int* __restrict__ top_ids, float* __restrict__ top_w) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  const int rows = E + (shared_gate ? 1 : 0);
  float* z = sh + (size_t)warp * rows;
  const A* x = h + (size_t)t * stride;
  for (int e = 0; e < rows; ++e) {
    const float* wr = w + (size_t)e * width;
    float a = 0.f;
    for (int c = lane; c < width; c += 32) a += wr[c] * bf_ld(x + c);
    a = warp_sum(a);
    if (lane == 0) z[e] = a;
  }
  __syncwarp();
  float* rw = route_w + (size_t)t * rows;
  for (int e = lane; e < rows; e += 32) rw[e] = 0.f;
  if (shared_gate && lane == 0) rw[E] = 1.f / (1.f + expf(-z[E]));
  __syncwarp();
  // the `top` largest, one after the other; the first is the softmax's maximum
  float zmax = 0.f, den = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -FLT_MAX;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (z[e] > best) { best = z[e]; at = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (k == 0) zmax = best;
    const float p = expf(best - zmax);
    den += p;
    if (lane == 0) {
      top_ids[(size_t)t * top + k] = at;
      top_w[(size_t)t * top + k] = p;
      z[at] = -FLT_MAX;
    }
    __syncwarp();
  }
  const float inv = 1.f / den;
  if (lane == 0) {
    for (int k = 0; k < top; ++k) {
      const float p = top_w[(size_t)t * top + k] * inv;
      top_w[(size_t)t * top + k] = p;
      rw[top_ids[(size_t)t * top + k]] = p;
    }
  }
}

BF_EXPORT int bf_moe_route(const void* h, long long stride, const float* w, int T, int width,
                           int E, int top, int shared_gate, float* route_w, int* top_ids,
                           float* top_w, int act_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top < 1 || top > E) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const size_t smem = (size_t)warps * (E + 1) * sizeof(float);
  const unsigned blocks = (unsigned)((T + warps - 1) / warps);
  if (act_dtype == BF_DTYPE_F32)
    moe_route_kernel<float><<<blocks, warps * 32, smem, stream>>>(
        (const float*)h, stride, w, T, width, E, top, shared_gate, route_w, top_ids, top_w);
  else
    moe_route_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)h, stride, w, T, width, E, top, shared_gate, route_w, top_ids,
        top_w);
  return bf_launch_status();
}

template <typename A>
__global__ void moe_act_kernel(const A* __restrict__ gu, const float* __restrict__ route_w,
                               A* __restrict__ act, int T, int F, int E, int ff, int rw_cols) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)T * F) return;
  const int t = (int)(i / F), c = (int)(i % F);
  const int e = c < E * ff ? c / ff : E;
  const float wgt = e < rw_cols ? route_w[(size_t)t * rw_cols + e] : 1.f;
  float r = 0.f;
  if (wgt != 0.f) {
    const float g = bf_ld(gu + (size_t)t * 2 * F + c), u = bf_ld(gu + (size_t)t * 2 * F + F + c);
    r = g / (1.f + expf(-g)) * u * wgt;
  }
  bf_st(act + i, r);
}

BF_EXPORT int bf_moe_act(const void* gu, const float* route_w, void* act, int T, int F, int E,
                         int ff, int rw_cols, int act_dtype, cudaStream_t stream) {
  if (T <= 0 || F <= 0) return 0;
  const long long n = (long long)T * F;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == BF_DTYPE_F32)
    moe_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, route_w, (float*)act, T,
                                                      F, E, ff, rw_cols);
  else
    moe_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, route_w, (__nv_bfloat16*)act, T, F, E, ff, rw_cols);
  return bf_launch_status();
}
