// Mixture of experts: the router and the weighting of the experts' activations.
//
// moe_route, a block per token (or four): logits z = W_router h in float (h in the activation type,
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

// One block per MR_TOKENS tokens: their rows go to shared memory as float; every warp takes a
// slice of the width and, row by row of the router, its share of each token's dot product
// (a router row is fetched once for all the block's tokens); the shares are then added in
// the warps' order, and one warp per token chooses.  A token's sums do not depend on which
// other tokens share its block.
#define MR_TOKENS 4
#define MR_WARPS 8

template <typename A>
__global__ void __launch_bounds__(MR_WARPS * 32) moe_route_kernel(
    const A* __restrict__ h, long long stride, const float* __restrict__ w, int T, int width,
    int E, int top, int shared_gate, int tokens_per_block, float* __restrict__ route_w,
    int* __restrict__ top_ids, float* __restrict__ top_w) {
  extern __shared__ __align__(16) float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * tokens_per_block;
  const int nt = min(tokens_per_block, T - t0);
  const int rows = E + (shared_gate ? 1 : 0);
  const int wp = (width + 3) & ~3;
  float* x = sh;                                   // [MR_TOKENS][wp]
  float* part = sh + (size_t)MR_TOKENS * wp;       // [MR_WARPS][MR_TOKENS][rows]
  float* zs = part + (size_t)MR_WARPS * MR_TOKENS * rows;   // [MR_TOKENS][rows]
  for (int k = 0; k < nt; ++k) {
    const A* src = h + (size_t)(t0 + k) * stride;
#pragma unroll 8
    for (int c = threadIdx.x; c < width; c += blockDim.x) x[(size_t)k * wp + c] = bf_ld(src + c);
  }
  __syncthreads();
  const bool vec = (width & 3) == 0 && (((uintptr_t)w) & 15) == 0;
  // this warp's slice of the width, in units of four columns (or of one without `vec`)
  const int units = vec ? width >> 2 : width;
  const int per = (units + MR_WARPS - 1) / MR_WARPS;
  const int lo = warp * per, hi = min(units, lo + per);
  for (int e = 0; e < rows; ++e) {
    const float* wr = w + (size_t)e * width;
    float a[MR_TOKENS];
#pragma unroll
    for (int k = 0; k < MR_TOKENS; ++k) a[k] = 0.f;
    if (vec) {
      // four pieces of the row a lane at a time, all fetched before any is used: the round
      // trips to L2 overlap (the sums keep the order of a plain walk)
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      for (int c = lo + lane; c < hi; c += 128) {
        float4 p[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          p[u] = c + 32 * u < hi ? w4[c + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (c + 32 * u < hi) {
#pragma unroll
            for (int k = 0; k < MR_TOKENS; ++k) {
              if (k < nt) {
                const float4 q = reinterpret_cast<const float4*>(x + (size_t)k * wp)[c + 32 * u];
                a[k] += p[u].x * q.x;
                a[k] += p[u].y * q.y;
                a[k] += p[u].z * q.z;
                a[k] += p[u].w * q.w;
              }
            }
          }
        }
      }
    } else {
      for (int c = lo + lane; c < hi; c += 32) {
        const float p = wr[c];
#pragma unroll
        for (int k = 0; k < MR_TOKENS; ++k)
          if (k < nt) a[k] += p * x[(size_t)k * wp + c];
      }
    }
#pragma unroll
    for (int k = 0; k < MR_TOKENS; ++k) {
      const float r = warp_sum(a[k]);
      if (lane == 0) part[((size_t)warp * MR_TOKENS + k) * rows + e] = r;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nt * rows; i += blockDim.x) {
    const int k = i / rows, e = i - k * rows;
    float r = 0.f;
    for (int wv = 0; wv < MR_WARPS; ++wv) r += part[((size_t)wv * MR_TOKENS + k) * rows + e];
    zs[(size_t)k * rows + e] = r;
  }
  __syncthreads();
  if (warp >= nt) return;
  const int t = t0 + warp;
  float* z = zs + (size_t)warp * rows;
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
  const int rows = E + (shared_gate ? 1 : 0);
  // few tokens: one a block, so that the step's blocks are many; else a router row serves four
  const int tpb = T >= 4 * 148 ? MR_TOKENS : 1;
  const size_t smem = ((size_t)MR_TOKENS * ((width + 3) & ~3) +
                       (size_t)(MR_WARPS + 1) * MR_TOKENS * rows) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const unsigned blocks = (unsigned)((T + tpb - 1) / tpb);
  if (act_dtype == BF_DTYPE_F32) {
    auto k = moe_route_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<blocks, MR_WARPS * 32, smem, stream>>>((const float*)h, stride, w, T, width, E, top,
                                               shared_gate, tpb, route_w, top_ids, top_w);
  } else {
    auto k = moe_route_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<blocks, MR_WARPS * 32, smem, stream>>>((const __nv_bfloat16*)h, stride, w, T, width, E,
                                               top, shared_gate, tpb, route_w, top_ids, top_w);
  }
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

// bfloat16 with F, ff and the experts' total a multiple of 8: eight columns a thread (they
// belong to one expert), 16-byte loads and stores.
__global__ void moe_act_bf16_vec_kernel(const __nv_bfloat16* __restrict__ gu,
                                        const float* __restrict__ route_w,
                                        __nv_bfloat16* __restrict__ act, int T, int F, int E,
                                        int ff, int rw_cols) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int F8 = F >> 3;
  if (i >= (long long)T * F8) return;
  const int t = (int)(i / F8), c = (int)(i % F8) << 3;
  const int e = c < E * ff ? c / ff : E;
  const float wgt = e < rw_cols ? route_w[(size_t)t * rw_cols + e] : 1.f;
  uint4 out = make_uint4(0u, 0u, 0u, 0u);
  if (wgt != 0.f) {
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + c);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (size_t)t * 2 * F + F + c);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      o2[j] = __floats2bfloat162_rn(g.x / (1.f + expf(-g.x)) * u.x * wgt,
                                    g.y / (1.f + expf(-g.y)) * u.y * wgt);
    }
  }
  *reinterpret_cast<uint4*>(act + (size_t)t * F + c) = out;
}

BF_EXPORT int bf_moe_act(const void* gu, const float* route_w, void* act, int T, int F, int E,
                         int ff, int rw_cols, int act_dtype, cudaStream_t stream) {
  if (T <= 0 || F <= 0) return 0;
  const long long n = (long long)T * F;
  const unsigned blocks = (unsigned)((n + 255) / 256);
  if (act_dtype == BF_DTYPE_BF16 && F % 8 == 0 && ff % 8 == 0 &&
      (((uintptr_t)gu | (uintptr_t)act) & 15) == 0) {
    moe_act_bf16_vec_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, route_w, (__nv_bfloat16*)act, T, F, E, ff, rw_cols);
    return bf_launch_status();
  }
  if (act_dtype == BF_DTYPE_F32)
    moe_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gu, route_w, (float*)act, T,
                                                      F, E, ff, rw_cols);
  else
    moe_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        (const __nv_bfloat16*)gu, route_w, (__nv_bfloat16*)act, T, F, E, ff, rw_cols);
  return bf_launch_status();
}
