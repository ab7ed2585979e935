// Norm on a sublayer's output: resid += rmsnorm(y) * w, and the stream as the next sublayer
// reads it.
//
// An arrangement whose sublayers read the residual stream itself and are normed on the way
// back (x <- x + N(sublayer(x))) needs, per sublayer, the norm of the sublayer's output, the
// add into the float stream, and the new stream in the activation type for the products of
// the next sublayer.  One kernel does the three: a block per row, the row of y kept in
// shared memory between the pass that sums the squares and the pass that adds.
//
//   inv = rsqrt(mean(y^2) + eps);  resid[c] += y[c] * inv * w[c];  act[c] = A(resid[c])
//
// `w` is the weight that multiplies (a family whose checkpoints hold the deviation from one adds the
// one when it loads them).  In a float engine `act` is null: the stream is its own reading.
#include "common.cuh"

template <typename A>
__global__ void rmsnorm_add_kernel(float* __restrict__ resid, const A* __restrict__ y,
                                   const float* __restrict__ w, A* __restrict__ act, int H,
                                   float eps) {
  extern __shared__ float sh[];
  float* row = sh;            // H floats
  float* scratch = sh + H;    // 33 floats
  const size_t r = blockIdx.x;
  const A* yr = y + r * H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = bf_ld(yr + c);
    row[c] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  float* x = resid + r * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = x[c] + row[c] * inv * w[c];
    x[c] = v;
    if (act) bf_st(act + r * H + c, v);
  }
}

// bf16 rows, H a multiple of 8: eight elements a thread and trip, 16-byte loads and stores,
// the row of y in registers between the passes.
template <int TRIPS>
__global__ void rmsnorm_add_bf16_vec_kernel(float* __restrict__ resid,
                                            const __nv_bfloat16* __restrict__ y,
                                            const float* __restrict__ w,
                                            __nv_bfloat16* __restrict__ act, int H, float eps) {
  __shared__ float scratch[33];
  const size_t r = blockIdx.x;
  const __nv_bfloat16* yr = y + r * H;
  float v[TRIPS][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < TRIPS; ++k) {
    const int c = (k * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      const uint4 q = *reinterpret_cast<const uint4*>(yr + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        v[k][2 * j] = f.x;
        v[k][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  float* x = resid + r * H;
#pragma unroll
  for (int k = 0; k < TRIPS; ++k) {
    const int c = (k * blockDim.x + threadIdx.x) * 8;
    if (c < H) {
      const float4 wa = *reinterpret_cast<const float4*>(w + c);
      const float4 wb = *reinterpret_cast<const float4*>(w + c + 4);
      float4 a = *reinterpret_cast<const float4*>(x + c);
      float4 b = *reinterpret_cast<const float4*>(x + c + 4);
      a.x += v[k][0] * inv * wa.x; a.y += v[k][1] * inv * wa.y;
      a.z += v[k][2] * inv * wa.z; a.w += v[k][3] * inv * wa.w;
      b.x += v[k][4] * inv * wb.x; b.y += v[k][5] * inv * wb.y;
      b.z += v[k][6] * inv * wb.z; b.w += v[k][7] * inv * wb.w;
      *reinterpret_cast<float4*>(x + c) = a;
      *reinterpret_cast<float4*>(x + c + 4) = b;
      if (act) {
        uint4 q;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
        h[0] = __floats2bfloat162_rn(a.x, a.y);
        h[1] = __floats2bfloat162_rn(a.z, a.w);
        h[2] = __floats2bfloat162_rn(b.x, b.y);
        h[3] = __floats2bfloat162_rn(b.z, b.w);
        *reinterpret_cast<uint4*>(act + r * H + c) = q;
      }
    }
  }
}

BF_EXPORT int bf_rmsnorm_add(float* resid, const void* y, const float* w, void* act, int rows,
                             int H, float eps, int act_dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (act_dtype == BF_DTYPE_BF16 && H % 8 == 0 && H <= 8 * 256 * 4 &&
      ((uintptr_t)resid & 15) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
      ((uintptr_t)act & 15) == 0) {
    const int threads = H >= 2048 ? 256 : 128;
    const int trips = (H / 8 + threads - 1) / threads;
    auto go = [&](auto kern) {
      kern<<<rows, threads, 0, stream>>>(resid, (const __nv_bfloat16*)y, w,
                                         (__nv_bfloat16*)act, H, eps);
      return bf_launch_status();
    };
    if (trips <= 1) return go(rmsnorm_add_bf16_vec_kernel<1>);
    if (trips == 2) return go(rmsnorm_add_bf16_vec_kernel<2>);
    return go(rmsnorm_add_bf16_vec_kernel<4>);
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32) {
    auto k = rmsnorm_add_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<rows, threads, smem, stream>>>(resid, (const float*)y, w, (float*)act, H, eps);
  } else {
    auto k = rmsnorm_add_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<rows, threads, smem, stream>>>(resid, (const __nv_bfloat16*)y, w, (__nv_bfloat16*)act,
                                       H, eps);
  }
  return bf_launch_status();
}

// The float stream in bfloat16, for the first sublayer that reads it (every later reading
// comes out of bf_rmsnorm_add).
__global__ void stream_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                      size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += step) out[i] = __float2bfloat16_rn(x[i]);
}

BF_EXPORT int bf_stream_to_bf16(const float* x, void* out, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  stream_to_bf16_kernel<<<(int)blocks, threads, 0, stream>>>(x, (__nv_bfloat16*)out, (size_t)n);
  return bf_launch_status();
}
