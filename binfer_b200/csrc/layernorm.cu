// Layer norm with weight and bias over the float residual stream, fused with the stream's
// pending adds:  v = x + d1 + d2;  y = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w + b.
//
// One block per row.  The row is summed in float, kept in shared memory between the passes
// (mean, then the mean of the squared deviations: no cancellation), and written back to the
// stream when asked.  `rows` picks the rows to norm (the output is then packed).
#include "common.cuh"

template <typename A>
__global__ void add_layernorm_kernel(float* __restrict__ resid, const A* __restrict__ d1,
                                     const A* __restrict__ d2, const float* __restrict__ w,
                                     const float* __restrict__ b, A* __restrict__ out,
                                     const int* __restrict__ rows, int H, float eps,
                                     int write_back) {
  extern __shared__ float sh[];
  float* row = sh;            // H floats
  float* scratch = sh + H;    // 33 floats
  bf_pdl_trigger();
  bf_pdl_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* x = resid + (size_t)r * H;
  const A* p1 = d1 ? d1 + (size_t)r * H : nullptr;
  const A* p2 = d2 ? d2 + (size_t)r * H : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = x[c];
    if (p1) v += bf_ld(p1 + c);
    if (p2) v += bf_ld(p2 + c);
    row[c] = v;
    if (write_back && (p1 || p2)) x[c] = v;
    s += v;
  }
  const float mean = block_sum(s, scratch) / (float)H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float dlt = row[c] - mean;
    ss += dlt * dlt;
  }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  A* o = out + (size_t)i * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    bf_st(o + c, (row[c] - mean) * inv * w[c] + (b ? b[c] : 0.f));
}

BF_EXPORT int bf_add_layernorm(float* resid, const void* d1, const void* d2, const float* w,
                               const float* b, void* out, const int* rows, int n_rows, int H,
                               float eps, int act_dtype, int write_back, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
  const size_t smem = (size_t)(H + 33) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32) {
    auto k = add_layernorm_kernel<float>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return bf_launch_pdl(k, dim3(n_rows), dim3(threads), smem, stream, resid, (const float*)d1,
                         (const float*)d2, w, b, (float*)out, rows, H, eps, write_back);
  }
  auto k = add_layernorm_kernel<__nv_bfloat16>;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return bf_launch_pdl(k, dim3(n_rows), dim3(threads), smem, stream, resid,
                       (const __nv_bfloat16*)d1, (const __nv_bfloat16*)d2, w, b,
                       (__nv_bfloat16*)out, rows, H, eps, write_back);
}
