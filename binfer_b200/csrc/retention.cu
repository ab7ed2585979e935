// Retention: linear attention with a fixed decay per head and no softmax,
//
//   S_t = decay_h S_{t-1} + k_t v_t^T        o_t = S_t^T q_t
//
// with q and k turned by a rotary angle of the token's position (the first 2 rot_half
// sizes of a head; k is then multiplied by k_scale).  The state S [dk, dv] per request and
// head is float and lives in the request's state slot, stored column by column
// ([dv][dk]: the dk numbers that one output column needs lie side by side), and is carried
// from step to step, so a prompt can be cut anywhere.
//
// retention_scan: a block owns `cols` output columns of one (request, head); a column is
// shared by KS adjacent lanes that each hold R consecutive state elements in registers.  The
// step's tokens are walked in order, in chunks of RET_CHUNK tokens whose q, k (rotated, in
// float) and v the block stages in shared memory; inside a chunk there is no block barrier,
// only the shuffle that adds the KS partial dot products of a column.  Every sum has an
// order that depends on the sizes alone, so the result does not depend on how the tokens
// were cut into steps.
//
// retention_out: each head's output divided by its root mean square (no weight), times
// silu of the gate projection, times out_scale, into a column block of `out`.
#include "common.cuh"

#define RET_CHUNK 16
#define RET_THREADS 256

template <typename A, int R>
__global__ void __launch_bounds__(RET_THREADS) retention_scan_kernel(
    const A* __restrict__ proj, long long stride, long long q_off, long long k_off,
    long long v_off, const float* __restrict__ decays, const float* __restrict__ inv_freq,
    int rot_half, const int* __restrict__ positions, float* __restrict__ state,
    long long state_stride, const int* __restrict__ q_start, const int* __restrict__ state_slots,
    int n_slots, float* __restrict__ o_raw, int H, int dk, int dv, int KS, float k_scale,
    int* __restrict__ err) {
  extern __shared__ float sh[];
  const int cols = RET_THREADS / KS;
  float* qs = sh;                           // [RET_CHUNK][dkp]
  const int dkp = KS * R;                   // dk rounded up to what the lanes of a column hold
  float* ks_ = qs + RET_CHUNK * dkp;        // [RET_CHUNK][dkp]
  float* vs = ks_ + RET_CHUNK * dkp;        // [RET_CHUNK][cols]
  const int b = blockIdx.z, h = blockIdx.y, col0 = blockIdx.x * cols;
  const int tid = threadIdx.x;
  const int col = col0 + tid / KS, part = tid % KS;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  int slot = state_slots[b];
  if (slot < 0 || slot >= n_slots) {
    if (tid == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  const float decay = decays[h];
  const bool live = col < dv;
  float* sp = state + (size_t)slot * state_stride + ((size_t)h * dv + (live ? col : 0)) * dk +
              (size_t)part * R;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) S[r] = (live && part * R + r < dk) ? sp[r] : 0.f;

  for (int c0 = 0; c0 < n; c0 += RET_CHUNK) {
    const int cn = min(RET_CHUNK, n - c0);
    __syncthreads();                        // the last chunk's readers are done
    for (int idx = tid; idx < cn * dkp; idx += RET_THREADS) {
      const int c = idx / dkp, i = idx % dkp;
      const int t = t0 + c0 + c;
      float qv = 0.f, kv = 0.f;
      if (i < dk) {
        const A* row = proj + (size_t)t * stride + (size_t)h * dk;
        qv = bf_ld(row + q_off + i);
        kv = bf_ld(row + k_off + i);
        if (i < 2 * rot_half) {
          const int m = i < rot_half ? i : i - rot_half;
          const int o = i < rot_half ? i + rot_half : i - rot_half;
          float sn, cs;
          sincosf((float)positions[t] * inv_freq[m], &sn, &cs);
          const float qo = bf_ld(row + q_off + o), ko = bf_ld(row + k_off + o);
          qv = i < rot_half ? qv * cs - qo * sn : qv * cs + qo * sn;
          kv = i < rot_half ? kv * cs - ko * sn : kv * cs + ko * sn;
        }
        kv *= k_scale;
      }
      qs[idx] = qv;
      ks_[idx] = kv;
    }
    for (int idx = tid; idx < cn * cols; idx += RET_THREADS) {
      const int c = idx / cols, j = idx % cols;
      vs[idx] = col0 + j < dv
                    ? bf_ld(proj + (size_t)(t0 + c0 + c) * stride + v_off + (size_t)h * dv + col0 + j)
                    : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < cn; ++c) {
      const float v = vs[c * cols + tid / KS];
      const float* qr = qs + c * dkp + part * R;
      const float* kr = ks_ + c * dkp + part * R;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        S[r] = decay * S[r] + kr[r] * v;
        S[r + 1] = decay * S[r + 1] + kr[r + 1] * v;
        a0 += S[r] * qr[r];
        a1 += S[r + 1] * qr[r + 1];
      }
      float a = a0 + a1;
      for (int o = 1; o < KS; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      if (part == 0 && live) o_raw[(size_t)(t0 + c0 + c) * H * dv + (size_t)h * dv + col] = a;
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r)
      if (part * R + r < dk) sp[r] = S[r];
  }
}

BF_EXPORT int bf_retention_scan(
    const void* proj, long long stride, long long q_off, long long k_off, long long v_off,
    const float* decays, const float* inv_freq, int rot_half, const int* positions, float* state,
    long long state_stride, const int* q_start, const int* state_slots, int n_slots, float* o_raw,
    int B, int H, int dk, int dv, float k_scale, int act_dtype, int* err, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dk <= 0 || dv <= 0 || dk > 1024) return (int)cudaErrorInvalidValue;
  const int R = dk <= 256 ? 8 : 32;
  int KS = 1;
  while (KS * R < dk) KS <<= 1;
  const int cols = RET_THREADS / KS;
  dim3 grid((dv + cols - 1) / cols, H, B);
  const size_t smem = (size_t)(2 * RET_CHUNK * KS * R + RET_CHUNK * cols) * sizeof(float);
#define RET_GO(AT, RR)                                                                        \
  if (smem > 48 * 1024)                                                                        \
    cudaFuncSetAttribute(retention_scan_kernel<AT, RR>,                                        \
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
  retention_scan_kernel<AT, RR><<<grid, RET_THREADS, smem, stream>>>(                          \
      (const AT*)proj, stride, q_off, k_off, v_off, decays, inv_freq, rot_half, positions,     \
      state, state_stride, q_start, state_slots, n_slots, o_raw, H, dk, dv, KS, k_scale, err)
  if (act_dtype == BF_DTYPE_F32) {
    if (R == 8) { RET_GO(float, 8); } else { RET_GO(float, 32); }
  } else {
    if (R == 8) { RET_GO(__nv_bfloat16, 8); } else { RET_GO(__nv_bfloat16, 32); }
  }
#undef RET_GO
  return bf_launch_status();
}

// One warp per (token, head).
template <typename A>
__global__ void retention_out_kernel(const float* __restrict__ o_raw, const A* __restrict__ proj,
                                     long long stride, long long g_off, A* __restrict__ out,
                                     long long out_stride, int T, int H, int dv, float eps,
                                     float out_scale) {
  const long long item = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= (long long)T * H) return;
  const int t = (int)(item / H), h = (int)(item % H);
  const float* o = o_raw + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += o[i] * o[i];
  const float f = rsqrtf(warp_sum(ss) / (float)dv + eps) * out_scale;
  const A* g = proj + (size_t)t * stride + g_off + (size_t)h * dv;
  A* dst = out + (size_t)t * out_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float z = bf_ld(g + i);
    bf_st(dst + i, o[i] * f * (z / (1.f + expf(-z))));
  }
}

BF_EXPORT int bf_retention_out(const float* o_raw, const void* proj, long long stride,
                               long long g_off, void* out, long long out_stride, int T, int H,
                               int dv, float eps, float out_scale, int act_dtype,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = 128;
  const long long blocks = ((long long)T * H * 32 + threads - 1) / threads;
  if (act_dtype == BF_DTYPE_F32)
    retention_out_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const float*)proj, stride, g_off, (float*)out, out_stride, T, H, dv, eps,
        out_scale);
  else
    retention_out_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const __nv_bfloat16*)proj, stride, g_off, (__nv_bfloat16*)out, out_stride, T, H,
        dv, eps, out_scale);
  return bf_launch_status();
}
