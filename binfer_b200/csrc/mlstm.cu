// The matrix memory with exponential gates (mLSTM): gate activations, the recurrence over a
// request's tokens with the state carried in a slot, and the output stage.
//
// Per head, with S [dk, dv], n [dk] and the stabiliser m (all zero for a new request), a
// token with query q, key k, value v and the log gates i (input) and f (forget) does
//
//   m' = max(f + m, i)
//   S' = exp(f + m - m') S + exp(i - m') k v^T        n' = exp(f + m - m') n + exp(i - m') k
//   o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
//
// State, gates and everything after the projections are float in both engine precisions.
// The recurrence runs token by token in one fixed order, so its result does not depend on
// how a prompt was cut into steps or on what else is in the batch.
//
// State layout of one slot: [head][dk * dv (S, row-major) | dk (n) | m | 3 unused].
#include "common.cuh"

// ----------------------------------------------------------------------------- gates
// gates[t, r] for r < heads:  cap tanh((w_r . h_t + b_r) / cap)          (log input gate)
//             for r >= heads: logsigmoid(cap tanh((w_r . h_t + b_r) / cap))  (log forget gate)
// One warp per (token, gate row); cap <= 0 means no cap.
template <typename A>
__global__ void mlstm_gates_kernel(const A* __restrict__ h, long long h_stride,
                                   const A* __restrict__ w, const float* __restrict__ bias,
                                   float* __restrict__ gates, int T, int width, int heads,
                                   float cap) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int n_gates = 2 * heads;
  if (warp >= T * n_gates) return;
  const int t = warp / n_gates, r = warp - t * n_gates;
  const A* x = h + (size_t)t * h_stride;
  const A* wr = w + (size_t)r * width;
  float acc = 0.f;
  for (int c = lane; c < width; c += 32) acc += bf_ld(x + c) * bf_ld(wr + c);
  acc = warp_sum(acc);
  if (lane == 0) {
    float z = acc + (bias ? bias[r] : 0.f);
    if (cap > 0.f) z = cap * tanhf(z / cap);
    if (r >= heads) z = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
    gates[(size_t)t * n_gates + r] = z;
  }
}

BF_EXPORT int bf_mlstm_gates(const void* h, long long h_stride, const void* w, const float* bias,
                             float* gates, int T, int width, int heads, float cap, int act_dtype,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long warps = (long long)T * 2 * heads;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (act_dtype == BF_DTYPE_F32)
    mlstm_gates_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        (const float*)h, h_stride, (const float*)w, bias, gates, T, width, heads, cap);
  else
    mlstm_gates_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)h, h_stride, (const __nv_bfloat16*)w, bias, gates, T, width, heads,
        cap);
  return bf_launch_status();
}

// ------------------------------------------------------------------------ the recurrence
// A block owns 32 columns of one head's S for one request and walks the request's tokens of
// this step.  Thread (warp g, lane c) keeps rows g, g + 4, g + 8, ... of column c in
// registers; n is spread over the block's threads (every block of a head keeps a copy, the
// first one stores it).  Two block barriers a token: the token's q and k are staged; the
// row groups' partial sums of S^T q and n . q are in shared memory.
#define MLSTM_COLS 32
#define MLSTM_GROUPS 4

template <typename A, int MAXJ>
__global__ void __launch_bounds__(MLSTM_COLS * MLSTM_GROUPS) mlstm_scan_kernel(
    const A* __restrict__ proj, long long stride, const float* __restrict__ gates,
    float* __restrict__ state, long long slot_stride, int state_size,
    const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_slots,
    float* __restrict__ o_raw, int H, int dk, int dv, float q_scale, int* __restrict__ err) {
  constexpr int NT = MLSTM_COLS * MLSTM_GROUPS;
  extern __shared__ float sh[];
  float* qs = sh;                    // dk
  float* ks = sh + dk;               // dk
  __shared__ float part[MLSTM_GROUPS][MLSTM_COLS];
  __shared__ float nqs[MLSTM_GROUPS];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int col = blockIdx.x * MLSTM_COLS + lane;
  const int head = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  float* st = state + (size_t)slot * slot_stride + (size_t)head * state_size;
  const bool live = col < dv;
  float S[MAXJ];
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int r = g + MLSTM_GROUPS * j;
    S[j] = (live && r < dk) ? st[(size_t)r * dv + col] : 0.f;
  }
  float* n_st = st + (size_t)dk * dv;
  float nreg[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = threadIdx.x + NT * i;
    nreg[i] = r < dk ? n_st[r] : 0.f;
  }
  float m = n_st[dk];
  const size_t q_off = (size_t)head * dk, k_off = (size_t)H * dk + (size_t)head * dk;
  const size_t v_off = 2 * (size_t)H * dk + (size_t)head * dv + col;
  for (int t = t0; t < t1; ++t) {
    const A* row = proj + (size_t)t * stride;
    for (int r = threadIdx.x; r < dk; r += NT) {
      qs[r] = bf_ld(row + q_off + r) * q_scale;
      ks[r] = bf_ld(row + k_off + r);
    }
    const float vc = live ? bf_ld(row + v_off) : 0.f;
    const float ig = gates[(size_t)t * 2 * H + head], fg = gates[(size_t)t * 2 * H + H + head];
    __syncthreads();
    const float m_new = fmaxf(fg + m, ig);
    const float a = expf(fg + m - m_new), bb = expf(ig - m_new);
    m = m_new;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < MAXJ; ++j) {
      const int r = g + MLSTM_GROUPS * j;
      if (r < dk) {
        S[j] = a * S[j] + bb * (ks[r] * vc);
        acc += S[j] * qs[r];
      }
    }
    part[g][lane] = acc;
    float nq = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = threadIdx.x + NT * i;
      if (r < dk) {
        nreg[i] = a * nreg[i] + bb * ks[r];
        nq += nreg[i] * qs[r];
      }
    }
    nq = warp_sum(nq);
    if (lane == 0) nqs[g] = nq;
    __syncthreads();
    if (g == 0 && live) {
      const float o = (part[0][lane] + part[1][lane]) + (part[2][lane] + part[3][lane]);
      const float dot = (nqs[0] + nqs[1]) + (nqs[2] + nqs[3]);
      const float den = fmaxf(fabsf(dot), expf(-m)) + 1e-6f;
      o_raw[((size_t)t * H + head) * dv + col] = o / den;
    }
  }
#pragma unroll
  for (int j = 0; j < MAXJ; ++j) {
    const int r = g + MLSTM_GROUPS * j;
    if (live && r < dk) st[(size_t)r * dv + col] = S[j];
  }
  if (blockIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = threadIdx.x + NT * i;
      if (r < dk) n_st[r] = nreg[i];
    }
    if (threadIdx.x == 0) n_st[dk] = m;
  }
}

// proj rows are [q: H dk | k: H dk | v: H dv | ...]; gates [T, 2 H] as bf_mlstm_gates leaves
// them; o_raw float [T, H dv].  dk at most 256.
BF_EXPORT int bf_mlstm_scan(const void* proj, long long stride, const float* gates, float* state,
                            long long slot_stride, int state_size, const int* q_start,
                            const int* state_slots, int num_slots, float* o_raw, int B, int H,
                            int dk, int dv, float q_scale, int act_dtype, int* err,
                            cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dk > 64 * MLSTM_GROUPS || dk <= 0 || dv <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((dv + MLSTM_COLS - 1) / MLSTM_COLS, H, B);
  const int threads = MLSTM_COLS * MLSTM_GROUPS;
  const size_t smem = 2 * (size_t)dk * sizeof(float);
#define GO(A, J)                                                                              \
  mlstm_scan_kernel<A, J><<<grid, threads, smem, stream>>>(                                   \
      (const A*)proj, stride, gates, state, slot_stride, state_size, q_start, state_slots,   \
      num_slots, o_raw, H, dk, dv, q_scale, err)
  const int rows = (dk + MLSTM_GROUPS - 1) / MLSTM_GROUPS;
  if (act_dtype == BF_DTYPE_F32) {
    if (rows <= 16) GO(float, 16); else if (rows <= 32) GO(float, 32); else GO(float, 64);
  } else {
    if (rows <= 16) GO(__nv_bfloat16, 16); else if (rows <= 32) GO(__nv_bfloat16, 32);
    else GO(__nv_bfloat16, 64);
  }
#undef GO
  return bf_launch_status();
}

// ------------------------------------------------------------------------- output stage
// out[t, h, c] = o_raw[t, h, c] / rms_h(o_raw[t, h, :]) * norm_w[h dv + c] * sigmoid(gate[t, h dv + c])
// with the gate's pre-activation at column g_off + h dv + c of the projection's row.
// One warp per (token, head).
template <typename A>
__global__ void mlstm_out_kernel(const float* __restrict__ o_raw, const A* __restrict__ proj,
                                 long long stride, long long g_off,
                                 const float* __restrict__ norm_w, A* __restrict__ out, int T,
                                 int H, int dv, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  const float* o = o_raw + ((size_t)t * H + h) * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += o[c] * o[c];
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)dv + eps);
  const A* gr = proj + (size_t)t * stride + g_off + (size_t)h * dv;
  A* dst = out + ((size_t)t * H + h) * dv;
  for (int c = lane; c < dv; c += 32) {
    const float z = bf_ld(gr + c);
    bf_st(dst + c, o[c] * inv * norm_w[(size_t)h * dv + c] / (1.f + expf(-z)));
  }
}

BF_EXPORT int bf_mlstm_out(const float* o_raw, const void* proj, long long stride,
                           long long g_off, const float* norm_w, void* out, int T, int H, int dv,
                           float eps, int act_dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = 128;
  const long long blocks = ((long long)T * H * 32 + threads - 1) / threads;
  if (act_dtype == BF_DTYPE_F32)
    mlstm_out_kernel<float><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const float*)proj, stride, g_off, norm_w, (float*)out, T, H, dv, eps);
  else
    mlstm_out_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, stream>>>(
        o_raw, (const __nv_bfloat16*)proj, stride, g_off, norm_w, (__nv_bfloat16*)out, T, H, dv,
        eps);
  return bf_launch_status();
}
