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
#include <type_traits>

#include "common.cuh"

// ----------------------------------------------------------------------------- gates
// gates[t, r] for r < heads:  cap tanh((w_r . h_t + b_r) / cap)          (log input gate)
//             for r >= heads: logsigmoid(cap tanh((w_r . h_t + b_r) / cap))  (log forget gate)
// One warp per (token, gate row); cap <= 0 means no cap.  (A warp that takes eight rows of a
// token, so as to read the token's input once, measured five times slower at 2,048 tokens and
// sixteen times slower at 8: too few warps, each a long chain.)
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

// The same recurrence without a block barrier per token.  A warp owns eight columns of S
// and keeps all of their rows among its lanes: lane l has the R consecutive rows l R .. l R +
// R - 1 (R = 4 or 8: key sizes up to 256) of all eight columns, 8 R values of S in
// registers.  A token then costs the lane six 16-byte reads of shared memory (its rows of k
// and q, the warp's eight values of v) for 24 R multiply-adds; the column sums of S^T q
// cross the lanes by a reduce-scatter (each exchange halves the values a lane still
// carries: nine shuffles for eight columns).  Every warp keeps n for itself, in the same
// rows, and walks the gates of a chunk of eight tokens by itself: the running maximum
// sequentially, the three exponentials of token t in lane t.  Tokens are staged eight at a
// time; while a chunk is worked on, the next one's q, k, v and gates are on their way in
// registers.  Arithmetic per token is the same whatever the chunking, so cuts still change
// no bit.  Key sizes: multiples of 8.
#define MLSTM2_CH 8
#define MLSTM2_COLS 32

__device__ __forceinline__ void mlstm_unpack8(const uint4 (&raw)[1], float (&x)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[0]);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(h[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ void mlstm_unpack8(const float4 (&raw)[2], float (&x)[8]) {
  x[0] = raw[0].x; x[1] = raw[0].y; x[2] = raw[0].z; x[3] = raw[0].w;
  x[4] = raw[1].x; x[5] = raw[1].y; x[6] = raw[1].z; x[7] = raw[1].w;
}

template <typename A, int R>
__global__ void __launch_bounds__(128) mlstm_scan2_kernel(
    const A* __restrict__ proj, long long stride, const float* __restrict__ gates,
    float* __restrict__ state, long long slot_stride, int state_size,
    const int* __restrict__ q_start, const int* __restrict__ state_slots, int num_slots,
    float* __restrict__ o_raw, int H, int dk, int dv, float q_scale, int* __restrict__ err) {
  constexpr int PAD = R == 8 ? 4 : 0;              // keeps the lanes' 16-byte reads off each
  constexpr int PITCH = 32 * (R + PAD);            // other's banks
  __shared__ __align__(16) float qs[MLSTM2_CH * PITCH];   // row r at (r / R) (R + PAD) + r % R
  __shared__ __align__(16) float ks[MLSTM2_CH * PITCH];
  __shared__ __align__(16) float vs[MLSTM2_CH * MLSTM2_COLS];
  __shared__ float gs[2 * MLSTM2_CH];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int colw = blockIdx.x * MLSTM2_COLS + warp * 8;    // the warp's first column
  const int head = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int slot = state_slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  float* st = state + (size_t)slot * slot_stride + (size_t)head * state_size;
  const bool whole = colw + 8 <= dv && (dv & 3) == 0;      // all eight columns, 16-byte rows
  float S[R][8];
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int r = lane * R + j;
    if (r < dk && whole) {
      const float4 x = *reinterpret_cast<const float4*>(st + (size_t)r * dv + colw);
      const float4 y = *reinterpret_cast<const float4*>(st + (size_t)r * dv + colw + 4);
      S[j][0] = x.x; S[j][1] = x.y; S[j][2] = x.z; S[j][3] = x.w;
      S[j][4] = y.x; S[j][5] = y.y; S[j][6] = y.z; S[j][7] = y.w;
    } else {
#pragma unroll
      for (int cc = 0; cc < 8; ++cc)
        S[j][cc] = (r < dk && colw + cc < dv) ? st[(size_t)r * dv + colw + cc] : 0.f;
    }
  }
  float* n_st = st + (size_t)dk * dv;
  float nreg[R];
#pragma unroll
  for (int j = 0; j < R; ++j) nreg[j] = lane * R + j < dk ? n_st[lane * R + j] : 0.f;
  float m = n_st[dk];
  const int dk8 = dk >> 3;
  const int items = MLSTM2_CH * 2 * dk8;           // 8-element pieces of a chunk's q and k
  const size_t v_off = 2 * (size_t)H * dk + (size_t)head * dv + (size_t)blockIdx.x * MLSTM2_COLS;
  // rows dk .. 32 R - 1 of every token stay zero
  for (int i = threadIdx.x; i < MLSTM2_CH * PITCH; i += 128) qs[i] = ks[i] = 0.f;

  // this thread's (at most four) 8-element pieces of a chunk's q and k: where each comes
  // from and where its two halves go, worked out once
  int it_tok[4], it_src[4], it_dst[4], it_dst2[4];
  bool it_k[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int i = threadIdx.x + 128 * k;
    const int tok = i / (2 * dk8), rest = i - tok * 2 * dk8;
    const int which = rest / dk8, r = (rest - which * dk8) * 8;
    it_tok[k] = i < items ? tok : MLSTM2_CH;       // MLSTM2_CH: no such piece
    it_src[k] = which * H * dk + head * dk + r;
    it_k[k] = which != 0;
    it_dst[k] = tok * PITCH + (r / R) * (R + PAD) + r % R;
    it_dst2[k] = tok * PITCH + ((r + 4) / R) * (R + PAD) + (r + 4) % R;
  }
  using Raw = typename std::conditional<sizeof(A) == 2, uint4, float4>::type;
  constexpr int RAWS = sizeof(A) == 2 ? 1 : 2;
  Raw raw[4][RAWS];
  float pre_v[2] = {0.f, 0.f}, pre_g = 0.f;
  auto fetch = [&](int tc) {                       // chunk starting at token tc
    const int n = min(MLSTM2_CH, t1 - tc);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (it_tok[k] < n) {
        const Raw* src = reinterpret_cast<const Raw*>(proj + (size_t)(tc + it_tok[k]) * stride +
                                                      it_src[k]);
#pragma unroll
        for (int x = 0; x < RAWS; ++x) raw[k][x] = src[x];
      }
    }
    const int vt = threadIdx.x >> 4, vc = threadIdx.x & 15;
#pragma unroll
    for (int x = 0; x < 2; ++x)
      pre_v[x] = (vt < n && blockIdx.x * MLSTM2_COLS + vc + 16 * x < dv)
                     ? bf_ld(proj + (size_t)(tc + vt) * stride + v_off + vc + 16 * x) : 0.f;
    const int gt = threadIdx.x & 7, gw = threadIdx.x >> 3;      // gw 0: input, 1: forget
    pre_g = (gw < 2 && gt < n) ? gates[(size_t)(tc + gt) * 2 * H + gw * H + head] : 0.f;
  };
  auto stage = [&](int n) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (it_tok[k] < n) {
        float x[8];
        mlstm_unpack8(raw[k], x);
        const float f = it_k[k] ? 1.f : q_scale;
        float* dst = it_k[k] ? ks : qs;
        *reinterpret_cast<float4*>(dst + it_dst[k]) =
            make_float4(x[0] * f, x[1] * f, x[2] * f, x[3] * f);
        *reinterpret_cast<float4*>(dst + it_dst2[k]) =
            make_float4(x[4] * f, x[5] * f, x[6] * f, x[7] * f);
      }
    }
    vs[(threadIdx.x >> 4) * MLSTM2_COLS + (threadIdx.x & 15)] = pre_v[0];
    vs[(threadIdx.x >> 4) * MLSTM2_COLS + (threadIdx.x & 15) + 16] = pre_v[1];
    if (threadIdx.x < 16) gs[threadIdx.x] = pre_g;
  };

  const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
  const int my_col = colw + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
  if (t0 < t1) fetch(t0);
  __syncthreads();                                 // the zeroed padding is in place
  for (int tc = t0; tc < t1; tc += MLSTM2_CH) {
    const int n = min(MLSTM2_CH, t1 - tc);
    stage(n);
    __syncthreads();
    if (tc + MLSTM2_CH < t1) fetch(tc + MLSTM2_CH);
    // the chunk's gates: m sequentially (every lane the same), then token t's factors in lane t
    float my_a = 1.f, my_b = 0.f, my_e = 1.f;
    {
      float mm = m;
#pragma unroll
      for (int tt = 0; tt < MLSTM2_CH; ++tt) {
        if (tt < n) {
          const float ig = gs[tt], fg = gs[MLSTM2_CH + tt];
          const float m_new = fmaxf(fg + mm, ig);
          if (lane == tt) {
            my_a = fg + mm - m_new;                // exponents for now
            my_b = ig - m_new;
            my_e = -m_new;
          }
          mm = m_new;
        }
      }
      m = mm;
      if (lane < n) {
        my_a = expf(my_a);
        my_b = expf(my_b);
        my_e = expf(my_e);
      }
    }
    const float4* k4 = reinterpret_cast<const float4*>(ks + lane * (R + PAD));
    const float4* q4 = reinterpret_cast<const float4*>(qs + lane * (R + PAD));
#pragma unroll 2
    for (int tt = 0; tt < n; ++tt) {
      const float a = __shfl_sync(0xffffffffu, my_a, tt);
      const float bb = __shfl_sync(0xffffffffu, my_b, tt);
      const float em = __shfl_sync(0xffffffffu, my_e, tt);
      float kr[R], qr[R], kv[8];
#pragma unroll
      for (int j = 0; j < R / 4; ++j) {
        const float4 kk = k4[tt * (PITCH / 4) + j], qq = q4[tt * (PITCH / 4) + j];
        kr[4 * j] = kk.x; kr[4 * j + 1] = kk.y; kr[4 * j + 2] = kk.z; kr[4 * j + 3] = kk.w;
        qr[4 * j] = qq.x; qr[4 * j + 1] = qq.y; qr[4 * j + 2] = qq.z; qr[4 * j + 3] = qq.w;
      }
      {
        const float4 x = *reinterpret_cast<const float4*>(vs + tt * MLSTM2_COLS + warp * 8);
        const float4 y = *reinterpret_cast<const float4*>(vs + tt * MLSTM2_COLS + warp * 8 + 4);
        kv[0] = bb * x.x; kv[1] = bb * x.y; kv[2] = bb * x.z; kv[3] = bb * x.w;
        kv[4] = bb * y.x; kv[5] = bb * y.y; kv[6] = bb * y.z; kv[7] = bb * y.w;
      }
      float acc[8];
      float nq = 0.f;
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) acc[cc] = 0.f;
#pragma unroll
      for (int j = 0; j < R; ++j) {
        nreg[j] = a * nreg[j] + bb * kr[j];
        nq += nreg[j] * qr[j];
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          S[j][cc] = a * S[j][cc] + kv[cc] * kr[j];
          acc[cc] += S[j][cc] * qr[j];
        }
      }
      // column sums over the lanes: each exchange halves what a lane carries
      float h4[4], h2[2], h1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float send = hi16 ? acc[i] : acc[i + 4];
        const float keep = hi16 ? acc[i + 4] : acc[i];
        h4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float send = hi8 ? h4[i] : h4[i + 2];
        const float keep = hi8 ? h4[i + 2] : h4[i];
        h2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
      }
      {
        const float send = hi4 ? h2[0] : h2[1];
        const float keep = hi4 ? h2[1] : h2[0];
        h1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
      }
      h1 += __shfl_xor_sync(0xffffffffu, h1, 2);
      h1 += __shfl_xor_sync(0xffffffffu, h1, 1);
      nq = warp_sum(nq);
      if ((lane & 3) == 0 && my_col < dv) {
        const float den = fmaxf(fabsf(nq), em) + 1e-6f;
        o_raw[((size_t)(tc + tt) * H + head) * dv + my_col] = h1 / den;
      }
    }
    __syncthreads();                               // the chunk is read; the next may be staged
  }
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int r = lane * R + j;
    if (r >= dk) continue;
    if (whole) {
      *reinterpret_cast<float4*>(st + (size_t)r * dv + colw) =
          make_float4(S[j][0], S[j][1], S[j][2], S[j][3]);
      *reinterpret_cast<float4*>(st + (size_t)r * dv + colw + 4) =
          make_float4(S[j][4], S[j][5], S[j][6], S[j][7]);
    } else {
#pragma unroll
      for (int cc = 0; cc < 8; ++cc)
        if (colw + cc < dv) st[(size_t)r * dv + colw + cc] = S[j][cc];
    }
  }
  if (blockIdx.x == 0 && warp == 0) {
#pragma unroll
    for (int j = 0; j < R; ++j)
      if (lane * R + j < dk) n_st[lane * R + j] = nreg[j];
    if (lane == 0) n_st[dk] = m;
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
  if (dk % 8 == 0 && stride % 8 == 0 && ((uintptr_t)proj & 15) == 0 && (H * dk) % 8 == 0 &&
      ((uintptr_t)state & 15) == 0 && slot_stride % 4 == 0 && state_size % 4 == 0) {
    dim3 grid2((dv + MLSTM2_COLS - 1) / MLSTM2_COLS, H, B);
#define GO2(A, J)                                                                             \
  mlstm_scan2_kernel<A, J><<<grid2, 128, 0, stream>>>(                                        \
      (const A*)proj, stride, gates, state, slot_stride, state_size, q_start, state_slots,   \
      num_slots, o_raw, H, dk, dv, q_scale, err)
    if (act_dtype == BF_DTYPE_F32) {
      if (dk <= 128) GO2(float, 4); else GO2(float, 8);
    } else {
      if (dk <= 128) GO2(__nv_bfloat16, 4); else GO2(__nv_bfloat16, 8);
    }
#undef GO2
    return bf_launch_status();
  }
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
