// Windowed attention with mean-pooled blocks of the keys behind the window, rotated values,
// a constant sink and a gate per head: the kernels around its cache, in their plain form.
//
// A query at position p of its request sees the tokens j with p - window < j <= p and,
// beside them, one key and value for every block of `pool` tokens that lies wholly before
// the window: block b (positions b pool .. b pool + pool - 1) is seen when
// b pool + pool - 1 <= p - window.  A block's key is the mean of its tokens' keys as the
// pages hold them, its value the mean of their values; the means live in a paged cache of
// their own (one entry per block) and are written by bf_pool_blocks in the step that
// completes the block.  Tokens and blocks share one softmax, whose denominator may hold a
// constant sink logit that has no value.  window 0: every token, no blocks.
//
// Values are kept rotated by their own position (the angles of a rotary encoding over the
// whole value head); a head's output, the weighted sum of such values, is turned back by the
// query's position before the head's gate multiplies it.
//
// Every sum runs in an order fixed by positions alone (blocks in ascending order in tiles
// of 32, then tokens in tiles of 32 whose edges are multiples of 32 from position 0), so
// the result does not depend on how the tokens were cut into steps or on the batch.
#include <float.h>

#include "common.cuh"

#define APW_MAX_ACC 8   // value head size <= 32 * APW_MAX_ACC

// Turn the pairs of x[0 .. 2 half) by sign * pos * inv_freq[m].  Pairs (m, m + half), or
// (2m, 2m + 1) when interleaved.  One warp; x in shared memory.
__device__ __forceinline__ void apw_rotate(float* x, int half, const float* __restrict__ inv_freq,
                                           float pos, float sign, int interleaved, int lane) {
  for (int m = lane; m < half; m += 32) {
    float s, c;
    sincosf(pos * inv_freq[m], &s, &c);
    s *= sign;
    const int iu = interleaved ? 2 * m : m, iv = interleaved ? 2 * m + 1 : m + half;
    const float u = x[iu], v = x[iv];
    x[iu] = u * c - v * s;
    x[iv] = v * c + u * s;
  }
}

// ------------------------------------------------------ after the projection: q, k, v
// proj rows: [q: nh dk | k: nkv dk | v: nkv dv | ...] (k and v only when the layer keeps a
// cache of its own).  Per-head RMSNorm of q and k (weights of size dk, or none), rotation of
// the first 2 rot_half entries, q to q_out [T, nh dk], k into its pages; v rotated over its
// whole head (v_inv_freq, dv / 2 angles; null: as projected) into its pages.
// Pages: [page][kv head][slot in page][d].  One warp per (token, head).
template <typename A>
__global__ void apw_encode_kernel(
    const A* __restrict__ proj, long long stride, const float* __restrict__ q_w,
    const float* __restrict__ k_w, const float* __restrict__ inv_freq, int rot_half,
    const float* __restrict__ v_inv_freq, int interleaved, const int* __restrict__ positions,
    const int* __restrict__ slots, A* __restrict__ q_out, A* __restrict__ k_cache,
    A* __restrict__ v_cache, int nh, int nkv, int dk, int dv, int page_size,
    long long num_slots, float eps, int* __restrict__ err) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int hh = blockIdx.y * warps + warp;
  if (hh >= nh + 2 * nkv) return;
  const int dmax = dk > dv ? dk : dv;
  float* x = sh + (size_t)warp * dmax;
  const bool is_q = hh < nh, is_k = !is_q && hh < nh + nkv;
  const int d = (is_q || is_k) ? dk : dv;
  const size_t off = is_q ? (size_t)hh * dk
                          : is_k ? (size_t)nh * dk + (size_t)(hh - nh) * dk
                                 : (size_t)(nh + nkv) * dk + (size_t)(hh - nh - nkv) * dv;
  const A* src = proj + (size_t)t * stride + off;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = bf_ld(src + i);
    x[i] = v;
    ss += v * v;
  }
  __syncwarp();
  const float pos = (float)positions[t];
  if (is_q || is_k) {
    const float* w = is_q ? q_w : k_w;
    if (w) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)d + eps);
      for (int i = lane; i < d; i += 32) x[i] = x[i] * inv * w[i];
      __syncwarp();
    }
    if (rot_half > 0) apw_rotate(x, rot_half, inv_freq, pos, 1.f, interleaved, lane);
  } else if (v_inv_freq) {
    apw_rotate(x, dv / 2, v_inv_freq, pos, 1.f, interleaved, lane);
  }
  __syncwarp();
  if (is_q) {
    A* dst = q_out + ((size_t)t * nh + hh) * dk;
    for (int i = lane; i < d; i += 32) bf_st(dst + i, x[i]);
    return;
  }
  const int slot = slots[t];
  if (slot < 0) return;
  if ((long long)slot >= num_slots) {
    if (lane == 0) atomicOr(err, BF_ERR_SLOT);
    return;
  }
  const int h = is_k ? hh - nh : hh - nh - nkv;
  const int page = slot / page_size, so = slot - page * page_size;
  A* dst = (is_k ? k_cache : v_cache) + (((size_t)page * nkv + h) * page_size + so) * d;
  for (int i = lane; i < d; i += 32) bf_st(dst + i, x[i]);
}

BF_EXPORT int bf_apw_encode(const void* proj, long long stride, const float* q_w,
                            const float* k_w, const float* inv_freq, int rot_half,
                            const float* v_inv_freq, int interleaved, const int* positions,
                            const int* slots, void* q_out, void* k_cache, void* v_cache, int T,
                            int nh, int nkv, int dk, int dv, int page_size, long long num_slots,
                            float eps, int act_dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (2 * rot_half > dk || (dv & 1)) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  const int total = nh + 2 * nkv;          // nkv 0: queries only
  dim3 grid(T, (total + warps - 1) / warps);
  const size_t smem = (size_t)warps * (dk > dv ? dk : dv) * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
  if (act_dtype == BF_DTYPE_F32)
    apw_encode_kernel<float><<<grid, warps * 32, smem, stream>>>(
        (const float*)proj, stride, q_w, k_w, inv_freq, rot_half, v_inv_freq, interleaved,
        positions, slots, (float*)q_out, (float*)k_cache, (float*)v_cache, nh, nkv, dk, dv,
        page_size, num_slots, eps, err);
  else
    apw_encode_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)proj, stride, q_w, k_w, inv_freq, rot_half, v_inv_freq,
        interleaved, positions, slots, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, nh, nkv, dk, dv, page_size, num_slots, eps, err);
  return bf_launch_status();
}

// ------------------------------------------------------------ means of completed blocks
// Request b of the batch held ctx_lens[b] - q_len tokens before this step and holds
// ctx_lens[b] after it: the blocks start / pool .. ctx_lens[b] / pool - 1 were completed by
// it.  For each, the mean over its tokens' keys (values), summed in ascending position in
// float, goes to entry `block` of the request's summary pages.
// grid (new blocks at most, kv head, request).
template <typename A>
__global__ void apw_pool_blocks_kernel(
    const A* __restrict__ k_cache, const A* __restrict__ v_cache, A* __restrict__ ks_cache,
    A* __restrict__ vs_cache, const int* __restrict__ q_start, const int* __restrict__ ctx_lens,
    const int* __restrict__ tables, int table_stride, const int* __restrict__ s_tables,
    int s_table_stride, int nkv, int dk, int dv, int page_size, int num_pages, int s_page_size,
    int s_num_pages, int pool, int* __restrict__ err) {
  const int b = blockIdx.z, g = blockIdx.y;
  const int end = ctx_lens[b], start = end - (q_start[b + 1] - q_start[b]);
  const int blk = start / pool + blockIdx.x;
  if (blk >= end / pool) return;
  const int* table = tables + (size_t)b * table_stride;
  const int sp = s_tables[(size_t)b * s_table_stride + blk / s_page_size];
  if (sp < 0 || sp >= s_num_pages) {
    if (threadIdx.x == 0) atomicOr(err, BF_ERR_PAGE);
    return;
  }
  const size_t s_row = ((size_t)sp * nkv + g) * s_page_size + blk % s_page_size;
  for (int c = threadIdx.x; c < dk + dv; c += blockDim.x) {
    const bool key = c < dk;
    const int d = key ? dk : dv, i = key ? c : c - dk;
    const A* cache = key ? k_cache : v_cache;
    float sum = 0.f;
    bool ok = true;
    for (int j = 0; j < pool; ++j) {
      const int pos = blk * pool + j;
      const int lp = pos / page_size;
      const int page = table[lp];
      if (page < 0 || page >= num_pages) {
        ok = false;
        break;
      }
      sum += bf_ld(cache + (((size_t)page * nkv + g) * page_size + (pos - lp * page_size)) * d + i);
    }
    if (!ok) {
      atomicOr(err, BF_ERR_PAGE);
      continue;
    }
    bf_st((key ? ks_cache : vs_cache) + s_row * d + i, sum / (float)pool);
  }
}

BF_EXPORT int bf_apw_pool_blocks(const void* k_cache, const void* v_cache, void* ks_cache,
                                 void* vs_cache, const int* q_start, const int* ctx_lens,
                                 const int* tables, int table_stride, const int* s_tables,
                                 int s_table_stride, int B, int max_new_blocks, int nkv, int dk,
                                 int dv, int page_size, int num_pages, int s_page_size,
                                 int s_num_pages, int pool, int act_dtype, int* err,
                                 cudaStream_t stream) {
  if (B <= 0 || max_new_blocks <= 0) return 0;
  if (pool <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid(max_new_blocks, nkv, B);
  const int threads = 128;
  if (act_dtype == BF_DTYPE_F32)
    apw_pool_blocks_kernel<float><<<grid, threads, 0, stream>>>(
        (const float*)k_cache, (const float*)v_cache, (float*)ks_cache, (float*)vs_cache, q_start,
        ctx_lens, tables, table_stride, s_tables, s_table_stride, nkv, dk, dv, page_size,
        num_pages, s_page_size, s_num_pages, pool, err);
  else
    apw_pool_blocks_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>(
        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)ks_cache,
        (__nv_bfloat16*)vs_cache, q_start, ctx_lens, tables, table_stride, s_tables,
        s_table_stride, nkv, dk, dv, page_size, num_pages, s_page_size, s_num_pages, pool, err);
  return bf_launch_status();
}

// ------------------------------------------------------------------------ the attention
// One warp per (query token, query head).  `gate`: pre-activations, one per (token, head),
// at gate[t * gate_stride + h] (null: no gate).  `has_sink`: exp(sink) joins the denominator.
template <typename A>
__global__ void apw_attention_kernel(
    const A* __restrict__ q, const A* __restrict__ k_cache, const A* __restrict__ v_cache,
    const A* __restrict__ ks_cache, const A* __restrict__ vs_cache,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions,
    const int* __restrict__ tables, int table_stride, const int* __restrict__ s_tables,
    int s_table_stride, const A* __restrict__ gate, long long gate_stride,
    const float* __restrict__ v_inv_freq, int interleaved, A* __restrict__ out, int nh, int nkv,
    int dk, int dv, int page_size, int num_pages, int s_page_size, int s_num_pages, int window,
    int pool, float scale, int has_sink, float sink, int* __restrict__ err) {
  extern __shared__ float sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int t = blockIdx.x;
  const int h = blockIdx.y * warps + warp;
  if (h >= nh) return;
  const int g = h / (nh / nkv);
  const int dmax = dk > dv ? dk : dv;
  float* qs = sh + (size_t)warp * dmax;
  const A* qrow = q + ((size_t)t * nh + h) * dk;
  for (int i = lane; i < dk; i += 32) qs[i] = bf_ld(qrow + i) * scale;
  __syncwarp();

  const int p = positions[t];
  const int b = seq_of_token[t];
  const int* table = tables + (size_t)b * table_stride;
  const int j0 = window > 0 ? max(0, p - window + 1) : 0;
  const int nb = (window > 0 && pool > 0 && p - window + 1 > 0) ? (p - window + 1) / pool : 0;
  const int* s_table = nb > 0 ? s_tables + (size_t)b * s_table_stride : nullptr;
  const int block_tiles = (nb + 31) >> 5;
  const int first_tile = j0 >> 5, last_tile = p >> 5;

  float m = -FLT_MAX, l = 0.f;
  float acc[APW_MAX_ACC];
#pragma unroll
  for (int c = 0; c < APW_MAX_ACC; ++c) acc[c] = 0.f;

  for (int it = 0; it < block_tiles + (last_tile - first_tile + 1); ++it) {
    const bool blocks = it < block_tiles;
    bool valid;
    long long krow = 0, vrow = 0;       // element offsets of this lane's key and value rows
    if (blocks) {
      const int blk = (it << 5) + lane;
      valid = blk < nb;
      if (valid) {
        const int lp = blk / s_page_size;
        const int page = s_table[lp];
        if (page < 0 || page >= s_num_pages) {
          atomicOr(err, BF_ERR_PAGE);
          valid = false;
        } else {
          const long long r = ((long long)page * nkv + g) * s_page_size + (blk - lp * s_page_size);
          krow = r * dk;
          vrow = r * dv;
        }
      }
    } else {
      const int j = ((first_tile + it - block_tiles) << 5) + lane;
      valid = j >= j0 && j <= p;
      if (valid) {
        const int lp = j / page_size;
        const int page = table[lp];
        if (page < 0 || page >= num_pages) {
          atomicOr(err, BF_ERR_PAGE);
          valid = false;
        } else {
          const long long r = ((long long)page * nkv + g) * page_size + (j - lp * page_size);
          krow = r * dk;
          vrow = r * dv;
        }
      }
    }
    const A* kc = blocks ? ks_cache : k_cache;
    const A* vc = blocks ? vs_cache : v_cache;
    float s = -FLT_MAX;
    if (valid) {
      const A* kr = kc + krow;
      float a = 0.f;
#pragma unroll 8
      for (int i = 0; i < dk; ++i) a += qs[i] * bf_ld(kr + i);
      s = a;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);
    const float pj = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int c = 0; c < APW_MAX_ACC; ++c) acc[c] *= corr;
    const unsigned live = __ballot_sync(0xffffffffu, valid);
    for (int jj = 0; jj < 32; ++jj) {
      if (!((live >> jj) & 1u)) continue;
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const long long rb = __shfl_sync(0xffffffffu, vrow, jj);
      const A* vr = vc + rb;
#pragma unroll
      for (int c = 0; c < APW_MAX_ACC; ++c) {
        const int i = lane + 32 * c;
        if (i < dv) acc[c] += pb * bf_ld(vr + i);
      }
    }
  }
  if (has_sink) {                               // in the denominator only
    const float m_new = fmaxf(m, sink);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sink - m_new);
#pragma unroll
    for (int c = 0; c < APW_MAX_ACC; ++c) acc[c] *= corr;
  }
  const float inv = 1.f / l;
  float* os = qs;                               // the query is no longer needed
  __syncwarp();
#pragma unroll
  for (int c = 0; c < APW_MAX_ACC; ++c) {
    const int i = lane + 32 * c;
    if (i < dv) os[i] = acc[c] * inv;
  }
  __syncwarp();
  if (v_inv_freq) {
    apw_rotate(os, dv / 2, v_inv_freq, (float)p, -1.f, interleaved, lane);
    __syncwarp();
  }
  float gt = 1.f;
  if (gate) gt = 1.f / (1.f + expf(-bf_ld(gate + (size_t)t * gate_stride + h)));
  A* o = out + ((size_t)t * nh + h) * dv;
  for (int i = lane; i < dv; i += 32) bf_st(o + i, os[i] * gt);
}

BF_EXPORT int bf_apw_attention(
    const void* q, const void* k_cache, const void* v_cache, const void* ks_cache,
    const void* vs_cache, const int* seq_of_token, const int* positions, const int* tables,
    int table_stride, const int* s_tables, int s_table_stride, const void* gate,
    long long gate_stride, const float* v_inv_freq, int interleaved, void* out, int T, int nh,
    int nkv, int dk, int dv, int page_size, int num_pages, int s_page_size, int s_num_pages,
    int window, int pool, float scale, int has_sink, float sink, int act_dtype, int* err,
    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dv > 32 * APW_MAX_ACC || dk > 1024 || nkv <= 0 || nh % nkv || (dv & 1))
    return (int)cudaErrorInvalidValue;
  if (pool > 0 && window > 0 && !ks_cache) return (int)cudaErrorInvalidValue;
  const int warps = 4;
  dim3 grid(T, (nh + warps - 1) / warps);
  const size_t smem = (size_t)warps * (dk > dv ? dk : dv) * sizeof(float);
  if (act_dtype == BF_DTYPE_F32)
    apw_attention_kernel<float><<<grid, warps * 32, smem, stream>>>(
        (const float*)q, (const float*)k_cache, (const float*)v_cache, (const float*)ks_cache,
        (const float*)vs_cache, seq_of_token, positions, tables, table_stride, s_tables,
        s_table_stride, (const float*)gate, gate_stride, v_inv_freq, interleaved, (float*)out, nh,
        nkv, dk, dv, page_size, num_pages, s_page_size, s_num_pages, window, pool, scale,
        has_sink, sink, err);
  else
    apw_attention_kernel<__nv_bfloat16><<<grid, warps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        (const __nv_bfloat16*)ks_cache, (const __nv_bfloat16*)vs_cache, seq_of_token, positions,
        tables, table_stride, s_tables, s_table_stride, (const __nv_bfloat16*)gate, gate_stride,
        v_inv_freq, interleaved, (__nv_bfloat16*)out, nh, nkv, dk, dv, page_size, num_pages,
        s_page_size, s_num_pages, window, pool, scale, has_sink, sink, err);
  return bf_launch_status();
}
