// Softmax attention over the paged cache with the pieces that sit between the projection and the
// scores in some designs:
//
//   * a short causal convolution over time on every channel of q, k and v, whose last taps - 1
//     inputs per request are kept in a state slot as a ring indexed by position;
//   * an RMS norm over the whole q projection and over the whole k projection (all heads at once);
//   * a factor on q that grows with the logarithm of the position;
//   * a bias per (distance, head) added to the scaled score, read from a table by distance;
//   * key and value heads of different sizes.
//
// Everything between the projection's stored result and the stored q, k, v is float32; scores,
// softmax and the weighted sum are float32.

#include "common.cuh"

#include <math.h>

// Keys [kv_heads][page_tokens][k_dim] then values [kv_heads][page_tokens][v_dim] per page and cache.
struct PagedCacheKV {
  void* k;
  void* v;
  const int32_t* block_table;
  long long page_stride;
  int table_stride;
  int page_tokens;
  int kv_heads;
  int k_dim;
  int v_dim;
};

__device__ __forceinline__ int cache_page(const PagedCacheKV& c, int seq, int pos) {
  return c.block_table[(long long)seq * c.table_stride + pos / c.page_tokens];
}

// ------------------------------------ convolution + whole-projection norms + cache write (per row)

// u: the step's projection rows [q | k | v] (C = qd + kd + vd channels).  For row t at position p
// of a request whose portion starts at position p0 (row t0):
//   y[c] = sum_j w[c][j] * U(p - taps + 1 + j)[c],  U(x) = 0 for x < 0, the step's own row for
//   x >= p0, and the ring entry x % (taps - 1) of the request's state otherwise.
// Then q = y_q / rms(y_q) * wq * (1 + coef * ln(floor((p + 1) / every) + 1)), k = y_k / rms(y_k) * wk,
// v = y_v; q goes to q_out, k and v into the cache.
template <typename T>
__global__ void __launch_bounds__(512) conv_norm_cache_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ conv_w,
                                       int taps, const float* __restrict__ ring, const float* __restrict__ q_norm_w,
                                       const float* __restrict__ k_norm_w, T* __restrict__ q_out, PagedCacheKV cache,
                                       const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start,
                                       int qd, int kd, int vd, float eps, float temp_coef, int temp_every,
                                       int write_cache) {
  pdl_launch_dependents();
  extern __shared__ float ys[];      // C floats + 32 scratch
  const int C = qd + kd + vd;
  float* scratch = ys + C;
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = row_seq[t], p = positions[t];
  const int slot = seq_slot[seq];
  const int p0 = p - (t - seq_q_start[seq]);
  const int hist = taps - 1;
  const float* ring_slot = ring + (long long)slot * (hist > 0 ? hist : 1) * C;
  float sq_q = 0.0f, sq_k = 0.0f;
  // most rows of a prompt's portion have all their taps inside the step's own rows: no case per tap
  const bool inside = p - hist >= p0;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float y = 0.0f;
    if (inside) {
      const T* col = u + (long long)(t - hist) * u_stride + c;
      const float* w = conv_w + (long long)c * taps;
      for (int j = 0; j < taps; ++j) y += w[j] * to_float(col[(long long)j * u_stride]);
    } else
    for (int j = 0; j < taps; ++j) {
      const int x = p - hist + j;
      if (x < 0) continue;
      float val;
      if (x >= p0) val = to_float(u[(long long)(t - (p - x)) * u_stride + c]);
      else val = ring_slot[(long long)(x % hist) * C + c];
      y += conv_w[(long long)c * taps + j] * val;
    }
    ys[c] = y;
    if (c < qd) sq_q += y * y;
    else if (c < qd + kd) sq_k += y * y;
  }
  const float tq = block_sum(sq_q, scratch);
  const float tk = block_sum(sq_k, scratch);
  const float rq = 1.0f / sqrtf(tq / (float)qd + eps) * (1.0f + temp_coef * logf((float)((p + 1) / temp_every + 1)));
  const float rk = 1.0f / sqrtf(tk / (float)kd + eps);
  const int page = cache_page(cache, seq, p);
  const int in_page = p % cache.page_tokens;
  const int G = cache.kv_heads;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    if (c < qd) {
      q_out[(long long)t * qd + c] = from_float<T>(ys[c] * rq * q_norm_w[c]);
    } else if (write_cache && page >= 0) {
      if (c < qd + kd) {
        const int e = c - qd, g = e / cache.k_dim, d = e - g * cache.k_dim;
        T* dst = (T*)cache.k + (long long)page * cache.page_stride + ((long long)g * cache.page_tokens + in_page) * cache.k_dim + d;
        *dst = from_float<T>(ys[c] * rk * k_norm_w[e]);
      } else {
        const int e = c - qd - kd, g = e / cache.v_dim, d = e - g * cache.v_dim;
        T* dst = (T*)cache.v + (long long)page * cache.page_stride + ((long long)g * cache.page_tokens + in_page) * cache.v_dim + d;
        *dst = from_float<T>(ys[c]);
      }
    }
  }
  (void)G;
}

extern "C" int llm_conv_norm_cache(const void* u, int dtype, long long u_stride, const float* conv_w, int taps,
                                   const float* ring, const float* q_norm_w, const float* k_norm_w, void* q_out,
                                   void* cache_k, void* cache_v, const int32_t* block_table, long long page_stride,
                                   int table_stride, int page_tokens, int kv_heads, int k_dim, int v_dim,
                                   const int32_t* positions, const int32_t* row_seq, const int32_t* seq_slot,
                                   const int32_t* seq_q_start, int n_tokens, int q_heads, float eps, float temp_coef,
                                   int temp_every, int write_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(taps >= 1 && temp_every >= 1, ERR_BAD_SIZE);
  const int qd = q_heads * k_dim, kd = kv_heads * k_dim, vd = kv_heads * v_dim;
  const int C = qd + kd + vd;
  const size_t smem = (size_t)(C + 32) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  const int threads = C >= 2048 ? 512 : (C >= 512 ? 256 : 128);
  PagedCacheKV cache{cache_k, cache_v, block_table, page_stride, table_stride, page_tokens, kv_heads, k_dim, v_dim};
#define LAUNCH(T)                                                                                                 \
  do {                                                                                                            \
    if (smem > 48 * 1024)                                                                                         \
      cudaFuncSetAttribute(conv_norm_cache_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    launch_kernel(conv_norm_cache_kernel<T>, n_tokens, threads, smem, stream, (const T*)u, u_stride, conv_w, taps, \
                  ring, q_norm_w, k_norm_w, (T*)q_out, cache, positions, row_seq, seq_slot, seq_q_start, qd, kd, vd, \
                  eps, temp_coef, temp_every, write_cache);                                                        \
  } while (0)
  if (dtype == DT_F32) LAUNCH(float);
  else if (dtype == DT_BF16) LAUNCH(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}

// The projection rows of each request's last taps - 1 positions go into its ring (entry position %
// (taps - 1)), after the convolution of the step has read the ring.
template <typename T>
__global__ void conv_ring_write_kernel(const T* __restrict__ u, long long u_stride, float* __restrict__ ring, int hist,
                                       int C, const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_kv_len) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = row_seq[t], p = positions[t];
  const int end = seq_kv_len[seq] > 0 ? seq_kv_len[seq] : p + 1;   // an idle row stands for itself
  if (p < end - hist) return;
  float* dst = ring + ((long long)seq_slot[seq] * hist + (p % hist)) * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) dst[c] = to_float(u[(long long)t * u_stride + c]);
}

extern "C" int llm_conv_ring_write(const void* u, int dtype, long long u_stride, float* ring, int taps, int channels,
                                   const int32_t* positions, const int32_t* row_seq, const int32_t* seq_slot,
                                   const int32_t* seq_kv_len, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || taps <= 1) return 0;
  const int threads = channels >= 1024 ? 256 : 128;
  if (dtype == DT_F32)
    launch_kernel(conv_ring_write_kernel<float>, n_tokens, threads, 0, stream, (const float*)u, u_stride, ring,
                  taps - 1, channels, positions, row_seq, seq_slot, seq_kv_len);
  else if (dtype == DT_BF16)
    launch_kernel(conv_ring_write_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16*)u,
                  u_stride, ring, taps - 1, channels, positions, row_seq, seq_slot, seq_kv_len);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------- attention with a distance bias

#define BA_WARPS 4

// One warp per (row, query head).  Keys are walked in blocks of 32 absolute positions (block b
// holds positions 32 b .. 32 b + 31), one key per lane: score = (q . k) * scale +
// bias[head][distance] (with `softcap` > 0 the scaled score first becomes softcap * tanh(score / softcap));
// online softmax over blocks; the value sum with one output channel group
// per lane.  Each sum's order depends on the sizes and on absolute key positions only.
template <typename T>
__global__ void __launch_bounds__(BA_WARPS * 32)
biased_attention_kernel(const T* __restrict__ q, T* __restrict__ out, long long out_stride, PagedCacheKV cache,
                        const float* __restrict__ bias, int bias_len, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ row_seq, int q_heads, int n_tokens, float scale, int window,
                        float out_scale, float softcap) {
  pdl_launch_dependents();
  extern __shared__ float q_sm[];   // [BA_WARPS][k_dim]
  const int dk = cache.k_dim, dv = cache.v_dim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long item = (long long)blockIdx.x * BA_WARPS + warp;
  pdl_wait();
  if (item >= (long long)n_tokens * q_heads) return;
  const int t = (int)(item / q_heads), h = (int)(item - (long long)t * q_heads);
  const int g = h / (q_heads / cache.kv_heads);
  const int seq = row_seq[t], p = positions[t];
  float* qs = q_sm + warp * dk;
  for (int d = lane; d < dk; d += 32) qs[d] = to_float(q[(long long)t * q_heads * dk + (long long)h * dk + d]);
  __syncwarp();
  const int first = window > 0 ? max(0, p - window + 1) : 0;
  const float* bias_h = bias ? bias + (long long)h * bias_len : nullptr;
  float m = -INFINITY, l = 0.0f;
  float acc[8];                      // value channels lane, lane + 32, ... (v_dim <= 256)
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  for (int b = first / 32; b * 32 <= p; ++b) {
    const int key = b * 32 + lane;
    const bool seen = key >= first && key <= p;
    float s = -INFINITY;
    int page = -1;
    if (seen) page = cache_page(cache, seq, key);
    if (seen && page >= 0) {
      const T* kr = (const T*)cache.k + (long long)page * cache.page_stride +
                    ((long long)g * cache.page_tokens + key % cache.page_tokens) * dk;
      float dot = 0.0f;
      for (int d = 0; d < dk; ++d) dot += qs[d] * to_float(kr[d]);
      s = dot * scale;
      if (softcap > 0.0f) s = softcap * tanhf(s / softcap);
      if (bias_h) s += bias_h[min(p - key, bias_len - 1)];
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float w = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + warp_sum(w);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= corr;
    m = m_new;
    const int last = min(31, p - b * 32);
    for (int kk = 0; kk <= last; ++kk) {
      const float wk = __shfl_sync(0xffffffffu, w, kk);
      const int pg = __shfl_sync(0xffffffffu, page, kk);
      if (wk == 0.0f || pg < 0) continue;
      const T* vr = (const T*)cache.v + (long long)pg * cache.page_stride +
                    ((long long)g * cache.page_tokens + (b * 32 + kk) % cache.page_tokens) * dv;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (d < dv) acc[j] += wk * to_float(vr[d]);
      }
    }
  }
  const float inv = l > 0.0f ? out_scale / l : 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = lane + 32 * j;
    if (d < dv) out[(long long)t * out_stride + (long long)h * dv + d] = from_float<T>(acc[j] * inv);
  }
}

extern "C" int llm_biased_attention(const void* q, void* out, int dtype, long long out_stride, void* cache_k,
                                    void* cache_v, const int32_t* block_table, long long page_stride, int table_stride,
                                    int page_tokens, int kv_heads, int k_dim, int v_dim, const float* bias, int bias_len,
                                    const int32_t* positions, const int32_t* row_seq, int q_heads, int n_tokens,
                                    float scale, int window, float out_scale, float softcap, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(v_dim <= 256 && k_dim >= 1 && kv_heads >= 1 && q_heads % kv_heads == 0, ERR_BAD_SIZE);
  LLM_HOST_CHECK(bias == nullptr || bias_len >= 1, ERR_BAD_SIZE);
  const size_t smem = (size_t)BA_WARPS * k_dim * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  PagedCacheKV cache{cache_k, cache_v, block_table, page_stride, table_stride, page_tokens, kv_heads, k_dim, v_dim};
  const long long items = (long long)n_tokens * q_heads;
  const int blocks = (int)((items + BA_WARPS - 1) / BA_WARPS);
  if (dtype == DT_F32)
    launch_kernel(biased_attention_kernel<float>, blocks, BA_WARPS * 32, smem, stream, (const float*)q, (float*)out,
                  out_stride, cache, bias, bias_len, positions, row_seq, q_heads, n_tokens, scale, window, out_scale, softcap);
  else if (dtype == DT_BF16)
    launch_kernel(biased_attention_kernel<__nv_bfloat16>, blocks, BA_WARPS * 32, smem, stream, (const __nv_bfloat16*)q,
                  (__nv_bfloat16*)out, out_stride, cache, bias, bias_len, positions, row_seq, q_heads, n_tokens, scale,
                  window, out_scale, softcap);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
