// Attention over a cached latent: per token the cache holds one vector [c | r], c the normed latent
// of `rank` entries from which every head's keys and values are linear maps (k_h = Uk_h c,
// v_h = Uv_h c), r a rotated key part of `rot` entries shared by all heads.  Nothing is expanded per
// cached token: the key map moves to the query side and the value map behind the weighted sum,
//
//   score_h(i, j) = ((Uk_h^T q_h) . c_j + qr_h . r_j) * scale,    o_h = Uv_h (sum_j p_h(i, j) c_j),
//
// so all heads read the same cached vectors (one key/value head of size rank + rot whose first
// `rank` entries are also the value).  The softmax may have a sink: exp(sink_h) joins the
// denominator, with no key and no value.  Scores, weights and sums are float32.
//
// Kernels: latent_prepare (norm of the latent, rotation of r and of the queries' rotated parts,
// cache write), per_head_linear (one small matrix per head applied to every token: the two maps),
// latent_attention (the softmax over the cached vectors).

#include "common.cuh"

#include <math.h>

#define LAT_THREADS 256
#define LAT_WARPS 8
#define LAT_MAX_CH 16      // value entries per lane: rank <= 512

// ------------------------------------------------------------------------------ prepare

// One block per token.  u holds the token's queries at q_col (per head `dim` plain entries, then
// `rot`), c_src its compressed row (`rank` entries to norm, then `rot`; null where the run reads a
// cache that another run wrote).  Rotated entries are paired (2i, 2i + 1), or with `halves`
// (i, i + rot_dims / 2).
template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_THREADS)
latent_prepare_kernel(const T* __restrict__ u, long long u_stride, int q_col, const T* __restrict__ c_src,
                      long long c_stride, int heads, int dim, int rot,
                      int rank, const TW* __restrict__ norm_w, float eps, const float* __restrict__ inv_freq,
                      int rot_dims, int halves, float mag, T* __restrict__ q_full, PagedCache cache,
                      const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int pos = positions[t], seq = row_seq[t];
  const T* row = u + (long long)t * u_stride;
  const int D = rank + rot;
  // the queries' rotated parts, behind the place of the mapped plain parts
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < heads * half; i += blockDim.x) {
    const int h = i / half, p = i - h * half;
    float sn, cs;
    sincosf((float)pos * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const T* x = row + q_col + (long long)h * (dim + rot) + dim;
    const int ia = halves ? p : 2 * p, ib = halves ? p + half : 2 * p + 1;
    const float a = to_float(x[ia]), b = to_float(x[ib]);
    T* dst = q_full + ((long long)t * heads + h) * D + rank;
    dst[ia] = from_float<T>(a * cs - b * sn);
    dst[ib] = from_float<T>(b * cs + a * sn);
  }
  for (int i = threadIdx.x; i < heads * (rot - rot_dims); i += blockDim.x) {
    const int h = i / (rot - rot_dims), c = rot_dims + i - h * (rot - rot_dims);
    q_full[((long long)t * heads + h) * D + rank + c] = row[q_col + (long long)h * (dim + rot) + dim + c];
  }
  // the latent and the shared rotated key part (a run that reads another run's cache has neither)
  if (!write_cache || !c_src) return;
  const T* x = c_src + (long long)t * c_stride;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(x[i]);
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)rank + eps);
  const long long off = cache_offset(cache, seq, pos, 0);
  if (off < 0) return;
  T* dst = (T*)cache.k + off;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<T>(to_float(x[i]) * scale * to_float(norm_w[i]));
  for (int p = threadIdx.x; p < half; p += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[p], &sn, &cs);
    sn *= mag;
    cs *= mag;
    const int ia = rank + (halves ? p : 2 * p), ib = rank + (halves ? p + half : 2 * p + 1);
    const float a = to_float(x[ia]), b = to_float(x[ib]);
    dst[ia] = from_float<T>(a * cs - b * sn);
    dst[ib] = from_float<T>(b * cs + a * sn);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = x[rank + c];
}

extern "C" int llm_latent_prepare(const void* u, int dtype, long long u_stride, int q_col, const void* c_src,
                                  long long c_stride, int heads, int dim,
                                  int rot, int rank, const void* norm_w, float eps, const float* inv_freq, int rot_dims,
                                  int halves, float mag, void* q_full, void* k_base, const int32_t* block_table,
                                  long long page_stride, int table_stride, int page_tokens, const int32_t* positions,
                                  const int32_t* row_seq, int write_cache, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= rot && (rot_dims == 0 || inv_freq), ERR_BAD_SIZE);
  LLM_HOST_CHECK(!write_cache || (c_src && norm_w), ERR_BAD_SIZE);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, rank + rot};
  if (dtype == DT_F32)
    launch_kernel(latent_prepare_kernel<float, float>, n_tokens, LAT_THREADS, 0, stream, (const float*)u, u_stride,
                  q_col, (const float*)c_src, c_stride, heads, dim, rot, rank, (const float*)norm_w, eps, inv_freq,
                  rot_dims, halves, mag, (float*)q_full, c, positions, row_seq, write_cache);
  else if (dtype == DT_BF16)
    launch_kernel(latent_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, n_tokens, LAT_THREADS, 0, stream,
                  (const __nv_bfloat16*)u, u_stride, q_col, (const __nv_bfloat16*)c_src, c_stride, heads, dim, rot, rank,
                  (const __nv_bfloat16*)norm_w, eps, inv_freq, rot_dims, halves, mag, (__nv_bfloat16*)q_full, c,
                  positions, row_seq, write_cache);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------ norm of a latent

// out[t, :] = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w: the norm of a compressed row that a product
// follows (queries that go through a latent of their own).  x may be a column view; a warp per row.
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
rows_rmsnorm_kernel(const T* __restrict__ x, long long x_stride, const TW* __restrict__ w, T* __restrict__ out,
                    long long out_stride, int rows, int width, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* xr = x + (long long)r * x_stride;
  float sq = 0.0f;
  for (int c = lane; c < width; c += 32) {
    const float v = to_float(xr[c]);
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
  for (int c = lane; c < width; c += 32)
    out[(long long)r * out_stride + c] = from_float<T>(to_float(xr[c]) * scale * to_float(w[c]));
}

extern "C" int llm_rows_rmsnorm(const void* x, long long x_stride, const void* w, void* out, long long out_stride,
                                int dtype, int rows, int width, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int blocks = (rows + 3) / 4;
  if (dtype == DT_F32)
    launch_kernel(rows_rmsnorm_kernel<float, float>, blocks, 128, 0, stream, (const float*)x, x_stride, (const float*)w,
                  (float*)out, out_stride, rows, width, eps);
  else if (dtype == DT_BF16)
    launch_kernel(rows_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, blocks, 128, 0, stream, (const __nv_bfloat16*)x,
                  x_stride, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, out_stride, rows, width, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ------------------------------------------------------------------------------ one matrix per head

// out[t, h, o] = sum_i x[t, h, i] * W_h[i, o] for every token t and head h, where head h's matrix is
// rows h * n_in .. of w [heads * n_in, n_out] (W_IN_ROWS: out = x W) or rows h * n_out .. of
// w [heads * n_out, n_in] (out = x W^T).  With `gate`: out *= sigmoid(gate[t, h * n_out + o]).
// A block takes 64 tokens x 64 outputs of one head, a thread 4 x 4 of them; float32 sums in the
// order of i.
#define PH_TILE 64
#define PH_K 16

template <typename T, bool W_IN_ROWS>
__global__ void __launch_bounds__(256)
per_head_linear_kernel(const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w,
                       T* __restrict__ out, long long o_row, long long o_head, const T* __restrict__ gate,
                       long long gate_row, int n_tokens, int n_in, int n_out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float xs[PH_K][PH_TILE + 4];
  __shared__ float ws[PH_K][PH_TILE + 4];
  const int h = blockIdx.z, t0 = blockIdx.x * PH_TILE, o0 = blockIdx.y * PH_TILE;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // tx: outputs, ty: tokens
  const T* wh = w + (long long)h * n_in * n_out;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < n_in; k0 += PH_K) {
    for (int e = threadIdx.x; e < PH_K * PH_TILE; e += 256) {
      {  // x tile: neighbouring threads read neighbouring inputs of one token
        const int kk = e % PH_K, tt = e / PH_K;
        const int t = t0 + tt, k = k0 + kk;
        xs[kk][tt] = (t < n_tokens && k < n_in) ? to_float(x[(long long)t * x_row + (long long)h * x_head + k]) : 0.0f;
      }
      if (W_IN_ROWS) {
        const int oo = e % PH_TILE, kk = e / PH_TILE;
        const int o = o0 + oo, k = k0 + kk;
        ws[kk][oo] = (o < n_out && k < n_in) ? to_float(wh[(long long)k * n_out + o]) : 0.0f;
      } else {
        const int kk = e % PH_K, oo = e / PH_K;
        const int o = o0 + oo, k = k0 + kk;
        ws[kk][oo] = (o < n_out && k < n_in) ? to_float(wh[(long long)o * n_in + k]) : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < PH_K; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = t0 + ty * 4 + i;
    if (t >= n_tokens) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int o = o0 + tx * 4 + j;
      if (o >= n_out) continue;
      float v = acc[i][j];
      if (gate) v = v / (1.0f + expf(-to_float(gate[(long long)t * gate_row + (long long)h * n_out + o])));
      out[(long long)t * o_row + (long long)h * o_head + o] = from_float<T>(v);
    }
  }
}

// The same for a step of few tokens (decoding), where a 64 x 64 tile would leave one thread block per
// head.  The head's inputs of all tokens wait in shared memory as float32.  W_IN_ROWS: grid (head, 64
// outputs); a thread takes one output (neighbouring threads neighbouring outputs of a weight row) and
// a quarter of the inputs, the quarters meet in shared memory.  Else: grid (head, 8 outputs); a warp
// takes one output, its lanes stride over the weight row's inputs.  Sums are float32.
#define PHF_TOKENS 16

template <typename T, bool W_IN_ROWS>
__global__ void __launch_bounds__(256)
per_head_linear_few_kernel(const T* __restrict__ x, long long x_row, long long x_head, const T* __restrict__ w,
                           T* __restrict__ out, long long o_row, long long o_head, const T* __restrict__ gate,
                           long long gate_row, int n_tokens, int n_in, int n_out) {
  pdl_launch_dependents();
  extern __shared__ float phf_smem[];      // x [n_tokens][n_in], then partial sums [4][PHF_TOKENS][64]
  float* xs = phf_smem;
  float* parts = phf_smem + n_tokens * n_in;
  const int h = blockIdx.x, o0 = blockIdx.y * (W_IN_ROWS ? 64 : 8);
  const T* wh = w + (long long)h * n_in * n_out;
  pdl_wait();
  for (int e = threadIdx.x; e < n_tokens * n_in; e += 256) {
    const int t = e / n_in, i = e - t * n_in;
    xs[e] = to_float(x[(long long)t * x_row + (long long)h * x_head + i]);
  }
  __syncthreads();
  float acc[PHF_TOKENS];
#pragma unroll
  for (int t = 0; t < PHF_TOKENS; ++t) acc[t] = 0.0f;
  if (W_IN_ROWS) {
    const int oo = threadIdx.x & 63, part = threadIdx.x >> 6, o = o0 + oo;
    const int per = (n_in + 3) / 4, i0 = part * per, i1 = min(n_in, i0 + per);
    if (o < n_out)
      for (int i = i0; i < i1; ++i) {
        const float wv = to_float(wh[(long long)i * n_out + o]);
#pragma unroll
        for (int t = 0; t < PHF_TOKENS; ++t)
          if (t < n_tokens) acc[t] = fmaf(xs[t * n_in + i], wv, acc[t]);
      }
#pragma unroll
    for (int t = 0; t < PHF_TOKENS; ++t)
      if (t < n_tokens) parts[(part * PHF_TOKENS + t) * 64 + oo] = acc[t];
    __syncthreads();
    for (int e = threadIdx.x; e < n_tokens * 64; e += 256) {
      const int t = e >> 6, c = e & 63, oc = o0 + c;
      if (oc >= n_out) continue;
      float v = (parts[(0 * PHF_TOKENS + t) * 64 + c] + parts[(1 * PHF_TOKENS + t) * 64 + c]) +
                (parts[(2 * PHF_TOKENS + t) * 64 + c] + parts[(3 * PHF_TOKENS + t) * 64 + c]);
      if (gate) v = v / (1.0f + expf(-to_float(gate[(long long)t * gate_row + (long long)h * n_out + oc])));
      out[(long long)t * o_row + (long long)h * o_head + oc] = from_float<T>(v);
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = o0 + warp;
    if (o < n_out) {
      for (int i = lane; i < n_in; i += 32) {
        const float wv = to_float(wh[(long long)o * n_in + i]);
#pragma unroll
        for (int t = 0; t < PHF_TOKENS; ++t)
          if (t < n_tokens) acc[t] = fmaf(xs[t * n_in + i], wv, acc[t]);
      }
#pragma unroll
      for (int t = 0; t < PHF_TOKENS; ++t)
        if (t < n_tokens) {
          float v = warp_sum(acc[t]);
          if (lane == (t & 31)) {
            if (gate) v = v / (1.0f + expf(-to_float(gate[(long long)t * gate_row + (long long)h * n_out + o])));
            out[(long long)t * o_row + (long long)h * o_head + o] = from_float<T>(v);
          }
        }
    }
  }
}

static int per_head_linear_mma(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows, void* out,
                               long long o_row, long long o_head, const void* gate, long long gate_row, int n_tokens,
                               int heads, int n_in, int n_out, cudaStream_t stream);
static bool per_head_mma_takes(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows, int n_in,
                               int n_out);

extern "C" int llm_per_head_linear(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows,
                                   void* out, long long o_row, long long o_head, const void* gate, long long gate_row,
                                   int dtype, int n_tokens, int heads, int n_in, int n_out, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const size_t few_smem = ((size_t)n_tokens * n_in + 4 * PHF_TOKENS * 64) * sizeof(float);
  if (n_tokens <= PHF_TOKENS && few_smem <= 48 * 1024 && (n_out + 7) / 8 <= 65535) {
    dim3 few_grid(heads, w_in_rows ? (n_out + 63) / 64 : (n_out + 7) / 8);
#define FEW(T, IN_ROWS)                                                                                               \
  launch_kernel(per_head_linear_few_kernel<T, IN_ROWS>, few_grid, 256, few_smem, stream, (const T*)x, x_row, x_head, \
                (const T*)w, (T*)out, o_row, o_head, (const T*)gate, gate_row, n_tokens, n_in, n_out)
    if (dtype == DT_F32) { if (w_in_rows) FEW(float, true); else FEW(float, false); }
    else if (dtype == DT_BF16) { if (w_in_rows) FEW(__nv_bfloat16, true); else FEW(__nv_bfloat16, false); }
    else return ERR_BAD_DTYPE;
#undef FEW
    return launch_status();
  }
  dim3 grid((n_tokens + PH_TILE - 1) / PH_TILE, (n_out + PH_TILE - 1) / PH_TILE, heads);
  LLM_HOST_CHECK(grid.y <= 65535 && grid.z <= 65535, ERR_BAD_SIZE);
  if (dtype == DT_BF16 && per_head_mma_takes(x, x_row, x_head, w, w_in_rows, n_in, n_out))
    return per_head_linear_mma(x, x_row, x_head, w, w_in_rows, out, o_row, o_head, gate, gate_row, n_tokens, heads, n_in,
                               n_out, stream);
#define GO(T, IN_ROWS)                                                                                             \
  launch_kernel(per_head_linear_kernel<T, IN_ROWS>, grid, 256, 0, stream, (const T*)x, x_row, x_head, (const T*)w, \
                (T*)out, o_row, o_head, (const T*)gate, gate_row, n_tokens, n_in, n_out)
  if (dtype == DT_F32) { if (w_in_rows) GO(float, true); else GO(float, false); }
  else if (dtype == DT_BF16) { if (w_in_rows) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
  else return ERR_BAD_DTYPE;
#undef GO
  return launch_status();
}

// ------------------------------------------------------------------------------ attention

// Grid (token, group of LAT_WARPS heads).  The block brings 32 cached vectors at a time into shared
// memory (as float32, a warp four of them), and each warp, one head, scores them (a lane one key),
// keeps a running maximum and sum, and adds the weighted first `rank` entries (a lane the entries
// lane, lane + 32, ...).  Key blocks start at multiples of 32 positions, so the order of a row's
// sums depends on positions only.
template <typename T, typename TW>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attention_kernel(const T* __restrict__ q, T* __restrict__ out, PagedCache cache, int rank,
                        const TW* __restrict__ sink, const int32_t* __restrict__ positions,
                        const int32_t* __restrict__ row_seq, int heads, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float lat_smem[];     // keys [32][D + 1], then q [LAT_WARPS][D]
  const int D = cache.head_dim, ld = D + 1;
  float* keys = lat_smem;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = lat_smem + 32 * ld + warp * D;
  const int t = blockIdx.x, h = blockIdx.y * LAT_WARPS + warp;
  const bool active = h < heads;
  if (active)
    for (int c = lane; c < D; c += 32) qs[c] = to_float(q[((long long)t * heads + h) * D + c]);
  const int pos = positions[t], seq = row_seq[t];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const T* kc = (const T*)cache.k;
  float m = -INFINITY, l = 0.0f;
  float acc[LAT_MAX_CH];
#pragma unroll
  for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] = 0.0f;
  for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
    __syncthreads();      // the last block's keys have been read
    for (int kk = warp; kk < 32; kk += LAT_WARPS) {
      const int j = j0 + kk;
      long long off = -1;
      if (j >= first && j <= pos) off = cache_offset(cache, seq, j, 0);
      float* dst = keys + kk * ld;
      if (off >= 0)
        for (int c = lane; c < D; c += 32) dst[c] = to_float(kc[off + c]);
      if (lane == 0) dst[D] = off >= 0 ? 1.0f : 0.0f;      // the spare entry says whether the key is there
    }
    __syncthreads();
    if (!active) continue;
    const float* mine = keys + lane * ld;
    float s = -INFINITY;
    if (mine[D] != 0.0f) {
      float dot = 0.0f;
      for (int c = 0; c < D; ++c) dot = fmaf(qs[c], mine[c], dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = (s == -INFINITY) ? 0.0f : expf(s - m_new);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] *= corr;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      if (pj == 0.0f) continue;
      const float* vj = keys + jj * ld;
#pragma unroll
      for (int i = 0; i < LAT_MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < rank) acc[i] = fmaf(pj, vj[c], acc[i]);
      }
    }
    m = m_new;
  }
  if (!active) return;
  if (sink) {
    const float sk = to_float(sink[h]);
    const float m_new = fmaxf(m, sk);
    const float corr = (m == -INFINITY) ? 0.0f : expf(m - m_new);
    l = l * corr + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < LAT_MAX_CH; ++i) acc[i] *= corr;
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
  for (int i = 0; i < LAT_MAX_CH; ++i) {
    const int c = lane + 32 * i;
    if (c < rank) out[((long long)t * heads + h) * rank + c] = from_float<T>(acc[i] * inv);
  }
}

// dtype: element type of q, out, the cache and the sinks.  q [tokens, heads, D = rank + rot], out
// [tokens, heads, rank].
extern "C" int llm_latent_attention(const void* q, void* out, int dtype, void* k_base, const int32_t* block_table,
                                    long long page_stride, int table_stride, int page_tokens, int D, int rank,
                                    const void* sink, const int32_t* positions, const int32_t* row_seq, int heads,
                                    int n_tokens, float scale, int window, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(rank >= 1 && rank <= D && rank <= 32 * LAT_MAX_CH, ERR_BAD_SIZE);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, D};
  const size_t smem = ((size_t)32 * (D + 1) + (size_t)LAT_WARPS * D) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  dim3 grid(n_tokens, (heads + LAT_WARPS - 1) / LAT_WARPS);
  LLM_HOST_CHECK(grid.y <= 65535, ERR_BAD_SIZE);
  if (dtype == DT_F32) {
    auto kernel = latent_attention_kernel<float, float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LAT_THREADS, smem, stream, (const float*)q, (float*)out, c, rank, (const float*)sink,
                  positions, row_seq, heads, scale, window);
  } else if (dtype == DT_BF16) {
    auto kernel = latent_attention_kernel<__nv_bfloat16, __nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LAT_THREADS, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, c, rank,
                  (const __nv_bfloat16*)sink, positions, row_seq, heads, scale, window);
  } else {
    return ERR_BAD_DTYPE;
  }
  return launch_status();
}

// ------------------------------------------------------------------------------ attention, tensor cores

// The same attention on mma.sync (bfloat16 operands, float32 sums) for bfloat16 steps whose sizes
// fit: D a multiple of 16, rank a multiple of 32 up to 512.  Grid (token x group of 16 heads, key
// split).  All 16 rows of a tile are one token's heads: they see the same keys, so a tile has one
// causal limit and one cached block serves all of them, as the K operand [keys][D] of S = Q K^T and,
// its first `rank` columns, as the V operand of O += P V, from the same shared memory.  Four warps:
// for S a warp takes a quarter of the block's keys (all D), for O a quarter of the value columns
// (all keys); P and the rows' maxima and sums cross between the warps through shared memory.  The
// running maximum and sum are kept (identically) by every warp; weights are base-2 exponentials of
// scores scaled by scale * log2(e).  Key blocks are KB positions wide and start at multiples of KB;
// the next block arrives by asynchronous copies while the current one is used.  With n_splits > 1 the
// key blocks are dealt to blockIdx.y in runs, every block writes (O, max, sum) unnormalised, and the
// merge kernel adds them up with the sink; else the block finishes its rows itself.
#define LM_THREADS 128
#define LM_MAX_NT 16

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16 bytes from global to shared memory, or 16 zero bytes
__device__ __forceinline__ void cp_async_16_or_zero(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
               "r"(bytes) : "memory");
}

template <int KB>
__global__ void __launch_bounds__(LM_THREADS)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out,
                            float* __restrict__ partial, PagedCache cache, int rank,
                            const __nv_bfloat16* __restrict__ sink, const int32_t* __restrict__ positions,
                            const int32_t* __restrict__ row_seq, int heads, int head_groups, float scale_log2,
                            int window, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t lm_smem[];
  constexpr int NT_S = KB / 32, PLD = KB + 8;
  const int D = cache.head_dim, ld = D + 8, chunks = D / 8;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lm_smem);      // [16][ld]
  __nv_bfloat16* ks = qs + 16 * ld;                                   // [2][KB][ld]
  __nv_bfloat16* ps = ks + 2 * KB * ld;                               // [16][PLD]
  float* red = reinterpret_cast<float*>(ps + 16 * PLD);               // [2][4][16]: maxima, sums
  long long* koff = reinterpret_cast<long long*>(red + 128);          // [2][KB]: a key's place in the pool, -1: none
  // later tokens read more keys: they start first, so that the short ones fill the launch's tail
  const int tile = gridDim.x - 1 - blockIdx.x, t = tile / head_groups, hg = tile - t * head_groups, split = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t], seq = row_seq[t];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int b_lo = first / KB, nb = pos / KB - b_lo + 1;
  const int per = (nb + n_splits - 1) / n_splits;
  const int b0 = b_lo + split * per, b1 = min(b_lo + nb, b0 + per);
  const __nv_bfloat16* kc = (const __nv_bfloat16*)cache.k;

  for (int idx = threadIdx.x; idx < 16 * chunks; idx += LM_THREADS) {
    const int r = idx / chunks, c = idx - r * chunks, h = hg * 16 + r;
    const bool valid = h < heads;
    cp_async_16_or_zero(qs + r * ld + c * 8, q + ((long long)t * heads + (valid ? h : 0)) * D + c * 8, valid);
  }
  auto offsets = [&](int b, int stage) {
    if (threadIdx.x < KB) {
      const int j = b * KB + threadIdx.x;
      long long off = -1;
      if (j >= first && j <= pos) {
        const int page = cache.block_table[(long long)seq * cache.table_stride + j / cache.page_tokens];
        if (page >= 0) off = (long long)page * cache.page_stride + (long long)(j % cache.page_tokens) * D;
      }
      koff[stage * KB + threadIdx.x] = off;
    }
  };
  auto copies = [&](int stage) {
    __nv_bfloat16* dst = ks + stage * KB * ld;
    for (int idx = threadIdx.x; idx < KB * chunks; idx += LM_THREADS) {
      const int kk = idx / chunks, c = idx - kk * chunks;
      const long long off = koff[stage * KB + kk];
      cp_async_16_or_zero(dst + kk * ld + c * 8, kc + (off >= 0 ? off : 0) + c * 8, off >= 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (b0 < b1) {
    offsets(b0, 0);
    __syncthreads();
    copies(0);
  } else {
    asm volatile("cp.async.commit_group;" ::: "memory");
  }

  const int r0 = lane >> 2;                 // this thread's rows: r0 and r0 + 8
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  float o[LM_MAX_NT][4];
#pragma unroll
  for (int i = 0; i < LM_MAX_NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  const int ntw = rank / 32, col0 = warp * (rank / 4);

  for (int b = b0; b < b1; ++b) {
    const int stage = (b - b0) & 1;
    if (b + 1 < b1) offsets(b + 1, stage ^ 1);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                         // block b (and q) have arrived; the other stage is free; offsets are seen
    if (b + 1 < b1) copies(stage ^ 1);
    // S = Q K^T for this warp's keys
    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    const __nv_bfloat16* kb = ks + (stage * KB + warp * (KB / 4)) * ld;
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t a[4];
      ldsm_x4(a, qs + (lane & 15) * ld + k0 + (lane >> 4) * 8);
      if constexpr (NT_S == 2) {
        uint32_t bb[4];
        ldsm_x4(bb, kb + ((lane & 7) + ((lane >> 4) & 1) * 8) * ld + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[0], a, bb[0], bb[1]);
        mma_bf16(s[1], a, bb[2], bb[3]);
      } else {
        uint32_t bb[2];
        ldsm_x2(bb, kb + (lane & 7) * ld + k0 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[0], a, bb[0], bb[1]);
      }
    }
    // scale, mask, the rows' maxima over this warp's keys
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < NT_S; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = warp * (KB / 4) + i * 8 + (lane & 3) * 2 + (e & 1);
        const float v = koff[stage * KB + key] >= 0 ? s[i][e] * scale_log2 : -INFINITY;
        s[i][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if ((lane & 3) == 0) {
      red[warp * 16 + r0] = mx0;
      red[warp * 16 + r0 + 8] = mx1;
    }
    __syncthreads();
    float n0 = m0, n1 = m1;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      n0 = fmaxf(n0, red[w * 16 + r0]);
      n1 = fmaxf(n1, red[w * 16 + r0 + 8]);
    }
    const float c0 = n0 == -INFINITY ? 1.0f : exp2f(m0 - n0), c1 = n1 == -INFINITY ? 1.0f : exp2f(m1 - n1);
    float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
    for (int i = 0; i < NT_S; ++i) {
      const float p0 = n0 == -INFINITY ? 0.0f : exp2f(s[i][0] - n0), p1 = n0 == -INFINITY ? 0.0f : exp2f(s[i][1] - n0);
      const float p2 = n1 == -INFINITY ? 0.0f : exp2f(s[i][2] - n1), p3 = n1 == -INFINITY ? 0.0f : exp2f(s[i][3] - n1);
      sum0 += p0 + p1;
      sum1 += p2 + p3;
      const int key = warp * (KB / 4) + i * 8 + (lane & 3) * 2;
      *reinterpret_cast<__nv_bfloat162*>(ps + r0 * PLD + key) = __floats2bfloat162_rn(p0, p1);
      *reinterpret_cast<__nv_bfloat162*>(ps + (r0 + 8) * PLD + key) = __floats2bfloat162_rn(p2, p3);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    if ((lane & 3) == 0) {
      red[64 + warp * 16 + r0] = sum0;
      red[64 + warp * 16 + r0 + 8] = sum1;
    }
    __syncthreads();
    l0 = l0 * c0 + red[64 + r0] + red[64 + 16 + r0] + red[64 + 32 + r0] + red[64 + 48 + r0];
    l1 = l1 * c1 + red[64 + r0 + 8] + red[64 + 16 + r0 + 8] + red[64 + 32 + r0 + 8] + red[64 + 48 + r0 + 8];
    m0 = n0;
    m1 = n1;
    // O = O * corr + P V for this warp's value columns
#pragma unroll
    for (int i = 0; i < LM_MAX_NT; ++i)
      if (i < ntw) {
        o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
      }
    const __nv_bfloat16* vb = ks + stage * KB * ld + col0;
#pragma unroll
    for (int kk = 0; kk < KB; kk += 16) {
      uint32_t a[4];
      ldsm_x4(a, ps + (lane & 15) * PLD + kk + (lane >> 4) * 8);
      const __nv_bfloat16* vrow = vb + (kk + (lane & 7) + ((lane >> 3) & 1) * 8) * ld;
#pragma unroll
      for (int i = 0; i < LM_MAX_NT; i += 2) {
        if (i + 1 < ntw) {
          uint32_t bb[4];
          ldsm_x4_trans(bb, vrow + i * 8 + ((lane >> 4) & 1) * 8);
          mma_bf16(o[i], a, bb[0], bb[1]);
          mma_bf16(o[i + 1], a, bb[2], bb[3]);
        } else if (i < ntw) {
          uint32_t bb[2];
          ldsm_x2_trans(bb, vrow + i * 8);
          mma_bf16(o[i], a, bb[0], bb[1]);
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  const int cq = (lane & 3) * 2;
  if (n_splits > 1) {
    float* dst = partial + ((long long)(tile * n_splits + split) * 16) * (rank + 2);
#pragma unroll
    for (int i = 0; i < LM_MAX_NT; ++i)
      if (i < ntw) {
        const int c = col0 + i * 8 + cq;
        *reinterpret_cast<float2*>(dst + (long long)r0 * (rank + 2) + c) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(dst + (long long)(r0 + 8) * (rank + 2) + c) = make_float2(o[i][2], o[i][3]);
      }
    if (warp == 0 && (lane & 3) == 0) {
      *reinterpret_cast<float2*>(dst + (long long)r0 * (rank + 2) + rank) = make_float2(m0, l0);
      *reinterpret_cast<float2*>(dst + (long long)(r0 + 8) * (rank + 2) + rank) = make_float2(m1, l1);
    }
    return;
  }
  const int h0 = hg * 16 + r0, h1 = h0 + 8;
  if (sink) {
    if (h0 < heads) {
      const float sk = __bfloat162float(sink[h0]) * 1.4426950408889634f, n = fmaxf(m0, sk);
      const float c = m0 == -INFINITY ? 0.0f : exp2f(m0 - n);
      l0 = l0 * c + exp2f(sk - n);
#pragma unroll
      for (int i = 0; i < LM_MAX_NT; ++i) { o[i][0] *= c; o[i][1] *= c; }
    }
    if (h1 < heads) {
      const float sk = __bfloat162float(sink[h1]) * 1.4426950408889634f, n = fmaxf(m1, sk);
      const float c = m1 == -INFINITY ? 0.0f : exp2f(m1 - n);
      l1 = l1 * c + exp2f(sk - n);
#pragma unroll
      for (int i = 0; i < LM_MAX_NT; ++i) { o[i][2] *= c; o[i][3] *= c; }
    }
  }
  const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
#pragma unroll
  for (int i = 0; i < LM_MAX_NT; ++i)
    if (i < ntw) {
      const int c = col0 + i * 8 + cq;
      if (h0 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((long long)t * heads + h0) * rank + c) =
            __floats2bfloat162_rn(o[i][0] * i0, o[i][1] * i0);
      if (h1 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + ((long long)t * heads + h1) * rank + c) =
            __floats2bfloat162_rn(o[i][2] * i1, o[i][3] * i1);
    }
}

// One block per (tile, row): the splits' (O, max, sum) and the sink -> the row's weighted latent.
// The splits' weights 2^(max_s - max) / sum are worked out once, in shared memory.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                              const __nv_bfloat16* __restrict__ sink, int heads, int head_groups, int rank,
                              int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float wt[64], red[2];      // n_splits <= 32 (two entries per split while they are reduced)
  const int tile = blockIdx.x >> 4, r = blockIdx.x & 15;
  const int t = tile / head_groups, h = (tile - t * head_groups) * 16 + r;
  if (h >= heads) return;
  const float* base = partial + ((long long)tile * n_splits * 16 + r) * (rank + 2);
  const long long step = (long long)16 * (rank + 2);
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const float m = s < n_splits ? base[s * step + rank] : -INFINITY;
    const float l = s < n_splits ? base[s * step + rank + 1] : 0.0f;
    const float sk = sink ? __bfloat162float(sink[h]) * 1.4426950408889634f : -INFINITY;
    const float top = fmaxf(warp_max(m), sk);
    const float wgt = m == -INFINITY ? 0.0f : exp2f(m - top);
    const float total = warp_sum(l * wgt) + (sink ? exp2f(sk - top) : 0.0f);
    wt[s] = wgt;
    if (s == 0) red[0] = total > 0.0f ? 1.0f / total : 0.0f;
  }
  __syncthreads();
  const float inv = red[0];
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.0f;
    for (int s = 0; s < n_splits; ++s) acc = fmaf(base[s * step + c], wt[s], acc);
    out[((long long)t * heads + h) * rank + c] = __float2bfloat16_rn(acc * inv);
  }
}

// The same attention for prompt portions whose latent has at most 256 entries.  A tile is four tokens
// of one request in a row, a warp one token's 16 heads; the four warps share the cached blocks in
// shared memory (a quarter of the reads of the kernel above) and nothing else: a warp scores all 32
// keys of a block for its rows, keeps its running maxima and sums in registers, turns its score
// fragments into the weights' operand fragments where they are, and adds into its own O (all value
// columns).  Keys from the first one that the tile's first token may see to the last token's own; a
// warp masks what its token may not see.  Grid (request x ceil(longest portion / 4), group of 16 heads).
template <int NT_MAX>
__global__ void __launch_bounds__(LM_THREADS, NT_MAX > 16 ? 2 : 3)
latent_attention_rows_kernel(const __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ out, PagedCache cache,
                             int rank, const __nv_bfloat16* __restrict__ sink, const int32_t* __restrict__ positions,
                             const int32_t* __restrict__ seq_q_start, const int32_t* __restrict__ seq_q_len,
                             const int32_t* __restrict__ row_seq, int heads, int tiles_per_seq, float scale_log2,
                             int window) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int KB = 32;
  extern __shared__ __align__(16) uint8_t lm_smem[];
  const int D = cache.head_dim, ld = D + 8, chunks = D / 8;
  __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(lm_smem);      // [64][ld]: warp w's rows are 16 w ..
  __nv_bfloat16* ks = qs + 64 * ld;                                   // [2][KB][ld]
  long long* koff = reinterpret_cast<long long*>(ks + 2 * KB * ld);   // [3][KB]: the warps run up to a block apart
  // a request's last tiles read the most keys: they start first, so that the short ones fill the launch's tail
  const int seq = blockIdx.x / tiles_per_seq, tok0 = (tiles_per_seq - 1 - (blockIdx.x - seq * tiles_per_seq)) * 4, hg = blockIdx.y;
  const int q_len = seq_q_len[seq];
  if (tok0 >= q_len) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row0 = seq_q_start[seq] + tok0;
  const int last = min(3, q_len - 1 - tok0);                // the tile's last token
  const int pos0 = positions[row0], pos_hi = pos0 + last;
  const int cache_seq = row_seq[row0];
  const bool mine = warp <= last;
  const int pos = pos0 + warp;                              // positions of a request's tokens follow one another
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int b0 = first_lo / KB, b1 = pos_hi / KB + 1;
  const __nv_bfloat16* kc = (const __nv_bfloat16*)cache.k;

  for (int idx = threadIdx.x; idx < 64 * chunks; idx += LM_THREADS) {
    const int r = idx / chunks, c = idx - r * chunks, w = r >> 4, h = hg * 16 + (r & 15);
    const bool valid = h < heads && w <= last;
    cp_async_16_or_zero(qs + r * ld + c * 8, q + ((row0 + (valid ? w : 0)) * heads + (valid ? h : 0)) * D + c * 8, valid);
  }
  auto offsets = [&](int b, int slot) {
    if (threadIdx.x < KB) {
      const int j = b * KB + threadIdx.x;
      long long off = -1;
      if (j >= first_lo && j <= pos_hi) {
        const int page = cache.block_table[(long long)cache_seq * cache.table_stride + j / cache.page_tokens];
        if (page >= 0) off = (long long)page * cache.page_stride + (long long)(j % cache.page_tokens) * D;
      }
      koff[slot * KB + threadIdx.x] = off;
    }
  };
  auto copies = [&](int stage, int slot) {
    __nv_bfloat16* dst = ks + stage * KB * ld;
    for (int idx = threadIdx.x; idx < KB * chunks; idx += LM_THREADS) {
      const int kk = idx / chunks, c = idx - kk * chunks;
      const long long off = koff[slot * KB + kk];
      cp_async_16_or_zero(dst + kk * ld + c * 8, kc + (off >= 0 ? off : 0) + c * 8, off >= 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  offsets(b0, 0);
  __syncthreads();
  copies(0, 0);

  const int r0 = lane >> 2, cq = (lane & 3) * 2;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
  float o[NT_MAX][4];
#pragma unroll
  for (int i = 0; i < NT_MAX; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  const int ntw = rank / 8;
  const __nv_bfloat16* qw = qs + warp * 16 * ld;

  for (int b = b0; b < b1; ++b) {
    const int stage = (b - b0) & 1, slot = (b - b0) % 3, next = (b - b0 + 1) % 3;
    if (b + 1 < b1) offsets(b + 1, next);      // a slot that no warp still reads: they are at most one block behind
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (b + 1 < b1) copies(stage ^ 1, next);
    if (!mine || b * KB > pos || (b + 1) * KB <= first) continue;      // nothing in this block for this warp's token
    const __nv_bfloat16* kb = ks + stage * KB * ld;
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
    for (int k0 = 0; k0 < D; k0 += 16) {
      uint32_t a[4], b01[4], b23[4];
      ldsm_x4(a, qw + (lane & 15) * ld + k0 + (lane >> 4) * 8);
      const __nv_bfloat16* kp = kb + ((lane & 7) + ((lane >> 4) & 1) * 8) * ld + k0 + ((lane >> 3) & 1) * 8;
      ldsm_x4(b01, kp);
      ldsm_x4(b23, kp + 16 * ld);
      mma_bf16(s[0], a, b01[0], b01[1]);
      mma_bf16(s[1], a, b01[2], b01[3]);
      mma_bf16(s[2], a, b23[0], b23[1]);
      mma_bf16(s[3], a, b23[2], b23[3]);
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = i * 8 + cq + (e & 1), j = b * KB + key;
        const float v = (koff[slot * KB + key] >= 0 && j >= first && j <= pos) ? s[i][e] * scale_log2 : -INFINITY;
        s[i][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);
    if (n0 == -INFINITY && n1 == -INFINITY) continue;
    const float c0 = n0 == -INFINITY ? 1.0f : exp2f(m0 - n0), c1 = n1 == -INFINITY ? 1.0f : exp2f(m1 - n1);
    float sum0 = 0.0f, sum1 = 0.0f;
    uint32_t pa[2][4];       // the weights as the A operand of P V: keys 0..15 and 16..31
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p0 = n0 == -INFINITY ? 0.0f : exp2f(s[i][0] - n0), p1 = n0 == -INFINITY ? 0.0f : exp2f(s[i][1] - n0);
      const float p2 = n1 == -INFINITY ? 0.0f : exp2f(s[i][2] - n1), p3 = n1 == -INFINITY ? 0.0f : exp2f(s[i][3] - n1);
      sum0 += p0 + p1;
      sum1 += p2 + p3;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
      pa[i >> 1][(i & 1) * 2] = *reinterpret_cast<const uint32_t*>(&lo);
      pa[i >> 1][(i & 1) * 2 + 1] = *reinterpret_cast<const uint32_t*>(&hi);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l0 = l0 * c0 + sum0;
    l1 = l1 * c1 + sum1;
    m0 = n0;
    m1 = n1;
#pragma unroll
    for (int i = 0; i < NT_MAX; ++i)
      if (i < ntw) {
        o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
      }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const __nv_bfloat16* vrow = kb + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + ((lane >> 4) & 1) * 8;
#pragma unroll
      for (int i = 0; i < NT_MAX; i += 2)
        if (i < ntw) {
          uint32_t bb[4];
          ldsm_x4_trans(bb, vrow + i * 8);
          mma_bf16(o[i], pa[kk], bb[0], bb[1]);
          mma_bf16(o[i + 1], pa[kk], bb[2], bb[3]);
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  if (!mine) return;
  const int h0 = hg * 16 + r0, h1 = h0 + 8;
  if (sink) {
    if (h0 < heads) {
      const float sk = __bfloat162float(sink[h0]) * 1.4426950408889634f, n = fmaxf(m0, sk);
      const float c = m0 == -INFINITY ? 0.0f : exp2f(m0 - n);
      l0 = l0 * c + exp2f(sk - n);
#pragma unroll
      for (int i = 0; i < NT_MAX; ++i) { o[i][0] *= c; o[i][1] *= c; }
    }
    if (h1 < heads) {
      const float sk = __bfloat162float(sink[h1]) * 1.4426950408889634f, n = fmaxf(m1, sk);
      const float c = m1 == -INFINITY ? 0.0f : exp2f(m1 - n);
      l1 = l1 * c + exp2f(sk - n);
#pragma unroll
      for (int i = 0; i < NT_MAX; ++i) { o[i][2] *= c; o[i][3] *= c; }
    }
  }
  const float i0 = l0 > 0.0f ? 1.0f / l0 : 0.0f, i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f;
  const long long t = row0 + warp;
#pragma unroll
  for (int i = 0; i < NT_MAX; ++i)
    if (i < ntw) {
      const int c = i * 8 + cq;
      if (h0 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + (t * heads + h0) * rank + c) = __floats2bfloat162_rn(o[i][0] * i0, o[i][1] * i0);
      if (h1 < heads)
        *reinterpret_cast<__nv_bfloat162*>(out + (t * heads + h1) * rank + c) = __floats2bfloat162_rn(o[i][2] * i1, o[i][3] * i1);
    }
}

extern "C" int llm_latent_attention_rows(const void* q, void* out, void* k_base, const int32_t* block_table,
                                         long long page_stride, int table_stride, int page_tokens, int D, int rank,
                                         const void* sink, const int32_t* positions, const int32_t* seq_q_start,
                                         const int32_t* seq_q_len, const int32_t* row_seq, int heads, int n_seqs,
                                         int max_q_len, float scale, int window, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return 0;
  LLM_HOST_CHECK(D % 16 == 0 && rank % 16 == 0 && rank >= 16 && rank <= 256 && rank <= D, ERR_BAD_SIZE);
  LLM_HOST_CHECK(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_base % 16) == 0 && page_stride % 8 == 0, ERR_BAD_ALIGN);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, D};
  const int tiles_per_seq = (max_q_len + 3) / 4, head_groups = (heads + 15) / 16;
  const size_t smem = (size_t)(64 + 2 * 32) * (D + 8) * 2 + (size_t)3 * 32 * sizeof(long long);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  dim3 grid((unsigned)((long long)n_seqs * tiles_per_seq), head_groups);
  LLM_HOST_CHECK(head_groups <= 65535, ERR_BAD_SIZE);
  const float scale_log2 = scale * 1.4426950408889634f;
#define GO(NT)                                                                                                       \
  do {                                                                                                               \
    auto kernel = latent_attention_rows_kernel<NT>;                                                                  \
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                            \
    launch_kernel(kernel, grid, LM_THREADS, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, c, rank,     \
                  (const __nv_bfloat16*)sink, positions, seq_q_start, seq_q_len, row_seq, heads, tiles_per_seq,      \
                  scale_log2, window);                                                                               \
  } while (0)
  if (rank <= 64) GO(8);
  else if (rank <= 128) GO(16);
  else GO(32);
#undef GO
  return launch_status();
}

// One matrix per head on mma.sync, for bfloat16 steps of many tokens whose rows are 16-byte aligned:
// a block takes 64 tokens x 64 outputs of one head, a warp 16 tokens; inputs and the head's weights
// arrive 32 inputs at a time by asynchronous copies, two stages deep; float32 sums.
template <bool W_IN_ROWS>
__global__ void __launch_bounds__(128)
per_head_linear_mma_kernel(const __nv_bfloat16* __restrict__ x, long long x_row, long long x_head,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long o_row,
                           long long o_head, const __nv_bfloat16* __restrict__ gate, long long gate_row, int n_tokens,
                           int n_in, int n_out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int XLD = 40, WLD = W_IN_ROWS ? 72 : 40, WROWS = W_IN_ROWS ? 32 : 64;
  __shared__ __align__(16) __nv_bfloat16 xs[2][64 * XLD];
  __shared__ __align__(16) __nv_bfloat16 ws[2][WROWS * WLD];
  const int h = blockIdx.z, t0 = blockIdx.x * 64, o0 = blockIdx.y * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const __nv_bfloat16* wh = w + (long long)h * n_in * n_out;
  auto copies = [&](int k0, int stage) {
    for (int e = threadIdx.x; e < 64 * 4; e += 128) {          // x: 64 tokens x 4 pieces of 8 inputs
      const int r = e >> 2, c = (e & 3) * 8, t = t0 + r, k = k0 + c;
      const bool valid = t < n_tokens && k < n_in;
      cp_async_16_or_zero(&xs[stage][r * XLD + c], x + (valid ? (long long)t * x_row + (long long)h * x_head + k : 0), valid);
    }
    if (W_IN_ROWS) {                                           // w: 32 inputs x 8 pieces of 8 outputs
      for (int e = threadIdx.x; e < 32 * 8; e += 128) {
        const int r = e >> 3, c = (e & 7) * 8, k = k0 + r, o = o0 + c;
        const bool valid = k < n_in && o < n_out;
        cp_async_16_or_zero(&ws[stage][r * WLD + c], wh + (valid ? (long long)k * n_out + o : 0), valid);
      }
    } else {                                                   // w: 64 outputs x 4 pieces of 8 inputs
      for (int e = threadIdx.x; e < 64 * 4; e += 128) {
        const int r = e >> 2, c = (e & 3) * 8, o = o0 + r, k = k0 + c;
        const bool valid = o < n_out && k < n_in;
        cp_async_16_or_zero(&ws[stage][r * WLD + c], wh + (valid ? (long long)o * n_in + k : 0), valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
  copies(0, 0);
  int stage = 0;
  for (int k0 = 0; k0 < n_in; k0 += 32, stage ^= 1) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                      // this stage has arrived, the other one has been read
    if (k0 + 32 < n_in) copies(k0 + 32, stage ^ 1);
#pragma unroll
    for (int kk = 0; kk < 32; kk += 16) {
      uint32_t a[4];
      ldsm_x4(a, &xs[stage][(warp * 16 + (lane & 15)) * XLD + kk + (lane >> 4) * 8]);
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        uint32_t b[4];
        if (W_IN_ROWS)
          ldsm_x4_trans(b, &ws[stage][(kk + (lane & 7) + ((lane >> 3) & 1) * 8) * WLD + i * 8 + ((lane >> 4) & 1) * 8]);
        else
          ldsm_x4(b, &ws[stage][(i * 8 + (lane & 7) + ((lane >> 4) & 1) * 8) * WLD + kk + ((lane >> 3) & 1) * 8]);
        mma_bf16(acc[i], a, b[0], b[1]);
        mma_bf16(acc[i + 1], a, b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int t = t0 + warp * 16 + (lane >> 2) + (e >= 2 ? 8 : 0), o = o0 + i * 8 + (lane & 3) * 2 + (e & 1);
      if (t >= n_tokens || o >= n_out) continue;
      float v = acc[i][e];
      if (gate) v = v / (1.0f + expf(-__bfloat162float(gate[(long long)t * gate_row + (long long)h * n_out + o])));
      out[(long long)t * o_row + (long long)h * o_head + o] = __float2bfloat16_rn(v);
    }
}

// Whether the mma.sync form can read these operands with 16-byte copies.
static bool per_head_mma_takes(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows, int n_in,
                               int n_out) {
  return ((uintptr_t)x % 16) == 0 && ((uintptr_t)w % 16) == 0 && x_row % 8 == 0 && x_head % 8 == 0 && n_in % 8 == 0 &&
         (w_in_rows ? n_out % 8 == 0 : true);
}

static int per_head_linear_mma(const void* x, long long x_row, long long x_head, const void* w, int w_in_rows, void* out,
                               long long o_row, long long o_head, const void* gate, long long gate_row, int n_tokens,
                               int heads, int n_in, int n_out, cudaStream_t stream) {
  dim3 grid((n_tokens + 63) / 64, (n_out + 63) / 64, heads);
  if (w_in_rows)
    launch_kernel(per_head_linear_mma_kernel<true>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_row, x_head,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row, o_head, (const __nv_bfloat16*)gate, gate_row,
                  n_tokens, n_in, n_out);
  else
    launch_kernel(per_head_linear_mma_kernel<false>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_row, x_head,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row, o_head, (const __nv_bfloat16*)gate, gate_row,
                  n_tokens, n_in, n_out);
  return launch_status();
}

// Floats of scratch a launch with these splits needs.
extern "C" long long llm_latent_attention_mma_scratch(int n_tokens, int heads, int rank, int n_splits) {
  return n_splits > 1 ? (long long)n_tokens * ((heads + 15) / 16) * n_splits * 16 * (rank + 2) : 0;
}

extern "C" int llm_latent_attention_mma(const void* q, void* out, float* partial, void* k_base,
                                        const int32_t* block_table, long long page_stride, int table_stride,
                                        int page_tokens, int D, int rank, const void* sink, const int32_t* positions,
                                        const int32_t* row_seq, int heads, int n_tokens, float scale, int window,
                                        int n_splits, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(D % 16 == 0 && rank % 32 == 0 && rank >= 32 && rank <= 32 * LM_MAX_NT && rank <= D, ERR_BAD_SIZE);
  LLM_HOST_CHECK(n_splits >= 1 && n_splits <= 32 && (n_splits == 1 || partial), ERR_BAD_SIZE);
  LLM_HOST_CHECK(((uintptr_t)q % 16) == 0 && ((uintptr_t)k_base % 16) == 0 && page_stride % 8 == 0, ERR_BAD_ALIGN);
  PagedCache c{k_base, k_base, block_table, page_stride, table_stride, page_tokens, 1, D};
  const int head_groups = (heads + 15) / 16;
  const int ld = D + 8;
  auto bytes = [&](int kb) {
    return (size_t)(16 + 2 * kb) * ld * 2 + (size_t)16 * (kb + 8) * 2 + 128 * sizeof(float) + (size_t)2 * kb * sizeof(long long);
  };
  const int kb = bytes(64) <= 56 * 1024 ? 64 : 32;
  const size_t smem = bytes(kb);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  dim3 grid((unsigned)((long long)n_tokens * head_groups), n_splits);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (kb == 64) {
    auto kernel = latent_attention_mma_kernel<64>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LM_THREADS, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, c, rank,
                  (const __nv_bfloat16*)sink, positions, row_seq, heads, head_groups, scale_log2, window, n_splits);
  } else {
    auto kernel = latent_attention_mma_kernel<32>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(kernel, grid, LM_THREADS, smem, stream, (const __nv_bfloat16*)q, (__nv_bfloat16*)out, partial, c, rank,
                  (const __nv_bfloat16*)sink, positions, row_seq, heads, head_groups, scale_log2, window, n_splits);
  }
  int status = launch_status();
  if (status || n_splits == 1) return status;
  launch_kernel(latent_attention_merge_kernel, (unsigned)((long long)n_tokens * head_groups * 16), 128, 0, stream,
                (const float*)partial, (__nv_bfloat16*)out, (const __nv_bfloat16*)sink, heads, head_groups, rank, n_splits);
  return launch_status();
}
