// What lies between the projections of a softmax-attention mixer and its attention kernel, for
// mixers that norm and rotate per head:
//
//   q_h <- rotate(rms_norm(q_h) * wq),  k_g <- rotate(rms_norm(k_g) * wk)       (norm weights shared by the heads)
//
// rotate turns the first `rot_dims` entries of a head pair by pair, entry 2i with entry 2i + 1 (or, with
// `halves`, entry i with entry i + rot_dims / 2), by the angle position * inv_freq[i], cos and sin
// multiplied by `mag`; the other entries pass.  With `maps` > 1 a head is that many units side by side
// (the maps of differential attention), each normed and turned by itself; the values belong to the head.  q goes
// to its buffer, k into the request's cache page, and the values - a projection of their own, or
// the keys as projected, before norm and rotation - beside it.  Grid (token, share of the token's heads).  Norm, angle and rotation are float32.
// `bias` (float32, indexed by the projection's column, or null) is added to q, k and v as they are read.
// Value mixing: with `v_mix_in` [tokens, kv_heads * v_dim] float32 the value becomes (1 - v_mix) v + v_mix *
// v_mix_in (another layer's values of the same token), and with `v_mix_out` the value as cached is also
// left there in float32 for later layers of the same step.
// Also here: the sigmoid gate on a mixer's output.

#include "common.cuh"

#include <math.h>

#define PREP_WARPS 4

template <typename T, typename TW>
__global__ void __launch_bounds__(PREP_WARPS * 32)
headnorm_rope_cache_kernel(const T* __restrict__ u, long long u_stride, int q_col, int k_col, int v_col,
                           const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
                           const float* __restrict__ inv_freq, int rot_dims, int halves, int maps, float mag,
                           T* __restrict__ q_out, PagedCache cache, int v_dim, const int32_t* __restrict__ positions,
                           const int32_t* __restrict__ row_seq, int q_heads, int write_cache,
                           const float* __restrict__ bias, const float* __restrict__ v_mix_in, float v_mix,
                           float* __restrict__ v_mix_out) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float head_smem[];  // PREP_WARPS * head_dim
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x, d = cache.head_dim / maps;      // a head holds `maps` units, each normed and turned by itself
  float* s = head_smem + warp * d;
  const int pos = positions[t], seq = row_seq[t];
  const T* row = u + (long long)t * u_stride;
  const int units = (q_heads + cache.kv_heads) * maps;
  for (int item = blockIdx.y * PREP_WARPS + warp; item < units; item += gridDim.y * PREP_WARPS) {
    const bool is_q = item < q_heads * maps;
    const int unit = is_q ? item : item - q_heads * maps;
    const int h = unit / maps, map = unit - h * maps;
    const T* x = row + (is_q ? q_col : k_col) + (long long)unit * d;
    const TW* w = is_q ? q_norm_w : k_norm_w;
    const float* bx = bias ? bias + (is_q ? q_col : k_col) + (long long)unit * d : nullptr;
    T* dst = nullptr;
    if (is_q) {
      dst = q_out + ((long long)t * q_heads * maps + unit) * d;
    } else if (write_cache) {
      const int page = cache.block_table[(long long)seq * cache.table_stride + pos / cache.page_tokens];
      if (page >= 0) {
        const long long slot = (long long)h * cache.page_tokens + (pos % cache.page_tokens);
        dst = (T*)cache.k + (long long)page * cache.page_stride + slot * cache.head_dim + map * d;
        if (map == 0) {
          T* vdst = (T*)cache.v + (long long)page * cache.page_stride + slot * v_dim;
          const T* vx = v_col >= 0 ? row + v_col + h * v_dim : x;
          if (!bias && !v_mix_in && !v_mix_out) {
            for (int c = lane; c < v_dim; c += 32) vdst[c] = vx[c];
          } else {
            const float* bv = bias ? (v_col >= 0 ? bias + v_col + h * v_dim : bx) : nullptr;
            const long long at = ((long long)t * cache.kv_heads + h) * v_dim;
            for (int c = lane; c < v_dim; c += 32) {
              float v = to_float(vx[c]) + (bv ? bv[c] : 0.0f);
              if (v_mix_in) v = (1.0f - v_mix) * v + v_mix * v_mix_in[at + c];
              if (v_mix_out) v_mix_out[at + c] = v;
              vdst[c] = from_float<T>(v);
            }
          }
        }
      }
    }
    if (!dst) continue;      // the whole warp takes the same way
    float sq = 0.0f;
    for (int c = lane; c < d; c += 32) {
      const float v = to_float(x[c]) + (bx ? bx[c] : 0.0f);
      s[c] = v;
      sq += v * v;
    }
    const float scale = w ? 1.0f / sqrtf(warp_sum(sq) / (float)d + eps) : 1.0f;
    __syncwarp();
    const int half = rot_dims / 2;
    for (int p = lane; p < half; p += 32) {
      float sn, cs;
      sincosf((float)pos * inv_freq[p], &sn, &cs);
      sn *= mag;
      cs *= mag;
      const int ia = halves ? p : 2 * p, ib = halves ? p + half : 2 * p + 1;
      const float a = s[ia] * scale * (w ? to_float(w[ia]) : 1.0f);
      const float b = s[ib] * scale * (w ? to_float(w[ib]) : 1.0f);
      dst[ia] = from_float<T>(a * cs - b * sn);
      dst[ib] = from_float<T>(b * cs + a * sn);
    }
    for (int c = rot_dims + lane; c < d; c += 32) dst[c] = from_float<T>(s[c] * scale * (w ? to_float(w[c]) : 1.0f));
    __syncwarp();
  }
}

// dtype: element type of u, q_out, the cache and the norm weights.
extern "C" int llm_headnorm_rope_cache(const void* u, int dtype, long long u_stride, int q_col, int k_col, int v_col,
                                       const void* q_norm_w, const void* k_norm_w, float eps, const float* inv_freq,
                                       int rot_dims, int halves, int maps, float mag, void* q_out, void* k_base,
                                       void* v_base,
                                       const int32_t* block_table, long long page_stride, int table_stride,
                                       int page_tokens, int kv_heads, int head_dim, int v_dim, const int32_t* positions,
                                       const int32_t* row_seq, int q_heads, int write_cache, int n_tokens,
                                       const float* bias, const float* v_mix_in, float v_mix, float* v_mix_out,
                                       cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(maps >= 1 && head_dim % maps == 0, ERR_BAD_SIZE);
  LLM_HOST_CHECK(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= head_dim / maps && (rot_dims == 0 || inv_freq), ERR_BAD_SIZE);
  LLM_HOST_CHECK(v_col >= 0 || (v_dim == head_dim && maps == 1), ERR_BAD_SIZE);
  const size_t smem = (size_t)PREP_WARPS * head_dim * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  PagedCache c{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  // few tokens: a token's heads are dealt to several blocks, so that the step still fills the GPU
  const int per_token = n_tokens >= 256 ? 1 : min(((q_heads + kv_heads) * maps + PREP_WARPS - 1) / PREP_WARPS, 16);
  const dim3 grid(n_tokens, per_token);
  if (dtype == DT_F32)
    launch_kernel(headnorm_rope_cache_kernel<float, float>, grid, PREP_WARPS * 32, smem, stream, (const float*)u,
                  u_stride, q_col, k_col, v_col, (const float*)q_norm_w, (const float*)k_norm_w, eps, inv_freq, rot_dims,
                  halves, maps, mag, (float*)q_out, c, v_dim, positions, row_seq, q_heads, write_cache, bias, v_mix_in, v_mix,
                  v_mix_out);
  else if (dtype == DT_BF16)
    launch_kernel(headnorm_rope_cache_kernel<__nv_bfloat16, __nv_bfloat16>, grid, PREP_WARPS * 32, smem, stream,
                  (const __nv_bfloat16*)u, u_stride, q_col, k_col, v_col, (const __nv_bfloat16*)q_norm_w,
                  (const __nv_bfloat16*)k_norm_w, eps, inv_freq, rot_dims, halves, maps, mag, (__nv_bfloat16*)q_out, c, v_dim,
                  positions, row_seq, q_heads, write_cache, bias, v_mix_in, v_mix, v_mix_out);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// x[t, c] *= sigmoid(gate[t, c]); gate may be a column view (rows `gate_stride` apart).
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, long long gate_stride, long long total,
                                    int width) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / width;
    const int c = (int)(i - t * width);
    const float z = to_float(gate[t * gate_stride + c]);
    x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-z)));
  }
}

extern "C" int llm_sigmoid_gate(void* x, const void* gate, int dtype, long long gate_stride, int rows, int width,
                                cudaStream_t stream) {
  const long long total = (long long)rows * width;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  if (dtype == DT_F32)
    launch_kernel(sigmoid_gate_kernel<float>, blocks, 256, 0, stream, (float*)x, (const float*)gate, gate_stride, total, width);
  else if (dtype == DT_BF16)
    launch_kernel(sigmoid_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)x,
                  (const __nv_bfloat16*)gate, gate_stride, total, width);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
