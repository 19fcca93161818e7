// Differential attention over the paged cache: every query head carries two maps, each a softmax
// attention of its own over the same values,
//
//   a_m = softmax_j((q_m . k_m,j) * scale) V,   m = 1, 2;   o = a_1 - lambda * a_2;
//   o <- o / sqrt(mean(o^2) + eps) * out_scale  (over the head's values, no weight);   o <- o * sigmoid(gate)
//
// A cached key head holds both maps side by side ([map 1 | map 2], 2 * dim entries), a value head
// `v_dim` entries; `heads / kv_heads` query heads share a key/value head.  Which keys a query at
// position p sees: j <= p and, with `window` > 0, j > p - window; with `chunk` > 0, j >= p - p % chunk
// (blocks of `chunk` positions counted from the sequence's first).  Scores, softmax weights, the
// difference, the norm and the gate are float32.
//
// Kernels: diff_attention_plain (a warp per (token, head), float32 throughout: the float32 path and
// sizes the tensor-core kernel does not take) and diff_attention_mma (bfloat16 on mma.sync).

#include "common.cuh"

#include <math.h>

constexpr int DA_WARPS = 4;
constexpr int DA_MAX_CH = 8;   // value sizes up to 256

__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  int first = 0;
  if (window > 0) first = max(first, pos - window + 1);
  if (chunk > 0) first = max(first, pos - pos % chunk);
  return first;
}

// One warp per (token, query head).  Keys are visited in blocks of 32 aligned to absolute
// positions, lane l scores key block * 32 + l for both maps, so the order of every sum depends on
// positions only and not on how a prompt was cut.
template <typename T>
__global__ void __launch_bounds__(DA_WARPS * 32)
diff_attention_plain_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ gate,
                            long long gate_stride, PagedCache cache, int v_dim,
                            const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq, int q_heads,
                            int n_tokens, float scale, int window, int chunk, float lambda, float eps,
                            float out_scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float q_smem[];  // DA_WARPS * head_dim (both maps)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * DA_WARPS + warp;
  const int d2 = cache.head_dim, d = d2 / 2;
  const bool active = item < (long long)n_tokens * q_heads;
  const int t = active ? (int)(item / q_heads) : 0;
  const int h = active ? (int)(item % q_heads) : 0;
  float* qs = q_smem + warp * d2;
  if (active)
    for (int c = lane; c < d2; c += 32) qs[c] = to_float(q[((long long)t * q_heads + h) * d2 + c]);
  __syncwarp();
  if (!active) return;

  const int pos = positions[t];
  const int slot = row_seq[t];
  const int kvh = h / (q_heads / cache.kv_heads);
  const int first = first_visible(pos, window, chunk);
  const T* kc = (const T*)cache.k;
  const T* vc = (const T*)cache.v;

  float m1 = -INFINITY, l1 = 0.0f, m2 = -INFINITY, l2 = 0.0f;
  float acc1[DA_MAX_CH], acc2[DA_MAX_CH];
#pragma unroll
  for (int i = 0; i < DA_MAX_CH; ++i) acc1[i] = acc2[i] = 0.0f;

  for (int j0 = (first / 32) * 32; j0 <= pos; j0 += 32) {
    const int j = j0 + lane;
    const bool visible = j >= first && j <= pos;
    float s1 = -INFINITY, s2 = -INFINITY;
    long long voff = -1;
    if (visible) {
      const int page = cache.block_table[(long long)slot * cache.table_stride + j / cache.page_tokens];
      if (page >= 0) {
        const long long in_page = (long long)kvh * cache.page_tokens + (j % cache.page_tokens);
        const long long koff = (long long)page * cache.page_stride + in_page * d2;
        voff = (long long)page * cache.page_stride + in_page * v_dim;
        float dot1 = 0.0f, dot2 = 0.0f;
        for (int c = 0; c < d; ++c) {
          dot1 = fmaf(qs[c], to_float(kc[koff + c]), dot1);
          dot2 = fmaf(qs[d + c], to_float(kc[koff + d + c]), dot2);
        }
        s1 = dot1 * scale;
        s2 = dot2 * scale;
      }
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float p1 = (s1 == -INFINITY) ? 0.0f : expf(s1 - n1);
    const float p2 = (s2 == -INFINITY) ? 0.0f : expf(s2 - n2);
    const float c1 = (m1 == -INFINITY) ? 0.0f : expf(m1 - n1);
    const float c2 = (m2 == -INFINITY) ? 0.0f : expf(m2 - n2);
    l1 = l1 * c1 + warp_sum(p1);
    l2 = l2 * c2 + warp_sum(p2);
#pragma unroll
    for (int i = 0; i < DA_MAX_CH; ++i) {
      acc1[i] *= c1;
      acc2[i] *= c2;
    }
    for (int jj = 0; jj < 32; ++jj) {
      const long long offj = __shfl_sync(0xffffffffu, voff, jj);
      const float pj1 = __shfl_sync(0xffffffffu, p1, jj);
      const float pj2 = __shfl_sync(0xffffffffu, p2, jj);
      if (offj < 0) continue;
#pragma unroll
      for (int i = 0; i < DA_MAX_CH; ++i) {
        const int c = lane + 32 * i;
        if (c < v_dim) {
          const float v = to_float(vc[offj + c]);
          acc1[i] = fmaf(pj1, v, acc1[i]);
          acc2[i] = fmaf(pj2, v, acc2[i]);
        }
      }
    }
    m1 = n1;
    m2 = n2;
  }
  const float i1 = l1 > 0.0f ? 1.0f / l1 : 0.0f, i2 = l2 > 0.0f ? 1.0f / l2 : 0.0f;
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < DA_MAX_CH; ++i) {
    const int c = lane + 32 * i;
    acc1[i] = c < v_dim ? acc1[i] * i1 - lambda * (acc2[i] * i2) : 0.0f;
    sq += acc1[i] * acc1[i];
  }
  const float norm = out_scale / sqrtf(warp_sum(sq) / (float)v_dim + eps);
#pragma unroll
  for (int i = 0; i < DA_MAX_CH; ++i) {
    const int c = lane + 32 * i;
    if (c < v_dim) {
      float o = acc1[i] * norm;
      if (gate) o /= 1.0f + expf(-to_float(gate[(long long)t * gate_stride + (long long)h * v_dim + c]));
      out[((long long)t * q_heads + h) * v_dim + c] = from_float<T>(o);
    }
  }
}

// q [tokens, heads, head_dim] with head_dim = 2 * dim (the cache's key head size); out [tokens, heads, v_dim];
// gate (or null) [tokens, >= heads * v_dim] with rows `gate_stride` apart.
extern "C" int llm_diff_attention_plain(const void* q, void* out, const void* gate, long long gate_stride, int dtype,
                                        void* k_base, void* v_base, const int32_t* block_table, long long page_stride,
                                        int table_stride, int page_tokens, int kv_heads, int head_dim, int v_dim,
                                        const int32_t* positions, const int32_t* row_seq, int q_heads, int n_tokens,
                                        float scale, int window, int chunk, float lambda, float eps, float out_scale,
                                        cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (v_dim > 32 * DA_MAX_CH || v_dim < 1 || head_dim % 2 || q_heads % kv_heads) return ERR_BAD_SIZE;
  const size_t smem = (size_t)DA_WARPS * head_dim * sizeof(float);
  if (smem > 48 * 1024) return ERR_BAD_SIZE;
  PagedCache c{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim};
  const long long items = (long long)n_tokens * q_heads;
  const unsigned blocks = (unsigned)((items + DA_WARPS - 1) / DA_WARPS);
  if (dtype == DT_F32)
    launch_kernel(diff_attention_plain_kernel<float>, blocks, DA_WARPS * 32, smem, stream, (const float*)q, (float*)out,
                  (const float*)gate, gate_stride, c, v_dim, positions, row_seq, q_heads, n_tokens, scale, window, chunk,
                  lambda, eps, out_scale);
  else if (dtype == DT_BF16)
    launch_kernel(diff_attention_plain_kernel<__nv_bfloat16>, blocks, DA_WARPS * 32, smem, stream,
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, gate_stride, c, v_dim,
                  positions, row_seq, q_heads, n_tokens, scale, window, chunk, lambda, eps, out_scale);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
