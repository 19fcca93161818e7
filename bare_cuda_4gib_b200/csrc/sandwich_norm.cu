// Norms of a residual stream whose sublayers are normed on both sides:
//
//   x <- x + rms_norm(y) * b,   h = rms_norm(x) * w          (y a sublayer's result, h the next one's input)
//
// as one kernel per sublayer boundary, and the embedding lookup followed by an RMS norm.  The
// stream, the sums of squares and both factors are float32; rms_norm(v) = v / sqrt(mean(v^2) + eps).
// One block of a fixed size per row: the order of every sum depends on the width only.

#include "common.cuh"

#include <math.h>

#define NORM_THREADS 256

template <typename TT, typename TW>
__global__ void __launch_bounds__(NORM_THREADS)
embed_rmsnorm_kernel(const TT* __restrict__ table, const int32_t* __restrict__ ids, const TW* __restrict__ weight,
                     float* __restrict__ out, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + hidden;
  const int t = blockIdx.x;
  const TT* row = table + (long long)ids[t] * hidden;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_float(row[i]);
    row_cache[i] = v;
    sq += v * v;
  }
  const float scale = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps);
  float* dst = out + (long long)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = row_cache[i] * scale * to_float(weight[i]);
}

// dtype: the table's element type; weight_dtype: the norm weight's (the table's, or float32 for a factor
// that was formed in float32).
extern "C" int llm_embed_rmsnorm(const void* table, const int32_t* ids, const void* weight, int dtype, int weight_dtype,
                                 float* out, int n_tokens, int hidden, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  if (dtype == DT_F32 && weight_dtype == DT_F32)
    launch_kernel(embed_rmsnorm_kernel<float, float>, n_tokens, NORM_THREADS, smem, stream, (const float*)table, ids,
                  (const float*)weight, out, hidden, eps);
  else if (dtype == DT_BF16 && weight_dtype == DT_BF16)
    launch_kernel(embed_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, n_tokens, NORM_THREADS, smem, stream,
                  (const __nv_bfloat16*)table, ids, (const __nv_bfloat16*)weight, out, hidden, eps);
  else if (dtype == DT_BF16 && weight_dtype == DT_F32)
    launch_kernel(embed_rmsnorm_kernel<__nv_bfloat16, float>, n_tokens, NORM_THREADS, smem, stream,
                  (const __nv_bfloat16*)table, ids, (const float*)weight, out, hidden, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// One block per output row r (stream row src = row_index[r] or r).  With y: the partial results are
// added in index order, normed with `post_w` and added into the stream, which is written back.
// With out: the norm of the (new) stream row with `next_w`.
template <typename TW, typename TO>
__global__ void __launch_bounds__(NORM_THREADS)
postnorm_add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ y, int n_partials,
                            long long partial_stride, const TW* __restrict__ post_w, float post_eps,
                            const TW* __restrict__ next_w, float next_eps, TO* __restrict__ out,
                            const int32_t* __restrict__ row_index, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + hidden;
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  float* x = residual + src * hidden;
  float sq = 0.0f;
  if (y) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = 0.0f;
      for (int p = 0; p < n_partials; ++p) v += y[p * partial_stride + src * hidden + i];
      row_cache[i] = v;
      sq += v * v;
    }
    const float s1 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + post_eps);
    sq = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = x[i] + row_cache[i] * s1 * to_float(post_w[i]);
      x[i] = v;
      row_cache[i] = v;
      sq += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = x[i];
      row_cache[i] = v;
      sq += v * v;
    }
  }
  if (!out) return;
  const float s2 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + next_eps);
  TO* dst = out + (long long)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    dst[i] = from_float<TO>(row_cache[i] * s2 * to_float(next_w[i]));
}

// The same with 16-byte accesses for bfloat16 weights and output: width a multiple of 4 up to 16 x the
// block size, every row's pieces in registers (a thread's sums are formed in another order than
// the kernel above forms them: float32 rounding under a bfloat16 result).
__device__ __forceinline__ float4 bf16x4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

__global__ void __launch_bounds__(NORM_THREADS)
postnorm_add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ y, int n_partials,
                                long long partial_stride, const __nv_bfloat16* __restrict__ post_w, float post_eps,
                                const __nv_bfloat16* __restrict__ next_w, float next_eps, __nv_bfloat16* __restrict__ out,
                                const int32_t* __restrict__ row_index, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const long long src = row_index ? row_index[r] : r;
  float4* x = reinterpret_cast<float4*>(residual + src * hidden);
  const int n4 = hidden / 4;
  float4 v[4], old[4];
  float sq = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * NORM_THREADS;
    if (i < n4) {
      old[j] = x[i];
      float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int p = 0; p < n_partials; ++p) {
        const float4 d = reinterpret_cast<const float4*>(y + p * partial_stride + src * hidden)[i];
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      }
      v[j] = a;
      sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  const float s1 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + post_eps);
  sq = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * NORM_THREADS;
    if (i < n4) {
      const float4 w = bf16x4(post_w + 4 * i);
      float4 a = old[j];
      a.x += v[j].x * s1 * w.x; a.y += v[j].y * s1 * w.y; a.z += v[j].z * s1 * w.z; a.w += v[j].w * s1 * w.w;
      x[i] = a;
      v[j] = a;
      sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  if (!out) return;
  const float s2 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + next_eps);
  uint2* dst = reinterpret_cast<uint2*>(out + (long long)r * hidden);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * NORM_THREADS;
    if (i < n4) {
      const float4 w = bf16x4(next_w + 4 * i);
      const __nv_bfloat162 lo = __floats2bfloat162_rn(v[j].x * s2 * w.x, v[j].y * s2 * w.y);
      const __nv_bfloat162 hi = __floats2bfloat162_rn(v[j].z * s2 * w.z, v[j].w * s2 * w.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      dst[i] = o;
    }
  }
}

// dtype: the element type of the norm weights and of `out` (the step's activation type).
extern "C" int llm_postnorm_add_rmsnorm(float* residual, const float* y, int n_partials, long long partial_stride,
                                        const void* post_w, float post_eps, const void* next_w, float next_eps,
                                        void* out, int dtype, const int32_t* row_index, int rows, int hidden,
                                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  LLM_HOST_CHECK(smem <= 48 * 1024, ERR_BAD_SIZE);
  LLM_HOST_CHECK((!y || post_w) && (!out || next_w), ERR_BAD_SIZE);
  if (dtype == DT_F32)
    launch_kernel(postnorm_add_rmsnorm_kernel<float, float>, rows, NORM_THREADS, smem, stream, residual, y, n_partials,
                  partial_stride, (const float*)post_w, post_eps, (const float*)next_w, next_eps, (float*)out, row_index,
                  hidden);
  else if (dtype == DT_BF16 && y && hidden % 4 == 0 && hidden <= 16 * NORM_THREADS && partial_stride % 4 == 0 &&
           ((uintptr_t)residual % 16) == 0 && ((uintptr_t)y % 16) == 0 && ((uintptr_t)post_w % 8) == 0 &&
           ((uintptr_t)next_w % 8) == 0 && ((uintptr_t)out % 8) == 0)
    launch_kernel(postnorm_add_rmsnorm_vec_kernel, rows, NORM_THREADS, 0, stream, residual, y, n_partials, partial_stride,
                  (const __nv_bfloat16*)post_w, post_eps, (const __nv_bfloat16*)next_w, next_eps, (__nv_bfloat16*)out,
                  row_index, hidden);
  else if (dtype == DT_BF16)
    launch_kernel(postnorm_add_rmsnorm_kernel<__nv_bfloat16, __nv_bfloat16>, rows, NORM_THREADS, smem, stream, residual,
                  y, n_partials, partial_stride, (const __nv_bfloat16*)post_w, post_eps, (const __nv_bfloat16*)next_w,
                  next_eps, (__nv_bfloat16*)out, row_index, hidden);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
