// The boundary between two sublayers of a stream that norms on both sides of every sublayer, gates
// every sublayer's result, and hands a weighted sum of all earlier layers' results on to the next layer:
//
//   y <- y * sigmoid(g + b)            (g the gate's projection of the sublayer's own input, b its bias)
//   x <- x + rms_norm(y) * p           (p the weight of the norm behind the sublayer)
//   X_k <- x;  x <- sum_{j <= k} a[j] X_j      (at a layer's end: X_0 is the embedding's output, X_k layer k - 1's)
//   h = rms_norm(x) * w                (the next sublayer's input, or the final norm of the wanted rows)
//
// as one kernel; each of the four steps may be left out.  rms_norm(v) = v / sqrt(mean(v^2) + eps).
// The stream, every X_j, the gate, the sums of squares and the factors p, w, a are float32.  One block of
// a fixed size per row: the order of every sum depends on the width only.

#include "common.cuh"

#include <math.h>

#define GS_THREADS 256

struct GatedStep {
  float* residual;            // [rows, hidden]
  const float* y;             // the sublayer's result as partial sums [n_partials][rows, hidden], or null
  int n_partials;
  long long partial_stride;
  const void* gate;           // [rows] x hidden pre-activations, rows `gate_stride` apart, or null
  long long gate_stride;
  const float* gate_bias;     // [hidden] or null
  const float* post_w;        // [hidden]
  float post_eps;
  float* history;             // entries `history_stride` elements apart, each [rows, hidden]
  long long history_stride;
  int store_at;               // entry that receives the row as it stands after the add (-1: none)
  const float* mix_w;         // [mix_n] or null: the row becomes sum_j mix_w[j] * entry j (entry mix_n - 1 is `store_at`)
  int mix_n;
  const float* next_w;        // [hidden] or null
  float next_eps;
  void* out;                  // [rows, hidden] or null
  const int32_t* row_index;   // output row r reads stream row row_index[r] (null: r)
  int hidden;
};

template <typename TG, typename TO>
__global__ void __launch_bounds__(GS_THREADS) gated_step_kernel(GatedStep a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_cache[];  // hidden floats + 32 scratch
  float* scratch = row_cache + a.hidden;
  const int r = blockIdx.x, hidden = a.hidden;
  const long long src = a.row_index ? a.row_index[r] : r;
  float* x = a.residual + src * hidden;
  float sq = 0.0f;
  if (a.y) {
    const TG* g = a.gate ? (const TG*)a.gate + src * a.gate_stride : nullptr;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = 0.0f;
      for (int p = 0; p < a.n_partials; ++p) v += a.y[p * a.partial_stride + src * hidden + i];
      if (g) v *= 1.0f / (1.0f + expf(-(to_float(g[i]) + (a.gate_bias ? a.gate_bias[i] : 0.0f))));
      row_cache[i] = v;
      sq += v * v;
    }
    const float s1 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + a.post_eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_cache[i] = x[i] + row_cache[i] * s1 * a.post_w[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_cache[i] = x[i];
  }
  // (a thread touches the same entries i in every loop, so no barrier is needed between them)
  if (a.store_at >= 0) {
    float* dst = a.history + a.store_at * a.history_stride + src * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = row_cache[i];
  }
  if (a.mix_w) {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = 0.0f;
      for (int j = 0; j + 1 < a.mix_n; ++j) v = fmaf(a.mix_w[j], a.history[j * a.history_stride + src * hidden + i], v);
      row_cache[i] = fmaf(a.mix_w[a.mix_n - 1], row_cache[i], v);
    }
  }
  sq = 0.0f;
  const bool changed = a.y || a.mix_w;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_cache[i];
    if (changed) x[i] = v;
    sq += v * v;
  }
  if (!a.out) return;
  const float s2 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + a.next_eps);
  TO* dst = (TO*)a.out + (long long)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_float<TO>(row_cache[i] * s2 * a.next_w[i]);
}

// The same in pieces of four entries (16-byte loads and stores of float32, 8-byte ones of bfloat16): a width
// that is a multiple of four, every pointer aligned for its pieces.  A thread keeps its pieces in registers
// (up to GS_PIECES of them: widths up to 4 * GS_PIECES * the block size); the sums of a thread are formed in
// the order of the kernel above, entry by entry within a piece.
#define GS_PIECES 4

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

template <typename TG, typename TO, int THREADS>
__global__ void __launch_bounds__(THREADS) gated_step_vec_kernel(GatedStep a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int r = blockIdx.x, hidden = a.hidden, n4 = hidden / 4;
  const long long src = a.row_index ? a.row_index[r] : r;
  float* x = a.residual + src * hidden;
  float4 v[GS_PIECES];
  float sq = 0.0f;
  if (a.y) {
    const TG* g = a.gate ? (const TG*)a.gate + src * a.gate_stride : nullptr;
#pragma unroll
    for (int j = 0; j < GS_PIECES; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i >= n4) break;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float* yp = a.y + src * hidden + 4 * i;
#pragma unroll 4
      for (int p = 0; p < a.n_partials; ++p) {
        const float4 d = load4(yp + p * a.partial_stride);
        acc.x += d.x; acc.y += d.y; acc.z += d.z; acc.w += d.w;
      }
      if (g) {
        const float4 gv = load4(g + 4 * i);
        const float4 b = a.gate_bias ? load4(a.gate_bias + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        acc.x *= sigmoid_f(gv.x + b.x); acc.y *= sigmoid_f(gv.y + b.y);
        acc.z *= sigmoid_f(gv.z + b.z); acc.w *= sigmoid_f(gv.w + b.w);
      }
      v[j] = acc;
      sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
    const float s1 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + a.post_eps);
#pragma unroll
    for (int j = 0; j < GS_PIECES; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i >= n4) break;
      const float4 old = load4(x + 4 * i), w = load4(a.post_w + 4 * i);
      v[j] = make_float4(old.x + v[j].x * s1 * w.x, old.y + v[j].y * s1 * w.y, old.z + v[j].z * s1 * w.z,
                         old.w + v[j].w * s1 * w.w);
    }
  } else {
#pragma unroll
    for (int j = 0; j < GS_PIECES; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i >= n4) break;
      v[j] = load4(x + 4 * i);
    }
  }
  if (a.store_at >= 0) {
    float* dst = a.history + a.store_at * a.history_stride + src * hidden;
#pragma unroll
    for (int j = 0; j < GS_PIECES; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i >= n4) break;
      store4(dst + 4 * i, v[j]);
    }
  }
  if (a.mix_w) {
    const float own = a.mix_w[a.mix_n - 1];
#pragma unroll
    for (int j = 0; j < GS_PIECES; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i >= n4) break;
      float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      const float* hp = a.history + src * hidden + 4 * i;
#pragma unroll 4
      for (int k = 0; k + 1 < a.mix_n; ++k) {
        const float4 d = load4(hp + k * a.history_stride);
        const float w = a.mix_w[k];
        acc.x = fmaf(w, d.x, acc.x); acc.y = fmaf(w, d.y, acc.y); acc.z = fmaf(w, d.z, acc.z); acc.w = fmaf(w, d.w, acc.w);
      }
      v[j] = make_float4(fmaf(own, v[j].x, acc.x), fmaf(own, v[j].y, acc.y), fmaf(own, v[j].z, acc.z), fmaf(own, v[j].w, acc.w));
    }
  }
  sq = 0.0f;
  const bool changed = a.y || a.mix_w;
#pragma unroll
  for (int j = 0; j < GS_PIECES; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i >= n4) break;
    if (changed) store4(x + 4 * i, v[j]);
    sq += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
  }
  if (!a.out) return;
  const float s2 = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + a.next_eps);
  TO* dst = (TO*)a.out + (long long)r * hidden;
#pragma unroll
  for (int j = 0; j < GS_PIECES; ++j) {
    const int i = threadIdx.x + j * THREADS;
    if (i >= n4) break;
    const float4 w = load4(a.next_w + 4 * i);
    store4(dst + 4 * i, make_float4(v[j].x * s2 * w.x, v[j].y * s2 * w.y, v[j].z * s2 * w.z, v[j].w * s2 * w.w));
  }
}

// gate_dtype: element type of the gate's projection; out_dtype: of `out`.
extern "C" int llm_gated_sandwich_step(float* residual, const float* y, int n_partials, long long partial_stride,
                                       const void* gate, int gate_dtype, long long gate_stride, const float* gate_bias,
                                       const float* post_w, float post_eps, float* history, long long history_stride,
                                       int store_at, const float* mix_w, int mix_n, const float* next_w, float next_eps,
                                       void* out, int out_dtype, const int32_t* row_index, int rows, int hidden,
                                       cudaStream_t stream) {
  if (rows <= 0) return 0;
  const size_t smem = (size_t)(hidden + 32) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
  LLM_HOST_CHECK((!y || post_w) && (!out || next_w) && (!gate || y), ERR_BAD_SIZE);
  LLM_HOST_CHECK((store_at < 0 && !mix_w) || history, ERR_BAD_SIZE);
  LLM_HOST_CHECK(!mix_w || (mix_n >= 1 && store_at == mix_n - 1), ERR_BAD_SIZE);
  GatedStep a{residual, y, n_partials, partial_stride, gate, gate_stride, gate_bias, post_w, post_eps, history,
              history_stride, store_at, mix_w, mix_n, next_w, next_eps, out, row_index, hidden};
  // pieces of four where every pointer allows them; few rows: a block of 1,024 threads a row, so that a
  // step of a handful of tokens does not wait on eight dependent loads a thread
  auto aligned = [](const void* p, int bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; };
  const int gbytes = gate_dtype == DT_BF16 ? 8 : 16, obytes = out_dtype == DT_BF16 ? 8 : 16;
  const bool vec = hidden % 4 == 0 && hidden <= 4 * GS_PIECES * 256 && aligned(residual, 16) && aligned(y, 16) &&
                   partial_stride % 4 == 0 && aligned(gate, gbytes) && gate_stride % 4 == 0 && aligned(gate_bias, 16) &&
                   aligned(post_w, 16) && aligned(history, 16) && history_stride % 4 == 0 && aligned(next_w, 16) &&
                   aligned(out, obytes);
  const bool wide = vec && rows <= 64 && hidden >= 2048;
#define STEP(TG, TO)                                                                                              \
  do {                                                                                                            \
    if (wide) {                                                                                                   \
      launch_kernel(gated_step_vec_kernel<TG, TO, 1024>, rows, 1024, 0, stream, a);                               \
    } else if (vec) {                                                                                             \
      launch_kernel(gated_step_vec_kernel<TG, TO, 256>, rows, 256, 0, stream, a);                                 \
    } else {                                                                                                      \
      if (smem > 48 * 1024)                                                                                       \
        cudaFuncSetAttribute(gated_step_kernel<TG, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      launch_kernel(gated_step_kernel<TG, TO>, rows, GS_THREADS, smem, stream, a);                                \
    }                                                                                                             \
  } while (0)
  const int gd = gate ? gate_dtype : out_dtype;
  if (gd == DT_F32 && out_dtype == DT_F32) STEP(float, float);
  else if (gd == DT_BF16 && out_dtype == DT_BF16) STEP(__nv_bfloat16, __nv_bfloat16);
  else if (gd == DT_F32 && out_dtype == DT_BF16) STEP(float, __nv_bfloat16);
  else if (gd == DT_BF16 && out_dtype == DT_F32) STEP(__nv_bfloat16, float);
  else return ERR_BAD_DTYPE;
#undef STEP
  return launch_status();
}
