// The pieces of a Mamba-2 mixer (state-space duality) around the engine's state scan.  The input
// projection of a token is [z: inner | x: inner | B: G * N | C: G * N | dt: H] with inner = H * P.
//
//   [x | B | C] <- silu(bias + causal convolution over time, per channel, `taps` taps)
//   dt_h <- softplus(dt_h + dt_bias_h);   a_h = exp(-exp(A_log_h) * dt_h)
//   S_h <- a_h S_h + (dt_h B_g) x_h^T  (N x P, g = h / (H / G));   y_h = S_h^T C_g + D_h x_h
//   out = rms_norm in `parts` equal parts of (y * silu(z)) * w
//
// mamba2_operands makes the scan's float32 operands from the projection (decay per token and head,
// k = B of the head's group, v = dt * x, q = C of the head's group) and keeps x for the D term; the scan
// (linear_attention.cu) walks the state; mamba2_finish adds D x, gates, norms and rounds.  The
// convolution's last taps - 1 inputs per request live in a state slot as a ring indexed by position
// (written by conv_ring_write of biased_attention.cu after this step's convolution has read it).
// Everything after the stored projection is float32.

#include "common.cuh"

#include <math.h>

__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(256)
mamba2_operands_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ conv_w,
                       const float* __restrict__ conv_b, int taps, const float* __restrict__ ring,
                       const float* __restrict__ dt_bias, const float* __restrict__ a_log, float* __restrict__ qf,
                       float* __restrict__ kf, float* __restrict__ vf, float* __restrict__ xc, float* __restrict__ decay,
                       const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_q_start, int H, int P, int N,
                       int G) {
  pdl_launch_dependents();
  extern __shared__ float sm[];      // C conv channels, then H step sizes
  const int inner = H * P, C = inner + 2 * G * N;
  float* ys = sm;
  float* dts = sm + C;
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = row_seq[t], p = positions[t];
  const int slot = seq_slot[seq];
  const int p0 = p - (t - seq_q_start[seq]);
  const int hist = taps - 1;
  const float* ring_slot = ring + (long long)slot * (hist > 0 ? hist : 1) * C;
  const T* row = u + (long long)t * u_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = softplus_f(to_float(row[inner + C + h]) + dt_bias[h]);
    dts[h] = dt;
    decay[(long long)t * H + h] = expf(-expf(a_log[h]) * dt);
  }
  const bool inside = p - hist >= p0;      // all taps inside the step's own rows
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float y = conv_b[c];
    const float* w = conv_w + (long long)c * taps;
    if (inside) {
      const T* col = row + inner + c - (long long)hist * u_stride;
      for (int j = 0; j < taps; ++j) y += w[j] * to_float(col[(long long)j * u_stride]);
    } else {
      for (int j = 0; j < taps; ++j) {
        const int x = p - hist + j;
        if (x < 0) continue;
        const float val = x >= p0 ? to_float(u[(long long)(t - (p - x)) * u_stride + inner + c])
                                  : ring_slot[(long long)(x % hist) * C + c];
        y += w[j] * val;
      }
    }
    ys[c] = silu_f(y);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < inner; c += blockDim.x) {
    const float x = ys[c];
    xc[(long long)t * inner + c] = x;
    vf[(long long)t * inner + c] = dts[c / P] * x;
  }
  const int per_group = H / G;
  for (int i = threadIdx.x; i < H * N; i += blockDim.x) {
    const int h = i / N, n = i - h * N, g = h / per_group;
    kf[(long long)t * H * N + i] = ys[inner + g * N + n];
    qf[(long long)t * H * N + i] = ys[inner + G * N + g * N + n];
  }
}

extern "C" int llm_mamba2_operands(const void* u, int dtype, long long u_stride, const float* conv_w, const float* conv_b,
                                   int taps, const float* ring, const float* dt_bias, const float* a_log, float* qf,
                                   float* kf, float* vf, float* xc, float* decay, const int32_t* positions,
                                   const int32_t* row_seq, const int32_t* seq_slot, const int32_t* seq_q_start,
                                   int n_tokens, int H, int P, int N, int G, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(taps >= 1 && H >= 1 && G >= 1 && H % G == 0 && P >= 1 && N >= 1, ERR_BAD_SIZE);
  const size_t smem = (size_t)(H * P + 2 * G * N + H) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
#define LAUNCH(T)                                                                                                   \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(mamba2_operands_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    launch_kernel(mamba2_operands_kernel<T>, n_tokens, 256, smem, stream, (const T*)u, u_stride, conv_w, conv_b, taps, \
                  ring, dt_bias, a_log, qf, kf, vf, xc, decay, positions, row_seq, seq_slot, seq_q_start, H, P, N, G); \
  } while (0)
  if (dtype == DT_F32) LAUNCH(float);
  else if (dtype == DT_BF16) LAUNCH(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}

// One block per token; a warp takes the norm's parts in turn.  y = scanned + D x, times silu(z), each
// part divided by its own root mean square, times w.
template <typename T>
__global__ void __launch_bounds__(256)
mamba2_finish_kernel(const float* __restrict__ scanned, const float* __restrict__ xc, const float* __restrict__ d_skip,
                     const T* __restrict__ z, long long z_stride, const float* __restrict__ norm_w, T* __restrict__ out,
                     long long out_stride, int inner, int P, int parts, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const int size = inner / parts;
  for (int part = warp; part < parts; part += n_warps) {
    const int c0 = part * size;
    float sq = 0.0f;
    for (int c = c0 + lane; c < c0 + size; c += 32) {
      const float y = (scanned[(long long)t * inner + c] + d_skip[c / P] * xc[(long long)t * inner + c]) *
                      silu_f(to_float(z[(long long)t * z_stride + c]));
      sq += y * y;
    }
    const float s = 1.0f / sqrtf(warp_sum(sq) / (float)size + eps);
    for (int c = c0 + lane; c < c0 + size; c += 32) {
      const float y = (scanned[(long long)t * inner + c] + d_skip[c / P] * xc[(long long)t * inner + c]) *
                      silu_f(to_float(z[(long long)t * z_stride + c]));
      out[(long long)t * out_stride + c] = from_float<T>(y * s * norm_w[c]);
    }
  }
}

extern "C" int llm_mamba2_finish(const float* scanned, const float* xc, const float* d_skip, const void* z, int dtype,
                                 long long z_stride, const float* norm_w, void* out, long long out_stride, int n_tokens,
                                 int inner, int P, int parts, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(parts >= 1 && inner % parts == 0 && P >= 1 && inner % P == 0, ERR_BAD_SIZE);
  const int threads = parts >= 8 ? 256 : (parts >= 4 ? 128 : (parts >= 2 ? 64 : 32));
  if (dtype == DT_F32)
    launch_kernel(mamba2_finish_kernel<float>, n_tokens, threads, 0, stream, scanned, xc, d_skip, (const float*)z,
                  z_stride, norm_w, (float*)out, out_stride, inner, P, parts, eps);
  else if (dtype == DT_BF16)
    launch_kernel(mamba2_finish_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, scanned, xc, d_skip,
                  (const __nv_bfloat16*)z, z_stride, norm_w, (__nv_bfloat16*)out, out_stride, inner, P, parts, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}
