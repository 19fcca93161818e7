// The pieces of a Mamba-2 mixer (state-space duality) around the engine's state scan.  The input
// projection of a token is [z: inner | x: inner | B: G * N | C: G * N | dt: H] with inner = H * P.
//
//   [x | B | C] <- silu(bias + causal convolution over time, per channel, `taps` taps)
//   dt_h <- softplus(dt_h + dt_bias_h);   a_h = exp(-exp(A_log_h) * dt_h)
//   S_h <- a_h S_h + (dt_h B_g) x_h^T  (N x P, g = h / (H / G));   y_h = S_h^T C_g + D_h x_h
//   out = rms_norm in `parts` equal parts of (y * silu(z)) * w
//
// (With `compact`, mamba2_operands instead leaves [x | B | C] once per token in bfloat16 with the step sizes and
// the decays' logarithms, for the chunked walk on the tensor cores of mamba2_chunked.cu.)
// mamba2_operands makes the scan's float32 operands from the projection (decay per token and head,
// k = B of the head's group, v = dt * x, q = C of the head's group) and keeps x for the D term; the scan
// (linear_attention.cu) walks the state; mamba2_finish adds D x, gates, norms and rounds.  The
// convolution's last inputs per request live in a state slot as a ring of `taps` entries indexed by
// position % taps (one entry more than a convolution reads back, so the entry a token writes is never one
// that the same step still reads); mamba2_ring_write fills it after a step's convolution.
// mamba2_step stands for operands, ring write and scan in steps of one token per request.
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
                       int G, __nv_bfloat16* __restrict__ compact, float* __restrict__ dt_out, float* __restrict__ la_out) {
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
  const float* ring_slot = ring + (long long)slot * taps * C;
  const T* row = u + (long long)t * u_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = softplus_f(to_float(row[inner + C + h]) + dt_bias[h]);
    dts[h] = dt;
    if (compact) {      // the chunked walk takes the step size and the decay's logarithm
      dt_out[(long long)t * H + h] = dt;
      la_out[(long long)t * H + h] = -expf(a_log[h]) * dt;
    } else {
      decay[(long long)t * H + h] = expf(-expf(a_log[h]) * dt);
    }
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
                                  : ring_slot[(long long)(x % taps) * C + c];
        y += w[j] * val;
      }
    }
    ys[c] = silu_f(y);
  }
  __syncthreads();
  if (compact) {
    // [x | B | C] once, rounded to bfloat16 (activations of the convolution), for the chunked walk
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      compact[(long long)t * C + c] = __float2bfloat16_rn(ys[c]);
      if (c < inner) xc[(long long)t * inner + c] = ys[c];
    }
    return;
  }
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
                                   int n_tokens, int H, int P, int N, int G, void* compact, float* dt_out, float* la_out,
                                   cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(taps >= 1 && H >= 1 && G >= 1 && H % G == 0 && P >= 1 && N >= 1, ERR_BAD_SIZE);
  const size_t smem = (size_t)(H * P + 2 * G * N + H) * sizeof(float);
  LLM_HOST_CHECK(smem <= 200 * 1024, ERR_BAD_SIZE);
#define LAUNCH(T)                                                                                                   \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(mamba2_operands_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    launch_kernel(mamba2_operands_kernel<T>, n_tokens, 256, smem, stream, (const T*)u, u_stride, conv_w, conv_b, taps, \
                  ring, dt_bias, a_log, qf, kf, vf, xc, decay, positions, row_seq, seq_slot, seq_q_start, H, P, N, G, \
                  (__nv_bfloat16*)compact, dt_out, la_out);                                                         \
  } while (0)
  if (dtype == DT_F32) LAUNCH(float);
  else if (dtype == DT_BF16) LAUNCH(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}

// One block per (token, part of the norm).  y = scanned + D x, times silu(z), the part divided by its own root
// mean square, times w.
template <typename T>
__global__ void __launch_bounds__(256)
mamba2_finish_kernel(const float* __restrict__ scanned, const float* __restrict__ xc, const float* __restrict__ d_skip,
                     const T* __restrict__ z, long long z_stride, const float* __restrict__ norm_w, T* __restrict__ out,
                     long long out_stride, int inner, int P, int parts, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x, part = blockIdx.y;
  const int size = inner / parts, c0 = part * size;
  float sq = 0.0f;
  for (int c = c0 + threadIdx.x; c < c0 + size; c += blockDim.x) {
    const float y = (scanned[(long long)t * inner + c] + d_skip[c / P] * xc[(long long)t * inner + c]) *
                    silu_f(to_float(z[(long long)t * z_stride + c]));
    sq += y * y;
  }
  const float s = 1.0f / sqrtf(block_sum(sq, scratch) / (float)size + eps);
  for (int c = c0 + threadIdx.x; c < c0 + size; c += blockDim.x) {
    const float y = (scanned[(long long)t * inner + c] + d_skip[c / P] * xc[(long long)t * inner + c]) *
                    silu_f(to_float(z[(long long)t * z_stride + c]));
    out[(long long)t * out_stride + c] = from_float<T>(y * s * norm_w[c]);
  }
}

extern "C" int llm_mamba2_finish(const float* scanned, const float* xc, const float* d_skip, const void* z, int dtype,
                                 long long z_stride, const float* norm_w, void* out, long long out_stride, int n_tokens,
                                 int inner, int P, int parts, float eps, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(parts >= 1 && parts <= 65535 && inner % parts == 0 && P >= 1 && inner % P == 0, ERR_BAD_SIZE);
  const int size = inner / parts;
  const int threads = size >= 1024 ? 256 : (size >= 256 ? 128 : (size >= 64 ? 64 : 32));
  const dim3 grid(n_tokens, parts);
  if (dtype == DT_F32)
    launch_kernel(mamba2_finish_kernel<float>, grid, threads, 0, stream, scanned, xc, d_skip, (const float*)z,
                  z_stride, norm_w, (float*)out, out_stride, inner, P, parts, eps);
  else if (dtype == DT_BF16)
    launch_kernel(mamba2_finish_kernel<__nv_bfloat16>, grid, threads, 0, stream, scanned, xc, d_skip,
                  (const __nv_bfloat16*)z, z_stride, norm_w, (__nv_bfloat16*)out, out_stride, inner, P, parts, eps);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// The projection rows [x | B | C] of each request's last taps - 1 positions go into its ring (entry position %
// taps).  Grid (row, slice of channels).
template <typename T>
__global__ void __launch_bounds__(256)
mamba2_ring_write_kernel(const T* __restrict__ u, long long u_stride, float* __restrict__ ring, int taps, int C,
                         const int32_t* __restrict__ positions, const int32_t* __restrict__ row_seq,
                         const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_kv_len) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int seq = row_seq[t], p = positions[t];
  const int end = seq_kv_len[seq] > 0 ? seq_kv_len[seq] : p + 1;   // an idle row stands for itself
  if (p < end - (taps - 1)) return;
  float* dst = ring + ((long long)seq_slot[seq] * taps + (p % taps)) * C;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x)
    dst[c] = to_float(u[(long long)t * u_stride + c]);
}

extern "C" int llm_mamba2_ring_write(const void* u, int dtype, long long u_stride, float* ring, int taps, int channels,
                                     const int32_t* positions, const int32_t* row_seq, const int32_t* seq_slot,
                                     const int32_t* seq_kv_len, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || taps <= 1) return 0;
  const dim3 grid(n_tokens, n_tokens >= 64 ? 1 : (channels + 1023) / 1024);
  if (dtype == DT_F32)
    launch_kernel(mamba2_ring_write_kernel<float>, grid, 256, 0, stream, (const float*)u, u_stride, ring, taps, channels,
                  positions, row_seq, seq_slot, seq_kv_len);
  else if (dtype == DT_BF16)
    launch_kernel(mamba2_ring_write_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)u, u_stride, ring,
                  taps, channels, positions, row_seq, seq_slot, seq_kv_len);
  else
    return ERR_BAD_DTYPE;
  return launch_status();
}

// ---------------------------------------------------------------- one token per request

// Grid (sequence, head); a block does all of one head of one token up to the scan's result: convolution and
// silu of its x channels and of its group's B and C channels, step size and decay, the state update S <- a S +
// dt B x^T in place, S^T C.  It leaves S^T C and x where mamba2_finish reads them, and puts the token's raw
// inputs into the ring (a group's B and C by the block of the group's first head).  A thread owns rows n, n + R,
// ... of one state column; the column's partial sums meet in shared memory and are added in a fixed order.
#define M2S_THREADS 256

template <typename T>
__global__ void __launch_bounds__(M2S_THREADS)
mamba2_step_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ conv_w,
                   const float* __restrict__ conv_b, int taps, float* __restrict__ ring, const float* __restrict__ dt_bias,
                   const float* __restrict__ a_log, float* __restrict__ state, float* __restrict__ scanned,
                   float* __restrict__ xc, const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_slot,
                   const int32_t* __restrict__ seq_q_start, int H, int P, int N, int G, int write_ring) {
  pdl_launch_dependents();
  extern __shared__ float sm[];
  const int inner = H * P, C = inner + 2 * G * N, per_group = H / G;
  const int h = blockIdx.y, g = h / per_group;
  const int W = P < M2S_THREADS ? P : M2S_THREADS, R = M2S_THREADS / W;
  float* xs = sm;                       // [P]   x after convolution and silu
  float* bs = xs + P;                   // [N]
  float* cs = bs + N;                   // [N]
  float* part = cs + N;                 // [R * W] partial sums of a column block
  pdl_wait();
  const int seq = blockIdx.x, t = seq_q_start[seq];
  const int p = positions[t], slot = seq_slot[seq], hist = taps - 1;
  const T* row = u + (long long)t * u_stride;
  float* ring_slot = ring + (long long)slot * taps * C;
  const float dt = softplus_f(to_float(row[inner + C + h]) + dt_bias[h]);
  const float decay = expf(-expf(a_log[h]) * dt);
  const bool owner = g * per_group == h;      // the group's first head keeps the group's B and C in the ring
  for (int i = threadIdx.x; i < P + 2 * N; i += blockDim.x) {
    int c;
    if (i < P) c = h * P + i;
    else {
      const int k = i - P, which = k / N;
      c = inner + which * G * N + g * N + (k - which * N);
    }
    const float now = to_float(row[inner + c]);
    float y = conv_b[c] + conv_w[(long long)c * taps + hist] * now;
    for (int j = 0; j < hist; ++j) {
      const int x = p - hist + j;
      if (x >= 0) y += conv_w[(long long)c * taps + j] * ring_slot[(long long)(x % taps) * C + c];
    }
    if (write_ring && hist > 0 && (i < P || owner)) ring_slot[(long long)(p % taps) * C + c] = now;
    xs[i] = silu_f(y);      // xs, bs and cs lie back to back
  }
  __syncthreads();
  for (int i = threadIdx.x; i < P; i += blockDim.x) xc[(long long)t * inner + h * P + i] = xs[i];
  const int rg = threadIdx.x / W, lc = threadIdx.x % W;
  float* S = state + ((long long)slot * H + h) * N * P;
  for (int c0 = 0; c0 < P; c0 += W) {
    const int col = c0 + lc;
    float acc = 0.0f;
    if (rg < R && col < P) {
      const float xv = dt * xs[col];
#pragma unroll 4
      for (int n = rg; n < N; n += R) {
        const float v = fmaf(decay, S[(long long)n * P + col], bs[n] * xv);
        S[(long long)n * P + col] = v;
        acc = fmaf(v, cs[n], acc);
      }
    }
    if (rg < R) part[rg * W + lc] = acc;
    __syncthreads();
    if (threadIdx.x < W && col < P) {
      float sum = 0.0f;
      for (int k = 0; k < R; ++k) sum += part[k * W + lc];
      scanned[(long long)t * inner + h * P + col] = sum;
    }
    __syncthreads();
  }
}

extern "C" long long llm_mamba2_step_shared_bytes(int H, int P, int N, int G) {
  if (G < 1 || H % G) return -1;
  const int W = P < M2S_THREADS ? P : M2S_THREADS, R = M2S_THREADS / W;
  return (long long)(P + 2 * N + R * W) * 4;
}

extern "C" int llm_mamba2_step(const void* u, int dtype, long long u_stride, const float* conv_w, const float* conv_b,
                               int taps, float* ring, const float* dt_bias, const float* a_log, float* state,
                               float* scanned, float* xc, const int32_t* positions, const int32_t* seq_slot,
                               const int32_t* seq_q_start, int n_seqs, int H, int P, int N, int G, int write_ring,
                               cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  const long long smem = llm_mamba2_step_shared_bytes(H, P, N, G);
  LLM_HOST_CHECK(smem > 0 && smem <= 200 * 1024 && taps >= 1 && H <= 65535, ERR_BAD_SIZE);
  const dim3 grid(n_seqs, H);
#define LAUNCH(T)                                                                                                   \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(mamba2_step_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    launch_kernel(mamba2_step_kernel<T>, grid, M2S_THREADS, (size_t)smem, stream, (const T*)u, u_stride, conv_w, conv_b, \
                  taps, ring, dt_bias, a_log, state, scanned, xc, positions, seq_slot, seq_q_start, H, P, N, G,      \
                  write_ring);                                                                                       \
  } while (0)
  if (dtype == DT_F32) LAUNCH(float);
  else if (dtype == DT_BF16) LAUNCH(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}
