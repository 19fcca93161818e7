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
// convolution's last inputs per request live in a state slot as a ring of `taps` entries indexed by
// position % taps (one entry more than a convolution reads back, so the entry a token writes is never one
// that the same step still reads); mamba2_ring_write fills it after a step's convolution.
// mamba2_step does all of it in one kernel for steps of one token per request.
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
  const float* ring_slot = ring + (long long)slot * taps * C;
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
                                  : ring_slot[(long long)(x % taps) * C + c];
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

// ---------------------------------------------------------------- one token per request, one kernel

// Grid (sequence, part of the norm); a block takes the heads of its part (the norm's parts hold whole
// heads), all of one token: convolution and silu of its x channels and of the B and C channels of the
// groups its heads read, step sizes and decays, the state update S <- a S + dt B x^T in place, y = S^T C
// + D x, the gate, the part's norm, the weight.  It also puts the token's raw [x | B | C] into the ring
// (a group's B and C by the block that holds the group's first head).  A thread owns rows n, n + R, ... of
// one state column; the column's partial sums meet in shared memory and are added in a fixed order.
#define M2S_THREADS 256

template <typename T>
__global__ void __launch_bounds__(M2S_THREADS)
mamba2_step_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ conv_w,
                   const float* __restrict__ conv_b, int taps, float* __restrict__ ring, const float* __restrict__ dt_bias,
                   const float* __restrict__ a_log, const float* __restrict__ d_skip, const float* __restrict__ norm_w,
                   float* __restrict__ state, T* __restrict__ out, long long out_stride,
                   const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_slot,
                   const int32_t* __restrict__ seq_q_start, int H, int P, int N, int G, int parts, float eps, int write_ring) {
  pdl_launch_dependents();
  extern __shared__ float sm[];
  const int inner = H * P, C = inner + 2 * G * N, hp = H / parts, per_group = H / G;
  const int h0 = blockIdx.y * hp, g0 = h0 / per_group, g1 = (h0 + hp - 1) / per_group, ng = g1 - g0 + 1;
  const int W = P < M2S_THREADS ? P : M2S_THREADS, R = M2S_THREADS / W;
  float* xs = sm;                       // [hp * P]   x after convolution and silu
  float* bs = xs + hp * P;              // [ng * N]
  float* cs = bs + ng * N;              // [ng * N]
  float* ys = cs + ng * N;              // [hp * P]
  float* dts = ys + hp * P;             // [hp], then decays [hp]
  float* part = dts + 2 * hp;           // [R * W] partial sums of a column block, then 32 scratch
  float* scratch = part + R * W;
  pdl_wait();
  const int seq = blockIdx.x, t = seq_q_start[seq];
  const int p = positions[t], slot = seq_slot[seq], hist = taps - 1;
  const T* row = u + (long long)t * u_stride;
  float* ring_slot = ring + (long long)slot * taps * C;
  for (int i = threadIdx.x; i < hp; i += blockDim.x) {
    const int h = h0 + i;
    const float dt = softplus_f(to_float(row[inner + C + h]) + dt_bias[h]);
    dts[i] = dt;
    dts[hp + i] = expf(-expf(a_log[h]) * dt);
  }
  // the block's channels: its heads' x, then B and C of the groups g0 .. g1
  const int nx = hp * P, nb = ng * N;
  for (int i = threadIdx.x; i < nx + 2 * nb; i += blockDim.x) {
    int c;
    bool owner = true;
    if (i < nx) c = h0 * P + i;
    else {
      const int k = i - nx, which = k / nb, e = k - which * nb, g = g0 + e / N;
      c = inner + which * G * N + g * N + e % N;
      owner = g * per_group >= h0 && g * per_group < h0 + hp;
    }
    const float now = to_float(row[inner + c]);
    float y = conv_b[c] + conv_w[(long long)c * taps + hist] * now;
    for (int j = 0; j < hist; ++j) {
      const int x = p - hist + j;
      if (x >= 0) y += conv_w[(long long)c * taps + j] * ring_slot[(long long)(x % taps) * C + c];
    }
    if (write_ring && owner && hist > 0) ring_slot[(long long)(p % taps) * C + c] = now;
    (i < nx ? xs : bs)[i < nx ? i : i - nx] = silu_f(y);      // bs and cs lie back to back
  }
  __syncthreads();
  const int rg = threadIdx.x / W, lc = threadIdx.x % W;
  for (int i = 0; i < hp; ++i) {
    const int h = h0 + i, g = h / per_group - g0;
    const float dt = dts[i], decay = dts[hp + i];
    float* S = state + ((long long)slot * H + h) * N * P;
    for (int c0 = 0; c0 < P; c0 += W) {
      const int col = c0 + lc;
      float acc = 0.0f;
      if (rg < R && col < P) {
        const float xv = dt * xs[i * P + col];
        for (int n = rg; n < N; n += R) {
          const float v = fmaf(decay, S[(long long)n * P + col], bs[g * N + n] * xv);
          S[(long long)n * P + col] = v;
          acc = fmaf(v, cs[g * N + n], acc);
        }
      }
      if (rg < R) part[rg * W + lc] = acc;
      __syncthreads();
      if (threadIdx.x < W && col < P) {
        float sum = 0.0f;
        for (int k = 0; k < R; ++k) sum += part[k * W + lc];
        ys[i * P + col] = sum;
      }
      __syncthreads();
    }
  }
  float sq = 0.0f;
  for (int i = threadIdx.x; i < nx; i += blockDim.x) {
    const int c = h0 * P + i;
    const float y = (ys[i] + d_skip[c / P] * xs[i]) * silu_f(to_float(row[c]));
    ys[i] = y;
    sq += y * y;
  }
  const float s = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nx + eps);
  for (int i = threadIdx.x; i < nx; i += blockDim.x) {
    const int c = h0 * P + i;
    out[(long long)t * out_stride + c] = from_float<T>(ys[i] * s * norm_w[c]);
  }
}

extern "C" long long llm_mamba2_step_shared_bytes(int H, int P, int N, int G, int parts) {
  if (parts < 1 || H % parts || G < 1 || H % G) return -1;
  const int hp = H / parts, per_group = H / G;
  const int ng = (hp + per_group - 1) / per_group + 1;      // at most this many groups under one part's heads
  const int W = P < M2S_THREADS ? P : M2S_THREADS, R = M2S_THREADS / W;
  return (long long)(2 * hp * P + 2 * ng * N + 2 * hp + R * W + 32) * 4;
}

extern "C" int llm_mamba2_step(const void* u, int dtype, long long u_stride, const float* conv_w, const float* conv_b,
                               int taps, float* ring, const float* dt_bias, const float* a_log, const float* d_skip,
                               const float* norm_w, float* state, void* out, long long out_stride,
                               const int32_t* positions, const int32_t* seq_slot, const int32_t* seq_q_start, int n_seqs,
                               int H, int P, int N, int G, int parts, float eps, int write_ring, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  const long long smem = llm_mamba2_step_shared_bytes(H, P, N, G, parts);
  LLM_HOST_CHECK(smem > 0 && smem <= 200 * 1024 && taps >= 1 && n_seqs <= 65535 * 32, ERR_BAD_SIZE);
  const dim3 grid(n_seqs, parts);
#define LAUNCH(T)                                                                                                   \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(mamba2_step_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    launch_kernel(mamba2_step_kernel<T>, grid, M2S_THREADS, (size_t)smem, stream, (const T*)u, u_stride, conv_w, conv_b, \
                  taps, ring, dt_bias, a_log, d_skip, norm_w, state, (T*)out, out_stride, positions, seq_slot,       \
                  seq_q_start, H, P, N, G, parts, eps, write_ring);                                                  \
  } while (0)
  if (dtype == DT_F32) LAUNCH(float);
  else if (dtype == DT_BF16) LAUNCH(__nv_bfloat16);
  else return ERR_BAD_DTYPE;
#undef LAUNCH
  return launch_status();
}
