// A mixture-of-experts feed-forward: every token goes through the `top` experts its router picks,
//
//   z = W_router h;   s = softmax(z) over all experts;   the `top` largest s are chosen (the lowest index
//   wins a tie);   weight_k = s_k * router_scale (not renormalised);
//   out = sum_k weight_k * W_down,e_k (act(W_gate,e_k h) * (W_up,e_k h)),   act(z) = z * sigmoid(z),
//
// plus, where the layer has one, a shared expert that every token uses, times sigmoid(w_sg . h).
// Router logits, softmax, weights and the shared gate are float32.
//
// Kernels: moe_route (a block per token: logits, softmax, choice, weights, shared gate), moe_sort (one
// block: tokens' slots grouped by expert, and the list of row tiles the grouped products walk),
// moe_grouped (the experts' products over those tiles in plain arithmetic, any element type: rows gathered
// by the list, one expert's matrix per tile; float32 sums in the order of the inner index, so a row's
// result does not depend on what else is in the step; bfloat16 steps run the tensor-core product of
// gemm_tcgen05.cu over the same list instead, on rows that moe_gather_rows put in the list's order), moe_combine (adds a token's slots in the order of k, and the shared expert).

#include "common.cuh"

#include <math.h>

#define MOE_MAX_EXPERTS 512
#define MOE_ROUTE_WARPS 4

// A lane's part of x . w over `n` entries, the warp's lanes together covering all of them: 16-byte pieces
// where both rows allow them (a lane takes every 32nd piece), single entries otherwise.  The order of the
// sum depends on n and the rows' alignment only.
template <typename T, typename TW>
__device__ __forceinline__ float lane_dot(const T* __restrict__ x, const TW* __restrict__ w, int n, int lane) {
  float dot = 0.0f;
  constexpr int V = 16 / sizeof(T);
  if (sizeof(T) == sizeof(TW) && n % V == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
    const uint4* x4 = reinterpret_cast<const uint4*>(x);
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
#pragma unroll 4
    for (int c = lane; c < n / V; c += 32) {
      const uint4 xa = x4[c], wa = w4[c];
      const T* xe = reinterpret_cast<const T*>(&xa);
      const TW* we = reinterpret_cast<const TW*>(&wa);
#pragma unroll
      for (int j = 0; j < V; ++j) dot = fmaf(to_float(xe[j]), to_float(we[j]), dot);
    }
    return dot;
  }
#pragma unroll 8
  for (int c = lane; c < n; c += 32) dot = fmaf(to_float(x[c]), to_float(w[c]), dot);
  return dot;
}

template <typename T, typename TW>
__global__ void __launch_bounds__(MOE_ROUTE_WARPS * 32)
moe_route_kernel(const T* __restrict__ h, long long h_stride, const TW* __restrict__ w_router,
                 const TW* __restrict__ w_shared_gate, int hidden, int experts, int top, float router_scale,
                 int32_t* __restrict__ ids, float* __restrict__ weights, float* __restrict__ shared_gate, int n_tokens,
                 const float* __restrict__ correction, int groups, int keep) {
  pdl_launch_dependents();
  pdl_wait();
  // a block per token: its warps share the experts' dot products (and the shared gate's, counted as one
  // more), each a warp's sum in a fixed order; the first warp then does the softmax and the choice
  __shared__ float s[MOE_MAX_EXPERTS];
  __shared__ float choice[MOE_MAX_EXPERTS];      // what the choice goes by; a chosen or barred expert holds -inf
  __shared__ float group_best[MOE_MAX_EXPERTS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* x = h + (long long)t * h_stride;
  for (int e = warp; e < experts + (w_shared_gate ? 1 : 0); e += MOE_ROUTE_WARPS) {
    const TW* w = e < experts ? w_router + (long long)e * hidden : w_shared_gate;
    const float dot = warp_sum(lane_dot(x, w, hidden, lane));
    if (lane == 0) {
      if (e < experts) s[e] = dot;
      else shared_gate[t] = 1.0f / (1.0f + expf(-dot));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  float mx = -INFINITY;
  for (int e = lane; e < experts; e += 32) mx = fmaxf(mx, s[e]);
  mx = warp_max(mx);
  float sum = 0.0f;
  for (int e = lane; e < experts; e += 32) {
    const float p = expf(s[e] - mx);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  // the score is the softmax; the choice goes by score + correction (where the router has one)
  for (int e = lane; e < experts; e += 32) {
    const float p = s[e] / sum;
    s[e] = p;
    choice[e] = correction ? p + correction[e] : p;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    // experts form `groups` equal groups of neighbours; a group counts by its best choice value, and only
    // the `keep` best groups stay eligible (the lowest index wins a tie)
    const int size = experts / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * size; e < (g + 1) * size; ++e) best = fmaxf(best, choice[e]);
      group_best[g] = best;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float best = -INFINITY;
      int at = groups;
      for (int g = lane; g < groups; g += 32) {
        const float v = group_best[g];
        if (isnan(v)) continue;      // kept already
        if (at == groups || v > best) best = v, at = g;
      }
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa < groups && (at == groups || ob > best || (ob == best && oa < at))) best = ob, at = oa;
      }
      if (lane == 0 && at < groups) group_best[at] = NAN;      // kept: marked, and out of the running
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (!isnan(group_best[e / size])) choice[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = experts;
    for (int e = lane; e < experts; e += 32)
      if (at == experts ? choice[e] > -INFINITY : choice[e] > best) best = choice[e], at = e;      // ascending e: the lowest index of a lane's ties stays
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (oa < experts && (at == experts || ob > best || (ob == best && oa < at))) best = ob, at = oa;
    }
    if (at >= experts) at = 0;      // fewer eligible experts than choices: cannot happen with a checked configuration
    if (lane == 0) {
      ids[(long long)t * top + k] = at;
      weights[(long long)t * top + k] = s[at] * router_scale;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
}

extern "C" int llm_moe_route(const void* h, int dtype, long long h_stride, const void* w_router, const void* w_shared_gate,
                             int w_dtype, int hidden, int experts, int top, float router_scale, int32_t* ids,
                             float* weights, float* shared_gate, int n_tokens, const float* correction, int groups,
                             int keep, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  LLM_HOST_CHECK(experts >= 1 && experts <= MOE_MAX_EXPERTS && top >= 1 && top <= experts, ERR_BAD_SIZE);
  LLM_HOST_CHECK(groups <= 1 || (experts % groups == 0 && keep >= 1 && keep <= groups && top <= keep * (experts / groups)),
                 ERR_BAD_SIZE);
  const int blocks = n_tokens;
#define ROUTE(T, TW)                                                                                                 \
  launch_kernel(moe_route_kernel<T, TW>, blocks, MOE_ROUTE_WARPS * 32, 0, stream, (const T*)h, h_stride,              \
                (const TW*)w_router, (const TW*)w_shared_gate, hidden, experts, top, router_scale, ids, weights,        \
                shared_gate, n_tokens, correction, groups, keep)
  if (dtype == DT_F32 && w_dtype == DT_F32) ROUTE(float, float);
  else if (dtype == DT_BF16 && w_dtype == DT_BF16) ROUTE(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == DT_BF16 && w_dtype == DT_F32) ROUTE(__nv_bfloat16, float);
  else return ERR_BAD_DTYPE;
#undef ROUTE
  return launch_status();
}

// ------------------------------------------------------------------------------ grouping by expert

// One block.  A slot is (token, k), slot index token * top + k.  `sorted` lists the slots expert by
// expert (inside an expert in ascending slot order); `tiles` lists (expert, first place in `sorted`,
// rows) for every tile of up to `tile_rows` rows, `tiles[0 .. 2]` of entry `n` being unused beyond
// `*n_tiles`.
#define MOE_SORT_THREADS 1024

__global__ void __launch_bounds__(MOE_SORT_THREADS)
moe_sort_kernel(const int32_t* __restrict__ ids, int n_slots, int experts, int tile_rows, int32_t* __restrict__ sorted,
                int32_t* __restrict__ tiles, int32_t* __restrict__ n_tiles) {
  // (`experts` counts the experts that have matrices: a slot whose id lies beyond them is listed nowhere)
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int count[MOE_MAX_EXPERTS], start[MOE_MAX_EXPERTS + 1], tile_start[MOE_MAX_EXPERTS + 1];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_slots; i += blockDim.x)
    if (ids[i] < experts) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, tl = 0;
    for (int e = 0; e < experts; ++e) {
      start[e] = at;
      tile_start[e] = tl;
      at += count[e];
      tl += (count[e] + tile_rows - 1) / tile_rows;
    }
    start[experts] = at;
    tile_start[experts] = tl;
    *n_tiles = tl;
  }
  __syncthreads();
  // places past the last listed slot name slot 0, so that whatever walks the whole list reads valid rows
  for (int i = start[experts] + threadIdx.x; i < n_slots; i += blockDim.x) sorted[i] = 0;
  // a warp per expert walks the slots in order, so the places inside an expert ascend with the slot
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int e = warp; e < experts; e += n_warps) {
    if (count[e] == 0) continue;
    int at = start[e];
    for (int i0 = 0; i0 < n_slots; i0 += 32) {
      const int i = i0 + lane;
      const bool mine = i < n_slots && ids[i] == e;
      const unsigned ballot = __ballot_sync(0xffffffffu, mine);
      if (mine) sorted[at + __popc(ballot & ((1u << lane) - 1u))] = i;
      at += __popc(ballot);
    }
    for (int k = lane; k < tile_start[e + 1] - tile_start[e]; k += 32) {
      int32_t* tile = tiles + 3 * (tile_start[e] + k);
      tile[0] = e;
      tile[1] = start[e] + k * tile_rows;
      tile[2] = min(tile_rows, count[e] - k * tile_rows);
    }
  }
}

extern "C" int llm_moe_sort(const int32_t* ids, int n_slots, int experts, int tile_rows, int32_t* sorted, int32_t* tiles,
                            int32_t* n_tiles, cudaStream_t stream) {
  if (n_slots <= 0) return 0;
  LLM_HOST_CHECK(experts >= 1 && experts <= MOE_MAX_EXPERTS && tile_rows >= 1, ERR_BAD_SIZE);
  launch_kernel(moe_sort_kernel, 1, MOE_SORT_THREADS, 0, stream, ids, n_slots, experts, tile_rows, sorted, tiles, n_tiles);
  return launch_status();
}

// ------------------------------------------------------------------------------ the experts' products

// SIMT form, any element type.  A block takes one tile of rows (one expert) and GM_BN output columns.
//   UP   (DOWN = false): row r of the tile is token sorted[first + r] / top of `a` [tokens, k];
//        GATED: w [experts][2 * n][k] (gate rows, then up rows); out[first + r, c] = act(gate) * up, [slots, n];
//        otherwise w [experts][n][k] and out[first + r, c] = relu(up)^2.
//   DOWN (DOWN = true):  row r is row first + r of `a` [slots, k]; w [experts][n][k];
//        out[sorted[first + r], c] = weight[sorted[first + r]] * sum, float32 [slots, n].
#define GM_BM 32
#define GM_BN 64
#define GM_BK 16

template <typename T, bool DOWN, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ a, long long a_stride, const T* __restrict__ w, void* __restrict__ out_,
                   const int32_t* __restrict__ sorted, const int32_t* __restrict__ tiles,
                   const int32_t* __restrict__ n_tiles, const float* __restrict__ weights, int top, int n, int k) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.x >= *n_tiles) return;
  const int expert = tiles[3 * blockIdx.x], first = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * GM_BN;
  __shared__ float As[GM_BK][GM_BM + 1];
  __shared__ float Wg[GM_BK][GM_BN + 1];
  __shared__ float Wu[GATED ? GM_BK : 1][GM_BN + 1];
  __shared__ int row_src[GM_BM];
  if (threadIdx.x < GM_BM) {
    const int r = threadIdx.x;
    int src = -1;
    if (r < rows) src = DOWN ? first + r : sorted[first + r] / top;
    row_src[r] = src;
  }
  __syncthreads();
  const T* wg = w + (long long)expert * (GATED ? 2 : 1) * n * k;
  const T* wu = wg + (long long)n * k;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // columns tx * 4 .., rows ty * 2 ..
  float acc_g[2][4] = {}, acc_u[2][4] = {};
  for (int k0 = 0; k0 < k; k0 += GM_BK) {
    for (int i = threadIdx.x; i < GM_BM * GM_BK; i += 256) {
      const int r = i / GM_BK, c = i % GM_BK;
      const int src = row_src[r];
      As[c][r] = (src >= 0 && k0 + c < k) ? to_float(a[(long long)src * a_stride + k0 + c]) : 0.0f;
    }
    for (int i = threadIdx.x; i < GM_BN * GM_BK; i += 256) {
      const int r = i / GM_BK, c = i % GM_BK;
      const bool ok = n0 + r < n && k0 + c < k;
      Wg[c][r] = ok ? to_float(wg[(long long)(n0 + r) * k + k0 + c]) : 0.0f;
      if (GATED) Wu[c][r] = ok ? to_float(wu[(long long)(n0 + r) * k + k0 + c]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < GM_BK; ++c) {
      float av[2], gv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 2; ++i) av[i] = As[c][ty * 2 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gv[j] = Wg[c][tx * 4 + j];
        if (GATED) uv[j] = Wu[c][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc_g[i][j] = fmaf(av[i], gv[j], acc_g[i][j]);
          if (GATED) acc_u[i][j] = fmaf(av[i], uv[j], acc_u[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = ty * 2 + i;
    if (r >= rows) continue;
    if (DOWN) {
      const int slot = sorted[first + r];
      const float wt = weights[slot];
      float* out = (float*)out_ + (long long)slot * n;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + tx * 4 + j < n) out[n0 + tx * 4 + j] = wt * acc_g[i][j];
    } else {
      T* out = (T*)out_ + (long long)(first + r) * n;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (n0 + tx * 4 + j < n) {
          const float g = acc_g[i][j];
          const float r = fmaxf(g, 0.0f);
          out[n0 + tx * 4 + j] = from_float<T>(GATED ? g / (1.0f + expf(-g)) * acc_u[i][j] : r * r);
        }
    }
  }
}

extern "C" int llm_moe_grouped(const void* a, long long a_stride, const void* w, void* out, int dtype, int down,
                               const int32_t* sorted, const int32_t* tiles, const int32_t* n_tiles, const float* weights,
                               int top, int n, int k, int max_tiles, int gated, cudaStream_t stream) {
  if (max_tiles <= 0) return 0;
  const dim3 grid(max_tiles, (n + GM_BN - 1) / GM_BN);
#define GROUPED(T, DOWN, GATED)                                                                                     \
  launch_kernel(moe_grouped_kernel<T, DOWN, GATED>, grid, 256, 0, stream, (const T*)a, a_stride, (const T*)w, out,  \
                sorted, tiles, n_tiles, weights, top, n, k)
  if (dtype == DT_F32) {
    if (down) GROUPED(float, true, false); else if (gated) GROUPED(float, false, true); else GROUPED(float, false, false);
  } else if (dtype == DT_BF16) {
    if (down) GROUPED(__nv_bfloat16, true, false);
    else if (gated) GROUPED(__nv_bfloat16, false, true);
    else GROUPED(__nv_bfloat16, false, false);
  } else {
    return ERR_BAD_DTYPE;
  }
#undef GROUPED
  return launch_status();
}

extern "C" int llm_moe_tile_rows() { return GM_BM; }

// ------------------------------------------------------------------------------ rows in the order of the list

// out[i, :] = a[sorted[i] / top, :] for the `n_slots` places of the list: the tokens' rows, expert by expert,
// which is the order the tensor-core grouped product reads them in.  16-byte pieces; `width` elements of
// `esize` bytes make a whole number of them.
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(const uint4* __restrict__ a, long long a_stride16, const int32_t* __restrict__ sorted, int top,
                       uint4* __restrict__ out, int row16, int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)n_slots * row16;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / row16), c = (int)(i % row16);
    out[i] = a[(long long)(sorted[r] / top) * a_stride16 + c];
  }
}

extern "C" int llm_moe_gather_rows(const void* a, long long a_stride_bytes, const int32_t* sorted, int top, void* out,
                                   int row_bytes, int n_slots, cudaStream_t stream) {
  if (n_slots <= 0) return 0;
  LLM_HOST_CHECK(row_bytes > 0 && row_bytes % 16 == 0 && a_stride_bytes % 16 == 0 && top >= 1, ERR_BAD_SIZE);
  LLM_HOST_CHECK(((uintptr_t)a & 15) == 0 && ((uintptr_t)out & 15) == 0, ERR_BAD_ALIGN);
  const long long total = (long long)n_slots * (row_bytes / 16);
  const int blocks = (int)((total + 255) / 256 < 2368 ? (total + 255) / 256 : 2368);
  launch_kernel(moe_gather_rows_kernel, blocks, 256, 0, stream, (const uint4*)a, a_stride_bytes / 16, sorted, top,
                (uint4*)out, row_bytes / 16, n_slots);
  return launch_status();
}

// ------------------------------------------------------------------------------ combine

// out[t, c] = sum_k y[t * top + k, c]  (+ shared_gate[t] * sum_p shared[p][t, c]), float32.
// With `ids`: a slot whose expert lies beyond `experts` is an identity expert, its result weight * h[t].
template <typename TS, typename TH>
__global__ void moe_combine_kernel(const float* __restrict__ y, int top, const TS* __restrict__ shared, int n_partials,
                                   long long partial_stride, const float* __restrict__ shared_gate,
                                   float* __restrict__ out, long long total, int hidden, const int32_t* __restrict__ ids,
                                   const float* __restrict__ weights, int experts, const TH* __restrict__ h,
                                   long long h_stride) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / hidden;
    const int c = (int)(i - t * hidden);
    float sum = 0.0f;
    for (int k = 0; k < top; ++k)
      sum += (ids && ids[t * top + k] >= experts) ? weights[t * top + k] * to_float(h[t * h_stride + c])
                                                  : y[(t * top + k) * hidden + c];
    if (shared) {
      float sh = 0.0f;
      for (int p = 0; p < n_partials; ++p) sh += to_float(shared[p * partial_stride + i]);
      sum += (shared_gate ? shared_gate[t] : 1.0f) * sh;
    }
    out[i] = sum;
  }
}

extern "C" int llm_moe_combine(const float* y, int top, const void* shared, int shared_dtype, int n_partials,
                               long long partial_stride, const float* shared_gate, float* out, int n_tokens, int hidden,
                               const int32_t* ids, const float* weights, int experts, const void* h, int h_dtype,
                               long long h_stride, cudaStream_t stream) {
  const long long total = (long long)n_tokens * hidden;
  if (total <= 0) return 0;
  LLM_HOST_CHECK(!ids || (weights && h), ERR_BAD_SIZE);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
#define COMBINE(TS, TH)                                                                                              \
  launch_kernel(moe_combine_kernel<TS, TH>, blocks, 256, 0, stream, y, top, (const TS*)shared, n_partials,           \
                partial_stride, shared_gate, out, total, hidden, ids, weights, experts, (const TH*)h, h_stride)
  const bool hf = !ids || h_dtype == DT_F32;
  if (ids && h_dtype != DT_F32 && h_dtype != DT_BF16) return ERR_BAD_DTYPE;
  if (!shared || shared_dtype == DT_F32) {
    if (hf) COMBINE(float, float); else COMBINE(float, __nv_bfloat16);
  } else if (shared_dtype == DT_BF16) {
    if (hf) COMBINE(__nv_bfloat16, float); else COMBINE(__nv_bfloat16, __nv_bfloat16);
  } else {
    return ERR_BAD_DTYPE;
  }
#undef COMBINE
  return launch_status();
}
