// The Mamba-2 recurrence of a step's portions in chunks, on the tensor cores (mma.sync m16n8k16, bfloat16
// operands, float32 sums), for bfloat16 steps.  Per head, with a = exp(la) the decay of a token (la = -e^(A_log) dt
// its logarithm), cum_i the sum of la over a chunk's tokens up to i, and S the state at the chunk's start:
//
//   y_i = sum_{j <= i} (C_i . B_j) exp(cum_i - cum_j) dt_j x_j  +  exp(cum_i) S^T C_i
//   S  <- exp(cum_last) S + sum_j B_j (exp(cum_last - cum_j) dt_j x_j)^T
//
// which is S_t = a_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t written out over a chunk of 64 tokens.  A block owns
// one request, one head and 32 (or 16) value columns and walks the request's chunks in order: the state's
// columns are independent, so blocks never wait on one another.  B, C and x arrive as bfloat16 (activations of
// the convolution); step sizes, decays, their exponentials and the state are float32.  Wherever a float32
// factor has to enter a product's operand (the masked weights (C_i . B_j) exp(..) dt_j, x times its decay to
// the chunk's end, the carried state) the operand is a bfloat16 number plus what its rounding left, two
// products, so it keeps 16 significant bits.  The state lives in registers across chunks (float32) and in
// shared memory as such a pair for the product with C.  A chunk's tiles arrive by cp.async while the chunk
// before them is being multiplied (two sets of stages).
//
// Built per model with -DSSD_N (state size) and -DSSD_P (value size of a head), multiples of 16, and
// optionally -DSSD_PC (value columns of a block).

#include "common.cuh"

#include <math.h>

#ifndef SSD_N
#define SSD_N 128
#endif
#ifndef SSD_P
#define SSD_P 64
#endif

namespace {

constexpr int N = SSD_N, P = SSD_P;
static_assert(N % 16 == 0 && N >= 16 && N <= 256, "SSD_N must be a multiple of 16 up to 256");
static_assert(P % 16 == 0 && P >= 16, "SSD_P must be a multiple of 16");
constexpr int L = 64;                         // tokens of a chunk
#ifndef SSD_PC
#define SSD_PC (SSD_P % 32 == 0 ? 32 : 16)
#endif
constexpr int PC = SSD_PC;                    // value columns of a block: 32, or 16 where the model's heads alone
                                              // would leave most SMs without a block
static_assert((PC == 16 || PC == 32) && P % PC == 0, "SSD_PC must be 16 or 32 and divide SSD_P");
constexpr int LDN = N + 8, LDP = PC + 8;      // padded rows (conflict-free ldmatrix)
constexpr int WARPS = 4, THREADS = WARPS * 32;
constexpr int MT_N = N / 16;                  // row tiles of the state
constexpr int MTW = (MT_N + WARPS - 1) / WARPS;   // of which a warp owns at most this many
constexpr int NT = PC / 8;                    // column tiles of a block's columns

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16 (or 4) bytes from global to shared memory without passing through registers; `valid` false fills zeros
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float rounded(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct SsdArgs {
  const __nv_bfloat16* x;      // [rows, heads * P]    after convolution and silu; rows `in_stride` apart, like b and c
  const __nv_bfloat16* b;      // [rows, groups * N]
  const __nv_bfloat16* c;      // [rows, groups * N]
  long long in_stride;
  const float* dt;             // [rows, heads]
  const float* la;             // [rows, heads]   logarithm of the token's decay
  float* state;                // [slots][heads][N][P]
  float* out;                  // [rows, heads * P]   S_t^T C_t
  const int32_t* seq_slot;
  const int32_t* seq_q_start;
  const int32_t* seq_q_len;
  int heads, groups;
};

__global__ void __launch_bounds__(THREADS) mamba2_chunked_kernel(SsdArgs a) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  // two sets of a chunk's tiles: the next chunk's arrive by cp.async while this chunk's products run
  __nv_bfloat16* Bs0 = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [2][L][LDN]
  __nv_bfloat16* Cs0 = Bs0 + 2 * L * LDN;                           // [2][L][LDN]
  __nv_bfloat16* Xs0 = Cs0 + 2 * L * LDN;                           // [2][L][LDP]  x
  __nv_bfloat16* Xh = Xs0 + 2 * L * LDP;                            // [L][LDP]  x times its decay to the chunk's end and dt: rounded ...
  __nv_bfloat16* Xl = Xh + L * LDP;                                 // ... and what the rounding left
  __nv_bfloat16* Sh = Xl + L * LDP;                                 // [N][LDP]  the state at the chunk's start, likewise
  __nv_bfloat16* Sl = Sh + N * LDP;
  float* cum = reinterpret_cast<float*>(Sl + N * LDP);              // [L]
  float* dts0 = cum + L;                                            // [2][L] step sizes
  float* las0 = dts0 + 2 * L;                                       // [2][L] logarithms of the decays

  pdl_launch_dependents();
  pdl_wait();
  const int col0 = blockIdx.x * PC, h = blockIdx.y, seq = blockIdx.z;
  const int q_len = a.seq_q_len[seq];
  if (q_len <= 0) return;
  const int q_start = a.seq_q_start[seq], slot = a.seq_slot[seq];
  const int H = a.heads, g = h / (H / a.groups);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;      // a thread's row within eight and its column pair
  const int mid = lane >> 3;
  const long long x_stride = a.in_stride, bc_stride = a.in_stride, out_stride = (long long)H * P;
  float* S_g = a.state + (((long long)slot * H + h) * N) * P + col0;

  // the state's tiles this warp owns, float32, for the whole walk
  float sreg[MTW][NT][4];
#pragma unroll
  for (int i = 0; i < MTW; ++i) {
    const int mt = warp + i * WARPS;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int n = mt * 16 + gq + (e >> 1) * 8, col = nt * 8 + tq * 2 + (e & 1);
        const float v = mt < MT_N ? S_g[(long long)n * P + col] : 0.0f;
        sreg[i][nt][e] = v;
        if (mt < MT_N) {
          const float hi = rounded(v);
          Sh[n * LDP + col] = __float2bfloat16_rn(v);
          Sl[n * LDP + col] = __float2bfloat16_rn(v - hi);
        }
      }
  }

  const int n_chunks = (q_len + L - 1) / L;
  constexpr int CN = N / 8, CP = PC / 8;
  // requests chunk `ch`'s B, C, x (rows past the portion's end are zero), step sizes and decays, and closes one group
  auto load_chunk = [&](int ch) {
    if (ch < n_chunks) {
      const int st = ch & 1, count = min(L, q_len - ch * L);
      const long long row0 = q_start + (long long)ch * L;
      __nv_bfloat16* Bd = Bs0 + st * L * LDN;
      __nv_bfloat16* Cd = Cs0 + st * L * LDN;
      __nv_bfloat16* Xd = Xs0 + st * L * LDP;
      for (int i = threadIdx.x; i < L * CN; i += THREADS) {
        const int r = i / CN, c8 = i % CN;
        const bool valid = r < count;
        const long long src = valid ? (row0 + r) * bc_stride + g * N + c8 * 8 : 0;
        cp_async16(Bd + r * LDN + c8 * 8, a.b + src, valid);
        cp_async16(Cd + r * LDN + c8 * 8, a.c + src, valid);
      }
      for (int i = threadIdx.x; i < L * CP; i += THREADS) {
        const int r = i / CP, c8 = i % CP;
        const bool valid = r < count;
        cp_async16(Xd + r * LDP + c8 * 8, a.x + (valid ? (row0 + r) * x_stride + h * P + col0 + c8 * 8 : 0), valid);
      }
      if (threadIdx.x < L) {
        const int r = threadIdx.x;
        const bool valid = r < count;
        const long long src = valid ? (row0 + r) * H + h : 0;
        cp_async4(dts0 + st * L + r, a.dt + src, valid);
        cp_async4(las0 + st * L + r, a.la + src, valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  load_chunk(0);
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int t0 = ch * L, count = min(L, q_len - t0);
    const long long row0 = q_start + t0;
    const __nv_bfloat16* Bs = Bs0 + (ch & 1) * L * LDN;
    const __nv_bfloat16* Cs = Cs0 + (ch & 1) * L * LDN;
    const __nv_bfloat16* Xs = Xs0 + (ch & 1) * L * LDP;
    const float* dts = dts0 + (ch & 1) * L;
    const float* las = las0 + (ch & 1) * L;
    load_chunk(ch + 1);      // into the other set, which every warp left at the last chunk's end
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();         // chunk `ch` has landed
    if (warp == 0) {      // the running sum over the chunk's 64 tokens: a lane takes two neighbours
      const float v0 = las[2 * lane], v1 = las[2 * lane + 1];
      float run = v0 + v1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += up;
      }
      cum[2 * lane] = run - v1;
      cum[2 * lane + 1] = run;
    }
    __syncthreads();
    const float cum_last = cum[L - 1];
    // x times exp(cum_last - cum_j) dt_j, as a rounded number and the rest
    for (int i = threadIdx.x; i < L * PC; i += THREADS) {
      const int r = i / PC, c = i % PC;
      const float v = __bfloat162float(Xs[r * LDP + c]) * (expf(cum_last - cum[r]) * dts[r]);
      const float hi = rounded(v);
      Xh[r * LDP + c] = __float2bfloat16_rn(v);
      Xl[r * LDP + c] = __float2bfloat16_rn(v - hi);
    }

    // ---- G = C B^T for this warp's 16 tokens against all 64
    float s[L / 8][4];
#pragma unroll
    for (int nt = 0; nt < L / 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < N / 16; ++ks) {
      uint32_t cf[4];
      ldmatrix_x4(cf, Cs + (warp * 16 + (lane & 15)) * LDN + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < L / 8; nt += 2) {
        uint32_t bf[4];
        ldmatrix_x4(bf, Bs + ((nt + (mid >> 1)) * 8 + (lane & 7)) * LDN + ks * 16 + (mid & 1) * 8);
        mma_bf16(s[nt], cf, bf[0], bf[1]);
        mma_bf16(s[nt + 1], cf, bf[2], bf[3]);
      }
    }
    // ---- the weights (C_i . B_j) exp(cum_i - cum_j) dt_j for j <= i, as A fragments: rounded, and the rest
    uint32_t wh[L / 16][4], wl[L / 16][4];
    const int i0 = warp * 16 + gq, i1 = i0 + 8;
    const float ci0 = cum[i0], ci1 = cum[i1];
#pragma unroll
    for (int nt = 0; nt < L / 8; ++nt) {
      float w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = (e >> 1) ? i1 : i0, j = nt * 8 + tq * 2 + (e & 1);
        w[e] = j <= i ? s[nt][e] * expf(((e >> 1) ? ci1 : ci0) - cum[j]) * dts[j] : 0.0f;
      }
      wh[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(w[0], w[1]);
      wh[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(w[2], w[3]);
      wl[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(w[0] - rounded(w[0]), w[1] - rounded(w[1]));
      wl[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(w[2] - rounded(w[2]), w[3] - rounded(w[3]));
    }
    __syncthreads();      // Xh and Xl are complete (the state's product below reads them)
    // ---- y = weights x  +  exp(cum_i) C S
    float o[NT][4], y2[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
      y2[nt][0] = y2[nt][1] = y2[nt][2] = y2[nt][3] = 0.0f;
    }
#pragma unroll
    for (int kk = 0; kk < L / 16; ++kk) {
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t xf[4];
        ldmatrix_x4_trans(xf, Xs + (kk * 16 + (mid & 1) * 8 + (lane & 7)) * LDP + (nt + (mid >> 1)) * 8);
        mma_bf16(o[nt], wh[kk], xf[0], xf[1]);
        mma_bf16(o[nt + 1], wh[kk], xf[2], xf[3]);
        mma_bf16(o[nt], wl[kk], xf[0], xf[1]);
        mma_bf16(o[nt + 1], wl[kk], xf[2], xf[3]);
      }
    }
#pragma unroll
    for (int ks = 0; ks < N / 16; ++ks) {
      uint32_t cf[4];
      ldmatrix_x4(cf, Cs + (warp * 16 + (lane & 15)) * LDN + ks * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t sf[4];
        ldmatrix_x4_trans(sf, Sh + (ks * 16 + (mid & 1) * 8 + (lane & 7)) * LDP + (nt + (mid >> 1)) * 8);
        mma_bf16(y2[nt], cf, sf[0], sf[1]);
        mma_bf16(y2[nt + 1], cf, sf[2], sf[3]);
        ldmatrix_x4_trans(sf, Sl + (ks * 16 + (mid & 1) * 8 + (lane & 7)) * LDP + (nt + (mid >> 1)) * 8);
        mma_bf16(y2[nt], cf, sf[0], sf[1]);
        mma_bf16(y2[nt + 1], cf, sf[2], sf[3]);
      }
    }
    {
      const float f0 = expf(ci0), f1 = expf(ci1);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int col = h * P + col0 + nt * 8 + tq * 2;
        if (i0 < count)
          *reinterpret_cast<float2*>(a.out + (row0 + i0) * out_stride + col) =
              make_float2(fmaf(f0, y2[nt][0], o[nt][0]), fmaf(f0, y2[nt][1], o[nt][1]));
        if (i1 < count)
          *reinterpret_cast<float2*>(a.out + (row0 + i1) * out_stride + col) =
              make_float2(fmaf(f1, y2[nt][2], o[nt][2]), fmaf(f1, y2[nt][3], o[nt][3]));
      }
    }
    // ---- the state: S <- exp(cum_last) S + B^T (x exp(cum_last - cum_j) dt_j), this warp's row tiles
    const float keep = expf(cum_last);
#pragma unroll
    for (int i = 0; i < MTW; ++i) {
      const int mt = warp + i * WARPS;
      if (mt >= MT_N) break;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sreg[i][nt][e] *= keep;
#pragma unroll
      for (int kk = 0; kk < L / 16; ++kk) {
        uint32_t bt[4];      // B^T as the row operand: the stored [token][n] tile, transposed on the way in
        ldmatrix_x4_trans(bt, Bs + (kk * 16 + (mid >> 1) * 8 + (lane & 7)) * LDN + mt * 16 + (mid & 1) * 8);
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          uint32_t xf[4];
          ldmatrix_x4_trans(xf, Xh + (kk * 16 + (mid & 1) * 8 + (lane & 7)) * LDP + (nt + (mid >> 1)) * 8);
          mma_bf16(sreg[i][nt], bt, xf[0], xf[1]);
          mma_bf16(sreg[i][nt + 1], bt, xf[2], xf[3]);
          ldmatrix_x4_trans(xf, Xl + (kk * 16 + (mid & 1) * 8 + (lane & 7)) * LDP + (nt + (mid >> 1)) * 8);
          mma_bf16(sreg[i][nt], bt, xf[0], xf[1]);
          mma_bf16(sreg[i][nt + 1], bt, xf[2], xf[3]);
        }
      }
    }
    __syncthreads();      // every warp has read the old state and this chunk's tiles
#pragma unroll
    for (int i = 0; i < MTW; ++i) {
      const int mt = warp + i * WARPS;
      if (mt >= MT_N) break;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int n = mt * 16 + gq + (e >> 1) * 8, col = nt * 8 + tq * 2 + (e & 1);
          const float v = sreg[i][nt][e];
          Sh[n * LDP + col] = __float2bfloat16_rn(v);
          Sl[n * LDP + col] = __float2bfloat16_rn(v - rounded(v));
        }
    }
    // (the next chunk's barriers come before anything reads the state again)
  }
#pragma unroll
  for (int i = 0; i < MTW; ++i) {
    const int mt = warp + i * WARPS;
    if (mt >= MT_N) break;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; e += 2) {
        const int n = mt * 16 + gq + (e >> 1) * 8, col = nt * 8 + tq * 2;
        *reinterpret_cast<float2*>(S_g + (long long)n * P + col) = make_float2(sreg[i][nt][e], sreg[i][nt][e + 1]);
      }
  }
}

constexpr size_t SMEM = (size_t)(4 * L * LDN + 4 * L * LDP + 2 * N * LDP) * 2 + 5 * L * 4;

}  // namespace

extern "C" int llm_mamba2_chunked_columns() { return PC; }

extern "C" int llm_mamba2_chunked(const void* x, const void* b, const void* c, long long in_stride, const float* dt,
                                  const float* la, float* state,
                                  float* out, const int32_t* seq_slot, const int32_t* seq_q_start, const int32_t* seq_q_len,
                                  int n_seqs, int heads, int groups, int state_size, int vdim, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  LLM_HOST_CHECK(state_size == N && vdim == P && groups >= 1 && heads % groups == 0, ERR_BAD_SIZE);
  LLM_HOST_CHECK(heads <= 65535 && n_seqs <= 65535 && in_stride % 8 == 0, ERR_BAD_SIZE);
  LLM_HOST_CHECK(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0 &&
                     ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(state)) & 7) == 0,
                 ERR_BAD_ALIGN);
  static bool configured = false;
  if (!configured) {
    if (SMEM > 48 * 1024 &&
        cudaFuncSetAttribute(mamba2_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return launch_status();
    configured = true;
  }
  SsdArgs a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)b, (const __nv_bfloat16*)c, in_stride, dt, la, state, out,
            seq_slot, seq_q_start, seq_q_len, heads, groups};
  launch_kernel(mamba2_chunked_kernel, dim3(P / PC, heads, n_seqs), THREADS, SMEM, stream, a);
  return launch_status();
}
