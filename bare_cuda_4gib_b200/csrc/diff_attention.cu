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
// sizes the tensor-core kernel does not take) and diff_attention_mma (bfloat16 on mma.sync, at the
// end of this file).

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

// ------------------------------------------------------------------ bfloat16 on the tensor cores
//
// Built with -DDA_DQ=<entries of one map> -DDA_DV=<value entries> (multiples of 16).  A thread block
// owns one tile of BM packed rows of one request and one key/value head (packed row R = token
// R / group, head R % group, so a key block loaded once serves every head of the group) and runs
// both maps: warps 0 .. NW/2-1 the first, the others the second, over the same staged keys and
// values.  Keys are visited in blocks of 64 positions aligned to absolute positions, copied from
// the request's pages with cp.async, two blocks in flight (up to four for single tokens).  Two shapes: 4 x 1 warps a map for
// prompts (BM = 64), 1 x 4 for steps of single tokens (BM = 16, each warp 16 of a block's 64
// keys).  All warps leave (maximum, sum, accumulator) in shared memory; one warp per row then
// merges them, subtracts, norms, gates and stores.  A block finds its tile by walking the step's
// sequences, so the grid depends on the step's shape only.
#ifdef DA_DQ

namespace {

constexpr int DQ = DA_DQ, DV = DA_DV;
static_assert(DQ % 16 == 0 && DQ >= 16 && DQ <= 128, "a map's size: a multiple of 16 up to 128");
static_assert(DV % 16 == 0 && DV >= 16 && DV <= 256, "the value size: a multiple of 16 up to 256");
constexpr int BN = 64;
constexpr int LDK = 2 * DQ + 8;  // padded rows (conflict-free ldmatrix)
constexpr int LDV = DV + 8;
// Key and value blocks in flight: two for prompts (the tensor cores are the limit there); steps of single
// tokens wait for memory and little else, so they keep as many as fit beside the queries, up to four.
template <int WARPS_M>
__host__ __device__ constexpr int stages_of() {
  if (WARPS_M > 1) return 2;
  constexpr int fit = (int)((200 * 1024 - 16 * LDK * 2) / (BN * (LDK + LDV) * 2));
  return fit >= 4 ? 4 : (fit >= 2 ? fit : 2);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;  // 0: filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
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
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct DiffArgs {
  const __nv_bfloat16* q;      // [tokens, q_heads, 2 * DQ]
  __nv_bfloat16* out;          // [tokens, q_heads * DV]
  const __nv_bfloat16* gate;   // null, or [tokens, >= q_heads * DV], rows gate_stride apart
  long long gate_stride;
  PagedCache cache;
  const int32_t* seq_q_start;
  const int32_t* seq_q_len;
  const int32_t* seq_kv_len;
  int n_seqs, q_heads;
  float scale_log2;
  int window, chunk;
  float lambda, eps, out_scale;
};

template <int WARPS_M, int WARPS_N>
constexpr size_t diff_smem_bytes() {
  constexpr int BM = 16 * WARPS_M;
  constexpr size_t stages = (size_t)stages_of<WARPS_M>() * BN * (LDK + LDV) * 2;
  constexpr size_t merge = (size_t)2 * WARPS_N * BM * (DV + 2) * 4;
  return (size_t)BM * LDK * 2 + (stages > merge ? stages : merge);
}

template <int WARPS_M, int WARPS_N>
__global__ void __launch_bounds__(2 * WARPS_M* WARPS_N * 32)
diff_attention_mma_kernel(DiffArgs a) {
  constexpr int NW = 2 * WARPS_M * WARPS_N, NT_THREADS = NW * 32;
  constexpr int BM = 16 * WARPS_M;
  constexpr int KEYS_W = BN / WARPS_N, NT = KEYS_W / 8;
  constexpr int STAGES = stages_of<WARPS_M>();
  constexpr int KCH = 2 * DQ / 8, VCH = DV / 8;  // 16-byte chunks per key and value row

  extern __shared__ __align__(16) uint8_t smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [BM][LDK]
  __nv_bfloat16* Ks = Qs + BM * LDK;                               // [STAGES][BN][LDK]
  __nv_bfloat16* Vs = Ks + STAGES * BN * LDK;                      // [STAGES][BN][LDV]
  __shared__ int tile_found[2];

  pdl_launch_dependents();
  pdl_wait();
  const int group = a.q_heads / a.cache.kv_heads;
  const int kvh = blockIdx.y;
  if (threadIdx.x == 0) {
    int left = blockIdx.x, seq = -1;
    for (int s = 0; s < a.n_seqs; ++s) {
      const int tiles = (a.seq_q_len[s] * group + BM - 1) / BM;
      if (left < tiles) {
        seq = s;
        break;
      }
      left -= tiles;
    }
    tile_found[0] = seq;
    tile_found[1] = left;
  }
  __syncthreads();
  const int seq = tile_found[0];
  if (seq < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mp = warp / (WARPS_M * WARPS_N);  // which map
  const int wm = (warp / WARPS_N) % WARPS_M, wn = warp % WARPS_N;
  const int q_start = a.seq_q_start[seq], q_len = a.seq_q_len[seq], kv_len = a.seq_kv_len[seq];
  const int row0 = tile_found[1] * BM;
  const int n_rows = q_len * group;
  const int pos0 = kv_len - q_len;
  const int tile_min_pos = pos0 + row0 / group;
  const int tile_max_pos = pos0 + min(q_len - 1, (row0 + BM - 1) / group);
  const int kb_begin = first_visible(tile_min_pos, a.window, a.chunk) / BN;
  const int kb_end = tile_max_pos / BN + 1;
  const int full_from = first_visible(tile_max_pos, a.window, a.chunk);  // every row sees [full_from, tile_min_pos]

  for (int i = threadIdx.x; i < BM * KCH; i += NT_THREADS) {
    const int r = i / KCH, c = i % KCH;
    const int R = row0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < n_rows) {
      const int token = R / group, head = kvh * group + R % group;
      v = *reinterpret_cast<const uint4*>(a.q + ((long long)(q_start + token) * a.q_heads + head) * (2 * DQ) + c * 8);
    }
    *reinterpret_cast<uint4*>(Qs + r * LDK + c * 8) = v;
  }

  const __nv_bfloat16* kc = reinterpret_cast<const __nv_bfloat16*>(a.cache.k);
  const __nv_bfloat16* vc = reinterpret_cast<const __nv_bfloat16*>(a.cache.v);
  const int page_tokens = a.cache.page_tokens;
  const int32_t* table_row = a.cache.block_table + (long long)seq * a.cache.table_stride;
  auto load_block = [&](int kb, int stage) {
    if (kb < kb_end) {
      __nv_bfloat16* ks = Ks + stage * BN * LDK;
      __nv_bfloat16* vs = Vs + stage * BN * LDV;
      const int key0 = kb * BN;
      // a thread's 16-byte pieces of the block: first the pages of all of them (independent loads), then the copies
      constexpr int PIECES = (BN * (KCH + VCH) + NT_THREADS - 1) / NT_THREADS;
      int page[PIECES];
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        const int key = key0 + (threadIdx.x + j * NT_THREADS) / (KCH + VCH);
        page[j] = key < kv_len ? __ldg(table_row + key / page_tokens) : -1;
      }
#pragma unroll
      for (int j = 0; j < PIECES; ++j) {
        const int i = threadIdx.x + j * NT_THREADS;
        if (i >= BN * (KCH + VCH)) break;
        const int r = i / (KCH + VCH), c = i % (KCH + VCH);
        const int key = key0 + r;
        const bool valid = page[j] >= 0;
        const long long page_base = valid ? (long long)page[j] * a.cache.page_stride : 0;
        const long long in_page = valid ? (long long)kvh * page_tokens + (key % page_tokens) : 0;
        if (c < KCH)
          cp_async16(ks + r * LDK + c * 8, kc + (valid ? page_base + in_page * (2 * DQ) + c * 8 : 0), valid);
        else
          cp_async16(vs + r * LDV + (c - KCH) * 8, vc + (valid ? page_base + in_page * DV + (c - KCH) * 8 : 0), valid);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) load_block(kb_begin + i, i);   // (a group each, empty behind the last block)
  __syncthreads();  // Q staged

  uint32_t qf[DQ / 16][4];
#pragma unroll
  for (int ks = 0; ks < DQ / 16; ++ks)
    ldmatrix_x4(qf[ks], Qs + (wm * 16 + (lane & 15)) * LDK + mp * DQ + ks * 16 + (lane >> 4) * 8);

  int row_pos[2], row_first[2];
  float m[2], l[2];
  float o[DV / 8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = row0 + wm * 16 + (lane >> 2) + h * 8;
    row_pos[h] = R < n_rows ? pos0 + R / group : -1;  // -1: sees nothing
    row_first[h] = R < n_rows ? first_visible(row_pos[h], a.window, a.chunk) : 0;
    m[h] = -INFINITY;
    l[h] = 0.0f;
  }
#pragma unroll
  for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  for (int kb = kb_begin; kb < kb_end; ++kb) {
    const int stage = (kb - kb_begin) % STAGES;
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();  // block kb has landed; everyone is done with block kb - 1, whose stage is filled next
    load_block(kb + STAGES - 1, (kb - kb_begin + STAGES - 1) % STAGES);
    const __nv_bfloat16* ks_ = Ks + stage * BN * LDK;
    const __nv_bfloat16* vs_ = Vs + stage * BN * LDV;
    const int key0 = kb * BN + wn * KEYS_W;

    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < DQ / 16; ++ks) {
#pragma unroll
      for (int nt = 0; nt < NT; nt += 2) {
        uint32_t kf[4];
        const int mid = lane >> 3;
        ldmatrix_x4(kf, ks_ + (wn * KEYS_W + (nt + (mid >> 1)) * 8 + (lane & 7)) * LDK + mp * DQ + ks * 16 + (mid & 1) * 8);
        mma_bf16(s[nt], qf[ks], kf[0], kf[1]);
        mma_bf16(s[nt + 1], qf[ks], kf[2], kf[3]);
      }
    }
    const bool all_visible = kb * BN + BN - 1 <= tile_min_pos && kb * BN >= full_from;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const bool visible = all_visible || (key <= row_pos[h] && key >= row_first[h]);
        const float v = visible ? s[nt][e] * a.scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.0f : m_new;
      corr[h] = fast_exp2(m[h] - m_use[h]);
      m[h] = m_new;
      l[h] *= corr[h];
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int i = 0; i < DV / 8; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
    }
    // a softmax weight enters the second product as a sum of two bfloat16 numbers (the weight rounded,
    // and what the rounding left), so it keeps 16 significant bits instead of 8
    uint32_t pf[NT / 2][4], pf_lo[NT / 2][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float p0 = fast_exp2(s[nt][0] - m_use[0]), p1 = fast_exp2(s[nt][1] - m_use[0]);
      const float p2 = fast_exp2(s[nt][2] - m_use[1]), p3 = fast_exp2(s[nt][3] - m_use[1]);
      l[0] += p0 + p1;
      l[1] += p2 + p3;
      pf[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
      pf_lo[nt / 2][(nt & 1) * 2 + 0] = pack_bf16(p0 - __bfloat162float(__float2bfloat16_rn(p0)),
                                                  p1 - __bfloat162float(__float2bfloat16_rn(p1)));
      pf_lo[nt / 2][(nt & 1) * 2 + 1] = pack_bf16(p2 - __bfloat162float(__float2bfloat16_rn(p2)),
                                                  p3 - __bfloat162float(__float2bfloat16_rn(p3)));
    }
#pragma unroll
    for (int kk = 0; kk < KEYS_W / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < DV / 8; dt += 2) {
        uint32_t vf[4];
        const int mid = lane >> 3;
        ldmatrix_x4_trans(vf, vs_ + (wn * KEYS_W + kk * 16 + (mid & 1) * 8 + (lane & 7)) * LDV + (dt + (mid >> 1)) * 8);
        mma_bf16(o[dt], pf[kk], vf[0], vf[1]);
        mma_bf16(o[dt + 1], pf[kk], vf[2], vf[3]);
        mma_bf16(o[dt], pf_lo[kk], vf[0], vf[1]);
        mma_bf16(o[dt + 1], pf_lo[kk], vf[2], vf[3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }

  // ---- every warp's state to shared memory (over the key and value stages), then one warp a row
  __syncthreads();
  float* red_o = reinterpret_cast<float*>(Ks);          // [2][WARPS_N][BM][DV]
  float* red_m = red_o + 2 * WARPS_N * BM * DV;         // [2][WARPS_N][BM]
  float* red_l = red_m + 2 * WARPS_N * BM;              // [2][WARPS_N][BM]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = wm * 16 + (lane >> 2) + h * 8;
    const int at = (mp * WARPS_N + wn) * BM + r;
    if ((lane & 3) == 0) {
      red_m[at] = m[h];
      red_l[at] = l[h];
    }
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      float* dst = red_o + (long long)at * DV + i * 8 + (lane & 3) * 2;
      dst[0] = o[i][h * 2 + 0];
      dst[1] = o[i][h * 2 + 1];
    }
  }
  __syncthreads();
  constexpr int CPL = (DV + 31) / 32;  // columns per lane
  for (int r = warp; r < BM; r += NW) {
    const int R = row0 + r;
    if (R >= n_rows) continue;
    float w[2][WARPS_N];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      float M = -INFINITY;
#pragma unroll
      for (int x = 0; x < WARPS_N; ++x) M = fmaxf(M, red_m[(p * WARPS_N + x) * BM + r]);
      float L = 0.0f;
#pragma unroll
      for (int x = 0; x < WARPS_N; ++x) {
        const float mw = red_m[(p * WARPS_N + x) * BM + r];
        w[p][x] = mw == -INFINITY ? 0.0f : fast_exp2(mw - M);
        L += red_l[(p * WARPS_N + x) * BM + r] * w[p][x];
      }
      const float inv = L > 0.0f ? 1.0f / L : 0.0f;
#pragma unroll
      for (int x = 0; x < WARPS_N; ++x) w[p][x] *= inv;
    }
    float d[CPL], sq = 0.0f;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = lane + 32 * i;
      float a1 = 0.0f, a2 = 0.0f;
      if (c < DV) {
#pragma unroll
        for (int x = 0; x < WARPS_N; ++x) {
          a1 = fmaf(red_o[(long long)(x * BM + r) * DV + c], w[0][x], a1);
          a2 = fmaf(red_o[(long long)((WARPS_N + x) * BM + r) * DV + c], w[1][x], a2);
        }
      }
      d[i] = a1 - a.lambda * a2;
      sq += d[i] * d[i];
    }
    const float norm = a.out_scale / sqrtf(warp_sum(sq) / (float)DV + a.eps);
    const int token = q_start + R / group, head = kvh * group + R % group;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = lane + 32 * i;
      if (c < DV) {
        float v = d[i] * norm;
        if (a.gate) v /= 1.0f + expf(-to_float(a.gate[(long long)token * a.gate_stride + (long long)head * DV + c]));
        a.out[((long long)token * a.q_heads + head) * DV + c] = __float2bfloat16_rn(v);
      }
    }
  }
}

}  // namespace

// As llm_diff_attention_plain, for bfloat16 with head_dim = 2 * DA_DQ and v_dim = DA_DV.  `single`:
// no sequence brings more than 16 / group tokens (the shape for steps of single tokens).
extern "C" int llm_diff_attention_mma(const void* q, void* out, const void* gate, long long gate_stride, void* k_base,
                                      void* v_base, const int32_t* block_table, long long page_stride, int table_stride,
                                      int page_tokens, int kv_heads, int head_dim, int v_dim,
                                      const int32_t* seq_q_start, const int32_t* seq_q_len, const int32_t* seq_kv_len,
                                      int n_seqs, int q_heads, int n_tokens, int single, float scale, int window,
                                      int chunk, float lambda, float eps, float out_scale, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (head_dim != 2 * DQ || v_dim != DV || q_heads % kv_heads) return ERR_BAD_SIZE;
  if (((uintptr_t)q | (uintptr_t)k_base | (uintptr_t)v_base) % 16 || page_stride % 8) return ERR_BAD_ALIGN;
  const int group = q_heads / kv_heads;
  DiffArgs a{(const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)gate, gate_stride,
             PagedCache{k_base, v_base, block_table, page_stride, table_stride, page_tokens, kv_heads, head_dim},
             seq_q_start, seq_q_len, seq_kv_len, n_seqs, q_heads, scale * 1.4426950408889634f, window, chunk, lambda, eps,
             out_scale};
  static bool raised = false;
  if (!raised) {
    cudaFuncSetAttribute(diff_attention_mma_kernel<4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)diff_smem_bytes<4, 1>());
    cudaFuncSetAttribute(diff_attention_mma_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)diff_smem_bytes<1, 4>());
    raised = true;
  }
  if (single) {
    launch_kernel(diff_attention_mma_kernel<1, 4>, dim3(n_seqs, kv_heads), 256, diff_smem_bytes<1, 4>(), stream, a);
  } else {
    // every sequence may leave one tile partly filled
    const unsigned tiles = (unsigned)(((long long)n_tokens * group + 63) / 64 + n_seqs);
    launch_kernel(diff_attention_mma_kernel<4, 1>, dim3(tiles, kv_heads), 256, diff_smem_bytes<4, 1>(), stream, a);
  }
  return launch_status();
}

#endif  // DA_DQ
