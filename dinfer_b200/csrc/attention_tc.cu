// Paged causal attention on the tensor cores, bfloat16, head sizes 32 / 64 / 128.
//
// One kernel body, two shapes of work:
//   * prompt portions (q_len > 1): a CTA owns 128 "rows" of one (request, kv head).  A row is a
//     (token, query head of the group) pair, so the query heads that share a kv head also share
//     every K/V tile read from the cache.  Eight warps of 16 rows walk the visible keys in tiles
//     of 64 with an online softmax (exp2 domain, 32-bit), K/V staged in shared memory by
//     cp.async with double buffering, fragments by ldmatrix, products by mma.m16n8k16.
//   * decoded tokens (q_len == 1): the rows are just the group's heads (<= 16), so the keys are
//     split instead: grid (split, kv head, request), each CTA takes a range of 64-key tiles and
//     each of its four warps 16 keys of every tile; warps merge in shared memory, splits through
//     a scratch buffer [B, H, splits, D + 2] of f32 partial sums that a second kernel folds.
// Both read keys through the request's block table, mask by position (causal, optional window)
// and never touch a key beyond the visible range (rows of a tile that are out of range are
// zero-filled, so stale or never-written cache contents cannot leak in).
//
// Counterparts in the reference: gqa_fa_v5_kernel (crates/kernels/cuda/gqa.cu:167-369) for prompts,
// gqa_decode_v3 + merge (crates/kernels/cuda/gqa_decode_v3_core.cuh:72-242, gqa.cu:1423-1461) for
// decoding; there the decode kernels compute on the CUDA cores and the group size is limited to 4.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int NT_DECODE = 128; // threads per CTA, decode shape
constexpr int NT_PROMPT = 256; // threads per CTA, prompt shape: eight warps of 16 rows
constexpr int BM = 128;        // rows per CTA (prompt shape)
constexpr int BN = 64;         // keys per tile
constexpr int TABLE_SLOTS = 2048;   // page-table entries of the CTA's key range kept in shared memory
constexpr int STAGES_PROMPT = 2;   // K/V tiles in flight per CTA
constexpr int STAGES_DECODE = 3;   // decode is bound by memory latency: one more tile in flight

struct Params {
  const __nv_bfloat16* q; int64_t ldq;
  __nv_bfloat16* out; int64_t ldo;
  const __nv_bfloat16* cache;
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int H, Hkv, group, block_size, window;
  float scale_log2;            // scale * log2(e)
  int splits;                  // decode shape only
  float* part_o; float* part_ml;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;      // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// 16-byte chunks of a row are XOR-swizzled by the row so that ldmatrix reads 8 rows without bank conflicts
template <int D> __device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int C = D / 8;
  constexpr int R = C >= 8 ? 1 : 8 / C;
  constexpr int M = C >= 8 ? 8 : C;
  return row * D + ((chunk ^ ((row / R) % M)) << 3);
}

// Stage one K and one V tile: keys [j0, j0 + 64) of kv head hk; rows outside [lo, hi) are zero-filled.
template <int D, int NT>
__device__ __forceinline__ void load_kv_tile(const Params& p, const int* table, const int* s_table, int table_first,
                                             int hk, int j0, int lo, int hi,
                                             __nv_bfloat16* sK, __nv_bfloat16* sV) {
  constexpr int C = D / 8;
  constexpr int ROWS = NT / C;
  const int chunk = threadIdx.x % C;
  const int64_t plane = (int64_t)p.Hkv * p.block_size * D;
#pragma unroll
  for (int r0 = 0; r0 < BN; r0 += ROWS) {
    const int row = r0 + threadIdx.x / C;
    const int j = j0 + row;
    bool ok = j >= lo && j < hi;
    int blk = 0;
    if (ok) {      // the CTA's slice of the page table sits in shared memory (no dependent global read per tile)
      const int e = j / p.block_size - table_first;
      blk = e < TABLE_SLOTS ? s_table[e] : table[j / p.block_size];
      ok = blk >= 0;
    }
    const __nv_bfloat16* src = p.cache;
    if (ok) src += (int64_t)blk * 2 * plane + ((int64_t)hk * p.block_size + j % p.block_size) * D + chunk * 8;
    cp_async16(sK + swz<D>(row, chunk), src, ok);
    cp_async16(sV + swz<D>(row, chunk), ok ? src + plane : src, ok);
  }
}

template <int D, bool DECODE>
__global__ void __launch_bounds__(DECODE ? NT_DECODE : NT_PROMPT, 2) attention_tc_kernel(const Params p) {
  constexpr int NT = DECODE ? NT_DECODE : NT_PROMPT;
  constexpr int STAGES = DECODE ? STAGES_DECODE : STAGES_PROMPT;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [BM][D] (16 rows when DECODE)
  __nv_bfloat16* sK = sQ + (DECODE ? 16 : BM) * D;                                  // [STAGES][BN][D]
  __nv_bfloat16* sV = sK + STAGES * BN * D;                                          // [STAGES][BN][D]
  constexpr int C = D / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z, hk = blockIdx.y;
  pdl_enter();
  const int t0 = p.cu_seqlens[b];
  const int q_len = p.cu_seqlens[b + 1] - t0;
  const int seq_len = p.seq_lens[b];
  const int hist = seq_len - q_len;
  if (DECODE ? (q_len != 1) : (q_len <= 1)) return;        // the other shape's kernel owns this request
  const int rows_total = q_len * p.group;
  const int row0 = DECODE ? 0 : blockIdx.x * BM;
  if (row0 >= rows_total) return;
  const int* table = p.block_table + (int64_t)b * p.max_blocks;

  // keys this CTA may need: [lo, hi)
  const int last_row = min(row0 + (DECODE ? 16 : BM), rows_total) - 1;
  const int first_tok = row0 / p.group, last_tok = last_row / p.group;
  int hi = hist + last_tok + 1;
  int lo = p.window > 0 ? max(0, hist + first_tok - p.window + 1) : 0;
  int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  if (DECODE) {
    const int n = tile_end - tile_begin;
    const int per = (n + p.splits - 1) / p.splits;
    tile_begin = tile_begin + blockIdx.x * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  const int n_tiles = max(0, tile_end - tile_begin);
  __shared__ int s_table[TABLE_SLOTS];
  const int table_first = (tile_begin * BN) / p.block_size;
  {
    const int last = (min(tile_end * BN, hi) - 1) / p.block_size;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NT) s_table[i] = table[table_first + i];
    __syncthreads();
  }

  // ---- stage Q (rows = (token, head of the group)) and the first K/V tile
  {
    constexpr int QROWS = DECODE ? 16 : BM;
    for (int i = threadIdx.x; i < QROWS * C; i += NT) {
      const int r = i / C, chunk = i % C;
      const int row = row0 + r;
      const bool ok = row < rows_total;
      const __nv_bfloat16* src = p.q;
      if (ok) src += (int64_t)(t0 + row / p.group) * p.ldq + (int64_t)(hk * p.group + row % p.group) * D + chunk * 8;
      cp_async16(sQ + swz<D>(r, chunk), src, ok);
    }
  }
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {      // Q rides in the first group
    if (i < n_tiles) load_kv_tile<D, NT>(p, table, s_table, table_first, hk, (tile_begin + i) * BN, lo, hi, sK + i * BN * D, sV + i * BN * D);
    cp_async_commit();
  }

  // per-thread softmax state for rows g and g + 8 of the warp's 16 rows
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  unsigned qf[DECODE ? D / 16 : 1][4];   // decode keeps Q's fragments; the prompt shape reloads them (registers)

  const int wrow = DECODE ? 0 : warp * 16;                 // first row of this warp inside the CTA's rows
  int pos_r[2];                                            // position of the query of rows g, g + 8 (-1: no row)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = row0 + wrow + g + 8 * i;
    pos_r[i] = row < rows_total ? hist + row / p.group : -1;
  }
  constexpr int NK = DECODE ? 16 : BN;                     // keys of a tile this warp works on
  const int key_off = DECODE ? warp * 16 : 0;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t % STAGES;
    if (t + STAGES - 1 < n_tiles)
      load_kv_tile<D, NT>(p, table, s_table, table_first, hk, (tile_begin + t + STAGES - 1) * BN, lo, hi,
                          sK + ((t + STAGES - 1) % STAGES) * BN * D, sV + ((t + STAGES - 1) % STAGES) * BN * D);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    if (DECODE && t == 0) {
#pragma unroll
      for (int ks = 0; ks < (DECODE ? D / 16 : 1); ++ks)
        ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], sQ + swz<D>(wrow + (lane & 15), ks * 2 + (lane >> 4)));
    }
    const __nv_bfloat16* kt = sK + buf * BN * D;
    const __nv_bfloat16* vt = sV + buf * BN * D;

    // S = Q K^T for NK keys: NK / 8 accumulator tiles of 16 x 8
    float s[NK / 8][4];
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      unsigned qa[4];
      if (DECODE) {
        qa[0] = qf[DECODE ? ks : 0][0]; qa[1] = qf[DECODE ? ks : 0][1]; qa[2] = qf[DECODE ? ks : 0][2]; qa[3] = qf[DECODE ? ks : 0][3];
      } else {
        ldmatrix_x4(qa[0], qa[1], qa[2], qa[3], sQ + swz<D>(wrow + (lane & 15), ks * 2 + (lane >> 4)));
      }
#pragma unroll
      for (int nb = 0; nb < NK / 16; ++nb) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, kt + swz<D>(key_off + nb * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
        mma_bf16(s[nb * 2], qa, b0, b1);
        mma_bf16(s[nb * 2 + 1], qa, b2, b3);
      }
    }
    // scale into the exp2 domain and mask by position
    const int jbase = (tile_begin + t) * BN + key_off;
    const bool need_mask = (jbase + NK - 1 > hist + first_tok) || (p.window > 0) || (jbase < lo) || DECODE;
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[i][e] * p.scale_log2;
        if (need_mask) {
          const int j = jbase + i * 8 + tq * 2 + (e & 1);
          const int pr = pos_r[e >> 1];
          const bool vis = j <= pr && j >= lo && (p.window <= 0 || j > pr - p.window);
          if (!vis) v = -INFINITY;
        }
        s[i][e] = v;
      }
    }
    // online softmax for rows g (e = 0, 1) and g + 8 (e = 2, 3)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = m_run[r];
#pragma unroll
      for (int i = 0; i < NK / 8; ++i) mx = fmaxf(mx, fmaxf(s[i][2 * r], s[i][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_use = mx == -INFINITY ? 0.f : mx;
      const float alpha = exp2f(m_run[r] - m_use);          // 0 when nothing was seen before
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NK / 8; ++i) {
        s[i][2 * r] = exp2f(s[i][2 * r] - m_use);
        s[i][2 * r + 1] = exp2f(s[i][2 * r + 1] - m_use);
        sum += s[i][2 * r] + s[i][2 * r + 1];
      }
      l_run[r] = l_run[r] * alpha + sum;
      m_run[r] = mx;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { o[i][2 * r] *= alpha; o[i][2 * r + 1] *= alpha; }
    }
    // O += P V
#pragma unroll
    for (int kb = 0; kb < NK / 16; ++kb) {
      unsigned a[4];
      a[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
      a[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
      a[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
      a[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
      for (int db = 0; db < D / 16; ++db) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vt + swz<D>(key_off + kb * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), db * 2 + (lane >> 4)));
        mma_bf16(o[db * 2], a, b0, b1);
        mma_bf16(o[db * 2 + 1], a, b2, b3);
      }
    }
    __syncthreads();          // everyone is done with this buffer before the next load overwrites it
  }
  cp_async_wait<0>();

  // the row sums live in four lanes each
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }

  if (!DECODE) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int row = row0 + wrow + g + 8 * r;
      if (row >= rows_total) continue;
      const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
      __nv_bfloat16* dst = p.out + (int64_t)(t0 + row / p.group) * p.ldo + (int64_t)(hk * p.group + row % p.group) * D;
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<unsigned*>(dst + i * 8 + tq * 2) = pack_bf16(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    }
    return;
  }

  // ---- decode: fold the four warps (each saw different keys), then write the result or the split's partial
  __syncthreads();
  float* sm_o = reinterpret_cast<float*>(smem_raw);         // [4][16][D]
  float* sm_m = sm_o + 4 * 16 * D;                          // [4][16]
  float* sm_l = sm_m + 4 * 16;                              // [4][16]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = g + 8 * r;
    if (tq == 0) { sm_m[warp * 16 + row] = m_run[r]; sm_l[warp * 16 + row] = l_run[r]; }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      sm_o[(warp * 16 + row) * D + i * 8 + tq * 2] = o[i][2 * r];
      sm_o[(warp * 16 + row) * D + i * 8 + tq * 2 + 1] = o[i][2 * r + 1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += NT) {
    const int row = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + row]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * 16 + row];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += sm_l[w * 16 + row] * f;
      acc += sm_o[(w * 16 + row) * D + d] * f;
    }
    const int head = hk * p.group + row;
    if (p.splits == 1) {
      p.out[(int64_t)t0 * p.ldo + (int64_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const int64_t slot = ((int64_t)b * p.H + head) * p.splits + blockIdx.x;
      p.part_o[slot * D + d] = acc;
      if (d == 0) { p.part_ml[slot * 2] = M; p.part_ml[slot * 2 + 1] = L; }
    }
  }
}

// Fold the splits of the decode shape: grid (H, B), one thread per element of the head.
template <int D>
__global__ void __launch_bounds__(D) attention_merge_kernel(const Params p) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  pdl_enter();
  const int t0 = p.cu_seqlens[b];
  if (p.cu_seqlens[b + 1] - t0 != 1) return;
  const int64_t base = ((int64_t)b * p.H + head) * p.splits;
  float M = -INFINITY;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, p.part_ml[(base + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = p.part_ml[(base + s) * 2];
    const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
    L += p.part_ml[(base + s) * 2 + 1] * f;
    acc += p.part_o[(base + s) * D + d] * f;
  }
  p.out[(int64_t)t0 * p.ldo + (int64_t)head * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

template <int D, bool DECODE> size_t smem_bytes() {
  const size_t tiles = (size_t)((DECODE ? 16 : BM) + 2 * (DECODE ? STAGES_DECODE : STAGES_PROMPT) * BN) * D * sizeof(__nv_bfloat16);
  const size_t fold = DECODE ? (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float) : 0;
  return tiles > fold ? tiles : fold;
}

template <int D>
int launch(const Params& p, int B, int max_q_len, bool any_decode, bool any_prefill, cudaStream_t stream) {
  if (any_prefill) {
    auto k = attention_tc_kernel<D, false>;
    const size_t sm = smem_bytes<D, false>();
    static bool opted = false;       // once per process: not a stream operation, kept out of graph captures
    if (!opted) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      if (e != cudaSuccess) return refuse((int)e, "attention_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
      opted = true;
    }
    dim3 grid(((int64_t)max_q_len * p.group + BM - 1) / BM, p.Hkv, B);
    launch_pdl(k, grid, dim3(NT_PROMPT), sm, stream, p);
  }
  if (any_decode) {
    auto k = attention_tc_kernel<D, true>;
    const size_t sm = smem_bytes<D, true>();
    static bool opted = false;       // once per process: not a stream operation, kept out of graph captures
    if (!opted) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
      if (e != cudaSuccess) return refuse((int)e, "attention_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
      opted = true;
    }
    dim3 grid(p.splits, p.Hkv, B);
    launch_pdl(k, grid, dim3(NT_DECODE), sm, stream, p);
    if (p.splits > 1) launch_pdl(attention_merge_kernel<D>, dim3(p.H, B), dim3(D), 0, stream, p);
  }
  return cuda_status("attention_tc");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// Head sizes this library takes; the caller falls back to the plain-arithmetic kernel otherwise.
DINFER_API int dinfer_attention_tc_supports(int D, int group) {
  return (D == 32 || D == 64 || D == 128) && group >= 1 && group <= 16;
}

// Floats of scratch a decode launch with `splits` > 1 needs: part_o then part_ml.
DINFER_API int64_t dinfer_attention_tc_scratch_floats(int B, int H, int D, int splits) {
  return splits > 1 ? (int64_t)B * H * splits * (D + 2) : 0;
}

// q rows of stride ldq (head h at h*D), out rows of stride ldo; cache [blocks, 2, Hkv, block, D] bf16;
// block_table [B, max_blocks]; cu_seqlens [B+1]; seq_lens [B] (length after this step).
// any_decode / any_prefill: whether the batch holds requests with q_len == 1 / q_len > 1.
// scratch: dinfer_attention_tc_scratch_floats() floats, or null when splits == 1.
DINFER_API int dinfer_attention_tc(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                   const int* block_table, int max_blocks, const int* cu_seqlens,
                                   const int* seq_lens, int B, int H, int Hkv, int D, int block_size,
                                   float scale, int window, int max_q_len, int any_decode, int any_prefill,
                                   int splits, float* scratch, cudaStream_t stream) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || block_size <= 0 || max_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_tc: bad sizes B=%d H=%d Hkv=%d block=%d", B, H, Hkv, block_size);
  if (!dinfer_attention_tc_supports(D, H / Hkv))
    return refuse(DINFER_BAD_ARGUMENT, "attention_tc: head_dim %d / group %d not supported (32, 64, 128; group <= 16)", D, H / Hkv);
  if ((ldq % 8) || (ldo % 2) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "attention_tc: q rows and the cache must be 16-byte aligned");
  if (splits < 1 || (splits > 1 && !scratch)) return refuse(DINFER_BAD_ARGUMENT, "attention_tc: splits=%d needs scratch", splits);
  if (Hkv > 65535 || B > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_tc: too many heads or requests for the grid");
  Params p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq; p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.H = H; p.Hkv = Hkv; p.group = H / Hkv;
  p.block_size = block_size; p.window = window; p.scale_log2 = scale * 1.4426950408889634f;
  p.splits = splits; p.part_o = scratch;
  p.part_ml = scratch ? scratch + (int64_t)B * H * splits * D : nullptr;
  if (D == 32) return launch<32>(p, B, max_q_len, any_decode, any_prefill, stream);
  if (D == 64) return launch<64>(p, B, max_q_len, any_decode, any_prefill, stream);
  return launch<128>(p, B, max_q_len, any_decode, any_prefill, stream);
}
