// Paged attention for decoded tokens (one query token per request), bfloat16, head sizes 64 / 128,
// group sizes up to 16, pages of a power-of-two size.
//
// The step is bound by reading K and V once, so the kernel is built to issue few instructions per
// byte: keys, not heads, fill the 16 rows of the tensor-core tile.
//     S^T[16 keys, 8 heads] = K[16 keys, D] * Q^T[D, 8 heads]          (A = K from shared memory)
//     O^T[D, 8 heads]      += V^T[D, 16 keys] * P^T[16 keys, 8 heads]  (A = V through ldmatrix.trans,
//                                                                       B = P^T by movmatrix.trans)
// so a group of up to 8 query heads costs one n8 tile and nothing is padded to 16 rows.
// Grid (split, kv head, request): a CTA walks a range of 64-key tiles with a 3-deep cp.async
// pipeline (the page-table slice of its keys staged in shared memory first); each of its four warps takes
// 16 keys of every tile with its own running max / sum; warps fold in shared memory; splits fold
// through f32 partials in scratch, by whichever CTA of the (request, kv head) arrives last (a counter
// in the same scratch, left at zero again for the next launch).
//
// Counterpart in the reference: gqa_decode_v3 + merge (crates/kernels/cuda/gqa_decode_v3_core.cuh:72-242,
// crates/kernels/cuda/gqa.cu:1423-1461), CUDA-core dot products with the group limited to 4.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "attention_decode_static.h"

using namespace dinfer;

namespace {

constexpr int NT = 128;
constexpr int BN = 64;
constexpr int STAGES = 3;
constexpr int TABLE_SLOTS = 1024;  // page-table entries of the CTA's key range kept in shared memory

struct Params {
  const __nv_bfloat16* q; int64_t ldq;
  __nv_bfloat16* out; int64_t ldo;
  const __nv_bfloat16* cache;
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int H, Hkv, group, block_size, bs_log2, window;
  float scale_log2;
  int splits;
  float* part_o;     // [B, H, splits, D]
  float* part_ml;    // [B, H, splits, 2]
  int* counters;     // [B, Hkv]
  int* status;       // device status word of the TMA variant (bounded waits)
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
  unsigned d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
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
__device__ __forceinline__ float fast_exp2(float x) {     // ex2.approx: -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int D> __device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int C = D / 8;
  return row * D + ((chunk ^ (row % (C >= 8 ? 8 : C))) << 3);
}

// keys [j0, j0 + 64) of kv head hk into one stage
// The page-table entries of the CTA's keys are staged in shared memory once (s_table, entry 0 = page
// `table_first`), so that a tile's loads do not wait for a dependent global read of the table.
template <int D>
__device__ __forceinline__ void load_tile(const Params& p, const int* table, const int* s_table, int table_first,
                                          int hk, int j0, int lo, int hi,
                                          __nv_bfloat16* sK, __nv_bfloat16* sV) {
  // a warp's copy instruction covers whole rows (C lanes per row, 16 bytes each), so every 32-byte
  // sector is asked for once
  constexpr int C = D / 8, ROWS = NT / C;
  const int chunk = threadIdx.x % C, r_in = threadIdx.x / C;
  const int64_t plane = (int64_t)p.Hkv * p.block_size * D;
  const int64_t head_off = (int64_t)hk * p.block_size * D + chunk * 8;
#pragma unroll
  for (int r0 = 0; r0 < BN; r0 += ROWS) {
    const int row = r0 + r_in;
    const int j = j0 + row;
    bool ok = j >= lo && j < hi;
    int blk = 0;
    if (ok) {
      const int e = (j >> p.bs_log2) - table_first;
      blk = e < TABLE_SLOTS ? s_table[e] : table[j >> p.bs_log2];
      ok = blk >= 0;
    }
    const __nv_bfloat16* src = p.cache;
    if (ok) src += (int64_t)blk * 2 * plane + head_off + (int64_t)(j & (p.block_size - 1)) * D;
    cp_async16(sK + swz<D>(row, chunk), src, ok);
    cp_async16(sV + swz<D>(row, chunk), ok ? src + plane : src, ok);
  }
}

template <int D, int NH8>      // NH8 tiles of 8 heads cover the group
__global__ void __launch_bounds__(NT, 2) attention_decode_kernel(const Params p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [STAGES][BN][D]
  __nv_bfloat16* sV = sK + STAGES * BN * D;                                   // [STAGES][BN][D]
  __shared__ int s_last;
  constexpr int NHEADS = NH8 * 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
  pdl_launch_dependents();
  // Before pdl_wait(): only what no kernel of this step writes (the batch's index arrays, copied to the
  // device before the step's first kernel, and cache pages of older tokens).  The newest token's K/V and
  // the q rows come from the kernel just before this one, so the tile that holds position `pos` and q
  // are read after the wait.
  const int t0 = p.cu_seqlens[b];
  if (p.cu_seqlens[b + 1] - t0 != 1) return;               // not a decoded token: another kernel's request
  const int seq_len = p.seq_lens[b];
  const int pos = seq_len - 1;
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0, hi = seq_len;
  const int* table = p.block_table + (int64_t)b * p.max_blocks;
  int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  {
    const int per = (tile_end - tile_begin + p.splits - 1) / p.splits;
    tile_begin += split * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  const int n_tiles = max(0, tile_end - tile_begin);
  __shared__ int s_table[TABLE_SLOTS];
  const int table_first = (tile_begin * BN) >> p.bs_log2;
  {
    const int last = (min(tile_end * BN, hi) - 1) >> p.bs_log2;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NT) s_table[i] = table[table_first + i];
    __syncthreads();
  }

  bool waited = false;
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) {
    if (i < n_tiles) {
      if (!waited && (tile_begin + i + 1) * BN > pos) { pdl_wait(); waited = true; }
      load_tile<D>(p, table, s_table, table_first, hk, (tile_begin + i) * BN, lo, hi, sK + i * BN * D, sV + i * BN * D);
    }
    cp_async_commit();
  }
  if (!waited) pdl_wait();

  // Q^T as the B operand: head nt*8 + g, dims ks*16 + {2tq, 2tq+1} and + 8
  unsigned qb[D / 16][NH8][2];
#pragma unroll
  for (int nt = 0; nt < NH8; ++nt) {
    const int head = nt * 8 + g;
    const __nv_bfloat16* qrow = p.q + (int64_t)t0 * p.ldq + (int64_t)(hk * p.group + head) * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qb[ks][nt][0] = head < p.group ? *reinterpret_cast<const unsigned*>(qrow + ks * 16 + 2 * tq) : 0u;
      qb[ks][nt][1] = head < p.group ? *reinterpret_cast<const unsigned*>(qrow + ks * 16 + 8 + 2 * tq) : 0u;
    }
  }

  float ot[D / 16][NH8][4];
#pragma unroll
  for (int i = 0; i < D / 16; ++i)
#pragma unroll
    for (int nt = 0; nt < NH8; ++nt) ot[i][nt][0] = ot[i][nt][1] = ot[i][nt][2] = ot[i][nt][3] = 0.f;
  float m_run[NH8][2], l_run[NH8][2];                       // heads nt*8 + 2tq + {0, 1}
#pragma unroll
  for (int nt = 0; nt < NH8; ++nt) { m_run[nt][0] = m_run[nt][1] = -INFINITY; l_run[nt][0] = l_run[nt][1] = 0.f; }
  const int key_off = warp * 16;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t % STAGES;
    cp_async_wait<STAGES - 2>();          // tile t has landed (this thread's part) ...
    __syncthreads();                      // ... everyone's part, and everyone is done with tile t-1:
    if (t + STAGES - 1 < n_tiles)         // its buffer takes tile t + STAGES - 1
      load_tile<D>(p, table, s_table, table_first, hk, (tile_begin + t + STAGES - 1) * BN, lo, hi,
                   sK + ((t + STAGES - 1) % STAGES) * BN * D, sV + ((t + STAGES - 1) % STAGES) * BN * D);
    cp_async_commit();
    const __nv_bfloat16* kt = sK + buf * BN * D;
    const __nv_bfloat16* vt = sV + buf * BN * D;
    const int jbase = (tile_begin + t) * BN + key_off;
    if (jbase < hi) {                                       // warp-uniform: this warp's 16 keys hold something
      float st[NH8][4], st2[NH8][4];                        // two accumulators: half the dependent chain
#pragma unroll
      for (int nt = 0; nt < NH8; ++nt) {
        st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.f;
        st2[nt][0] = st2[nt][1] = st2[nt][2] = st2[nt][3] = 0.f;
      }
#pragma unroll
      for (int ks = 0; ks < D / 16; ks += 2) {
        unsigned a[4], a2[4];
        ldmatrix_x4(a, kt + swz<D>(key_off + (lane & 15), ks * 2 + (lane >> 4)));
        ldmatrix_x4(a2, kt + swz<D>(key_off + (lane & 15), (ks + 1) * 2 + (lane >> 4)));
#pragma unroll
        for (int nt = 0; nt < NH8; ++nt) {
          mma_bf16(st[nt], a, qb[ks][nt][0], qb[ks][nt][1]);
          mma_bf16(st2[nt], a2, qb[ks + 1][nt][0], qb[ks + 1][nt][1]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < NH8; ++nt) {
        st[nt][0] += st2[nt][0]; st[nt][1] += st2[nt][1]; st[nt][2] += st2[nt][2]; st[nt][3] += st2[nt][3];
      }
      const bool vis0 = jbase + g >= lo && jbase + g <= pos;
      const bool vis1 = jbase + g + 8 >= lo && jbase + g + 8 <= pos;
      bool rescale = false;
      float alpha[NH8][2];
      unsigned pb[NH8][2];
#pragma unroll
      for (int nt = 0; nt < NH8; ++nt) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float s0 = vis0 ? st[nt][c] * p.scale_log2 : -INFINITY;
          const float s1 = vis1 ? st[nt][c + 2] * p.scale_log2 : -INFINITY;
          float mx = fmaxf(s0, s1);
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
          const float m_new = fmaxf(m_run[nt][c], mx);
          const float m_use = m_new == -INFINITY ? 0.f : m_new;
          alpha[nt][c] = fast_exp2(m_run[nt][c] - m_use);
          rescale |= m_new != m_run[nt][c];
          const float p0 = fast_exp2(s0 - m_use), p1 = fast_exp2(s1 - m_use);
          l_run[nt][c] = l_run[nt][c] * alpha[nt][c] + p0 + p1;
          m_run[nt][c] = m_new;
          st[nt][c] = p0;
          st[nt][c + 2] = p1;
        }
        pb[nt][0] = movmatrix_trans(pack_bf16(st[nt][0], st[nt][1]));
        pb[nt][1] = movmatrix_trans(pack_bf16(st[nt][2], st[nt][3]));
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int i = 0; i < D / 16; ++i)
#pragma unroll
          for (int nt = 0; nt < NH8; ++nt) {
            ot[i][nt][0] *= alpha[nt][0]; ot[i][nt][1] *= alpha[nt][1];
            ot[i][nt][2] *= alpha[nt][0]; ot[i][nt][3] *= alpha[nt][1];
          }
      }
#pragma unroll
      for (int db = 0; db < D / 16; ++db) {
        unsigned a[4];
        ldmatrix_x4_trans(a, vt + swz<D>(key_off + (lane & 7) + ((lane >> 4) << 3), db * 2 + ((lane >> 3) & 1)));
#pragma unroll
        for (int nt = 0; nt < NH8; ++nt) mma_bf16(ot[db][nt], a, pb[nt][0], pb[nt][1]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- fold the four warps
  float* sm_o = reinterpret_cast<float*>(smem_raw);          // [4][NHEADS][D]
  float* sm_m = sm_o + 4 * NHEADS * D;                       // [4][NHEADS]
  float* sm_l = sm_m + 4 * NHEADS;
#pragma unroll
  for (int nt = 0; nt < NH8; ++nt) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float l = l_run[nt][c];
      l += __shfl_xor_sync(0xffffffffu, l, 4);
      l += __shfl_xor_sync(0xffffffffu, l, 8);
      l += __shfl_xor_sync(0xffffffffu, l, 16);
      const int head = nt * 8 + 2 * tq + c;
      if (g == 0) { sm_m[warp * NHEADS + head] = m_run[nt][c]; sm_l[warp * NHEADS + head] = l; }
#pragma unroll
      for (int i = 0; i < D / 16; ++i) {
        sm_o[(warp * NHEADS + head) * D + i * 16 + g] = ot[i][nt][c];
        sm_o[(warp * NHEADS + head) * D + i * 16 + g + 8] = ot[i][nt][c + 2];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += NT) {
    const int head = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * NHEADS + head]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * NHEADS + head];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      L += sm_l[w * NHEADS + head] * f;
      acc += sm_o[(w * NHEADS + head) * D + d] * f;
    }
    const int gh = hk * p.group + head;
    if (p.splits == 1) {
      p.out[(int64_t)t0 * p.ldo + (int64_t)gh * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    } else {
      const int64_t slot = ((int64_t)b * p.H + gh) * p.splits + split;
      p.part_o[slot * D + d] = acc;
      if (d == 0) { p.part_ml[slot * 2] = M; p.part_ml[slot * 2 + 1] = L; }
    }
  }
  if (p.splits == 1) return;

  // ---- fold the splits: the CTA that arrives last does it
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(&p.counters[b * p.Hkv + hk], 1) == p.splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // weights of the splits first (one (head, split) pair per thread, all loads independent), then the sums
  float* sm_f = reinterpret_cast<float*>(smem_raw);           // [group][splits] factor, then [group] 1 / L
  float* sm_inv = sm_f + NHEADS * 32;
  float* sm_l2 = sm_inv + NHEADS;
  for (int i = threadIdx.x; i < p.group * p.splits; i += NT) {
    const int head = i / p.splits, sp = i % p.splits;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + ((int64_t)b * p.H + hk * p.group + head) * p.splits + sp);
    sm_f[head * 32 + sp] = ml.x;                              // the split's maximum
    sm_l2[head * 32 + sp] = ml.y;                             // and its sum
  }
  __syncthreads();
  if (threadIdx.x < p.group) {
    const int head = threadIdx.x;
    float M = -INFINITY;
    for (int sp = 0; sp < p.splits; ++sp) M = fmaxf(M, sm_f[head * 32 + sp]);
    float L = 0.f;
    for (int sp = 0; sp < p.splits; ++sp) {
      const float ms = sm_f[head * 32 + sp];
      const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
      L += sm_l2[head * 32 + sp] * f;
      sm_f[head * 32 + sp] = f;
    }
    sm_inv[head] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < p.group * D; idx += NT) {
    const int head = idx / D, d = idx % D;
    const int gh = hk * p.group + head;
    const float* po = p.part_o + ((int64_t)b * p.H + gh) * p.splits * D + d;
    float acc = 0.f;
#pragma unroll 8
    for (int sp = 0; sp < p.splits; ++sp) acc += __ldcg(po + sp * D) * sm_f[head * 32 + sp];
    p.out[(int64_t)t0 * p.ldo + (int64_t)gh * D + d] = __float2bfloat16_rn(acc * sm_inv[head]);
  }
  if (threadIdx.x == 0) p.counters[b * p.Hkv + hk] = 0;      // ready for the next launch
}

// ------------------------------------------------------------------------------------------------
// The same computation with the tiles brought in by TMA: a fifth warp's elected lane requests every
// page of a tile (one box per page, 64-wide half and K / V) through a tensor map over the layer's
// cache, tiles ride an mbarrier ring (full: bytes landed; empty: the four compute warps are done), and
// the compute warps issue no address arithmetic or copies at all and meet at no CTA-wide barrier per
// tile.  Shared-memory tiles have TMA's 128-byte swizzle: [half][key][128 bytes].  Pages of at least
// 8 tokens (a swizzle atom is 8 rows).  Every mbarrier wait is bounded (status word).
// With key splits the CTAs of a (request, kv head) are one thread-block cluster: each owns a share of
// the (head, dim) outputs, the others store their unnormalised sums of that share (and their maxima
// and sums) into its shared memory, and after one cluster barrier every CTA folds and writes its share.
constexpr int NT_TMA = 160;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  uint64_t start = 0;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 255) == 255) {
      uint64_t now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (start == 0) start = now;
      else if (now - start > 2000000000ull) return false;
    }
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// ---- thread-block cluster: the CTAs of one (request, kv head) that split its keys
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
constexpr int MAX_CLUSTER_SPLITS = 16;
// floats of the receive buffer of a CTA: its share of the (head, dim) sums from every split, then
// every split's (maximum, sum) of every head
__host__ __device__ constexpr int fold_share(int group, int D, int splits) { return (group * D + splits - 1) / splits; }
__host__ __device__ constexpr int fold_recv_floats(int group, int D, int splits) {
  return splits * fold_share(group, D, splits) + splits * group * 2;
}
// byte offset of (key row, 16-byte chunk c of the head) inside a [half][64 keys][128 B] tile with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int c) {
  return (uint32_t)((c >> 3) * (BN * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

template <int D, int NH8>
__global__ void __launch_bounds__(NT_TMA, 2)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const Params p) {
  constexpr int NHF = D / 64;                                 // 64-wide halves of the head
  constexpr uint32_t KV_BYTES = NHF * BN * 128;               // one of K / V of a tile
  constexpr int NHEADS = NH8 * 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];   // aligned to 1024 by hand below
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ int s_table[TABLE_SLOTS];
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int b = blockIdx.z, hk = blockIdx.y, split = blockIdx.x;
  pdl_launch_dependents();
  // before pdl_wait(): only the batch's index arrays and cache pages of older tokens (see the other kernel)
  const int t0 = p.cu_seqlens[b];
  if (p.cu_seqlens[b + 1] - t0 != 1) return;                  // the whole cluster leaves: same request
  // first phase of the cluster barrier: this CTA runs, its shared memory may be written by the others
  if (p.splits > 1) cluster_arrive_relaxed();
  const int seq_len = p.seq_lens[b];
  const int pos = seq_len - 1;
  const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0, hi = seq_len;
  const int* table = p.block_table + (int64_t)b * p.max_blocks;
  int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  {
    const int per = (tile_end - tile_begin + p.splits - 1) / p.splits;
    tile_begin += split * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  const int n_tiles = max(0, tile_end - tile_begin);
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - smem_u32(smem_raw));
  const int table_first = (tile_begin * BN) >> p.bs_log2;
  {
    const int last = (min(tile_end * BN, hi) - 1) >> p.bs_log2;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NT_TMA) s_table[i] = table[table_first + i];
    // a page that is skipped leaves its rows as they were: they must hold finite numbers (0 * V)
    uint4* z = reinterpret_cast<uint4*>(gbase);
    for (int i = threadIdx.x; i < (int)(2 * STAGES * KV_BYTES / 16); i += NT_TMA) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 4); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();

  float ot[D / 16][NH8][4];
  float m_run[NH8][2], l_run[NH8][2];
#pragma unroll
  for (int i = 0; i < D / 16; ++i)
#pragma unroll
    for (int nt = 0; nt < NH8; ++nt) ot[i][nt][0] = ot[i][nt][1] = ot[i][nt][2] = ot[i][nt][3] = 0.f;
#pragma unroll
  for (int nt = 0; nt < NH8; ++nt) { m_run[nt][0] = m_run[nt][1] = -INFINITY; l_run[nt][0] = l_run[nt][1] = 0.f; }

  if (warp == 4) {
    // ---- TMA producer: the whole warp.  A tile is (64 / page rows) pages x (K, V) x 64-wide halves of
    // copies; each lane owns up to two of them, so they are requested side by side instead of one after
    // another from a single thread (that serial issue, not the memory, bounded the kernel).
    const int br = min(p.block_size, BN), boxes = BN / br;
    constexpr int PER_BOX = 2 * NHF;                          // K/V x halves
    const int n_ops = boxes * PER_BOX;                        // <= 64
    bool waited = false, alive = true;
    for (int t = 0; t < n_tiles && alive; ++t) {
      const int s = t % STAGES;
      const int j0 = (tile_begin + t) * BN;
      if (!waited && j0 + BN > pos) { pdl_wait(); waited = true; }        // the newest token's page
      bool ok = true;
      if (lane == 0) ok = mbar_wait(smem_u32(&empty_bar[s]), ((t / STAGES) & 1) ^ 1);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) { if (lane == 0) { s_abort = 1; atomicExch(p.status, 21); } alive = false; break; }
      const uint32_t bar = smem_u32(&full_bar[s]);
      const uint32_t sk = base + s * 2 * KV_BYTES;
      int row[2]; uint32_t dst[2]; int col[2]; bool valid[2];
      uint32_t bytes = 0;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int o = lane + 32 * u;
        valid[u] = false;
        if (o < n_ops) {
          const int x = o / PER_BOX, r = o % PER_BOX, kv = r / NHF, h = r % NHF;
          const int key = j0 + x * br;
          if (key < hi && key + br > lo) {
            const int e = (key >> p.bs_log2) - table_first;
            const int blk = e < TABLE_SLOTS ? s_table[e] : table[key >> p.bs_log2];
            if (blk >= 0) {
              valid[u] = true;
              row[u] = ((blk * 2 + kv) * p.Hkv + hk) * p.block_size + (key & (p.block_size - 1));
              col[u] = h * 64;
              dst[u] = sk + kv * KV_BYTES + h * (BN * 128) + x * br * 128;
              bytes += br * 128;
            }
          }
        }
      }
      bytes = __reduce_add_sync(0xffffffffu, bytes);
      if (lane == 0) {
        if (bytes == 0) mbar_arrive(bar); else mbar_expect_tx(bar, bytes);
      }
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if (valid[u]) tma_load_2d(dst[u], &map_kv, col[u], row[u], bar);
    }
    if (!waited) pdl_wait();
  } else {                                                    // ---- four compute warps, 16 keys of every tile each
    pdl_wait();                                               // q comes from the kernel before this one
    unsigned qb[D / 16][NH8][2];
#pragma unroll
    for (int nt = 0; nt < NH8; ++nt) {
      const int head = nt * 8 + g;
      const __nv_bfloat16* qrow = p.q + (int64_t)t0 * p.ldq + (int64_t)(hk * p.group + head) * D;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        qb[ks][nt][0] = head < p.group ? *reinterpret_cast<const unsigned*>(qrow + ks * 16 + 2 * tq) : 0u;
        qb[ks][nt][1] = head < p.group ? *reinterpret_cast<const unsigned*>(qrow + ks * 16 + 8 + 2 * tq) : 0u;
      }
    }
    const int key_off = warp * 16;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t % STAGES;
      if (!mbar_wait(smem_u32(&full_bar[s]), (t / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 22); ok = false; break; }
      const unsigned char* kt = gbase + s * 2 * KV_BYTES;
      const unsigned char* vt = kt + KV_BYTES;
      const int jbase = (tile_begin + t) * BN + key_off;
      if (jbase < hi) {
        float st[NH8][4], st2[NH8][4];
#pragma unroll
        for (int nt = 0; nt < NH8; ++nt) {
          st[nt][0] = st[nt][1] = st[nt][2] = st[nt][3] = 0.f;
          st2[nt][0] = st2[nt][1] = st2[nt][2] = st2[nt][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ks += 2) {
          unsigned a[4], a2[4];
          ldmatrix_x4(a, kt + sw128(key_off + (lane & 15), ks * 2 + (lane >> 4)));
          ldmatrix_x4(a2, kt + sw128(key_off + (lane & 15), (ks + 1) * 2 + (lane >> 4)));
#pragma unroll
          for (int nt = 0; nt < NH8; ++nt) {
            mma_bf16(st[nt], a, qb[ks][nt][0], qb[ks][nt][1]);
            mma_bf16(st2[nt], a2, qb[ks + 1][nt][0], qb[ks + 1][nt][1]);
          }
        }
#pragma unroll
        for (int nt = 0; nt < NH8; ++nt) {
          st[nt][0] += st2[nt][0]; st[nt][1] += st2[nt][1]; st[nt][2] += st2[nt][2]; st[nt][3] += st2[nt][3];
        }
        const bool vis0 = jbase + g >= lo && jbase + g <= pos;
        const bool vis1 = jbase + g + 8 >= lo && jbase + g + 8 <= pos;
        bool rescale = false;
        float alpha[NH8][2];
        unsigned pb[NH8][2];
#pragma unroll
        for (int nt = 0; nt < NH8; ++nt) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const float s0 = vis0 ? st[nt][c] * p.scale_log2 : -INFINITY;
            const float s1 = vis1 ? st[nt][c + 2] * p.scale_log2 : -INFINITY;
            float mx = fmaxf(s0, s1);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float m_new = fmaxf(m_run[nt][c], mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            alpha[nt][c] = fast_exp2(m_run[nt][c] - m_use);
            rescale |= m_new != m_run[nt][c];
            const float p0 = fast_exp2(s0 - m_use), p1 = fast_exp2(s1 - m_use);
            l_run[nt][c] = l_run[nt][c] * alpha[nt][c] + p0 + p1;
            m_run[nt][c] = m_new;
            st[nt][c] = p0;
            st[nt][c + 2] = p1;
          }
          pb[nt][0] = movmatrix_trans(pack_bf16(st[nt][0], st[nt][1]));
          pb[nt][1] = movmatrix_trans(pack_bf16(st[nt][2], st[nt][3]));
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
          for (int i = 0; i < D / 16; ++i)
#pragma unroll
            for (int nt = 0; nt < NH8; ++nt) {
              ot[i][nt][0] *= alpha[nt][0]; ot[i][nt][1] *= alpha[nt][1];
              ot[i][nt][2] *= alpha[nt][0]; ot[i][nt][3] *= alpha[nt][1];
            }
        }
#pragma unroll
        for (int db = 0; db < D / 16; ++db) {
          unsigned a[4];
          ldmatrix_x4_trans(a, vt + sw128(key_off + (lane & 7) + ((lane >> 4) << 3), db * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int nt = 0; nt < NH8; ++nt) mma_bf16(ot[db][nt], a, pb[nt][0], pb[nt][1]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&empty_bar[s]));     // this warp is done with the stage
    }
  }
  __syncthreads();

  // ---- fold the four warps (the tiles' shared memory is free now)
  float* sm_o = reinterpret_cast<float*>(gbase);             // [4][NHEADS][D]
  float* sm_m = sm_o + 4 * NHEADS * D;                       // [4][NHEADS]
  float* sm_l = sm_m + 4 * NHEADS;
  if (warp < 4) {
#pragma unroll
    for (int nt = 0; nt < NH8; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float l = l_run[nt][c];
        l += __shfl_xor_sync(0xffffffffu, l, 4);
        l += __shfl_xor_sync(0xffffffffu, l, 8);
        l += __shfl_xor_sync(0xffffffffu, l, 16);
        const int head = nt * 8 + 2 * tq + c;
        if (g == 0) { sm_m[warp * NHEADS + head] = m_run[nt][c]; sm_l[warp * NHEADS + head] = l; }
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
          sm_o[(warp * NHEADS + head) * D + i * 16 + g] = ot[i][nt][c];
          sm_o[(warp * NHEADS + head) * D + i * 16 + g + 8] = ot[i][nt][c + 2];
        }
      }
    }
  }
  __syncthreads();
  const bool clustered = p.splits > 1;
  const int share = fold_share(p.group, D, p.splits);        // (head, dim) outputs per CTA of the cluster
  const uint32_t recv_base = base + 2 * STAGES * KV_BYTES;   // beyond the tiles: others write it while tiles still land
  if (clustered) cluster_wait_acquire();                     // every CTA of the cluster runs
  if (!s_abort) {
    for (int idx = threadIdx.x; idx < p.group * D; idx += NT_TMA) {
      const int head = idx / D, d = idx % D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * NHEADS + head]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sm_m[w * NHEADS + head];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += sm_l[w * NHEADS + head] * f;
        acc += sm_o[(w * NHEADS + head) * D + d] * f;
      }
      if (!clustered) {
        p.out[(int64_t)t0 * p.ldo + (int64_t)(hk * p.group + head) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
      } else {
        const int owner = idx / share;
        st_cluster_f32(map_to_cta(recv_base, owner) + (uint32_t)((split * share + idx - owner * share) * 4), acc);
        if (d == 0) {                                         // this head's maximum and sum, to every CTA
          const uint32_t off = recv_base + (uint32_t)((p.splits * share + (split * p.group + head) * 2) * 4);
          for (int o = 0; o < p.splits; ++o) {
            const uint32_t dst = map_to_cta(off, o);
            st_cluster_f32(dst, M);
            st_cluster_f32(dst + 4, L);
          }
        }
      }
    }
  }
  if (!clustered) return;

  // ---- second phase: all partial sums of this CTA's share have arrived
  cluster_arrive_release();
  cluster_wait_acquire();
  if (s_abort) return;
  {
    const float* recv = reinterpret_cast<const float*>(gbase + 2 * STAGES * KV_BYTES);
    const float* recv_ml = recv + p.splits * share;
    const int rank = (int)cluster_ctarank();                  // = split: the cluster spans the grid's x
    const int mine = min(share, p.group * D - rank * share);
    for (int i = threadIdx.x; i < mine; i += NT_TMA) {
      const int idx = rank * share + i;
      const int head = idx / D, d = idx % D;
      float M = -INFINITY;
      for (int sp = 0; sp < p.splits; ++sp) M = fmaxf(M, recv_ml[(sp * p.group + head) * 2]);
      float L = 0.f, acc = 0.f;
      for (int sp = 0; sp < p.splits; ++sp) {
        const float ms = recv_ml[(sp * p.group + head) * 2];
        const float f = ms == -INFINITY ? 0.f : exp2f(ms - M);
        L += recv_ml[(sp * p.group + head) * 2 + 1] * f;
        acc += recv[sp * share + i] * f;
      }
      p.out[(int64_t)t0 * p.ldo + (int64_t)(hk * p.group + head) * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  }
  return fn;
}

template <int D, int NH8>
int launch_tma(const CUtensorMap& map, const Params& p, int B, cudaStream_t stream) {
  auto k = attention_decode_tma_kernel<D, NH8>;
  // tiles (the four warps' fold reuses them: it is smaller), then the cluster's receive buffer
  static_assert((size_t)(4 * NH8 * 8 * D + 2 * 4 * NH8 * 8) * sizeof(float) <= (size_t)2 * STAGES * (D / 64) * BN * 128,
                "the fold of the four warps fits the tiles");
  const size_t tiles = (size_t)2 * STAGES * (D / 64) * BN * 128 + 1024;
  const size_t sm = tiles + (p.splits > 1 ? (size_t)fold_recv_floats(p.group, D, p.splits) * sizeof(float) : 0);
  static bool opted = false;
  if (!opted) {
    const size_t most = tiles + (size_t)fold_recv_floats(NH8 * 8, D, MAX_CLUSTER_SPLITS) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) return refuse((int)e, "attention_decode: shared memory opt-in failed: %s", cudaGetErrorString(e));
    e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);     // clusters of up to 16
    if (e != cudaSuccess) return refuse((int)e, "attention_decode: cluster size opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  if (p.splits > 8) {
    // beyond the portable cluster size: ask once per size whether such a cluster fits this GPU
    static int fits[MAX_CLUSTER_SPLITS + 1] = {0};            // 0 = not asked, 1 = yes, -1 = no
    if (!fits[p.splits]) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(p.splits, p.Hkv, B); cfg.blockDim = dim3(NT_TMA); cfg.dynamicSmemBytes = sm;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = p.splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int n = 0;
      const cudaError_t q = cudaOccupancyMaxActiveClusters(&n, k, &cfg);
      if (q != cudaSuccess) (void)cudaGetLastError();
      fits[p.splits] = (q == cudaSuccess && n > 0) ? 1 : -1;
    }
    if (fits[p.splits] < 0)
      return refuse(DINFER_BAD_ARGUMENT, "attention_decode: a cluster of %d CTAs does not fit this GPU; use at most 8 key splits", p.splits);
  }
  cudaError_t e = launch_pdl_cluster(k, dim3(p.splits, p.Hkv, B), dim3(NT_TMA), dim3(p.splits, 1, 1), sm, stream, map, p);
  if (e != cudaSuccess) return refuse((int)e, "attention_decode: launch failed: %s", cudaGetErrorString(e));
  return cuda_status("attention_decode");
}

template <int D, int NH8>
int launch(const Params& p, int B, cudaStream_t stream) {
  auto k = attention_decode_kernel<D, NH8>;
  size_t sm = (size_t)2 * STAGES * BN * D * sizeof(__nv_bfloat16);
  const size_t fold = (size_t)(4 * NH8 * 8 * D + 2 * 4 * NH8 * 8) * sizeof(float);
  if (fold > sm) sm = fold;
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return refuse((int)e, "attention_decode: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  launch_pdl(k, dim3(p.splits, p.Hkv, B), dim3(NT), sm, stream, p);
  return cuda_status("attention_decode");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

DINFER_API int dinfer_attention_decode_supports(int D, int group, int block_size) {
  return (D == 64 || D == 128) && group >= 1 && group <= 16 && block_size > 0 && (block_size & (block_size - 1)) == 0;
}

// Scratch for `splits` > 1: floats [B*H*splits*(D+2)] then ints [B*Hkv] that must be zero before the
// first launch (every launch leaves them zero).  Launches that share the scratch must not overlap.
DINFER_API int64_t dinfer_attention_decode_scratch_bytes(int B, int H, int Hkv, int D, int splits) {
  return splits > 1 ? ((int64_t)B * H * splits * (D + 2) + (int64_t)B * Hkv) * 4 : 0;
}

// What the cp.async variant takes (shared by the two entry points that launch it); 0 or a refusal.
static int check_decode_arguments(const void* q, int64_t ldq, int64_t ldo, const void* cache, int max_blocks, int B, int H,
                                  int Hkv, int D, int block_size, int splits) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || max_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode: bad sizes B=%d H=%d Hkv=%d", B, H, Hkv);
  if (!dinfer_attention_decode_supports(D, H / Hkv, block_size))
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode: head_dim %d, group %d, block_size %d not supported "
                  "(head_dim 64 or 128, group <= 16, power-of-two pages)", D, H / Hkv, block_size);
  if ((ldq % 2) || (ldo % 2) || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(cache) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode: q rows must be 4-byte and the cache 16-byte aligned");
  if (splits > 32) return refuse(DINFER_BAD_ARGUMENT, "attention_decode: at most 32 key splits, got %d", splits);
  if (splits < 1) return refuse(DINFER_BAD_ARGUMENT, "attention_decode: splits=%d", splits);
  if (Hkv > 65535 || B > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_decode: too many heads or requests for the grid");
  return 0;
}

// Requests whose portion is not exactly one token are skipped (left to the prompt kernel).
DINFER_API int dinfer_attention_decode(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                       const int* block_table, int max_blocks, const int* cu_seqlens,
                                       const int* seq_lens, int B, int H, int Hkv, int D, int block_size,
                                       float scale, int window, int splits, float* scratch_floats,
                                       int* scratch_counters, cudaStream_t stream) {
  if (int rc = check_decode_arguments(q, ldq, ldo, cache, max_blocks, B, H, Hkv, D, block_size, splits)) return rc;
  if (splits > 1 && (!scratch_floats || !scratch_counters))
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode: splits=%d needs scratch", splits);
  Params p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq; p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.H = H; p.Hkv = Hkv; p.group = H / Hkv;
  p.block_size = block_size; p.bs_log2 = 0;
  while ((1 << p.bs_log2) < block_size) ++p.bs_log2;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.splits = splits;
  p.part_o = scratch_floats;
  p.part_ml = scratch_floats ? scratch_floats + (int64_t)B * H * splits * D : nullptr;
  p.counters = scratch_counters; p.status = nullptr;
  const int nh8 = (p.group + 7) / 8;
  if (D == 64) return nh8 == 1 ? launch<64, 1>(p, B, stream) : launch<64, 2>(p, B, stream);
  return nh8 == 1 ? launch<128, 1>(p, B, stream) : launch<128, 2>(p, B, stream);
}

// The TMA variant (pages of at least 8 tokens): no scratch (the splits fold inside a cluster, at most
// 16 of them), plus the number of pages of the cache tensor (for the tensor map) and the device status
// word that a bounded wait sets when it runs out.
DINFER_API int dinfer_attention_decode_tma(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                           int64_t num_blocks, const int* block_table, int max_blocks,
                                           const int* cu_seqlens, const int* seq_lens, int B, int H, int Hkv, int D,
                                           int block_size, float scale, int window, int splits, int* status,
                                           cudaStream_t stream) {
  if (B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || max_blocks <= 0 || num_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: bad sizes B=%d H=%d Hkv=%d", B, H, Hkv);
  if (!dinfer_attention_decode_supports(D, H / Hkv, block_size) || block_size < 8)
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: head_dim %d, group %d, block_size %d not supported "
                  "(head_dim 64 or 128, group <= 16, power-of-two pages of at least 8)", D, H / Hkv, block_size);
  if ((ldq % 2) || (ldo % 2) || (reinterpret_cast<uintptr_t>(q) & 3) || (reinterpret_cast<uintptr_t>(cache) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: q rows must be 4-byte and the cache 16-byte aligned");
  if (splits < 1 || splits > MAX_CLUSTER_SPLITS)
    return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: 1 to %d key splits (one cluster), got %d", MAX_CLUSTER_SPLITS, splits);
  if (!status) return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: a status word is required");
  if (Hkv > 65535 || B > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: too many heads or requests for the grid");
  const int64_t cache_rows = num_blocks * 2 * Hkv * block_size;
  if (cache_rows > 0x7fffffffLL) return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: the cache has too many rows for a tensor map coordinate");
  EncodeTiledFn fn = encode_fn();
  if (!fn) return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap map;
  {
    const int br = block_size < BN ? block_size : BN;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)cache_rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)br};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "attention_decode_tma: tensor map of the cache failed with %d", (int)r);
  }
  Params p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq; p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.H = H; p.Hkv = Hkv; p.group = H / Hkv;
  p.block_size = block_size; p.bs_log2 = 0;
  while ((1 << p.bs_log2) < block_size) ++p.bs_log2;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.splits = splits;
  p.part_o = nullptr; p.part_ml = nullptr; p.counters = nullptr; p.status = status;
  const int nh8 = (p.group + 7) / 8;
  if (D == 64) return nh8 == 1 ? launch_tma<64, 1>(map, p, B, stream) : launch_tma<64, 2>(map, p, B, stream);
  return nh8 == 1 ? launch_tma<128, 1>(map, p, B, stream) : launch_tma<128, 2>(map, p, B, stream);
}

// ---- the entry point that allocates nothing (see attention_decode_static.h)
// The scratch of the split-key kernel as a fixed array in the library's device image.  In host code the
// name below is only a handle; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_decode_static_scratch[DINFER_DECODE_STATIC_SCRATCH_BYTES];

DINFER_API int dinfer_attention_decode_static(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                              const int* block_table, int max_blocks, const int* cu_seqlens,
                                              const int* seq_lens, int B, int H, int Hkv, int D, int block_size,
                                              float scale, int window, int splits, cudaStream_t stream) {
  constexpr int MAX_DEVICES = 64;
  static unsigned char* base[MAX_DEVICES] = {nullptr};
  static std::mutex base_lock;                    // two host threads may make their first calls together
  // everything is checked before anything is queued on the caller's stream
  if (int rc = check_decode_arguments(q, ldq, ldo, cache, max_blocks, B, H, Hkv, D, block_size, splits)) return rc;
  const int64_t floats = splits > 1 ? (int64_t)B * H * splits * (D + 2) : 0;
  const int64_t counters = splits > 1 ? (int64_t)B * Hkv : 0;
  if (floats > (int64_t)DINFER_DECODE_STATIC_FLOATS || counters > DINFER_DECODE_STATIC_COUNTERS)
    return refuse(DINFER_BAD_ARGUMENT,
                  "attention_decode_static: needs %lld floats and %lld counters of scratch, the fixed array holds %lld and %d "
                  "(fewer requests or splits, or the entry point that takes scratch from the caller)",
                  (long long)floats, (long long)counters, (long long)DINFER_DECODE_STATIC_FLOATS, DINFER_DECODE_STATIC_COUNTERS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
    return refuse(e != cudaSuccess ? (int)e : DINFER_BAD_ARGUMENT, "attention_decode_static: no usable current device (%d)", dev);
  unsigned char* mine;
  {
    std::lock_guard<std::mutex> hold(base_lock);
    if (!base[dev]) {                             // once per device, with that device current
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
      if (e != cudaSuccess || !p)
        return refuse((int)e, "attention_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      base[dev] = static_cast<unsigned char*>(p);
    }
    mine = base[dev];
  }
  float* fl = reinterpret_cast<float*>(mine);
  int* ct = reinterpret_cast<int*>(mine + (size_t)DINFER_DECODE_STATIC_FLOATS * 4);
  if (splits > 1) {                               // the counters must start at zero whatever the last call left
    e = cudaMemsetAsync(ct, 0, (size_t)counters * sizeof(int), stream);
    if (e != cudaSuccess) return refuse((int)e, "attention_decode_static: clearing the counters failed: %s", cudaGetErrorString(e));
  }
  return dinfer_attention_decode(q, ldq, out, ldo, cache, block_table, max_blocks, cu_seqlens, seq_lens, B, H, Hkv, D,
                                 block_size, scale, window, splits, splits > 1 ? fl : nullptr, splits > 1 ? ct : nullptr,
                                 stream);
}
