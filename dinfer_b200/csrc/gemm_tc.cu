// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 on the 5th-generation tensor cores:
// TMA (cp.async.bulk.tensor, 128-byte swizzle) stages K-major operand tiles in shared memory,
// one elected thread issues tcgen05.mma (kind::f16) with the f32 accumulator in tensor memory,
// tcgen05.commit hands shared-memory stages back to the producer, and four epilogue warps read the
// accumulator with tcgen05.ld.  No load is multicast.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue,
// warps 2..5 = epilogue (TMEM lane quarter = warp index mod 4).
//
// Two kernels:
//   * decoding (at most 64 tokens), gemm_tc_kernel: the 128 tile rows are WEIGHT rows and the (16..64)
//     columns are tokens (cta_group::1, 128 x N_TILE x 16), so that a handful of tokens still fills the
//     tensor-core tile and each CTA streams its weight rows from HBM exactly once; K may be split across up to
//     8 CTAs, which then form a thread-block cluster: every CTA owns a share of the tile's 128 rows, the others
//     store their partial sums of those rows into its shared memory (st.shared::cluster), and after one
//     cluster barrier each CTA adds its share up, always in split order, and writes it.  With `act` the
//     weight rows are (gate, up) pairs and the same epilogue writes silu(gate) * up, half as wide, so
//     the gated feed-forward needs no kernel between its two products.  Two more epilogues take the
//     RMSNorm between two products apart so that it needs no kernel either: `resid` adds the product into
//     the 32-bit residual, writes the new residual times the norm's weight (rounded) for the next product
//     and leaves each row's partial sums of squares; `ss_in` multiplies the next product's result by
//     rsqrt(mean of squares + eps) of its row, which commutes with the product.
//   * prompts (more tokens), gemm_tc_pair_kernel: the tile rows are tokens; two SMs share a 256 x 256 tile
//     (cta_group::2), persistent over tiles, with the same gated epilogue (see the kernel).
//
// Every wait on an mbarrier is bounded: on time-out the kernel records a code in a status word,
// lets copies in flight land, frees its tensor memory and returns (the host reads the status word).
//
// The reference uses cuBLASLt for these products (crates/kernels/src/gemm.rs:649-690) and mma.sync
// kernels for small M (crates/kernels/cuda/gemm_small_m.cu:148-285); its tcgen05 code
// (crates/kernels/cuda/umma.cuh) serves other architectures and stages by cp.async.
#include <cuda.h>

#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int TILE_M = 128;      // rows of the accumulator tile = TMEM lanes
constexpr int BLOCK_K = 64;      // one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int NTHREADS = 192;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct GemmParams {
  void* out; int64_t ldc;        // [tokens, N] row-major, bf16 or f32
  int tokens, N, K;
  int k_blocks_per_split, splits;
  int act;                       // 1: weight rows come in (gate, up) pairs and out[t, j] = silu(gate_j) * up_j, N / 2 wide
  // residual mode (decode orientation): the product is added into resid [tokens, ldr] (f32) and out gets the new
  // residual times norm_w, rounded; the sums of squares of the rows this CTA owns go to ss_out[part][token]
  float* resid; int64_t ldr;
  const void* norm_w; int norm_w_f32;
  float* ss_out;
  // scaled mode: x holds rows that still lack their division by the root mean square; out is multiplied by
  // rsqrt(sum over parts of ss_in[part][token] * inv_size + eps)
  const float* ss_in; int ss_parts;
  int ss_stride;                 // floats between the parts of ss_out / ss_in
  float inv_size, eps;
  int* status;                   // device status word: 0 = fine
};

// ---- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after `limit` polls or about two seconds, whichever comes first.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = WAIT_LIMIT) {
  uint64_t start = 0;
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 255) == 255) {
      const uint64_t now = global_ns();
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
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// ---- thread-block cluster: barrier phases and stores into another CTA's shared memory
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

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte swizzle:
// start address >> 4, leading byte offset 1 (unused with swizzle), stride byte offset 1024 B (8 rows),
// descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: f32 accumulator, bf16 A and B, both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <typename T> __device__ __forceinline__ T out_cast(float v);
template <> __device__ __forceinline__ float out_cast<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 out_cast<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float norm_weight(const GemmParams& p, int n) {
  return p.norm_w_f32 ? reinterpret_cast<const float*>(p.norm_w)[n]
                      : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.norm_w)[n]);
}
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }
// the prompt epilogue's: fast exponential and division, as the reference's gate kernel has them
// (crates/kernels/cuda/common.cuh:55); the quotient is 0 where 1 + e^-g passes 2^126, as is its limit
__device__ __forceinline__ float silu_mul_fast(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

template <int N_TILE> constexpr int tmem_cols() { return N_TILE <= 32 ? 32 : (N_TILE <= 64 ? 64 : (N_TILE <= 128 ? 128 : 256)); }
// Rows of the tile that one CTA of a split-K cluster owns, and the floats of its receive buffer
// [splits][N_TILE][rows]: splits * ceil(128 / splits) <= RECV_ROWS for every split count up to 8.
constexpr int MAX_SPLITS = 8;
constexpr int RECV_ROWS = 136;
__host__ __device__ constexpr int rows_per_cta(int splits) { return (TILE_M + splits - 1) / splits; }
template <int N_TILE, int STAGES> constexpr size_t gemm_smem_bytes(bool with_recv) {
  return (size_t)STAGES * (TILE_M * BLOCK_K + N_TILE * BLOCK_K) * 2 + 1024      // + slack to align to 1024
         + (with_recv ? (size_t)N_TILE * RECV_ROWS * 4 : 0);
}

// grid: (tiles of the 128-row operand, tiles of the N_TILE-row operand, K splits)
template <int N_TILE, int STAGES, typename OutT>
__global__ void __launch_bounds__(NTHREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_rstd[64];                                // scaled mode: per token column of this tile
  __shared__ float s_share[128];                              // [threads of a column][N_TILE]
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  constexpr uint32_t A_BYTES = TILE_M * BLOCK_K * 2, B_BYTES = N_TILE * BLOCK_K * 2;
  const uint32_t recv_base = smem_base + STAGES * (A_BYTES + B_BYTES);       // split-K receive buffer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a0 = blockIdx.x * TILE_M, b0 = blockIdx.y * N_TILE;
  const int total_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int kb_begin = blockIdx.z * p.k_blocks_per_split;
  const int kb_end = min(total_kb, kb_begin + p.k_blocks_per_split);
  const int n_kb = max(0, kb_end - kb_begin);
  pdl_launch_dependents();
  // split K: the CTAs of a tile are one cluster.  First phase of its barrier: every CTA has started,
  // so its shared memory may be written from the others (waited for just before those stores).
  const bool clustered = p.splits > 1 || p.resid != nullptr;   // the residual epilogue lives in the fold
  if (clustered) cluster_arrive_relaxed();

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    mbar_init(smem_u32(&tmem_full_bar), 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(tmem_cols<N_TILE>()) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == 0) {
    if (lane == 0) {                                            // ---- TMA producer
      // The weights do not depend on the kernels before this one: their first tiles are requested
      // at once, while the preceding kernel may still be running; the activations only after it has
      // completed (pdl_wait).  Both land on the same barrier of their stage.
      const int ahead = min(STAGES, n_kb);
      for (int i = 0; i < ahead; ++i) {
        const uint32_t bar = smem_u32(&full_bar[i]);
        mbar_expect_tx(bar, A_BYTES + B_BYTES);
        const uint32_t sa = smem_base + i * (A_BYTES + B_BYTES);
        tma_load_2d(sa, &map_a, (kb_begin + i) * BLOCK_K, a0, bar);
      }
      pdl_wait();
      for (int i = 0; i < ahead; ++i) {
        const uint32_t bar = smem_u32(&full_bar[i]);
        const uint32_t sa = smem_base + i * (A_BYTES + B_BYTES);
        tma_load_2d(sa + A_BYTES, &map_b, (kb_begin + i) * BLOCK_K, b0, bar);
      }
      for (int i = ahead; i < n_kb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) & 1) ^ 1)) { s_abort = 1; atomicExch(p.status, 1); break; }
        const uint32_t bar = smem_u32(&full_bar[s]);
        mbar_expect_tx(bar, A_BYTES + B_BYTES);
        const uint32_t sa = smem_base + s * (A_BYTES + B_BYTES);
        tma_load_2d(sa, &map_a, (kb_begin + i) * BLOCK_K, a0, bar);
        tma_load_2d(sa + A_BYTES, &map_b, (kb_begin + i) * BLOCK_K, b0, bar);
      }
    } else {
      pdl_enter();
    }
  } else if (warp == 1) {
    pdl_enter();
    if (lane == 0) {                                            // ---- MMA issue
      constexpr uint32_t idesc = instr_desc_bf16(TILE_M, N_TILE);
      bool ok = true;
      for (int i = 0; i < n_kb && ok; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 2); ok = false; break; }
        tcgen05_fence_after();
        const uint32_t sa = smem_base + s * (A_BYTES + B_BYTES);
        const uint64_t da = smem_desc_k_sw128(sa), db = smem_desc_k_sw128(sa + A_BYTES);
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k)              // +32 bytes per 16-element K step, in 16-byte units
          tcgen05_mma_f16(tmem, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tcgen05_commit(smem_u32(&empty_bar[s]));                // the stage is free once these MMAs have read it
      }
      if (ok) tcgen05_commit(smem_u32(&tmem_full_bar));          // accumulator complete
    }
  } else {                                                      // ---- epilogue: TMEM -> registers -> global
    pdl_enter();
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                          // accumulator row = TMEM lane
    if (p.ss_in) {
      // scaled mode: while the products run, one thread per token column adds that row's partial sums of
      // squares (always in the same order) and keeps 1 / rms
      // 128 / N_TILE threads share a column: thread k of them takes the parts k, k + that many, ... (loads in
      // flight side by side), then the first adds the shares up in order
      constexpr int TPC = 128 / N_TILE;
      const int e = (warp - 2) * 32 + lane;
      const int c = e % N_TILE, k = e / N_TILE;
      float sum = 0.f;
      if (b0 + c < p.tokens) {
        const float* src = p.ss_in + b0 + c;
        for (int q0 = k; q0 < p.ss_parts; q0 += 16 * TPC) {
          float v[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int q = q0 + u * TPC;
            v[u] = q < p.ss_parts ? __ldcg(src + (int64_t)q * p.ss_stride) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) sum += v[u];
        }
      }
      s_share[k * N_TILE + c] = sum;
      asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps
      if (k == 0) {
        float total = 0.f;
#pragma unroll
        for (int j = 0; j < TPC; ++j) total += s_share[j * N_TILE + c];
        s_rstd[c] = rsqrtf(total * p.inv_size + p.eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    bool ok = true;
    if (n_kb > 0) {
      ok = mbar_wait(smem_u32(&tmem_full_bar), 0);
      if (!ok && lane == 0) { s_abort = 1; atomicExch(p.status, 3); }
      tcgen05_fence_after();
    }
    if (clustered) cluster_wait_acquire();                      // all CTAs of the cluster run: stores may go out
    if (ok) {
      OutT* out = reinterpret_cast<OutT*>(p.out);
      const int rows_per = rows_per_cta(p.splits);
      const int owner = r / rows_per;                           // the CTA that adds up this row
      const uint32_t recv_remote = clustered ? map_to_cta(recv_base, owner) : 0u;
      const uint32_t my_rank = clustered ? cluster_ctarank() : 0u;
#pragma unroll 1
      for (int c0 = 0; c0 < N_TILE; c0 += 16) {
        uint32_t v[16];
        if (n_kb > 0) {
          tmem_ld_32x32b_x16(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
        {
          const int n = a0 + r;                                 // weight row; the columns are tokens
          if (!clustered && p.ss_in) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * s_rstd[c0 + j]);
          }
          if (!clustered && p.act) {
            // the up row of a pair sits in the next lane
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g = __uint_as_float(v[j]);
              const float u = __shfl_down_sync(0xffffffffu, g, 1);
              if (!(lane & 1) && n + 1 < p.N && b0 + c0 + j < p.tokens)
                out[(int64_t)(b0 + c0 + j) * p.ldc + (n >> 1)] = out_cast<OutT>(silu_mul(g, u));
            }
          } else if (!clustered) {
            if (n < p.N) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (b0 + c0 + j < p.tokens) out[(int64_t)(b0 + c0 + j) * p.ldc + n] = out_cast<OutT>(__uint_as_float(v[j]));
            }
          } else {
            // recv[split][token column][row of the owner's share]: consecutive lanes, consecutive words
            const uint32_t dst = recv_remote + (uint32_t)(((my_rank * N_TILE + c0) * rows_per + (r - owner * rows_per)) * 4);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (b0 + c0 + j < p.tokens) st_cluster_f32(dst + (uint32_t)(j * rows_per * 4), __uint_as_float(v[j]));
          }
        }
      }
    }
    tcgen05_fence_before();
  }

  // ---- split K: after the second barrier phase the partial sums of this CTA's rows are all here
  if (clustered) {
    __syncwarp();
    if (warp < 2) cluster_wait_acquire();                       // first phase (the epilogue warps have passed it)
    const int rank = (int)cluster_ctarank();
    const int rows_per = rows_per_cta(p.splits);
    const int rows_mine = min(rows_per, TILE_M - rank * rows_per);
    const int cols = min(N_TILE, p.tokens - b0);                // token columns that exist
    // residual mode: what this thread will add to is requested before the barrier, not behind it
    constexpr int PRE = 4;
    float pre_r[PRE], pre_w[PRE];
    if (p.resid) {
#pragma unroll
      for (int k = 0; k < PRE; ++k) {
        const int i = threadIdx.x + k * NTHREADS;
        pre_r[k] = 0.f; pre_w[k] = 0.f;
        if (i < cols * rows_mine) {
          const int c = i / rows_mine, rl = i - c * rows_mine;
          const int n = a0 + rank * rows_per + rl;
          if (n < p.N) { pre_r[k] = p.resid[(int64_t)(b0 + c) * p.ldr + n]; pre_w[k] = norm_weight(p, n); }
        }
      }
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    if (!s_abort) {
      OutT* out = reinterpret_cast<OutT*>(p.out);
      const float* recv = reinterpret_cast<const float*>(smem_dyn + (recv_base - smem_u32(smem_dyn)));
      if (p.resid) {
        // residual mode: the new residual, the next product's input, and the squares, which go through the
        // (now free) first receive slot so that one thread per token column adds them up in a fixed order
        float* sq = const_cast<float*>(recv);
        const int total = cols * rows_mine;
        int k = 0;
        for (int i = threadIdx.x; i < total; i += NTHREADS, ++k) {
          const int c = i / rows_mine, rl = i - c * rows_mine;
          const int n = a0 + rank * rows_per + rl;
          float acc = 0.f;
          for (int s = 0; s < p.splits; ++s) acc += recv[(s * N_TILE + c) * rows_per + rl];
          float v2 = 0.f;
          if (n < p.N) {
            const int64_t t = b0 + c;
            const float r0 = k < PRE ? pre_r[k] : p.resid[t * p.ldr + n];
            const float w = k < PRE ? pre_w[k] : norm_weight(p, n);
            const float v = r0 + acc;
            p.resid[t * p.ldr + n] = v;
            out[t * p.ldc + n] = out_cast<OutT>(v * w);
            v2 = v * v;
          }
          sq[c * rows_per + rl] = v2;
        }
        __syncthreads();
        if ((int)threadIdx.x < cols) {
          float sum = 0.f;
          for (int rl = 0; rl < rows_mine; ++rl) sum += sq[threadIdx.x * rows_per + rl];
          p.ss_out[(int64_t)((int)blockIdx.x * p.splits + rank) * p.ss_stride + b0 + threadIdx.x] = sum;
        }
      } else if (p.act) {                                       // (gate, up) pairs: rows_per is even (host)
        const int pairs_mine = rows_mine >> 1;
        for (int i = threadIdx.x; i < cols * pairs_mine; i += NTHREADS) {
          const int c = i / pairs_mine, pr = i - c * pairs_mine;
          float g = 0.f, u = 0.f;
          for (int s = 0; s < p.splits; ++s) {
            const float2 v = *reinterpret_cast<const float2*>(recv + (s * N_TILE + c) * rows_per + 2 * pr);
            g += v.x;
            u += v.y;
          }
          if (p.ss_in) { g *= s_rstd[c]; u *= s_rstd[c]; }
          const int n = a0 + rank * rows_per + 2 * pr;
          if (n + 1 < p.N) out[(int64_t)(b0 + c) * p.ldc + (n >> 1)] = out_cast<OutT>(silu_mul(g, u));
        }
      } else {
        for (int i = threadIdx.x; i < cols * rows_mine; i += NTHREADS) {
          const int c = i / rows_mine, rl = i - c * rows_mine;
          float acc = 0.f;
          for (int s = 0; s < p.splits; ++s) acc += recv[(s * N_TILE + c) * rows_per + rl];
          if (p.ss_in) acc *= s_rstd[c];
          const int n = a0 + rank * rows_per + rl;
          if (n < p.N) out[(int64_t)(b0 + c) * p.ldc + n] = out_cast<OutT>(acc);
        }
      }
    }
  }

  __syncthreads();
  if (warp == 1) {
    if (s_abort) {                                              // let copies and MMAs in flight finish before the memory goes back
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols<N_TILE>()) : "memory");
  }
}

// ---- prompts, two SMs on one tile: the CTAs of a cluster of two share a 256 x 256 output tile
// (tcgen05.mma.cta_group::2).  Each CTA stages its own 128 token rows and its own 128 of the 256 weight rows,
// so a stage is 32 KB instead of 48 and every byte of the weight tile is fetched by one SM of the pair only;
// the leader (cluster rank 0) issues the MMAs for both, which leave 128 accumulator rows in each CTA's tensor
// memory.  TMA completions of both CTAs count on the leader's barrier; tcgen05.commit hands stages and
// accumulators back to both CTAs at once.  No load is multicast.
// CTAs are persistent: a pair walks over tiles (token tile fastest, so that pairs running at the same time read the
// same few weight tiles from L2), the shared-memory ring runs on across tiles, and the accumulator is double-buffered
// in tensor memory (2 x 256 columns): the epilogue warps drain tile i while the MMAs of tile i + 1 run.  With GATED
// the weight rows are (gate, up) pairs and the epilogue writes silu(gate) * up, half as wide.
// (Narrower tiles, chosen so that the last round of tiles leaves fewer SMs idle, were measured and are slower at
// every shape.)
constexpr int NT = 256;                                                       // columns of the pair's tile
constexpr int C_STAGES = 6, C_ACC_BUFS = 2, C_TMEM_COLS = NT * C_ACC_BUFS;
constexpr uint32_t C_A_BYTES = TILE_M * BLOCK_K * 2, C_B_BYTES = (NT / 2) * BLOCK_K * 2;   // this CTA's rows of both operands
constexpr size_t C_SMEM_BYTES = (size_t)C_STAGES * (C_A_BYTES + C_B_BYTES) + 1024;

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  uint64_t start = 0;
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
    if ((i & 255) == 255) {
      const uint64_t now = global_ns();
      if (start == 0) start = now;
      else if (now - start > 2000000000ull) return false;
    }
  }
  return false;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// the completion is counted on a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {     // arrives on this barrier in both CTAs
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <typename OutT, bool GATED>
__global__ void __launch_bounds__(NTHREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t full_bar[C_STAGES], empty_bar[C_STAGES], acc_full_bar[C_ACC_BUFS], acc_empty_bar[C_ACC_BUFS];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                      // 0 = leader
  const int m_tiles = (p.tokens + 255) / 256, n_tiles = (p.N + NT - 1) / NT;
  const int tiles = m_tiles * n_tiles;
  const int total_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  pdl_enter();

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    for (int s = 0; s < C_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int b = 0; b < C_ACC_BUFS; ++b) { mbar_init(smem_u32(&acc_full_bar[b]), 1); mbar_init(smem_u32(&acc_empty_bar[b]), 8); }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(C_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive_release();                                     // both CTAs' barriers and tensor memory are ready
  cluster_wait_acquire();
  tcgen05_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == 0) {
    if (lane == 0) {                                            // ---- TMA producer (both CTAs)
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * NT + (int)rank * (NT / 2);
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const uint32_t s = it % C_STAGES;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / C_STAGES) & 1) ^ 1)) { s_abort = 1; atomicExch(p.status, 1); ok = false; break; }
          if (rank == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * (C_A_BYTES + C_B_BYTES));
          const uint32_t bar = map_to_cta(smem_u32(&full_bar[s]), 0);
          const uint32_t sa = smem_base + s * (C_A_BYTES + C_B_BYTES);
          tma_load_2d_pair(sa, &map_a, kb * BLOCK_K, m0, bar);
          tma_load_2d_pair(sa + C_A_BYTES, &map_b, kb * BLOCK_K, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {                               // ---- MMA issue (the leader, for both CTAs)
      constexpr uint32_t idesc = instr_desc_bf16(256, NT);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++lt) {
        const uint32_t b = lt % C_ACC_BUFS;
        if (!mbar_wait_cluster(smem_u32(&acc_empty_bar[b]), ((lt / C_ACC_BUFS) & 1) ^ 1)) { s_abort = 1; atomicExch(p.status, 2); break; }
        tcgen05_fence_after();
        const uint32_t acc = tmem + b * NT;
        for (int kb = 0; kb < total_kb; ++kb, ++it) {
          const uint32_t s = it % C_STAGES;
          if (!mbar_wait_cluster(smem_u32(&full_bar[s]), (it / C_STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 2); ok = false; break; }
          tcgen05_fence_after();
          const uint32_t sa = smem_base + s * (C_A_BYTES + C_B_BYTES);
          const uint64_t da = smem_desc_k_sw128(sa), db = smem_desc_k_sw128(sa + C_A_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
            tcgen05_mma_f16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tcgen05_commit_pair(smem_u32(&empty_bar[s]));
        }
        if (ok) tcgen05_commit_pair(smem_u32(&acc_full_bar[b]));
      }
    }
  } else {                                                      // ---- epilogue (both CTAs, 128 rows each)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    OutT* out = reinterpret_cast<OutT*>(p.out);
    const bool vec = sizeof(OutT) == 2 && (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
    const int n_out = GATED ? p.N / 2 : p.N;
    uint32_t lt = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++lt) {
      const uint32_t b = lt % C_ACC_BUFS;
      const int m0 = (tile % m_tiles) * 256 + (int)rank * 128, n0 = (tile / m_tiles) * NT;
      if (total_kb > 0) {
        if (!mbar_wait(smem_u32(&acc_full_bar[b]), (lt / C_ACC_BUFS) & 1)) {
          if (lane == 0) { s_abort = 1; atomicExch(p.status, 3); }
          break;
        }
        tcgen05_fence_after();
      }
      const int t = m0 + r;
      const uint32_t acc = tmem + ((uint32_t)(quarter * 32) << 16) + b * NT;
#pragma unroll 1
      for (int c0 = 0; c0 < NT; c0 += 32) {
        uint32_t v[2][16];
        if (total_kb > 0) {
          tmem_ld_32x32b_x16(acc + c0, v[0]);
          tmem_ld_32x32b_x16(acc + c0 + 16, v[1]);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) { v[0][j] = 0u; v[1][j] = 0u; }
        }
        if (t >= p.tokens) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if constexpr (GATED) {
            const int o0 = (n0 + c0 + h * 16) >> 1;
            OutT* dst = out + (int64_t)t * p.ldc + o0;
            float y[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) y[j] = silu_mul_fast(__uint_as_float(v[h][2 * j]), __uint_as_float(v[h][2 * j + 1]));
            if (vec && o0 + 8 <= n_out) {
              uint4 w0;
              __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&w0);
#pragma unroll
              for (int j = 0; j < 4; ++j) h0[j] = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
              *reinterpret_cast<uint4*>(dst) = w0;
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (o0 + j < n_out) dst[j] = out_cast<OutT>(y[j]);
            }
          } else {
            const int o0 = n0 + c0 + h * 16;
            OutT* dst = out + (int64_t)t * p.ldc + o0;
            if (vec && o0 + 16 <= n_out) {
              uint4 w0, w1;
              __nv_bfloat162* h0 = reinterpret_cast<__nv_bfloat162*>(&w0);
              __nv_bfloat162* h1 = reinterpret_cast<__nv_bfloat162*>(&w1);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                h0[j] = __floats2bfloat162_rn(__uint_as_float(v[h][2 * j]), __uint_as_float(v[h][2 * j + 1]));
                h1[j] = __floats2bfloat162_rn(__uint_as_float(v[h][8 + 2 * j]), __uint_as_float(v[h][8 + 2 * j + 1]));
              }
              reinterpret_cast<uint4*>(dst)[0] = w0;
              reinterpret_cast<uint4*>(dst)[1] = w1;
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (o0 + j < n_out) dst[j] = out_cast<OutT>(__uint_as_float(v[h][j]));
            }
          }
        }
      }
      // read: the leader may let the MMAs of a later tile overwrite this accumulator in both CTAs
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty_bar[b]), 0));
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive_release();                                     // neither CTA leaves while the other may still signal it
  cluster_wait_acquire();
  if (warp == 1) {
    if (s_abort) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C_TMEM_COLS) : "memory");
  }
}

// ---- host side
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

// bf16 matrix [rows, K] with row stride ld (elements); box = 64 columns x box_rows rows, 128-byte swizzle
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BLOCK_K, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r);
  return 0;
}

template <int N_TILE, int STAGES, typename OutT>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, dim3 grid, cudaStream_t stream) {
  auto k = gemm_tc_kernel<N_TILE, STAGES, OutT>;
  const size_t sm = gemm_smem_bytes<N_TILE, STAGES>(p.splits > 1 || p.resid != nullptr);
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes<N_TILE, STAGES>(true));
    if (e != cudaSuccess) return refuse((int)e, "gemm_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  cudaError_t e = launch_pdl_cluster(k, grid, dim3(NTHREADS), dim3(1, 1, p.splits), sm, stream, ma, mb, p);
  if (e != cudaSuccess) return refuse((int)e, "gemm_tc: launch failed: %s", cudaGetErrorString(e));
  return cuda_status("gemm_tc");
}

// What every bounded wait of this file does when it runs out, on its own: one CTA allocates tensor memory, waits
// on an mbarrier that nobody arrives at (at most `polls` polls), records code 2, frees its tensor memory and
// returns.  Launched by tests of the failure path only.
__global__ void __launch_bounds__(64) wait_probe_kernel(int* status, uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t s_tmem_base;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (threadIdx.x == 0 && !mbar_wait(smem_u32(&bar), 0, polls)) atomicExch(status, 2);
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(s_tmem_base), "r"(32) : "memory");
}

int num_sms() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

// clusters of two CTAs of `kernel` that the device runs at a time
int cluster_pairs_resident(const void* kernel, size_t smem) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * num_sms()); cfg.blockDim = dim3(NTHREADS); cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

template <typename OutT, bool GATED>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  auto k = gemm_tc_pair_kernel<OutT, GATED>;
  static int max_pairs = 0;
  if (!max_pairs) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C_SMEM_BYTES);
    if (e != cudaSuccess) return refuse((int)e, "gemm_tc: shared memory opt-in failed: %s", cudaGetErrorString(e));
    const int n = cluster_pairs_resident(reinterpret_cast<const void*>(k), C_SMEM_BYTES);
    if (n <= 0) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: no cluster of two CTAs fits this device");
    max_pairs = n;
  }
  const int tiles = ((p.tokens + 255) / 256) * ((p.N + NT - 1) / NT);
  dim3 grid(2 * (tiles < max_pairs ? tiles : max_pairs));
  cudaError_t e = launch_pdl_cluster(k, grid, dim3(NTHREADS), dim3(2, 1, 1), C_SMEM_BYTES, stream, ma, mb, p);
  if (e != cudaSuccess) return refuse((int)e, "gemm_tc: launch failed: %s", cudaGetErrorString(e));
  return cuda_status("gemm_tc");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// x [tokens, K] (row stride ldx), w [N, K] (row stride ldw), both bf16; out [tokens, N] (row stride ldc)
// bf16 (out_f32 = 0) or f32.  tokens <= 64: decode orientation with `splits` K splits (at most 8: the
// CTAs of a tile form a cluster).  More tokens: prompt orientation (two SMs on a tile), splits ignored.
// act = 1 (N even): the rows of w are (gate, up) pairs and out is [tokens, N / 2],
// out[t, j] = silu(x w_{2j}) * (x w_{2j+1}).
// status: a device int that a kernel sets non-zero when one of its bounded waits ran out.
//
// The two halves of an RMSNorm between two decode products (tokens <= 64, see the kernel's header):
//   resid != null: resid [tokens, ldr] f32 += product; out = (new residual) * norm_w (bf16 or f32 vector of N);
//                  ss_out[part * ss_stride + token] = sum of squares of the new residual over the part's rows,
//                  for part < dinfer_gemm_tc_parts(tokens, N, K, splits);
//   ss_in != null: out *= rsqrt(sum_{part < ss_parts} ss_in[part * ss_stride + token] * inv_size + eps).
DINFER_API int dinfer_gemm_tc_fused(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldc,
                                    int out_f32, int tokens, int N, int K, int splits, int act, float* resid, int64_t ldr,
                                    const void* norm_w, int norm_w_f32, float* ss_out, const float* ss_in, int ss_parts,
                                    int ss_stride, float inv_size, float eps, int* status, cudaStream_t stream) {
  if (tokens < 0 || N <= 0 || K <= 0) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: bad sizes tokens=%d N=%d K=%d", tokens, N, K);
  if (tokens == 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldw % 8) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: K and the row strides must be multiples of 8 and the bases 16-byte aligned "
                  "(TMA); K=%d ldx=%lld ldw=%lld", K, (long long)ldx, (long long)ldw);
  if (!status) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: a status word is required");
  if (act && (N & 1))
    return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: the gated epilogue takes an even N (N=%d)", N);
  if ((resid || ss_in) && tokens > 64)
    return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: the norm epilogues take at most 64 tokens, got %d", tokens);
  if (resid && (act || !norm_w || !ss_out || ss_stride < tokens))
    return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: the residual epilogue needs the norm's weight and room for the sums, and no gate");
  if (ss_in && (ss_parts <= 0 || ss_stride < tokens))
    return refuse(DINFER_BAD_ARGUMENT, "gemm_tc: the scaled epilogue needs the parts of the sums (parts=%d stride=%d)", ss_parts, ss_stride);
  GemmParams p;
  p.act = act ? 1 : 0;
  p.resid = resid; p.ldr = ldr; p.norm_w = norm_w; p.norm_w_f32 = norm_w_f32; p.ss_out = ss_out;
  p.ss_in = ss_in; p.ss_parts = ss_parts; p.ss_stride = ss_stride; p.inv_size = inv_size; p.eps = eps;
  p.out = out; p.ldc = ldc; p.tokens = tokens; p.N = N; p.K = K; p.status = status;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  CUtensorMap ma, mb;
  int rc;
  if (tokens <= 64) {
    const int n_tile = tokens <= 16 ? 16 : (tokens <= 32 ? 32 : 64);
    if (splits < 1) splits = 1;
    if (splits > MAX_SPLITS) splits = MAX_SPLITS;
    if (splits > total_kb) splits = total_kb;
    for (;;) {
      p.k_blocks_per_split = (total_kb + splits - 1) / splits;
      p.splits = (total_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
      // with the gated epilogue a (gate, up) pair must stay in one CTA: 128 / splits rows each, a power of two
      if (!act || !(p.splits & (p.splits - 1))) break;
      --splits;
    }
    if ((rc = make_map(&ma, w, N, K, ldw, TILE_M))) return rc;
    if ((rc = make_map(&mb, x, tokens, K, ldx, n_tile))) return rc;
    dim3 grid((N + TILE_M - 1) / TILE_M, (tokens + n_tile - 1) / n_tile, p.splits);
#define GO(NT_, ST_) (out_f32 ? launch<NT_, ST_, float>(ma, mb, p, grid, stream) \
                              : launch<NT_, ST_, __nv_bfloat16>(ma, mb, p, grid, stream))
    // Four stages leave room for two CTAs of a split launch on an SM; a launch with more CTAs than that
    // takes three stages, of which three CTAs fit (as many bytes in flight, one wave instead of two).
    if (n_tile == 16) return (p.splits > 1 && (int64_t)grid.x * grid.y * grid.z > 264) ? GO(16, 3) : GO(16, 4);
    if (n_tile == 32) return GO(32, 4);
    return p.splits > 1 ? GO(64, 3) : GO(64, 4);              // with the receive buffer, two CTAs fit with three stages
#undef GO
  }
  p.k_blocks_per_split = total_kb;
  p.splits = 1;
  if ((rc = make_map(&ma, x, tokens, K, ldx, TILE_M))) return rc;
  if ((rc = make_map(&mb, w, N, K, ldw, NT / 2))) return rc;
  if (act) return out_f32 ? launch_pair<float, true>(ma, mb, p, stream) : launch_pair<__nv_bfloat16, true>(ma, mb, p, stream);
  return out_f32 ? launch_pair<float, false>(ma, mb, p, stream) : launch_pair<__nv_bfloat16, false>(ma, mb, p, stream);
}

DINFER_API int dinfer_gemm_tc(const void* x, int64_t ldx, const void* w, int64_t ldw, void* out, int64_t ldc,
                              int out_f32, int tokens, int N, int K, int splits, int act, int* status,
                              cudaStream_t stream) {
  return dinfer_gemm_tc_fused(x, ldx, w, ldw, out, ldc, out_f32, tokens, N, K, splits, act, nullptr, 0, nullptr, 0,
                              nullptr, nullptr, 0, 0, 0.f, 0.f, status, stream);
}

// For tests of the failure path: a wait of at most `polls` polls (1..65536) that nothing ends; the kernel gives
// up, sets *status = 2, frees its tensor memory and returns.
DINFER_API int dinfer_gemm_tc_wait_probe(int* status, int polls, cudaStream_t stream) {
  if (!status) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc_wait_probe: a status word is required");
  if (polls < 1 || polls > 65536) return refuse(DINFER_BAD_ARGUMENT, "gemm_tc_wait_probe: polls must be in 1..65536, got %d", polls);
  wait_probe_kernel<<<1, 64, 0, stream>>>(status, (uint32_t)polls);
  return cuda_status("gemm_tc_wait_probe");
}

// Parts of the sums of squares the residual epilogue writes for these sizes: 128-row tiles times effective K splits.
DINFER_API int dinfer_gemm_tc_parts(int tokens, int N, int K, int splits) {
  if (tokens <= 0 || tokens > 64 || N <= 0 || K <= 0) return 0;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (splits < 1) splits = 1;
  if (splits > MAX_SPLITS) splits = MAX_SPLITS;
  if (splits > total_kb) splits = total_kb;
  const int per = (total_kb + splits - 1) / splits;
  return ((N + TILE_M - 1) / TILE_M) * ((total_kb + per - 1) / per);
}
