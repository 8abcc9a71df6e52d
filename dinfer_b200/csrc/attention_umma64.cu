// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// bfloat16, head size 64 or 128, group sizes that divide 128, pages of 8..64 tokens (power of two).
// The kernel for short contexts: key tiles of 64, so that the tiles on the diagonal (all there is of a short
// prompt) carry half the masked scores of the 128-key kernel in attention_umma.cu, and less to set up per CTA
// (a 128-token prompt alone 9 against 15 us, 32 of them 20 against 31 us at 16 heads over 8); beyond some 1024
// keys per row the other kernel's longer tiles win.  The grid counts the batch's row-tile pairs, as there.
//
// A CTA owns 2 x 128 rows of one (request, kv head); a row is a (token, query head of the group) pair, so
// the heads of a group share every K/V tile.  Per 64-key tile and 128-row group:
//     S[128, 64]  = Q K^T          tcgen05.mma, Q and K K-major in shared memory, S in tensor memory
//     P = softmax step             one thread per row (= TMEM lane): tcgen05.ld, mask, exp2, P -> shared memory (bf16)
//     O[128, D]  += P V            tcgen05.mma accumulating in tensor memory, V used as it lies in the cache
//                                  ([key][d] = MN-major B operand); O is rescaled in place only when a row's
//                                  maximum grows by more than 2^8
// Warp roles (352 threads): warp 0 = TMA producer (Q once through a 3-D map over [token][head][d]; K/V page
// by page through a 2-D map over the layer's cache, looked up in the block table), warp 1 = TMEM
// allocation + MMA issue for row tile A, warp 10 = MMA issue for row tile B (a tile's chain of products
// hangs on one issuing thread; two threads keep the tiles from waiting for each other), warps 2..5 and
// 6..9 = the softmax / output groups of the two row tiles.  K tiles
// and V tiles ride a 3-stage mbarrier ring each (K runs two tiles ahead of V).  S is double-buffered in
// tensor memory: the MMA thread issues Q K^T of tile j+2 right behind P V of tile j, so a group's softmax
// of tile j+1 finds its S ready when it has handed P of tile j over, and the tensor core works for one
// group while the other computes.  No cluster launch, no multicast.  Every mbarrier wait is bounded.
//
// Counterpart in the reference: gqa_fa_v5_kernel (crates/kernels/cuda/gqa.cu:167-369, mma.sync) for this
// head size; its tcgen05 attention (crates/kernels/cuda/gqa_fa_sm100.cu) exists for D = 256 only and stages
// by cp.async.
#include <cuda.h>

#include "common.cuh"
#include "umma_attention.cuh"

using namespace dinfer;
using namespace dinfer_umma;

namespace {

constexpr int BM = 128, BN = 64, STAGES = 3, NTHREADS = 352;   // BM rows per softmax group, two groups per CTA
constexpr int MMA_WARP_B = 10;                                  // the second MMA issuer (the first is warp 1)
constexpr int TABLE_SLOTS = 2048;

struct Params {
  __nv_bfloat16* out; int64_t ldo;
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int B, H, Hkv, group, block_size, bs_log2, window;
  float scale_log2;
  int* status;
};

template <int D> constexpr size_t smem_bytes() {
  return (size_t)(2 * BM * D * 2 + 2 * STAGES * BN * D * 2 + 2 * BM * BN * 2) + 1024;
}

// Two row tiles (A, B) of 128 rows per CTA, each with its own softmax warpgroup; the MMA thread feeds
// them alternately, so one group's softmax runs while the tensor core works for the other.
// O accumulates in tensor memory across tiles; a row's reference maximum is only raised when it grows
// by more than 2^8 (the accumulator and the running sum are then rescaled in place), so P stays below
// 256 and the rescale is rare.
template <int D>
__global__ void __launch_bounds__(NTHREADS, 1)
attention_umma64_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Params p) {
  constexpr int NH = D / 64;                          // 64-wide halves of the head
  constexpr uint32_t Q_HALF = BM * 128, KV_HALF = BN * 128;
  constexpr uint32_t Q_BYTES = NH * Q_HALF, KV_BYTES = NH * KV_HALF, P_BYTES = BM * BN * 2;
  constexpr int TMEM_COLS = 512, O_COL = 256;                  // S of (tile w, buffer b) at (2w + b) * 64; O_A 256, O_B 384
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES],
      s_full[2][2], p_full[2], pv_done[2], o_full[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_table[TABLE_SLOTS];
  __shared__ int s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hk = blockIdx.x;
  pdl_enter();
  // The grid's y counts the row-tile pairs of the whole batch (an upper bound of them): which request's pair this
  // is comes from the portions' lengths, summed by every warp for itself.  Requests that bring one token have no
  // pair (they belong to the decode kernel), so a step with many of them launches no CTAs for them.
  int b = -1, pair = 0, pairs_b = 0;
  {
    const int y = blockIdx.y;
    int before = 0;
    for (int i0 = 0; i0 < p.B; i0 += 32) {
      const int i = i0 + lane;
      int n = 0;
      if (i < p.B) {
        const int ql = p.cu_seqlens[i + 1] - p.cu_seqlens[i];
        n = ql > 1 ? (ql * p.group + 2 * BM - 1) / (2 * BM) : 0;
      }
      int incl = n;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      const int chunk = __shfl_sync(0xffffffffu, incl, 31);
      if (y < before + chunk) {
        const unsigned hit = __ballot_sync(0xffffffffu, y >= before + incl - n && y < before + incl);
        const int src = __ffs(hit) - 1;
        b = i0 + src;
        pair = y - before - __shfl_sync(0xffffffffu, incl - n, src);
        pairs_b = __shfl_sync(0xffffffffu, n, src);
        break;
      }
      before += chunk;
    }
  }
  if (b < 0) return;                                   // beyond the batch's pairs
  const int t0 = p.cu_seqlens[b];
  const int q_len = p.cu_seqlens[b + 1] - t0;
  const int rows_total = q_len * p.group;
  // CTAs start in the order of blockIdx (x fastest): every kv head of a request's longest (latest) row tile
  // first, so that the long CTAs do not start last and leave the other SMs idle at the end
  const int row0 = (pairs_b - 1 - pair) * 2 * BM;
  const int hist = p.seq_lens[b] - q_len;
  const int* table = p.block_table + (int64_t)b * p.max_blocks;
  const bool b_on = row0 + BM < rows_total;            // the second row tile exists
  const int first_tok = row0 / p.group;
  const int last_tok_a = (min(row0 + BM, rows_total) - 1) / p.group;
  const int last_tok = (min(row0 + 2 * BM, rows_total) - 1) / p.group;
  const int hi = hist + last_tok + 1;
  const int hi_a = hist + last_tok_a + 1;
  const int lo = p.window > 0 ? max(0, hist + first_tok - p.window + 1) : 0;
  const int tile_begin = lo / BN, tile_end = (hi + BN - 1) / BN;
  const int n_tiles = tile_end - tile_begin;           // tiles of B (or of A when B does not exist)
  const int n_tiles_a = (hi_a + BN - 1) / BN - tile_begin;

  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = sQ + 2 * Q_BYTES, sV = sK + STAGES * KV_BYTES, sP = sV + STAGES * KV_BYTES;

  // page-table slice of this CTA's keys, and zeroed K/V stages (a page that is skipped leaves its slot as it
  // was: it must hold finite numbers, because a masked key still meets 0 * V)
  const int table_first = (tile_begin * BN) >> p.bs_log2;
  {
    const int last = (min(tile_end * BN, hi) - 1) >> p.bs_log2;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NTHREADS) s_table[i] = table[table_first + i];
    uint4* z = reinterpret_cast<uint4*>(smem_dyn + (sK - smem_u32(smem_dyn)));
    for (int i = threadIdx.x; i < (int)(2 * STAGES * KV_BYTES / 16); i += NTHREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1); mbar_init(smem_u32(&k_empty[s]), 2);       // empty: both MMA issuers
      mbar_init(smem_u32(&v_full[s]), 1); mbar_init(smem_u32(&v_empty[s]), 2);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(smem_u32(&s_full[w][0]), 1);
      mbar_init(smem_u32(&s_full[w][1]), 1);
      mbar_init(smem_u32(&p_full[w]), 128);
      mbar_init(smem_u32(&pv_done[w]), 1);
      mbar_init(smem_u32(&o_full[w]), 1);
    }
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the zero fill above, before TMA writes the same bytes
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = s_tmem_base;

  if (warp == 0) {
    // ---- TMA producer: the whole warp.  Q once (lane 0); then per tile one copy per page, K / V and
    // 64-wide half, spread over the lanes so that they are requested side by side.
    if (lane == 0) {
      const uint32_t qb = smem_u32(&q_full);
      mbar_expect_tx(qb, (b_on ? 2 : 1) * Q_BYTES);
      for (int w = 0; w < (b_on ? 2 : 1); ++w)
        for (int h = 0; h < NH; ++h)
          tma_load_3d(sQ + w * Q_BYTES + h * Q_HALF, &map_q, h * 64, hk * p.group, t0 + first_tok + w * (BM / p.group), qb);
    }
    const int br = min(p.block_size, BN);                          // rows of one K/V box
    const int boxes = BN / br;
    const int n_ops = boxes * NH;                                  // copies of one of K / V of a tile, <= 16
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int s = j % STAGES;
      const int j0 = (tile_begin + j) * BN;
      // this lane's copy: page x of the tile, 64-wide half h (the same for K and for V)
      bool valid = false;
      int row_k = 0, col = 0; uint32_t off = 0;
      if (lane < n_ops) {
        const int x = lane / NH, h = lane % NH;
        const int key = j0 + x * br;
        if (key < hi && key + br > lo) {
          const int e = (key >> p.bs_log2) - table_first;
          const int blk = e < TABLE_SLOTS ? s_table[e] : table[key >> p.bs_log2];
          if (blk >= 0) {
            valid = true;
            row_k = (blk * 2 * p.Hkv + hk) * p.block_size + (key & (p.block_size - 1));
            col = h * 64;
            off = s * KV_BYTES + h * KV_HALF + x * br * 128;
          }
        }
      }
      const uint32_t bytes = __reduce_add_sync(0xffffffffu, valid ? (uint32_t)(br * 128) : 0u);
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        bool ok = true;
        if (lane == 0) ok = mbar_wait(smem_u32(kv == 0 ? &k_empty[s] : &v_empty[s]), ((j / STAGES) & 1) ^ 1);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { if (lane == 0) { s_abort = 1; atomicExch(p.status, 11); } alive = false; break; }
        const uint32_t bar = smem_u32(kv == 0 ? &k_full[s] : &v_full[s]);
        if (lane == 0) {
          if (bytes == 0) mbar_arrive(bar); else mbar_expect_tx(bar, bytes);
        }
        __syncwarp();
        if (valid) tma_load_2d((kv == 0 ? sK : sV) + off, &map_kv, col, row_k + kv * p.Hkv * p.block_size, bar);
      }
    }
  } else if (warp == 1 || warp == MMA_WARP_B) {
    if (lane == 0) {
      // ---- MMA issue: one thread per row tile (warp 1: tile A, the last warp: tile B).  Each runs its tile's
      // chain on its own, so neither waits for the other's softmax; the K and V stages go back to the producer
      // when both have committed (or, past the end of its tile, plainly arrived on) their empty barriers.
      const int w = warp == 1 ? 0 : 1;
      const int n_w = w == 0 ? n_tiles_a : (b_on ? n_tiles : 0);
      constexpr uint32_t idesc_qk = idesc_bf16(BM, BN, 0), idesc_pv = idesc_bf16(BM, D, 1);
      // descriptors differ from these bases by constants (16-byte units in the low field)
      const uint64_t dq = desc_k_major(sQ + w * Q_BYTES), dk = desc_k_major(sK);
      const uint64_t dp = desc_k_major(sP + w * P_BYTES), dv = desc_mn_major(sV, KV_HALF);
      const uint32_t o_tmem = tmem + O_COL + w * 128;
      auto issue_qk = [&](int t) {                                  // S_w[t % 2] = Q_w K(t)^T
        const uint64_t dks = dk + (uint64_t)((t % STAGES) * (KV_BYTES >> 4));
        const uint32_t s_tmem = tmem + (2 * w + (t & 1)) * BN;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          tc_mma(s_tmem, dq + (uint64_t)(((k / 4) * Q_HALF + (k % 4) * 32) >> 4),
                 dks + (uint64_t)(((k / 4) * KV_HALF + (k % 4) * 32) >> 4), idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(smem_u32(&s_full[w][t & 1]));
      };
      auto issue_pv = [&](int s, int j) {
        const uint64_t dvs = dv + (uint64_t)(s * (KV_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          tc_mma(o_tmem, dp + (uint64_t)(k * 2), dvs + (uint64_t)((k * 16 * 128) >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
      };
      bool ok = true;
      if (n_w > 0 && !mbar_wait(smem_u32(&q_full), 0)) { s_abort = 1; atomicExch(p.status, 12); ok = false; }
      // prologue: S of this row tile's first two key tiles
      for (int t = 0; t < 2 && t < n_tiles && ok; ++t) {
        if (t < n_w) {
          if (!mbar_wait(smem_u32(&k_full[t % STAGES]), 0)) { s_abort = 1; atomicExch(p.status, 12); ok = false; break; }
          tc_fence_after();
          issue_qk(t);
          tc_commit(smem_u32(&k_empty[t % STAGES]));
        } else {                                                   // not this tile's key tile: hand the stage back once it is full
          if (!mbar_wait(smem_u32(&k_full[t % STAGES]), 0)) { s_abort = 1; atomicExch(p.status, 12); ok = false; break; }
          mbar_arrive(smem_u32(&k_empty[t % STAGES]));
        }
      }
      // Past the end of its own row tile an issuer still takes every stage in step (it waits for the stage
      // to be full before it arrives on its empty barrier), so that a barrier never gets two arrivals of one
      // issuer in one phase.
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % STAGES;
        if (j < n_w) {
          if (!mbar_wait(smem_u32(&p_full[w]), j & 1)) { s_abort = 1; atomicExch(p.status, 13); ok = false; break; }
          if (!mbar_wait(smem_u32(&v_full[s]), (j / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); ok = false; break; }
          tc_fence_after();
          issue_pv(s, j);
          tc_commit(smem_u32(&pv_done[w]));                         // P_w is free again, O_w is quiet until the next P V
          if (j + 1 == n_w) tc_commit(smem_u32(&o_full[w]));         // this row tile's last P V
          tc_commit(smem_u32(&v_empty[s]));
        } else {
          if (!mbar_wait(smem_u32(&v_full[s]), (j / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); ok = false; break; }
          mbar_arrive(smem_u32(&v_empty[s]));
        }
        if (j + 2 < n_tiles) {
          const int s2 = (j + 2) % STAGES;
          if (j + 2 < n_w) {                                         // S of tile j + 2 into the buffer tile j just left
            if (!mbar_wait(smem_u32(&k_full[s2]), ((j + 2) / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); ok = false; break; }
            tc_fence_after();
            issue_qk(j + 2);
            tc_commit(smem_u32(&k_empty[s2]));
          } else {
            if (!mbar_wait(smem_u32(&k_full[s2]), ((j + 2) / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); ok = false; break; }
            mbar_arrive(smem_u32(&k_empty[s2]));
          }
        }
      }
    }
  } else {                                                          // ---- softmax and output: one thread per row
    const int w = (warp - 2) >> 2;                                  // row tile A (warps 2..5) or B (warps 6..9)
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int row = row0 + w * BM + r;
    const bool row_ok = row < rows_total;
    const int pos = row_ok ? hist + row / p.group : -1;
    const int n_w = w == 0 ? n_tiles_a : (b_on ? n_tiles : 0);
    const int first_tok_w = (row0 + w * BM) / p.group;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + 2 * w * BN, o_addr = lane_addr + O_COL + w * 128;
    unsigned char* prow = smem_dyn + (sP - smem_u32(smem_dyn)) + w * P_BYTES + r * 128;
    float m_run = -INFINITY, l_run = 0.f;                           // reference maximum (scaled, log2 units), running sum
    bool ok = true;
    for (int j = 0; j < n_w && ok; ++j) {
      if (!mbar_wait(smem_u32(&s_full[w][j & 1]), (j >> 1) & 1)) { s_abort = 1; atomicExch(p.status, 15); ok = false; break; }
      tc_fence_after();
      float s0[32], s1[32];
      tmem_ld32(s_addr + (j & 1) * BN, s0);
      tmem_ld32(s_addr + (j & 1) * BN + 32, s1);
      tmem_ld_wait();
      const int jbase = (tile_begin + j) * BN;
      const bool need_mask = (jbase + BN - 1 > hist + first_tok_w) || p.window > 0 || jbase < lo;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int ja = jbase + i, jc = jbase + 32 + i;
          if (!(ja <= pos && ja >= lo && (p.window <= 0 || ja > pos - p.window))) s0[i] = -INFINITY;
          if (!(jc <= pos && jc >= lo && (p.window <= 0 || jc > pos - p.window))) s1[i] = -INFINITY;
        }
      }
      // maximum of the raw scores (the scale is positive), as eight short chains instead of one long one
      float mq[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mq[i] = fmaxf(s0[i], s1[i]);
#pragma unroll
      for (int i = 8; i < 32; ++i) mq[i & 7] = fmaxf(mq[i & 7], fmaxf(s0[i], s1[i]));
      float mx = fmaxf(fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])), fmaxf(fmaxf(mq[4], mq[5]), fmaxf(mq[6], mq[7])));
      mx *= p.scale_log2;
      // raise the reference maximum only when it grows by more than 8 (in log2 units)
      const bool raise = mx > m_run + 8.f;
      bool pv_seen = j == 0;                                        // P V of tile j-1 known to be complete
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // O_w must be quiet: P V of tile j-1 complete (P V of tile j waits for our P)
        if (!mbar_wait(smem_u32(&pv_done[w]), (j - 1) & 1)) { s_abort = 1; atomicExch(p.status, 15); ok = false; break; }
        tc_fence_after();
        pv_seen = true;
        const float alpha = raise ? fast_exp2(m_run - mx) : 1.f;     // m_run = -inf gives 0
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tmem_ld32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(o_addr + c * 32, o);
        }
        tmem_st_wait();
      }
      if (raise) m_run = mx;
      const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
      float sq[8];                                                  // eight partial sums: short dependency chains
#pragma unroll
      for (int i = 0; i < 8; ++i) sq[i] = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        s0[i] = fast_exp2(fmaf(s0[i], p.scale_log2, neg_m));         // masked: -inf stays -inf, 2^-inf = 0
        s1[i] = fast_exp2(fmaf(s1[i], p.scale_log2, neg_m));
        sq[i & 7] += s0[i] + s1[i];
      }
      l_run += ((sq[0] + sq[1]) + (sq[2] + sq[3])) + ((sq[4] + sq[5]) + (sq[6] + sq[7]));
      // the P V of tile j-1 must have read P before it is overwritten
      if (!pv_seen) {
        if (!mbar_wait(smem_u32(&pv_done[w]), (j - 1) & 1)) { s_abort = 1; atomicExch(p.status, 15); ok = false; break; }
      }
      // P row r: 64 keys = 8 chunks of 16 bytes, swizzled like a K-major tile with 128-byte rows
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float* src = c < 4 ? s0 + c * 8 : s1 + (c - 4) * 8;
        uint4 v;
        v.x = pack_bf16(src[0], src[1]); v.y = pack_bf16(src[2], src[3]);
        v.z = pack_bf16(src[4], src[5]); v.w = pack_bf16(src[6], src[7]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = v;
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(&p_full[w]));
    }
    if (ok && n_w > 0) {
      if (!mbar_wait(smem_u32(&o_full[w]), 0)) { s_abort = 1; atomicExch(p.status, 16); ok = false; }
      tc_fence_after();
    }
    if (ok && n_w > 0) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* dst = row_ok ? p.out + (int64_t)(t0 + row / p.group) * p.ldo + (int64_t)(hk * p.group + row % p.group) * D
                                  : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        tmem_ld32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack_bf16(o[q4 * 8] * inv, o[q4 * 8 + 1] * inv); v.y = pack_bf16(o[q4 * 8 + 2] * inv, o[q4 * 8 + 3] * inv);
            v.z = pack_bf16(o[q4 * 8 + 4] * inv, o[q4 * 8 + 5] * inv); v.w = pack_bf16(o[q4 * 8 + 6] * inv, o[q4 * 8 + 7] * inv);
            reinterpret_cast<uint4*>(dst + c * 32)[q4] = v;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (s_abort) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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

template <int D>
int launch(const CUtensorMap& mq, const CUtensorMap& mkv, const Params& p, dim3 grid, cudaStream_t stream) {
  auto k = attention_umma64_kernel<D>;
  constexpr size_t sm = smem_bytes<D>();
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return refuse((int)e, "attention_umma64: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  launch_pdl(k, grid, dim3(NTHREADS), sm, stream, mq, mkv, p);
  return cuda_status("attention_umma64");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

DINFER_API int dinfer_attention_umma64_supports(int D, int group, int block_size) {
  return (D == 64 || D == 128) && group >= 1 && group <= 128 && (128 % group) == 0 && block_size >= 8 &&
         block_size <= 64 && (block_size & (block_size - 1)) == 0;
}

// Prompt portions (q_len > 1) only; requests that bring one token are skipped.
// q: [T, ...] rows of stride ldq with head h at h*D (all H heads); cache [num_blocks, 2, Hkv, block, D] bf16.
DINFER_API int dinfer_attention_umma64(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                     int64_t num_blocks, const int* block_table, int max_blocks,
                                     const int* cu_seqlens, const int* seq_lens, int T, int B, int H, int Hkv, int D,
                                     int block_size, float scale, int window, int max_q_len, int pair_bound,
                                     int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || max_blocks <= 0 || num_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: bad sizes T=%d B=%d H=%d Hkv=%d", T, B, H, Hkv);
  const int group = H / Hkv;
  if (!(scale > 0.f)) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: the score scale must be positive, got %g", (double)scale);
  if (!dinfer_attention_umma64_supports(D, group, block_size))
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: head_dim %d, group %d, block_size %d not supported "
                  "(head_dim 64 or 128, group dividing 128, power-of-two pages of 8 to 64)", D, group, block_size);
  if ((ldq % 8) || (ldo % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: rows and bases must be 16-byte aligned");
  if (!status) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: a status word is required");

  const int64_t cache_rows = num_blocks * 2 * Hkv * block_size;
  if (cache_rows > 0x7fffffffLL) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: the cache has too many rows for a tensor map coordinate");
  EncodeTiledFn fn = encode_fn();
  if (!fn) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap mq, mkv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)ldq * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(BM / group)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: tensor map of q failed with %d", (int)r);
  }
  {
    const int br = block_size < BN ? block_size : BN;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)cache_rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)br};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: tensor map of the cache failed with %d", (int)r);
  }
  Params p;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.H = H; p.Hkv = Hkv; p.group = group; p.block_size = block_size;
  p.bs_log2 = 0;
  while ((1 << p.bs_log2) < block_size) ++p.bs_log2;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status; p.B = B;
  // pairs of 128-row tiles in the batch: the caller's bound, or every request taken for the longest
  int64_t pairs = pair_bound > 0 ? pair_bound : (int64_t)B * (((int64_t)max_q_len * group + 2 * BM - 1) / (2 * BM));
  if (pairs > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_umma64: %lld row-tile pairs are too many for the grid", (long long)pairs);
  dim3 grid(Hkv, (unsigned)pairs, 1);
  return D == 64 ? launch<64>(mq, mkv, p, grid, stream) : launch<128>(mq, mkv, p, grid, stream);
}
