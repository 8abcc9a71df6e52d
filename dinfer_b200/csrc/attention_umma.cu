// Paged causal attention for prompt portions on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// bfloat16, head size 64 or 128, group sizes that divide 128, pages of 8 tokens or more (a power of two).
//
// A CTA owns 2 x 128 rows of one (request, kv head); a row is a (token, query head of the group) pair, so
// the heads of a group share every K/V tile.  Per 128-key tile and 128-row tile:
//     S[128, 128] = Q K^T          tcgen05.mma, Q and K K-major in shared memory, S in tensor memory
//     P = softmax step             two threads per row (= TMEM lane), 64 keys each: tcgen05.ld, mask, the row's
//                                  maximum (the halves' maxima meet in shared memory), exp2; P goes back into
//                                  tensor memory as bfloat16, over columns of S its thread has read (tcgen05.st)
//     O[128, D]  += P V            tcgen05.mma with A = P from tensor memory and B = V as it lies in the cache
//                                  ([key][d] = MN-major operand); O is rescaled in place only when a row's
//                                  maximum grows by more than 2^8
// Tensor memory (512 columns): S of row tile A, S of row tile B, O of A, O of B, 128 columns each.
// Warp roles (608 threads, at most 96 registers each): warp 0 = Q once (a 3-D map over [token][head][d]) and the K
// tiles, warp 18 = the V tiles (page by page through a 2-D map over the layer's cache, looked up in the block
// table; each on its own 2-stage mbarrier ring), warp 1 = TMEM allocation + MMA issue, warps 2..17 = softmax and
// output: (row tile, half of the keys) by groups of four warps, TMEM lane quarter = warp index mod 4.
// A row tile's chain is  Q K^T -> softmax -> P V, Q K^T of the next tile -> ...; the one issuing thread serves the two
// row tiles strictly in turn and puts P V and the next Q K^T into the tensor pipe together, which runs them in order:
// the next S overwrites P only after P V has read it, and the tensor core works for one row tile while the
// other's softmax computes.  Every mbarrier wait is bounded; the named barriers between the two warps of a row
// are passed by both even after a wait has run out.
// With key_splits > 1 the launch is a cluster of that many CTAs on one row-tile pair: each takes a run of the
// pair's key tiles, and the partial results (O, reference maximum, sum) are folded through distributed shared
// memory behind two cluster barriers, each CTA writing out a share of the 256 rows.  No multicast.
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

constexpr int BM = 128, BN = 128, STAGES = 2, NTHREADS = 608;   // BM rows per row tile, two row tiles per CTA
constexpr int V_WARP = 18;                                     // the second producer warp (the first is warp 0)
constexpr int TABLE_SLOTS = 2048;

struct Params {
  __nv_bfloat16* out; int64_t ldo;
  const int* block_table; int max_blocks;
  const int* cu_seqlens; const int* seq_lens;
  int B, H, Hkv, group, block_size, bs_log2, window;
  int ksplit;                          // CTAs of a cluster that share a row-tile pair's keys (1, 2, 4 or 8)
  float scale_log2;
  int* status;
};

template <int D> constexpr size_t smem_bytes() {
  return (size_t)(2 * BM * D * 2 + 2 * STAGES * BN * D * 2) + 1024;      // Q of both row tiles, K and V stages
}

// Two row tiles (A, B) of 128 rows per CTA, each with eight softmax warps.  O accumulates in tensor memory
// across tiles; a row's reference maximum is only raised when it grows by more than 2^8 (the accumulator and
// the running sums are then rescaled in place), so P stays below 256 and the rescale is rare.
template <int D>
__global__ void __maxnreg__(96)
attention_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Params p) {
  constexpr int NH = D / 64;                          // 64-wide halves of the head
  constexpr uint32_t Q_HALF = BM * 128, KV_HALF = BN * 128;
  constexpr uint32_t Q_BYTES = NH * Q_HALF, KV_BYTES = NH * KV_HALF;
  constexpr int TMEM_COLS = 512, O_COL = 256;                  // S (and P over it) of row tile w at w * 128; O_A 256, O_B 384
  extern __shared__ unsigned char smem_dyn[];
  __shared__ __align__(8) uint64_t q_full, k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES],
      s_full[2], p_full[2], o_full[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_table[TABLE_SLOTS];
  __shared__ int s_abort;
  __shared__ float s_sum[2][2][BM];                       // a row's running sum, by the halves of its keys
  __shared__ float s_max[2][2][2][BM];                    // a tile's row maxima, by the halves of its keys
  __shared__ float x_max[2 * BM], x_sum[2 * BM];          // what the other CTAs of a cluster found for the rows this one writes
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = p.ksplit > 1 ? (int)cluster_ctarank() : 0;   // the cluster spans ksplit neighbours of the grid's x
  const int hk = blockIdx.x / p.ksplit;
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
  // the key tiles of the pair, dealt out to the cluster's CTAs in runs of `per` (a CTA may get none)
  const int tile_first = lo / BN;
  const int n_all = (hi + BN - 1) / BN - tile_first;   // tiles of B (or of A when B does not exist)
  const int n_all_a = (hi_a + BN - 1) / BN - tile_first;
  // The launch's split is an upper bound (a graph is captured for the longest request there may be): a pair is
  // shared by as many CTAs as leave each at least four tiles; the cluster's other CTAs have nothing to do with it.
  int ks = p.ksplit;
  while (ks > 1 && n_all < 4 * ks) ks >>= 1;
  if (rank >= ks) return;
  const int per = (n_all + ks - 1) / ks;
  const int tile_begin = tile_first + rank * per;
  const int n_tiles = max(0, min(per, n_all - rank * per));
  const int n_tiles_a = max(0, min(per, n_all_a - rank * per));

  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = sQ + 2 * Q_BYTES, sV = sK + STAGES * KV_BYTES;

  // page-table slice of this CTA's keys, and zeroed K/V stages (a page that is skipped leaves its slot as it
  // was: it must hold finite numbers, because a masked key still meets 0 * V)
  const int table_first = (tile_begin * BN) >> p.bs_log2;
  {
    const int last = (min((tile_begin + n_tiles) * BN, hi) - 1) >> p.bs_log2;
    for (int i = threadIdx.x; i < TABLE_SLOTS && table_first + i <= last; i += NTHREADS) s_table[i] = table[table_first + i];
    uint4* z = reinterpret_cast<uint4*>(smem_dyn + (sK - smem_u32(smem_dyn)));
    for (int i = threadIdx.x; i < (int)(2 * STAGES * KV_BYTES / 16); i += NTHREADS) z[i] = make_uint4(0, 0, 0, 0);
  }
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1); mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1); mbar_init(smem_u32(&v_empty[s]), 1);
    }
    for (int w = 0; w < 2; ++w) {
      mbar_init(smem_u32(&s_full[w]), 1);
      mbar_init(smem_u32(&p_full[w]), 256);
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

  if (warp == 0 || warp == V_WARP) {
    // ---- TMA producers: warp 0 brings Q (once, lane 0) and the K tiles, another warp the V tiles, each walking
    // its own ring; per tile one copy per page and 64-wide half, spread over the lanes.  (A copy of a page's
    // 2 KB takes the issuing warp some 85 cycles: two warps issue side by side.)
    const int kv = warp == 0 ? 0 : 1;
    if (kv == 0 && lane == 0) {
      const uint32_t qb = smem_u32(&q_full);
      mbar_expect_tx(qb, (b_on ? 2 : 1) * Q_BYTES);
      for (int w = 0; w < (b_on ? 2 : 1); ++w)
        for (int h = 0; h < NH; ++h)
          tma_load_3d(sQ + w * Q_BYTES + h * Q_HALF, &map_q, h * 64, hk * p.group, t0 + first_tok + w * (BM / p.group), qb);
    }
    const int br = min(p.block_size, BN);                          // rows of one K/V box
    const int boxes = BN / br;
    const int n_ops = boxes * NH;                                  // copies of one of K / V of a tile, <= 32
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int s = j % STAGES;
      const int j0 = (tile_begin + j) * BN;
      // this lane's copy: page x of the tile, 64-wide half h
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
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issue: one thread, the two row tiles strictly in turn: P V of tile j and, right behind it, Q K^T
      // of tile j + 1 for row tile A, then the same for row tile B.  The tensor pipe runs them in that order, so a
      // row tile's next S overwrites its P only after P V has read it, and while the pipe works for one row tile
      // the other's softmax computes: the turns keep the two a half step apart.
      constexpr uint32_t idesc_qk = idesc_bf16(BM, BN, 0), idesc_pv = idesc_bf16(BM, D, 1);
      // descriptors differ from these bases by constants (16-byte units in the low field)
      const uint64_t dq = desc_k_major(sQ), dk = desc_k_major(sK);
      const uint64_t dv = desc_mn_major(sV, KV_HALF);
      const int n_of[2] = {n_tiles_a, b_on ? n_tiles : 0};
      auto issue_qk = [&](int w, int t) {                           // S_w = Q_w K(t)^T
        const uint64_t dqs = dq + (uint64_t)(w * (Q_BYTES >> 4));
        const uint64_t dks = dk + (uint64_t)((t % STAGES) * (KV_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          tc_mma(tmem + w * BN, dqs + (uint64_t)(((k / 4) * Q_HALF + (k % 4) * 32) >> 4),
                 dks + (uint64_t)(((k / 4) * KV_HALF + (k % 4) * 32) >> 4), idesc_qk, k > 0 ? 1u : 0u);
        tc_commit(smem_u32(&s_full[w]));
      };
      auto issue_pv = [&](int w, int s, int j) {                    // O_w += P_w V(j), P from the columns of S_w
        const uint64_t dvs = dv + (uint64_t)(s * (KV_BYTES >> 4));
        const uint32_t s_tmem = tmem + w * BN, o_tmem = tmem + O_COL + w * 128;
#pragma unroll
        for (int k = 0; k < BN / 16; ++k)
          tc_mma_ts(o_tmem, s_tmem + (k / 4) * 64 + (k % 4) * 8, dvs + (uint64_t)((k * 16 * 128) >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
      };
      bool ok = true;
      if (!mbar_wait(smem_u32(&q_full), 0)) { s_abort = 1; atomicExch(p.status, 12); ok = false; }
      if (ok && n_tiles > 0) {                                      // S of the first key tile, for both row tiles
        if (!mbar_wait(smem_u32(&k_full[0]), 0)) { s_abort = 1; atomicExch(p.status, 12); ok = false; }
        else {
          tc_fence_after();
          for (int w = 0; w < 2; ++w)
            if (n_of[w] > 0) issue_qk(w, 0);
          tc_commit(smem_u32(&k_empty[0]));
        }
      }
      // V of a tile and K of the next are there long before the tile's P.  The thread looks for them while it would
      // wait anyway (between the two row tiles' turns of the step before), so that nothing but the issue itself
      // stands between a row tile's P and its next S.
      bool ahead = false;                                           // V(j) and K(j + 1) already seen
      // The wait for a row tile's P is a tight loop of looks (this thread has nothing else to do, and a suspended
      // wait wakes up late); between looks it sees to the next step's V and K.
      auto wait_p = [&](int w, int j, uint32_t v_next, uint32_t v_par, uint32_t k_next, uint32_t k_par, bool look) {
        const uint32_t bar = smem_u32(&p_full[w]);
        uint64_t start = 0;
        for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
          if (mbar_test(bar, j & 1)) return true;
          if (look && !ahead) ahead = mbar_test(v_next, v_par) && (k_next == 0 || mbar_test(k_next, k_par));
          if ((i & 255) == 255) {
            const uint64_t now = global_ns();
            if (start == 0) start = now;
            else if (now - start > 2000000000ull) return false;
          }
        }
        return false;
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % STAGES, s1 = (j + 1) % STAGES;
        if (!ahead) {
          if (!mbar_spin(smem_u32(&v_full[s]), (j / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); break; }
          if (j + 1 < n_tiles && !mbar_spin(smem_u32(&k_full[s1]), ((j + 1) / STAGES) & 1)) { s_abort = 1; atomicExch(p.status, 14); break; }
        }
        ahead = false;
        const bool look = j + 1 < n_tiles;                          // V(j + 1) and K(j + 2) went out a step ago
        const uint32_t v_next = smem_u32(&v_full[s1]), v_par = ((j + 1) / STAGES) & 1;
        const uint32_t k_next = j + 2 < n_tiles ? smem_u32(&k_full[s]) : 0u, k_par = ((j + 2) / STAGES) & 1;
        for (int w = 0; w < 2 && ok; ++w) {
          if (j < n_of[w]) {
            if (!wait_p(w, j, v_next, v_par, k_next, k_par, look && w == 1)) { s_abort = 1; atomicExch(p.status, 13); ok = false; break; }
            tc_fence_after();
            issue_pv(w, s, j);
            if (j + 1 == n_of[w]) tc_commit(smem_u32(&o_full[w]));   // this row tile's last P V
          }
          if (j + 1 < n_of[w]) issue_qk(w, j + 1);                   // the next S, queued right behind this P V
        }
        if (!ok) break;
        // the stages go back when the products issued so far have read them
        tc_commit(smem_u32(&v_empty[s]));
        if (j + 1 < n_tiles) tc_commit(smem_u32(&k_empty[s1]));
      }
    }
  } else {
    // ---- softmax and output: two threads per row.  Both read the row's 128 scores for its maximum (so they
    // agree on it without talking), then each takes the exponentials, the sum and the P columns of its own 64
    // keys, and its own half of the columns of O when O is rescaled and when it is written.
    const int idx = (warp - 2) >> 2;                                // 0..3: (row tile, half of the keys)
    const int w = idx >> 1, h = idx & 1;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int row = row0 + w * BM + r;
    const bool row_ok = row < rows_total;
    const int pos = row_ok ? hist + row / p.group : -1;
    const int n_w = w == 0 ? n_tiles_a : (b_on ? n_tiles : 0);
    const int first_tok_w = (row0 + w * BM) / p.group;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + w * BN, o_addr = lane_addr + O_COL + w * 128 + h * (D / 2);
    const int pair_bar = 1 + w * 4 + quarter;                       // named barrier of the two warps on these 32 rows
    float m_run = -INFINITY, l_run = 0.f;                           // reference maximum (scaled, log2 units), running sum of this half
    bool ok = true;
    // A warp that gives up a wait keeps walking the loop for the pair barriers alone, so that the warp it shares
    // its rows with never waits for it in vain.
    for (int j = 0; j < n_w; ++j) {
      if (ok && !__all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[w]), j & 1))) { s_abort = 1; atomicExch(p.status, 15); ok = false; }
      tc_fence_after();
      const int jbase = (tile_begin + j) * BN;
      const bool need_mask = (jbase + BN - 1 > hist + first_tok_w) || p.window > 0 || jbase < lo;
      // this thread's 64 scores; their maximum (raw: the scale is positive), as eight short chains
      float v0[32], v1[32];
      float mx = -INFINITY;
      if (ok) {
        tmem_ld32(s_addr + h * 64, v0);
        tmem_ld32(s_addr + h * 64 + 32, v1);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int ja = jbase + h * 64 + i, jc = ja + 32;
            if (!(ja <= pos && ja >= lo && (p.window <= 0 || ja > pos - p.window))) v0[i] = -INFINITY;
            if (!(jc <= pos && jc >= lo && (p.window <= 0 || jc > pos - p.window))) v1[i] = -INFINITY;
          }
        }
        float mq[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mq[i] = fmaxf(v0[i], v1[i]);
#pragma unroll
        for (int i = 8; i < 32; ++i) mq[i & 7] = fmaxf(mq[i & 7], fmaxf(v0[i], v1[i]));
        mx = fmaxf(fmaxf(fmaxf(mq[0], mq[1]), fmaxf(mq[2], mq[3])), fmaxf(fmaxf(mq[4], mq[5]), fmaxf(mq[6], mq[7])));
      }
      // the row's maximum is the larger of its two halves': through shared memory (two slots in turn, so that a
      // thread a tile ahead does not overwrite what its partner has yet to read)
      s_max[j & 1][w][h][r] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      if (!ok) continue;
      mx = fmaxf(mx, s_max[j & 1][w][1 - h][r]) * p.scale_log2;
      // raise the reference maximum only when it grows by more than 8 (in log2 units)
      const bool raise = mx > m_run + 8.f;
      if (j > 0 && __any_sync(0xffffffffu, raise)) {
        // O_w is quiet: the P V of tile j-1 went through the tensor pipe before the Q K^T that made this S
        const float alpha = raise ? fast_exp2(m_run - mx) : 1.f;     // m_run = -inf gives 0
        l_run *= alpha;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {                           // 16 columns at a time: the scores stay in registers
          uint32_t o[16];
          tmem_ld16(o_addr + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(o_addr + c * 16, o);
        }
      }
      if (raise) m_run = mx;
      const float neg_m = m_run == -INFINITY ? 0.f : -m_run;
      // P = 2^(s * scale - m) rounded to bfloat16, two keys to a column, over the first 32 columns of this
      // thread's half of S
      float sq[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) sq[i] = 0.f;
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = fast_exp2(fmaf(v0[i], p.scale_log2, neg_m));         // masked: 2^-inf = 0
          const float e1 = fast_exp2(fmaf(v0[i + 1], p.scale_log2, neg_m));
          sq[(i >> 1) & 7] += e0 + e1;
          pk[i >> 1] = pack_bf16(e0, e1);
        }
        tmem_st16(s_addr + h * 64, pk);
      }
      {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = fast_exp2(fmaf(v1[i], p.scale_log2, neg_m));
          const float e1 = fast_exp2(fmaf(v1[i + 1], p.scale_log2, neg_m));
          sq[(i >> 1) & 7] += e0 + e1;
          pk[i >> 1] = pack_bf16(e0, e1);
        }
        tmem_st16(s_addr + h * 64 + 16, pk);
      }
      l_run += ((sq[0] + sq[1]) + (sq[2] + sq[3])) + ((sq[4] + sq[5]) + (sq[6] + sq[7]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_full[w]));
    }
    if (ok && n_w > 0) {
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&o_full[w]), 0))) { s_abort = 1; atomicExch(p.status, 16); ok = false; }
      tc_fence_after();
    }
    // the row's sum is the two halves' (the reference maximum is the same in both)
    s_sum[w][h][r] = l_run;
    asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
    const float l_own = n_w > 0 ? s_sum[w][0][r] + s_sum[w][1][r] : 0.f;
    __nv_bfloat16* dst = row_ok ? p.out + (int64_t)(t0 + row / p.group) * p.ldo + (int64_t)(hk * p.group + row % p.group) * D + h * (D / 2)
                                : nullptr;
    if (ks == 1) {
      if (ok && n_w > 0) {
        const float inv = l_own > 0.f ? 1.f / l_own : 0.f;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
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
    } else {
      // ---- the cluster's CTAs hold partial results of the same rows over different keys.  The 256 rows are dealt
      // out in runs of 32 (one warp's): CTA `dest` writes the run out, the others send it their unnormalised O, their
      // reference maximum and their sum through distributed shared memory, into the K/V stages, which are free once
      // every CTA's products have completed (the first cluster barrier).  Layout of what a CTA receives:
      // [sender][4-column group][row of the CTA's runs] float4, so that a warp's stores and loads are contiguous.
      constexpr int C4 = D / 4;
      const int run = w * 4 + quarter;
      const int runs_per = 8 / ks;
      const int dest = run / runs_per;
      const int rows_r = runs_per * 32;
      const int rloc = (run % runs_per) * 32 + lane;
      const bool mine = ok && n_w > 0;                              // O_w of this CTA holds something
      cluster_sync_all();
      if (dest != rank) {
        const int slot = rank < dest ? rank : rank - 1;
        if (mine) {
          const uint32_t remote = map_to_rank(sK, (uint32_t)dest) + (uint32_t)(((slot * C4 + h * (C4 / 2)) * rows_r + rloc) * 16);
#pragma unroll
          for (int c = 0; c < D / 64; ++c) {
            float o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              st_cluster_f32x4(remote + (uint32_t)((c * 8 + q4) * rows_r * 16), o[q4 * 4], o[q4 * 4 + 1], o[q4 * 4 + 2], o[q4 * 4 + 3]);
          }
        }
        if (h == 0) {
          st_cluster_f32(map_to_rank(smem_u32(&x_max[slot * rows_r + rloc]), (uint32_t)dest), mine ? m_run : -INFINITY);
          st_cluster_f32(map_to_rank(smem_u32(&x_sum[slot * rows_r + rloc]), (uint32_t)dest), mine ? l_own : 0.f);
        }
      }
      cluster_sync_all();
      if (dest == rank && ok) {
        float m_all = mine ? m_run : -INFINITY;
        for (int sl = 0; sl < ks - 1; ++sl) m_all = fmaxf(m_all, x_max[sl * rows_r + rloc]);
        const float a_own = (mine && m_run > -INFINITY) ? fast_exp2(m_run - m_all) : 0.f;
        float l_all = l_own * a_own;
        for (int sl = 0; sl < ks - 1; ++sl) {
          const float l_p = x_sum[sl * rows_r + rloc];
          if (l_p > 0.f) l_all += l_p * fast_exp2(x_max[sl * rows_r + rloc] - m_all);
        }
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        const float4* recv = reinterpret_cast<const float4*>(smem_dyn + (sK - smem_u32(smem_dyn)));
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          float o[32];
          if (mine) {                                               // the whole warp or none of it: tcgen05.ld is a warp's instruction
            tmem_ld32(o_addr + c * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = a_own != 0.f ? o[i] * a_own : 0.f;   // a row without a key holds anything
          for (int sl = 0; sl < ks - 1; ++sl) {
            const float l_p = x_sum[sl * rows_r + rloc];
            if (l_p > 0.f) {
              const float a_p = fast_exp2(x_max[sl * rows_r + rloc] - m_all);
#pragma unroll
              for (int q4 = 0; q4 < 8; ++q4) {
                const float4 v = recv[(sl * C4 + h * (C4 / 2) + c * 8 + q4) * rows_r + rloc];
                o[q4 * 4] = fmaf(a_p, v.x, o[q4 * 4]); o[q4 * 4 + 1] = fmaf(a_p, v.y, o[q4 * 4 + 1]);
                o[q4 * 4 + 2] = fmaf(a_p, v.z, o[q4 * 4 + 2]); o[q4 * 4 + 3] = fmaf(a_p, v.w, o[q4 * 4 + 3]);
              }
            }
          }
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
  }
  if (ks > 1 && (warp < 2 || warp == V_WARP)) {             // the other warps pass the cluster's two barriers too
    cluster_sync_all();
    cluster_sync_all();
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
  static_assert((size_t)2 * STAGES * BN * D * 2 >= (size_t)7 * 32 * D * 4, "the K/V stages hold what seven senders bring");
  auto k = attention_umma_kernel<D>;
  constexpr size_t sm = smem_bytes<D>();
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    if (e != cudaSuccess) return refuse((int)e, "attention_umma: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  launch_pdl_cluster(k, grid, dim3(NTHREADS), dim3(p.ksplit, 1, 1), sm, stream, mq, mkv, p);
  return cuda_status("attention_umma");
}

template <int D>
int max_clusters(int key_splits) {
  auto k = attention_umma_kernel<D>;
  constexpr size_t sm = smem_bytes<D>();
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  if (e != cudaSuccess) return -refuse((int)e, "attention_umma: shared memory opt-in failed: %s", cudaGetErrorString(e));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(key_splits * 64, 1, 1); cfg.blockDim = dim3(NTHREADS); cfg.dynamicSmemBytes = sm;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = key_splits; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int n = 0;
  e = cudaOccupancyMaxActiveClusters(&n, k, &cfg);
  if (e != cudaSuccess) return -refuse((int)e, "attention_umma: cluster occupancy query failed: %s", cudaGetErrorString(e));
  return n;
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// How many clusters of key_splits CTAs of this kernel the device runs at a time (negative: an error code).
DINFER_API int dinfer_attention_umma_max_clusters(int D, int key_splits) {
  if ((D != 64 && D != 128) || (key_splits != 1 && key_splits != 2 && key_splits != 4 && key_splits != 8))
    return -refuse(DINFER_BAD_ARGUMENT, "attention_umma: no such kernel (head_dim %d, key_splits %d)", D, key_splits);
  return D == 64 ? max_clusters<64>(key_splits) : max_clusters<128>(key_splits);
}

DINFER_API int dinfer_attention_umma_supports(int D, int group, int block_size) {
  return (D == 64 || D == 128) && group >= 1 && group <= 128 && (128 % group) == 0 && block_size >= 8 &&
         (block_size & (block_size - 1)) == 0;
}

// Prompt portions (q_len > 1) only; requests that bring one token are skipped.
// pair_bound: an upper bound of the batch's row-tile pairs, sum over the portions of ceil(tokens * group / 256)
// (0: B times the longest portion's); CTAs beyond the pairs there are return at once.
// key_splits (1, 2, 4 or 8): that many CTAs of a cluster share the keys of a row-tile pair and fold their results
// through distributed shared memory; for steps with fewer row tiles than the device has SMs.
// q: [T, ...] rows of stride ldq with head h at h*D (all H heads); cache [num_blocks, 2, Hkv, block, D] bf16.
DINFER_API int dinfer_attention_umma(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                     int64_t num_blocks, const int* block_table, int max_blocks,
                                     const int* cu_seqlens, const int* seq_lens, int T, int B, int H, int Hkv, int D,
                                     int block_size, float scale, int window, int max_q_len, int pair_bound,
                                     int key_splits, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv || max_blocks <= 0 || num_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma: bad sizes T=%d B=%d H=%d Hkv=%d", T, B, H, Hkv);
  const int group = H / Hkv;
  if (!(scale > 0.f)) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: the score scale must be positive, got %g", (double)scale);
  if (!dinfer_attention_umma_supports(D, group, block_size))
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma: head_dim %d, group %d, block_size %d not supported "
                  "(head_dim 64 or 128, group dividing 128, power-of-two pages of at least 8)", D, group, block_size);
  if ((ldq % 8) || (ldo % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15) ||
      (reinterpret_cast<uintptr_t>(cache) & 15))
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma: rows and bases must be 16-byte aligned");
  if (!status) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: a status word is required");
  if (key_splits != 1 && key_splits != 2 && key_splits != 4 && key_splits != 8)
    return refuse(DINFER_BAD_ARGUMENT, "attention_umma: key_splits must be 1, 2, 4 or 8, got %d", key_splits);
  if ((int64_t)Hkv * key_splits > 0x7fffffffLL) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: too many heads for the grid");
  const int64_t cache_rows = num_blocks * 2 * Hkv * block_size;
  if (cache_rows > 0x7fffffffLL) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: the cache has too many rows for a tensor map coordinate");
  EncodeTiledFn fn = encode_fn();
  if (!fn) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap mq, mkv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T};
    cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)ldq * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(BM / group)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: tensor map of q failed with %d", (int)r);
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
    if (r != CUDA_SUCCESS) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: tensor map of the cache failed with %d", (int)r);
  }
  Params p;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.block_table = block_table; p.max_blocks = max_blocks;
  p.cu_seqlens = cu_seqlens; p.seq_lens = seq_lens; p.H = H; p.Hkv = Hkv; p.group = group; p.block_size = block_size;
  p.bs_log2 = 0;
  while ((1 << p.bs_log2) < block_size) ++p.bs_log2;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = status;
  p.ksplit = key_splits; p.B = B;
  // pairs of 128-row tiles in the batch: the caller's bound, or every request taken for the longest
  int64_t pairs = pair_bound > 0 ? pair_bound : (int64_t)B * (((int64_t)max_q_len * group + 2 * BM - 1) / (2 * BM));
  if (pairs > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_umma: %lld row-tile pairs are too many for the grid", (long long)pairs);
  dim3 grid(Hkv * key_splits, (unsigned)pairs, 1);
  return D == 64 ? launch<64>(mq, mkv, p, grid, stream) : launch<128>(mq, mkv, p, grid, stream);
}
