// Sampling on f32 logits.  A row is shared by a thread-block cluster of ROW_CTAS CTAs of 1024 threads:
// every CTA keeps its contiguous slice of the row (scaled by 1/temperature) in shared memory, so the
// row is read from memory once, and the CTAs exchange their partial results through each other's
// shared memory (st.shared::cluster + one cluster barrier per exchange).
//
//   dinfer_argmax      greedy, ties to the lowest index
//   dinfer_sample      temperature -> min_p -> top-k -> top-p -> inverse CDF in vocabulary order,
//                      the uniform number from Philox4x32-10 keyed by the request's seed and
//                      counted by the number of tokens the request has produced, so a request's
//                      tokens do not depend on its place in the batch; rows whose temperature is
//                      <= 1e-5 are greedy
//   dinfer_penalties   repetition / frequency / presence penalties from the token history
//   dinfer_logit_bias  per-request additive biases on given tokens
//   dinfer_logprobs    log-probability and rank of the chosen token and the k most likely tokens
//
// Same contract as the reference (crates/kernels/cuda/sampling.cu:13-56,60-133,143-157,196-283,
// 322-349; order of operations models/qwen3/src/executor.rs:552-605).  Unlike it the logits are not
// rewritten: the three filters reduce to one keep-threshold on the scaled logits.  The top-k and the
// top-p threshold are each found by a radix-16 descent over the order-preserving 32-bit image of a
// float (eight rounds, every round one pass over shared memory): the largest value t such that the
// kept entries >= t number at least k (have at least the share p of the mass).  A small k (up to 512)
// takes a short way instead: a histogram names the bin of the k-th largest entry, the entries from
// there up are collected in every CTA, and both thresholds are counted out among them.  All sums are
// taken in a fixed order (thread, warp, CTA rank), so the same logits, seed and count give the same token.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int BLOCK = 1024;
constexpr int ROW_CTAS = 8;                 // cluster size: CTAs that share a row
constexpr int MAX_SLICE = 48 * 1024;        // floats of a row slice that shared memory holds (192 KB)
constexpr int XCH = 16;                     // floats a CTA hands to the others per exchange
constexpr int ARGMAX_MANY_ROWS = 40;        // from so many rows on the argmax runs a CTA per row

// ---- cluster plumbing
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t local_addr, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// What the CTAs of a row share: two exchange buffers used alternately (a CTA may write the next
// exchange while a slower one still reads the last) and the block-level scratch.
struct Shared {
  float xchg[2][ROW_CTAS][XCH];
  float warp_part[32][XCH];
  float blk[XCH];
  float warp_tot[32];
  int pick[4];
  int turn;
};

// Every CTA contributes n <= XCH floats (valid in threads 0..n-1 as `mine`); afterwards
// sh.xchg[turn][r][j] holds the contribution j of CTA r, the same in every CTA.  Returns the buffer.
__device__ float (*exchange(Shared& sh, float mine, int n, uint32_t rank))[XCH] {
  const int t = sh.turn;
  if ((int)threadIdx.x < n) {
#pragma unroll
    for (uint32_t r = 0; r < ROW_CTAS; ++r) st_cluster_f32(smem_u32(&sh.xchg[t][rank][threadIdx.x]), r, mine);
  }
  cluster_sync_all();
  __syncthreads();
  if (threadIdx.x == 0) sh.turn = t ^ 1;
  __syncthreads();
  return sh.xchg[t];
}

// Deterministic block sum of a per-thread vector v[0..N): warp shuffle tree, then the warps in order.
// The result is in sh.blk[0..N) for all threads.
template <int N>
__device__ void block_sum_vec(Shared& sh, float (&v)[N]) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < N; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[j] += __shfl_xor_sync(0xffffffffu, v[j], o);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int j = 0; j < N; ++j) sh.warp_part[warp][j] = v[j];
  }
  __syncthreads();
  if ((int)threadIdx.x < N) {
    float s = 0.f;
    for (int w = 0; w < BLOCK / 32; ++w) s += sh.warp_part[w][threadIdx.x];
    sh.blk[threadIdx.x] = s;
  }
  __syncthreads();
}

// Sum over the whole row of a per-thread vector: block sum, exchange, CTAs in rank order.
template <int N>
__device__ void row_sum_vec(Shared& sh, float (&v)[N], uint32_t rank, float (&out)[N]) {
  block_sum_vec<N>(sh, v);
  const float mine = (int)threadIdx.x < N ? sh.blk[threadIdx.x] : 0.f;
  float (*x)[XCH] = exchange(sh, mine, N, rank);
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float s = 0.f;
#pragma unroll
    for (int r = 0; r < ROW_CTAS; ++r) s += x[r][j];
    out[j] = s;
  }
}

// order-preserving image of a float: a < b  <=>  key(a) < key(b)   (-0 is folded into +0 by the caller)
__device__ __forceinline__ uint32_t float_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// argmax over the row (ties to the lowest index), the same in every CTA of the cluster
__device__ int row_argmax(Shared& sh, const float* xs, int n_mine, int first, uint32_t rank) {
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < n_mine; i += BLOCK) best = better(best, ArgMax{xs[i], first + i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sh.warp_part[warp][0] = best.v; sh.warp_part[warp][1] = __int_as_float(best.i); }
  __syncthreads();
  if (warp == 0) {
    best = ArgMax{sh.warp_part[lane][0], __float_as_int(sh.warp_part[lane][1])};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    if (lane == 0) { sh.blk[0] = best.v; sh.blk[1] = __int_as_float(best.i); }
  }
  __syncthreads();
  const float mine = threadIdx.x < 2 ? sh.blk[threadIdx.x] : 0.f;
  float (*x)[XCH] = exchange(sh, mine, 2, rank);
  ArgMax all{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r) all = better(all, ArgMax{x[r][0], __float_as_int(x[r][1])});
  return all.i == 0x7fffffff ? 0 : all.i;
}

__device__ __forceinline__ uint32_t mulhilo(uint32_t a, uint32_t b, uint32_t* hi) {
  const uint64_t p = (uint64_t)a * b;
  *hi = (uint32_t)(p >> 32);
  return (uint32_t)p;
}

// counter (offset_lo, offset_hi, 0, 0), key (seed_lo, seed_hi), ten rounds, u = (c0 >> 8) / 2^24
__device__ float philox_uniform(uint64_t seed, uint64_t offset) {
  uint32_t c0 = (uint32_t)offset, c1 = (uint32_t)(offset >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, hi1;
    const uint32_t lo0 = mulhilo(0xD2511F53u, c0, &hi0);
    const uint32_t lo1 = mulhilo(0xCD9E8D57u, c2, &hi1);
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (float)(c0 >> 8) * (1.f / 16777216.f);
}

// The slice of the row this CTA owns: ids [first, first + n_mine).  Thread t owns the contiguous
// ids [t*seg, (t+1)*seg) of the slice, so thread order, then CTA rank, is vocabulary order.
struct Slice {
  const float* xs;      // scaled values in shared memory, or null: read the row and scale on the fly
  const float* row;
  float inv_t;
  int first, n_mine, seg;
  __device__ __forceinline__ float at(int i) const { return xs ? xs[i] : row[first + i] * inv_t + 0.f; }
};

// The largest value t such that the entries x >= max(t, floor_) weigh at least `target`, where an
// entry weighs 1 (MASS = false) or exp(x - m) (MASS = true).  Radix-16 descent over float_key:
// `above` is the weight of the entries beyond the digits fixed so far.
template <bool MASS>
__device__ float radix_threshold(Shared& sh, const Slice& sl, uint32_t rank, float m, float floor_, float target) {
  uint32_t prefix = 0;
  float above = 0.f;
  const int i0 = min(sl.n_mine, (int)threadIdx.x * sl.seg), i1 = min(sl.n_mine, i0 + sl.seg);
#pragma unroll 1
  for (int shift = 28; shift >= 0; shift -= 4) {
    float h[16];
#pragma unroll
    for (int d = 0; d < 16; ++d) h[d] = 0.f;
    for (int i = i0; i < i1; ++i) {
      const float x = sl.at(i);
      if (!(x >= floor_)) continue;
      const uint32_t k = float_key(x);
      if (shift < 28 && (k >> (shift + 4)) != (prefix >> (shift + 4))) continue;
      const float w = MASS ? expf(x - m) : 1.f;
      const int dgt = (k >> shift) & 15;
#pragma unroll
      for (int d = 0; d < 16; ++d) h[d] += dgt == d ? w : 0.f;
    }
    float tot[16];
    row_sum_vec<16>(sh, h, rank, tot);
    int chosen = 0;
    float run = above;
    bool found = false;
#pragma unroll
    for (int d = 15; d >= 0; --d) {
      if (!found) {
        if (run + tot[d] >= target) { chosen = d; found = true; }
        else run += tot[d];
      }
    }
    if (!found) { chosen = 0; run -= tot[0]; }          // less than the target in all: keep everything
    above = run;
    prefix |= (uint32_t)chosen << shift;
  }
  return key_float(prefix);
}

// ---- the short way to a top-k threshold (and the top-p threshold behind it) when k is small
// One pass counts the kept entries by the upper 12 bits of their key (a histogram in shared memory; the CTAs
// read each other's counts), which names the bin that holds the k-th largest entry; the entries from that bin
// up, at most CAND_MAX of them, are copied into every CTA in vocabulary order, and the thresholds are found
// among them by direct counting.  With more entries than that from the bin up, the radix descent does it.
constexpr int CAND_MAX = 1024;
constexpr int HIST_BITS = 12, HIST_BINS = 1 << HIST_BITS, BINS_PER_CTA = HIST_BINS / ROW_CTAS;
static_assert(BINS_PER_CTA <= BLOCK, "a thread per bin of a CTA's share");

struct Candidates {
  uint32_t hist[HIST_BINS];
  float x[CAND_MAX];                  // the candidates, the same list in every CTA of the row
  float w[CAND_MAX];                  // their weights exp(x - m), 0 below the floor
  int warp_tot[BLOCK / 32];
  int n;
  float thr;
};

__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}

// inclusive prefix sum of v over the threads of the block, in thread order; `total` is the block's sum
__device__ int block_scan_inclusive(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += u;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < BLOCK / 32; ++w) {
    const int t = warp_tot[w];
    if (w < warp) before += t;
    all += t;
  }
  total = all;
  return incl + before;
}

// Fills c.x with the kept entries (x >= floor_) from the bin of the k-th largest up; returns their number, or -1
// if they are more than CAND_MAX.  With fewer than k kept entries all of them are candidates.
__device__ int gather_candidates(Shared& sh, Candidates& c, const Slice& sl, uint32_t rank, float floor_, int k) {
  const int i0 = min(sl.n_mine, (int)threadIdx.x * sl.seg), i1 = min(sl.n_mine, i0 + sl.seg);
  for (int i = threadIdx.x; i < HIST_BINS; i += BLOCK) c.hist[i] = 0u;
  __syncthreads();
  for (int i = i0; i < i1; ++i) {
    const float x = sl.at(i);
    if (x >= floor_) atomicAdd(&c.hist[float_key(x) >> (32 - HIST_BITS)], 1u);
  }
  __syncthreads();
  cluster_sync_all();
  // this CTA adds up the bins [rank * BINS_PER_CTA, +BINS_PER_CTA) over all CTAs; thread u takes them from the top
  int v = 0;
  const int bin = (int)rank * BINS_PER_CTA + (BINS_PER_CTA - 1 - (int)threadIdx.x);
  if ((int)threadIdx.x < BINS_PER_CTA) {
#pragma unroll
    for (uint32_t r = 0; r < ROW_CTAS; ++r) v += (int)ld_cluster_u32(smem_u32(&c.hist[bin]), r);
  }
  int mine_total;
  const int incl = block_scan_inclusive(v, c.warp_tot, mine_total);     // entries of my bins from `bin` up
  float (*x)[XCH] = exchange(sh, threadIdx.x == 0 ? (float)mine_total : 0.f, 1, rank);
  int above = 0, kept = 0;
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r) {
    const int t = (int)x[r][0];
    kept += t;
    if (r > (int)rank) above += t;
  }
  // the bin where the count from the top reaches k: at most one thread of the row finds it
  if (threadIdx.x < 2) sh.blk[threadIdx.x] = -1.f;
  __syncthreads();
  if ((int)threadIdx.x < BINS_PER_CTA && v > 0 && above + incl - v < k && above + incl >= k) {
    sh.blk[0] = (float)bin;
    sh.blk[1] = (float)(above + incl);
  }
  __syncthreads();
  x = exchange(sh, threadIdx.x < 2 ? sh.blk[threadIdx.x] : 0.f, 2, rank);
  int pivot_bin = 0, n = kept;                           // fewer than k kept: all of them
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r)
    if (x[r][0] >= 0.f) { pivot_bin = (int)x[r][0]; n = (int)x[r][1]; }
  if (n > CAND_MAX) return -1;
  // copy them into every CTA, in vocabulary order
  int cnt = 0;
  for (int i = i0; i < i1; ++i) {
    const float xv = sl.at(i);
    cnt += xv >= floor_ && (int)(float_key(xv) >> (32 - HIST_BITS)) >= pivot_bin;
  }
  int cta_total;
  const int my_end = block_scan_inclusive(cnt, c.warp_tot, cta_total);
  x = exchange(sh, threadIdx.x == 0 ? (float)cta_total : 0.f, 1, rank);
  int base = 0;
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r)
    if (r < (int)rank) base += (int)x[r][0];
  int at = base + my_end - cnt;
  for (int i = i0; i < i1 && cnt > 0; ++i) {
    const float xv = sl.at(i);
    if (xv >= floor_ && (int)(float_key(xv) >> (32 - HIST_BITS)) >= pivot_bin) {
      const uint32_t dst = smem_u32(&c.x[at]);
#pragma unroll
      for (uint32_t r = 0; r < ROW_CTAS; ++r) st_cluster_f32(dst, r, xv);
      ++at;
    }
  }
  cluster_sync_all();
  __syncthreads();
  return n;
}

// the k-th largest of the n candidates (all kept if they are fewer than k)
__device__ float topk_of_candidates(Candidates& c, int n, int k) {
  if (threadIdx.x == 0) c.thr = -INFINITY;
  __syncthreads();
  if (k <= n && (int)threadIdx.x < n) {
    const float v = c.x[threadIdx.x];
    int before = 0;                                      // candidates that come before this one, larger first
    for (int j = 0; j < n; ++j) {
      const float xj = c.x[j];
      before += xj > v || (xj == v && j < (int)threadIdx.x);
    }
    if (before == k - 1) c.thr = v;
  }
  __syncthreads();
  return c.thr;
}

// the largest candidate value v >= floor_ such that the candidates >= v hold at least the share p of the mass of
// those >= floor_; every thread adds the masses in the same order
__device__ float topp_of_candidates(Candidates& c, int n, float m, float floor_, float p) {
  for (int j = threadIdx.x; j < n; j += BLOCK) c.w[j] = c.x[j] >= floor_ ? expf(c.x[j] - m) : 0.f;
  __syncthreads();
  float best = -INFINITY;
  if ((int)threadIdx.x < n) {
    const float v = c.x[threadIdx.x];
    float denom = 0.f, mass = 0.f;
    for (int j = 0; j < n; ++j) {
      const float wj = c.w[j];
      denom += wj;
      if (c.x[j] >= v) mass += wj;
    }
    if (v >= floor_ && mass >= p * denom) best = v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) c.w[threadIdx.x >> 5] = best;            // the weights are done with
  __syncthreads();
  float all = -INFINITY;
#pragma unroll
  for (int w = 0; w < BLOCK / 32; ++w) all = fmaxf(all, c.w[w]);
  __syncthreads();
  return all;
}

__global__ void __launch_bounds__(BLOCK)
argmax_kernel(const float* __restrict__ logits, int64_t ld, int* __restrict__ out, int vocab) {
  extern __shared__ __align__(16) float xs_dyn[];
  __shared__ Shared sh;
  pdl_enter();
  const uint32_t rank = cluster_ctarank();
  const int b = blockIdx.x / ROW_CTAS;
  const float* row = logits + (int64_t)b * ld;
  const int per = (vocab + ROW_CTAS - 1) / ROW_CTAS;
  const int first = min(vocab, (int)rank * per), n_mine = min(vocab, first + per) - first;
  if (threadIdx.x == 0) sh.turn = 0;
  __syncthreads();
  cluster_sync_all();                                    // every CTA runs before any writes into its memory
  const int r = row_argmax(sh, row + first, n_mine, first, rank);
  if (rank == 0 && threadIdx.x == 0) out[b] = r;
  cluster_sync_all();                                    // nobody leaves while others may still write to it
}

// Many rows: a CTA per row (no cluster: with 8 CTAs a row, 64 rows are two waves of CTAs that mostly wait for each
// other), four floats a load where the row allows.
__global__ void __launch_bounds__(BLOCK)
argmax_many_kernel(const float* __restrict__ logits, int64_t ld, int* __restrict__ out, int vocab) {
  __shared__ float part_v[BLOCK / 32];
  __shared__ int part_i[BLOCK / 32];
  pdl_enter();
  const int b = blockIdx.x;
  const float* row = logits + (int64_t)b * ld;
  ArgMax best{-INFINITY, 0x7fffffff};
  if (!(reinterpret_cast<uintptr_t>(row) & 15)) {
    const int n4 = vocab >> 2;
    const float4* row4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < n4; i += BLOCK) {
      const float4 v = row4[i];
      best = better(best, ArgMax{v.x, 4 * i});
      best = better(best, ArgMax{v.y, 4 * i + 1});
      best = better(best, ArgMax{v.z, 4 * i + 2});
      best = better(best, ArgMax{v.w, 4 * i + 3});
    }
    for (int i = 4 * n4 + threadIdx.x; i < vocab; i += BLOCK) best = better(best, ArgMax{row[i], i});
  } else {
    for (int i = threadIdx.x; i < vocab; i += BLOCK) best = better(best, ArgMax{row[i], i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { part_v[warp] = best.v; part_i[warp] = best.i; }
  __syncthreads();
  if (warp == 0) {
    best = ArgMax{part_v[lane], part_i[lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    if (lane == 0) out[b] = best.i == 0x7fffffff ? 0 : best.i;
  }
}

__global__ void __launch_bounds__(BLOCK)
sample_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ offsets,
              int* __restrict__ out, int vocab, int cache_slice) {
  extern __shared__ __align__(16) float xs_dyn[];
  __shared__ Shared sh;
  __shared__ Candidates cand;
  pdl_enter();
  const uint32_t rank = cluster_ctarank();
  const int b = blockIdx.x / ROW_CTAS;
  const float* row = logits + (int64_t)b * ld;
  const int per = (vocab + ROW_CTAS - 1) / ROW_CTAS;
  const int first = min(vocab, (int)rank * per), n_mine = min(vocab, first + per) - first;
  if (threadIdx.x == 0) sh.turn = 0;
  __syncthreads();
  cluster_sync_all();                                    // every CTA runs before any writes into its memory
  const float temp = temperature[b];
  if (temp <= 1e-5f) {
    const int r = row_argmax(sh, row + first, n_mine, first, rank);
    if (rank == 0 && threadIdx.x == 0) out[b] = r;
    cluster_sync_all();
    return;
  }
  const float inv_t = 1.f / temp;
  Slice sl;
  sl.row = row; sl.inv_t = inv_t; sl.first = first; sl.n_mine = n_mine;
  sl.seg = (per + BLOCK - 1) / BLOCK;
  sl.xs = cache_slice ? xs_dyn : nullptr;

  // one pass over the row: scaled values into shared memory, maximum and smallest finite value
  float m = -INFINITY, lo = INFINITY;
  for (int i = threadIdx.x; i < n_mine; i += BLOCK) {
    const float x = row[first + i] * inv_t + 0.f;        // + 0: -0 becomes +0 (one image per value)
    if (cache_slice) xs_dyn[i] = x;
    m = fmaxf(m, x);
    if (x > -INFINITY) lo = fminf(lo, x);
  }
  {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sh.warp_part[warp][0] = m; sh.warp_part[warp][1] = lo; }
    __syncthreads();
    if (threadIdx.x < 2) {
      float v = sh.warp_part[0][threadIdx.x];
      for (int w = 1; w < BLOCK / 32; ++w) v = threadIdx.x == 0 ? fmaxf(v, sh.warp_part[w][0]) : fminf(v, sh.warp_part[w][1]);
      sh.blk[threadIdx.x] = v;
    }
    __syncthreads();
    const float mine = threadIdx.x < 2 ? sh.blk[threadIdx.x] : 0.f;
    float (*x)[XCH] = exchange(sh, mine, 2, rank);
    m = -INFINITY; lo = INFINITY;
#pragma unroll
    for (int r = 0; r < ROW_CTAS; ++r) { m = fmaxf(m, x[r][0]); lo = fminf(lo, x[r][1]); }
  }

  // keep-threshold on x: min_p, then top-k, then top-p on what top-k and min_p left
  float thr = -INFINITY;
  const float mp = min_p ? min_p[b] : 0.f;
  if (mp > 0.f) thr = m + logf(mp);                      // p_i >= min_p * p_max
  const int k = top_k ? top_k[b] : -1;
  int n_cand = -1;                                       // >= 0: cand holds every entry from the top-k threshold up
  if (k > 0 && k < vocab) {
    if (k <= CAND_MAX / 2) n_cand = gather_candidates(sh, cand, sl, rank, thr, k);
    if (n_cand >= 0) thr = fmaxf(thr, topk_of_candidates(cand, n_cand, k));
    else thr = fmaxf(thr, radix_threshold<false>(sh, sl, rank, m, thr, (float)k));
  }
  const float p = top_p ? top_p[b] : 1.f;
  const int i0 = min(n_mine, (int)threadIdx.x * sl.seg), i1 = min(n_mine, i0 + sl.seg);
  if (p < 1.f && p > 0.f && n_cand >= 0) {
    thr = fmaxf(thr, topp_of_candidates(cand, n_cand, m, thr, p));
  } else if (p < 1.f && p > 0.f) {
    float d1[1] = {0.f}, denom[1];
    for (int i = i0; i < i1; ++i) {
      const float x = sl.at(i);
      if (x >= thr) d1[0] += expf(x - m);
    }
    row_sum_vec<1>(sh, d1, rank, denom);
    thr = fmaxf(thr, radix_threshold<true>(sh, sl, rank, m, thr, p * denom[0]));
  }

  // inverse CDF in vocabulary order: threads in order within a CTA, CTAs in rank order
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = sl.at(i);
    if (x >= thr) mine += expf(x - m);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float incl = mine;                                     // inclusive scan over the lanes of the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) sh.warp_tot[warp] = incl;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < BLOCK / 32; ++w) s += sh.warp_tot[w];
    sh.blk[0] = s;
  }
  __syncthreads();
  float (*x)[XCH] = exchange(sh, threadIdx.x == 0 ? sh.blk[0] : 0.f, 1, rank);
  float total = 0.f;
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r) total += x[r][0];
  const float target = philox_uniform(seeds[b], offsets[b]) * total;
  // the CTA whose share of the cumulative mass reaches the target; beyond the total by rounding: the
  // last CTA that keeps anything, at the end of its share
  int owner = -1, last_nonzero = -1;
  float before = 0.f, before_last = 0.f, run = 0.f;
#pragma unroll
  for (int r = 0; r < ROW_CTAS; ++r) {
    const float t = x[r][0];
    if (t > 0.f) { last_nonzero = r; before_last = run; }
    if (owner < 0 && t > 0.f && run + t >= target) { owner = r; before = run; }
    run += t;
  }
  bool clamp = false;
  if (owner < 0) { owner = last_nonzero; before = before_last; clamp = true; }
  if (owner == (int)rank) {
    // within this CTA: the warp, then the lane, then the entry
    if (threadIdx.x == 0) {
      float cum = before;
      int w_own = -1;
      float w_before = before;
      int w_last = -1;
      float w_before_last = before;
      for (int w = 0; w < BLOCK / 32; ++w) {
        const float t = sh.warp_tot[w];
        if (t > 0.f) { w_last = w; w_before_last = cum; }
        if (w_own < 0 && !clamp && t > 0.f && cum + t >= target) { w_own = w; w_before = cum; }
        cum += t;
      }
      if (w_own < 0) { w_own = w_last; w_before = w_before_last; sh.pick[2] = 1; } else sh.pick[2] = 0;
      sh.pick[0] = w_own;
      sh.blk[1] = w_before;
    }
    __syncthreads();
    if (warp == sh.pick[0]) {
      const bool clamp_w = sh.pick[2] != 0;
      const float base = sh.blk[1];
      const float excl = incl - mine;                    // mass of the lanes before this one
      // the first lane whose inclusive sum reaches the target (or the last lane that keeps anything)
      const bool hit = !clamp_w && mine > 0.f && base + incl >= target;
      const unsigned hits = __ballot_sync(0xffffffffu, hit);
      const unsigned keeps = __ballot_sync(0xffffffffu, mine > 0.f);
      int l_own;
      bool clamp_l = false;
      if (hits) l_own = __ffs(hits) - 1;
      else { l_own = 31 - __clz(keeps); clamp_l = true; }
      if (lane == l_own) {
        float cum = base + excl;
        int last = -1;
        for (int i = i0; i < i1; ++i) {
          const float xv = sl.at(i);
          if (xv >= thr) {
            cum += expf(xv - m);
            last = i;
            if (!clamp_l && cum >= target) break;
          }
        }
        out[b] = first + (last < 0 ? 0 : last);
      }
    }
  }
  if (owner < 0 && rank == 0 && threadIdx.x == 0) out[b] = 0;   // nothing kept at all (no finite logit)
  cluster_sync_all();                                    // nobody leaves while others may still write to it
}

// history of row b: ids[offsets[b] .. offsets[b+1]), the first prompt_len[b] of them the prompt.
__global__ void penalties_kernel(float* __restrict__ logits, int64_t ld, const int* __restrict__ ids,
                                 const int* __restrict__ offsets, const int* __restrict__ prompt_len,
                                 const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres, int vocab) {
  const int b = blockIdx.x;
  const float r = rep[b], f = freq[b], pr = pres[b];
  if (r == 1.f && f == 0.f && pr == 0.f) return;
  float* row = logits + (int64_t)b * ld;
  const int lo = offsets[b], hi = offsets[b + 1], np = prompt_len[b];
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const int t = ids[i];
    if (t < 0 || t >= vocab) continue;
    bool first = true;                       // each distinct token is handled by its first occurrence
    for (int j = lo; j < i; ++j) if (ids[j] == t) { first = false; break; }
    if (!first) continue;
    int cnt = 0;
    for (int j = lo + np; j < hi; ++j) cnt += ids[j] == t;
    float v = row[t];
    if (r != 1.f) v = v > 0.f ? v / r : v * r;
    if (cnt > 0) v -= f * (float)cnt + pr;
    row[t] = v;
  }
}

// logits[rows[i], ids[i]] += bias[i]; a (row, id) pair appears once.
__global__ void logit_bias_kernel(float* __restrict__ logits, int64_t ld, const int* __restrict__ rows,
                                  const int* __restrict__ ids, const float* __restrict__ bias, int n, int vocab) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int t = ids[i];
  if (t >= 0 && t < vocab) logits[(int64_t)rows[i] * ld + t] += bias[i];
}

// Log-probabilities of a row under log_softmax of the logits as given (no temperature, no filter): the chosen
// token's, how many tokens are strictly more likely (its rank), and the k most likely in descending order, ties
// to the lower id.  One CTA per row.  The k best are found one after the other, each as the best entry that comes
// after the last one in that order, so nothing has to be remembered but the last winner.
constexpr int LP_MAX_K = 32;
__global__ void logprobs_kernel(const float* __restrict__ logits, int64_t ld, const int* __restrict__ chosen, int k,
                                int* __restrict__ out_ids, float* __restrict__ out_lp, int* __restrict__ out_rank,
                                int vocab) {
  __shared__ float s_f[BLOCK / 32];
  __shared__ int s_i[BLOCK / 32];
  __shared__ float s_m, s_lse, s_last_v;
  __shared__ int s_last_i;
  const int b = blockIdx.x;
  const float* row = logits + (int64_t)b * ld;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // maximum
  float m = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += BLOCK) m = fmaxf(m, row[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) s_f[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = s_f[0];
    for (int w = 1; w < BLOCK / 32; ++w) v = fmaxf(v, s_f[w]);
    s_m = v;
  }
  __syncthreads();
  m = s_m;
  // log of the sum of exponentials, and the rank of the chosen token (sums in a fixed order)
  const int c = chosen[b];
  const bool c_ok = c >= 0 && c < vocab;
  const float xc = c_ok ? row[c] : -INFINITY;
  float d = 0.f;
  int gt = 0;
  for (int i = threadIdx.x; i < vocab; i += BLOCK) {
    const float v = row[i];
    if (v > -INFINITY) d += expf(v - m);
    gt += v > xc;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    d += __shfl_xor_sync(0xffffffffu, d, o);
    gt += __shfl_xor_sync(0xffffffffu, gt, o);
  }
  if (lane == 0) { s_f[warp] = d; s_i[warp] = gt; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.f;
    int cnt = 0;
    for (int w = 0; w < BLOCK / 32; ++w) { sum += s_f[w]; cnt += s_i[w]; }
    s_lse = m + logf(sum);
    out_ids[(int64_t)b * (k + 1)] = c;
    out_lp[(int64_t)b * (k + 1)] = xc - s_lse;
    out_rank[b] = cnt;
    s_last_v = INFINITY;                  // before the first entry of the order
    s_last_i = -1;
  }
  __syncthreads();
  for (int j = 0; j < k; ++j) {
    const float last_v = s_last_v;
    const int last_i = s_last_i;
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < vocab; i += BLOCK) {
      const float v = row[i];
      if (v < last_v || (v == last_v && i > last_i)) best = better(best, ArgMax{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    __syncthreads();                      // the last round's readers of s_f / s_i are done
    if (lane == 0) { s_f[warp] = best.v; s_i[warp] = best.i; }
    __syncthreads();
    if (threadIdx.x == 0) {
      ArgMax a{s_f[0], s_i[0]};
      for (int w = 1; w < BLOCK / 32; ++w) a = better(a, ArgMax{s_f[w], s_i[w]});
      const bool any = a.i != 0x7fffffff;  // fewer than k entries in the row: the rest is marked -1
      out_ids[(int64_t)b * (k + 1) + 1 + j] = any ? a.i : -1;
      out_lp[(int64_t)b * (k + 1) + 1 + j] = any ? a.v - s_lse : -INFINITY;
      s_last_v = any ? a.v : -INFINITY;
      s_last_i = any ? a.i : 0x7fffffff;
    }
    __syncthreads();
  }
}

template <typename... KArgs, typename... Args>
int launch_rows(void (*kernel)(KArgs...), int rows, size_t smem, cudaStream_t stream, const char* what, Args... args) {
  cudaError_t e = launch_pdl_cluster(kernel, dim3(rows * ROW_CTAS), dim3(BLOCK), dim3(ROW_CTAS, 1, 1), smem, stream, args...);
  if (e != cudaSuccess) return refuse((int)e, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return cuda_status(what);
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

DINFER_API int dinfer_argmax(const float* logits, int64_t ld, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  if (rows >= ARGMAX_MANY_ROWS) {
    cudaError_t e = launch_pdl(argmax_many_kernel, dim3(rows), dim3(BLOCK), 0, stream, logits, ld, out, vocab);
    if (e != cudaSuccess) return refuse((int)e, "argmax: launch failed: %s", cudaGetErrorString(e));
    return cuda_status("argmax");
  }
  return launch_rows(argmax_kernel, rows, 0, stream, "argmax", logits, ld, out, vocab);
}

// temperature [rows]; top_k (<=0: off), top_p, min_p may be null; seeds, offsets [rows] uint64.
DINFER_API int dinfer_sample(const float* logits, int64_t ld, const float* temperature, const int* top_k,
                             const float* top_p, const float* min_p, const uint64_t* seeds,
                             const uint64_t* offsets, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  // a row slice that fits shared memory is kept there (read once); a longer one is read again every pass
  const int per = (vocab + ROW_CTAS - 1) / ROW_CTAS;
  const int cache_slice = per <= MAX_SLICE ? 1 : 0;
  const size_t smem = cache_slice ? (size_t)per * sizeof(float) : 0;
  static bool opted = false;
  if (!opted) {
    cudaError_t e = cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MAX_SLICE * (int)sizeof(float));
    if (e != cudaSuccess) return refuse((int)e, "sample: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted = true;
  }
  return launch_rows(sample_kernel, rows, smem, stream, "sample", logits, ld, temperature, top_k, top_p, min_p, seeds,
                     offsets, out, vocab, cache_slice);
}

DINFER_API int dinfer_penalties(float* logits, int64_t ld, const int* ids, const int* offsets,
                                const int* prompt_len, const float* rep, const float* freq, const float* pres,
                                int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "penalties: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  penalties_kernel<<<rows, 256, 0, stream>>>(logits, ld, ids, offsets, prompt_len, rep, freq, pres, vocab);
  return cuda_status("penalties");
}

// rows, ids, bias [n]: logits[rows[i], ids[i]] += bias[i] (the reference adds its logit_bias before the penalties:
// crates/core/src/sample.rs:104-106).
DINFER_API int dinfer_logit_bias(float* logits, int64_t ld, const int* rows, const int* ids, const float* bias, int n,
                                 int vocab, cudaStream_t stream) {
  if (n < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "logit_bias: bad sizes n=%d vocab=%d", n, vocab);
  if (n == 0) return 0;
  logit_bias_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, ld, rows, ids, bias, n, vocab);
  return cuda_status("logit_bias");
}

// chosen [rows]; out_ids, out_lp [rows, k + 1]: column 0 the chosen token, then the k most likely, descending;
// out_rank [rows]: tokens strictly more likely than the chosen one (crates/kernels/cuda/sampling.cu:381-430).
DINFER_API int dinfer_logprobs(const float* logits, int64_t ld, const int* chosen, int k, int* out_ids, float* out_lp,
                               int* out_rank, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "logprobs: bad sizes rows=%d vocab=%d", rows, vocab);
  if (k < 0 || k > LP_MAX_K) return refuse(DINFER_BAD_ARGUMENT, "logprobs: k must be in [0, %d], got %d", LP_MAX_K, k);
  if (rows == 0) return 0;
  logprobs_kernel<<<rows, BLOCK, 0, stream>>>(logits, ld, chosen, k, out_ids, out_lp, out_rank, vocab);
  return cuda_status("logprobs");
}
