// Sampling on f32 logits, one 1024-thread block per row.
//
//   dinfer_argmax      greedy, ties to the lowest index
//   dinfer_sample      temperature -> min_p -> top-k -> top-p -> inverse CDF in vocabulary order,
//                      the uniform number from Philox4x32-10 keyed by the request's seed and
//                      counted by the number of tokens the request has produced, so a request's
//                      tokens do not depend on its place in the batch; rows whose temperature is
//                      <= 1e-5 are greedy
//   dinfer_penalties   repetition / frequency / presence penalties from the token history
//
// Same contract as the reference (crates/kernels/cuda/sampling.cu:13-56,60-133,143-157,196-283,
// 322-349; order of operations models/qwen3/src/executor.rs:552-605).  Unlike it the logits are not
// rewritten: the three filters reduce to one keep-threshold on the scaled logits.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int BLOCK = 1024;

struct ArgMax { float v; int i; };

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ int block_argmax(const float* row, int vocab, float* sv, int* si) {
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += BLOCK) best = better(best, ArgMax{row[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
  __syncthreads();
  if (warp == 0) {
    best = ArgMax{sv[lane], si[lane]};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      best = better(best, ArgMax{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)});
    if (lane == 0) si[0] = best.i == 0x7fffffff ? 0 : best.i;
  }
  __syncthreads();
  return si[0];
}

__global__ void __launch_bounds__(BLOCK) argmax_kernel(const float* __restrict__ logits, int64_t ld,
                                                       int* __restrict__ out, int vocab) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_enter();
  const int r = block_argmax(logits + (int64_t)blockIdx.x * ld, vocab, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = r;
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

// Count and softmax mass of the scaled logits x = v * inv_t with x >= t (and x >= floor).
__device__ void count_mass(const float* row, int vocab, float inv_t, float m, float t, float floor_,
                           float* red, float* count, float* mass) {
  float c = 0.f, s = 0.f;
  for (int i = threadIdx.x; i < vocab; i += BLOCK) {
    const float x = row[i] * inv_t;
    if (x >= t && x >= floor_) { c += 1.f; s += expf(x - m); }
  }
  *count = block_sum(c, red);
  *mass = block_sum(s, red);
}

__global__ void __launch_bounds__(BLOCK)
sample_kernel(const float* __restrict__ logits, int64_t ld, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ offsets,
              int* __restrict__ out, int vocab) {
  __shared__ float red[33];
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float seg_sum[BLOCK];
  __shared__ int choice;
  pdl_enter();
  const int b = blockIdx.x;
  const float* row = logits + (int64_t)b * ld;
  const float temp = temperature[b];
  if (temp <= 1e-5f) {
    const int r = block_argmax(row, vocab, sv, si);
    if (threadIdx.x == 0) out[b] = r;
    return;
  }
  const float inv_t = 1.f / temp;
  float m = -INFINITY, lo = INFINITY;
  for (int i = threadIdx.x; i < vocab; i += BLOCK) {
    const float x = row[i] * inv_t;
    m = fmaxf(m, x);
    if (x > -INFINITY) lo = fminf(lo, x);
  }
  m = block_max(m, red);
  lo = -block_max(-lo, red);

  // keep-threshold on x: min_p, then top-k, then top-p on what top-k and min_p left
  float thr = -INFINITY;
  const float mp = min_p ? min_p[b] : 0.f;
  if (mp > 0.f) thr = m + logf(mp);                      // p_i >= min_p * p_max
  const int k = top_k ? top_k[b] : -1;
  if (k > 0 && k < vocab) {
    float a = fmaxf(lo, thr), hi = m;                     // largest t with count(x >= t) >= k
    for (int it = 0; it < 48 && hi > a; ++it) {
      const float mid = 0.5f * (a + hi);
      float c, s;
      count_mass(row, vocab, inv_t, m, mid, thr, red, &c, &s);
      if (c >= (float)k) a = mid; else hi = mid;
    }
    thr = fmaxf(thr, a);
  }
  const float p = top_p ? top_p[b] : 1.f;
  if (p < 1.f && p > 0.f) {
    float c, denom;
    count_mass(row, vocab, inv_t, m, -INFINITY, thr, red, &c, &denom);
    float a = fmaxf(lo, thr), hi = m;                     // largest t with mass(x >= t) >= p * denom
    for (int it = 0; it < 48 && hi > a; ++it) {
      const float mid = 0.5f * (a + hi);
      float s;
      count_mass(row, vocab, inv_t, m, mid, thr, red, &c, &s);
      if (s >= p * denom) a = mid; else hi = mid;
    }
    thr = fmaxf(thr, a);
  }

  // inverse CDF in vocabulary order: thread t owns the contiguous ids [t*seg, (t+1)*seg)
  const int seg = (vocab + BLOCK - 1) / BLOCK;
  const int i0 = threadIdx.x * seg, i1 = min(vocab, i0 + seg);
  float mine = 0.f;
  for (int i = i0; i < i1; ++i) {
    const float x = row[i] * inv_t;
    if (x >= thr) mine += expf(x - m);
  }
  seg_sum[threadIdx.x] = mine;
  if (threadIdx.x == 0) choice = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int t = 0; t < BLOCK; ++t) total += seg_sum[t];
    const float target = philox_uniform(seeds[b], offsets[b]) * total;
    float before = 0.f;
    int owner = -1;
    for (int t = 0; t < BLOCK; ++t) {
      if (seg_sum[t] > 0.f && before + seg_sum[t] >= target) { owner = t; break; }
      before += seg_sum[t];
    }
    red[0] = target;
    red[1] = before;
    si[0] = owner;
  }
  __syncthreads();
  const int owner = si[0];
  if (owner == (int)threadIdx.x) {
    float cum = red[1];
    const float target = red[0];
    int last = -1;
    for (int i = i0; i < i1; ++i) {
      const float x = row[i] * inv_t;
      if (x >= thr) {
        cum += expf(x - m);
        last = i;
        if (cum >= target) break;
      }
    }
    choice = last;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int c = choice;
    if (c < 0) {   // the target lies a rounding above the total: the last kept token
      for (int i = vocab - 1; i >= 0; --i) if (row[i] * inv_t >= thr) { c = i; break; }
      if (c < 0) c = 0;
    }
    out[b] = c;
  }
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

}  // namespace

DINFER_DEFINE_LAST_ERROR()

DINFER_API int dinfer_argmax(const float* logits, int64_t ld, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  launch_pdl(argmax_kernel, dim3(rows), dim3(BLOCK), 0, stream, logits, ld, out, vocab);
  return cuda_status("argmax");
}

// temperature [rows]; top_k (<=0: off), top_p, min_p may be null; seeds, offsets [rows] uint64.
DINFER_API int dinfer_sample(const float* logits, int64_t ld, const float* temperature, const int* top_k,
                             const float* top_p, const float* min_p, const uint64_t* seeds,
                             const uint64_t* offsets, int* out, int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  launch_pdl(sample_kernel, dim3(rows), dim3(BLOCK), 0, stream, logits, ld, temperature, top_k, top_p, min_p, seeds, offsets, out, vocab);
  return cuda_status("sample");
}

DINFER_API int dinfer_penalties(float* logits, int64_t ld, const int* ids, const int* offsets,
                                const int* prompt_len, const float* rep, const float* freq, const float* pres,
                                int rows, int vocab, cudaStream_t stream) {
  if (rows < 0 || vocab <= 0 || ld < vocab) return refuse(DINFER_BAD_ARGUMENT, "penalties: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return 0;
  penalties_kernel<<<rows, 256, 0, stream>>>(logits, ld, ids, offsets, prompt_len, rep, freq, pres, vocab);
  return cuda_status("penalties");
}
