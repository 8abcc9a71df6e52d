// Paged causal attention for any head size, any group size, 32-bit or bfloat16 storage:
// the plain-arithmetic path (no tensor cores).  It is the whole attention of the 32-bit model and
// the fallback of the bfloat16 model for head sizes the tensor-core kernels refuse.
//
// One warp owns one (token, query head): the lanes split the head's D elements, keys are visited
// four at a time in position order with an online softmax; scores, softmax and the output sum are
// 32-bit (expf, not the fast intrinsic).  A query at position p sees the keys [max(0, p-window+1), p]
// of its own request, read through the request's block table.
//
// Counterpart in the reference: the any-D reference kernels crates/kernels/cuda/gqa.cu:956-1118.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int WARPS = 4;
constexpr int KEYS = 4;

template <typename T, int C>   // C = ceil(D / 32) elements per lane
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int64_t ldq, T* __restrict__ out, int64_t ldo,
                         const T* __restrict__ cache, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ positions,
                         int num_reqs, int H, int Hkv, int D, int block_size, float scale, int window) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= H) return;
  // request of this token: last b with cu_seqlens[b] <= t
  int lo = 0, hi = num_reqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int* table = block_table + (int64_t)lo * max_blocks;
  const int hk = h / (H / Hkv);
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float qv[C], acc[C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    qv[c] = e < D ? to_f32<T>(q[(int64_t)t * ldq + (int64_t)h * D + e]) * scale : 0.f;
    acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int64_t plane = (int64_t)Hkv * block_size * D;       // one of k / v of one block
  for (int j0 = first; j0 <= pos; j0 += KEYS) {
    const T* kp[KEYS];
    float s[KEYS];
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      const int j = j0 + u;
      kp[u] = nullptr;
      s[u] = 0.f;
      // a page the table does not hold (-1: a dummy row of a captured graph, a page a window has passed) is no key
      const int64_t blk = j <= pos ? table[j / block_size] : -1;
      if (blk >= 0) {
        kp[u] = cache + blk * 2 * plane + ((int64_t)hk * block_size + j % block_size) * D;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < D) s[u] += qv[c] * to_f32<T>(kp[u][e]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < KEYS; ++u) s[u] = kp[u] ? warp_sum(s[u]) : -INFINITY;
    float m_new = m;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) m_new = fmaxf(m_new, s[u]);
    if (m_new == -INFINITY) continue;                            // no key so far
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] *= alpha;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      if (kp[u]) {
        const float p = expf(s[u] - m_new);
        l += p;
        const T* vp = kp[u] + plane;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < D) acc[c] += p * to_f32<T>(vp[e]);
        }
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;                      // a row without keys gives zeros
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    if (e < D) out[(int64_t)t * ldo + (int64_t)h * D + e] = from_f32<T>(acc[c] * inv);
  }
}

template <typename T, int C>
int launch(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache, const int* block_table,
           int max_blocks, const int* cu_seqlens, const int* positions, int T_, int B, int H, int Hkv,
           int D, int block_size, float scale, int window, cudaStream_t stream) {
  dim3 grid(T_, (H + WARPS - 1) / WARPS);
  attention_generic_kernel<T, C><<<grid, WARPS * 32, 0, stream>>>(
      (const T*)q, ldq, (T*)out, ldo, (const T*)cache, block_table, max_blocks, cu_seqlens, positions,
      B, H, Hkv, D, block_size, scale, window);
  return cuda_status("attention_generic");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q: [T, ...] rows of stride ldq, head h at h*D; out likewise with stride ldo.
// cache [num_blocks, 2, Hkv, block_size, D]; block_table [B, max_blocks] int32;
// cu_seqlens [B+1] int32 (token offsets of the requests); positions [T] int32.
// window <= 0: all keys.
DINFER_API int dinfer_attention_generic(const void* q, int64_t ldq, void* out, int64_t ldo, const void* cache,
                                        const int* block_table, int max_blocks, const int* cu_seqlens,
                                        const int* positions, int T, int B, int H, int Hkv, int D,
                                        int block_size, float scale, int window, int dtype,
                                        cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || Hkv <= 0 || D <= 0 || block_size <= 0 || max_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_generic: bad sizes T=%d B=%d H=%d Hkv=%d D=%d block=%d",
                  T, B, H, Hkv, D, block_size);
  if (H % Hkv) return refuse(DINFER_BAD_ARGUMENT, "attention_generic: heads %d not divisible by kv heads %d", H, Hkv);
  if (D > 512) return refuse(DINFER_BAD_ARGUMENT, "attention_generic: head_dim %d above the limit 512", D);
  if ((H + WARPS - 1) / WARPS > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_generic: too many heads");
  if (T == 0) return 0;
  const int c = (D + 31) / 32;
#define GO(C) return launch<T_, C>(q, ldq, out, ldo, cache, block_table, max_blocks, cu_seqlens, positions, \
                                   T, B, H, Hkv, D, block_size, scale, window, stream)
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    if (c <= 1) GO(1);
    else if (c <= 2) GO(2);
    else if (c <= 4) GO(4);
    else if (c <= 8) GO(8);
    else GO(16);
  });
#undef GO
  return 0;
}
