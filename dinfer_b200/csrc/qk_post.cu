// After the q/k/v projection, in one pass over a token's heads: per-head RMSNorm of q and k,
// neox rotation of the first `rot` dims by the angle table row of the token's position, q and k
// written back in place, and k and v written to the token's slot of the paged cache.
// Every piece is optional (null weight / null table / null cache), so the same kernel serves a
// mixer without head norm, without rotation, or one that reads another layer's cache.
//
// Cache layout, per layer: [num_blocks, 2 (k, v), Hkv, block_size, D]; slot = block*block_size + offset.
// Counterpart in the reference: crates/kernels/cuda/qkv_post.cu:26-91 (D in {128, 256} only there).
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int WARPS = 8;
constexpr int MAX_D = 512;

template <typename TA, typename TW>
__global__ void __launch_bounds__(WARPS * 32)
qk_post_kernel(TA* __restrict__ qkv, int64_t ld, const int* __restrict__ positions,
               const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, float eps,
               const float* __restrict__ cos_sin, int rot,
               TA* __restrict__ cache, const int* __restrict__ slots, int block_size,
               int H, int Hkv, int D) {
  __shared__ float sm[WARPS][MAX_D];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * WARPS + warp;
  if (head >= H + 2 * Hkv) return;
  const int kind = head < H ? 0 : (head < H + Hkv ? 1 : 2);   // q, k, v
  TA* x = qkv + (int64_t)t * ld + (int64_t)head * D;
  float* xs = sm[warp];

  const TW* w = kind == 0 ? q_weight : (kind == 1 ? k_weight : nullptr);
  float ss = 0.f;
  for (int e = lane; e < D; e += 32) {
    const float v = to_f32<TA>(x[e]);
    xs[e] = v;
    ss += v * v;
  }
  if (w) {
    ss = warp_sum(ss);
    const float rinv = rsqrtf(ss / (float)D + eps);
    for (int e = lane; e < D; e += 32) xs[e] = xs[e] * rinv * to_f32<TW>(w[e]);
  }
  __syncwarp();

  TA* dst = nullptr;
  if (cache && kind != 0) {
    const int slot = slots[t];
    if (slot >= 0) {
      const int64_t blk = slot / block_size, off = slot % block_size;
      const int hk = kind == 1 ? head - H : head - H - Hkv;
      dst = cache + ((((blk * 2 + (kind - 1)) * Hkv + hk) * block_size + off) * (int64_t)D);
    }
  }
  const bool rotate = cos_sin != nullptr && kind != 2;
  const int half = rot >> 1;
  const float* cs = rotate ? cos_sin + (int64_t)positions[t] * rot : nullptr;
  for (int e = lane; e < D; e += 32) {
    float v = xs[e];
    if (rotate && e < rot) {
      if (e < half) v = v * cs[e] - xs[e + half] * cs[half + e];
      else          v = v * cs[e - half] + xs[e - half] * cs[e];
    }
    const TA r = from_f32<TA>(v);
    if (kind != 2 && (w || rotate)) x[e] = r;
    if (dst) dst[e] = r;
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// qkv [T, >= (H+2Hkv)*D] act dtype with row stride ld, laid out q heads | k heads | v heads.
// positions [T] int32; q_weight/k_weight [D] or null; cos_sin [max_pos, rot] f32 (cos | sin) or null;
// cache (act dtype) or null; slots [T] int32 (negative = do not write).
DINFER_API int dinfer_qk_post(void* qkv, int64_t ld, const int* positions, const void* q_weight,
                              const void* k_weight, float eps, const float* cos_sin, int rot,
                              void* cache, const int* slots, int block_size,
                              int T, int H, int Hkv, int D, int act_dtype, int w_dtype,
                              cudaStream_t stream) {
  if (T < 0 || H <= 0 || Hkv < 0 || D <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "qk_post: bad sizes T=%d H=%d Hkv=%d D=%d", T, H, Hkv, D);
  if (D > MAX_D) return refuse(DINFER_BAD_ARGUMENT, "qk_post: head_dim %d above the limit %d", D, MAX_D);
  if (cos_sin && (rot <= 0 || rot > D || (rot & 1)))
    return refuse(DINFER_BAD_ARGUMENT, "qk_post: rotary dim %d must be even and at most head_dim %d", rot, D);
  if (ld < (int64_t)(H + 2 * Hkv) * D) return refuse(DINFER_BAD_ARGUMENT, "qk_post: row stride below the row's width");
  if (cache && block_size <= 0) return refuse(DINFER_BAD_ARGUMENT, "qk_post: block_size %d", block_size);
  if (T == 0) return 0;
  const int heads = H + 2 * Hkv;
  if ((heads + WARPS - 1) / WARPS > 65535) return refuse(DINFER_BAD_ARGUMENT, "qk_post: too many heads");
  dim3 grid(T, (heads + WARPS - 1) / WARPS);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      qk_post_kernel<TA, TW><<<grid, WARPS * 32, 0, stream>>>(
          (TA*)qkv, ld, positions, (const TW*)q_weight, (const TW*)k_weight, eps, cos_sin, rot,
          (TA*)cache, slots, block_size, H, Hkv, D);
      return cuda_status("qk_post");
    }));
  return 0;
}
