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

// eight consecutive elements at once
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 x = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[2 * j] = f.x; v[2 * j + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 x;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<uint4*>(p) = x;
}

// One warp per (token, head); a lane owns runs of 8 elements (VEC8) or single elements.
template <typename TA, typename TW, bool VEC8>
__global__ void __launch_bounds__(WARPS * 32)
qk_post_kernel(TA* __restrict__ qkv, int64_t ld, const int* __restrict__ positions,
               const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, float eps,
               const float* __restrict__ cos_sin, int rot, int interleaved,
               TA* __restrict__ cache, const int* __restrict__ slots, int block_size,
               int H, int Hkv, int D) {
  __shared__ __align__(16) float sm[WARPS][MAX_D];
  pdl_enter();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * WARPS + warp;
  if (head >= H + 2 * Hkv) return;
  const int kind = head < H ? 0 : (head < H + Hkv ? 1 : 2);   // q, k, v
  TA* x = qkv + (int64_t)t * ld + (int64_t)head * D;
  float* xs = sm[warp];
  constexpr int STEP = VEC8 ? 8 : 1;

  const TW* w = kind == 0 ? q_weight : (kind == 1 ? k_weight : nullptr);
  float ss = 0.f;
  for (int e = lane * STEP; e < D; e += 32 * STEP) {
    if (VEC8) {
      float v[8];
      load8<TA>(x + e, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) { xs[e + j] = v[j]; ss += v[j] * v[j]; }
    } else {
      const float v = to_f32<TA>(x[e]);
      xs[e] = v;
      ss += v * v;
    }
  }
  if (w) {
    ss = warp_sum(ss);
    const float rinv = rsqrtf(ss / (float)D + eps);
    for (int e = lane * STEP; e < D; e += 32 * STEP) {
#pragma unroll
      for (int j = 0; j < STEP; ++j) xs[e + j] = xs[e + j] * rinv * to_f32<TW>(w[e + j]);
    }
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
  const bool rewrite = kind != 2 && (w || rotate);
  const int half = rot >> 1;
  const float* cs = rotate ? cos_sin + (int64_t)positions[t] * rot : nullptr;
  for (int e0 = lane * STEP; e0 < D; e0 += 32 * STEP) {
    float r[8];
#pragma unroll
    for (int j = 0; j < STEP; ++j) {
      const int e = e0 + j;
      float v = xs[e];
      if (rotate && e < rot) {
        if (interleaved) {                                    // pairs (2i, 2i + 1), angle i
          const int i = e >> 1;
          v = (e & 1) ? v * cs[i] + xs[e - 1] * cs[half + i] : v * cs[i] - xs[e + 1] * cs[half + i];
        } else if (e < half) {                                // pairs (i, i + rot/2), angle i
          v = v * cs[e] - xs[e + half] * cs[half + e];
        } else {
          v = v * cs[e - half] + xs[e - half] * cs[e];
        }
      }
      r[j] = v;
    }
    if (VEC8) {
      if (rewrite) store8<TA>(x + e0, r);
      if (dst) store8<TA>(dst + e0, r);
    } else {
      const TA o = from_f32<TA>(r[0]);
      if (rewrite) x[e0] = o;
      if (dst) dst[e0] = o;
    }
  }
}

// Fast shape: bfloat16/f32 with D = 32 * EPL and the rotation over the whole head.  A lane owns EPL
// consecutive elements in registers; its rotation partner (D/2 away) sits 16 lanes across.  A warp takes
// HPW consecutive heads of one token and requests all of them before it works on the first, so that
// enough bytes are in flight for prompts (one 8-byte load per lane and head is not).
constexpr int HPW = 4;

template <typename TA, typename TW, int EPL>
__global__ void __launch_bounds__(WARPS * 32)
qk_post_lanes_kernel(TA* __restrict__ qkv, int64_t ld, const int* __restrict__ positions,
                     const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, float eps,
                     const float* __restrict__ cos_sin, TA* __restrict__ cache, const int* __restrict__ slots,
                     int block_size, int H, int Hkv) {
  constexpr int D = 32 * EPL;
  struct alignas(sizeof(TA) * EPL) Vec { TA v[EPL]; };
  struct alignas(sizeof(TW) * EPL) WVec { TW v[EPL]; };
  struct alignas(sizeof(float) * EPL) FVec { float v[EPL]; };
  pdl_enter();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head0 = (blockIdx.y * WARPS + warp) * HPW;
  const int heads = H + 2 * Hkv;
  if (head0 >= heads) return;
  TA* row = qkv + (int64_t)t * ld + lane * EPL;
  Vec in[HPW];
#pragma unroll
  for (int u = 0; u < HPW; ++u)
    if (head0 + u < heads) in[u] = *reinterpret_cast<const Vec*>(row + (int64_t)(head0 + u) * D);
  FVec c, sn;
  const bool has_table = cos_sin != nullptr;
  if (has_table) {
    const float* cs = cos_sin + (int64_t)positions[t] * D;
    const int i = (lane & 15) * EPL;                          // index of the pair inside the half
    c = *reinterpret_cast<const FVec*>(cs + i);
    sn = *reinterpret_cast<const FVec*>(cs + D / 2 + i);
  }
  const int slot = cache ? slots[t] : -1;
#pragma unroll
  for (int u = 0; u < HPW; ++u) {
    const int head = head0 + u;
    if (head >= heads) break;
    const int kind = head < H ? 0 : (head < H + Hkv ? 1 : 2);
    float v[EPL];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) { v[j] = to_f32<TA>(in[u].v[j]); ss += v[j] * v[j]; }
    const TW* w = kind == 0 ? q_weight : (kind == 1 ? k_weight : nullptr);
    if (w) {
      ss = warp_sum(ss);
      const float rinv = rsqrtf(ss / (float)D + eps);
      const WVec wv = *reinterpret_cast<const WVec*>(w + lane * EPL);
#pragma unroll
      for (int j = 0; j < EPL; ++j) v[j] = v[j] * rinv * to_f32<TW>(wv.v[j]);
    }
    const bool rotate = has_table && kind != 2;
    if (rotate) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);
        v[j] = lane < 16 ? v[j] * c.v[j] - other * sn.v[j] : v[j] * c.v[j] + other * sn.v[j];
      }
    }
    Vec out;
#pragma unroll
    for (int j = 0; j < EPL; ++j) out.v[j] = from_f32<TA>(v[j]);
    if (kind != 2 && (w || rotate)) *reinterpret_cast<Vec*>(row + (int64_t)head * D) = out;
    if (kind != 0 && slot >= 0) {
      const int64_t blk = slot / block_size, off = slot % block_size;
      const int hk = kind == 1 ? head - H : head - H - Hkv;
      TA* dst = cache + ((((blk * 2 + (kind - 1)) * Hkv + hk) * block_size + off) * (int64_t)D) + lane * EPL;
      *reinterpret_cast<Vec*>(dst) = out;
    }
  }
}

// Head size 128 in bfloat16, the rotation over the whole head: half a warp per head.  A lane owns four consecutive
// elements of the head's first half and the four elements 64 further on, which are their rotation partners, so the
// rotation needs no exchange between lanes (two 8-byte accesses a head).  A warp takes HALF_HP pairs of heads (one
// where the tokens are few: a decode step is a chain of latencies, more warps make it shorter) of one
// token and requests all of them before it works on the first.  Value heads are only copied into the cache.
constexpr int FEW_TOKENS = 128;

__device__ __forceinline__ void unpack4(const uint2& x, float (&v)[4]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ uint2 pack4(const float (&v)[4]) {
  uint2 x;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&x);
  h[0] = __floats2bfloat162_rn(v[0], v[1]);
  h[1] = __floats2bfloat162_rn(v[2], v[3]);
  return x;
}

template <typename TW, int HALF_HP>
__global__ void __launch_bounds__(WARPS * 32)
qk_post_half_warp_kernel(__nv_bfloat16* __restrict__ qkv, int64_t ld, const int* __restrict__ positions,
                         const TW* __restrict__ q_weight, const TW* __restrict__ k_weight, float eps,
                         const float* __restrict__ cos_sin, __nv_bfloat16* __restrict__ cache,
                         const int* __restrict__ slots, int block_size, int H, int Hkv) {
  constexpr int D = 128;
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int side = lane >> 4, l = lane & 15;
  const int head0 = (blockIdx.y * WARPS + warp) * 2 * HALF_HP + side;
  const int heads = H + 2 * Hkv;
  // What no kernel of the step writes (the token's position and slot, its row of the angle table, the norm weights)
  // is fetched while the kernel before this one may still be running; the q/k/v rows only after it has completed.
  pdl_launch_dependents();
  float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool has_table = cos_sin != nullptr;
  if (has_table) {
    const float* cs = cos_sin + (int64_t)positions[t] * D + l * 4;
    c = *reinterpret_cast<const float4*>(cs);
    sn = *reinterpret_cast<const float4*>(cs + D / 2);
  }
  const float cv[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
  const int slot = cache ? slots[t] : -1;
  const int64_t blk = slot >= 0 ? slot / block_size : 0, off = slot >= 0 ? slot % block_size : 0;
  float wq[2][4], wk[2][4];                                    // this lane's norm weights: [half of the head][element]
  auto weights = [&](const TW* w, float (&dst)[2][4]) {
    if (!w) {
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[0][j] = dst[1][j] = 1.f;
    } else if constexpr (sizeof(TW) == 2) {
      unpack4(*reinterpret_cast<const uint2*>(w + l * 4), dst[0]);
      unpack4(*reinterpret_cast<const uint2*>(w + D / 2 + l * 4), dst[1]);
    } else {
      const float4 x = *reinterpret_cast<const float4*>(w + l * 4), y = *reinterpret_cast<const float4*>(w + D / 2 + l * 4);
      dst[0][0] = x.x; dst[0][1] = x.y; dst[0][2] = x.z; dst[0][3] = x.w;
      dst[1][0] = y.x; dst[1][1] = y.y; dst[1][2] = y.z; dst[1][3] = y.w;
    }
  };
  weights(q_weight, wq);
  weights(k_weight, wk);
  pdl_wait();
  __nv_bfloat16* row = qkv + (int64_t)t * ld + l * 4;          // this lane's elements of the first half
  uint2 lo[HALF_HP], hi[HALF_HP];
#pragma unroll
  for (int u = 0; u < HALF_HP; ++u)
    if (head0 + 2 * u < heads) {
      lo[u] = *reinterpret_cast<const uint2*>(row + (int64_t)(head0 + 2 * u) * D);
      hi[u] = *reinterpret_cast<const uint2*>(row + (int64_t)(head0 + 2 * u) * D + D / 2);
    }
#pragma unroll
  for (int u = 0; u < HALF_HP; ++u) {
    const int head = head0 + 2 * u;
    const bool live = head < heads;                            // (the other half of the warp may still have a head)
    const int kind = head < H ? 0 : (head < H + Hkv ? 1 : 2);
    const TW* w = !live ? nullptr : (kind == 0 ? q_weight : (kind == 1 ? k_weight : nullptr));
    const bool rotate = has_table && live && kind != 2;
    uint2 out_lo = lo[u], out_hi = hi[u];
    float a[4], b[4];
    float ss = 0.f;
    if (live && kind != 2) {
      unpack4(lo[u], a);
      unpack4(hi[u], b);
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += a[j] * a[j] + b[j] * b[j];
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // over the head's 16 lanes
    if (live && kind != 2) {
      if (w) {
        const float rinv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a[j] = a[j] * rinv * (kind == 0 ? wq[0][j] : wk[0][j]);
          b[j] = b[j] * rinv * (kind == 0 ? wq[1][j] : wk[1][j]);
        }
      }
      if (rotate) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float x = a[j], y = b[j];
          a[j] = x * cv[j] - y * sv[j];
          b[j] = y * cv[j] + x * sv[j];
        }
      }
      out_lo = pack4(a);
      out_hi = pack4(b);
      if (w || rotate) {
        *reinterpret_cast<uint2*>(row + (int64_t)head * D) = out_lo;
        *reinterpret_cast<uint2*>(row + (int64_t)head * D + D / 2) = out_hi;
      }
    }
    if (live && kind != 0 && slot >= 0) {
      const int hk = kind == 1 ? head - H : head - H - Hkv;
      __nv_bfloat16* dst = cache + ((((blk * 2 + (kind - 1)) * Hkv + hk) * block_size + off) * (int64_t)D) + l * 4;
      *reinterpret_cast<uint2*>(dst) = out_lo;
      *reinterpret_cast<uint2*>(dst + D / 2) = out_hi;
    }
  }
}

template <typename TA, typename TW>
void launch_lanes(dim3 grid, cudaStream_t stream, TA* qkv, int64_t ld, const int* positions, const TW* qw,
                  const TW* kw, float eps, const float* cos_sin, TA* cache, const int* slots, int block_size,
                  int H, int Hkv, int D) {
  const int threads = WARPS * 32;
  if (D == 32) launch_pdl(qk_post_lanes_kernel<TA, TW, 1>, grid, dim3(threads), 0, stream, qkv, ld, positions, qw, kw, eps, cos_sin, cache, slots, block_size, H, Hkv);
  else if (D == 64) launch_pdl(qk_post_lanes_kernel<TA, TW, 2>, grid, dim3(threads), 0, stream, qkv, ld, positions, qw, kw, eps, cos_sin, cache, slots, block_size, H, Hkv);
  else if (D == 128) launch_pdl(qk_post_lanes_kernel<TA, TW, 4>, grid, dim3(threads), 0, stream, qkv, ld, positions, qw, kw, eps, cos_sin, cache, slots, block_size, H, Hkv);
  else launch_pdl(qk_post_lanes_kernel<TA, TW, 8>, grid, dim3(threads), 0, stream, qkv, ld, positions, qw, kw, eps, cos_sin, cache, slots, block_size, H, Hkv);
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// qkv [T, >= (H+2Hkv)*D] act dtype with row stride ld, laid out q heads | k heads | v heads.
// positions [T] int32; q_weight/k_weight [D] or null; cos_sin [max_pos, rot] f32 (cos | sin) or null;
// cache (act dtype) or null; slots [T] int32 (negative = do not write).
// interleaved = 0: the rotation pairs element i with i + rot/2 (neox); 1: element 2i with 2i + 1.
DINFER_API int dinfer_qk_post_styled(void* qkv, int64_t ld, const int* positions, const void* q_weight,
                                     const void* k_weight, float eps, const float* cos_sin, int rot, int interleaved,
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
      const bool aligned = ld % 8 == 0 && !(reinterpret_cast<uintptr_t>(qkv) & 31) &&
                           !(reinterpret_cast<uintptr_t>(cache) & 31) && !(reinterpret_cast<uintptr_t>(q_weight) & 31) &&
                           !(reinterpret_cast<uintptr_t>(k_weight) & 31) && !(reinterpret_cast<uintptr_t>(cos_sin) & 31);
      if constexpr (sizeof(TA) == 2) {
        if (aligned && !interleaved && (!cos_sin || rot == D) && D == 128) {
          const int hp = T <= FEW_TOKENS ? 1 : 3;
          const dim3 half_grid(T, (heads + WARPS * 2 * hp - 1) / (WARPS * 2 * hp));
          launch_pdl(hp == 1 ? qk_post_half_warp_kernel<TW, 1> : qk_post_half_warp_kernel<TW, 3>, half_grid, dim3(WARPS * 32), 0,
                     stream, (__nv_bfloat16*)qkv, ld, positions,
                     (const TW*)q_weight, (const TW*)k_weight, eps, cos_sin, (__nv_bfloat16*)cache, slots, block_size, H, Hkv);
          return cuda_status("qk_post");
        }
      }
      if (aligned && !interleaved && (!cos_sin || rot == D) && (D == 32 || D == 64 || D == 128 || D == 256)) {
        const dim3 lanes_grid(T, (heads + WARPS * HPW - 1) / (WARPS * HPW));
        launch_lanes<TA, TW>(lanes_grid, stream, (TA*)qkv, ld, positions, (const TW*)q_weight, (const TW*)k_weight, eps,
                             cos_sin, (TA*)cache, slots, block_size, H, Hkv, D);
        return cuda_status("qk_post");
      }
      // 8-wide accesses need rows, heads and cache slots that start on 32-byte (f32) / 16-byte (bf16) bounds
      const bool vec8 = D % 8 == 0 && ld % 8 == 0 && !(reinterpret_cast<uintptr_t>(qkv) & 31) &&
                        !(reinterpret_cast<uintptr_t>(cache) & 31);
      if (vec8)
        qk_post_kernel<TA, TW, true><<<grid, WARPS * 32, 0, stream>>>(
            (TA*)qkv, ld, positions, (const TW*)q_weight, (const TW*)k_weight, eps, cos_sin, rot, interleaved,
            (TA*)cache, slots, block_size, H, Hkv, D);
      else
        qk_post_kernel<TA, TW, false><<<grid, WARPS * 32, 0, stream>>>(
            (TA*)qkv, ld, positions, (const TW*)q_weight, (const TW*)k_weight, eps, cos_sin, rot, interleaved,
            (TA*)cache, slots, block_size, H, Hkv, D);
      return cuda_status("qk_post");
    }));
  return 0;
}

DINFER_API int dinfer_qk_post(void* qkv, int64_t ld, const int* positions, const void* q_weight,
                              const void* k_weight, float eps, const float* cos_sin, int rot,
                              void* cache, const int* slots, int block_size,
                              int T, int H, int Hkv, int D, int act_dtype, int w_dtype,
                              cudaStream_t stream) {
  return dinfer_qk_post_styled(qkv, ld, positions, q_weight, k_weight, eps, cos_sin, rot, 0, cache, slots, block_size, T, H,
                               Hkv, D, act_dtype, w_dtype, stream);
}
