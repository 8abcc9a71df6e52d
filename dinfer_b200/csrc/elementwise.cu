// Embedding gather into the 32-bit residual stream, and the SwiGLU gate.
// Counterparts in the reference: crates/kernels/cuda/activation.cu:121-129 (embedding, an id out of
// range reads row 0) and :80-99 (silu_and_mul).
// A negative id -(r + 1) names row r of `prev`, the tokens the previous step sampled, which are still on
// the device when this step is launched before the host has read them (the reference's asynchronous
// scheduling feeds its placeholders the same way: crates/core/src/sched/mod.rs:645-668).
#include "common.cuh"

using namespace dinfer;

namespace {

template <typename TW>
__global__ void embedding_kernel(const int* __restrict__ ids, const int* __restrict__ prev, int prev_rows,
                                 const TW* __restrict__ table, float* __restrict__ out, int h, int vocab, float scale) {
  pdl_enter();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 && prev != nullptr && -id - 1 < prev_rows) id = prev[-id - 1];
  if (id < 0 || id >= vocab) id = 0;
  const TW* row = table + (int64_t)id * h;
  float* o = out + (int64_t)t * h;
  for (int i = threadIdx.x; i < h; i += blockDim.x) o[i] = to_f32<TW>(row[i]) * scale;
}

__global__ void softcap_kernel(float* __restrict__ x, int64_t n, float cap) {
  pdl_enter();
  const float inv = 1.f / cap;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] * inv);
}

// out[t, i] = silu(gate_i) * up_i; silu(g) = g / (1 + exp(-g)) in 32-bit, one rounding.  The row of x holds
// gate and up as two halves (gate_i at i, up_i at I + i) or in pairs (gate_i at 2i, up_i at 2i + 1).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ x, T* __restrict__ out, int inter, int64_t ldx, int pairs) {
  const int t = blockIdx.x;
  const T* row = x + (int64_t)t * ldx;
  T* o = out + (int64_t)t * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    const float a = to_f32<T>(pairs ? row[2 * i] : row[i]);
    const float b = to_f32<T>(pairs ? row[2 * i + 1] : row[inter + i]);
    o[i] = from_f32<T>(a / (1.f + expf(-a)) * b);
  }
}

// out[t, n] += bias[n]: the bias of a linear part (none of the Qwen3 dense model's products has one; a mixer
// or feed-forward of another architecture may), added in 32-bit with one rounding
template <typename T, typename TB>
__global__ void add_bias_kernel(T* __restrict__ out, int64_t ld, const TB* __restrict__ bias, int n) {
  pdl_enter();
  T* row = out + (int64_t)blockIdx.x * ld;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x)
    row[i] = from_f32<T>(to_f32<T>(row[i]) + to_f32<TB>(bias[i]));
}

// bfloat16 in pairs: 16 inputs (two 16-byte loads) -> 8 outputs (one 16-byte store) per thread
__global__ void silu_mul_pairs_bf16_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                           int inter8, int64_t ldx, int inter) {
  pdl_enter();
  const int t = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
  uint4* o = reinterpret_cast<uint4*>(out + (int64_t)t * inter);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter8; i += gridDim.y * blockDim.x) {
    const uint4 a = src[2 * i], b = src[2 * i + 1];
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    float r[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g0 = __bfloat1622float2(pa[j]), g1 = __bfloat1622float2(pb[j]);
      r[j] = g0.x / (1.f + expf(-g0.x)) * g0.y;
      r[4 + j] = g1.x / (1.f + expf(-g1.x)) * g1.y;
    }
    uint4 w;
    __nv_bfloat162* pw = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
    for (int j = 0; j < 4; ++j) pw[j] = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
    o[i] = w;
  }
}

// bfloat16, 8 elements (16 bytes) per thread: the shape prompts run at
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                       int inter8, int64_t ldx, int inter) {
  pdl_enter();
  const int t = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx);
  const uint4* u = reinterpret_cast<const uint4*>(x + (int64_t)t * ldx + inter);
  uint4* o = reinterpret_cast<uint4*>(out + (int64_t)t * inter);
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter8; i += gridDim.y * blockDim.x) {
    const uint4 a = g[i], b = u[i];
    uint4 r;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
      pr[j] = __floats2bfloat162_rn(fa.x / (1.f + expf(-fa.x)) * fb.x, fa.y / (1.f + expf(-fa.y)) * fb.y);
    }
    o[i] = r;
  }
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = from_f32<TD>(to_f32<TS>(src[i]));
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// ids [T] int32; table [vocab, h]; out [T, h] f32; prev [prev_rows] int32 or null (see the head of the file).
// out[t] = table[ids[t]] * scale (scale 1 for a model that does not scale its embedding)
DINFER_API int dinfer_embedding(const int* ids, const int* prev, int prev_rows, const void* table, float* out, int T,
                                int h, int vocab, int table_dtype, float scale, cudaStream_t stream) {
  if (T < 0 || h <= 0 || vocab <= 0) return refuse(DINFER_BAD_ARGUMENT, "embedding: bad sizes T=%d h=%d vocab=%d", T, h, vocab);
  if (T == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  DINFER_DISPATCH_DTYPE(table_dtype, TW, {
    launch_pdl(embedding_kernel<TW>, dim3(T), dim3(threads), 0, stream, ids, prev, prev_rows, (const TW*)table, out, h, vocab, scale);
    return cuda_status("embedding");
  });
  return 0;
}

// x [T, 2*inter] with row stride ldx; out [T, inter].  pairs = 0: gate first, then up; 1: (gate_i, up_i) pairs.
DINFER_API int dinfer_silu_mul(const void* x, void* out, int T, int inter, int64_t ldx, int dtype, int pairs,
                               cudaStream_t stream) {
  if (T < 0 || inter <= 0 || ldx < 2 * (int64_t)inter)
    return refuse(DINFER_BAD_ARGUMENT, "silu_mul: bad sizes T=%d inter=%d ldx=%lld", T, inter, (long long)ldx);
  if (T == 0) return 0;
  const int threads = 256;
  int bx = (inter + threads - 1) / threads;
  if (bx > 64) bx = 64;
  if (pairs && dtype == DINFER_BF16 && inter % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    int by = (inter / 8 + threads - 1) / threads;
    if (by > 64) by = 64;
    launch_pdl(silu_mul_pairs_bf16_kernel, dim3(T, by), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
               (__nv_bfloat16*)out, inter / 8, ldx, inter);
    return cuda_status("silu_mul");
  }
  if (!pairs && dtype == DINFER_BF16 && inter % 8 == 0 && ldx % 8 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) &&
      !(reinterpret_cast<uintptr_t>(out) & 15)) {
    int by = (inter / 8 + threads - 1) / threads;
    if (by > 64) by = 64;
    launch_pdl(silu_mul_bf16x8_kernel, dim3(T, by), dim3(threads), 0, stream, (const __nv_bfloat16*)x,
               (__nv_bfloat16*)out, inter / 8, ldx, inter);
    return cuda_status("silu_mul");
  }
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    silu_mul_kernel<T_><<<dim3(T, bx), threads, 0, stream>>>((const T_*)x, (T_*)out, inter, ldx, pairs);
    return cuda_status("silu_mul");
  });
  return 0;
}

// dst[i] = (dst type) src[i]
DINFER_API int dinfer_cast(const void* src, void* dst, int64_t n, int src_dtype, int dst_dtype,
                           cudaStream_t stream) {
  if (n < 0) return refuse(DINFER_BAD_ARGUMENT, "cast: negative length");
  if (n == 0) return 0;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  DINFER_DISPATCH_DTYPE(src_dtype, TS,
    DINFER_DISPATCH_DTYPE(dst_dtype, TD, {
      cast_kernel<TS, TD><<<(int)blocks, 256, 0, stream>>>((const TS*)src, (TD*)dst, n);
      return cuda_status("cast");
    }));
  return 0;
}

// x[i] = cap * tanh(x[i] / cap) in place over n 32-bit values (logits with a soft cap)
DINFER_API int dinfer_softcap(float* x, int64_t n, float cap, cudaStream_t stream) {
  if (n < 0 || !(cap > 0.f)) return refuse(DINFER_BAD_ARGUMENT, "softcap: n=%lld cap=%g", (long long)n, (double)cap);
  if (n == 0) return 0;
  int64_t blocks = (n + 1023) / 1024;
  if (blocks > 4096) blocks = 4096;
  launch_pdl(softcap_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, x, n, cap);
  return cuda_status("softcap");
}

// out [T, N] (row stride ld, act dtype) += bias [N] (bias dtype)
DINFER_API int dinfer_add_bias(void* out, int64_t ld, const void* bias, int T, int N, int act_dtype, int bias_dtype,
                               cudaStream_t stream) {
  if (T < 0 || N <= 0 || ld < N) return refuse(DINFER_BAD_ARGUMENT, "add_bias: bad sizes T=%d N=%d", T, N);
  if (T == 0) return 0;
  dim3 grid(T, (N + 1023) / 1024 > 64 ? 64 : (N + 1023) / 1024);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(bias_dtype, TB, {
      launch_pdl(add_bias_kernel<TA, TB>, grid, dim3(256), 0, stream, (TA*)out, ld, (const TB*)bias, N);
      return cuda_status("add_bias");
    }));
  return 0;
}
