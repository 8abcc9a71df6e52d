// RMSNorm over rows of the 32-bit residual stream, with the residual add and the row gather
// fused in.  One block per output row.
//
//   v      = residual[src] + delta[src]          (delta optional; src = rows[r] or r)
//   residual[src] = v                            (only when delta is given and rows is not)
//   out[r] = T( v * rsqrt(mean(v^2) + eps) * w ) (one rounding, after the weight multiply)
//
// Sum of squares, rsqrt and products are 32-bit.  Counterpart in the reference:
// crates/kernels/cuda/norm.cu:41-116 (rmsnorm / fused_add_rmsnorm / gather_rmsnorm), which keeps
// the residual in bf16; here it stays in 32-bit so that the sum is exact to rounding of one add.
#include "common.cuh"

using namespace dinfer;

namespace {

// four consecutive elements at once (16 bytes of f32, 8 bytes of bf16)
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 x;
  *reinterpret_cast<__nv_bfloat162*>(&x.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&x.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = x;
}

template <typename TA, typename TW, int VEC>
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta, const int* __restrict__ rows,
               const TW* __restrict__ weight, TA* __restrict__ out, int h, float eps, int stash) {
  extern __shared__ float sm_row[];
  __shared__ float red[33];
  pdl_enter();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (int64_t)src * h;
  const TA* del = delta ? delta + (int64_t)src * h : nullptr;
  const bool writeback = (delta != nullptr) && (rows == nullptr);
  TA* o = out + (int64_t)r * h;

  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float v[4];
    if (VEC == 4) {
      load4<float>(res + i, v);
      if (del) {
        float d[4];
        load4<TA>(del + i, d);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += d[j];
        if (writeback) store4<float>(res + i, v);
      }
    } else {
      v[0] = res[i];
      if (del) {
        v[0] += to_f32<TA>(del[i]);
        if (writeback) res[i] = v[0];
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      ss += v[j] * v[j];
      if (stash) sm_row[i + j] = v[j];
    }
  }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)h + eps);
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float v[4], w[4];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      if (stash) v[j] = sm_row[i + j];
      else v[j] = res[i + j] + ((del && !writeback) ? to_f32<TA>(del[i + j]) : 0.f);
    }
    if (VEC == 4) {
      load4<TW>(weight + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = v[j] * rinv * w[j];
      store4<TA>(o + i, v);
    } else {
      o[i] = from_f32<TA>(v[0] * rinv * to_f32<TW>(weight[i]));
    }
  }
}

template <typename TA, typename TW>
int launch(float* residual, const void* delta, const int* rows, const void* weight, void* out,
           int num_rows, int h, float eps, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec4 = (h % 4 == 0) && al(residual) && al(delta) && al(weight) && al(out);
  const int per = vec4 ? 4 : 1;
  int threads = (h / per + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  const size_t row_bytes = (size_t)h * sizeof(float);
  const int stash = row_bytes <= 64 * 1024;
  const size_t smem = stash ? row_bytes : 0;
  auto k4 = rmsnorm_kernel<TA, TW, 4>;
  auto k1 = rmsnorm_kernel<TA, TW, 1>;
  auto k = vec4 ? k4 : k1;
  static bool opted[2] = {false, false};   // once per process and kernel, kept out of graph captures
  if (smem > 48 * 1024 && !opted[vec4]) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return refuse((int)e, "rmsnorm: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted[vec4] = true;
  }
  launch_pdl(k, dim3(num_rows), dim3(threads), smem, stream, residual, (const TA*)delta, rows, (const TW*)weight, (TA*)out, h, eps, stash);
  return cuda_status("rmsnorm");
}

// Plain RMSNorm of rows that are not the residual stream (toy parts, tests): x of type TA.
template <typename TA, typename TW>
__global__ void rmsnorm_plain_kernel(const TA* __restrict__ x, const TW* __restrict__ weight,
                                     TA* __restrict__ out, int h, float eps) {
  __shared__ float red[33];
  const TA* row = x + (int64_t)blockIdx.x * h;
  float ss = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) { const float v = to_f32<TA>(row[i]); ss += v * v; }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)h + eps);
  for (int i = threadIdx.x; i < h; i += blockDim.x)
    out[(int64_t)blockIdx.x * h + i] = from_f32<TA>(to_f32<TA>(row[i]) * rinv * to_f32<TW>(weight[i]));
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// residual [*, h] f32 (updated in place when delta is given and rows is null); delta [*, h] act
// dtype or null; rows [num_rows] int32 or null; weight [h]; out [num_rows, h] act dtype.
DINFER_API int dinfer_rmsnorm(float* residual, const void* delta, const int* rows, const void* weight,
                              void* out, int num_rows, int h, float eps, int act_dtype, int w_dtype,
                              cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "rmsnorm: bad sizes rows=%d h=%d", num_rows, h);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW,
      return launch<TA, TW>(residual, delta, rows, weight, out, num_rows, h, eps, stream)));
  return 0;
}

DINFER_API int dinfer_rmsnorm_plain(const void* x, const void* weight, void* out, int num_rows, int h,
                                    float eps, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "rmsnorm_plain: bad sizes rows=%d h=%d", num_rows, h);
  if (num_rows == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      rmsnorm_plain_kernel<TA, TW><<<num_rows, threads, 0, stream>>>((const TA*)x, (const TW*)weight, (TA*)out, h, eps);
      return cuda_status("rmsnorm_plain");
    }));
  return 0;
}
