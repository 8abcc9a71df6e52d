// Shared helpers of the kernel libraries.  Every library is one .cu file built into its own
// shared object with a C ABI: `extern "C" int dinfer_<op>(pointers..., sizes..., cudaStream_t)`.
// A call returns 0, a positive cudaError_t, or a negative refusal code; the text of the last
// refusal or CUDA error of the calling thread is read with dinfer_last_error().
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>

#define DINFER_API extern "C" __attribute__((visibility("default")))

enum DinferDtype : int { DINFER_F32 = 0, DINFER_BF16 = 1 };

enum DinferStatus : int {
  DINFER_OK = 0,
  DINFER_BAD_ARGUMENT = -1,   // a size or option the kernel does not take
  DINFER_BAD_DTYPE = -2,
  DINFER_DEVICE_STATUS = -3,  // a kernel recorded a fault in its status word
};

namespace dinfer {

inline char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

inline int refuse(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int cuda_status(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(error_buffer(), 512, "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}

// ---- element types: storage in T, arithmetic in float ----
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace dinfer

// ---- programmatic dependent launch: a kernel launched through launch_pdl may start while the kernel
// before it on the stream is still running; everything it does before pdl_wait() must be independent
// of all earlier work (no read of their outputs, no write at all).  pdl_wait() returns when the
// preceding kernels have completed and their writes are visible; pdl_launch_dependents() lets the
// NEXT kernel begin its own independent part.  Without the launch attribute both are no-ops.
namespace dinfer {
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// the usual opening of a kernel with nothing to do ahead of its inputs
__device__ __forceinline__ void pdl_enter() { pdl_launch_dependents(); pdl_wait(); }

// `cluster`: thread-block cluster dimensions (all 1 = no cluster attribute).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x; attr[n].val.clusterDim.y = cluster.y; attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  // DINFER_NO_PDL=1 (read once) launches without the attribute: a switch for measuring what the overlap buys
  static const bool off = [] { const char* e = getenv("DINFER_NO_PDL"); return e && e[0] == '1'; }();
  if (!off) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr; cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  return launch_pdl_cluster(kernel, grid, block, dim3(1, 1, 1), smem, stream, args...);
}
}  // namespace dinfer

// One of these per library gives Python the text of the last refusal.
#define DINFER_DEFINE_LAST_ERROR() \
  DINFER_API const char* dinfer_last_error() { return dinfer::error_buffer(); }

// Call `expr` with T bound to the element type that `code` names.
#define DINFER_DISPATCH_DTYPE(code, T, ...)                                  \
  do {                                                                       \
    if ((code) == DINFER_F32) { using T = float; __VA_ARGS__; }              \
    else if ((code) == DINFER_BF16) { using T = __nv_bfloat16; __VA_ARGS__; }\
    else return dinfer::refuse(DINFER_BAD_DTYPE, "unknown dtype code %d", (int)(code)); \
  } while (0)
