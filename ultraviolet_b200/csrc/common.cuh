// Shared device/host helpers for libuvdecode (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/uvdecode.h"

namespace uv {

// ---- per-thread last CUDA error, surfaced through uv_last_cuda_error()
void set_last_cuda_error(int e);

inline int check_launch() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_last_cuda_error((int)e);
    return UV_ERR_CUDA;
  }
  return UV_OK;
}

// ---- programmatic dependent launch: a kernel launched through launch_pdl may be scheduled while its predecessor
// on the stream is still draining; it must call pdl_wait() before it touches anything the predecessor wrote (or
// writes anything the predecessor reads).  pdl_trigger() lets the successor start being scheduled.  Both are no-ops
// for ordinary launches.  The launch attribute is opt-in: UVDECODE_PDL=1 in the environment turns it on.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr, cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);  // errors surface through check_launch()
}

// launch_pdl plus a thread-block cluster shape (cluster.x * y * z == 1: no cluster attribute)
// (pdl: -1 = the process-wide setting, 0 / 1 = this launch without / with the attribute)
template <typename... KArgs, typename... Args>
inline void launch_cluster_pdl(int pdl, void (*kern)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                               cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = (pdl < 0 ? pdl_enabled() : pdl != 0) ? 1 : 0;
  int n = 1;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster.x, attr[1].val.clusterDim.y = cluster.y, attr[1].val.clusterDim.z = cluster.z;
    n = 2;
  }
  cfg.attrs = attr, cfg.numAttrs = n;
  cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline void launch_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t st,
                           Args... args) {
  launch_cluster_pdl(-1, kern, grid, block, cluster, smem, st, args...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- element conversion
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// round-trip through the activation dtype: the reference rounds after every elementwise op in half precision
template <typename T> __device__ __forceinline__ float rnd(float x) { return to_f32<T>(from_f32<T>(x)); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One (row, head) vector -> int8 + fp16 scale, bit-exact with the reference quantiser
// (ultraviolet/kernels/kv_quant.py:12-19).  Called by a full warp; lane i owns elements [i*E, i*E + E) where
// E = max(1, hd / 32); lanes beyond hd / E pass zeros.  Returns the fp16 scale bits; q[] holds the lane's bytes.
template <int E>
__device__ __forceinline__ uint16_t quantize_lane(const float (&x)[E], int8_t (&q)[E]) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(x[i]));
  amax = warp_max(amax);
  const __half s16 = __float2half_rn(__fdiv_rn(amax, 127.0f));
  const float sf = fmaxf(__half2float(s16), 1e-30f);
#pragma unroll
  for (int i = 0; i < E; ++i) {
    float r = rintf(__fdiv_rn(x[i], sf));
    r = fminf(fmaxf(r, -127.0f), 127.0f);
    q[i] = (int8_t)__float2int_rn(r);
  }
  return __half_as_ushort(s16);
}

}  // namespace uv
