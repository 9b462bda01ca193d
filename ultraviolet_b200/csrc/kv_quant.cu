// Fused KV quantise + append (per-token-per-head symmetric int8, fp16 scales).
// One warp owns one (row, kv head) vector: max-reduce by shuffles, exact fp32 division by the fp16-rounded scale,
// packed byte stores.  K and V of a decode step go through one launch.
#include "common.cuh"

namespace uv {

template <typename T, int E>
__device__ __forceinline__ void load_vec(const T* __restrict__ src, int lane, int hd, float (&x)[E]) {
  const int base = lane * E;
#pragma unroll
  for (int i = 0; i < E; ++i) x[i] = (base + i < hd) ? to_f32<T>(src[base + i]) : 0.f;
}

template <int E>
__device__ __forceinline__ void store_q(int8_t* __restrict__ dst, int lane, int hd, const int8_t (&q)[E]) {
  const int base = lane * E;
  if (base >= hd) return;
  if constexpr (E == 4) {
    *reinterpret_cast<char4*>(dst + base) = make_char4(q[0], q[1], q[2], q[3]);
  } else if constexpr (E == 2) {
    *reinterpret_cast<char2*>(dst + base) = make_char2(q[0], q[1]);
  } else {
#pragma unroll
    for (int i = 0; i < E; ++i) dst[base + i] = q[i];
  }
}

// Generic scatter: row i -> cache row idx[i] (identity when idx == nullptr).
template <typename T, int E>
__global__ void __launch_bounds__(128) kv_quant_scatter_kernel(
    const T* __restrict__ x, int64_t x_stride, int64_t n_rows, int hd, int8_t* __restrict__ cache,
    uint16_t* __restrict__ scale, const int64_t* __restrict__ idx, int64_t n_cache_rows, int* __restrict__ oob) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float v[E];
  int8_t q[E];
  load_vec<T, E>(x + row * x_stride, lane, hd, v);
  const uint16_t s = quantize_lane<E>(v, q);
  const int64_t dst = idx ? idx[row] : row;
  if (dst < 0 || dst >= n_cache_rows) {
    if (lane == 0 && oob) atomicAdd(oob, 1);
    return;
  }
  store_q<E>(cache + dst * hd, lane, hd, q);
  if (lane == 0) scale[dst] = s;
}

// Decode-time append: warp w of the grid handles (b, h, which) with which = 0 (K) / 1 (V).
template <typename T, int E>
__global__ void __launch_bounds__(128) kv_append_kernel(
    const T* __restrict__ k_new, const T* __restrict__ v_new, int64_t k_stride, int64_t v_stride,
    int8_t* __restrict__ k_cache, int8_t* __restrict__ v_cache, uint16_t* __restrict__ k_scale,
    uint16_t* __restrict__ v_scale, const int64_t* __restrict__ pos, int n_bk, int KH, int hd, int S, int ring,
    int* __restrict__ oob) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (item >= 2 * n_bk) return;
  const int which = item & 1;
  const int bk = item >> 1;
  const int b = bk / KH;
  int64_t p = pos[b];
  if (ring) p = ((p % S) + S) % S;
  float v[E];
  int8_t q[E];
  const T* src = which ? v_new + (int64_t)bk * v_stride : k_new + (int64_t)bk * k_stride;
  load_vec<T, E>(src, lane, hd, v);
  const uint16_t s = quantize_lane<E>(v, q);
  if (p < 0 || p >= S) {
    if (lane == 0 && oob) atomicAdd(oob, 1);
    return;
  }
  const int64_t dst = (int64_t)bk * S + p;
  store_q<E>((which ? v_cache : k_cache) + dst * hd, lane, hd, q);
  if (lane == 0) (which ? v_scale : k_scale)[dst] = s;
}

template <typename T>
static int launch_scatter(const void* x, int64_t x_stride, int64_t n_rows, int hd, int8_t* cache, uint16_t* scale,
                          const int64_t* idx, int64_t n_cache_rows, int* oob, cudaStream_t st) {
  const unsigned grid = (unsigned)((n_rows + 3) / 4);
  const T* xp = static_cast<const T*>(x);
#define UV_GO(E) kv_quant_scatter_kernel<T, E><<<grid, 128, 0, st>>>(xp, x_stride, n_rows, hd, cache, scale, idx, \
                                                                    n_cache_rows, oob)
  if (hd <= 32) UV_GO(1);
  else if (hd <= 64) UV_GO(2);
  else if (hd <= 128) UV_GO(4);
  else UV_GO(8);
#undef UV_GO
  return check_launch();
}

template <typename T>
static int launch_append(const void* k_new, const void* v_new, int64_t ks, int64_t vs, int8_t* kc, int8_t* vc,
                         uint16_t* ksc, uint16_t* vsc, const int64_t* pos, int B, int KH, int hd, int S, int ring,
                         int* oob, cudaStream_t st) {
  const int n_bk = B * KH;
  const unsigned grid = (unsigned)((2 * n_bk + 3) / 4);
  const T* kp = static_cast<const T*>(k_new);
  const T* vp = static_cast<const T*>(v_new);
#define UV_GO(E) kv_append_kernel<T, E><<<grid, 128, 0, st>>>(kp, vp, ks, vs, kc, vc, ksc, vsc, pos, n_bk, KH, hd, S, \
                                                             ring, oob)
  if (hd <= 32) UV_GO(1);
  else if (hd <= 64) UV_GO(2);
  else if (hd <= 128) UV_GO(4);
  else UV_GO(8);
#undef UV_GO
  return check_launch();
}

}  // namespace uv

extern "C" int uv_kv_quant_scatter(const void* x, int x_dtype, int64_t x_stride, int64_t n_rows, int hd,
                                   int8_t* cache, uint16_t* scale, const int64_t* flat_idx, int64_t n_cache_rows,
                                   int* oob_count, void* stream) {
  if (n_rows == 0) return UV_OK;
  if (!x || !cache || !scale || n_rows < 0 || n_cache_rows < 0) return UV_ERR_ARG;
  if (hd < 1 || hd > 256) return UV_ERR_SHAPE;
  if (hd > 32 && hd % (hd <= 64 ? 2 : hd <= 128 ? 4 : 8)) return UV_ERR_SHAPE;
  if (hd > 32 && (reinterpret_cast<uintptr_t>(cache) % (hd <= 64 ? 2 : 4))) return UV_ERR_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (x_dtype) {
    case UV_F32: return uv::launch_scatter<float>(x, x_stride, n_rows, hd, cache, scale, flat_idx, n_cache_rows,
                                                  oob_count, st);
    case UV_F16: return uv::launch_scatter<__half>(x, x_stride, n_rows, hd, cache, scale, flat_idx, n_cache_rows,
                                                   oob_count, st);
    case UV_BF16: return uv::launch_scatter<__nv_bfloat16>(x, x_stride, n_rows, hd, cache, scale, flat_idx,
                                                          n_cache_rows, oob_count, st);
    default: return UV_ERR_DTYPE;
  }
}

extern "C" int uv_kv_append(const void* k_new, const void* v_new, int dtype, int64_t k_stride, int64_t v_stride,
                            int8_t* k_cache, int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale,
                            const int64_t* pos, int B, int KH, int hd, int S, int ring, int* oob_count,
                            void* stream) {
  if (B == 0) return UV_OK;
  if (!k_new || !v_new || !k_cache || !v_cache || !k_scale || !v_scale || !pos || B < 0 || KH < 1 || S < 1)
    return UV_ERR_ARG;
  if (hd < 1 || hd > 256) return UV_ERR_SHAPE;
  if (hd > 32 && hd % (hd <= 64 ? 2 : hd <= 128 ? 4 : 8)) return UV_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case UV_F32: return uv::launch_append<float>(k_new, v_new, k_stride, v_stride, k_cache, v_cache, k_scale,
                                                 v_scale, pos, B, KH, hd, S, ring, oob_count, st);
    case UV_F16: return uv::launch_append<__half>(k_new, v_new, k_stride, v_stride, k_cache, v_cache, k_scale,
                                                  v_scale, pos, B, KH, hd, S, ring, oob_count, st);
    case UV_BF16: return uv::launch_append<__nv_bfloat16>(k_new, v_new, k_stride, v_stride, k_cache, v_cache,
                                                         k_scale, v_scale, pos, B, KH, hd, S, ring, oob_count, st);
    default: return UV_ERR_DTYPE;
  }
}
