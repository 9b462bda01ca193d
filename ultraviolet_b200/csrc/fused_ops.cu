// Fused row-wise kernels of one decode step (everything between the GEMMs):
//   uv_embed_norm     token embedding gather + the two RMS norms that open the step
//   uv_qkv_post       value-embedding gate, per-head QK RMS norm, partial RoPE, int8 quantise + cache append
//   uv_resid_norm     lambda-weighted residual add + RMS norm (output feeds the next GEMM)
//   uv_swiglu         silu(gate) * up
// All of them keep the reference's rounding points: every elementwise result is rounded to the activation dtype
// where the reference's half-precision torch ops round (ultraviolet/kernels/fast_decode.py:272-334,
// ultraviolet/model.py:302-320, :567-571, :388-391), norms accumulate in fp32 with eps = 2^-23.
#include "common.cuh"

namespace uv {

constexpr float RMS_EPS = 1.1920929e-07f;  // torch.finfo(float32).eps: F.rms_norm's default in fp32 opmath

template <typename T> struct Vec2;
template <> struct Vec2<__half> { using type = __half2; };
template <> struct Vec2<__nv_bfloat16> { using type = __nv_bfloat162; };

template <typename T> __device__ __forceinline__ float2 ld2(const T* p) {
  typename Vec2<T>::type v = *reinterpret_cast<const typename Vec2<T>::type*>(p);
  return make_float2(to_f32<T>(v.x), to_f32<T>(v.y));
}
template <typename T> __device__ __forceinline__ void st2(T* p, float a, float b) {
  typename Vec2<T>::type v;
  v.x = from_f32<T>(a);
  v.y = from_f32<T>(b);
  *reinterpret_cast<typename Vec2<T>::type*>(p) = v;
}

// ------------------------------------------------------------------------------------------------ embed + norms
// A warp owns a row; rows of up to ROW_MAX elements live in registers as 16-byte vectors (lane owns elements
// 8*lane + 256*j .. +7): one global read and one write per element, three or four memory instructions per lane.
constexpr int ROW_MAX = 1024;
constexpr int ROW_J = ROW_MAX / 256;

template <typename T> __device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const typename Vec2<T>::type* h = reinterpret_cast<const typename Vec2<T>::type*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) v[2 * i] = to_f32<T>(h[i].x), v[2 * i + 1] = to_f32<T>(h[i].y);
}
template <typename T> __device__ __forceinline__ void st8(T* p, const float (&v)[8]) {
  uint4 u;
  typename Vec2<T>::type* h = reinterpret_cast<typename Vec2<T>::type*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i].x = from_f32<T>(v[2 * i]), h[i].y = from_f32<T>(v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// x = rms_norm(embed[tok]); xn = rms_norm(x)   (fast_decode.py:284 and the first layer's pre-norm, :303)
template <typename T>
__global__ void __launch_bounds__(128) embed_norm_kernel(const int64_t* __restrict__ tok, const T* __restrict__ embed,
                                                         int64_t vocab, int d, T* __restrict__ x, T* __restrict__ xn,
                                                         int B) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (row >= B) return;
  int64_t t = tok[row];
  if (t < 0 || t >= vocab) t = 0;  // out-of-range ids read row 0 instead of faulting
  const T* e = embed + t * d;
  float v[ROW_J][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    const int i = 8 * lane + 256 * j;
    if (i < d) {
      ld8<T>(e + i, v[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += v[j][k] * v[j][k];
    }
  }
  float inv = rsqrtf(warp_sum(ss) / (float)d + RMS_EPS);
  ss = 0.f;
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    if (8 * lane + 256 * j < d) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[j][k] = rnd<T>(v[j][k] * inv);
        ss += v[j][k] * v[j][k];
      }
    }
  }
  inv = rsqrtf(warp_sum(ss) / (float)d + RMS_EPS);
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    const int i = 8 * lane + 256 * j;
    if (i < d) {
      st8<T>(x + (int64_t)row * d + i, v[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[j][k] *= inv;
      st8<T>(xn + (int64_t)row * d + i, v[j]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ residual + norm
// h = l0 * x + l1 * a (each product and the sum rounded to T, Block.finish, model.py:567-571); hn = rms_norm(h)
template <typename T>
__global__ void __launch_bounds__(128) resid_norm_kernel(const T* __restrict__ x, const T* __restrict__ a,
                                                         const float* __restrict__ lambdas, int d,
                                                         T* __restrict__ h, T* __restrict__ hn, int B) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (row >= B) return;
  const float l0 = lambdas[0], l1 = lambdas[1];
  const int64_t ro = (int64_t)row * d;
  float v[ROW_J][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    const int i = 8 * lane + 256 * j;
    if (i < d) {
      float xv[8], av[8];
      ld8<T>(x + ro + i, xv);
      ld8<T>(a + ro + i, av);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        v[j][k] = rnd<T>(rnd<T>(l0 * xv[k]) + rnd<T>(l1 * av[k]));
        ss += v[j][k] * v[j][k];
      }
    }
  }
  const float inv = rsqrtf(warp_sum(ss) / (float)d + RMS_EPS);
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    const int i = 8 * lane + 256 * j;
    if (i < d) {
      st8<T>(h + ro + i, v[j]);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[j][k] *= inv;
      st8<T>(hn + ro + i, v[j]);
    }
  }
}

// ------------------------------------------------------------------------------------------------ SwiGLU
// act = silu(g) * u with gu = [g | u] (B, 2f) (MLP.forward fused branch, model.py:388-391)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gu, int f, T* __restrict__ act,
                                                     int64_t n_pairs) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // pair index over (B, f/2)
  pdl_wait();
  pdl_trigger();
  if (i >= n_pairs) return;
  const int half_f = f / 2;
  const int64_t row = i / half_f;
  const int col = (int)(i % half_f) * 2;
  const float2 g = ld2<T>(gu + row * 2 * f + col);
  const float2 u = ld2<T>(gu + row * 2 * f + f + col);
  const float s0 = rnd<T>(g.x / (1.0f + __expf(-g.x))), s1 = rnd<T>(g.y / (1.0f + __expf(-g.y)));
  st2<T>(act + row * f + col, s0 * u.x, s1 * u.y);
}

// ------------------------------------------------------------------------------------------------ QKV post
// One warp per (row b, head slot): slots [0, H) are query heads, [H, H+K) key heads, [H+K, H+2K) value heads of the
// packed GEMM output qkv (B, (H+2K)*hd).  In place: q <- rope(rms_norm(q)); k <- rope(rms_norm(k)); v <- v + ve gate.
// K and V are also quantised and appended to the int8 cache at the row's slot (Attention.qkv, model.py:302-320;
// kv_write, kv_quant.py:26-36; slot rule fast_decode.py:292-294).
struct QkvPostParams {
  void* qkv;
  const void* xn;            // (B, d) pre-norm activations (value-embedding gate input)
  const int64_t* tok;        // (B,)
  const void* value_embed;   // (vocab, K*hd) or null
  const void* ve_gate;       // (K, ve_ch) or null when the layer has no value embedding
  const float* inv_freq;     // (n_pairs,) or null when the layer is NoPE
  const int64_t* pos;        // (B,)
  int8_t* k_cache;
  int8_t* v_cache;
  uint16_t* k_scale;
  uint16_t* v_scale;
  const int64_t* row_map;
  int* oob;
  int64_t vocab;
  int B, H, K, d, S, S_alloc, ring, ve_ch, n_pairs;
};

template <typename T, int HD>
__global__ void __launch_bounds__(128) qkv_post_kernel(const __grid_constant__ QkvPostParams P) {
  constexpr int E = HD >= 32 ? HD / 32 : 1;
  const int lane = threadIdx.x & 31;
  const int slots = P.H + 2 * P.K;
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (item >= P.B * slots) return;
  const int b = item / slots, hs = item % slots;
  const bool act = lane * E < HD;
  T* vec = static_cast<T*>(P.qkv) + ((int64_t)b * slots + hs) * HD;
  float x[E];
#pragma unroll
  for (int i = 0; i < E; ++i) x[i] = act ? to_f32<T>(vec[lane * E + i]) : 0.f;

  const bool is_v = hs >= P.H + P.K;
  if (is_v) {
    if (P.ve_gate != nullptr) {
      const int kh = hs - P.H - P.K;
      const T* xr = static_cast<const T*>(P.xn) + (int64_t)b * P.d;
      const T* gw = static_cast<const T*>(P.ve_gate) + (int64_t)kh * P.ve_ch;
      float acc = 0.f;
      for (int ch = lane; ch < P.ve_ch; ch += 32) acc += to_f32<T>(xr[ch]) * to_f32<T>(gw[ch]);
      acc = rnd<T>(warp_sum(acc));
      const float g = rnd<T>(2.0f * rnd<T>(1.0f / (1.0f + __expf(-acc))));
      int64_t t = P.tok[b];
      if (t < 0 || t >= P.vocab) t = 0;
      const T* ve = static_cast<const T*>(P.value_embed) + (t * P.K + kh) * HD;
#pragma unroll
      for (int i = 0; i < E; ++i)
        if (act) x[i] = rnd<T>(x[i] + rnd<T>(g * to_f32<T>(ve[lane * E + i])));
    }
  } else {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < E; ++i) ss += x[i] * x[i];
    const float inv = rsqrtf(warp_sum(ss) / (float)HD + RMS_EPS);
#pragma unroll
    for (int i = 0; i < E; ++i) x[i] = rnd<T>(x[i] * inv);
    if (P.inv_freq != nullptr) {
      // half-split pairing: dim j < n_pairs rotates with dim j + n_pairs (apply_rope, model.py:219-226)
      const int pl = P.n_pairs / E;  // lanes holding x1
      const float pf = (float)P.pos[b];
#pragma unroll
      for (int i = 0; i < E; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, x[i], pl);
        const int dim = lane * E + i;
        if (dim < 2 * P.n_pairs) {
          const int j = dim < P.n_pairs ? dim : dim - P.n_pairs;
          const float th = pf * P.inv_freq[j];
          const float cs = rnd<T>(cosf(th)), sn = rnd<T>(sinf(th));
          // x1' = x1*c - x2*s ; x2' = x1*s + x2*c, each product and the sum rounded
          x[i] = dim < P.n_pairs ? rnd<T>(rnd<T>(x[i] * cs) - rnd<T>(other * sn))
                                 : rnd<T>(rnd<T>(other * sn) + rnd<T>(x[i] * cs));
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < E; ++i)
    if (act) vec[lane * E + i] = from_f32<T>(x[i]);

  if (hs >= P.H && P.k_cache != nullptr) {  // key or value head: quantise + append
    const bool isv = is_v;
    const int kh = isv ? hs - P.H - P.K : hs - P.H;
    int8_t q8[E];
    const uint16_t s = quantize_lane<E>(x, q8);
    int64_t p = P.pos[b];
    if (P.ring) p = ((p % P.S) + P.S) % P.S;
    if (p < 0 || p >= P.S) {
      if (lane == 0 && P.oob) atomicAdd(P.oob, 1);
      return;
    }
    const int64_t cb = P.row_map ? P.row_map[b] : b;
    const int64_t dst = (cb * P.K + kh) * P.S_alloc + p;  // rows may be allocated longer than S
    int8_t* crow = (isv ? P.v_cache : P.k_cache) + dst * HD;
    if (act) {
      if constexpr (E == 4) *reinterpret_cast<char4*>(crow + lane * 4) = make_char4(q8[0], q8[1], q8[2], q8[3]);
      else if constexpr (E == 2) *reinterpret_cast<char2*>(crow + lane * 2) = make_char2(q8[0], q8[1]);
      else crow[lane] = q8[0];
    }
    if (lane == 0) (isv ? P.v_scale : P.k_scale)[dst] = s;
  }
}

template <typename T>
static int launch_qkv_post(const QkvPostParams& P, int hd, cudaStream_t st) {
  const unsigned grid = (unsigned)(((int64_t)P.B * (P.H + 2 * P.K) + 3) / 4);
  switch (hd) {
    case 16: launch_pdl(qkv_post_kernel<T, 16>, dim3(grid), dim3(128), 0, st, P); break;
    case 32: launch_pdl(qkv_post_kernel<T, 32>, dim3(grid), dim3(128), 0, st, P); break;
    case 64: launch_pdl(qkv_post_kernel<T, 64>, dim3(grid), dim3(128), 0, st, P); break;
    case 128: launch_pdl(qkv_post_kernel<T, 128>, dim3(grid), dim3(128), 0, st, P); break;
    default: return UV_ERR_SHAPE;
  }
  return check_launch();
}

}  // namespace uv

using namespace uv;

extern "C" int uv_embed_norm(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x,
                             void* xn, int B, void* stream) {
  if (B == 0) return UV_OK;
  if (!tok || !embed || !x || !xn || B < 0 || vocab < 1) return UV_ERR_ARG;
  if (d < 8 || (d & 7) || d > ROW_MAX) return UV_ERR_SHAPE;  // rows are moved as 16-byte vectors
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((B + 3) / 4);
  if (dtype == UV_F16)
    launch_pdl(embed_norm_kernel<__half>, dim3(grid), dim3(128), 0, st, tok, static_cast<const __half*>(embed), vocab,
               d, static_cast<__half*>(x), static_cast<__half*>(xn), B);
  else if (dtype == UV_BF16)
    launch_pdl(embed_norm_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, tok,
               static_cast<const __nv_bfloat16*>(embed), vocab, d, static_cast<__nv_bfloat16*>(x),
               static_cast<__nv_bfloat16*>(xn), B);
  else return UV_ERR_DTYPE;
  return check_launch();
}

extern "C" int uv_resid_norm(const void* x, const void* a, const float* lambdas, int dtype, int d, void* h, void* hn,
                             int B, void* stream) {
  if (B == 0) return UV_OK;
  if (!x || !a || !lambdas || !h || !hn || B < 0) return UV_ERR_ARG;
  if (d < 8 || (d & 7) || d > ROW_MAX) return UV_ERR_SHAPE;  // rows are moved as 16-byte vectors
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((B + 3) / 4);
  if (dtype == UV_F16)
    launch_pdl(resid_norm_kernel<__half>, dim3(grid), dim3(128), 0, st, static_cast<const __half*>(x),
               static_cast<const __half*>(a), lambdas, d, static_cast<__half*>(h), static_cast<__half*>(hn), B);
  else if (dtype == UV_BF16)
    launch_pdl(resid_norm_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(x),
               static_cast<const __nv_bfloat16*>(a), lambdas, d, static_cast<__nv_bfloat16*>(h),
               static_cast<__nv_bfloat16*>(hn), B);
  else return UV_ERR_DTYPE;
  return check_launch();
}

extern "C" int uv_swiglu(const void* gu, int dtype, int f, void* act, int B, void* stream) {
  if (B == 0) return UV_OK;
  if (!gu || !act || B < 0) return UV_ERR_ARG;
  if (f < 2 || (f & 1)) return UV_ERR_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n = (int64_t)B * (f / 2);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (dtype == UV_F16)
    launch_pdl(swiglu_kernel<__half>, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(gu), f,
               static_cast<__half*>(act), n);
  else if (dtype == UV_BF16)
    launch_pdl(swiglu_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(gu), f,
               static_cast<__nv_bfloat16*>(act), n);
  else return UV_ERR_DTYPE;
  return check_launch();
}

extern "C" int uv_qkv_post(void* qkv, const void* xn, const int64_t* tok, const void* value_embed,
                           const void* ve_gate, const float* inv_freq, const int64_t* pos, int8_t* k_cache,
                           int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale, const int64_t* row_map,
                           int* oob_count, int dtype, int64_t vocab, int B, int H, int K, int hd, int d, int S,
                           int S_alloc, int ring, int ve_ch, int n_pairs, void* stream) {
  if (B == 0) return UV_OK;
  if (!qkv || !pos || B < 0 || H < 1 || K < 1) return UV_ERR_ARG;
  if (ve_gate && (!xn || !tok || !value_embed || ve_ch < 1)) return UV_ERR_ARG;
  if (k_cache && (!v_cache || !k_scale || !v_scale || S < 1)) return UV_ERR_ARG;
  if (hd != 16 && hd != 32 && hd != 64 && hd != 128) return UV_ERR_SHAPE;
  if (inv_freq) {
    const int E = hd >= 32 ? hd / 32 : 1;
    const int pl = n_pairs / E;
    if (n_pairs < 1 || 2 * n_pairs > hd || n_pairs % E || (pl & (pl - 1))) return UV_ERR_SHAPE;
  }
  QkvPostParams P{};
  P.qkv = qkv, P.xn = xn, P.tok = tok, P.value_embed = value_embed, P.ve_gate = ve_gate, P.inv_freq = inv_freq;
  P.pos = pos, P.k_cache = k_cache, P.v_cache = v_cache, P.k_scale = k_scale, P.v_scale = v_scale, P.row_map = row_map, P.oob = oob_count;
  P.vocab = vocab, P.B = B, P.H = H, P.K = K, P.d = d, P.S = S, P.S_alloc = S_alloc > S ? S_alloc : S, P.ring = ring, P.ve_ch = ve_ch, P.n_pairs = n_pairs;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_F16) return launch_qkv_post<__half>(P, hd, st);
  if (dtype == UV_BF16) return launch_qkv_post<__nv_bfloat16>(P, hd, st);
  return UV_ERR_DTYPE;
}
