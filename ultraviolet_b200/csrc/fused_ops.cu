// Fused row-wise kernels of one decode step (everything between the GEMMs):
//   uv_embed_norm     token embedding gather + the two RMS norms that open the step
//   uv_qkv_post       value-embedding gate, per-head QK RMS norm, partial RoPE, int8 quantise + cache append
//   uv_resid_norm     lambda-weighted residual add + RMS norm (output feeds the next GEMM)
//   uv_swiglu         silu(gate) * up
// All of them keep the reference's rounding points: every elementwise result is rounded to the activation dtype
// where the reference's half-precision torch ops round (ultraviolet/kernels/fast_decode.py:272-334,
// ultraviolet/model.py:302-320, :567-571, :388-391), norms accumulate in fp32 with eps = 2^-23.
#include <stdlib.h>

#include "common.cuh"
#include "qkv_post.cuh"

namespace uv {

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
                                                         int B, const int64_t* __restrict__ pos,
                                                         const float* __restrict__ inv_freq, int n_pairs,
                                                         float* __restrict__ rope_cs, float* __restrict__ ss_out,
                                                         int ss_parts, int ss_ld) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (row >= B) return;
  if (rope_cs != nullptr) {
    // the step's RoPE table: cos / sin of pos * inv_freq rounded to T, as apply_rope's operands are
    // (fast_decode.py:286-290); every layer's q / k rotation reads it instead of evaluating cosf / sinf
    const float pf = (float)pos[row];
    for (int j = lane; j < n_pairs; j += 32) {
      const float th = pf * inv_freq[j];
      rope_cs[(int64_t)row * 2 * n_pairs + j] = rnd<T>(cosf(th));
      rope_cs[(int64_t)row * 2 * n_pairs + n_pairs + j] = rnd<T>(sinf(th));
    }
  }
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
  ss = warp_sum(ss);
  if (ss_out != nullptr && lane < ss_parts) {
    // the row's sum of squares in the per-tile form the tensor-core GEMMs read (deferred RMS norm): all of it in
    // part 0, zeros in the others
    ss_out[(int64_t)lane * ss_ld + row] = lane == 0 ? ss : 0.f;
  }
  inv = rsqrtf(ss / (float)d + RMS_EPS);
#pragma unroll
  for (int j = 0; j < ROW_J; ++j) {
    const int i = 8 * lane + 256 * j;
    if (i < d) {
      st8<T>(x + (int64_t)row * d + i, v[j]);
      if (xn != nullptr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[j][k] *= inv;
        st8<T>(xn + (int64_t)row * d + i, v[j]);
      }
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

// act = silu(g) * u of the gate|up projection of UN-normalised rows h: [g | u] = (h . W^T) * rs with
// rs = rsqrt(mean(h^2) + eps) formed here.  A row is cut over SWR_SPLIT CTAs of SWR_THREADS threads (each re-forms rs
// from the 1-2 KB row: cheaper than one long CTA per row).  Every thread first requests everything it will need -- its
// 16-byte pieces of h and of g and u -- so the sum of squares and the projection arrive in one round trip.
constexpr int SWR_THREADS = 64;
constexpr int SWR_SPLIT = 4;
constexpr int SWR_HV = 2;     // 16-byte pieces of h per thread: d <= 8 * 64 * 2 = 1024 without the tail loop
constexpr int SWR_VMAX = 2;   // 8-feature vectors per thread: f <= 8 * 64 * 2 * SWR_SPLIT = 4096 on this path

template <typename T>
__global__ void __launch_bounds__(SWR_THREADS) swiglu_rs_kernel(const T* __restrict__ gu, const T* __restrict__ hrow,
                                                                int d, int f, T* __restrict__ act) {
  __shared__ float red[SWR_THREADS / 32];
  const int row = blockIdx.x / SWR_SPLIT, part = blockIdx.x % SWR_SPLIT;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  pdl_trigger();
  const T* hr = hrow + (int64_t)row * d;
  const T* g = gu + (int64_t)row * 2 * f;
  const int nvec = f / 8;
  const int per = (nvec + SWR_SPLIT - 1) / SWR_SPLIT, v0 = part * per;
  const int v1 = v0 + per < nvec ? v0 + per : nvec;
  float hv[SWR_HV][8], gv[SWR_VMAX][8], uv[SWR_VMAX][8];
  // all loads first
#pragma unroll
  for (int j = 0; j < SWR_HV; ++j) {
    const int i = 8 * (tid + j * SWR_THREADS);
    if (i < d) {
      ld8<T>(hr + i, hv[j]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) hv[j][k] = 0.f;
    }
  }
#pragma unroll
  for (int j = 0; j < SWR_VMAX; ++j) {
    const int v = v0 + tid + j * SWR_THREADS;
    if (v < v1) {
      ld8<T>(g + 8 * v, gv[j]);
      ld8<T>(g + f + 8 * v, uv[j]);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < SWR_HV; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += hv[j][k] * hv[j][k];
  for (int i = 8 * (tid + SWR_HV * SWR_THREADS); i < d; i += 8 * SWR_THREADS) {  // rows wider than 1024 elements
    float more[8];
    ld8<T>(hr + i, more);
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += more[k] * more[k];
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < SWR_THREADS / 32; ++w) tot += red[w];
  const float rs = rsqrtf(tot / (float)d + RMS_EPS);
#pragma unroll
  for (int j = 0; j < SWR_VMAX; ++j) {
    const int v = v0 + tid + j * SWR_THREADS;
    if (v < v1) {
      float o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float g0 = rnd<T>(gv[j][k] * rs), u0 = rnd<T>(uv[j][k] * rs);
        o[k] = rnd<T>(g0 / (1.0f + __expf(-g0))) * u0;
      }
      st8<T>(act + (int64_t)row * f + 8 * v, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------ QKV post
// One warp per (row b, head slot), in place on the packed GEMM output; the arithmetic lives in qkv_post.cuh.
// W warps per CTA, one (row, item) per warp.  COOP (xn_raw launches whose items per row are a multiple of W): the W
// items of a CTA belong to ONE row, whose sum of squares the CTA forms once -- every thread one 16-byte piece -- instead
// of each warp reading the whole row for itself (18 readers per 1.3 KB row otherwise: at a few thousand rows that
// redundant L2 traffic is what the launch costs).
template <typename T, int HD, bool TABLE, int W, bool COOP>
__global__ void __launch_bounds__(W * 32) qkv_post_kernel(const __grid_constant__ QkvPostParams P) {
  constexpr int E = HD >= 32 ? HD / 32 : 1;
  const int lane = threadIdx.x & 31;
  const int slots = P.H + 2 * P.K;
  const int per_row = slots + (P.gate_out ? P.H : 0);  // head slots, then one gate item per query head
  const int item = blockIdx.x * W + (threadIdx.x >> 5);
  pdl_wait();
  pdl_trigger();
  if (item >= P.B * per_row) return;  // (COOP: the item count is a multiple of W, so this is CTA-uniform)
  const int b = item / per_row, hs = item % per_row;
  const bool raw = P.xn_raw != 0;
  // the slot's own values are requested before the row reduction below needs its loads: one round trip, not two
  const bool act0 = lane * E < HD;
  float x0[E];
  if (hs < slots) {
    const T* vec0 = static_cast<const T*>(P.qkv) + ((int64_t)b * slots + hs) * HD;
#pragma unroll
    for (int i = 0; i < E; ++i) x0[i] = act0 ? to_f32<T>(vec0[lane * E + i]) : 0.f;
  }
  // so is where a key / value slot will land (position, cache row): three more loads off the tail of the chain
  QkvSlot dest{};
  const bool appends = hs >= P.H && hs < slots && P.k_cache != nullptr;
  if (appends) dest = qkv_post_slot(P, b);
  float rs = 1.0f;
  if constexpr (COOP) {
    __shared__ float part[W];
    const uint4* row = reinterpret_cast<const uint4*>(static_cast<const T*>(P.xn) + (int64_t)b * P.d);
    float ss = 0.f;
    for (int p = threadIdx.x; p * 8 < P.d; p += W * 32) {
      const uint4 u = row[p];
      const T* v = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float f = to_f32<T>(v[k]);
        ss += f * f;
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < W; ++w) tot += part[w];
    rs = rsqrtf(tot / (float)P.d + RMS_EPS);
  } else {
    if (raw) rs = row_rms_factor<T>(static_cast<const T*>(P.xn) + (int64_t)b * P.d, P.d, lane);
  }
  if (hs >= slots) {
    const int head = hs - slots;
    const float g = head_gate<T>(static_cast<const T*>(P.xn) + (int64_t)b * P.d,
                                 static_cast<const T*>(P.gate_w) + (int64_t)head * P.gate_ch, P.gate_ch, lane, rs,
                                 raw);
    if (lane == 0) P.gate_out[(int64_t)b * P.H + head] = g;
    return;
  }
  const bool act = lane * E < HD;
  T* vec = static_cast<T*>(P.qkv) + ((int64_t)b * slots + hs) * HD;
  float x[E];
#pragma unroll
  for (int i = 0; i < E; ++i) x[i] = x0[i];
  if (raw) {  // the projection of the un-normalised row, scaled: what the GEMM on the normalised row would hold
#pragma unroll
    for (int i = 0; i < E; ++i) x[i] = rnd<T>(x[i] * rs);
  }
  qkv_post_compute<T, HD, TABLE>(P, b, hs, lane, x, rs, raw);
#pragma unroll
  for (int i = 0; i < E; ++i)
    if (act) vec[lane * E + i] = from_f32<T>(x[i]);
  if (appends) qkv_post_append<T, HD>(P, b, hs, lane, x, &dest);
}

template <typename T>
static int launch_qkv_post(const QkvPostParams& P, int hd, cudaStream_t st) {
  const int per_row = P.H + 2 * P.K + (P.gate_out ? P.H : 0);
  const int64_t items = (int64_t)P.B * per_row;
  // cooperative row reduction when the launch defers the norm and a row's items fill whole CTAs of 6 or 4 warps
  static const bool coop_on = [] {
    const char* v = getenv("UVDECODE_QKV_POST_COOP");
    return !(v && v[0] == '0');
  }();
  const int coop = (P.xn_raw && coop_on) ? (per_row % 6 == 0 ? 6 : (per_row % 4 == 0 ? 4 : 0)) : 0;
  const int wpc = coop ? coop : 4;
  const unsigned grid = (unsigned)((items + wpc - 1) / wpc);
  // with the step's RoPE table the kernel carries no cosf / sinf code at all
#define UV_QKV_POST_W(HD_, TABLE_)                                                                              \
  do {                                                                                                          \
    if (coop == 6) launch_pdl(qkv_post_kernel<T, HD_, TABLE_, 6, true>, dim3(grid), dim3(192), 0, st, P);       \
    else if (coop == 4) launch_pdl(qkv_post_kernel<T, HD_, TABLE_, 4, true>, dim3(grid), dim3(128), 0, st, P);  \
    else launch_pdl(qkv_post_kernel<T, HD_, TABLE_, 4, false>, dim3(grid), dim3(128), 0, st, P);                \
  } while (0)
#define UV_QKV_POST(HD_)                       \
  case HD_:                                    \
    if (P.rope_cs) UV_QKV_POST_W(HD_, true);   \
    else UV_QKV_POST_W(HD_, false);            \
    break;
  switch (hd) {
    UV_QKV_POST(16)
    UV_QKV_POST(32)
    UV_QKV_POST(64)
    UV_QKV_POST(128)
    default: return UV_ERR_SHAPE;
  }
#undef UV_QKV_POST
#undef UV_QKV_POST_W
  return check_launch();
}

}  // namespace uv

using namespace uv;

extern "C" int uv_embed_norm_rope(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x,
                                  void* xn, int B, const int64_t* pos, const float* inv_freq, int n_pairs,
                                  float* rope_cs, void* stream) {
  if (!xn) return B == 0 ? UV_OK : UV_ERR_ARG;
  return uv_embed_norm_ss(tok, embed, dtype, vocab, d, x, xn, B, pos, inv_freq, n_pairs, rope_cs, nullptr, 0, 0,
                          stream);
}

extern "C" int uv_embed_norm_ss(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x,
                                void* xn, int B, const int64_t* pos, const float* inv_freq, int n_pairs,
                                float* rope_cs, float* ss_out, int ss_parts, int ss_ld, void* stream) {
  if (B == 0) return UV_OK;
  if (!tok || !embed || !x || B < 0 || vocab < 1) return UV_ERR_ARG;
  if (!xn && !ss_out) return UV_ERR_ARG;
  if (ss_out && (ss_parts < 1 || ss_parts > 32 || ss_ld < B)) return UV_ERR_ARG;
  if (rope_cs && (!pos || !inv_freq || n_pairs < 1)) return UV_ERR_ARG;
  if (d < 8 || (d & 7) || d > ROW_MAX) return UV_ERR_SHAPE;  // rows are moved as 16-byte vectors
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((B + 3) / 4);
  if (dtype == UV_F16)
    launch_pdl(embed_norm_kernel<__half>, dim3(grid), dim3(128), 0, st, tok, static_cast<const __half*>(embed), vocab,
               d, static_cast<__half*>(x), static_cast<__half*>(xn), B, pos, inv_freq, n_pairs, rope_cs, ss_out, ss_parts,
               ss_ld);
  else if (dtype == UV_BF16)
    launch_pdl(embed_norm_kernel<__nv_bfloat16>, dim3(grid), dim3(128), 0, st, tok,
               static_cast<const __nv_bfloat16*>(embed), vocab, d, static_cast<__nv_bfloat16*>(x),
               static_cast<__nv_bfloat16*>(xn), B, pos, inv_freq, n_pairs, rope_cs, ss_out, ss_parts, ss_ld);
  else return UV_ERR_DTYPE;
  return check_launch();
}

extern "C" int uv_embed_norm(const int64_t* tok, const void* embed, int dtype, int64_t vocab, int d, void* x,
                             void* xn, int B, void* stream) {
  return uv_embed_norm_rope(tok, embed, dtype, vocab, d, x, xn, B, nullptr, nullptr, 0, nullptr, stream);
}

extern "C" int uv_qkv_post_args(const uv_qkv_args* a, void* stream) {
  if (!a) return UV_ERR_ARG;
  if (a->B == 0) return UV_OK;
  QkvPostParams P{};
  const int rc = qkv_post_params(&P, a->qkv, a->xn, a->tok, a->value_embed, a->ve_gate, a->inv_freq, a->pos, a->k_cache,
                                 a->v_cache, a->k_scale, a->v_scale, a->row_map, a->oob_count, a->vocab, a->B, a->H,
                                 a->K, a->hd, a->d, a->S, a->S_alloc, a->ring, a->ve_ch, a->n_pairs);
  if (rc != UV_OK) return rc;
  P.rope_cs = a->inv_freq ? a->rope_cs : nullptr;
  if (a->gate_out) {
    if (!a->gate_w || !a->xn || a->gate_ch < 1 || a->gate_ch > a->d) return UV_ERR_ARG;
    P.gate_w = a->gate_w, P.gate_out = a->gate_out, P.gate_ch = a->gate_ch;
  }
  P.last_pos = a->last_pos;
  if (a->xn_raw) {
    if (!a->xn || a->d < 8 || (a->d & 7) || !aligned16(a->xn)) return UV_ERR_ARG;
    P.xn_raw = 1;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == UV_F16) return launch_qkv_post<__half>(P, a->hd, st);
  if (a->dtype == UV_BF16) return launch_qkv_post<__nv_bfloat16>(P, a->hd, st);
  return UV_ERR_DTYPE;
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

extern "C" int uv_swiglu_rs(const void* gu, const void* h, int dtype, int d, int f, void* act, int B, void* stream) {
  if (B == 0) return UV_OK;
  if (!gu || !h || !act || B < 0) return UV_ERR_ARG;
  if (f < 8 || (f & 7) || f > 8 * SWR_THREADS * SWR_VMAX * SWR_SPLIT || d < 8 || (d & 7)) return UV_ERR_SHAPE;
  if (!aligned16(h) || !aligned16(gu) || !aligned16(act)) return UV_ERR_ALIGN;  // rows move as 16-byte vectors
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_F16)
    launch_pdl(swiglu_rs_kernel<__half>, dim3((unsigned)B * SWR_SPLIT), dim3(SWR_THREADS), 0, st, static_cast<const __half*>(gu),
               static_cast<const __half*>(h), d, f, static_cast<__half*>(act));
  else if (dtype == UV_BF16)
    launch_pdl(swiglu_rs_kernel<__nv_bfloat16>, dim3((unsigned)B * SWR_SPLIT), dim3(SWR_THREADS), 0, st,
               static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(h), d, f,
               static_cast<__nv_bfloat16*>(act));
  else return UV_ERR_DTYPE;
  return check_launch();
}

extern "C" int uv_qkv_post(void* qkv, const void* xn, const int64_t* tok, const void* value_embed,
                           const void* ve_gate, const float* inv_freq, const int64_t* pos, int8_t* k_cache,
                           int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale, const int64_t* row_map,
                           int* oob_count, int dtype, int64_t vocab, int B, int H, int K, int hd, int d, int S,
                           int S_alloc, int ring, int ve_ch, int n_pairs, void* stream) {
  if (B == 0) return UV_OK;
  QkvPostParams P{};
  const int rc = qkv_post_params(&P, qkv, xn, tok, value_embed, ve_gate, inv_freq, pos, k_cache, v_cache, k_scale,
                                 v_scale, row_map, oob_count, vocab, B, H, K, hd, d, S, S_alloc, ring, ve_ch, n_pairs);
  if (rc != UV_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_F16) return launch_qkv_post<__half>(P, hd, st);
  if (dtype == UV_BF16) return launch_qkv_post<__nv_bfloat16>(P, hd, st);
  return UV_ERR_DTYPE;
}
