// Per-head post-processing of the packed QKV projection, shared by uv_qkv_post (its own launch) and uv_qkv_attn
// (the same work done in the prologue of the attention kernel).  One warp per (row b, head slot): slots [0, H) are
// query heads, [H, H+K) key heads, [H+K, H+2K) value heads of qkv (B, (H+2K)*hd).
//   q <- rope(rms_norm(q)); k <- rope(rms_norm(k)); v <- v + 2*sigmoid(xn[:ve_ch] . ve_gate) * value_embed[tok]
// (Attention.qkv, ultraviolet/model.py:302-320), then K and V quantised and appended to the int8 cache at the row's
// slot (kv_write, ultraviolet/kernels/kv_quant.py:26-36; slot rule ultraviolet/kernels/fast_decode.py:292-294).
// Every elementwise result is rounded to the activation dtype where the reference's half-precision ops round.
#pragma once

#include "common.cuh"

namespace uv {

constexpr float RMS_EPS = 1.1920929e-07f;  // torch.finfo(float32).eps: F.rms_norm's default in fp32 opmath

struct QkvPostParams {
  void* qkv;
  const void* xn;            // (B, d) pre-norm activations (value-embedding gate input)
  const int64_t* tok;        // (B,)
  const void* value_embed;   // (vocab, K*hd) or null
  const void* ve_gate;       // (K, ve_ch) or null when the layer has no value embedding
  const float* inv_freq;     // (n_pairs,) or null when the layer is NoPE
  const float* rope_cs;      // optional (B, 2*n_pairs): cos then sin of pos*inv_freq, already rounded to the
                             // activation dtype (uv_embed_norm_rope writes it once per step)
  const int64_t* pos;        // (B,)
  int8_t* k_cache;
  int8_t* v_cache;
  uint16_t* k_scale;
  uint16_t* v_scale;
  const int64_t* row_map;
  int* oob;
  int64_t vocab;
  int B, H, K, d, S, S_alloc, ring, ve_ch, n_pairs;
  // optional: the attention output gate of every query head, 2*sigmoid(xn[b, :gate_ch] . gate_w[head]), computed
  // here (it depends on xn only) so that the attention epilogue loads one float instead of two 128-channel rows
  const void* gate_w;        // (H, gate_ch)
  float* gate_out;           // (B, H)
  int gate_ch;
  // optional, packed prefill: last position of the row's sequence in this launch; ring caches then keep only the
  // newest S positions of a sequence (no two rows of one launch write one slot)
  const int64_t* last_pos;
  // xn holds the UN-normalised residual rows: every warp forms its row's RMS-norm factor itself, scales the raw
  // projection by it (the GEMM ran on the un-normalised rows) and reads normalised gate inputs on the fly
  int xn_raw;
};

// rsqrt(mean(row^2) + eps) of one activation row of d elements (d % 8 == 0, 16-byte aligned rows); full warp
template <typename T>
__device__ __forceinline__ float row_rms_factor(const T* row, int d, int lane) {
  float ss = 0.f;
  // rows of up to 1024 elements: four guarded 16-byte loads per lane, all in flight together
  uint4 u[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = 8 * lane + 256 * j;
    u[j] = i < d ? *reinterpret_cast<const uint4*>(row + i) : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const T* v = reinterpret_cast<const T*>(&u[j]);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float f = to_f32<T>(v[k]);
      ss += f * f;
    }
  }
  for (int i = 8 * lane + 1024; i < d; i += 256) {
    const uint4 w = *reinterpret_cast<const uint4*>(row + i);
    const T* v = reinterpret_cast<const T*>(&w);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float f = to_f32<T>(v[k]);
      ss += f * f;
    }
  }
  return rsqrtf(warp_sum(ss) / (float)d + RMS_EPS);
}

// The head gate of Attention.post (ultraviolet/model.py:330-333) with its rounding points; lane-strided products,
// then a warp sum.  Full warp; every lane returns the gate.
// scaled: gx is the UN-normalised activation row and xs its RMS-norm factor; the normalised value is formed (and
// rounded, as the stored one would be) on the fly.
template <typename T>
__device__ __forceinline__ float head_gate(const T* gx, const T* gw, int gate_ch, int lane, float xs = 1.0f,
                                           bool scaled = false) {
  float acc = 0.f;
  for (int ch = lane; ch < gate_ch; ch += 32) {
    const float xv = scaled ? rnd<T>(to_f32<T>(gx[ch]) * xs) : to_f32<T>(gx[ch]);
    acc += xv * to_f32<T>(gw[ch]);
  }
  acc = rnd<T>(warp_sum(acc));
  return rnd<T>(2.0f * rnd<T>(1.0f / (1.0f + __expf(-acc))));
}

// Host-side argument check + parameter block (shared by the two entry points).
inline int qkv_post_params(QkvPostParams* out, void* qkv, const void* xn, const int64_t* tok, const void* value_embed,
                           const void* ve_gate, const float* inv_freq, const int64_t* pos, int8_t* k_cache,
                           int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale, const int64_t* row_map,
                           int* oob_count, int64_t vocab, int B, int H, int K, int hd, int d, int S, int S_alloc,
                           int ring, int ve_ch, int n_pairs) {
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
  P.pos = pos, P.k_cache = k_cache, P.v_cache = v_cache, P.k_scale = k_scale, P.v_scale = v_scale;
  P.row_map = row_map, P.oob = oob_count;
  P.vocab = vocab, P.B = B, P.H = H, P.K = K, P.d = d, P.S = S, P.S_alloc = S_alloc > S ? S_alloc : S;
  P.ring = ring, P.ve_ch = ve_ch, P.n_pairs = n_pairs;
  *out = P;
  return UV_OK;
}

// x: the slot's raw projection values held by a warp (lane owns elements [lane*E, lane*E + E)), replaced by the
// post-processed values.  Called by a full warp.
// TABLE: the rotation always reads P.rope_cs (the caller checked that it is there), so that no cosf / sinf code
// is compiled into the kernel.
// scaled: P.xn holds the un-normalised activation rows and xs is row b's RMS-norm factor (see head_gate).
template <typename T, int HD, bool TABLE = false>
__device__ __forceinline__ void qkv_post_compute(const QkvPostParams& P, int b, int hs, int lane,
                                                 float (&x)[HD >= 32 ? HD / 32 : 1], float xs = 1.0f,
                                                 bool scaled = false) {
  constexpr int E = HD >= 32 ? HD / 32 : 1;
  const bool act = lane * E < HD;
  if (hs >= P.H + P.K) {
    if (P.ve_gate != nullptr) {
      const int kh = hs - P.H - P.K;
      const T* xr = static_cast<const T*>(P.xn) + (int64_t)b * P.d;
      const T* gw = static_cast<const T*>(P.ve_gate) + (int64_t)kh * P.ve_ch;
      // the embedding row hangs off the token id (two dependent loads): started before the gate's reduction
      int64_t t = P.tok[b];
      if (t < 0 || t >= P.vocab) t = 0;
      const T* ve = static_cast<const T*>(P.value_embed) + (t * P.K + kh) * HD;
      float vev[E];
#pragma unroll
      for (int i = 0; i < E; ++i) vev[i] = act ? to_f32<T>(ve[lane * E + i]) : 0.f;
      float acc = 0.f;
      for (int ch = lane; ch < P.ve_ch; ch += 32) {
        const float xv = scaled ? rnd<T>(to_f32<T>(xr[ch]) * xs) : to_f32<T>(xr[ch]);
        acc += xv * to_f32<T>(gw[ch]);
      }
      acc = rnd<T>(warp_sum(acc));
      const float g = rnd<T>(2.0f * rnd<T>(1.0f / (1.0f + __expf(-acc))));
#pragma unroll
      for (int i = 0; i < E; ++i)
        if (act) x[i] = rnd<T>(x[i] + rnd<T>(g * vev[i]));
    }
    return;
  }
  // the rotation's table entries do not depend on x: requested before the norm's reduction, not after it
  float cs_pre[E], sn_pre[E];
  const bool table = P.inv_freq != nullptr && (TABLE || P.rope_cs != nullptr);
#pragma unroll
  for (int i = 0; i < E; ++i) {
    cs_pre[i] = 1.f, sn_pre[i] = 0.f;
    const int dim = lane * E + i;
    if (table && dim < 2 * P.n_pairs) {
      const int j = dim < P.n_pairs ? dim : dim - P.n_pairs;
      cs_pre[i] = P.rope_cs[(int64_t)b * 2 * P.n_pairs + j];
      sn_pre[i] = P.rope_cs[(int64_t)b * 2 * P.n_pairs + P.n_pairs + j];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < E; ++i) ss += x[i] * x[i];
  const float inv = rsqrtf(warp_sum(ss) / (float)HD + RMS_EPS);
#pragma unroll
  for (int i = 0; i < E; ++i) x[i] = rnd<T>(x[i] * inv);
  if (P.inv_freq != nullptr) {
    // half-split pairing: dim j < n_pairs rotates with dim j + n_pairs (apply_rope, model.py:219-226)
    const int pl = P.n_pairs / E;  // lanes holding x1
    const float pf = table ? 0.f : (float)P.pos[b];
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, x[i], pl);
      const int dim = lane * E + i;
      if (dim < 2 * P.n_pairs) {
        const int j = dim < P.n_pairs ? dim : dim - P.n_pairs;
        float cs, sn;
        if (table) {
          cs = cs_pre[i], sn = sn_pre[i];
        } else {
          const float th = pf * P.inv_freq[j];
          cs = rnd<T>(cosf(th)), sn = rnd<T>(sinf(th));
        }
        // x1' = x1*c - x2*s ; x2' = x1*s + x2*c, each product and the sum rounded
        x[i] = dim < P.n_pairs ? rnd<T>(rnd<T>(x[i] * cs) - rnd<T>(other * sn))
                               : rnd<T>(rnd<T>(other * sn) + rnd<T>(x[i] * cs));
      }
    }
  }
}

// Store a quantised key / value slot (lane owns bytes [lane*E, lane*E + E)) and its scale at the cache row of batch
// entry b.  Full warp.
// Where batch entry b's key / value lands: its position, its cache row and (packed prefill) the last position of its
// sequence -- three independent loads a caller can request early and hand to qkv_post_store.
struct QkvSlot {
  int64_t pos, row, last;
};
__device__ __forceinline__ QkvSlot qkv_post_slot(const QkvPostParams& P, int b) {
  QkvSlot q;
  q.pos = P.pos[b];
  q.row = P.row_map ? P.row_map[b] : b;
  q.last = (P.ring && P.last_pos != nullptr) ? P.last_pos[b] : -1;
  return q;
}

template <int HD>
__device__ __forceinline__ void qkv_post_store(const QkvPostParams& P, int b, int hs, int lane,
                                               const int8_t (&q8)[HD >= 32 ? HD / 32 : 1], uint16_t s,
                                               const QkvSlot* pre = nullptr) {
  constexpr int E = HD >= 32 ? HD / 32 : 1;
  const bool act = lane * E < HD;
  const bool isv = hs >= P.H + P.K;
  const int kh = isv ? hs - P.H - P.K : hs - P.H;
  const QkvSlot sl = pre ? *pre : qkv_post_slot(P, b);
  int64_t p = sl.pos;
  if (P.ring) {
    if (sl.last >= 0 && p + P.S <= sl.last) return;  // a newer token of this launch owns the slot
    p = ((p % P.S) + P.S) % P.S;
  }
  if (p < 0 || p >= P.S) {
    if (lane == 0 && P.oob) atomicAdd(P.oob, 1);
    return;
  }
  const int64_t cb = sl.row;
  const int64_t dst = (cb * P.K + kh) * P.S_alloc + p;  // rows may be allocated longer than S
  int8_t* crow = (isv ? P.v_cache : P.k_cache) + dst * HD;
  if (act) {
    if constexpr (E == 4) *reinterpret_cast<char4*>(crow + lane * 4) = make_char4(q8[0], q8[1], q8[2], q8[3]);
    else if constexpr (E == 2) *reinterpret_cast<char2*>(crow + lane * 2) = make_char2(q8[0], q8[1]);
    else crow[lane] = q8[0];
  }
  if (lane == 0) (isv ? P.v_scale : P.k_scale)[dst] = s;
}

// Quantise a post-processed key / value slot and append it to the cache row of batch entry b.  Full warp.
template <typename T, int HD>
__device__ __forceinline__ void qkv_post_append(const QkvPostParams& P, int b, int hs, int lane,
                                                const float (&x)[HD >= 32 ? HD / 32 : 1],
                                                const QkvSlot* pre = nullptr) {
  constexpr int E = HD >= 32 ? HD / 32 : 1;
  int8_t q8[E];
  const uint16_t s = quantize_lane<E>(x, q8);
  qkv_post_store<HD>(P, b, hs, lane, q8, s, pre);
}

}  // namespace uv
