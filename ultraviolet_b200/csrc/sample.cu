// Fused softcap + sampling + behaviour log-prob over the raw LM-head output, one CTA per sequence.
//
//   z = a * sigmoid((x + b) / c)                      softcap (MathLM.logits, ultraviolet/model.py:824-827)
//   T <= 0 : token = argmax z (first index on ties)    sample(), ultraviolet/model.py:1197-1198
//   T  > 0 : e = exp((z - a) / T); token = first index whose running sum of e reaches (1 - u) * sum(e)
//            (the inverse-CDF draw of fused_sample, ultraviolet/kernels/fused_sample.py:31-58); with top_p < 1 the
//            draw is restricted to the nucleus of sample() (model.py:1203-1208): tokens whose strictly-larger mass
//            is below top_p, ties with the cut kept; with top_k > 0 only the k largest logits (ties with the k-th
//            kept) take part, and top_p then applies to that renormalised set (model.py:1201-1208)
//   logp   = (z_tok - a) / T - log(sum e)              untruncated softmax, as the rollout log records it
//                                                      (model.py:1160-1169); T <= 0 reports it at T = 1
// u comes from the caller (one uniform per row) or from Philox4x32-10 keyed by (seed; row key, step), so a
// sequence's random stream depends only on its own key and token index, never on the slot or batch it runs in.
#include <stdlib.h>

#include "common.cuh"

namespace uv {

constexpr int SAMPLE_THREADS = 256;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
  c[0] = n0, c[1] = lo1, c[2] = n2, c[3] = lo0;
}
// Philox4x32-10 (Salmon et al., SC'11): counter = (step, row key), key = seed; returns a uniform in [0, 1)
__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t row_key, uint64_t step) {
  uint32_t c[4] = {(uint32_t)step, (uint32_t)(step >> 32), (uint32_t)row_key, (uint32_t)(row_key >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

struct SampleParams {
  const void* x;
  int64_t x_stride;
  int B, V;
  float a, b, c, inv_t, top_p;
  int top_k;  // 0 = no limit
  int greedy;
  int greedy_fast;  // host-decided: the vectorised arg-max path (needs no shared memory: launched with none)
  int plain_fast;   // host-decided: T > 0 without top-k / top-p over 16-bit logits: the draw without shared memory
  int precapped;  // input rows are already softcapped logits z (sample(), model.py:1194-1211); a = row maximum
  const float* u;
  uint64_t seed;
  const int64_t* row_keys;
  const int64_t* steps;
  int64_t* tok;
  float* logp;
  int64_t* inc_a;  // optional per-row counters advanced by one after the draw (cache position, Philox step)
  int64_t* inc_b;
};

__device__ __forceinline__ float block_sum(float v, float* red, int tid) {
  v = warp_sum(v);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += red[w];
  return t;
}

template <typename T>
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const __grid_constant__ SampleParams P) {
  extern __shared__ float e_sm[];  // V + V/CH floats: chunk t of CH values starts at t * (CH + 1) (bank skew)
  __shared__ float red[SAMPLE_THREADS / 32];
  __shared__ float red_v[SAMPLE_THREADS / 32];
  __shared__ int red_i[SAMPLE_THREADS / 32];
  __shared__ float scan_w[SAMPLE_THREADS / 32];
  __shared__ int s_tok;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int row = blockIdx.x;
  const int V = P.V, CH = V / SAMPLE_THREADS;
  // chunk index of element i: a shift when CH is a power of two (every vocabulary in use), else a division
  const int ch_shift = (CH & (CH - 1)) == 0 ? 31 - __clz(CH) : -1;
  auto chunk_of = [&](int i) { return ch_shift >= 0 ? i >> ch_shift : i / CH; };
  pdl_wait();
  pdl_trigger();
  const T* xr = static_cast<const T*>(P.x) + (int64_t)row * P.x_stride;
  const float inv_c = 1.0f / P.c;
  float cap_a = P.a;
  auto zof = [&](int i) {
    const float x = to_f32<T>(xr[i]);
    return P.precapped ? x : __fdividef(P.a, 1.0f + __expf(-(x + P.b) * inv_c));
  };
  if (P.precapped) {  // no analytic bound on z: take the row maximum as the reference point of the exponentials
    float m = -INFINITY;
    for (int i = tid; i < V; i += SAMPLE_THREADS) m = fmaxf(m, to_f32<T>(xr[i]));
    m = warp_max(m);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < SAMPLE_THREADS / 32; ++w) m = fmaxf(m, red[w]);
    cap_a = m;
    __syncthreads();
  }

  if constexpr (sizeof(T) == 2)
  if (P.greedy_fast) {
    // greedy over the softcap: no cumulative sums needed, so nothing is parked in shared memory -- one vectorised
    // pass (8 values per 16-byte load) for the arg-max and the normaliser of the log-prob
    float best = -INFINITY, sum = 0.f;
    int best_i = 0x7fffffff;
    constexpr int UN = 4;  // 16-byte loads in flight per thread: the row is read in two round trips, not eight
    for (int i0 = tid * 8; i0 < V; i0 += SAMPLE_THREADS * 8 * UN) {
      uint4 u4[UN];
#pragma unroll
      for (int j = 0; j < UN; ++j) {
        const int i = i0 + j * SAMPLE_THREADS * 8;
        if (i < V) u4[j] = *reinterpret_cast<const uint4*>(xr + i);
      }
#pragma unroll
      for (int j = 0; j < UN; ++j) {
        const int i = i0 + j * SAMPLE_THREADS * 8;
        if (i >= V) break;
        const T* v = reinterpret_cast<const T*>(&u4[j]);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float z = __fdividef(P.a, 1.0f + __expf(-(to_f32<T>(v[k]) + P.b) * inv_c));
          if (z > best) best = z, best_i = i + k;
          sum += __expf((z - P.a) * P.inv_t);
        }
      }
    }
    const float S_all = block_sum(sum, red, tid);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) best = ob, best_i = oi;
    }
    if (lane == 0) red_v[warp] = best, red_i[warp] = best_i;
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
        if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) best = red_v[w], best_i = red_i[w];
      P.tok[row] = best_i;
      P.logp[row] = (best - P.a) * P.inv_t - logf(S_all);
      if (P.inc_a) P.inc_a[row] += 1;
      if (P.inc_b) P.inc_b[row] += 1;
    }
    return;
  }

  if constexpr (sizeof(T) == 2)
  if (P.plain_fast) {
    // T > 0, no truncation: nothing is parked in shared memory.  Element i belongs to (slab k, thread t, j) with
    // i = k * 2048 + t * 8 + j, so index order is slab-major, then thread, then j.  Pass 1 keeps one partial sum per
    // slab in registers (coalesced 16-byte loads); one batched block reduction gives every slab's sum; the slab that
    // holds the target is re-read (it sits in L2), scanned over the threads in order, and the owning thread walks its
    // eight values.  Same rule as the general path: first index whose running sum reaches (1 - u) * S.
    constexpr int SLAB = SAMPLE_THREADS * 8, KMAX = 24;   // V <= 49152
    __shared__ float slab_w[SAMPLE_THREADS / 32][KMAX];
    __shared__ float slab_s[KMAX];
    const int nslab = V / SLAB;
    float part[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; ++k) part[k] = 0.f;
    auto e8 = [&](const uint4& u4, float (&e)[8]) {
      const T* v = reinterpret_cast<const T*>(&u4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float z = __fdividef(P.a, 1.0f + __expf(-(to_f32<T>(v[j]) + P.b) * inv_c));
        e[j] = __expf((z - P.a) * P.inv_t);
      }
    };
#pragma unroll
    for (int k0 = 0; k0 < KMAX; k0 += 4) {
      uint4 u4[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (k0 + q < nslab) u4[q] = *reinterpret_cast<const uint4*>(xr + (k0 + q) * SLAB + tid * 8);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (k0 + q < nslab) {
          float e[8];
          e8(u4[q], e);
          part[k0 + q] = ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
        }
    }
#pragma unroll
    for (int k = 0; k < KMAX; ++k)
      if (k < nslab) {
        const float w = warp_sum(part[k]);
        if (lane == 0) slab_w[warp][k] = w;
      }
    if (tid == 0) s_tok = V - 1;
    __syncthreads();
    if (tid < nslab) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SAMPLE_THREADS / 32; ++w) t += slab_w[w][tid];
      slab_s[tid] = t;
    }
    __syncthreads();
    float S_all = 0.f;
    for (int k = 0; k < nslab; ++k) S_all += slab_s[k];
    const float u = P.u ? P.u[row] : philox_uniform(P.seed, (uint64_t)P.row_keys[row], (uint64_t)P.steps[row]);
    const float target = (1.0f - u) * S_all;
    int ks = nslab - 1;
    float base = 0.f, run = 0.f;
    for (int k = 0; k < nslab; ++k) {  // the first slab whose cumulative sum reaches the target (uniform in the CTA)
      if (run + slab_s[k] >= target) {
        ks = k;
        break;
      }
      run += slab_s[k];
    }
    base = run;
    // ---- the slab: per-thread sums in index order, block scan, then the owner's eight values
    float e[8];
    e8(*reinterpret_cast<const uint4*>(xr + ks * SLAB + tid * 8), e);
    const float mine = ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) scan_w[warp] = incl;
    __syncthreads();
    float wbase = 0.f;
    for (int w = 0; w < warp; ++w) wbase += scan_w[w];
    incl += wbase + base;
    const float excl = incl - mine;
    if (excl < target && target <= incl) {
      float cs = excl;
      int found = ks * SLAB + tid * 8 + 7;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        cs += e[j];
        if (cs >= target) {
          found = ks * SLAB + tid * 8 + j;
          break;
        }
      }
      atomicMin(&s_tok, found);
    }
    __syncthreads();
    if (tid == 0) {
      const int t = s_tok;
      P.tok[row] = t;
      P.logp[row] = (zof(t) - P.a) * P.inv_t - logf(S_all);
      if (P.inc_a) P.inc_a[row] += 1;  // every thread read steps[row] before the barrier above
      if (P.inc_b) P.inc_b[row] += 1;
    }
    return;
  }

  // ---- pass 1: softcap, exp, argmax (coalesced reads; e parked in shared memory)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool vec = false;
  if constexpr (sizeof(T) == 2) vec = (reinterpret_cast<uintptr_t>(xr) & 3) == 0 && V % 2 == 0 && CH % 2 == 0;
  if (vec) {
    // 4-byte loads (two values), eight in flight per thread before any of them is used: the stores to shared
    // memory below would otherwise keep the compiler from hoisting the next load over them.  Two values per lane
    // keep the shared-memory stores at a 2-way bank conflict.
    if constexpr (sizeof(T) == 2) {
      constexpr int UN = 8;
      for (int i0 = tid * 2; i0 < V; i0 += SAMPLE_THREADS * 2 * UN) {
        uint32_t w[UN];
#pragma unroll
        for (int j = 0; j < UN; ++j) {
          const int i = i0 + j * SAMPLE_THREADS * 2;
          if (i < V) w[j] = *reinterpret_cast<const uint32_t*>(xr + i);
        }
#pragma unroll
        for (int j = 0; j < UN; ++j) {
          const int i = i0 + j * SAMPLE_THREADS * 2;
          if (i >= V) break;
          const T* v = reinterpret_cast<const T*>(&w[j]);
          float* dst = e_sm + i + chunk_of(i);  // two consecutive entries of one chunk
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float x = to_f32<T>(v[k]);
            const float z = P.precapped ? x : __fdividef(P.a, 1.0f + __expf(-(x + P.b) * inv_c));
            if (z > best) best = z, best_i = i + k;  // ascending per thread: first index wins within a thread
            dst[k] = __expf((z - cap_a) * P.inv_t);
          }
        }
      }
    }
  } else {
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
      const float z = zof(i);
      if (z > best) best = z, best_i = i;  // strided ascending per thread: first index wins within a thread
      e_sm[i + chunk_of(i)] = __expf((z - cap_a) * P.inv_t);
    }
  }
  if (tid == 0) s_tok = V - 1;
  __syncthreads();

  // ---- per-thread contiguous chunk sums and block scan
  float* chunk = e_sm + tid * (CH + 1);
  auto chunk_sum = [&](float cut) {
    float s = 0.f;
    for (int j = 0; j < CH; ++j) {
      const float e = chunk[j];
      s += e >= cut ? e : 0.f;
    }
    return s;
  };
  float mine = chunk_sum(0.f);
  const float S_full = block_sum(mine, red, tid);

  if (P.greedy) {
    // block argmax with first-index ties
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) best = ob, best_i = oi;
    }
    if (lane == 0) red_v[warp] = best, red_i[warp] = best_i;
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
        if (red_v[w] > best || (red_v[w] == best && red_i[w] < best_i)) best = red_v[w], best_i = red_i[w];
      P.tok[row] = best_i;
      P.logp[row] = (best - cap_a) * P.inv_t - logf(S_full);
      if (P.inc_a) P.inc_a[row] += 1;
      if (P.inc_b) P.inc_b[row] += 1;
    }
    return;
  }

  // ---- top-k: the k-th largest e as a float bit pattern = the smallest cut with fewer than k entries above it
  float cut = 0.f, S = S_full;
  if (P.top_k > 0 && P.top_k < V) {
    const float kf = (float)P.top_k;  // counts are exact in fp32 (V < 2^24)
    uint32_t lo = 0u, hi = 0x3f800001u;  // e <= 1: nothing lies above hi; e > 0 (or 0 when it underflowed)
    {
      float n0 = 0.f;
      for (int j = 0; j < CH; ++j) n0 += chunk[j] > 0.f ? 1.f : 0.f;
      if (block_sum(n0, red, tid) < kf) hi = 0u;  // fewer than k non-zero entries: everything stays
    }
    while (hi - lo > 1u) {
      const uint32_t mid = lo + (hi - lo) / 2u;
      const float cm = __uint_as_float(mid);
      float n = 0.f;
      for (int j = 0; j < CH; ++j) n += chunk[j] > cm ? 1.f : 0.f;
      if (block_sum(n, red, tid) < kf) hi = mid;
      else lo = mid;
    }
    cut = __uint_as_float(hi);
    mine = chunk_sum(cut);
    S = block_sum(mine, red, tid);
  }
  // ---- nucleus: smallest cut whose strictly-larger mass (inside the top-k set) is below top_p * S
  if (P.top_p < 1.0f) {
    const float lim = P.top_p * S, cut_k = cut;
    uint32_t lo = 0u, hi = 0x3f800001u;  // mass_above(hi) = 0 < lim always (e <= 1)
    while (hi - lo > 1u) {
      const uint32_t mid = lo + (hi - lo) / 2u;
      const float cm = __uint_as_float(mid);
      float s = 0.f;
      for (int j = 0; j < CH; ++j) {
        const float e = chunk[j];
        s += (e > cm && e >= cut_k) ? e : 0.f;
      }
      const float above = block_sum(s, red, tid);
      if (above < lim) hi = mid;
      else lo = mid;
    }
    cut = fmaxf(__uint_as_float(hi), cut_k);
    mine = chunk_sum(cut);
    S = block_sum(mine, red, tid);
  }

  // ---- inverse CDF: exclusive scan of the chunk sums, then the owning thread walks its chunk
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) scan_w[warp] = incl;
  __syncthreads();
  float base = 0.f;
  for (int w = 0; w < warp; ++w) base += scan_w[w];
  incl += base;
  const float excl = incl - mine;
  float u = P.u ? P.u[row] : philox_uniform(P.seed, (uint64_t)P.row_keys[row], (uint64_t)P.steps[row]);
  const float target = (1.0f - u) * S;
  if (excl < target && target <= incl) {
    float cs = excl;
    int found = tid * CH + CH - 1;
    for (int j = 0; j < CH; ++j) {
      const float e = chunk[j];
      cs += e >= cut ? e : 0.f;
      if (cs >= target && e >= cut) {
        found = tid * CH + j;
        break;
      }
    }
    atomicMin(&s_tok, found);
  }
  __syncthreads();
  if (tid == 0) {
    int t = s_tok;
    if (cut > 0.f && e_sm[t + t / CH] < cut) {  // rounding left the target past the last kept entry
      for (t = V - 1; t > 0 && e_sm[t + t / CH] < cut; --t) {}
    }
    P.tok[row] = t;
    P.logp[row] = (zof(t) - cap_a) * P.inv_t - logf(S_full);
    if (P.inc_a) P.inc_a[row] += 1;  // every thread read steps[row] before the barrier above
    if (P.inc_b) P.inc_b[row] += 1;
  }
}

}  // namespace uv

namespace uv {
static bool plain_fast_disabled() {
  static const bool off = [] {
    const char* v = getenv("UVDECODE_SAMPLE_PLAIN_FAST");  // "0": always the general (shared-memory) path
    return v && v[0] == '0';
  }();
  return off;
}
}  // namespace uv

extern "C" int uv_sample(const void* x, int x_dtype, int64_t x_stride, int B, int V, int precapped, float cap_a,
                         float cap_b, float cap_c, float temperature, float top_p, const float* u, uint64_t seed,
                         const int64_t* row_keys, const int64_t* steps, int64_t* tok_out, float* logp_out,
                         int64_t* inc_a, int64_t* inc_b, void* stream) {
  return uv_sample_topk(x, x_dtype, x_stride, B, V, precapped, cap_a, cap_b, cap_c, temperature, 0, top_p, u, seed,
                        row_keys, steps, tok_out, logp_out, inc_a, inc_b, stream);
}

extern "C" int uv_sample_topk(const void* x, int x_dtype, int64_t x_stride, int B, int V, int precapped, float cap_a,
                              float cap_b, float cap_c, float temperature, int top_k, float top_p, const float* u,
                              uint64_t seed, const int64_t* row_keys, const int64_t* steps, int64_t* tok_out,
                              float* logp_out, int64_t* inc_a, int64_t* inc_b, void* stream) {
  using namespace uv;
  if (B == 0) return UV_OK;
  if (top_k < 0) return UV_ERR_ARG;
  if (!x || !tok_out || !logp_out || B < 0) return UV_ERR_ARG;
  if (V < SAMPLE_THREADS || V % SAMPLE_THREADS || V > 49152) return UV_ERR_SHAPE;
  const bool greedy = !(temperature > 0.f);
  if (!greedy && !u && (!row_keys || !steps)) return UV_ERR_ARG;
  if (!precapped && !(cap_a > 0.f && cap_c > 0.f)) return UV_ERR_ARG;
  if (!precapped && !greedy && cap_a / temperature > 80.f) return UV_ERR_ARG;  // exp((z - a)/T) leaves fp32 range
  if (!(top_p > 0.f)) return UV_ERR_ARG;
  SampleParams P{};
  P.x = x, P.x_stride = x_stride, P.B = B, P.V = V;
  P.a = cap_a, P.b = cap_b, P.c = cap_c;
  P.inv_t = greedy ? 1.0f : 1.0f / temperature;
  P.top_p = top_p, P.top_k = top_k, P.greedy = greedy ? 1 : 0, P.precapped = precapped ? 1 : 0;
  P.u = u, P.seed = seed, P.row_keys = row_keys, P.steps = steps, P.tok = tok_out, P.logp = logp_out;
  P.inc_a = inc_a, P.inc_b = inc_b;
  // greedy over 16-bit logits whose rows start on 16-byte boundaries: one vectorised pass, no shared memory, so
  // more rows are resident per SM
  P.greedy_fast = greedy && !precapped && x_dtype != UV_F32 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                  (x_stride * 2) % 16 == 0 && V % 8 == 0;
  // T > 0 without truncation over 16-bit logits in whole 2048-element slabs: the draw needs no shared memory either
  P.plain_fast = !greedy && !precapped && top_k == 0 && !(top_p < 1.0f) && x_dtype != UV_F32 &&
                 (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (x_stride * 2) % 16 == 0 &&
                 V % (SAMPLE_THREADS * 8) == 0 && V / (SAMPLE_THREADS * 8) <= 24 && !plain_fast_disabled();
  const size_t smem = (P.greedy_fast || P.plain_fast) ? 0 : (size_t)(V + V / (V / SAMPLE_THREADS) + 1) * sizeof(float);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define UV_GO(T)                                                                                              \
  do {                                                                                                        \
    if (smem > 48 * 1024) {                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(sample_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                           (int)smem);                                                        \
      if (e != cudaSuccess) {                                                                                 \
        set_last_cuda_error((int)e);                                                                          \
        return UV_ERR_CUDA;                                                                                   \
      }                                                                                                       \
    }                                                                                                         \
    launch_pdl(sample_kernel<T>, dim3((unsigned)B), dim3(SAMPLE_THREADS), smem, st, P);                       \
  } while (0)
  if (x_dtype == UV_F32) UV_GO(float);
  else if (x_dtype == UV_F16) UV_GO(__half);
  else if (x_dtype == UV_BF16) UV_GO(__nv_bfloat16);
  else return UV_ERR_DTYPE;
#undef UV_GO
  return check_launch();
}
