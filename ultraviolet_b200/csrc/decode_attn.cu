// Split-K single-query (flash-decode) attention over the slot-indexed int8 KV cache, sm_100a.
//
// Work decomposition: one CTA per (cache row b, kv head h, split).  The row's valid positions [lo, hi] are cut into
// 128-key tiles aligned to multiples of 128 in position space; a split owns a contiguous run of tiles.  Tiles
// stream HBM -> shared memory through the bulk-copy (TMA) engine into a 3-stage ring (cp.async.bulk + mbarrier
// complete_tx), K / V / both scale vectors as four linear copies per tile, trimmed to the row's valid range at
// 8-key granularity; a ring whose length is not a multiple of the tile gets the tile that crosses slot S - 1 as two
// pieces.  Caches whose geometry breaks the 16-byte rules of the bulk engine (row or ring length not a multiple of
// 8 slots, unaligned views) take a two-stage cp.async path with the same shared memory layout.
//
// Math: the G query heads of a kv group form the M rows of warp-level tensor-core tiles.
//   S = Q K^T runs on the int8 pipe (mma.sync.m16n8k32.s8): each query head is split once per CTA into two int8
//   parts (q ~= s1*q1 + s1/254*q2, error <= max|q|/64516) so the cache bytes are the B operand as they are -- no
//   dequantisation of K at all.  With G <= 8 the two parts share one MMA (rows 0..7 / 8..15).
//   O += P V runs on the fp16 pipe (mma.sync.m16n8k16): keys are the N dimension of S, so the score accumulators
//   are already the A fragment of P; int8 V is dequantised in registers (xor 0x80 + byte permute into the mantissa
//   of 1024.0, minus 1152) through a 4x4 byte transpose that rides on the same permutes.
// The per-key K scale multiplies the S columns, the V scale is folded into P.  Head dims are consumed in a permuted
// order that Q shares (dot products are order free) so every lane reads contiguous 16-byte pieces of a key row.
//
// Each of the 4 warps owns 32 keys of every tile with its own online-softmax state (the accumulator is rescaled
// only when a row maximum moves); tiles fully inside [lo, hi] take a mask-free path.  Warp states are merged
// through shared memory with log-sum-exp weights, and splits > 1 are merged by a second small kernel.
#include <mutex>
#include <type_traits>

#include <stdlib.h>

#include "common.cuh"
#include "qkv_post.cuh"

namespace uv {

#ifndef UV_ATTN_TILE
#define UV_ATTN_TILE 128
#endif
#ifndef UV_ATTN_NSTAGE
#define UV_ATTN_NSTAGE 3
#endif
#ifndef UV_ATTN_NWARP
#define UV_ATTN_NWARP 4
#endif
constexpr int TILE = UV_ATTN_TILE;   // keys per pipeline stage
constexpr int NSTAGE = UV_ATTN_NSTAGE;
constexpr int NWARP = UV_ATTN_NWARP;
constexpr int NTHREAD = (NWARP + 1) * 32;  // NWARP consumer warps + one warp that issues the bulk copies
constexpr int WKEYS = TILE / NWARP;  // keys one warp consumes per stage
constexpr unsigned long long WAIT_NS = 200ull * 1000 * 1000;  // a tile that has not landed after 200 ms is abandoned
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_GAP = 6.0f;  // 2^6 * (largest fp16 scale 65504/127) still fits fp16

struct AttnParams {
  const void* q;
  const int8_t* k;
  const int8_t* v;
  const __half* ks;
  const __half* vs;
  const int64_t* pos;
  const int64_t* starts;
  const int64_t* row_map;  // optional: cache row of batch entry b (q / out / pos / starts stay batch-indexed)
  void* out;
  float* ws_o;
  float* ws_m;
  float* ws_l;
  int* status;
  int* counters;  // per (b, kv head) arrival counters for the fused split merge; zero on entry, zero on exit
  int64_t sqb, sqh, skb, skh, sks, svb, svh, svs, ssb, ssh, stb, sth, sob, soh;
  int B, H, KH, G, S, window, ring, splits;
  float scale_log2;
  // fused epilogue
  const void* v_cur;
  int64_t v_cur_sb, v_cur_sh;
  const float* xsa_alpha;
  float xsa_eps;
  const void* gate_x;
  int64_t gate_x_stride;
  const void* gate_w;
  int gate_ch;
  const float* gate_vals;  // (B, H) gates already computed (uv_qkv_post_args): replaces gate_x / gate_w
  int cluster;  // the splits of one cache row form a thread-block cluster and merge through distributed shared memory
  // uv_qkv_attn: the kernel first post-processes the row's raw QKV projection (q / k / v of this step) and appends
  // the new key and value to the cache; q and the current v are then taken from shared memory
  int has_pre;
  QkvPostParams pre;
};

// ------------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Poll with a wall-clock bound: never an unbounded spin.  false = the expected bytes did not arrive in WAIT_NS.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  unsigned long long t_begin = 0;
  for (int i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 127) == 127) {
      const unsigned long long now = global_ns();
      if (t_begin == 0) t_begin = now;
      else if (now - t_begin > WAIT_NS) return false;
    }
  }
}

// Named CTA barrier for a subset of the warps (id 1: the consumer warps).
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Thread-block cluster: hardware barrier (no spinning) and loads from a peer CTA's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_peer_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// two bytes (already xor 0x80) selected from x -> half2 of the signed values: 0x64xx is 1024 + xx, minus 1152
__device__ __forceinline__ uint32_t bias_pair(uint32_t x, uint32_t sel) {
  uint32_t w = __byte_perm(x, 0x64646464u, sel);
  __half2 h = __hsub2(*reinterpret_cast<__half2*>(&w), __half2half2(__ushort_as_half(0x6480)));
  return *reinterpret_cast<uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------------------ row finalisation
// One warp holds z (one query head's output, lane owns dims lane + 32*i), applies the optional XSA / head-gate
// epilogue with the reference's rounding points (Attention.post, ultraviolet/model.py:322-333) and stores it.
template <typename QT, int HD>
__device__ __forceinline__ void finalize_row(float (&z)[(HD + 31) / 32], int lane, int b, int head, int kvh,
                                             const AttnParams& P, const QT* v_stage = nullptr) {
  constexpr int EPL = (HD + 31) / 32;
  const bool act = (HD >= 32) || lane < HD;
#pragma unroll
  for (int i = 0; i < EPL; ++i) z[i] = rnd<QT>(z[i]);  // the attention output itself is in the activation dtype
  if (P.xsa_alpha != nullptr) {
    // the current token's unquantised v: from the caller's tensor, or from the shared-memory copy the fused
    // prologue left
    const QT* vc = v_stage ? v_stage
                           : static_cast<const QT*>(P.v_cur) + (int64_t)b * P.v_cur_sb + (int64_t)kvh * P.v_cur_sh;
    float vv[EPL], n2 = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      vv[i] = act ? to_f32<QT>(vc[lane + 32 * i]) : 0.f;
      n2 += vv[i] * vv[i];
    }
    n2 = warp_sum(n2);
    const float inv = 1.0f / fmaxf(sqrtf(n2), P.xsa_eps);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      vv[i] *= inv;
      dot += z[i] * vv[i];
    }
    dot = warp_sum(dot);
    const float a = P.xsa_alpha[head];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = rnd<QT>(z[i] - a * dot * vv[i]);
  }
  if (P.gate_vals != nullptr) {
    const float g = P.gate_vals[(int64_t)b * P.H + head];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = rnd<QT>(z[i] * g);
  } else if (P.gate_w != nullptr) {
    const float g = head_gate<QT>(static_cast<const QT*>(P.gate_x) + (int64_t)b * P.gate_x_stride,
                                  static_cast<const QT*>(P.gate_w) + (int64_t)head * P.gate_ch, P.gate_ch, lane);
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = rnd<QT>(z[i] * g);
  }
  QT* o = static_cast<QT*>(P.out) + (int64_t)b * P.sob + (int64_t)head * P.soh;
#pragma unroll
  for (int i = 0; i < EPL; ++i)
    if (act) o[lane + 32 * i] = from_f32<QT>(z[i]);
}

// ------------------------------------------------------------------------------------------------ split merge
// Log-sum-exp merge of the split partials of one (b, kv head): warp per query head, then the shared epilogue.
// Partials were written by other CTAs: read them through L2 (ld.global.cg).
template <typename QT, int HD>
__device__ __forceinline__ void combine_rows(const AttnParams& P, int bk, int warp, int lane,
                                             const QT* v_stage = nullptr) {
  constexpr int EPL = (HD + 31) / 32;
  const int b = bk / P.KH, h = bk % P.KH;
  for (int row = warp; row < P.G && warp < NWARP; row += NWARP) {
    const int64_t base = (int64_t)bk * P.splits * P.G + row;
    float mx = -INFINITY;
    for (int s = lane; s < P.splits; s += 32) mx = fmaxf(mx, __ldcg(P.ws_m + base + (int64_t)s * P.G));
    mx = warp_max(mx);
    float lsum = 0.f, z[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = 0.f;
    if (mx != -INFINITY) {
      for (int s = 0; s < P.splits; ++s) {
        const int64_t wrow = base + (int64_t)s * P.G;
        const float m = __ldcg(P.ws_m + wrow);
        if (m == -INFINITY) continue;
        const float wt = ex2(m - mx);
        lsum += wt * __ldcg(P.ws_l + wrow);
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const int d = lane + 32 * i;
          if (HD >= 32 || d < HD) z[i] += wt * __ldcg(P.ws_o + wrow * HD + d);
        }
      }
      const float inv = 1.0f / lsum;
#pragma unroll
      for (int i = 0; i < EPL; ++i) z[i] *= inv;
    }
    finalize_row<QT, HD>(z, lane, b, h * P.G + row, h, P, v_stage);
  }
}

// Called by every CTA of a split launch after its partials are written: the CTA that arrives last merges.
template <typename QT, int HD>
__device__ __forceinline__ void arrive_and_merge(const AttnParams& P, int bk, int tid, const QT* v_stage = nullptr) {
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(P.counters + bk, 1) == P.splits - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  combine_rows<QT, HD>(P, bk, tid >> 5, tid & 31, v_stage);
  if (tid == 0) P.counters[bk] = 0;
}

// Cluster merge: every split CTA of a cache row has left its partial (o[G][HD], m[G], l[G], fp32) at `part` in its
// own shared memory.  After a cluster barrier the CTA of rank j merges query heads j, j + splits, ... reading its
// peers' partials through distributed shared memory, and runs the epilogue; a second barrier keeps every CTA (and
// its shared memory) alive until all peers have read it.  Called by ALL threads of ALL CTAs of the cluster.
template <typename QT, int HD>
__device__ __forceinline__ void cluster_merge(const AttnParams& P, const float* part, int bk, int sid, int warp,
                                              int lane, const QT* v_stage = nullptr) {
  constexpr int EPL = (HD + 31) / 32;
  const int G = P.G, b = bk / P.KH, h = bk % P.KH;
  cluster_sync_all();
  const uint32_t po = smem_u32(part), pm = po + (uint32_t)(G * HD) * 4u, pl = pm + (uint32_t)G * 4u;
  for (int row = sid + warp * P.splits; row < G; row += (NWARP + 1) * P.splits) {
    // lane s holds split s's running maximum and sum (splits <= 8 <= 32)
    float m_s = -INFINITY, l_s = 0.f;
    if (lane < P.splits) {
      m_s = ld_peer_f32(pm + (uint32_t)row * 4u, (uint32_t)lane);
      l_s = ld_peer_f32(pl + (uint32_t)row * 4u, (uint32_t)lane);
    }
    const float mx = warp_max(m_s);
    const float wt_s = (m_s == -INFINITY) ? 0.f : ex2(m_s - mx);
    const float lsum = warp_sum(wt_s * l_s);
    float z[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = 0.f;
    if (mx != -INFINITY) {
#pragma unroll 8
      for (int s = 0; s < P.splits; ++s) {
        const float wt = __shfl_sync(0xffffffffu, wt_s, s);
        if (wt == 0.f) continue;  // an empty split never wrote its o
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const int d = lane + 32 * i;
          if (HD >= 32 || d < HD) z[i] += wt * ld_peer_f32(po + (uint32_t)(row * HD + d) * 4u, (uint32_t)s);
        }
      }
      const float inv = 1.0f / lsum;
#pragma unroll
      for (int i = 0; i < EPL; ++i) z[i] *= inv;
    }
    finalize_row<QT, HD>(z, lane, b, h * G + row, h, P, v_stage);
  }
  cluster_sync_all();
}

// ------------------------------------------------------------------------------------------------ split kernel
template <int HD> struct StageLayout {
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = TILE * HD;
  static constexpr int KS_OFF = 2 * TILE * HD;
  static constexpr int VS_OFF = 2 * TILE * HD + 2 * TILE;
  static constexpr int BYTES = 2 * TILE * HD + 4 * TILE;
};

// Two-part symmetric int8 split of one query head slice held by a quad: q ~= s1*q1 + (s1/254)*q2 with
// |error| <= max|q| / 64516, so Q K^T runs on the int8 tensor-core path against the raw cache bytes.
template <int N>
__device__ __forceinline__ void split_q(const float (&qv)[N], uint32_t (&w1)[N / 4], uint32_t (&w2)[N / 4],
                                        float& f1, float& f2, float scale_log2) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(qv[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float s1 = amax > 0.f ? amax / 127.0f : 1.0f;
  const float inv1 = 1.0f / s1, inv2 = 254.0f / s1;
#pragma unroll
  for (int w = 0; w < N / 4; ++w) {
    uint32_t p1 = 0u, p2 = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x = qv[4 * w + i];
      const float a = fminf(fmaxf(rintf(x * inv1), -127.f), 127.f);
      const float b = fminf(fmaxf(rintf((x - a * s1) * inv2), -127.f), 127.f);
      p1 |= ((uint32_t)(__float2int_rn(a) & 0xff)) << (8 * i);
      p2 |= ((uint32_t)(__float2int_rn(b) & 0xff)) << (8 * i);
    }
    w1[w] = p1, w2[w] = p2;
  }
  f1 = s1 * scale_log2;
  f2 = s1 * (1.0f / 254.0f) * scale_log2;
}

__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first k-step of a tile: C = 0, so the accumulators need no clearing
__device__ __forceinline__ void imma16832_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

template <typename QT, int HD, bool GP16, bool BULK, bool PRE>
__global__ void __launch_bounds__(NTHREAD) attn_split_kernel(const __grid_constant__ AttnParams P) {
  using L = StageLayout<HD>;
  constexpr int QN = HD / 4;         // query dims per lane = bytes of a key row per lane
  constexpr int QW = HD / 16;        // 32-bit words of a key row per lane
  constexpr int ISTEPS = (QW + 1) / 2;  // k32 int8 MMA steps of Q K^T
  constexpr int NT_S = WKEYS / 8;    // n8 score tiles per warp per stage
  constexpr int NT_O = HD / 8;       // n8 tiles of O = bytes of a value row per lane
  constexpr int ROWS = GP16 ? 16 : 8;
  constexpr int NH = GP16 ? 2 : 1;   // row halves (heads r and r + 8)
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t bars[NSTAGE];   // "full": a tile has landed (transaction bytes)
  __shared__ __align__(8) uint64_t empty[NSTAGE];  // "empty": every consumer warp is done with the stage

  __shared__ int s_dead;                            // a tile of this CTA never landed (bounded wait ran out)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool producer = warp == NWARP;  // the copy-issuing warp never computes
  // This CTA's split partial for the cluster merge sits behind the stage ring (and the staged q / k / v of the
  // fused form), never inside it: peers address it at the same offset in every CTA, and a CTA that gave up on a tile
  // can publish an empty partial without touching shared memory that an abandoned copy may still write.
  constexpr size_t PART_OFF =
      ((size_t)(BULK ? NSTAGE : 2) * L::BYTES + (PRE ? (size_t)(ROWS + 2) * HD * sizeof(QT) + 2 * HD + 16 : 0) + 15) &
      ~(size_t)15;
  float* const part = reinterpret_cast<float*>(smem + PART_OFF);
  const int r = lane >> 2, c = lane & 3;
  const int bk = blockIdx.x, sid = blockIdx.y;
  const int b = bk / P.KH, h = bk % P.KH;
  const int G = P.G;
  pdl_wait();     // positions, q and the newest cache entries come from the kernels before this one
  pdl_trigger();
  // what the epilogue will read at the very end of the chain (the current token's v, the head gates, the XSA
  // coefficients): pulled towards the SM now, while the tiles stream
  if (tid == 0 && P.xsa_alpha != nullptr && P.v_cur != nullptr)
    asm volatile("prefetch.global.L1 [%0];" ::"l"(static_cast<const QT*>(P.v_cur) + (int64_t)b * P.v_cur_sb +
                                                   (int64_t)h * P.v_cur_sh));
  if (tid == 32 && P.gate_vals != nullptr)
    asm volatile("prefetch.global.L1 [%0];" ::"l"(P.gate_vals + (int64_t)b * P.H + (int64_t)h * G));
  if (tid == 64 && P.xsa_alpha != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(P.xsa_alpha + (int64_t)h * G));

  // ---- the row's key range and this split's tiles
  const int64_t p = P.pos[b];
  int64_t lo = P.starts[b];
  if (lo < 0) lo = 0;
  if (P.window > 0 && p - P.window + 1 > lo) lo = p - P.window + 1;
  int64_t hi = p;
  if (P.ring) {
    if (p - P.S + 1 > lo) lo = p - P.S + 1;  // older positions have been overwritten
  } else if (hi > P.S - 1) {
    hi = P.S - 1;
  }
  int64_t t0 = 0, t1 = 0;
  int owner_sid = 0;  // the split whose tiles hold position p (it appends the new key / value in the fused form)
  if (hi >= lo) {
    const int64_t t_lo = lo / TILE, t_hi = hi / TILE;
    const int64_t per = (t_hi - t_lo + P.splits) / P.splits;  // ceil(n_tiles / splits)
    t0 = t_lo + (int64_t)sid * per;
    t1 = t0 + per < t_hi + 1 ? t0 + per : t_hi + 1;
    if (p == hi) owner_sid = (int)((t_hi - t_lo) / per);
  }
  const int ntile = t1 > t0 ? (int)(t1 - t0) : 0;

  // ---- fused form (uv_qkv_attn): the consumer warps post-process the row's raw q / k / v head slots, leave them in
  //      shared memory behind the stage ring ([G] query heads, key, value) and, in the owning split, append the
  //      quantised key and value to the cache.  Splits of one row repeat the arithmetic; only the owner writes.
//      No copy waits for that write: every tile is requested up front, and the entry at p is patched into the
//      landed tile from shared memory.
  QT* const pre_stage = reinterpret_cast<QT*>(smem + (size_t)NSTAGE * L::BYTES);  // [G + 2][HD] activations,
  int8_t* const pre_q8 = reinterpret_cast<int8_t*>(pre_stage + (ROWS + 2) * HD);     // then [2][HD] int8 (k, v)
  uint16_t* const pre_sc = reinterpret_cast<uint16_t*>(pre_q8 + 2 * HD);             // and their two fp16 scales
  const QT* v_stage = nullptr;
  auto pre_items = [&]() {
    constexpr int E = HD >= 32 ? HD / 32 : 1;
    constexpr int MAXI = (ROWS + 2 + NWARP - 1) / NWARP;
    const int slots = P.pre.H + 2 * P.pre.K;
    const QT* raw = static_cast<const QT*>(P.pre.qkv) + (int64_t)b * slots * HD;
    const bool act = lane * E < HD;
    float x[MAXI][E];
    int hs[MAXI];
#pragma unroll
    for (int n = 0; n < MAXI; ++n) {  // all loads first: one round trip for the warp's items
      const int it = warp + n * NWARP;
      hs[n] = it < G ? h * G + it : (it == G ? P.pre.H + h : P.pre.H + P.pre.K + h);
#pragma unroll
      for (int i = 0; i < E; ++i)
        x[n][i] = (it < G + 2 && act) ? to_f32<QT>(raw[(int64_t)hs[n] * HD + lane * E + i]) : 0.f;
    }
#pragma unroll
    for (int n = 0; n < MAXI; ++n) {
      const int it = warp + n * NWARP;
      if (it >= G + 2) continue;  // warp-uniform
      qkv_post_compute<QT, HD, true>(P.pre, b, hs[n], lane, x[n]);
#pragma unroll
      for (int i = 0; i < E; ++i)
        if (act) pre_stage[it * HD + lane * E + i] = from_f32<QT>(x[n][i]);
      if (it >= G) {
        // the quantised entry stays in shared memory too: the warp that consumes position p patches it into the
        // landed tile, so no copy has to wait for the global write below
        int8_t q8[E];
        const uint16_t s = quantize_lane<E>(x[n], q8);
#pragma unroll
        for (int i = 0; i < E; ++i)
          if (act) pre_q8[(it - G) * HD + lane * E + i] = q8[i];
        if (lane == 0) pre_sc[it - G] = s;
        if (sid == owner_sid) qkv_post_store<HD>(P.pre, b, hs[n], lane, q8, s);
      }
    }
  };
  if constexpr (PRE) {
    v_stage = pre_stage + (G + 1) * HD;
    if (ntile == 0) {
      if (!producer) pre_items();
      __syncthreads();
    }
  }

  // An empty row, an inactive split, or a CTA whose tile copy timed out: zeros (unsplit) or an empty partial.
  auto empty_result = [&]() {
    if (P.splits == 1) {
      for (int i = tid; i < G * HD; i += NTHREAD) {
        QT* o = static_cast<QT*>(P.out) + (int64_t)b * P.sob + (int64_t)(h * G + i / HD) * P.soh;
        o[i % HD] = from_f32<QT>(0.f);
      }
    } else if (P.cluster) {
      if (tid < G) {
        part[G * HD + tid] = -INFINITY;
        part[G * HD + G + tid] = 0.f;
      }
      cluster_merge<QT, HD>(P, part, bk, sid, warp, lane, v_stage);
    } else {
      if (tid < G) {
        const int64_t row = ((int64_t)bk * P.splits + sid) * G + tid;
        P.ws_m[row] = -INFINITY;
        P.ws_l[row] = 0.f;
      }
      if (P.counters) arrive_and_merge<QT, HD>(P, bk, tid, v_stage);
    }
  };
  if (ntile == 0) {
    empty_result();
    return;
  }

  // ---- Q: lane (r, c) owns dims [c*HD/4, (c+1)*HD/4) of head r (and r + 8), split into two int8 parts.
  //      G <= 8: rows 0..7 of the A operand carry part 1 and rows 8..15 part 2 of the same head.
  uint32_t q1w[NH][QW], q2w[NH][QW];
  float f1[NH], f2[NH];
  const int64_t cb = P.row_map ? P.row_map[b] : b;  // cache row
  const int8_t* kbase = P.k + cb * P.skb + (int64_t)h * P.skh;
  const int8_t* vbase = P.v + cb * P.svb + (int64_t)h * P.svh;
  const __half* ksbase = P.ks + cb * P.ssb + (int64_t)h * P.ssh;
  const __half* vsbase = P.vs + cb * P.stb + (int64_t)h * P.sth;

  if constexpr (BULK) {
    if (tid == 0) {
      s_dead = 0;
#pragma unroll
      for (int s = 0; s < NSTAGE; ++s) {
        mbar_init(smem_u32(&bars[s]), 1);
        mbar_init(smem_u32(&empty[s]), NWARP);
      }
      fence_barrier_init();
    }
    __syncthreads();
  }

  // issue the four linear copies of tile ti into stage s (one thread)
  auto issue = [&](int64_t ti, int s) {
    const int64_t T0 = ti * TILE;
    int64_t a = (T0 > lo ? T0 : lo) & ~(int64_t)7;
    int64_t e = (T0 + TILE < hi + 1 ? T0 + TILE : hi + 1);
    e = (e + 7) & ~(int64_t)7;
    const uint32_t cnt = (uint32_t)(e - a);
    const int64_t slot = P.ring ? a % P.S : a;
    const uint32_t off = (uint32_t)(a - T0);
    const uint32_t bar = smem_u32(&bars[s]);
    const uint32_t st = smem_u32(smem + (size_t)s * L::BYTES);
    fence_proxy_async();
    mbar_expect_tx(bar, cnt * (2 * HD + 4));
    // A ring whose length is not a multiple of the tile lets a tile's positions run past slot S - 1: the copy is
    // cut there and continues at slot 0 (S is a multiple of 8, so both pieces keep the 16-byte rules; a tile spans
    // at most S + 8 positions, so it wraps once).
    uint32_t c1 = cnt;
    if (P.ring && slot + (int64_t)cnt > P.S) c1 = (uint32_t)(P.S - slot);
    bulk_g2s(st + L::K_OFF + off * HD, kbase + slot * HD, c1 * HD, bar);
    bulk_g2s(st + L::V_OFF + off * HD, vbase + slot * HD, c1 * HD, bar);
    bulk_g2s(st + L::KS_OFF + off * 2, ksbase + slot, c1 * 2, bar);
    bulk_g2s(st + L::VS_OFF + off * 2, vsbase + slot, c1 * 2, bar);
    if (c1 < cnt) {
      const uint32_t c2 = cnt - c1, off2 = off + c1;
      bulk_g2s(st + L::K_OFF + off2 * HD, kbase, c2 * HD, bar);
      bulk_g2s(st + L::V_OFF + off2 * HD, vbase, c2 * HD, bar);
      bulk_g2s(st + L::KS_OFF + off2 * 2, ksbase, c2 * 2, bar);
      bulk_g2s(st + L::VS_OFF + off2 * 2, vsbase, c2 * 2, bar);
    }
  };

  // plain-load path (caches whose geometry breaks the bulk engine's 16-byte rules): every thread moves 16-byte
  // pieces of the valid keys of tile ti into stage s with cp.async, so the copy of the next tile runs under the
  // math of the current one; the 2-byte scales travel through registers (loaded when the tile is requested, stored
  // one iteration later, just before the tile is consumed).
  constexpr int SC_PER_THREAD = (2 * TILE + NTHREAD - 1) / NTHREAD;
  __half sc_reg[SC_PER_THREAD];
  auto load_generic = [&](int64_t ti, int s) {
    const int64_t T0 = ti * TILE;
    unsigned char* st = smem + (size_t)s * L::BYTES;
    constexpr int CH = HD / 16;  // 16-byte chunks per row
    for (int i = tid; i < TILE * CH * 2; i += NTHREAD) {
      const int which = i / (TILE * CH);
      const int j = (i % (TILE * CH)) / CH, ch = i % CH;
      const int64_t t = T0 + j;
      if (t < lo || t > hi) continue;
      const int64_t slot = P.ring ? t % P.S : t;
      const int8_t* src = which ? vbase + slot * P.svs : kbase + slot * P.sks;
      const uint32_t dst = smem_u32(st + (which ? L::V_OFF : L::K_OFF) + j * HD + ch * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + ch * 16) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
    for (int n = 0; n < SC_PER_THREAD; ++n) {
      const int i = tid + n * NTHREAD;
      const int which = i / TILE, j = i % TILE;
      const int64_t t = T0 + j;
      sc_reg[n] = __ushort_as_half(0);
      if (i < 2 * TILE && t >= lo && t <= hi) {
        const int64_t slot = P.ring ? t % P.S : t;
        sc_reg[n] = which ? vsbase[slot] : ksbase[slot];
      }
    }
  };
  auto store_scales = [&](int s) {
    unsigned char* st = smem + (size_t)s * L::BYTES;
#pragma unroll
    for (int n = 0; n < SC_PER_THREAD; ++n) {
      const int i = tid + n * NTHREAD;
      if (i < 2 * TILE) reinterpret_cast<__half*>(st + (i / TILE ? L::VS_OFF : L::KS_OFF))[i % TILE] = sc_reg[n];
    }
  };

  // ---- per-warp online softmax state
  float o_acc[NT_O][4];  // full m16n8 accumulator quads (rows 8..15 stay zero when G <= 8): no register shuffling
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[NH], l_run[NH];
#pragma unroll
  for (int j = 0; j < NH; ++j) {
    m_run[j] = -INFINITY;
    l_run[j] = 0.f;
  }

  // one warp's WKEYS keys of one stage.  EDGE: some keys fall outside [lo, hi] (first / last tile of the row).
  auto block = [&](const unsigned char* st, int lo_rel, int hi_rel, auto edge_tag) {
    constexpr bool EDGE = decltype(edge_tag)::value;
    const int k0 = WKEYS * warp;
    // ---- S = Q K^T on the int8 pipe
    int acc1[NT_S][4], acc2[GP16 ? NT_S : 1][4];
#pragma unroll
    for (int t = 0; t < NT_S; ++t) {
      const unsigned char* krow = st + L::K_OFF + (k0 + 8 * t + r) * HD + c * QN;
      uint32_t kw[QW];
      if constexpr (QW == 1) {
        kw[0] = *reinterpret_cast<const uint32_t*>(krow);
      } else if constexpr (QW == 2) {
        const uint2 u = *reinterpret_cast<const uint2*>(krow);
        kw[0] = u.x, kw[1] = u.y;
      } else {
#pragma unroll
        for (int j4 = 0; j4 < QW / 4; ++j4) {
          const uint4 u = *reinterpret_cast<const uint4*>(krow + 16 * j4);
          kw[4 * j4] = u.x, kw[4 * j4 + 1] = u.y, kw[4 * j4 + 2] = u.z, kw[4 * j4 + 3] = u.w;
        }
      }
#pragma unroll
      for (int j = 0; j < ISTEPS; ++j) {
        const bool two = 2 * j + 1 < QW;
        const uint32_t b0 = kw[2 * j], b1 = two ? kw[two ? 2 * j + 1 : 0] : 0u;
        const int j1 = two ? 2 * j + 1 : 0;
        if constexpr (GP16) {
          if (j == 0) {
            imma16832_z(acc1[t], q1w[0][0], q1w[1][0], two ? q1w[0][j1] : 0u, two ? q1w[1][j1] : 0u, b0, b1);
            imma16832_z(acc2[t], q2w[0][0], q2w[1][0], two ? q2w[0][j1] : 0u, two ? q2w[1][j1] : 0u, b0, b1);
          } else {
            imma16832(acc1[t], q1w[0][2 * j], q1w[1][2 * j], two ? q1w[0][j1] : 0u, two ? q1w[1][j1] : 0u, b0, b1);
            imma16832(acc2[t], q2w[0][2 * j], q2w[1][2 * j], two ? q2w[0][j1] : 0u, two ? q2w[1][j1] : 0u, b0, b1);
          }
        } else {
          if (j == 0)
            imma16832_z(acc1[t], q1w[0][0], q2w[0][0], two ? q1w[0][j1] : 0u, two ? q2w[0][j1] : 0u, b0, b1);
          else
            imma16832(acc1[t], q1w[0][2 * j], q2w[0][2 * j], two ? q1w[0][j1] : 0u, two ? q2w[0][j1] : 0u, b0, b1);
        }
      }
    }
    // ---- per-key scales (K: fp32 multipliers of the S columns; V: raw half2, multiplied into P in fp16)
    float ksf[NT_S][2];
    uint32_t vsh[NT_S];
#pragma unroll
    for (int t = 0; t < NT_S; ++t) {
      const int kk = 8 * t + 2 * c;
      const float2 kf = __half22float2(*reinterpret_cast<const __half2*>(st + L::KS_OFF + (k0 + kk) * 2));
      ksf[t][0] = kf.x, ksf[t][1] = kf.y;
      vsh[t] = *reinterpret_cast<const uint32_t*>(st + L::VS_OFF + (k0 + kk) * 2);
      if constexpr (EDGE) {  // keys outside [lo, hi] may sit on bytes no copy has written: zero their V scale
        const bool ok0 = kk >= lo_rel && kk <= hi_rel, ok1 = kk + 1 >= lo_rel && kk + 1 <= hi_rel;
        vsh[t] &= (ok0 ? 0x0000ffffu : 0u) | (ok1 ? 0xffff0000u : 0u);
      }
    }
    // ---- online softmax per row half; P (fp16, V scale folded in) becomes the A operand of P V
    uint32_t pa[WKEYS / 16][4];
#pragma unroll
    for (int u = 0; u < WKEYS / 16; ++u) pa[u][0] = pa[u][1] = pa[u][2] = pa[u][3] = 0u;
#pragma unroll
    for (int hr = 0; hr < NH; ++hr) {
      float sc[NT_S][2];
      float mx = -INFINITY;
#pragma unroll
      for (int t = 0; t < NT_S; ++t)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float v;
          if constexpr (GP16)
            v = (__int2float_rn(acc1[t][2 * hr + e]) * f1[hr] + __int2float_rn(acc2[t][2 * hr + e]) * f2[hr]) *
                ksf[t][e];
          else
            v = (__int2float_rn(acc1[t][e]) * f1[0] + __int2float_rn(acc1[t][2 + e]) * f2[0]) * ksf[t][e];
          if constexpr (EDGE) {
            const int kk = 8 * t + 2 * c + e;
            v = (kk >= lo_rel && kk <= hi_rel) ? v : -INFINITY;
          }
          sc[t][e] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      // The running maximum is only raised when a row's new maximum beats it by more than RESCALE_GAP (log2
      // units), so p <= 2^RESCALE_GAP and the accumulator rescale is rare; the final ratio O / l is unaffected.
      if (__any_sync(0xffffffffu, mx > m_run[hr] + RESCALE_GAP)) {
        const float m_new = mx > m_run[hr] + RESCALE_GAP ? mx : m_run[hr];
        const float alpha = ex2(m_run[hr] - m_new);  // 1 for rows that keep their maximum, 0 on the first block
        l_run[hr] *= alpha;
#pragma unroll
        for (int i = 0; i < NT_O; ++i) {
          o_acc[i][2 * hr] *= alpha;
          o_acc[i][2 * hr + 1] *= alpha;
        }
        m_run[hr] = m_new;
      }
      const float m_use = m_run[hr];
      float ls = 0.f;
#pragma unroll
      for (int t = 0; t < NT_S; ++t) {
        const float p0 = ex2(sc[t][0] - m_use), p1 = ex2(sc[t][1] - m_use);  // masked keys: ex2(-inf) = 0
        ls += p0 + p1;
        const __half2 ph = __floats2half2_rn(p0, p1);
        const __half2 pv = __hmul2(ph, *reinterpret_cast<const __half2*>(&vsh[t]));
        pa[t / 2][2 * (t & 1) + hr] = *reinterpret_cast<const uint32_t*>(&pv);
      }
      l_run[hr] += ls;
    }
    // ---- O += P V: lane (r, c) reads HD/8 bytes at dim offset r*HD/8 of keys 2c, 2c+1, 2c+8, 2c+9 of each
    //      16-key step and transposes them into B fragments (n8 tile i <-> dim r*HD/8 + i)
#pragma unroll
    for (int u = 0; u < WKEYS / 16; ++u) {
      const unsigned char* vrow = st + L::V_OFF + (k0 + 16 * u + 2 * c) * HD + r * (HD / 8);
      constexpr int VW = (NT_O + 3) / 4;  // 32-bit words per row piece
      uint32_t va[VW], vb[VW], vc[VW], vd[VW];
      auto ld = [&](const unsigned char* ptr, uint32_t(&w)[VW]) {
        if constexpr (NT_O == 2) {
          w[0] = *reinterpret_cast<const uint16_t*>(ptr);
        } else if constexpr (NT_O == 4) {
          w[0] = *reinterpret_cast<const uint32_t*>(ptr);
        } else if constexpr (NT_O == 8) {
          const uint2 q2 = *reinterpret_cast<const uint2*>(ptr);
          w[0] = q2.x, w[1] = q2.y;
        } else {
#pragma unroll
          for (int j4 = 0; j4 < VW / 4; ++j4) {
            const uint4 q4 = *reinterpret_cast<const uint4*>(ptr + 16 * j4);
            w[4 * j4] = q4.x, w[4 * j4 + 1] = q4.y, w[4 * j4 + 2] = q4.z, w[4 * j4 + 3] = q4.w;
          }
        }
      };
      ld(vrow, va);
      ld(vrow + HD, vb);
      ld(vrow + 8 * HD, vc);
      ld(vrow + 9 * HD, vd);
#pragma unroll
      for (int w = 0; w < VW; ++w) {
        const uint32_t xa = va[w] ^ 0x80808080u, xb = vb[w] ^ 0x80808080u;
        const uint32_t xc = vc[w] ^ 0x80808080u, xd = vd[w] ^ 0x80808080u;
#pragma unroll
        for (int hw = 0; hw < 2; ++hw) {  // byte pairs (0,1) and (2,3) of the word
          if (4 * w + 2 * hw >= NT_O) break;
          const uint32_t tab = __byte_perm(xa, xb, hw ? 0x7362 : 0x5140);  // (A_i, B_i, A_i+1, B_i+1)
          const uint32_t tcd = __byte_perm(xc, xd, hw ? 0x7362 : 0x5140);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = 4 * w + 2 * hw + e;
            const uint32_t b0 = bias_pair(tab, e ? 0x4342 : 0x4140);
            const uint32_t b1 = bias_pair(tcd, e ? 0x4342 : 0x4140);
            mma16816(o_acc[i], pa[u][0], pa[u][1], pa[u][2], pa[u][3], b0, b1);
          }
        }
      }
    }
  };

  bool dead = false;
  if constexpr (BULK) {
    // The producer warp runs ahead of the consumers by up to NSTAGE tiles: it refills a stage as soon as all
    // consumer warps have released it, so consumer warps drift freely instead of meeting at a CTA barrier per tile.
    if (producer) {
      if (lane == 0) {
        for (int j = 0; j < ntile; ++j) {
          const int s = j % NSTAGE, k = j / NSTAGE;
          if (k > 0 && !mbar_wait_bounded(smem_u32(&empty[s]), (uint32_t)((k - 1) & 1))) {
            dead = true;  // consumers will time out on the full barrier and flag the launch as well
            break;
          }
          issue(t0 + j, s);
        }
      }
    } else if constexpr (PRE) {
      pre_items();
      named_bar_sync(1, NWARP * 32);  // every consumer warp reads the q heads (and the new entry) the others staged
    }
  }
  // the first tiles are in flight: consumers load and split Q under their latency
  if (!producer)
#pragma unroll
  for (int hr = 0; hr < NH; ++hr) {
    float qv[QN];
    const int head = r + 8 * hr;
    const QT* qb = PRE
                       ? pre_stage + head * HD + c * QN
                       : static_cast<const QT*>(P.q) + (int64_t)b * P.sqb + (int64_t)(h * G + head) * P.sqh + c * QN;
#pragma unroll
    for (int i = 0; i < QN; i += 2) {
      if (head < G) {
        qv[i] = to_f32<QT>(qb[i]), qv[i + 1] = to_f32<QT>(qb[i + 1]);
      } else {
        qv[i] = qv[i + 1] = 0.f;
      }
    }
    split_q<QN>(qv, q1w[hr], q2w[hr], f1[hr], f2[hr], P.scale_log2);
  }


  if constexpr (BULK) {
    if (!producer) {
      for (int it = 0; it < ntile; ++it) {
        const int s = it % NSTAGE;
        if (!dead) {  // warp-uniform: a warp whose tile never landed stops consuming and flags the launch
          const bool got = mbar_wait_bounded(smem_u32(&bars[s]), (uint32_t)((it / NSTAGE) & 1));
          dead = !__all_sync(0xffffffffu, got);
        }
        if (!dead) {
          const unsigned char* st = smem + (size_t)s * L::BYTES;
          const int64_t kb0 = (t0 + it) * TILE + WKEYS * warp;  // position of this warp's first key
          if constexpr (PRE) {
            // The tile was copied while the cache entry at p was being rewritten: the warp that consumes
            // position p (no other warp reads it) overwrites that entry in the landed tile with the staged bytes.
            if (p == hi && p >= kb0 && p < kb0 + WKEYS) {
              unsigned char* sw = smem + (size_t)s * L::BYTES;
              const int kk = (int)(p - (t0 + it) * TILE);
              for (int w = lane; w < HD / 2; w += 32) {
                const uint32_t v = reinterpret_cast<const uint32_t*>(pre_q8)[w];
                if (w < HD / 4) *reinterpret_cast<uint32_t*>(sw + L::K_OFF + kk * HD + 4 * w) = v;
                else *reinterpret_cast<uint32_t*>(sw + L::V_OFF + kk * HD + 4 * (w - HD / 4)) = v;
              }
              if (lane == 0) *reinterpret_cast<uint16_t*>(sw + L::KS_OFF + kk * 2) = pre_sc[0];
              if (lane == 1) *reinterpret_cast<uint16_t*>(sw + L::VS_OFF + kk * 2) = pre_sc[1];
              __syncwarp();
            }
          }
          if (kb0 + WKEYS - 1 >= lo && kb0 <= hi) {
            if (kb0 < lo || kb0 + WKEYS - 1 > hi) {
              const int64_t lr = lo - kb0, hr_ = hi - kb0;
              block(st, lr < 0 ? 0 : (int)lr, hr_ > WKEYS ? WKEYS : (int)hr_, std::true_type{});
            } else {
              block(st, 0, WKEYS, std::false_type{});
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&empty[s]));  // release the stage (also when skipped or dead)
      }
    }
  } else {
    // two stages: tile it + 1 is copied while tile it is consumed; one CTA barrier per tile
    load_generic(t0, 0);
    for (int it = 0; it < ntile; ++it) {
      const int s = it & 1;
      asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's pieces of tile it have landed
      store_scales(s);
      __syncthreads();  // tile it is complete for everyone, and every warp is done with tile it - 1 (stage s ^ 1)
      if (it + 1 < ntile) load_generic(t0 + it + 1, s ^ 1);
      if (producer) continue;
      const unsigned char* st = smem + (size_t)s * L::BYTES;
      const int64_t kb0 = (t0 + it) * TILE + WKEYS * warp;
      if (kb0 + WKEYS - 1 < lo || kb0 > hi) continue;
      if (kb0 < lo || kb0 + WKEYS - 1 > hi) {
        const int64_t lr = lo - kb0, hr_ = hi - kb0;
        block(st, lr < 0 ? 0 : (int)lr, hr_ > WKEYS ? WKEYS : (int)hr_, std::true_type{});
      } else {
        block(st, 0, WKEYS, std::false_type{});
      }
    }
  }

  if constexpr (BULK) {
    if (dead && lane == 0) {
      if (P.status) atomicOr(P.status, 1);
      s_dead = 1;
    }
  }

  __syncthreads();
  if constexpr (BULK) {
    // A tile was abandoned: its copy may still land, so the stage ring is not reused.  The CTA reports an empty
    // result (the status bit says the launch's output is undefined) and still takes part in the split merge, which
    // its peers wait for.
    if (s_dead) {
      empty_result();
      return;
    }
  }
  // ---- merge the warps' states through shared memory (aliases the stage ring: every copy has landed)
  float* mg_o = reinterpret_cast<float*>(smem);                    // [NWARP][ROWS][HD]
  float* mg_m = mg_o + NWARP * ROWS * HD;                          // [NWARP][ROWS]
  float* mg_l = mg_m + NWARP * ROWS;
  if (!producer)
#pragma unroll
  for (int hr = 0; hr < NH; ++hr) {
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int row = r + 8 * hr;
    if (c == 0) {
      mg_m[warp * ROWS + row] = m_run[hr];
      mg_l[warp * ROWS + row] = l;
    }
    float* orow = mg_o + (warp * ROWS + row) * HD;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      orow[(2 * c) * (HD / 8) + i] = o_acc[i][2 * hr];
      orow[(2 * c + 1) * (HD / 8) + i] = o_acc[i][2 * hr + 1];
    }
  }
  __syncthreads();

  constexpr int EPL = (HD + 31) / 32;
  for (int row = warp; row < G && !producer; row += NWARP) {
    float mw[NWARP], mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      mw[w] = mg_m[w * ROWS + row];
      mx = fmaxf(mx, mw[w]);
    }
    float lsum = 0.f, z[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) z[i] = 0.f;
#pragma unroll
    for (int w = 0; w < NWARP; ++w) {
      const float wt = (mw[w] == -INFINITY) ? 0.f : ex2(mw[w] - mx);
      lsum += wt * mg_l[w * ROWS + row];
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (HD >= 32 || d < HD) z[i] += wt * mg_o[(w * ROWS + row) * HD + d];
      }
    }
    if (P.splits == 1) {
      const float inv = 1.0f / lsum;
#pragma unroll
      for (int i = 0; i < EPL; ++i) z[i] *= inv;
      finalize_row<QT, HD>(z, lane, b, h * G + row, h, P, v_stage);
    } else if (P.cluster) {
      if (lane == 0) {
        part[G * HD + row] = mx;
        part[G * HD + G + row] = lsum;
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (HD >= 32 || d < HD) part[row * HD + d] = z[i];
      }
    } else {
      const int64_t wrow = ((int64_t)bk * P.splits + sid) * G + row;
      if (lane == 0) {
        P.ws_m[wrow] = mx;
        P.ws_l[wrow] = lsum;
      }
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int d = lane + 32 * i;
        if (HD >= 32 || d < HD) P.ws_o[wrow * HD + d] = z[i];
      }
    }
  }
  if (P.splits > 1) {
    if (P.cluster)
      cluster_merge<QT, HD>(P, part, bk, sid, warp, lane, v_stage);
    else if (P.counters)
      arrive_and_merge<QT, HD>(P, bk, tid, v_stage);
  }
}

template <typename QT, int HD>
__global__ void __launch_bounds__(NTHREAD) attn_combine_kernel(const __grid_constant__ AttnParams P) {
  combine_rows<QT, HD>(P, blockIdx.x, threadIdx.x >> 5, threadIdx.x & 31);
}

// ------------------------------------------------------------------------------------------------ host side
template <typename QT, int HD>
static int launch_attn(const AttnParams& P, bool bulk, cudaStream_t st) {
  using L = StageLayout<HD>;
  const bool gp16 = P.G > 8;
  const int rows = gp16 ? 16 : 8;
  // the stage ring (reused for the warp-merge arrays once every copy has landed) ...
  const size_t merge = (size_t)NWARP * rows * (HD + 2) * sizeof(float);
  size_t smem = (size_t)(bulk ? NSTAGE : 2) * L::BYTES;
  static_assert((size_t)NWARP * 16 * (HD + 2) * sizeof(float) <= 2 * (size_t)L::BYTES, "merge arrays fit the ring");
  (void)merge;
  // ... staged q heads, key and value (activations), the quantised key / value and their scales (fused form) ...
  if (P.has_pre) smem += (size_t)(rows + 2) * HD * sizeof(QT) + 2 * HD + 16;
  // ... and this CTA's split partial for the cluster merge (o[rows][HD], m[rows], l[rows])
  smem = ((smem + 15) & ~(size_t)15) + (size_t)rows * (HD + 2) * sizeof(float);
  dim3 grid((unsigned)(P.B * P.KH), (unsigned)P.splits);
  const dim3 cluster(1, P.cluster ? (unsigned)P.splits : 1u, 1);
#define UV_LAUNCH(GP, BK, PR)                                                                              \
  do {                                                                                                     \
    auto kern = attn_split_kernel<QT, HD, GP, BK, PR>;                                                     \
    if (smem > 48 * 1024) {                                                                                \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
      if (e != cudaSuccess) {                                                                              \
        set_last_cuda_error((int)e);                                                                       \
        return UV_ERR_CUDA;                                                                                \
      }                                                                                                    \
    }                                                                                                      \
    launch_cluster(kern, grid, dim3(NTHREAD), cluster, smem, st, P);                                                    \
  } while (0)
  if (gp16) {
    if (bulk && P.has_pre) UV_LAUNCH(true, true, true);
    else if (bulk) UV_LAUNCH(true, true, false);
    else UV_LAUNCH(true, false, false);
  } else {
    if (bulk && P.has_pre) UV_LAUNCH(false, true, true);
    else if (bulk) UV_LAUNCH(false, true, false);
    else UV_LAUNCH(false, false, false);
  }
#undef UV_LAUNCH
  int rc = check_launch();
  if (rc != UV_OK) return rc;
  if (P.splits > 1 && !P.counters && !P.cluster) {
    attn_combine_kernel<QT, HD><<<(unsigned)(P.B * P.KH), NTHREAD, 0, st>>>(P);
    rc = check_launch();
  }
  return rc;
}

template <typename QT>
static int dispatch_hd(const AttnParams& P, int hd, bool bulk, cudaStream_t st) {
  switch (hd) {
    case 16: return launch_attn<QT, 16>(P, bulk, st);
    case 32: return launch_attn<QT, 32>(P, bulk, st);
    case 64: return launch_attn<QT, 64>(P, bulk, st);
    case 128: return launch_attn<QT, 128>(P, bulk, st);
    default: return UV_ERR_SHAPE;
  }
}

}  // namespace uv

extern "C" size_t uv_decode_attn_workspace_bytes(int B, int KH, int G, int hd, int num_splits) {
  if (num_splits <= 1 || B <= 0 || KH <= 0 || G <= 0 || hd <= 0) return 0;
  return (size_t)B * KH * num_splits * G * (size_t)(hd + 2) * sizeof(float);
}

namespace uv {
static bool cluster_merge_enabled() {
  static const bool on = [] {
    const char* v = getenv("UVDECODE_CLUSTER_MERGE");  // "0" falls back to the workspace + arrival-counter merge
    return !(v && v[0] == '0');
  }();
  return on;
}
}  // namespace uv

extern "C" int uv_default_splits(int n_bk, int ctx, int n_sm) {
  if (n_bk < 1) n_bk = 1;
  if (n_sm < 1) n_sm = 148;
  const int tiles = (ctx + uv::TILE - 1) / uv::TILE;
  // All CTAs resident at once (4 per SM): a launch that spills into a second wave pays that wave's whole latency.
  int s = 4 * n_sm / n_bk;
  if (s > tiles / 2) s = tiles / 2;  // at least two tiles per split
  if (s > 64) s = 64;
  if (s < 1) s = 1;
  // Up to 8 splits merge inside a thread-block cluster, ~3.5 us cheaper than the workspace merge: more than 8 only
  // pays when 8 per row would leave most of the SMs without a CTA.
  if (s > 8) s = (16 * n_bk <= n_sm) ? (s < 16 ? s : 16) : 8;
  const int per = (tiles + s - 1) / s;  // tiles per split; the fewest splits with that much work each
  s = (tiles + per - 1) / per;
  // a split launch costs ~3 us more than an unsplit one (cluster scheduling + merge) and a tile ~0.9 us: splitting
  // pays only when it takes at least four tiles off every CTA's serial chain
  if (tiles - per < 4) s = 1;
  return s < 1 ? 1 : s;
}

// bulk-copy (TMA) path: tiles must be linear and every piece 16-byte aligned
static bool attn_bulk_ok(const uv_attn_args* a) {
  using namespace uv;
  bool bulk = a->sks == a->hd && a->svs == a->hd;
  // rows are read in whole 8-slot groups: a linear row's allocation (S_alloc slots, >= S) must cover the group that
  // holds slot S - 1, a ring's length must be a multiple of 8 (a tile that crosses slot S - 1 is fetched in two pieces)
  const int s_alloc = a->S_alloc > a->S ? a->S_alloc : a->S;
  bulk = bulk && (a->ring ? a->S % 8 == 0 : s_alloc % 8 == 0);
  bulk = bulk && aligned16(a->k_cache) && aligned16(a->v_cache) && ((a->skb | a->skh | a->svb | a->svh) & 15) == 0;
  bulk = bulk && aligned16(a->k_scale) && aligned16(a->v_scale) &&
         ((a->ssb | a->ssh | a->stb | a->sth) & 7) == 0;  // scale rows start on 16-byte boundaries (fp16 elements)
  return bulk;
}

extern "C" int uv_decode_attn_uses_bulk(const uv_attn_args* a) {
  if (!a || !a->k_cache || !a->v_cache || !a->k_scale || !a->v_scale) return UV_ERR_ARG;
  return attn_bulk_ok(a) ? 1 : 0;
}

// pre != nullptr: the caller wants uv_qkv_post's work done in the kernel's prologue.  *fused tells it whether that
// happened; when the launch cannot take the fused form (plain-load path, or more than 8 splits without arrival
// counters) nothing is launched, *fused = false and the caller runs the two-launch form.
static int decode_attn_impl(const uv_attn_args* a, void* stream, bool allow_cluster,
                            const uv::QkvPostParams* pre = nullptr, bool* fused = nullptr) {
  using namespace uv;
  if (!a) return UV_ERR_ARG;
  if (a->B == 0) return UV_OK;
  if (!a->q || !a->k_cache || !a->v_cache || !a->pos || !a->starts || !a->out) return UV_ERR_ARG;
  if (a->B < 0 || a->H < 1 || a->KH < 1 || a->S < 1 || a->H % a->KH || a->num_splits < 1 || a->window < 0)
    return UV_ERR_ARG;
  if (a->kv_dtype != UV_I8) return UV_ERR_DTYPE;
  if (!a->k_scale || !a->v_scale) return UV_ERR_ARG;
  if (a->q_dtype != UV_F16 && a->q_dtype != UV_BF16) return UV_ERR_DTYPE;
  const int G = a->H / a->KH, hd = a->hd;
  if (G > 16) return UV_ERR_SHAPE;
  if (hd != 16 && hd != 32 && hd != 64 && hd != 128) return UV_ERR_SHAPE;
  // q / out: pairs are read as 32-bit words
  if ((reinterpret_cast<uintptr_t>(a->q) & 3) || (a->sqb & 1) || (a->sqh & 1)) return UV_ERR_ALIGN;
  // cache rows are read in 16-byte pieces on every path
  if (!aligned16(a->k_cache) || !aligned16(a->v_cache) || (a->skb | a->skh | a->sks | a->svb | a->svh | a->svs) & 15)
    return UV_ERR_ALIGN;
  if ((a->xsa_alpha && !a->v_cur) || (a->gate_w && !a->gate_vals && (!a->gate_x || a->gate_ch < 1)))
    return UV_ERR_ARG;

  AttnParams P{};
  P.q = a->q, P.k = static_cast<const int8_t*>(a->k_cache), P.v = static_cast<const int8_t*>(a->v_cache);
  P.ks = reinterpret_cast<const __half*>(a->k_scale), P.vs = reinterpret_cast<const __half*>(a->v_scale);
  P.pos = a->pos, P.starts = a->starts, P.row_map = a->row_map, P.out = a->out;
  P.sqb = a->sqb, P.sqh = a->sqh, P.skb = a->skb, P.skh = a->skh, P.sks = a->sks;
  P.svb = a->svb, P.svh = a->svh, P.svs = a->svs, P.ssb = a->ssb, P.ssh = a->ssh, P.stb = a->stb, P.sth = a->sth;
  P.sob = a->sob, P.soh = a->soh;
  P.B = a->B, P.H = a->H, P.KH = a->KH, P.G = G, P.S = a->S, P.window = a->window, P.ring = a->ring ? 1 : 0;
  P.splits = a->num_splits;
  P.scale_log2 = a->scale * LOG2E;
  P.status = a->status;
  P.counters = a->num_splits > 1 ? a->counters : nullptr;
  P.v_cur = a->v_cur, P.v_cur_sb = a->v_cur_sb, P.v_cur_sh = a->v_cur_sh, P.xsa_alpha = a->xsa_alpha, P.xsa_eps = a->xsa_eps;
  P.gate_x = a->gate_x, P.gate_x_stride = a->gate_x_stride, P.gate_w = a->gate_w, P.gate_ch = a->gate_ch;
  P.gate_vals = a->gate_vals;
  // up to 8 splits (the portable cluster size) merge inside a thread-block cluster and need no workspace
  P.cluster = (allow_cluster && P.splits > 1 && P.splits <= 8 && cluster_merge_enabled()) ? 1 : 0;
  if (P.splits > 1 && !P.cluster) {
    const size_t need = uv_decode_attn_workspace_bytes(a->B, a->KH, G, hd, P.splits);
    if (!a->workspace || a->workspace_bytes < need) return UV_ERR_WORKSPACE;
    if (!aligned16(a->workspace)) return UV_ERR_ALIGN;
    const size_t rows = (size_t)a->B * a->KH * P.splits * G;
    P.ws_o = static_cast<float*>(a->workspace);
    P.ws_m = P.ws_o + rows * hd;
    P.ws_l = P.ws_m + rows;
  }
  const bool bulk = attn_bulk_ok(a);
  if (pre != nullptr) {
    // one launch needs: the bulk-copy path, a merge that runs inside the launch, and the step's RoPE table
    const bool ok = bulk && (P.splits == 1 || P.cluster || P.counters) && (!pre->inv_freq || pre->rope_cs);
    *fused = ok;
    if (!ok) return UV_OK;
    P.has_pre = 1;
    P.pre = *pre;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->q_dtype == UV_F16) return dispatch_hd<__half>(P, hd, bulk, st);
  return dispatch_hd<__nv_bfloat16>(P, hd, bulk, st);
}


// ------------------------------------------------------------------------------------------------ built-in scratch
extern "C" int uv_decode_attn(const uv_attn_args* a, void* stream) { return decode_attn_impl(a, stream, true); }

extern "C" int uv_qkv_attn(const uv_qkv_args* qa, const uv_attn_args* a, void* stream) {
  using namespace uv;
  if (!qa || !a) return UV_ERR_ARG;
  if (a->B == 0) return UV_OK;
  // the two argument blocks must describe the same step of the same cache
  const int slots = qa->H + 2 * qa->K;
  if (qa->B != a->B || qa->H != a->H || qa->K != a->KH || qa->hd != a->hd || qa->dtype != a->q_dtype ||
      qa->S != a->S || (qa->ring != 0) != (a->ring != 0) || qa->pos != a->pos || qa->row_map != a->row_map ||
      static_cast<const void*>(qa->k_cache) != a->k_cache || static_cast<const void*>(qa->v_cache) != a->v_cache ||
      qa->k_scale != a->k_scale || qa->v_scale != a->v_scale)
    return UV_ERR_ARG;
  // q and the current v are slots of the packed projection
  const size_t esz = 2;
  if (a->q != qa->qkv || a->sqb != (int64_t)slots * qa->hd || a->sqh != qa->hd) return UV_ERR_ARG;
  if (a->xsa_alpha &&
      (a->v_cur != static_cast<const char*>(qa->qkv) + (size_t)(qa->H + qa->K) * qa->hd * esz ||
       a->v_cur_sb != (int64_t)slots * qa->hd || a->v_cur_sh != qa->hd))
    return UV_ERR_ARG;
  // contiguous cache rows of S_alloc slots (what uv_qkv_post addresses) must be what the attention strides say
  const int s_alloc = qa->S_alloc > qa->S ? qa->S_alloc : qa->S;
  if (a->sks != a->hd || a->svs != a->hd || a->skh != (int64_t)s_alloc * a->hd || a->svh != a->skh ||
      a->skb != a->skh * a->KH || a->svb != a->skb || a->ssh != s_alloc || a->sth != s_alloc ||
      a->ssb != (int64_t)s_alloc * a->KH || a->stb != a->ssb)
    return UV_ERR_ARG;
  QkvPostParams qp{};
  int rc = qkv_post_params(&qp, qa->qkv, qa->xn, qa->tok, qa->value_embed, qa->ve_gate, qa->inv_freq, qa->pos,
                           qa->k_cache, qa->v_cache, qa->k_scale, qa->v_scale, qa->row_map, qa->oob_count, qa->vocab,
                           qa->B, qa->H, qa->K, qa->hd, qa->d, qa->S, qa->S_alloc, qa->ring, qa->ve_ch, qa->n_pairs);
  if (rc != UV_OK) return rc;
  if (!qa->k_cache) return UV_ERR_ARG;
  qp.rope_cs = qa->inv_freq ? qa->rope_cs : nullptr;  // without the table the two-launch form runs
  bool fused = false;
  rc = decode_attn_impl(a, stream, true, &qp, &fused);
  if (rc != UV_OK || fused) return rc;
  rc = uv_qkv_post(qa->qkv, qa->xn, qa->tok, qa->value_embed, qa->ve_gate, qa->inv_freq, qa->pos, qa->k_cache,
                   qa->v_cache, qa->k_scale, qa->v_scale, qa->row_map, qa->oob_count, qa->dtype, qa->vocab, qa->B,
                   qa->H, qa->K, qa->hd, qa->d, qa->S, qa->S_alloc, qa->ring, qa->ve_ch, qa->n_pairs, stream);
  if (rc != UV_OK) return rc;
  return decode_attn_impl(a, stream, true);
}

// uv_decode_attn_static: split-K decode attention for callers that may not allocate device memory at all.
// The split partials and the arrival counters live in this file-scope device array instead of a caller workspace.
// Every GPU that loads the library holds the array (4 MiB + 16 KiB) until the process exits.
#define UV_STATIC_PARTIAL_BYTES (4u << 20)
#define UV_STATIC_MAX_ROWS 4096
static __device__ __align__(256) unsigned char uv_static_scratch[UV_STATIC_PARTIAL_BYTES +
                                                                 UV_STATIC_MAX_ROWS * sizeof(int)];

namespace uv {
constexpr int MAX_DEVICES = 64;
static void* g_static_ptr[MAX_DEVICES] = {nullptr};
static std::mutex g_static_mu;

// Device address of uv_static_scratch on the CURRENT device.  The array's name is only a host-side handle; the
// address a kernel can use comes from cudaGetSymbolAddress, looked up once per device and cached.
static int static_scratch_ptr(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    set_last_cuda_error((int)(e != cudaSuccess ? e : cudaErrorInvalidDevice));
    return UV_ERR_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, uv_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_cuda_error((int)e);
      return UV_ERR_CUDA;
    }
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return UV_OK;
}
}  // namespace uv

extern "C" int uv_decode_attn_static(const uv_attn_args* a, void* stream) {
  using namespace uv;
  if (!a) return UV_ERR_ARG;
  if (a->B <= 0 || a->KH <= 0 || a->H <= 0 || a->num_splits < 1) return a->B == 0 ? UV_OK : UV_ERR_ARG;
  if (a->H % a->KH) return UV_ERR_ARG;
  const size_t need = uv_decode_attn_workspace_bytes(a->B, a->KH, a->H / a->KH, a->hd, a->num_splits);
  if (need > UV_STATIC_PARTIAL_BYTES || (int64_t)a->B * a->KH > UV_STATIC_MAX_ROWS) return UV_ERR_STATIC_LIMIT;
  void* base = nullptr;
  const int rc = static_scratch_ptr(&base);
  if (rc != UV_OK) return rc;
  uv_attn_args b = *a;
  b.workspace = base;
  b.workspace_bytes = UV_STATIC_PARTIAL_BYTES;
  b.counters = nullptr;
  if (a->num_splits > 1) {
    // the array keeps whatever the previous call left: the arrival counters must start at zero
    b.counters = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + UV_STATIC_PARTIAL_BYTES);
    cudaError_t e = cudaMemsetAsync(b.counters, 0, (size_t)a->B * a->KH * sizeof(int),
                                    static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
      set_last_cuda_error((int)e);
      return UV_ERR_CUDA;
    }
  }
  return decode_attn_impl(&b, stream, false);  // the split partials go through the built-in array
}
