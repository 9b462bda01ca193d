// Decode-step GEMMs on the 5th-generation tensor cores with the step's row-wise kernels fused into their epilogues
// (sm_100a: tcgen05.mma + TMEM accumulators + TMA operand tiles).
//
// Tiling ("weights on the lanes"): C^T = W . X^T.  The MMA's M dimension is 128 rows of the WEIGHT matrix (one output
// feature per TMEM lane), its N dimension a tile of BN batch rows.  A CTA therefore streams a slab of weights that
// no other CTA of its batch tile reads, and the part of its traffic that depends on the previous kernel -- the BN
// activation rows -- is small.  That split is what makes programmatic dependent launch pay: the CTA is scheduled
// while its predecessor drains, allocates TMEM, and requests its WEIGHT tiles (which no kernel of the step writes)
// before griddepcontrol.wait; only the activation tiles are requested after it.
//
// Split-K: the K range can be cut over a thread-block cluster (grid.z = cluster.z = KS <= 8).  Every CTA leaves its
// fp32 partial tile in its own shared memory; after one cluster barrier rank r sums batch columns
// [r * BN / KS, (r + 1) * BN / KS) of all partials through distributed shared memory (all KS loads in flight at once)
// and runs the epilogue for them.  (Pushing the columns to their owners with st.shared::cluster instead measured
// 1.5-2 us slower per launch: 32 scalar remote stores per thread.)
//
// Epilogues (thread = TMEM lane = feature reads its BN columns, scales them, and parks them transposed in shared
// memory; then a warp owns a batch row of 128 features):
//   STORE    c = acc                                               (building block / tests)
//   QKV      everything uv_qkv_post does for the two 64-wide head slots of the tile: per-head RMS norm, RoPE,
//            value-embedding gate, int8 quantise + cache append, attention head gates
//   SWIGLU   act = silu(g) * u for a tile of 64 gate + 64 up features
//   RESID    h = l0 * x + l1 * acc (Block.finish, ultraviolet/model.py:567-571) + this tile's share of sum(h^2)
// "Deferred RMS norm": the GEMMs that consume a normalised activation (QKV, gate|up, LM head) read the UN-normalised
// residual stream and multiply their accumulator columns by rs[b] = rsqrt(mean(h[b]^2) + eps), assembled from the
// per-tile sums of squares the producing RESID epilogue (or uv_embed_norm) left behind.  No kernel of the step then
// needs a whole activation row at once, so nothing has to reduce across CTAs.
//
// Every mbarrier wait is bounded (200 ms); a wait that runs out sets status bit 2, the CTA skips its stores, still
// joins the cluster barriers its peers count on and frees its TMEM columns.
#include "qkv_post.cuh"
#include "tcgen05.cuh"

namespace uv {

constexpr int SW_THREADS = 128;
constexpr int SW_MAX_STAGES = 12;
constexpr int SW_PITCH = 132;  // floats per transposed row: 128 features + 4 (keeps 16-byte alignment, skews banks)

enum { SW_EPI_STORE = 0, SW_EPI_QKV = 1, SW_EPI_SWIGLU = 2, SW_EPI_RESID = 3 };

struct GemmSwParams {
  int M, N, K;             // batch rows, weight rows covered by the launch, reduction length
  int stages, ksplit;
  int* status;
  // deferred norm of the INPUT activation: rs[b] = rsqrt(sum_j ss_in[j * ss_in_ld + b] / ss_in_dim + eps)
  const float* ss_in;
  int ss_in_parts, ss_in_ld, ss_in_dim;
  // 1: no producer left sums of squares behind -- the CTA forms sum(x[b]^2) over its K range from the activation
  // tiles it holds in shared memory anyway (every K block of the CTA must stay resident: stages >= its K blocks)
  // and the ranks of a split-K cluster add their parts up through distributed shared memory
  int ss_self;
  int pdl;                 // host side only: -1 process default, 0 / 1 launch without / with the PDL attribute
  // STORE / SWIGLU / RESID output (M, ldo)
  void* out;
  int64_t ldo;
  int f;                   // SWIGLU: features (weight rows f + n are the "up" rows of gate row n)
  // RESID
  const void* resid;       // x (M, ldo)
  const float* lambdas;    // l0, l1
  float* ss_out;           // (N / 128, ss_out_ld): sum of h^2 over this tile's 128 features
  int ss_out_ld;
  // QKV
  QkvPostParams post;      // post.xn = the un-normalised residual stream (its rows are scaled by rs[b] on the fly)
};

__device__ __forceinline__ void sw_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float sw_ld_peer_f1(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ float2 sw_ld_peer_f2(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float2 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ float4 sw_ld_peer_f4(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// grid (N / 128 [SWIGLU: f / 64], ceil(M / BN), ksplit); cluster (1, 1, ksplit)
// NT threads: warps 0..3 run the main loop (copy thread, MMA thread, row factors) and read the accumulator out of
// TMEM; warps 4.. (QKV epilogue only) do nothing until the accumulator is parked in shared memory and then take
// their share of the epilogue's (row, head slot) items, each of which is a ~1 us chain of dependent shuffles and
// loads that only parallelism across warps hides.
template <int BN, int EPI, int NT>
__global__ void __launch_bounds__(NT) gemm_sw_kernel(const __grid_constant__ CUtensorMap tm_w,
                                                     const __grid_constant__ CUtensorMap tm_x,
                                                     const GemmSwParams P) {
  using T = __nv_bfloat16;
  constexpr int W_BYTES = 128 * TC_BK * 2;   // 16 KB of weights per K block
  constexpr int X_BYTES = BN * TC_BK * 2;
  constexpr int STAGE = W_BYTES + X_BYTES;
  constexpr int TCOLS = BN < 32 ? 32 : BN;   // TMEM columns: a power of two >= 32
  extern __shared__ __align__(1024) unsigned char sw_smem[];
  __shared__ __align__(8) uint64_t full_bar[SW_MAX_STAGES], empty_bar[SW_MAX_STAGES], accum_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ float rs_sm[BN];
  __shared__ float ssp_sm[BN];   // ss_self: this CTA's share of sum(x[b]^2)
  __shared__ int dead_sm;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ft = blockIdx.x, b0 = blockIdx.y * BN, kr = blockIdx.z;
  const int n0 = EPI == SW_EPI_SWIGLU ? ft * 64 : ft * 128;
  const int nk_all = P.K / TC_BK;
  const int per = (nk_all + P.ksplit - 1) / P.ksplit;
  const int kb0 = kr * per;
  const int nk = nk_all - kb0 < per ? (nk_all - kb0 > 0 ? nk_all - kb0 : 0) : per;
  const int NS = P.stages;
  const uint32_t base = (tc_smem_u32(sw_smem) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      tc_mbar_init(tc_smem_u32(&full_bar[s]), 1);
      tc_mbar_init(tc_smem_u32(&empty_bar[s]), 1);
    }
    tc_mbar_init(tc_smem_u32(&accum_bar), 1);
    dead_sm = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_slot)),
                 "r"((uint32_t)TCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  pdl_trigger();   // the next kernel of the step may be scheduled now: it only touches its own weights until its wait

  auto load_w = [&](int kb, int s) {
    const uint32_t bar = tc_smem_u32(&full_bar[s]);
    const uint32_t sw = base + (uint32_t)s * STAGE;
    tc_mbar_expect_tx(bar, (uint32_t)STAGE);
    if constexpr (EPI == SW_EPI_SWIGLU) {
      tc_tma_load_2d(sw, &tm_w, (kb0 + kb) * TC_BK, n0, bar);                       // 64 gate rows
      tc_tma_load_2d(sw + W_BYTES / 2, &tm_w, (kb0 + kb) * TC_BK, P.f + n0, bar);   // the same features' up rows
    } else {
      tc_tma_load_2d(sw, &tm_w, (kb0 + kb) * TC_BK, n0, bar);
    }
  };
  auto load_x = [&](int kb, int s) {
    tc_tma_load_2d(base + (uint32_t)s * STAGE + W_BYTES, &tm_x, (kb0 + kb) * TC_BK, b0, tc_smem_u32(&full_bar[s]));
  };

  bool ok = true;
  const int pre = nk < NS ? nk : NS;  // K blocks whose weights are requested before the predecessor has finished
  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_x) : "memory");
    for (int kb = 0; kb < pre; ++kb) load_w(kb, kb);
  }
  pdl_wait();      // everything below may read what the previous kernel wrote

  if (warp == 0 && lane == 0) {
    // ---- copy thread
    for (int kb = 0; kb < pre; ++kb) load_x(kb, kb);
    for (int kb = pre; kb < nk; ++kb) {
      const int s = kb % NS;
      if (!tc_mbar_wait(tc_smem_u32(&empty_bar[s]), (uint32_t)((kb / NS - 1) & 1))) {
        ok = false;
        break;
      }
      load_w(kb, s);
      load_x(kb, s);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA thread
    const uint32_t idesc = tc_idesc(128, BN);
    for (int kb = 0; kb < nk; ++kb) {
      const int s = kb % NS;
      if (!tc_mbar_wait(tc_smem_u32(&full_bar[s]), (uint32_t)((kb / NS) & 1))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t sw = base + (uint32_t)s * STAGE, sx = sw + W_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k)
        tc_mma(tmem, tc_smem_desc(sw + k * 32), tc_smem_desc(sx + k * 32), idesc, (uint32_t)((kb | k) != 0));
      tc_commit(tc_smem_u32(&empty_bar[s]));
    }
    if (ok && nk > 0) tc_commit(tc_smem_u32(&accum_bar));
  } else if (warp == 2 || warp == 3) {
    // ---- the other two main-loop warps: rs[b] of this CTA's batch rows from the producer's per-tile sums of squares, or
    //      (ss_self) the sums of squares themselves, read off the activation tiles as they land: a batch row of a K
    //      block is one 128-byte row of the tile (the swizzle permutes 16-byte pieces inside it, which a sum ignores)
    if (P.ss_self) {
      // 8 lanes share a row (one 16-byte piece each: a warp reads 4 whole rows = 512 contiguous bytes per load)
      constexpr int PASSES = (BN + 7) / 8;   // 64 threads cover 8 rows per pass
      float part[PASSES];
#pragma unroll
      for (int i = 0; i < PASSES; ++i) part[i] = 0.f;
      const int t64 = tid - 64;
      for (int kb = 0; kb < nk && ok; ++kb) {
        const int s = kb % NS;
        if (!tc_mbar_wait(tc_smem_u32(&full_bar[s]), (uint32_t)((kb / NS) & 1))) {
          ok = false;
          break;
        }
        const unsigned char* xt = sw_smem + (base - tc_smem_u32(sw_smem)) + (size_t)s * STAGE + W_BYTES;
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
          const int j = i * 8 + (t64 >> 3);
          if (j < BN) {
            const uint4 u = *reinterpret_cast<const uint4*>(xt + (size_t)j * 128 + (t64 & 7) * 16);
            const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[e]));
              part[i] += f.x * f.x + f.y * f.y;
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < PASSES; ++i) {
        float v = part[i];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        const int j = i * 8 + (t64 >> 3);
        if ((t64 & 7) == 0 && j < BN) ssp_sm[j] = v;
      }
    }
    for (int j = tid - 64; j < BN; j += 64) {
      float r = 1.0f;
      if (P.ss_in != nullptr && b0 + j < P.M) {
        float ss = 0.f;
        for (int p = 0; p < P.ss_in_parts; ++p) ss += P.ss_in[(int64_t)p * P.ss_in_ld + b0 + j];
        r = rsqrtf(ss / (float)P.ss_in_dim + RMS_EPS);
      }
      rs_sm[j] = r;
    }
  }
  __syncwarp();
  const int rows_per = BN / P.ksplit;
  if constexpr (EPI == SW_EPI_QKV) {
    // While the accumulator is still being formed: pull what this warp's epilogue rows will read (positions, cache
    // rows, the rotation table row, the gate inputs and weights, the value-embedding row) towards the SM, so that the
    // epilogue's dependent loads find them close by instead of paying an L2 round trip each, item after item.
    const QkvPostParams& Q = P.post;
    auto pf = [](const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); };
    const int slots = Q.H + 2 * Q.K;
    for (int it = warp; it < 2 * rows_per; it += NT / 32) {
      const int b = b0 + kr * rows_per + (it >> 1);
      if (b >= P.M) continue;
      if (lane == 0) pf(Q.pos + b);
      if (lane == 1 && Q.row_map) pf(Q.row_map + b);
      if (lane == 2 && Q.last_pos) pf(Q.last_pos + b);
      if (lane == 3 && Q.rope_cs) pf(Q.rope_cs + (int64_t)b * 2 * Q.n_pairs);
      if (lane >= 4 && lane < 8 && Q.xn) {  // the first channels of the row: head gates and the value-embedding gate
        const int off = (lane - 4) * 64;
        if (off < Q.d) pf(static_cast<const T*>(Q.xn) + (int64_t)b * Q.d + off);
      }
      if (lane >= 8 && lane < 10) {         // gate weights of the item's head slot
        const int hs = 2 * ft + (it & 1), off = (lane - 8) * 64;
        if (hs < Q.H && Q.gate_out != nullptr && off < Q.gate_ch)
          pf(static_cast<const T*>(Q.gate_w) + (int64_t)hs * Q.gate_ch + off);
      }
      if (lane == 12 && Q.ve_gate != nullptr) {
        const int hs = 2 * ft + (it & 1);
        if (hs >= Q.H + Q.K && hs < slots) {
          const int kh = hs - Q.H - Q.K;
          pf(static_cast<const T*>(Q.ve_gate) + (int64_t)kh * Q.ve_ch);
          int64_t t = Q.tok[b];
          if (t < 0 || t >= Q.vocab) t = 0;
          pf(static_cast<const T*>(Q.value_embed) + (t * Q.K + kh) * 64);
        }
      }
    }
  }
  if (nk > 0 && warp < 4) ok = tc_mbar_wait(tc_smem_u32(&accum_bar), 0) && ok;  // warps 4.. sleep at the barrier below
  if (!ok) dead_sm = 1;
  tc_fence_after();
  __syncthreads();
  const bool dead = dead_sm != 0;
  if (dead && tid == 0 && P.status) atomicOr(P.status, 4);

  // ---- stage 1: thread = feature (TMEM lane) parks its BN columns, transposed, as T32[b][feature] behind the
  //      stage ring
  float* T32 = reinterpret_cast<float*>(sw_smem + (base - tc_smem_u32(sw_smem)) + (size_t)NS * STAGE);
  const uint32_t t32_addr = tc_smem_u32(T32);
  if (!dead && warp < 4) {
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t v[32];
      if (nk > 0) {
        tc_ld32(taddr + c0, v);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) T32[(c0 + j) * SW_PITCH + tid] = __uint_as_float(v[j]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TCOLS) : "memory");
  if (P.ksplit > 1) sw_cluster_sync();

  // ---- stage 2: rank kr finishes batch rows [kr * rows_per, (kr + 1) * rows_per) of the tile; a warp owns a row,
  //      a lane 4 consecutive features
  auto row_factor = [&](int bl) {
    float rs = rs_sm[bl];
    if (P.ss_self) {
      float ss = 0.f;
      if (P.ksplit > 1) {
        const uint32_t a = tc_smem_u32(&ssp_sm[bl]);
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if (p < P.ksplit) ss += sw_ld_peer_f1(a, (uint32_t)p);
      } else {
        ss = ssp_sm[bl];
      }
      rs = rsqrtf(ss / (float)P.K + RMS_EPS);
    }
    return rs;
  };
  if constexpr (EPI == SW_EPI_QKV) {
    // an item = one 64-wide head slot of one batch row (two slots per 128-feature tile); lane l holds features
    // 2l, 2l + 1 of the slot, as the row kernels do
    const QkvPostParams& Q = P.post;
    const int slots = Q.H + 2 * Q.K;
    if (!dead)
      for (int it = warp; it < 2 * rows_per; it += NT / 32) {
        const int bl = kr * rows_per + (it >> 1), b = b0 + bl, hs = 2 * ft + (it & 1);
        if (b >= P.M || hs >= slots) continue;  // warp-uniform
        float2 acc;
        if (P.ksplit > 1) {
          float2 q[8];
          const uint32_t a = t32_addr + (uint32_t)(bl * SW_PITCH + (it & 1) * 64 + 2 * lane) * 4u;
#pragma unroll
          for (int p = 0; p < 8; ++p)
            if (p < P.ksplit) q[p] = sw_ld_peer_f2(a, (uint32_t)p);
          acc = q[0];
#pragma unroll
          for (int p = 1; p < 8; ++p)
            if (p < P.ksplit) acc.x += q[p].x, acc.y += q[p].y;
        } else {
          acc = *reinterpret_cast<const float2*>(T32 + bl * SW_PITCH + (it & 1) * 64 + 2 * lane);
        }
        const float rs = row_factor(bl);
        float x[2] = {rnd<T>(acc.x * rs), rnd<T>(acc.y * rs)};  // the projection as the reference holds it (rounded)
        qkv_post_compute<T, 64, true>(Q, b, hs, lane, x, rs, true);
        T* vec = static_cast<T*>(Q.qkv) + ((int64_t)b * slots + hs) * 64;
        *reinterpret_cast<__nv_bfloat162*>(vec + 2 * lane) = __floats2bfloat162_rn(x[0], x[1]);
        if (hs >= Q.H && Q.k_cache != nullptr) qkv_post_append<T, 64>(Q, b, hs, lane, x);
        if (hs < Q.H && Q.gate_out != nullptr) {
          const float gt = head_gate<T>(static_cast<const T*>(Q.xn) + (int64_t)b * Q.d,
                                        static_cast<const T*>(Q.gate_w) + (int64_t)hs * Q.gate_ch, Q.gate_ch, lane,
                                        rs, true);
          if (lane == 0) Q.gate_out[(int64_t)b * Q.H + hs] = gt;
        }
      }
  } else if (!dead)
    for (int rr = warp; rr < rows_per; rr += NT / 32) {
      const int bl = kr * rows_per + rr, b = b0 + bl;
      if (b >= P.M) continue;  // warp-uniform
      float4 acc;
      if (P.ksplit > 1) {
        float4 q[8];
        const uint32_t a = t32_addr + (uint32_t)(bl * SW_PITCH + 4 * lane) * 4u;
#pragma unroll
        for (int p = 0; p < 8; ++p)
          if (p < P.ksplit) q[p] = sw_ld_peer_f4(a, (uint32_t)p);
        acc = q[0];
#pragma unroll
        for (int p = 1; p < 8; ++p)
          if (p < P.ksplit) acc.x += q[p].x, acc.y += q[p].y, acc.z += q[p].z, acc.w += q[p].w;
      } else {
        acc = *reinterpret_cast<const float4*>(T32 + bl * SW_PITCH + 4 * lane);
      }
      const float rs = row_factor(bl);
      // the GEMM result as the reference holds it: rounded to the activation dtype
      float c[4] = {rnd<T>(acc.x * rs), rnd<T>(acc.y * rs), rnd<T>(acc.z * rs), rnd<T>(acc.w * rs)};
      if constexpr (EPI == SW_EPI_STORE) {
        T* o = static_cast<T*>(P.out) + (int64_t)b * P.ldo + n0 + 4 * lane;
        const __nv_bfloat162 h0 = __floats2bfloat162_rn(c[0], c[1]), h1 = __floats2bfloat162_rn(c[2], c[3]);
        *reinterpret_cast<uint2*>(o) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
      } else if constexpr (EPI == SW_EPI_RESID) {
        const T* xr = static_cast<const T*>(P.resid) + (int64_t)b * P.ldo + n0 + 4 * lane;
        const uint2 xu = *reinterpret_cast<const uint2*>(xr);
        const __nv_bfloat162 x0 = *reinterpret_cast<const __nv_bfloat162*>(&xu.x);
        const __nv_bfloat162 x1 = *reinterpret_cast<const __nv_bfloat162*>(&xu.y);
        const float xv[4] = {__bfloat162float(x0.x), __bfloat162float(x0.y), __bfloat162float(x1.x),
                             __bfloat162float(x1.y)};
        const float l0 = P.lambdas[0], l1 = P.lambdas[1];
        float hv[4], ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          hv[i] = rnd<T>(rnd<T>(l0 * xv[i]) + rnd<T>(l1 * c[i]));
          ss += hv[i] * hv[i];
        }
        T* o = static_cast<T*>(P.out) + (int64_t)b * P.ldo + n0 + 4 * lane;
        const __nv_bfloat162 h0 = __floats2bfloat162_rn(hv[0], hv[1]), h1 = __floats2bfloat162_rn(hv[2], hv[3]);
        *reinterpret_cast<uint2*>(o) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        ss = warp_sum(ss);
        if (lane == 0) P.ss_out[(int64_t)ft * P.ss_out_ld + b] = ss;
      } else if constexpr (EPI == SW_EPI_SWIGLU) {
        // features 0..63 of the tile are gate rows, 64..127 the up rows of the same features: lanes 0..15 hold
        // gates 4*lane.., lanes 16..31 the matching ups
        float u[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) u[i] = __shfl_down_sync(0xffffffffu, c[i], 16);
        if (lane < 16) {
          float a[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) a[i] = rnd<T>(c[i] / (1.0f + __expf(-c[i]))) * u[i];
          T* o = static_cast<T*>(P.out) + (int64_t)b * P.ldo + n0 + 4 * lane;
          const __nv_bfloat162 h0 = __floats2bfloat162_rn(a[0], a[1]), h1 = __floats2bfloat162_rn(a[2], a[3]);
          *reinterpret_cast<uint2*>(o) =
              make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
        }
      }
    }
  if (P.ksplit > 1) sw_cluster_sync();  // peers may still be reading this CTA's partial
}

template <int BN, int EPI>
static int launch_sw(const CUtensorMap& tw, const CUtensorMap& tx, const GemmSwParams& P, dim3 grid, cudaStream_t st) {
  // QKV epilogue: one warp per (row, slot) item of the CTA where the register file allows (2 * BN / ksplit items)
  constexpr int NT = EPI == SW_EPI_QKV ? 512 : SW_THREADS;
  auto kern = gemm_sw_kernel<BN, EPI, NT>;
  const size_t ring = (size_t)P.stages * (128 * TC_BK * 2 + BN * TC_BK * 2);
  const size_t t32 = (size_t)BN * SW_PITCH * sizeof(float);
  const size_t smem = ring + t32 + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_last_cuda_error((int)e);
    return UV_ERR_CUDA;
  }
  launch_cluster_pdl(P.pdl, kern, grid, dim3(NT), dim3(1, 1, (unsigned)P.ksplit), smem, st, tw, tx, P);
  return check_launch();
}

// BN / split-K / stage choice: enough CTAs to cover the SMs once, all of a CTA's K blocks resident when they fit
static void sw_plan(int M, int n_tiles, int K, int bn_hint, int ks_hint, int* bn, int* ks, int* stages) {
  int b = bn_hint > 0 ? bn_hint : (M <= 320 ? 32 : 64);
  const int btiles = (M + b - 1) / b;
  const int nk = K / TC_BK;
  int s = ks_hint > 0 ? ks_hint : 1;
  if (ks_hint <= 0) {
    while (s < 8 && n_tiles * btiles * s * 2 <= 148 && nk / (s * 2) >= 2 && b % (s * 2) == 0) s *= 2;
  }
  while (s > 1 && (b % s != 0)) --s;
  const int per = (nk + s - 1) / s;
  const size_t stage = (size_t)128 * TC_BK * 2 + (size_t)b * TC_BK * 2;
  int st = per;
  const int cap = (int)((220 * 1024 - (size_t)b * SW_PITCH * sizeof(float)) / stage);
  if (st > cap) st = cap;
  if (st > SW_MAX_STAGES) st = SW_MAX_STAGES;
  if (st < 1) st = 1;
  *bn = b, *ks = s, *stages = st;
}

static int sw_checks(const void* x, int64_t ldx, const void* w, int M, int N, int K) {
  if (!x || !w || M < 1 || N < 1 || K < 1) return UV_ERR_ARG;
  if (K % TC_BK || N % 128) return UV_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(w) || (ldx * 2) % 16) return UV_ERR_ALIGN;
  return UV_OK;
}

static void sw_norm_in(GemmSwParams& P, const float* ss_in, int parts, int ld, int dim) {
  P.ss_in = ss_in, P.ss_in_parts = parts, P.ss_in_ld = ld, P.ss_in_dim = dim;
}

#define UV_SW_DISPATCH(EPI_, grid_)                                                     \
  do {                                                                                  \
    if (bn == 32) return launch_sw<32, EPI_>(tw, tx, P, grid_, st);                     \
    if (bn == 64) return launch_sw<64, EPI_>(tw, tx, P, grid_, st);                     \
    if (bn == 128) return launch_sw<128, EPI_>(tw, tx, P, grid_, st);                   \
    return UV_ERR_SHAPE;                                                                \
  } while (0)

}  // namespace uv

using namespace uv;

extern "C" int uv_gemm_sw(const void* x, int64_t ldx, const void* w, void* c, int64_t ldc, int dtype, int M, int N,
                          int K, const float* ss_in, int ss_parts, int ss_ld, int bn_hint, int ks_hint, int* status,
                          void* stream) {
  if (M == 0 || N == 0) return UV_OK;
  if (dtype != UV_BF16) return UV_ERR_DTYPE;
  int rc = sw_checks(x, ldx, w, M, N, K);
  if (rc != UV_OK) return rc;
  if (!c || (ldc & 3)) return UV_ERR_ALIGN;
  int bn, ks, stages;
  sw_plan(M, N / 128, K, bn_hint, ks_hint, &bn, &ks, &stages);
  CUtensorMap tw, tx;
  if (!make_map(&tw, w, N, K, K, 128) || !make_map(&tx, x, M, K, ldx, bn)) return UV_ERR_CUDA;
  GemmSwParams P{};
  P.pdl = -1;
  P.M = M, P.N = N, P.K = K, P.stages = stages, P.ksplit = ks, P.status = status, P.out = c, P.ldo = ldc;
  sw_norm_in(P, ss_in, ss_parts, ss_ld, K);
  const dim3 grid((unsigned)(N / 128), (unsigned)((M + bn - 1) / bn), (unsigned)ks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  UV_SW_DISPATCH(SW_EPI_STORE, grid);
}

extern "C" int uv_gemm_sw_resid(const void* a, int64_t lda, const void* w, const void* x, const float* lambdas,
                                void* h, int64_t ldh, float* ss_out, int ss_out_ld, int dtype, int M, int N, int K,
                                int bn_hint, int ks_hint, int* status, void* stream) {
  if (M == 0 || N == 0) return UV_OK;
  if (dtype != UV_BF16) return UV_ERR_DTYPE;
  int rc = sw_checks(a, lda, w, M, N, K);
  if (rc != UV_OK) return rc;
  if (!x || !lambdas || !h || !ss_out || (ldh & 3) || ss_out_ld < M) return UV_ERR_ARG;
  int bn, ks, stages;
  sw_plan(M, N / 128, K, bn_hint, ks_hint, &bn, &ks, &stages);
  CUtensorMap tw, tx;
  if (!make_map(&tw, w, N, K, K, 128) || !make_map(&tx, a, M, K, lda, bn)) return UV_ERR_CUDA;
  GemmSwParams P{};
  P.pdl = -1;
  P.M = M, P.N = N, P.K = K, P.stages = stages, P.ksplit = ks, P.status = status, P.out = h, P.ldo = ldh;
  P.resid = x, P.lambdas = lambdas, P.ss_out = ss_out, P.ss_out_ld = ss_out_ld;
  const dim3 grid((unsigned)(N / 128), (unsigned)((M + bn - 1) / bn), (unsigned)ks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  UV_SW_DISPATCH(SW_EPI_RESID, grid);
}

extern "C" int uv_gemm_sw_swiglu(const void* h, int64_t ldh, const void* w_gu, void* act, int dtype, int M, int K,
                                 int f, const float* ss_in, int ss_parts, int ss_ld, int bn_hint, int* status,
                                 void* stream) {
  if (M == 0 || f == 0) return UV_OK;
  if (dtype != UV_BF16) return UV_ERR_DTYPE;
  int rc = sw_checks(h, ldh, w_gu, M, 128, K);
  if (rc != UV_OK) return rc;
  if (!act || f % 64) return UV_ERR_SHAPE;
  int bn, ks, stages;
  sw_plan(M, f / 64, K, bn_hint, 1, &bn, &ks, &stages);
  CUtensorMap tw, tx;
  if (!make_map(&tw, w_gu, 2 * (int64_t)f, K, K, 64) || !make_map(&tx, h, M, K, ldh, bn)) return UV_ERR_CUDA;
  GemmSwParams P{};
  P.pdl = -1;
  P.M = M, P.N = 2 * f, P.K = K, P.stages = stages, P.ksplit = 1, P.status = status, P.out = act, P.ldo = f, P.f = f;
  sw_norm_in(P, ss_in, ss_parts, ss_ld, K);
  const dim3 grid((unsigned)(f / 64), (unsigned)((M + bn - 1) / bn), 1u);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  UV_SW_DISPATCH(SW_EPI_SWIGLU, grid);
}

extern "C" int uv_gemm_sw_qkv(const void* x, int64_t ldx, const void* wqkv, const uv_qkv_args* qa, const float* ss_in,
                              int ss_parts, int ss_ld, int bn_hint, int ks_hint, int* status, void* stream) {
  if (!qa) return UV_ERR_ARG;
  if (qa->B == 0) return UV_OK;
  if (qa->dtype != UV_BF16) return UV_ERR_DTYPE;
  if (qa->hd != 64) return UV_ERR_SHAPE;
  const int M = qa->B, K = qa->d, slots = qa->H + 2 * qa->K;
  const int N = (slots * 64 + 127) / 128 * 128;  // an odd slot count leaves the last tile half used
  if ((slots & 1) != 0) return UV_ERR_SHAPE;     // (the weight rows of such a tile would not exist)
  int rc = sw_checks(x, ldx, wqkv, M, N, K);
  if (rc != UV_OK) return rc;
  if (qa->inv_freq && !qa->rope_cs) return UV_ERR_ARG;  // RoPE layers need the step's table
  GemmSwParams P{};
  P.pdl = -1;
  rc = qkv_post_params(&P.post, qa->qkv, x, qa->tok, qa->value_embed, qa->ve_gate, qa->inv_freq, qa->pos, qa->k_cache,
                       qa->v_cache, qa->k_scale, qa->v_scale, qa->row_map, qa->oob_count, qa->vocab, qa->B, qa->H,
                       qa->K, qa->hd, qa->d, qa->S, qa->S_alloc, qa->ring, qa->ve_ch, qa->n_pairs);
  if (rc != UV_OK) return rc;
  P.post.rope_cs = qa->inv_freq ? qa->rope_cs : nullptr;
  P.post.last_pos = qa->last_pos;
  if (qa->gate_out) {
    if (!qa->gate_w || qa->gate_ch < 1 || qa->gate_ch > qa->d) return UV_ERR_ARG;
    P.post.gate_w = qa->gate_w, P.post.gate_out = qa->gate_out, P.post.gate_ch = qa->gate_ch;
  }
  int bn, ks, stages;
  sw_plan(M, N / 128, K, bn_hint, ks_hint, &bn, &ks, &stages);
  CUtensorMap tw, tx;
  if (!make_map(&tw, wqkv, N, K, K, 128) || !make_map(&tx, x, M, K, ldx, bn)) return UV_ERR_CUDA;
  P.M = M, P.N = N, P.K = K, P.stages = stages, P.ksplit = ks, P.status = status;
  sw_norm_in(P, ss_in, ss_parts, ss_ld, K);
  if (!ss_in) {
    // no producer of sums of squares (the residual stream was updated by a library GEMM): the kernel forms them
    // from its own activation tiles, which must all stay resident; its weight tiles are worth requesting while the
    // predecessor drains, so this launch carries the PDL attribute whatever the process default is
    while (stages < (K / TC_BK + ks - 1) / ks && ks < 8 && ks_hint <= 0) {  // cut K further until a CTA's share fits
      sw_plan(M, N / 128, K, bn, ks * 2, &bn, &ks, &stages);
      P.stages = stages, P.ksplit = ks;
    }
    if (stages < (K / TC_BK + ks - 1) / ks) return UV_ERR_SHAPE;
    P.ss_self = 1, P.ss_in_dim = K;
    P.pdl = ss_parts < 0 ? 0 : 1;   // ss_parts = -1 with a null ss_in: launch without the attribute (A/B switch)
  }
  const dim3 grid((unsigned)(N / 128), (unsigned)((M + bn - 1) / bn), (unsigned)ks);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  UV_SW_DISPATCH(SW_EPI_QKV, grid);
}
