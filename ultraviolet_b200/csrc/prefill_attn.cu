// Packed variable-length causal attention for prompt prefill, sm_100a.
//
// The prompts of a refill batch are packed back to back into one (M, (H + 2K) * hd) matrix of post-processed
// q | k | v rows (uv_qkv_post has normalised / rotated q and k and added the value embedding to v, and has written
// the int8 cache entries).  Token i of a sequence attends to tokens max(0, i - window + 1) .. i of the SAME sequence,
// using the UNQUANTISED keys and values of the chunk -- what the reference's prefill does (its trunk runs SDPA or
// the packed varlen kernel on the activations and quantises only what it stores:
// ultraviolet/kernels/fast_decode.py:70-163, ultraviolet/kernels/varlen_attn.py:38-92).
//
// One CTA = 16 query tokens of one sequence x one kv head; warp g owns query head h*G + g, so the G heads of a group
// share every key / value tile that the CTA stages (GQA).  Keys stream through shared memory in 64-key tiles with
// two-stage cp.async; S = Q K^T and O += P V run on the tensor cores (mma.sync.m16n8k16, fp32 accumulation) with
// ldmatrix operand fetches from padded rows; online softmax in fp32; the epilogue is the decode kernel's (XSA with
// the token's own v, per-head output gate, Attention.post: ultraviolet/model.py:322-333).
//
// Tiles are found from two prefix-sum arrays that either the host or the device scheduler builds: cu_seqlens
// (first packed row of every sequence) and tile_cu (first 16-token tile of every sequence); blocks past the last
// tile exit.  Nothing here waits on anything but its own cp.async groups.
#include "common.cuh"

namespace uv {

constexpr int PF_QT = 16;   // query tokens per CTA
constexpr int PF_KT = 64;   // keys per shared-memory tile

struct PrefillAttnParams {
  const void* qkv;
  int64_t ld;                // row stride of qkv, elements
  const int32_t* cu_seqlens; // (n_seq + 1)
  const int32_t* tile_cu;    // (n_seq + 1): tile_cu[s] = sum over s' < s of ceil(len_s' / 16)
  int n_seq;
  void* out;                 // (M, H * hd)
  int64_t ldo;
  int H, K, G, window;
  float scale_log2;
  const float* xsa_alpha;    // (H,) or null
  float xsa_eps;
  const float* gate_vals;    // (M, H) or null
};

template <typename T> struct MmaType;
template <> struct MmaType<__half> {
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};
template <> struct MmaType<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
};

__device__ __forceinline__ uint32_t pf_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pf_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void pf_ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ float pf_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// grid (n_tiles upper bound, K); block 32 * G threads
template <typename QT, int HD>
__global__ void __launch_bounds__(512) prefill_attn_kernel(const __grid_constant__ PrefillAttnParams P) {
  constexpr int ROWB = HD * 2 + 16;       // padded shared-memory row (bytes): conflict-free ldmatrix, 16-byte aligned
  constexpr int TILEB = PF_KT * ROWB;     // one K (or V) tile
  constexpr int KS = HD / 16;             // k16 steps of Q K^T
  constexpr int NT_S = PF_KT / 8;         // n8 score tiles per key tile
  constexpr int NT_O = HD / 8;            // n8 output tiles
  extern __shared__ __align__(16) unsigned char pf_smem[];  // [2 stages][K tile | V tile]
  using M = MmaType<QT>;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tg = lane & 3;
  const int kvh = blockIdx.y;
  const int nthr = blockDim.x;
  pdl_wait();
  pdl_trigger();

  // ---- which sequence / query tile: binary search of the tile prefix sums
  const int tile = blockIdx.x;
  if (tile >= P.tile_cu[P.n_seq]) return;
  int lo_s = 0, hi_s = P.n_seq;  // invariant: tile_cu[lo_s] <= tile < tile_cu[hi_s]
  while (hi_s - lo_s > 1) {
    const int mid = (lo_s + hi_s) >> 1;
    if (P.tile_cu[mid] <= tile) lo_s = mid;
    else hi_s = mid;
  }
  const int seq = lo_s;
  const int row0 = P.cu_seqlens[seq];
  const int len = P.cu_seqlens[seq + 1] - row0;
  const int q0 = (tile - P.tile_cu[seq]) * PF_QT;  // first query token (index inside the sequence)
  if (q0 >= len) return;

  const QT* base = static_cast<const QT*>(P.qkv);
  const int head = kvh * P.G + warp;               // this warp's query head
  const int kcol = (P.H + kvh) * HD, vcol = (P.H + P.K + kvh) * HD;

  // ---- Q fragments (A operand, rows = query tokens g and g + 8)
  uint32_t qa[KS][4];
  {
    const int i0 = q0 + g, i1 = q0 + g + 8;
    const QT* r0 = base + (int64_t)(row0 + (i0 < len ? i0 : len - 1)) * P.ld + head * HD;
    const QT* r1 = base + (int64_t)(row0 + (i1 < len ? i1 : len - 1)) * P.ld + head * HD;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      qa[ks][0] = *reinterpret_cast<const uint32_t*>(r0 + 16 * ks + 2 * tg);
      qa[ks][1] = *reinterpret_cast<const uint32_t*>(r1 + 16 * ks + 2 * tg);
      qa[ks][2] = *reinterpret_cast<const uint32_t*>(r0 + 16 * ks + 8 + 2 * tg);
      qa[ks][3] = *reinterpret_cast<const uint32_t*>(r1 + 16 * ks + 8 + 2 * tg);
    }
  }

  // ---- key range of the tile: causal (+ window) over the same sequence
  const int q_last = (q0 + PF_QT - 1 < len ? q0 + PF_QT - 1 : len - 1);
  int k_first = 0;
  if (P.window > 0 && q0 - P.window + 1 > 0) k_first = q0 - P.window + 1;
  const int t_first = k_first / PF_KT, t_last = q_last / PF_KT;

  // stage a key tile: every thread moves 16-byte pieces of K and V rows; rows past the sequence are zero-filled
  // (a masked probability is an exact zero, but 0 * garbage could still be a NaN in P V)
  auto load_tile = [&](int t, int s) {
    unsigned char* dst = pf_smem + (size_t)s * 2 * TILEB;
    constexpr int CH = HD / 8;  // 16-byte chunks per row
    for (int i = tid; i < PF_KT * CH * 2; i += nthr) {
      const int which = i / (PF_KT * CH);
      const int j = (i % (PF_KT * CH)) / CH, ch = i % CH;
      const int key = t * PF_KT + j;
      unsigned char* d = dst + which * TILEB + j * ROWB + ch * 16;
      if (key < len) {
        const QT* src = base + (int64_t)(row0 + key) * P.ld + (which ? vcol : kcol) + ch * 8;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(pf_smem_u32(d)), "l"(src) : "memory");
      } else {
        *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  float o_acc[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  load_tile(t_first, 0);
  for (int t = t_first; t <= t_last; ++t) {
    const int s = (t - t_first) & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // tile t is complete for every warp; every warp is done with tile t - 1 (stage s ^ 1)
    if (t < t_last) load_tile(t + 1, s ^ 1);
    const uint32_t ks_base = pf_smem_u32(pf_smem + (size_t)s * 2 * TILEB);
    const uint32_t vs_base = ks_base + TILEB;

    // ---- S = Q K^T (16 x 64 per warp)
    float sc[NT_S][4];
#pragma unroll
    for (int n = 0; n < NT_S; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {
        // four 8x8 matrices: (keys 16np + 0..7, dims 16ks + 0..7 | + 8..15), (keys 16np + 8..15, same dims)
        const int m = lane >> 3, r = lane & 7;
        const uint32_t addr = ks_base + (uint32_t)((16 * np + (m >> 1) * 8 + r) * ROWB + (16 * ks + (m & 1) * 8) * 2);
        uint32_t b0, b1, b2, b3;
        pf_ldsm_x4(addr, b0, b1, b2, b3);
        M::mma(sc[2 * np], qa[ks], b0, b1);
        M::mma(sc[2 * np + 1], qa[ks], b2, b3);
      }
    }
    // ---- mask + online softmax (rows g and g + 8 of the warp's 16 query tokens)
    const int kb = t * PF_KT;
    const bool edge = (kb + PF_KT - 1 > q0) || (P.window > 0 && kb < q0 + PF_QT - P.window);
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      const int qi = q0 + g + 8 * hr;
      float mx = -INFINITY;
#pragma unroll
      for (int n = 0; n < NT_S; ++n)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float v = sc[n][2 * hr + e] * P.scale_log2;
          if (edge) {
            const int kj = kb + 8 * n + 2 * tg + e;
            const bool ok = kj <= qi && (P.window <= 0 || kj > qi - P.window);
            v = ok ? v : -INFINITY;
          }
          sc[n][2 * hr + e] = v;
          mx = fmaxf(mx, v);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hr], mx);
      // a row with no valid key yet keeps m = -inf: use 0 as the reference point so that ex2(-inf - 0) = 0
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = pf_ex2(m_run[hr] - m_use);  // m_run = -inf -> 0
      l_run[hr] *= alpha;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        o_acc[i][2 * hr] *= alpha;
        o_acc[i][2 * hr + 1] *= alpha;
      }
      m_run[hr] = m_new;
      float ls = 0.f;
#pragma unroll
      for (int n = 0; n < NT_S; ++n) {
        const float p0 = pf_ex2(sc[n][2 * hr] - m_use), p1 = pf_ex2(sc[n][2 * hr + 1] - m_use);
        ls += p0 + p1;
        sc[n][2 * hr] = p0, sc[n][2 * hr + 1] = p1;
      }
      l_run[hr] += ls;
    }
    // ---- O += P V: the score accumulators of two n8 tiles are the A fragment of one 16-key step
#pragma unroll
    for (int kk = 0; kk < PF_KT / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = M::pack(sc[2 * kk][0], sc[2 * kk][1]);
      pa[1] = M::pack(sc[2 * kk][2], sc[2 * kk][3]);
      pa[2] = M::pack(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
      pa[3] = M::pack(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        // transposed fetch: (keys 16kk + 0..7 | + 8..15, dims 16np + 0..7), then the same keys for dims 16np + 8..15
        const int m = lane >> 3, r = lane & 7;
        const uint32_t addr = vs_base + (uint32_t)((16 * kk + (m & 1) * 8 + r) * ROWB + (16 * np + (m >> 1) * 8) * 2);
        uint32_t b0, b1, b2, b3;
        pf_ldsm_x4_t(addr, b0, b1, b2, b3);
        M::mma(o_acc[2 * np], pa, b0, b1);
        M::mma(o_acc[2 * np + 1], pa, b2, b3);
      }
    }
  }

  // ---- epilogue per query row: normalise, round, XSA with the token's own v, head gate, store
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const int qi = q0 + g + 8 * hr;
    float l = l_run[hr];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const bool live = qi < len;               // quad-uniform
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    float z[NT_O][2];
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      z[i][0] = rnd<QT>(o_acc[i][2 * hr] * inv);
      z[i][1] = rnd<QT>(o_acc[i][2 * hr + 1] * inv);
    }
    const int64_t row = row0 + (live ? qi : len - 1);
    if (P.xsa_alpha != nullptr) {
      const QT* vr = base + row * P.ld + vcol;
      float vv[NT_O][2], n2 = 0.f;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        vv[i][0] = to_f32<QT>(vr[8 * i + 2 * tg]);
        vv[i][1] = to_f32<QT>(vr[8 * i + 2 * tg + 1]);
        n2 += vv[i][0] * vv[i][0] + vv[i][1] * vv[i][1];
      }
      n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
      n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
      const float vinv = 1.0f / fmaxf(sqrtf(n2), P.xsa_eps);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        vv[i][0] *= vinv, vv[i][1] *= vinv;
        dot += z[i][0] * vv[i][0] + z[i][1] * vv[i][1];
      }
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      const float a = P.xsa_alpha[head];
#pragma unroll
      for (int i = 0; i < NT_O; ++i) {
        z[i][0] = rnd<QT>(z[i][0] - a * dot * vv[i][0]);
        z[i][1] = rnd<QT>(z[i][1] - a * dot * vv[i][1]);
      }
    }
    if (P.gate_vals != nullptr) {
      const float gt = P.gate_vals[row * P.H + head];
#pragma unroll
      for (int i = 0; i < NT_O; ++i) z[i][0] = rnd<QT>(z[i][0] * gt), z[i][1] = rnd<QT>(z[i][1] * gt);
    }
    if (live) {
      QT* o = static_cast<QT*>(P.out) + row * P.ldo + head * HD;
#pragma unroll
      for (int i = 0; i < NT_O; ++i)
        *reinterpret_cast<uint32_t*>(o + 8 * i + 2 * tg) = M::pack(z[i][0], z[i][1]);
    }
  }
}

template <typename QT>
static int launch_prefill(const PrefillAttnParams& P, int hd, int max_tiles, cudaStream_t st) {
  const dim3 grid((unsigned)max_tiles, (unsigned)P.K), block((unsigned)(32 * P.G));
#define UV_PF(HD_)                                                                                              \
  case HD_: {                                                                                                   \
    const size_t smem = (size_t)2 * 2 * PF_KT * (HD_ * 2 + 16);                                                 \
    auto kern = prefill_attn_kernel<QT, HD_>;                                                                   \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
      if (e != cudaSuccess) {                                                                                   \
        set_last_cuda_error((int)e);                                                                            \
        return UV_ERR_CUDA;                                                                                     \
      }                                                                                                         \
    }                                                                                                           \
    launch_pdl(kern, grid, block, smem, st, P);                                                                 \
    break;                                                                                                      \
  }
  switch (hd) {
    UV_PF(16)
    UV_PF(32)
    UV_PF(64)
    UV_PF(128)
    default: return UV_ERR_SHAPE;
  }
#undef UV_PF
  return check_launch();
}

}  // namespace uv

extern "C" int uv_prefill_attn(const uv_prefill_attn_args* a, void* stream) {
  using namespace uv;
  if (!a) return UV_ERR_ARG;
  if (a->n_seq == 0 || a->max_tiles == 0) return UV_OK;
  if (!a->qkv || !a->cu_seqlens || !a->tile_cu || !a->out || a->n_seq < 0 || a->max_tiles < 0) return UV_ERR_ARG;
  if (a->H < 1 || a->K < 1 || a->H % a->K || a->window < 0) return UV_ERR_ARG;
  const int G = a->H / a->K;
  if (G > 16) return UV_ERR_SHAPE;
  // rows are moved in 16-byte pieces and pairs are read / written as 32-bit words
  if (!aligned16(a->qkv) || (a->ld * 2) % 16 || (reinterpret_cast<uintptr_t>(a->out) & 3) || (a->ldo & 1))
    return UV_ERR_ALIGN;
  PrefillAttnParams P{};
  P.qkv = a->qkv, P.ld = a->ld, P.cu_seqlens = a->cu_seqlens, P.tile_cu = a->tile_cu, P.n_seq = a->n_seq;
  P.out = a->out, P.ldo = a->ldo, P.H = a->H, P.K = a->K, P.G = G, P.window = a->window;
  P.scale_log2 = a->scale * 1.4426950408889634f;
  P.xsa_alpha = a->xsa_alpha, P.xsa_eps = a->xsa_eps, P.gate_vals = a->gate_vals;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == UV_F16) return launch_prefill<__half>(P, a->hd, a->max_tiles, st);
  if (a->dtype == UV_BF16) return launch_prefill<__nv_bfloat16>(P, a->hd, a->max_tiles, st);
  return UV_ERR_DTYPE;
}
