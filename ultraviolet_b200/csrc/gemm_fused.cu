// Skinny GEMMs of the decode step with the row-wise work fused into their epilogues (sm_100a).
//
// A decode step multiplies a few hundred activation rows by each weight matrix: the GEMMs are latency bound and
// every separate elementwise kernel between them costs a full dependent launch.  Three kernels, one mainloop:
//
//   uv_gemm_qkv        C = xn . Wqkv^T, one CTA column per head slot (64 outputs = one head), epilogue = the whole
//                      of qkv_post (value-embedding gate, per-head RMS norm, RoPE, int8 quantise + cache append)
//   uv_gemm_swiglu     C = hn . [Wg ; Wu]^T with gate / up rows interleaved inside the tile so that each thread owns
//                      (g, u) pairs, epilogue act = silu(g) * u
//   uv_gemm_resid_norm C = a . W^T (wo or down), N split over a thread-block cluster; epilogue h = l0*x + l1*C and
//                      hn = rms_norm(h), the per-row sum of squares reduced across the cluster through distributed
//                      shared memory (cluster barrier, no spinning)
//
// Mainloop: A (M, K) and W (N, K) row-major in the activation dtype, K-blocks of 64 elements streamed with cp.async
// (16-byte chunks, XOR-swizzled rows) through a 3-stage ring, fragments by ldmatrix, mma.sync.m16n8k16 with fp32
// accumulation.  The GEMM result is rounded to the activation dtype before the epilogue, as the reference's
// F.linear outputs are (ultraviolet/model.py:302-320, :388-391, :567-571).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace uv {

constexpr int GK = 64;      // K elements per pipeline stage (128 bytes per row)
constexpr int GSTAGE = 3;
constexpr float RMS_EPS_G = 1.1920929e-07f;

enum { EPI_QKV = 0, EPI_SWIGLU = 1, EPI_RESID = 2 };

struct GemmParams {
  const void* A;       // (M, K)
  const void* W;       // (N, K)
  int M, N, K;
  int64_t lda, ldw;
  // EPI_SWIGLU
  void* act;           // (M, f)
  int f;
  // EPI_RESID
  const void* x;       // (M, N) residual input
  const float* lambdas;
  void* h;
  void* hn;
  // EPI_QKV (fields of uv_qkv_post)
  void* qkv;           // (M, N) output
  const int64_t* tok;
  const void* value_embed;
  const void* ve_gate;
  const float* inv_freq;
  const int64_t* pos;
  int8_t* k_cache;
  int8_t* v_cache;
  uint16_t* k_scale;
  uint16_t* v_scale;
  const int64_t* row_map;
  int* oob;
  int64_t vocab;
  int H, KH, S, S_alloc, ring, ve_ch, n_pairs;
};

template <typename T> __device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                                uint32_t b1);
template <> __device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                                     uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // zero-fill rows beyond M / N
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// byte offset of 16-byte chunk `ch` (0..7) of tile row `row` (128-byte rows, XOR swizzle against bank conflicts)
__device__ __forceinline__ uint32_t swz(int row, int ch) { return (uint32_t)(row * 128 + ((ch ^ (row & 7)) << 4)); }

// W row feeding tile row i of CTA column `bn`
template <int EPI, int BN> __device__ __forceinline__ int w_row(const GemmParams& P, int bn, int i) {
  if constexpr (EPI == EPI_SWIGLU) return (i & 1 ? P.f : 0) + bn * (BN / 2) + (i >> 1);  // g, u interleaved
  return bn * BN + i;
}

template <typename T, int BM, int BN, int WM, int WN, int EPI>
__global__ void __launch_bounds__(WM* WN * 32) gemm_fused_kernel(const __grid_constant__ GemmParams P) {
  constexpr int NT = WM * WN * 32;
  constexpr int TM = BM / WM, TN = BN / WN, MI = TM / 16, NI = TN / 8;
  static_assert(TM % 16 == 0 && TN % 8 == 0, "warp tile");
  constexpr int A_BYTES = BM * 128, B_BYTES = BN * 128, ST_BYTES = A_BYTES + B_BYTES;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / WN, wn = warp % WN;
  const int bm = blockIdx.x, bn = blockIdx.y;
  const int g = lane >> 2, c = lane & 3;
  const T* A = static_cast<const T*>(P.A);
  const T* W = static_cast<const T*>(P.W);
  const int nk = P.K / GK;

  auto load_stage = [&](int kb, int s) {
    const uint32_t sa = smem_addr(smem + s * ST_BYTES), sb = sa + A_BYTES;
    for (int i = tid; i < BM * 8; i += NT) {
      const int row = i >> 3, ch = i & 7;
      const int gr = bm * BM + row;
      const bool ok = gr < P.M;
      cp_async16(sa + swz(row, ch), A + (int64_t)(ok ? gr : 0) * P.lda + kb * GK + ch * 8, ok);
    }
    for (int i = tid; i < BN * 8; i += NT) {
      const int row = i >> 3, ch = i & 7;
      const int wr = w_row<EPI, BN>(P, bn, row);
      const bool ok = wr < P.N;
      cp_async16(sb + swz(row, ch), W + (int64_t)(ok ? wr : 0) * P.ldw + kb * GK + ch * 8, ok);
    }
  };

  float acc[MI][NI][4];
#pragma unroll
  for (int i = 0; i < MI; ++i)
#pragma unroll
    for (int j = 0; j < NI; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

  pdl_wait();
  pdl_trigger();
#pragma unroll
  for (int s = 0; s < GSTAGE - 1; ++s) {
    if (s < nk) load_stage(s, s);
    cp_async_commit();
  }
  for (int kb = 0; kb < nk; ++kb) {
    cp_async_wait<GSTAGE - 2>();
    __syncthreads();  // stage kb has landed for everyone; stage kb-1 is free
    if (kb + GSTAGE - 1 < nk) load_stage(kb + GSTAGE - 1, (kb + GSTAGE - 1) % GSTAGE);
    cp_async_commit();
    const uint32_t sa = smem_addr(smem + (kb % GSTAGE) * ST_BYTES), sb = sa + A_BYTES;
#pragma unroll
    for (int k16 = 0; k16 < GK / 16; ++k16) {
      uint32_t af[MI][4];
#pragma unroll
      for (int i = 0; i < MI; ++i) {
        const int row = wm * TM + i * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        ldsm_x4(af[i], sa + swz(row, k16 * 2 + (lane >> 4)));
      }
#pragma unroll
      for (int j = 0; j < NI; j += 2) {
        if (j + 1 < NI) {
          uint32_t bf[4];
          const int row = wn * TN + j * 8 + (lane & 7) + 8 * (lane >> 4);
          ldsm_x4(bf, sb + swz(row, k16 * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int i = 0; i < MI; ++i) {
            mma_16816<T>(acc[i][j], af[i], bf[0], bf[1]);
            mma_16816<T>(acc[i][j + 1], af[i], bf[2], bf[3]);
          }
        } else {
          uint32_t bf[2];
          const int row = wn * TN + j * 8 + (lane & 7);
          ldsm_x2(bf, sb + swz(row, k16 * 2 + ((lane >> 3) & 1)));
#pragma unroll
          for (int i = 0; i < MI; ++i) mma_16816<T>(acc[i][j], af[i], bf[0], bf[1]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // the stage ring is free: the epilogues reuse it

  // ================================================================================================ epilogues
  if constexpr (EPI == EPI_SWIGLU) {
    // thread owns (g, u) at tile columns (2c, 2c+1) of every n8 tile: act column = (wn*TN + j*8)/2 + c
    T* stage = reinterpret_cast<T*>(smem);  // [BM][BN/2]
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const float gv = rnd<T>(acc[i][j][2 * hrow]), uvv = rnd<T>(acc[i][j][2 * hrow + 1]);
          const float sv = rnd<T>(gv / (1.0f + __expf(-gv)));
          const int row = wm * TM + i * 16 + g + 8 * hrow, col = (wn * TN + j * 8) / 2 + c;
          stage[row * (BN / 2) + col] = from_f32<T>(sv * uvv);
        }
    __syncthreads();
    constexpr int CH = (BN / 2) / 8;  // 16-byte chunks per row
    T* act = static_cast<T*>(P.act);
    for (int i = tid; i < BM * CH; i += NT) {
      const int row = i / CH, ch = i % CH, gr = bm * BM + row;
      if (gr < P.M)
        *reinterpret_cast<uint4*>(act + (int64_t)gr * P.f + bn * (BN / 2) + ch * 8) =
            *reinterpret_cast<const uint4*>(stage + row * (BN / 2) + ch * 8);
    }
  } else if constexpr (EPI == EPI_RESID) {
    // h = rnd(rnd(l0*x) + rnd(l1*rnd(C))) on this CTA's BN columns; row sums of squares meet across the cluster
    __shared__ float rowsum[BM];
    float* hs = reinterpret_cast<float*>(smem);  // [BM][BN] h values (fp32 copies of the rounded results)
    const float l0 = P.lambdas[0], l1 = P.lambdas[1];
    const T* X = static_cast<const T*>(P.x);
    for (int i = tid; i < BM; i += NT) rowsum[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const int row = wm * TM + i * 16 + g + 8 * hrow, gr = bm * BM + row;
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const int col = wn * TN + j * 8 + 2 * c, gc = bn * BN + col;
          float x0 = 0.f, x1 = 0.f;
          if (gr < P.M) {
            const T* xp = X + (int64_t)gr * P.N + gc;
            x0 = to_f32<T>(xp[0]), x1 = to_f32<T>(xp[1]);
          }
          const float h0 = rnd<T>(rnd<T>(l0 * x0) + rnd<T>(l1 * rnd<T>(acc[i][j][2 * hrow])));
          const float h1 = rnd<T>(rnd<T>(l0 * x1) + rnd<T>(l1 * rnd<T>(acc[i][j][2 * hrow + 1])));
          hs[row * BN + col] = h0, hs[row * BN + col + 1] = h1;
          ss += h0 * h0 + h1 * h1;
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (c == 0) atomicAdd(&rowsum[row], ss);  // WN warps share a row
      }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();  // every CTA of the row block has its partial sums in place
    const unsigned nrank = cluster.num_blocks();
    T* Hh = static_cast<T*>(P.h);
    T* Hn = static_cast<T*>(P.hn);
    constexpr int CH = BN / 8;
    for (int i = tid; i < BM * CH; i += NT) {
      const int row = i / CH, ch = i % CH, gr = bm * BM + row;
      float tot = 0.f;
      for (unsigned rk = 0; rk < nrank; ++rk) tot += cluster.map_shared_rank(rowsum, rk)[row];
      const float inv = rsqrtf(tot / (float)P.N + RMS_EPS_G);
      if (gr < P.M) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = hs[row * BN + ch * 8 + k];
        __align__(16) T o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = from_f32<T>(v[k]);
        *reinterpret_cast<uint4*>(Hh + (int64_t)gr * P.N + bn * BN + ch * 8) = *reinterpret_cast<const uint4*>(o);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = from_f32<T>(v[k] * inv);
        *reinterpret_cast<uint4*>(Hn + (int64_t)gr * P.N + bn * BN + ch * 8) = *reinterpret_cast<const uint4*>(o);
      }
    }
    cluster.sync();  // nobody leaves while a peer may still read its rowsum
  } else {
    // EPI_QKV: BN == head_dim == 64: the tile column is one head slot.  C -> shared (rounded), then a warp per row
    // with lane owning dims (2*lane, 2*lane+1): the arithmetic of uv_qkv_post.
    static_assert(EPI != EPI_QKV || BN == 64, "one head of 64 dims per tile column");
    float* cs = reinterpret_cast<float*>(smem);  // [BM][64]
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
          const int row = wm * TM + i * 16 + g + 8 * hrow, col = wn * TN + j * 8 + 2 * c;
          cs[row * 64 + col] = rnd<T>(acc[i][j][2 * hrow]);
          cs[row * 64 + col + 1] = rnd<T>(acc[i][j][2 * hrow + 1]);
        }
    __syncthreads();
    const int hs_ = bn;  // head slot: [0, H) query heads, [H, H+KH) key heads, then value heads
    const int slots = P.H + 2 * P.KH;
    const bool is_v = hs_ >= P.H + P.KH, is_k = !is_v && hs_ >= P.H;
    for (int row = warp; row < BM; row += NT / 32) {
      const int b = bm * BM + row;
      if (b >= P.M) break;
      float x[2] = {cs[row * 64 + 2 * lane], cs[row * 64 + 2 * lane + 1]};
      if (is_v) {
        if (P.ve_gate != nullptr) {
          const int kh = hs_ - P.H - P.KH;
          const T* xr = static_cast<const T*>(P.A) + (int64_t)b * P.lda;
          const T* gw = static_cast<const T*>(P.ve_gate) + (int64_t)kh * P.ve_ch;
          float a = 0.f;
          for (int ch = lane; ch < P.ve_ch; ch += 32) a += to_f32<T>(xr[ch]) * to_f32<T>(gw[ch]);
          a = rnd<T>(warp_sum(a));
          const float gt = rnd<T>(2.0f * rnd<T>(1.0f / (1.0f + __expf(-a))));
          int64_t t = P.tok[b];
          if (t < 0 || t >= P.vocab) t = 0;
          const T* ve = static_cast<const T*>(P.value_embed) + (t * P.KH + kh) * 64;
#pragma unroll
          for (int i = 0; i < 2; ++i) x[i] = rnd<T>(x[i] + rnd<T>(gt * to_f32<T>(ve[2 * lane + i])));
        }
      } else {
        float ss = warp_sum(x[0] * x[0] + x[1] * x[1]);
        const float inv = rsqrtf(ss / 64.0f + RMS_EPS_G);
        x[0] = rnd<T>(x[0] * inv), x[1] = rnd<T>(x[1] * inv);
        if (P.inv_freq != nullptr) {
          const int pl = P.n_pairs / 2;
          const float pf = (float)P.pos[b];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, x[i], pl);
            const int dim = 2 * lane + i;
            if (dim < 2 * P.n_pairs) {
              const int jj = dim < P.n_pairs ? dim : dim - P.n_pairs;
              const float th = pf * P.inv_freq[jj];
              const float csn = rnd<T>(cosf(th)), sn = rnd<T>(sinf(th));
              x[i] = dim < P.n_pairs ? rnd<T>(rnd<T>(x[i] * csn) - rnd<T>(other * sn))
                                     : rnd<T>(rnd<T>(other * sn) + rnd<T>(x[i] * csn));
            }
          }
        }
      }
      T* dst = static_cast<T*>(P.qkv) + ((int64_t)b * slots + hs_) * 64 + 2 * lane;
      dst[0] = from_f32<T>(x[0]), dst[1] = from_f32<T>(x[1]);
      if ((is_k || is_v) && P.k_cache != nullptr) {
        const int kh = is_v ? hs_ - P.H - P.KH : hs_ - P.H;
        int8_t q8[2];
        const uint16_t sc = quantize_lane<2>(x, q8);
        int64_t p = P.pos[b];
        if (P.ring) p = ((p % P.S) + P.S) % P.S;
        if (p < 0 || p >= P.S) {
          if (lane == 0 && P.oob) atomicAdd(P.oob, 1);
          continue;
        }
        const int64_t cb = P.row_map ? P.row_map[b] : b;
        const int64_t d = (cb * P.KH + kh) * P.S_alloc + p;
        *reinterpret_cast<char2*>((is_v ? P.v_cache : P.k_cache) + d * 64 + 2 * lane) = make_char2(q8[0], q8[1]);
        if (lane == 0) (is_v ? P.v_scale : P.k_scale)[d] = sc;
      }
    }
  }
}

template <typename KernelT>
static int launch_gemm(KernelT kern, dim3 grid, int threads, size_t smem, int cluster_y, const GemmParams& P,
                       cudaStream_t st) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
      set_last_cuda_error((int)e);
      return UV_ERR_CUDA;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid, cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = smem, cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster_y > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1, attr[na].val.clusterDim.y = cluster_y, attr[na].val.clusterDim.z = 1;
    ++na;
  }
  attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[na].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  ++na;
  cfg.attrs = attr, cfg.numAttrs = na;
  cudaLaunchKernelEx(&cfg, kern, P);
  return check_launch();
}

template <typename T> static int gemm_qkv(const GemmParams& P, cudaStream_t st) {
  constexpr int BM = 32, BN = 64;
  dim3 grid((P.M + BM - 1) / BM, P.N / BN);
  return launch_gemm(gemm_fused_kernel<T, BM, BN, 2, 2, EPI_QKV>, grid, 128, GSTAGE * (BM + BN) * 128, 1, P, st);
}
template <typename T> static int gemm_swiglu(const GemmParams& P, cudaStream_t st) {
  constexpr int BM = 128, BN = 64;
  dim3 grid((P.M + BM - 1) / BM, P.f / (BN / 2));
  return launch_gemm(gemm_fused_kernel<T, BM, BN, 4, 2, EPI_SWIGLU>, grid, 256, GSTAGE * (BM + BN) * 128, 1, P, st);
}
template <typename T> static int gemm_resid(const GemmParams& P, cudaStream_t st) {
  constexpr int BM = 32, BN = 80;
  dim3 grid((P.M + BM - 1) / BM, P.N / BN);
  return launch_gemm(gemm_fused_kernel<T, BM, BN, 2, 2, EPI_RESID>, grid, 128, GSTAGE * (BM + BN) * 128,
                     (int)grid.y, P, st);
}

}  // namespace uv

using namespace uv;

static bool gemm_common_ok(const void* A, const void* W, int M, int N, int K, int64_t lda, int64_t ldw) {
  return A && W && M > 0 && N > 0 && K > 0 && K % GK == 0 && lda % 8 == 0 && ldw % 8 == 0 && aligned16(A) &&
         aligned16(W);
}

extern "C" int uv_gemm_qkv(const void* xn, int64_t ldx, const void* wqkv, void* qkv, const int64_t* tok,
                           const void* value_embed, const void* ve_gate, const float* inv_freq, const int64_t* pos,
                           int8_t* k_cache, int8_t* v_cache, uint16_t* k_scale, uint16_t* v_scale,
                           const int64_t* row_map, int* oob_count, int dtype, int64_t vocab, int B, int H, int KH,
                           int hd, int d, int S, int S_alloc, int ring, int ve_ch, int n_pairs, void* stream) {
  if (B == 0) return UV_OK;
  if (hd != 64) return UV_ERR_SHAPE;  // one 64-dim head per tile column; other sizes use uv_qkv_post
  const int N = (H + 2 * KH) * hd;
  if (!gemm_common_ok(xn, wqkv, B, N, d, ldx, d) || !qkv || !pos || H < 1 || KH < 1) return UV_ERR_ARG;
  if (ve_gate && (!tok || !value_embed || ve_ch < 1)) return UV_ERR_ARG;
  if (k_cache && (!v_cache || !k_scale || !v_scale || S < 1)) return UV_ERR_ARG;
  if (inv_freq && (n_pairs < 2 || 2 * n_pairs > hd || (n_pairs & 1) || ((n_pairs / 2) & (n_pairs / 2 - 1))))
    return UV_ERR_SHAPE;
  GemmParams P{};
  P.A = xn, P.W = wqkv, P.M = B, P.N = N, P.K = d, P.lda = ldx, P.ldw = d;
  P.qkv = qkv, P.tok = tok, P.value_embed = value_embed, P.ve_gate = ve_gate, P.inv_freq = inv_freq, P.pos = pos;
  P.k_cache = k_cache, P.v_cache = v_cache, P.k_scale = k_scale, P.v_scale = v_scale, P.row_map = row_map;
  P.oob = oob_count, P.vocab = vocab, P.H = H, P.KH = KH, P.S = S, P.S_alloc = S_alloc > S ? S_alloc : S;
  P.ring = ring, P.ve_ch = ve_ch, P.n_pairs = n_pairs;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_BF16) return gemm_qkv<__nv_bfloat16>(P, st);
  if (dtype == UV_F16) return gemm_qkv<__half>(P, st);
  return UV_ERR_DTYPE;
}

extern "C" int uv_gemm_swiglu(const void* hn, int64_t ldh, const void* w_gu, void* act, int dtype, int B, int d, int f,
                              void* stream) {
  if (B == 0) return UV_OK;
  if (!gemm_common_ok(hn, w_gu, B, 2 * f, d, ldh, d) || !act) return UV_ERR_ARG;
  if (f % 32 || !aligned16(act)) return UV_ERR_SHAPE;
  GemmParams P{};
  P.A = hn, P.W = w_gu, P.M = B, P.N = 2 * f, P.K = d, P.lda = ldh, P.ldw = d, P.act = act, P.f = f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_BF16) return gemm_swiglu<__nv_bfloat16>(P, st);
  if (dtype == UV_F16) return gemm_swiglu<__half>(P, st);
  return UV_ERR_DTYPE;
}

extern "C" int uv_gemm_resid_norm(const void* a, int64_t lda, const void* w, int K, const void* x,
                                  const float* lambdas, void* h, void* hn, int dtype, int B, int d, void* stream) {
  if (B == 0) return UV_OK;
  if (!gemm_common_ok(a, w, B, d, K, lda, K) || !x || !lambdas || !h || !hn) return UV_ERR_ARG;
  if (d % 80 || d / 80 > 8 || !aligned16(h) || !aligned16(hn)) return UV_ERR_SHAPE;  // cluster of <= 8 CTAs x 80
  GemmParams P{};
  P.A = a, P.W = w, P.M = B, P.N = d, P.K = K, P.lda = lda, P.ldw = K, P.x = x, P.lambdas = lambdas, P.h = h, P.hn = hn;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == UV_BF16) return gemm_resid<__nv_bfloat16>(P, st);
  if (dtype == UV_F16) return gemm_resid<__half>(P, st);
  return UV_ERR_DTYPE;
}
