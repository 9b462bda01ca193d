// Skinny bf16 GEMM on the 5th-generation tensor cores (sm_100a): C (M, N) = A (M, K) . W (N, K)^T, fp32 accumulation
// in tensor memory.
//
//   * operands move global -> shared memory as 2-D TMA tiles (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//     into a ring of STAGES K-blocks of 64 elements, each completion counted by an mbarrier (complete_tx);
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x BN x 16 per instruction) with the
//     accumulator tile (128 lanes x BN fp32 columns) living in TMEM; tcgen05.commit hands a stage back to the copy
//     thread and finally publishes the finished accumulator;
//   * the four warps read the accumulator back with tcgen05.ld (32 lanes x 32 columns each), round it to the
//     activation dtype and run the epilogue: plain store, or SwiGLU when the tile holds gate and up columns of the
//     same features.
//
// The CTA tile is 128 rows of A (every MMA uses all 128 TMEM lanes: one activation row per epilogue thread, which is
// what row-wise epilogues want) by BN rows of W.  Every wait is bounded; a wait that runs out sets a status bit,
// skips the rest and still frees the TMEM columns.
#include <mutex>

#include "tcgen05.cuh"

namespace uv {

constexpr int TC_BM = 128;
constexpr int TC_THREADS = 128;

enum { TC_EPI_STORE = 0, TC_EPI_SWIGLU = 1 };

struct GemmTcParams {
  void* out;        // EPI_STORE: C (M, N), EPI_SWIGLU: act (M, f)
  int64_t ldo;
  int M, N, K;      // N = rows of W covered by the launch (EPI_SWIGLU: 2 * f)
  int f;
  int* status;
};

// 32 bf16 of one output row: four 16-byte stores when the row allows it
__device__ __forceinline__ void tc_store64(__nv_bfloat16* dst, const uint32_t (&pk)[16]) {
  if ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      reinterpret_cast<uint4*>(dst)[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
  } else {
#pragma unroll
    for (int q = 0; q < 16; ++q) reinterpret_cast<uint32_t*>(dst)[q] = pk[q];
  }
}

template <int BN> struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;  // 16 KB
  static constexpr int W_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE = A_BYTES + W_BYTES;
};

// grid (N / BN, M / 128); EPI_SWIGLU: the BN columns of a tile are BN/2 gate features followed by the same BN/2
// up features (two TMA boxes of W rows).
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                             const __grid_constant__ CUtensorMap tm_w,
                                                             const GemmTcParams P) {
  using S = TcSmem<BN>;
  constexpr int TCOLS = BN < 32 ? 32 : BN;  // TMEM columns: a power of two, at least 32
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], accum_bar;
  __shared__ uint32_t tmem_slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * (EPI == TC_EPI_SWIGLU ? BN / 2 : BN), m0 = blockIdx.y * TC_BM;
  const int nk = P.K / TC_BK;
  // the dynamic shared memory base is only 16-byte aligned by contract: round up to the 1024 bytes the swizzle wants
  const uint32_t base = (tc_smem_u32(tc_smem) + 1023u) & ~1023u;

  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      tc_mbar_init(tc_smem_u32(&full_bar[s]), 1);
      tc_mbar_init(tc_smem_u32(&empty_bar[s]), 1);
    }
    tc_mbar_init(tc_smem_u32(&accum_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // one warp allocates (and later frees) the accumulator's TMEM columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_slot)),
                 "r"((uint32_t)TCOLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  pdl_wait();
  pdl_trigger();

  bool ok = true;
  if (warp == 0 && lane == 0) {
    // ---- copy thread: K-blocks into the ring
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_w) : "memory");
    for (int kb = 0; kb < nk; ++kb) {
      const int s = kb % STAGES;
      if (kb >= STAGES && !tc_mbar_wait(tc_smem_u32(&empty_bar[s]), (uint32_t)((kb / STAGES - 1) & 1))) {
        ok = false;
        break;
      }
      const uint32_t bar = tc_smem_u32(&full_bar[s]);
      const uint32_t sa = base + (uint32_t)s * S::STAGE, sw = sa + S::A_BYTES;
      tc_mbar_expect_tx(bar, (uint32_t)S::STAGE);
      tc_tma_load_2d(sa, &tm_a, kb * TC_BK, m0, bar);
      if constexpr (EPI == TC_EPI_SWIGLU) {
        tc_tma_load_2d(sw, &tm_w, kb * TC_BK, n0, bar);                              // gate rows
        tc_tma_load_2d(sw + S::W_BYTES / 2, &tm_w, kb * TC_BK, P.f + n0, bar);        // up rows
      } else {
        tc_tma_load_2d(sw, &tm_w, kb * TC_BK, n0, bar);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA thread
    const uint32_t idesc = tc_idesc(TC_BM, BN);
    for (int kb = 0; kb < nk; ++kb) {
      const int s = kb % STAGES;
      if (!tc_mbar_wait(tc_smem_u32(&full_bar[s]), (uint32_t)((kb / STAGES) & 1))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t sa = base + (uint32_t)s * S::STAGE, sw = sa + S::A_BYTES;
#pragma unroll
      for (int k = 0; k < TC_BK / 16; ++k)  // 16 elements = 32 bytes further along the swizzled row
        tc_mma(tmem, tc_smem_desc(sa + k * 32), tc_smem_desc(sw + k * 32), idesc, (uint32_t)((kb | k) != 0));
      tc_commit(tc_smem_u32(&empty_bar[s]));  // the stage is free once these MMAs have read it
    }
    if (ok) tc_commit(tc_smem_u32(&accum_bar));
  }
  __syncwarp();

  // ---- epilogue: thread = one row of the tile (TMEM lane), BN accumulator columns
  ok = tc_mbar_wait(tc_smem_u32(&accum_bar), 0) && ok;
  tc_fence_after();
  if (ok) {
    const int row = m0 + warp * 32 + lane;
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(P.out);
    if constexpr (EPI == TC_EPI_SWIGLU) {
      constexpr int HB = BN / 2;  // features per tile
      static_assert(HB % 32 == 0 || HB == 16, "gate / up halves are read in 32-column pieces");
#pragma unroll
      for (int c0 = 0; c0 < HB; c0 += 32) {
        uint32_t g[32], u[32];
        tc_ld32(taddr + c0, g);
        tc_ld32(taddr + HB + c0, u);
        if (row < P.M) {
          __nv_bfloat16* dst = out + (int64_t)row * P.ldo + n0 + c0;
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            // the GEMM result and silu(g) are rounded to bf16 where the reference's separate ops round
            const float g0 = rnd<__nv_bfloat16>(__uint_as_float(g[j])), g1 = rnd<__nv_bfloat16>(__uint_as_float(g[j + 1]));
            const float u0 = rnd<__nv_bfloat16>(__uint_as_float(u[j])), u1 = rnd<__nv_bfloat16>(__uint_as_float(u[j + 1]));
            const float s0 = rnd<__nv_bfloat16>(g0 / (1.0f + __expf(-g0))), s1 = rnd<__nv_bfloat16>(g1 / (1.0f + __expf(-g1)));
            const __nv_bfloat162 h = __floats2bfloat162_rn(s0 * u0, s1 * u1);
            pk[j / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
          tc_store64(dst, pk);
        }
      }
    } else {
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t v[32];
        tc_ld32(taddr + c0, v);
        if (row < P.M) {
          __nv_bfloat16* dst = out + (int64_t)row * P.ldo + n0 + c0;
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
            pk[j / 2] = *reinterpret_cast<const uint32_t*>(&h);
          }
          tc_store64(dst, pk);
        }
      }
    }
  } else if (tid == 0 && P.status) {
    atomicOr(P.status, 4);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TCOLS) : "memory");
}

template <int BN, int STAGES, int EPI>
static int launch_tc(const CUtensorMap& ta, const CUtensorMap& tw, const GemmTcParams& P, dim3 grid, cudaStream_t st) {
  auto kern = gemm_tc_kernel<BN, STAGES, EPI>;
  const size_t smem = (size_t)STAGES * TcSmem<BN>::STAGE + 1024;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_last_cuda_error((int)e);
    return UV_ERR_CUDA;
  }
  launch_pdl(kern, grid, dim3(TC_THREADS), smem, st, ta, tw, P);
  return check_launch();
}

}  // namespace uv

using namespace uv;

static int tc_common_checks(const void* a, int64_t lda, const void* w, int64_t ldw, int M, int K) {
  if (!a || !w || M < 1 || K < 1) return UV_ERR_ARG;
  if (K % TC_BK) return UV_ERR_SHAPE;
  if (!aligned16(a) || !aligned16(w) || (lda * 2) % 16 || (ldw * 2) % 16) return UV_ERR_ALIGN;
  return UV_OK;
}

extern "C" int uv_gemm_tc(const void* a, int64_t lda, const void* w, int64_t ldw, void* c, int64_t ldc, int dtype,
                          int M, int N, int K, int* status, void* stream) {
  if (M == 0 || N == 0) return UV_OK;
  if (dtype != UV_BF16) return UV_ERR_DTYPE;
  int rc = tc_common_checks(a, lda, w, ldw, M, K);
  if (rc != UV_OK) return rc;
  if (!c || N % 64 || (ldc & 1)) return UV_ERR_SHAPE;
  CUtensorMap ta, tw;
  if (!make_map(&ta, a, M, K, lda, TC_BM) || !make_map(&tw, w, N, K, ldw, 64)) return UV_ERR_CUDA;
  GemmTcParams P{};
  P.out = c, P.ldo = ldc, P.M = M, P.N = N, P.K = K, P.status = status;
  const dim3 grid((unsigned)(N / 64), (unsigned)((M + TC_BM - 1) / TC_BM));
  return launch_tc<64, 6, TC_EPI_STORE>(ta, tw, P, grid, static_cast<cudaStream_t>(stream));
}

extern "C" int uv_gemm_tc_swiglu(const void* a, int64_t lda, const void* w_gu, void* act, int dtype, int M, int K,
                                 int f, int* status, void* stream) {
  if (M == 0 || f == 0) return UV_OK;
  if (dtype != UV_BF16) return UV_ERR_DTYPE;
  int rc = tc_common_checks(a, lda, w_gu, K, M, K);
  if (rc != UV_OK) return rc;
  if (!act || f % 32) return UV_ERR_SHAPE;
  CUtensorMap ta, tw;
  if (!make_map(&ta, a, M, K, lda, TC_BM) || !make_map(&tw, w_gu, 2 * (int64_t)f, K, K, 32)) return UV_ERR_CUDA;
  GemmTcParams P{};
  P.out = act, P.ldo = f, P.M = M, P.N = 2 * f, P.K = K, P.f = f, P.status = status;
  const dim3 grid((unsigned)(f / 32), (unsigned)((M + TC_BM - 1) / TC_BM));
  return launch_tc<64, 6, TC_EPI_SWIGLU>(ta, tw, P, grid, static_cast<cudaStream_t>(stream));
}
