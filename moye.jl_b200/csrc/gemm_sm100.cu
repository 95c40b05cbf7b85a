// Dense tiled GEMM for sm_100a: D = alpha * A.B^T (+ beta*C), A:(M,K) and B:(N,K) K-major.
//
// This kernel is the Blackwell re-design of MoYe's `matmul_kernel` (reference
// examples/gemm.jl:4-64).  The roles of the reference's steps map as follows:
//   @tile mA (bM,bK) (blockIdx.x, :)           -> TMA tensor-map box + tile coordinates
//   copyto!(sA, gA) ; cp_async_wait ; sync     -> cp.async.bulk.tensor into a 128B-swizzled
//                                                 smem ring, mbarrier full/empty pipeline
//   gemm!(rC, sA, sB, rC) / FMA triple loop    -> tcgen05.mma, accumulator in tensor memory
//   copyto!(gC, rC)                            -> tcgen05.ld -> registers -> smem -> TMA store
//
// One persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (also owns
// the TMEM allocation), warps 2-5 = epilogue.  The accumulator is double-buffered in TMEM
// so the epilogue of tile i overlaps the main loop of tile i+1.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "common.h"
#include "ptx.cuh"

namespace moye {

struct GemmArgs {
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int group_m;
  uint32_t idesc;
  float alpha;  // alpha * scale_a * scale_b
  float beta;
  const void* C;
  long long c_sm, c_sn;  // strides of C in elements
  int* status;
  int a_mn, b_mn;  // 1: the operand is MN-major (stride 1 along M / N) instead of K-major
  const float* bias;  // fused epilogue: D = act(alpha*acc + beta*C + bias)
  int bias_mode;      // 0 none, 1 one value per column n (length N), 2 one value per row m (length M)
  int act;            // 0 none, 1 relu, 2 gelu (erf form), 3 silu
  void* D;            // output pointer and element strides, for the kernels that store D with plain stores
  long long d_sm, d_sn;
};

// The activations of the fused epilogue, on the fp32 value before the output conversion.
__device__ __forceinline__ float apply_act(float x, int act) {
  if (act == 1) return fmaxf(x, 0.f);
  if (act == 2) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  if (act == 3) return x / (1.f + __expf(-x));
  return x;
}

// Wait-site codes reported through the status word.
enum : int { SITE_PROD_EMPTY = 101, SITE_MMA_ACC = 102, SITE_MMA_FULL = 103, SITE_EPI_ACC = 104 };

__device__ __forceinline__ void tile_coord(int t, int m_tiles, int n_tiles, int group_m, int& mi, int& ni) {
  // Grouped raster: tiles that run concurrently cover `group_m` row-blocks x a few
  // column-blocks, so their A and B panels are shared through L2.
  const int per_group = group_m * n_tiles;
  const int grp = t / per_group;
  const int first_m = grp * group_m;
  const int gsz = min(group_m, m_tiles - first_m);
  const int r = t - grp * per_group;
  mi = first_m + r % gsz;
  ni = r / gsz;
  if (grp & 1) ni = n_tiles - 1 - ni;  // serpentine: a new group starts on the B tiles the last one ended on
}

template <typename OutT>
__device__ __forceinline__ OutT cvt_out(float f);
template <>
__device__ __forceinline__ float cvt_out<float>(float f) { return f; }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }
template <>
__device__ __forceinline__ __half cvt_out<__half>(float f) { return __float2half_rn(f); }

template <typename OutT>
__device__ __forceinline__ float load_c_as_float(const void* C, long long off) {
  return static_cast<float>(reinterpret_cast<const OutT*>(C)[off]);
}


// One operand tile of `rows` x BK into shared memory at `dst`.  K-major: one box {BK, rows}.
// MN-major: the tile is split into chunks of 128 bytes along MN, each a box {128 B, BK rows}.
template <int ELEM, int BK, bool MN_POSSIBLE>
__device__ __forceinline__ void load_operand(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int mn, int row0,
                                             int rows, int kb) {
  if (!MN_POSSIBLE || !mn) {
    tma_load_2d(dst, tm, bar, kb * BK, row0);
  } else {
    constexpr int CH = 128 / ELEM;  // elements per 128-byte chunk
    for (int c = 0; c * CH < rows; ++c) tma_load_2d(dst + c * (BK * 128), tm, bar, row0 + c * CH, kb * BK);
  }
}
template <int ELEM, int BK, bool MN_POSSIBLE>
__device__ __forceinline__ void load_operand_pair(uint8_t* dst, const CUtensorMap* tm, uint32_t bar, int mn, int row0,
                                                  int rows, int kb) {
  if (!MN_POSSIBLE || !mn) {
    tma_load_2d_pair(dst, tm, bar, kb * BK, row0);
  } else {
    constexpr int CH = 128 / ELEM;
    for (int c = 0; c * CH < rows; ++c) tma_load_2d_pair(dst + c * (BK * 128), tm, bar, row0 + c * CH, kb * BK);
  }
}
// Descriptors of an operand tile are `base + (smem address >> 4) + k * kstep` for the k-th UMMA_K slice: the
// majorness only changes the constants, so the MMA-issuing thread (whose instruction count is on the critical
// path) runs the same straight-line code for K-major and MN-major operands.
struct OperandDesc {
  uint64_t base;   // descriptor of a tile at shared-memory address 0
  uint32_t kstep;  // K advance of one instruction, in 16-byte units
};
template <int BK, int UMMA_K>
__device__ __forceinline__ OperandDesc make_operand_desc(int mn) {
  OperandDesc d;
  if (!mn) {
    d.base = umma_desc_k_sw128(0);
    d.kstep = 2;  // 32 bytes inside the swizzled row
  } else {
    d.base = (BK == 32) ? umma_desc_mn_sw128_atom32(0, BK * 128)  // 32-bit elements (tf32): 32-byte swizzle atoms
                        : umma_desc_mn_sw128(0, BK * 128);
    d.kstep = (UMMA_K * 128) >> 4;  // UMMA_K rows of 128 bytes further
  }
  return d;
}

// Epilogue of one accumulator tile for one warp: its 32 TMEM lanes x BN columns go
// TMEM -> registers -> (alpha, beta, convert) -> staging tile in shared memory -> TMA store.
// After the last TMEM read the accumulator is handed back: an arrive on `acc_empty_local`, or,
// when `acc_empty_remote` is non-zero, on that shared::cluster address (the pair leader's barrier).
template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN, int NBUF = 2, bool RELEASE = true>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& g, const CUtensorMap* tmD, uint32_t t_addr, int m0,
                                              int n0, uint8_t* my_buf, int& nstore, int lane,
                                              uint64_t* acc_empty_local, uint32_t acc_empty_remote) {
  constexpr int EPI_BUF = 4096;
  constexpr bool INT_OUT = (KIND == KIND_I8);
  // columns handled per TMA store: a 128-byte row for N-major output, 32 for M-major
  constexpr int SC = OUT_M_MAJOR ? 32 : (128 / (int)sizeof(OutT));
  constexpr int SUB = SC / 32;
#pragma unroll 1
  for (int c = 0; c < BN / SC; ++c) {
    uint8_t* sb = my_buf + (nstore % NBUF) * EPI_BUF;
    if (lane == 0) tma_store_wait_read<NBUF - 1>();  // the store that last used `sb` has drained
    __syncwarp();
#pragma unroll
    for (int s = 0; s < SUB; ++s) {
      uint32_t v[32];
      const int col0 = c * SC + s * 32;
      tmem_ld_x32(t_addr + col0, v);
      tmem_ld_wait();
      if (RELEASE && c == BN / SC - 1 && s == SUB - 1) {
        // last read of this accumulator: hand it back to the MMA warp
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (acc_empty_remote != 0u) mbar_arrive_remote(acc_empty_remote);
          else mbar_arrive(acc_empty_local);
        }
      }
      if (g.beta != 0.f) {
        const int row = m0 + lane;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int col = n0 + col0 + j;
          if (row < g.M && col < g.N) {
            const long long off = (long long)row * g.c_sm + (long long)col * g.c_sn;
            if constexpr (INT_OUT) {
              v[j] = (uint32_t)((int)v[j] + reinterpret_cast<const int*>(g.C)[off]);
            } else {
              float cin = load_c_as_float<OutT>(g.C, off);
              v[j] = __float_as_uint(__uint_as_float(v[j]) * g.alpha + g.beta * cin);
            }
          }
        }
      } else if constexpr (!INT_OUT) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * g.alpha);
      }
      if constexpr (!INT_OUT) {
        if (g.bias_mode | g.act) {  // uniform over the grid: the plain GEMM pays one predicated branch per chunk
          const int row = m0 + lane;
          const float brow = (g.bias_mode == 2 && row < g.M) ? __ldg(g.bias + row) : 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = n0 + col0 + j;
            float x = __uint_as_float(v[j]) + brow;
            if (g.bias_mode == 1 && col < g.N) x += __ldg(g.bias + col);
            v[j] = __float_as_uint(apply_act(x, g.act));
          }
        }
      }
      if constexpr (OUT_M_MAJOR) {
        // staging tile is [32 columns][32 rows], rows contiguous: conflict-free
        if constexpr (INT_OUT) {
          int* so = reinterpret_cast<int*>(sb);
#pragma unroll
          for (int j = 0; j < 32; ++j) so[j * 32 + lane] = (int)v[j];
        } else {
          OutT* so = reinterpret_cast<OutT*>(sb);
#pragma unroll
          for (int j = 0; j < 32; ++j) so[j * 32 + lane] = cvt_out<OutT>(__uint_as_float(v[j]));
        }
      } else {
        // staging tile is [32 rows][128 bytes] in the 128-byte swizzle the store map expects
        uint8_t* rowp = sb + lane * 128;
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            *reinterpret_cast<uint4*>(rowp + ((j ^ (lane & 7)) << 4)) = w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              OutT lo = cvt_out<OutT>(__uint_as_float(v[8 * j + 2 * e]));
              OutT hi = cvt_out<OutT>(__uint_as_float(v[8 * j + 2 * e + 1]));
              w[e] = (uint32_t)(*reinterpret_cast<uint16_t*>(&lo)) |
                     ((uint32_t)(*reinterpret_cast<uint16_t*>(&hi)) << 16);
            }
            const int chunk = s * 4 + j;
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      if constexpr (OUT_M_MAJOR)
        tma_store_2d(tmD, sb, m0, n0 + c * SC);
      else
        tma_store_2d(tmD, sb, n0 + c * SC, m0);
      tma_store_commit();
    }
    ++nstore;
  }
}

template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmD, const GemmArgs g) {
  constexpr int BM = 128;
  constexpr int ELEM = (KIND == KIND_F16) ? 2 : (KIND == KIND_TF32 ? 4 : 1);
  constexpr int BK = 128 / ELEM;       // one 128-byte swizzle row of K per stage
  constexpr int UMMA_K = 32 / ELEM;    // K of one tcgen05.mma
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int EPI_BUF = 4096;        // one staging buffer of one epilogue warp
  constexpr uint32_t TMEM_COLS = 2 * BN;
  static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile N");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns must be a power of two");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + 8 * EPI_BUF);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = g.m_tiles * g.n_tiles;

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // the K-major-only loop is compiled separately: the producer's issue rate is on the critical path
      auto produce = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          int mi, ni;
          tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
          for (int kb = 0; kb < g.k_blocks; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITE_PROD_EMPTY)) { ok = false; break; }
            mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
            uint8_t* sa = smem + stage * STAGE_BYTES;
            load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, mi * BM, BM, kb);
            load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, ni * BN, BN, kb);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      };
      if (g.a_mn | g.b_mn) produce(std::true_type{});
      else produce(std::false_type{});
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      auto issue = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;  // false: K-major constants fold at compile time
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int lt = 0;
        const OperandDesc da = make_operand_desc<BK, UMMA_K>(MN ? g.a_mn : 0), db = make_operand_desc<BK, UMMA_K>(MN ? g.b_mn : 0);
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++lt) {
          const int buf = lt & 1;
          const uint32_t aphase = (lt >> 1) & 1;
          if (!mbar_wait(&acc_empty[buf], aphase ^ 1, g.status, SITE_MMA_ACC)) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < g.k_blocks; ++kb) {
            if (!mbar_wait(&full[stage], phase, g.status, SITE_MMA_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES) >> 4);
  #pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc_mma_ss<KIND>(d_tmem, ad + k * da.kstep, bd + k * db.kstep, g.idesc, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit(&empty[stage]);  // frees the smem stage once these MMAs have read it
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) tc_commit(&acc_full[buf]);
        }
      };
      if (g.a_mn | g.b_mn) issue(std::true_type{});
      else issue(std::false_type{});
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // the TMEM lane quarter this warp may read
    uint8_t* my_buf = epi + (warp - 2) * 2 * EPI_BUF;
    int nstore = 0;
    int lt = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++lt) {
      int mi, ni;
      tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
      const int buf = lt & 1;
      const uint32_t aphase = (lt >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], aphase, g.status, SITE_EPI_ACC)) break;
      tc_fence_after_sync();
      const int m0 = mi * BM + q * 32;
      const int n0 = ni * BN;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      epilogue_tile<KIND, OutT, OUT_M_MAJOR, BN>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, &acc_empty[buf], 0u);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ---------------------------------------------------------------- teardown
  if (*reinterpret_cast<volatile int*>(g.status) != 0) {
    // A wait gave up somewhere: give copies still in flight time to land before the CTA
    // (and its shared memory) goes away.
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// Split-K on thread-block clusters, for products whose output has far fewer tiles than the GPU has SMs
// (a few hundred rows against a mid-sized weight matrix): a cluster of S CTAs owns one 128 x BN tile, CTA r
// accumulates K blocks [r*KB/S, (r+1)*KB/S) in tensor memory, every CTA then stages its raw fp32 / s32
// accumulator in its own shared memory (the pipeline stages are free by then), and after a cluster barrier CTA r
// sums rows [r*128/S, (r+1)*128/S) over the S staged tiles through distributed shared memory -- always in rank
// order, so the result does not depend on timing -- applies the epilogue and stores D.  No global workspace, no
// atomics, no waiting on other clusters.  The reference has no split-K form; the arithmetic is the same `gemm!`
// tower (src/algorithm/blas.jl:39-88) with the K loop cut into S consecutive pieces.
enum : int { SITES_PROD_EMPTY = 131, SITES_MMA_FULL = 133, SITES_EPI_ACC = 134 };

template <typename OutT>
__device__ __forceinline__ void store_out4(void* D, long long off, long long sn, const float (&v)[4], int count, bool vec) {
  OutT* d = reinterpret_cast<OutT*>(D) + off;
  if (vec && count == 4) {
    if constexpr (sizeof(OutT) == 4) {
      *reinterpret_cast<float4*>(d) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      OutT h[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = cvt_out<OutT>(v[e]);
      uint2 w;
      w.x = (uint32_t)(*reinterpret_cast<uint16_t*>(&h[0])) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&h[1])) << 16);
      w.y = (uint32_t)(*reinterpret_cast<uint16_t*>(&h[2])) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&h[3])) << 16);
      *reinterpret_cast<uint2*>(d) = w;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (e < count) d[e * sn] = cvt_out<OutT>(v[e]);
  }
}

template <int KIND, typename OutT, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const GemmArgs g) {
  constexpr int BM = 128;
  constexpr int ELEM = (KIND == KIND_F16) ? 2 : (KIND == KIND_TF32 ? 4 : 1);
  constexpr int BK = 128 / ELEM;
  constexpr int UMMA_K = 32 / ELEM;
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = BN * 128;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int PITCH = BN * 4 + 16;  // bytes of one staged accumulator row; the 16-byte pad spreads rows over banks
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr bool INT_OUT = (KIND == KIND_I8);
  static_assert(BM * PITCH <= STAGES * STAGE_BYTES, "the staged accumulator must fit into the pipeline stages");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = (int)cluster_nctarank();
  const int rank = (int)cluster_ctarank();
  const int tile = blockIdx.x / S;
  const int mi = tile % g.m_tiles, ni = tile / g.m_tiles;
  const int kb0 = (int)((long long)g.k_blocks * rank / S);
  const int kb1 = (int)((long long)g.k_blocks * (rank + 1) / S);
  const bool have = kb1 > kb0;

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITES_PROD_EMPTY)) break;
        mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
        uint8_t* sa = smem + stage * STAGE_BYTES;
        load_operand<ELEM, BK, true>(sa, &tmA, &full[stage], g.a_mn, mi * BM, BM, kb);
        load_operand<ELEM, BK, true>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, ni * BN, BN, kb);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && have) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const OperandDesc da = make_operand_desc<BK, UMMA_K>(g.a_mn), db = make_operand_desc<BK, UMMA_K>(g.b_mn);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[stage], phase, g.status, SITES_MMA_FULL)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
        const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          tc_mma_ss<KIND>(tmem_base, ad + k * da.kstep, bd + k * db.kstep, g.idesc, (kb > kb0 || k != 0) ? 1u : 0u);
        tc_commit(&empty[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (ok) tc_commit(acc_full);  // arrives once every MMA above has completed, i.e. has read its stage
    }
  } else {
    // epilogue warps: stage this CTA's raw accumulator (zeros if it had no K block) as [128 rows][BN] 32-bit words
    const int q = warp & 3;
    bool ok = true;
    if (have) ok = mbar_wait(acc_full, 0, g.status, SITES_EPI_ACC);
    tc_fence_after_sync();
    uint8_t* rowp = smem + (q * 32 + lane) * PITCH;
    const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t v[32];
      if (have && ok) {
        tmem_ld_x32(t_addr + c * 32, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(rowp + c * 128 + j * 16) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  }

  // every thread of every CTA of the cluster passes here, whatever happened above
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();

  if (warp >= 2) {
    // Thread (rr, c4) owns the 16-byte column group c4 of rows rr, rr + RSTEP, ... of this CTA's share: its column
    // bias and its addresses are set up once, every pass adds constants.  These four warps run alone on their
    // schedulers, so the loop is kept short and the loads of several passes are issued together.
    const int et = threadIdx.x - 64;
    constexpr int V = BN / 4;        // 16-byte groups per row
    constexpr int RSTEP = 128 / V;   // rows covered by one pass of the 128 threads
    const int rows_per = BM / S;
    const int c4 = et % V;
    const int row0 = rank * rows_per + et / V;
    const int gn = ni * BN + c4 * 4;
    const int count = g.N - gn < 4 ? g.N - gn : 4;  // columns of this group inside D (<= 0: none)
    const bool vec = g.d_sn == 1 && (g.d_sm & 3) == 0 && (reinterpret_cast<uintptr_t>(g.D) & (4 * sizeof(OutT) - 1)) == 0;
    const uint32_t local0 = smem_u32(smem + row0 * PITCH + c4 * 16);
    uint32_t peer[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) peer[p] = mapa_shared(local0, (uint32_t)(p < S ? p : 0));
    float bcol[4] = {0.f, 0.f, 0.f, 0.f};
    if (!INT_OUT && g.bias_mode == 1) {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < count) bcol[e] = __ldg(g.bias + gn + e);
    }
    const bool plain = g.beta == 0.f && g.act == 0 && g.bias_mode != 2;
    const float alpha = g.alpha;
    const int passes = rows_per / RSTEP;
    auto reduce = [&](auto s_tag) {
      constexpr int SS = decltype(s_tag)::value;
      constexpr int UNR = SS == 8 ? 2 : 4;  // passes whose loads are in flight together
#pragma unroll 1
      for (int ps = 0; ps < passes; ps += UNR) {
        uint4 part[UNR][SS];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
#pragma unroll
          for (int p = 0; p < SS; ++p)
            part[u][p] = ld_shared_cluster_v4(peer[p] + (uint32_t)((ps + u < passes ? ps + u : ps) * RSTEP * PITCH));
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
          const int gm = mi * BM + row0 + (ps + u) * RSTEP;
          if (ps + u >= passes || gm >= g.M || count <= 0) continue;
          const long long off = (long long)gm * g.d_sm + (long long)gn * g.d_sn;
          if constexpr (INT_OUT) {
            int acc[4] = {0, 0, 0, 0};
#pragma unroll
            for (int p = 0; p < SS; ++p) {
              acc[0] += (int)part[u][p].x; acc[1] += (int)part[u][p].y; acc[2] += (int)part[u][p].z; acc[3] += (int)part[u][p].w;
            }
            int* d = reinterpret_cast<int*>(g.D) + off;
            if (g.beta != 0.f) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (e < count) acc[e] += reinterpret_cast<const int*>(g.C)[(long long)gm * g.c_sm + (long long)(gn + e) * g.c_sn];
            }
            if (vec && count == 4) {
              *reinterpret_cast<int4*>(d) = make_int4(acc[0], acc[1], acc[2], acc[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (e < count) d[e * g.d_sn] = acc[e];
            }
          } else {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int p = 0; p < SS; ++p) {  // rank order: the sum does not depend on timing
              acc[0] += __uint_as_float(part[u][p].x); acc[1] += __uint_as_float(part[u][p].y);
              acc[2] += __uint_as_float(part[u][p].z); acc[3] += __uint_as_float(part[u][p].w);
            }
            if (plain) {
#pragma unroll
              for (int e = 0; e < 4; ++e) acc[e] = fmaf(acc[e], alpha, bcol[e]);
            } else {
              const float brow = g.bias_mode == 2 ? __ldg(g.bias + gm) : 0.f;
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                float x = acc[e] * alpha + brow + bcol[e];
                if (g.beta != 0.f && e < count)
                  x += g.beta * load_c_as_float<OutT>(g.C, (long long)gm * g.c_sm + (long long)(gn + e) * g.c_sn);
                acc[e] = apply_act(x, g.act);
              }
            }
            store_out4<OutT>(g.D, off, g.d_sn, acc, count, vec);
          }
        }
      }
    };
    if (S == 2) reduce(std::integral_constant<int, 2>{});
    else if (S == 4) reduce(std::integral_constant<int, 4>{});
    else reduce(std::integral_constant<int, 8>{});
  }

  // the peers may still be reading this CTA's staged tile
  cluster_arrive();
  cluster_wait();
  if (*reinterpret_cast<volatile int*>(g.status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs (tcgen05 cta_group::2).  A cluster of two CTAs owns a 256 x BN
// output tile: each CTA holds its 128 rows of A and of the accumulator and HALF of the B tile
// (BN/2 rows); the tensor cores of the pair read both halves of B.  Per 64-wide K block a
// CTA therefore loads 16 KB + BN/2 * 128 B instead of 16 KB + BN * 128 B, which is what the
// single-CTA kernel runs out of (its L2 -> SM operand feed).  Only the leader CTA (cluster
// rank 0) issues MMAs.  Signalling across the pair:
//   full[s]      (leader)   count 2: one arrive.expect_tx per CTA; the peer's TMA loads complete on
//                           the leader's barrier (cp.async.bulk.tensor ... cta_group::2)
//   empty[s]     (each CTA) tcgen05.commit by the leader, once to its own and once to the peer's barrier
//   acc_full[b]  (each CTA) likewise
//   acc_empty[b] (leader)   count 8: the four epilogue warps of both CTAs
// No multicast is used anywhere.
enum : int { SITE2_PROD_EMPTY = 111, SITE2_MMA_ACC = 112, SITE2_MMA_FULL = 113, SITE2_EPI_ACC = 114 };

template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmD, const GemmArgs g) {
  constexpr int BM = 128;              // rows per CTA; the pair covers 256
  constexpr int ELEM = (KIND == KIND_F16) ? 2 : (KIND == KIND_TF32 ? 4 : 1);
  constexpr int BK = 128 / ELEM;
  constexpr int UMMA_K = 32 / ELEM;
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = (BN / 2) * 128;  // this CTA's half of the B tile
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int EPI_BUF = 4096;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  static_assert(BN % 32 == 0 && BN >= 64 && BN <= 256, "tile N");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + 8 * EPI_BUF);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int num_tiles = g.m_tiles * g.n_tiles;  // m_tiles counts 256-row pair tiles here

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_holder, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();  // both CTAs' barriers are initialised and both halves of the TMEM pair are allocated
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      // the K-major-only loop is compiled separately: the producer's issue rate is on the critical path
      auto produce = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const uint32_t leader_full0 = mapa_shared(smem_u32(&full[0]), 0);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
          int mi, ni;
          tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
          const int row_a = mi * 256 + (int)rank * BM;
          const int row_b = ni * BN + (int)rank * (BN / 2);
          for (int kb = 0; kb < g.k_blocks; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITE2_PROD_EMPTY)) { ok = false; break; }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            if (rank == 0) {
              mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
              load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, row_a, BM, kb);
              load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, row_b, BN / 2, kb);
            } else {
              const uint32_t leader_full = leader_full0 + stage * 8;
              mbar_arrive_expect_tx_remote(leader_full, STAGE_BYTES);
              load_operand_pair<ELEM, BK, MN>(sa, &tmA, leader_full, g.a_mn, row_a, BM, kb);
              load_operand_pair<ELEM, BK, MN>(sa + A_BYTES, &tmB, leader_full, g.b_mn, row_b, BN / 2, kb);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      };
      if (g.a_mn | g.b_mn) produce(std::true_type{});
      else produce(std::false_type{});
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      auto issue = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;  // false: K-major constants fold at compile time
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int lt = 0;
        const OperandDesc da = make_operand_desc<BK, UMMA_K>(MN ? g.a_mn : 0), db = make_operand_desc<BK, UMMA_K>(MN ? g.b_mn : 0);
        const uint32_t empty_local = smem_u32(&empty[0]), empty_peer = mapa_shared(empty_local, 1);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++lt) {
          const int buf = lt & 1;
          const uint32_t aphase = (lt >> 1) & 1;
          if (!mbar_wait(&acc_empty[buf], aphase ^ 1, g.status, SITE2_MMA_ACC)) break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < g.k_blocks; ++kb) {
            if (!mbar_wait(&full[stage], phase, g.status, SITE2_MMA_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES) >> 4);
  #pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              tc_mma_ss2<KIND>(d_tmem, ad + k * da.kstep, bd + k * db.kstep, g.idesc, (kb | k) != 0 ? 1u : 0u);
            }
            tc_commit2(empty_local + stage * 8);  // frees this stage in the leader ...
            tc_commit2(empty_peer + stage * 8);   // ... and in the peer
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) {
            const uint32_t f_local = smem_u32(&acc_full[buf]);
            tc_commit2(f_local);
            tc_commit2(mapa_shared(f_local, 1));
          }
        }
      };
      if (g.a_mn | g.b_mn) issue(std::true_type{});
      else issue(std::false_type{});
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    uint8_t* my_buf = epi + (warp - 2) * 2 * EPI_BUF;
    int nstore = 0;
    int lt = 0;
    for (int t = cluster_id; t < num_tiles; t += num_clusters, ++lt) {
      int mi, ni;
      tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
      const int buf = lt & 1;
      const uint32_t aphase = (lt >> 1) & 1;
      if (!mbar_wait(&acc_full[buf], aphase, g.status, SITE2_EPI_ACC)) break;
      tc_fence_after_sync();
      const int m0 = mi * 256 + (int)rank * BM + q * 32;
      const int n0 = ni * BN;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const uint32_t remote = rank == 0 ? 0u : mapa_shared(smem_u32(&acc_empty[buf]), 0);
      epilogue_tile<KIND, OutT, OUT_M_MAJOR, BN>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, &acc_empty[buf], remote);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  // ---------------------------------------------------------------- teardown
  if (*reinterpret_cast<volatile int*>(g.status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  // neither CTA may leave while its partner can still signal its barriers or read its operands
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------------------------------
// CTA pairs on 256 x 512 tiles.  The pair kernel above is limited by how fast operands reach the
// SMs (32 KB per SM and K block at 64 B/clk when the tensor pipe is busy, against a measured
// L2 -> SM ceiling of about 68 B/clk/SM).  Doubling the tile along N lets two 256-wide MMAs share
// every A stage: 48 KB per SM feed 1024 MMA cycles (47 B/clk).  The price is tensor memory: the
// 128 x 512 fp32 accumulator of a CTA is all 512 columns, so it cannot be double-buffered.  The
// two 256-column halves are drained by two epilogue warpgroups at the same time and handed back
// separately, so the next tile's first half starts while the second is still draining.
// Column j of half h belongs to global column n0 + (j / 128) * 256 + h * 128 + j % 128: that way
// each CTA's share of B for both halves is ONE contiguous 256-row box.
enum : int { SITEW_PROD_EMPTY = 121, SITEW_MMA_ACC = 122, SITEW_MMA_FULL = 123, SITEW_EPI_ACC = 124 };

template <int KIND, typename OutT, bool OUT_M_MAJOR, int STAGES>
__global__ void __launch_bounds__(320, 1)
gemm_tcgen05_2cta_wide_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                              const __grid_constant__ CUtensorMap tmD, const GemmArgs g) {
  constexpr int BM = 128;
  constexpr int ELEM = (KIND == KIND_F16) ? 2 : (KIND == KIND_TF32 ? 4 : 1);
  constexpr int BK = 128 / ELEM;
  constexpr int UMMA_K = 32 / ELEM;
  constexpr int A_BYTES = BM * 128;
  constexpr int B_BYTES = 256 * 128;  // this CTA's 256 rows of the 512-row B tile
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int EPI_BUF = 4096;
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + 8 * EPI_BUF);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;       // [1]
  uint64_t* acc_empty = bars + 2 * STAGES + 1;  // [2], one per half
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 3);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;
  const int num_tiles = g.m_tiles * g.n_tiles;

  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    mbar_init(&acc_full[0], 1);
    mbar_init(&acc_empty[0], 8);
    mbar_init(&acc_empty[1], 8);
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmD);
  }
  if (warp == 1) {
    tmem_alloc2(tmem_holder, TMEM_COLS);
    tmem_relinquish2();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      // the K-major-only loop is compiled separately: the producer's issue rate is on the critical path
      auto produce = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const uint32_t leader_full0 = mapa_shared(smem_u32(&full[0]), 0);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
          int mi, ni;
          tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
          const int row_a = mi * 256 + (int)rank * BM;
          const int row_b = ni * 512 + (int)rank * 256;
          for (int kb = 0; kb < g.k_blocks; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITEW_PROD_EMPTY)) { ok = false; break; }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            if (rank == 0) {
              mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
              load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, row_a, BM, kb);
              load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, row_b, 256, kb);
            } else {
              const uint32_t leader_full = leader_full0 + stage * 8;
              mbar_arrive_expect_tx_remote(leader_full, STAGE_BYTES);
              load_operand_pair<ELEM, BK, MN>(sa, &tmA, leader_full, g.a_mn, row_a, BM, kb);
              load_operand_pair<ELEM, BK, MN>(sa + A_BYTES, &tmB, leader_full, g.b_mn, row_b, 256, kb);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      };
      if (g.a_mn | g.b_mn) produce(std::true_type{});
      else produce(std::false_type{});
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      auto issue = [&](auto mn_tag) {
        constexpr bool MN = decltype(mn_tag)::value;  // false: K-major constants fold at compile time
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int lt = 0;
        const OperandDesc da = make_operand_desc<BK, UMMA_K>(MN ? g.a_mn : 0), db = make_operand_desc<BK, UMMA_K>(MN ? g.b_mn : 0);
        const uint32_t empty_local = smem_u32(&empty[0]), empty_peer = mapa_shared(empty_local, 1);
        for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++lt) {
          const uint32_t aphase = lt & 1;
          for (int kb = 0; kb < g.k_blocks && ok; ++kb) {
            if (!mbar_wait(&full[stage], phase, g.status, SITEW_MMA_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
  #pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (kb == 0) {  // this half of the accumulator must have been drained by both CTAs
                if (!mbar_wait(&acc_empty[h], aphase ^ 1, g.status, SITEW_MMA_ACC)) { ok = false; break; }
                tc_fence_after_sync();
              }
              const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES + h * (128 * 128)) >> 4);
  #pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                tc_mma_ss2<KIND>(tmem_base + h * 256, ad + k * da.kstep, bd + k * db.kstep, g.idesc,
                                 (kb | k) != 0 ? 1u : 0u);
              }
            }
            if (!ok) break;
            tc_commit2(empty_local + stage * 8);
            tc_commit2(empty_peer + stage * 8);
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) {
            const uint32_t f_local = smem_u32(&acc_full[0]);
            tc_commit2(f_local);
            tc_commit2(mapa_shared(f_local, 1));
          }
        }
      };
      if (g.a_mn | g.b_mn) issue(std::true_type{});
      else issue(std::false_type{});
    }
  } else {
    // ------------------------------------------------------------ epilogue: warps 2..5 drain half 0, 6..9 half 1
    const int q = warp & 3;
    const int h = (warp - 2) >> 2;
    uint8_t* my_buf = epi + (warp - 2) * EPI_BUF;
    int nstore = 0;
    int lt = 0;
    for (int t = cluster_id; t < num_tiles; t += num_clusters, ++lt) {
      int mi, ni;
      tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
      if (!mbar_wait(&acc_full[0], lt & 1, g.status, SITEW_EPI_ACC)) break;
      tc_fence_after_sync();
      const int m0 = mi * 256 + (int)rank * BM + q * 32;
      const int n0 = ni * 512 + h * 128;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * 256;
      const uint32_t remote = rank == 0 ? 0u : mapa_shared(smem_u32(&acc_empty[h]), 0);
      epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, 1, false>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u);
      epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, 1, true>(g, &tmD, t_addr + 128, m0, n0 + 256, my_buf, nstore, lane,
                                                           &acc_empty[h], remote);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  if (*reinterpret_cast<volatile int*>(g.status) != 0) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------- host side

template <int BN>
constexpr int stages_for() {
  return (227 * 1024 - 8 * 4096 - 1024 - 256) / (128 * 128 + BN * 128);
}

template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN>
static int launch_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                       const GemmArgs& args, cudaStream_t stream) {
  constexpr int STAGES = stages_for<BN>();
  static_assert(STAGES >= 3, "pipeline too shallow");
  constexpr int SMEM = STAGES * (128 * 128 + BN * 128) + 8 * 4096 + 256 + 1024;
  auto kern = gemm_tcgen05_kernel<KIND, OutT, OUT_M_MAJOR, BN, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  const int grid = tiles < h->num_sms ? tiles : h->num_sms;
  kern<<<grid, 192, SMEM, stream>>>(ta, tb, td, args);
  MOYE_CUDA(cudaGetLastError());
  return MOYE_OK;
}

template <int KIND, typename OutT, bool OUT_M_MAJOR>
static int launch_bn(int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                     const GemmArgs& args, cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_inst<KIND, OutT, OUT_M_MAJOR, 256>(h, ta, tb, td, args, stream);
    case 128: return launch_inst<KIND, OutT, OUT_M_MAJOR, 128>(h, ta, tb, td, args, stream);
    case 64: return launch_inst<KIND, OutT, OUT_M_MAJOR, 64>(h, ta, tb, td, args, stream);
    default: MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile_n must be 64, 128 or 256 (got %d)", bn);
  }
}

template <int KIND, typename OutT>
static int launch_major(bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                        const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream) {
  return m_major ? launch_bn<KIND, OutT, true>(bn, h, ta, tb, td, args, stream)
                 : launch_bn<KIND, OutT, false>(bn, h, ta, tb, td, args, stream);
}


template <int BN>
constexpr int stages_for_pair() {
  return (227 * 1024 - 8 * 4096 - 1024 - 256) / (128 * 128 + (BN / 2) * 128);
}

template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN>
static int launch_pair_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmArgs& args, cudaStream_t stream) {
  constexpr int STAGES = stages_for_pair<BN>();
  constexpr int SMEM = STAGES * (128 * 128 + (BN / 2) * 128) + 8 * 4096 + 256 + 1024;
  auto kern = gemm_tcgen05_2cta_kernel<KIND, OutT, OUT_M_MAJOR, BN, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  int clusters = h->num_sms / 2;
  if (clusters > tiles) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, td, args));
  return MOYE_OK;
}

template <int KIND, typename OutT, bool OUT_M_MAJOR>
static int launch_pair_bn(int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                          const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_pair_inst<KIND, OutT, OUT_M_MAJOR, 256>(h, ta, tb, td, args, stream);
    case 128: return launch_pair_inst<KIND, OutT, OUT_M_MAJOR, 128>(h, ta, tb, td, args, stream);
    default: MOYE_FAIL(MOYE_ERR_INVALID_ARG, "CTA pairs take tile_n 128 or 256 (got %d)", bn);
  }
}

template <int KIND, typename OutT>
static int launch_pair_major(bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                             const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream) {
  return m_major ? launch_pair_bn<KIND, OutT, true>(bn, h, ta, tb, td, args, stream)
                 : launch_pair_bn<KIND, OutT, false>(bn, h, ta, tb, td, args, stream);
}


template <int KIND, typename OutT, bool OUT_M_MAJOR>
static int launch_wide_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmArgs& args, cudaStream_t stream) {
  constexpr int STAGES = 4;
  constexpr int SMEM = STAGES * (128 * 128 + 256 * 128) + 8 * 4096 + 256 + 1024;
  auto kern = gemm_tcgen05_2cta_wide_kernel<KIND, OutT, OUT_M_MAJOR, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  int clusters = h->num_sms / 2;
  if (clusters > tiles) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(320, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, td, args));
  return MOYE_OK;
}

template <int KIND, typename OutT>
static int launch_wide_major(bool m_major, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                             const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream) {
  return m_major ? launch_wide_inst<KIND, OutT, true>(h, ta, tb, td, args, stream)
                 : launch_wide_inst<KIND, OutT, false>(h, ta, tb, td, args, stream);
}

template <int KIND, typename OutT, int BN>
static int launch_splitk_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                              int split, cudaStream_t stream) {
  constexpr int STAGES = (227 * 1024 - 1024 - 256) / (128 * 128 + BN * 128);
  constexpr int SMEM = STAGES * (128 * 128 + BN * 128) + 256 + 1024;
  auto kern = gemm_tcgen05_splitk_kernel<KIND, OutT, BN, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // a cluster of `split` CTAs, each with a whole SM's shared memory, must fit into one GPC: ask once per size
  for (; split >= 2; split /= 2) {
    attr[0].val.clusterDim.x = (unsigned)split;
    cfg.gridDim = dim3((unsigned)(tiles * split), 1, 1);
    const uint64_t key = (reinterpret_cast<uint64_t>(reinterpret_cast<const void*>(kern)) << 4) ^ (uint64_t)split;
    int fit = -1;
    {
      std::lock_guard<std::mutex> lk(h->mu);
      auto it = h->cluster_fit.find(key);
      if (it != h->cluster_fit.end()) fit = it->second;
    }
    if (fit < 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
      }
      fit = n;
      std::lock_guard<std::mutex> lk(h->mu);
      h->cluster_fit[key] = fit;
    }
    if (fit >= 1) break;
  }
  if (split < 2) MOYE_FAIL(MOYE_ERR_CUDA, "no cluster of 2 or more CTAs with %d bytes of shared memory fits this device", SMEM);
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, args));
  return MOYE_OK;
}

template <int KIND, typename OutT>
static int launch_splitk_bn(int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                            int split, cudaStream_t stream) {
  if (bn == 256) return launch_splitk_inst<KIND, OutT, 256>(h, ta, tb, args, split, stream);
  if (bn == 128) return launch_splitk_inst<KIND, OutT, 128>(h, ta, tb, args, split, stream);
  MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the split-K path takes tile_n 128 or 256 (got %d)", bn);
}

int launch_gemm_skinny(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                       const moye_gemm_params_t* p, cudaStream_t stream);

int launch_gemm(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                const moye_tensor_t* C, const moye_gemm_params_t* pp, cudaStream_t stream) {
  moye_gemm_params_t p = {1.f, 0.f, 1.f, 1.f, 0, 0, 0, 0, nullptr};
  if (pp) p = *pp;
  const int act = p.flags & MOYE_EPI_ACT_MASK, bias_mode = (p.flags & MOYE_EPI_BIAS_MASK) >> 4;
  if ((p.flags & ~(MOYE_EPI_ACT_MASK | MOYE_EPI_BIAS_MASK)) != 0 || act > MOYE_EPI_SILU || bias_mode > 2)
    MOYE_FAIL(MOYE_ERR_INVALID_ARG, "unknown bits in flags (0x%x)", p.flags);
  if (p.path < 0 || p.path > 5) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "path must be 0..5 (got %d)", p.path);
  if (bias_mode != 0 && !p.bias) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "a bias mode is set but bias is NULL");
  if (bias_mode != 0 && (reinterpret_cast<uintptr_t>(p.bias) & 3) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "bias must be 4-byte aligned");
  if (A->rank != 2 || B->rank != 2 || D->rank != 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "A, B, D must be rank 2");
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K || D->shape[0] != M || D->shape[1] != N)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "shape mismatch: A (%lld,%lld) B (%lld,%lld) D (%lld,%lld)", (long long)M,
              (long long)K, (long long)N, (long long)B->shape[1], (long long)D->shape[0], (long long)D->shape[1]);
  if (M <= 0 || N <= 0 || K <= 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "empty GEMM");
  if (M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "extent too large");
  if (!A->ptr || !B->ptr || !D->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null data pointer");
  if (A->dtype != B->dtype) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "A and B must have the same dtype");

  int kind;
  uint32_t ab_fmt, c_fmt;
  switch (A->dtype) {
    case MOYE_F16: kind = KIND_F16; ab_fmt = 0; c_fmt = 1; break;
    case MOYE_BF16: kind = KIND_F16; ab_fmt = 1; c_fmt = 1; break;
    case MOYE_S8: kind = KIND_I8; ab_fmt = 1; c_fmt = 2; break;
    case MOYE_E4M3: kind = KIND_F8; ab_fmt = 0; c_fmt = 1; break;
    case MOYE_F32: kind = KIND_TF32; ab_fmt = 2; c_fmt = 1; break;  // operands are read as tf32 (10-bit mantissa)
    default: MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "operand dtype %d is not supported by the tcgen05 path", A->dtype);
  }
  const int out = D->dtype;
  const bool out_ok = (A->dtype == MOYE_F16 && (out == MOYE_F32 || out == MOYE_F16)) ||
                      (A->dtype == MOYE_BF16 && (out == MOYE_F32 || out == MOYE_BF16)) ||
                      (A->dtype == MOYE_S8 && out == MOYE_S32) ||
                      (A->dtype == MOYE_E4M3 && (out == MOYE_BF16 || out == MOYE_F32)) ||
                      (A->dtype == MOYE_F32 && out == MOYE_F32);
  if (!out_ok) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "output dtype %d not supported for operand dtype %d", out, A->dtype);
  // K-major (stride 1 along K) or MN-major (stride 1 along M / N, MoYe's column-major default)
  const bool a_mn = A->stride[1] != 1 || (K == 1 && A->stride[0] == 1 && M > 1);
  const bool b_mn = B->stride[1] != 1 || (K == 1 && B->stride[0] == 1 && N > 1);
  if ((a_mn && A->stride[0] != 1) || (b_mn && B->stride[0] != 1))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "A and B need a unit stride along K or along M / N; got A (%lld,%lld), B (%lld,%lld)",
              (long long)A->stride[0], (long long)A->stride[1], (long long)B->stride[0], (long long)B->stride[1]);
  bool m_major;
  if (D->stride[0] == 1 && (D->stride[1] != 1 || N == 1)) m_major = true;
  else if (D->stride[1] == 1) m_major = false;
  else MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "D must have a unit stride in one mode");

  float alpha = p.alpha * p.scale_a * p.scale_b;
  if (kind == KIND_I8) {
    if (alpha != 1.f || (p.beta != 0.f && p.beta != 1.f))
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the s8 -> s32 path is exact integer arithmetic: alpha must be 1, beta 0 or 1");
    if (act != 0 || bias_mode != 0)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the s8 -> s32 path takes no bias or activation (its epilogue is exact integer arithmetic)");
  }
  if (p.beta != 0.f) {
    if (!C || !C->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "beta != 0 needs C");
    if (C->rank != 2 || C->shape[0] != M || C->shape[1] != N || C->dtype != D->dtype)
      MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "C must match D in shape and dtype");
  }

  if (p.path == 2 && (a_mn || b_mn)) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "the skinny path takes K-major operands");
  // Automatic choice for decode shapes, from measurements at M = 1 .. 128 (bf16, weights from 2048 x 8192 to
  // 28672 x 8192).  The dense kernel on single CTAs streams one tile per CTA over the whole of K, so it is only as
  // fast as its row of tiles is wide.  The stream-K kernel deals equal runs of (row-block, K-block) units to all
  // SMs; it is the fastest form up to 16 rows (X tiles of 2 KB): on the largest weights (16 x 28672 x 8192: 77 us
  // against 81-86), wherever the row of tiles is short, and with very few rows (M = 1 at 28672 x 8192: 75 against
  // 99).  From 17 rows its X tiles and its epilogue grow with M and the split-K kernel (below) or the dense
  // kernel take over (4096 x 4096 weights, M = 64: 16.6 us split-K, 25 stream-K, 25 dense).
  bool use_skinny = p.path == 2;
  if (p.path == 0 && p.tile_n == 0 && p.beta == 0.f && kind == KIND_F16 && M <= 16 && !a_mn && !b_mn && N >= 128 && K >= 512) {
    const long long nk = (long long)N * K;
    const long long tiles256 = (N + 255) / 256;
    const long long tiles = tiles256 >= (long long)h->num_sms * 2 / 3 ? tiles256 : (N + 127) / 128;
    use_skinny = (M <= 16 && nk >= (64ll << 20)) || (M <= 16 && tiles <= 64 && K >= 1024 && nk >= (8ll << 20)) ||
                 (M <= 4 && nk >= (8ll << 20));
  }
  if (use_skinny) return launch_gemm_skinny(h, D, A, B, &p, stream);

  int bn = p.tile_n;
  if (bn == 0) {
    bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
    // one row of tiles (M <= 128): 256-wide tiles only if there are enough of them to occupy most SMs; otherwise
    // 128-wide tiles double the CTAs that stream B (14336 x 4096 weights, M = 64: 29 us against 35.5)
    if (M <= 128 && bn == 256 && (N + 255) / 256 < (long long)h->num_sms * 2 / 3) bn = 128;
  }
  // path 4 = CTA pairs on 256 x 512 tiles.  Chosen automatically when it fills the SM pairs at least as well as
  // 256 x 256 tiles do: it needs less operand traffic per flop and measured about 8 % faster on full waves.
  bool wide = p.path == 4;
  if (p.path == 0 && M > 128 && bn == 256 && N >= 512) {
    const long long clusters = h->num_sms / 2;
    auto fill = [&](long long tm, long long tn) {
      const long long tiles = ((M + tm - 1) / tm) * ((N + tn - 1) / tn);
      const long long waves = (tiles + clusters - 1) / clusters;
      return (double)M * (double)N / ((double)waves * clusters * tm * tn);
    };
    wide = fill(256, 512) * 1.08 >= fill(256, 256);
  }
  if (wide) bn = 256;
  // path 5 = split-K on clusters (128 x tile_n tiles, `split_k` CTAs per tile).  Chosen automatically when the
  // output has so few tiles that the other kernels would leave most SMs idle and K is long enough to cut (at least
  // 8 blocks per CTA): the tile width (256, 128) and split (4, 2) that put the most CTAs on the SMs without
  // exceeding them (4096 x 4096 weights, M = 128: 16.7 us with 32 tiles x 4 against 25-27 unsplit; M = 512: 27
  // against 31).  Clusters of 8 measured slower than clusters of 4 with the same number of CTAs and are only used
  // on request.
  const int kb_total = (int)((K + 128 / dtype_bytes(A->dtype) - 1) / (128 / dtype_bytes(A->dtype)));
  int split = 0;
  if (p.path == 5) {
    if (p.split_k != 0 && p.split_k != 2 && p.split_k != 4 && p.split_k != 8)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "split_k must be 0, 2, 4 or 8 (got %d)", p.split_k);
    if (p.tile_n != 0 && p.tile_n != 128 && p.tile_n != 256)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the split-K path takes tile_n 0, 128 or 256 (got %d)", p.tile_n);
  }
  if (p.path == 5 || (p.path == 0 && !wide && p.tile_n == 0)) {
    long long best_ctas = 0;
    for (int bn_c = 256; bn_c >= 128; bn_c /= 2) {
      if (p.tile_n != 0 && bn_c != p.tile_n) continue;
      if (bn_c == 256 && N <= 128) continue;
      const long long tiles_c = ((M + 127) / 128) * ((N + bn_c - 1) / bn_c);
      for (int sp = 4; sp >= 2; sp /= 2) {
        if (p.split_k != 0 && sp != p.split_k) continue;
        if (tiles_c * sp <= h->num_sms && kb_total >= 8 * sp) {
          if (tiles_c * sp > best_ctas) { best_ctas = tiles_c * sp; split = sp; bn = bn_c; }
          break;
        }
      }
    }
    if (p.path == 5 && split == 0) {  // asked for explicitly: honour it even where it is not the fast choice
      split = p.split_k ? p.split_k : 2;
      bn = p.tile_n ? p.tile_n : (N > 128 ? 256 : 128);
    }
  }
  const bool pair = !split && (wide || p.path == 3 || (p.path == 0 && M > 128 && bn >= 128));
  if (pair && bn < 128) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "CTA pairs take tile_n 128 or 256 (got %d)", bn);
  const int eb = dtype_bytes(A->dtype);
  if (b_mn && eb == 1) {
    // an MN-major tile is loaded in chunks of 128 bytes along N = 128 8-bit elements: a CTA's share of B must be
    // at least that wide (single CTAs: tile_n >= 128; pairs: tile_n 256, i.e. 128 columns per CTA); a narrower
    // request is widened
    const int need = pair ? 256 : 128;
    if (bn < need) bn = need;
  }
  const int bk = 128 / eb;
  CUtensorMap ta, tb, td;
  const int ch = 128 / eb;  // elements in one 128-byte chunk
  // MN-major 32-bit tiles have one legal shared-memory form: the 128-byte swizzle with 32-byte atoms
  const int mn_swizzle = eb == 4 ? TMAP_SWIZZLE_128B_ATOM_32B : TMAP_SWIZZLE_128B;
  if (a_mn) {
    if (int rc = make_tmap_2d(h, &ta, A->ptr, A->dtype, M, K, (uint64_t)A->stride[1] * eb, ch, bk, mn_swizzle)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &ta, A->ptr, A->dtype, K, M, (uint64_t)A->stride[0] * eb, bk, 128, true)) return rc;
  }
  if (b_mn) {
    if (int rc = make_tmap_2d(h, &tb, B->ptr, B->dtype, N, K, (uint64_t)B->stride[1] * eb, ch, bk, mn_swizzle)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &tb, B->ptr, B->dtype, K, N, (uint64_t)B->stride[0] * eb, bk,
                              wide ? 256 : (pair ? bn / 2 : bn), true))
      return rc;
  }
  const int ob = dtype_bytes(out);
  if (m_major) {
    if (int rc = make_tmap_2d(h, &td, D->ptr, out, M, N, (uint64_t)D->stride[1] * ob, 32, 32, false)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &td, D->ptr, out, N, M, (uint64_t)D->stride[0] * ob, 128 / ob, 32, true)) return rc;
  }

  GemmArgs a;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.m_tiles = pair ? (int)((M + 255) / 256) : (int)((M + 127) / 128);
  a.n_tiles = wide ? (int)((N + 511) / 512) : (int)((N + bn - 1) / bn);
  a.k_blocks = (int)((K + bk - 1) / bk);
  // Tile groups: all column tiles of `group_m` row tiles run before the next group, so the group's A panel
  // (rows x K) is re-used from L2 while B streams through.  Size the panel at about 32 MB: the 126 MB L2 is two 63 MB halves, and a 67 MB panel measurably thrashes (DRAM reads 1.1 GB -> 1.3-1.4 GB at 8192^3).
  {
    const long long rows_per_tile = pair ? 256 : 128;
    long long gm = (32ll << 20) / ((long long)K * eb * rows_per_tile);
    if (gm < 4) gm = 4;
    if (gm > a.m_tiles) gm = a.m_tiles;
    a.group_m = (int)gm;
  }
  a.idesc = (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
            ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((pair ? 256 : 128) >> 4) << 24);
  a.a_mn = a_mn ? 1 : 0;
  a.b_mn = b_mn ? 1 : 0;
  a.bias = bias_mode ? p.bias : nullptr;
  a.bias_mode = bias_mode;
  a.act = act;
  a.alpha = alpha;
  a.beta = p.beta;
  a.C = (p.beta != 0.f) ? C->ptr : nullptr;
  a.c_sm = (p.beta != 0.f) ? C->stride[0] : 0;
  a.c_sn = (p.beta != 0.f) ? C->stride[1] : 0;
  a.status = h->d_status;
  a.D = D->ptr;
  a.d_sm = D->stride[0];
  a.d_sn = D->stride[1];

  if (split) {
    if (kind == KIND_F16) {
      if (out == MOYE_F32) return launch_splitk_bn<KIND_F16, float>(bn, h, ta, tb, a, split, stream);
      if (out == MOYE_F16) return launch_splitk_bn<KIND_F16, __half>(bn, h, ta, tb, a, split, stream);
      return launch_splitk_bn<KIND_F16, __nv_bfloat16>(bn, h, ta, tb, a, split, stream);
    } else if (kind == KIND_TF32) {
      return launch_splitk_bn<KIND_TF32, float>(bn, h, ta, tb, a, split, stream);
    } else if (kind == KIND_I8) {
      return launch_splitk_bn<KIND_I8, int>(bn, h, ta, tb, a, split, stream);
    } else {
      if (out == MOYE_F32) return launch_splitk_bn<KIND_F8, float>(bn, h, ta, tb, a, split, stream);
      return launch_splitk_bn<KIND_F8, __nv_bfloat16>(bn, h, ta, tb, a, split, stream);
    }
  }
  if (wide) {
    if (kind == KIND_F16) {
      if (out == MOYE_F32) return launch_wide_major<KIND_F16, float>(m_major, h, ta, tb, td, a, stream);
      if (out == MOYE_F16) return launch_wide_major<KIND_F16, __half>(m_major, h, ta, tb, td, a, stream);
      return launch_wide_major<KIND_F16, __nv_bfloat16>(m_major, h, ta, tb, td, a, stream);
    } else if (kind == KIND_TF32) {
      return launch_wide_major<KIND_TF32, float>(m_major, h, ta, tb, td, a, stream);
    } else if (kind == KIND_I8) {
      return launch_wide_major<KIND_I8, int>(m_major, h, ta, tb, td, a, stream);
    } else {
      if (out == MOYE_F32) return launch_wide_major<KIND_F8, float>(m_major, h, ta, tb, td, a, stream);
      return launch_wide_major<KIND_F8, __nv_bfloat16>(m_major, h, ta, tb, td, a, stream);
    }
  }
  if (pair) {
    if (kind == KIND_F16) {
      if (out == MOYE_F32) return launch_pair_major<KIND_F16, float>(m_major, bn, h, ta, tb, td, a, stream);
      if (out == MOYE_F16) return launch_pair_major<KIND_F16, __half>(m_major, bn, h, ta, tb, td, a, stream);
      return launch_pair_major<KIND_F16, __nv_bfloat16>(m_major, bn, h, ta, tb, td, a, stream);
    } else if (kind == KIND_TF32) {
      return launch_pair_major<KIND_TF32, float>(m_major, bn, h, ta, tb, td, a, stream);
    } else if (kind == KIND_I8) {
      return launch_pair_major<KIND_I8, int>(m_major, bn, h, ta, tb, td, a, stream);
    } else {
      if (out == MOYE_F32) return launch_pair_major<KIND_F8, float>(m_major, bn, h, ta, tb, td, a, stream);
      return launch_pair_major<KIND_F8, __nv_bfloat16>(m_major, bn, h, ta, tb, td, a, stream);
    }
  }
  if (kind == KIND_F16) {
    if (out == MOYE_F32) return launch_major<KIND_F16, float>(m_major, bn, h, ta, tb, td, a, stream);
    if (out == MOYE_F16) return launch_major<KIND_F16, __half>(m_major, bn, h, ta, tb, td, a, stream);
    return launch_major<KIND_F16, __nv_bfloat16>(m_major, bn, h, ta, tb, td, a, stream);
  } else if (kind == KIND_TF32) {
    return launch_major<KIND_TF32, float>(m_major, bn, h, ta, tb, td, a, stream);
  } else if (kind == KIND_I8) {
    return launch_major<KIND_I8, int>(m_major, bn, h, ta, tb, td, a, stream);
  } else {
    if (out == MOYE_F32) return launch_major<KIND_F8, float>(m_major, bn, h, ta, tb, td, a, stream);
    return launch_major<KIND_F8, __nv_bfloat16>(m_major, bn, h, ta, tb, td, a, stream);
  }
}

}  // namespace moye
