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
#include "gemm_common.cuh"

namespace moye {

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
  griddep_launch();  // programmatic dependent launch: see launch_dependent(); nothing above touches global memory
  griddep_wait();
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
            load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, mi * BM, BM, kb, g.status);
            load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, ni * BN, BN, kb, g.status);
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
  MOYE_CUDA(launch_dependent(kern, dim3((unsigned)grid), dim3(192), SMEM, stream, ta, tb, td, args));
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


int launch_dense_single(int kind, int out, bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta,
                        const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& a, cudaStream_t stream) {
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
