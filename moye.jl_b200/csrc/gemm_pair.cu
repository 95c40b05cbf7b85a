#include "gemm_common.cuh"

namespace moye {

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
  griddep_launch();  // programmatic dependent launch: nothing above touches global memory
  griddep_wait();
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
              load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, row_a, BM, kb, g.status);
              load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, row_b, BN / 2, kb, g.status);
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
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits for the previous grid itself
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_without_pdl() ? 1 : 2;
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


int launch_dense_pair(int kind, int out, bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta,
                      const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& a, cudaStream_t stream) {
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

}  // namespace moye
