#include "gemm_common.cuh"

namespace moye {

// ------------------------------------------------------------------------------------------
// CTA pairs on 256 x 512 tiles.  The pair kernel on 256 x 256 tiles (gemm_pair.cu) is limited by how fast operands reach the
// SMs (32 KB per SM and K block at 64 B/clk when the tensor pipe is busy, against a measured
// L2 -> SM ceiling of about 68 B/clk/SM).  Doubling the tile along N lets two 256-wide MMAs share
// every A stage: 48 KB per SM feed 1024 MMA cycles (47 B/clk).  The price is tensor memory: the
// 128 x 512 fp32 accumulator of a CTA is all 512 columns, so it cannot be double-buffered.  The
// two 256-column halves are drained by two epilogue warpgroups at the same time and handed back
// separately, so the next tile's first half starts while the second is still draining.
// Column j of half h belongs to global column n0 + (j / 128) * 256 + h * 128 + j % 128: that way
// each CTA's share of B for both halves is ONE contiguous 256-row box.
//
// K-split tail.  With T tiles on P CTA pairs the last wave is only partly filled (4096^3: 128 tiles on 74 pairs is
// 1.73 waves run as 2).  The tiles of the full waves are dealt out whole as before.  The remaining R = `sk_tiles`
// tiles are shared by ALL pairs in chains: a chain of L tiles is worked by L + 1 pairs; pair i of the chain first
// computes the head [0, h(i)) of the chain's tile i and then the tail [h(i-1), k_blocks) of its tile i-1 (the first
// pair has no tail, the last no head), with h(i) = (i+1) t - i k_blocks - lead.  Every pair of a chain is busy for t
// K blocks (the first `lead` fewer): t = ceil((L k_blocks + lead) / (L + 1)).  So a tile has exactly two
// contributors, and the one with the head is done at least `lead` K blocks before the one with the tail reaches its
// epilogue.  All heads start together at K block 0, like whole tiles do, and all tails run the same distance ahead
// of them, so the pairs that share an operand panel still fetch the same part of it at about the same time.
//
// Putting the two pieces together (per epilogue warp; an atomic ticket tells who came first; nobody spins):
//   linear epilogue, 32-bit D: the head's owner runs the epilogue on its piece alone and stores D; the tail's owner
//     scales its piece by alpha and adds it to D with a TMA reduction -- no scratch traffic at all;
//   otherwise: the head's owner leaves its raw accumulator in the workspace, the tail's owner adds it to its own,
//     still in tensor memory, on the way out.
// Should the tail's owner ever come first, it leaves its raw accumulator in the workspace and the late one finishes
// the tile.  The value is always a sum of the two pieces, so it does not depend on timing; integer kinds stay
// exact.  The reference has no counterpart: its launch covers C with one CTA per tile (examples/gemm.jl:66-89) and
// leaves the wave arithmetic to the hardware.
enum : int { SITEW_PROD_EMPTY = 121, SITEW_MMA_ACC = 122, SITEW_MMA_FULL = 123, SITEW_EPI_ACC = 124 };

// The work items of one CTA pair in order: whole tiles first, then its one or two pieces of K-split tiles.  The
// producer, the MMA issuer and the epilogue warps each walk their own copy and see the same sequence.
struct WideSched {
  int t, step, full_tiles, kb;
  int head_tile, head_to;    // piece 1: K blocks [0, head_to) of K-split tile `head_tile` (-1: none)
  int tail_tile, tail_from;  // piece 2: K blocks [tail_from, kb) of K-split tile `tail_tile` (-1: none)
  __device__ __forceinline__ void init(const GemmArgs& g, int cluster_id, int num_clusters) {
    kb = g.k_blocks;
    full_tiles = g.m_tiles * g.n_tiles - g.sk_tiles;
    t = cluster_id;
    step = num_clusters;
    tail_tile = head_tile = -1;
    tail_from = head_to = 0;
    if (g.sk_tiles == 0) return;
    // chains: the first `extra` have base + 1 tiles (and base + 2 pairs), the others base tiles
    const int base = g.sk_tiles / g.sk_chains, extra = g.sk_tiles % g.sk_chains;
    int c, i, len, tile0, tt;
    if (cluster_id < extra * (base + 2)) {
      c = cluster_id / (base + 2); i = cluster_id - c * (base + 2); len = base + 1; tile0 = c * (base + 1); tt = g.sk_t_long;
    } else {
      const int q = cluster_id - extra * (base + 2);
      c = extra + q / (base + 1); i = q - (c - extra) * (base + 1); len = base; tile0 = extra * (base + 1) + (c - extra) * base;
      tt = g.sk_t_short;
    }
    if (c >= g.sk_chains) return;  // more pairs than the chains need: this one only had whole tiles
    if (i < len) { head_tile = tile0 + i; head_to = (i + 1) * tt - i * kb - g.sk_lead; }
    if (i >= 1) { tail_tile = tile0 + i - 1; tail_from = i * tt - (i - 1) * kb - g.sk_lead; }
  }
  __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1) {
    if (t < full_tiles) {
      tile = t; kb0 = 0; kb1 = kb; t += step;
      return true;
    }
    if (head_tile >= 0) {
      tile = full_tiles + head_tile; kb0 = 0; kb1 = head_to; head_tile = -1;
      return true;
    }
    if (tail_tile >= 0) {
      tile = full_tiles + tail_tile; kb0 = tail_from; kb1 = kb; tail_tile = -1;
      return true;
    }
    return false;
  }
};

// A pair's partial accumulator goes to the workspace as it sits in the epilogue warps' registers: 8 chunks of 32
// columns (first the 128 columns at `t_addr`, then the 128 at `t_addr + 128`), word (chunk, j, lane).
__device__ __forceinline__ void sk_write_partial(uint32_t t_addr, uint32_t* dst, int lane, uint64_t* acc_empty_local,
                                                 uint32_t acc_empty_remote) {
#pragma unroll 1
  for (int cc = 0; cc < 8; ++cc) {
    uint32_t v[32];
    tmem_ld_x32(t_addr + (cc < 4 ? cc * 32 : 128 + (cc - 4) * 32), v);
    tmem_ld_wait();
    if (cc == 7) {
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (acc_empty_remote != 0u) mbar_arrive_remote(acc_empty_remote);
        else mbar_arrive(acc_empty_local);
      }
    }
    uint32_t* p = dst + cc * 1024 + lane;
#pragma unroll
    for (int j = 0; j < 32; ++j) __stcg(p + j * 32, v[j]);
  }
}

// The epilogue of a K-split tile for one warp that came second: both 128-column pieces of its half.
template <int KIND, typename OutT, bool OUT_M_MAJOR, int MODE, int NBUF>
__device__ __forceinline__ void sk_finish_tile(const GemmArgs& g, const CUtensorMap* tmD, uint32_t t_addr, int m0, int n0,
                                               uint8_t* my_buf, int& nstore, int lane, uint64_t* acc_empty_local,
                                               uint32_t acc_empty_remote, const uint32_t* own, const uint32_t* other,
                                               bool own_in_tmem) {
  FixUp fx;
  fx.own = own;
  fx.other = other;
  fx.own_in_tmem = own_in_tmem;
  fx.release = false;
  fx.chunk0 = 0;
  epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, false, MODE>(g, tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u, &fx);
  fx.release = true;
  fx.chunk0 = 4;
  epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, true, MODE>(g, tmD, t_addr + 128, m0, n0 + 256, my_buf, nstore, lane,
                                                             acc_empty_local, acc_empty_remote, &fx);
}

template <int KIND, typename OutT, bool OUT_M_MAJOR, int STAGES, int NBUF>
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + 8 * NBUF * EPI_BUF);
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
  // Programmatic dependent launch: a pair that finds a free SM pair starts as soon as the CTAs of the stream's
  // previous grid leave it and has its barriers and tensor memory ready when that grid completes; nothing above
  // touches global memory, everything below comes after the wait.
  griddep_launch();
  griddep_wait();
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
        WideSched sched;
        sched.init(g, cluster_id, num_clusters);
        int t, kb0, kb1;
        while (ok && sched.next(t, kb0, kb1)) {
          int mi, ni;
          tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
          const int row_a = mi * 256 + (int)rank * BM;
          const int row_b = ni * 512 + (int)rank * 256;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITEW_PROD_EMPTY)) { ok = false; break; }
            uint8_t* sa = smem + stage * STAGE_BYTES;
            if (rank == 0) {
              mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
              load_operand<ELEM, BK, MN>(sa, &tmA, &full[stage], g.a_mn, row_a, BM, kb, g.status);
              load_operand<ELEM, BK, MN>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, row_b, 256, kb, g.status);
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
        WideSched sched;
        sched.init(g, cluster_id, num_clusters);
        int t, kb0, kb1;
        for (; ok && sched.next(t, kb0, kb1); ++lt) {
          const uint32_t aphase = lt & 1;
          for (int kb = kb0; kb < kb1 && ok; ++kb) {
            if (!mbar_wait(&full[stage], phase, g.status, SITEW_MMA_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
  #pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (kb == kb0) {  // this half of the accumulator must have been drained by both CTAs
                if (!mbar_wait(&acc_empty[h], aphase ^ 1, g.status, SITEW_MMA_ACC)) { ok = false; break; }
                tc_fence_after_sync();
              }
              const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES + h * (128 * 128)) >> 4);
  #pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                tc_mma_ss2<KIND>(tmem_base + h * 256, ad + k * da.kstep, bd + k * db.kstep, g.idesc,
                                 ((kb - kb0) | k) != 0 ? 1u : 0u);
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
    uint8_t* my_buf = epi + (warp - 2) * NBUF * EPI_BUF;
    int nstore = 0;
    int lt = 0;
    WideSched sched;
    sched.init(g, cluster_id, num_clusters);
    int t, kb0, kb1;
    for (; sched.next(t, kb0, kb1); ++lt) {
      int mi, ni;
      tile_coord(t, g.m_tiles, g.n_tiles, g.group_m, mi, ni);
      if (!mbar_wait(&acc_full[0], lt & 1, g.status, SITEW_EPI_ACC)) break;
      tc_fence_after_sync();
      const int m0 = mi * 256 + (int)rank * BM + q * 32;
      const int n0 = ni * 512 + h * 128;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + h * 256;
      const uint32_t remote = rank == 0 ? 0u : mapa_shared(smem_u32(&acc_empty[h]), 0);
      if (kb0 == 0 && kb1 == g.k_blocks) {
        epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, false>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u);
        epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, true>(g, &tmD, t_addr + 128, m0, n0 + 256, my_buf, nstore, lane,
                                                             &acc_empty[h], remote);
        continue;
      }
      // ---- one of the two pieces of a K-split tile
      const int st = t - sched.full_tiles;
      const int wslot = (int)rank * 8 + (warp - 2);  // this warp's place in a slab and among the tile's tickets
      int* ticket = g.sk_tickets + st * 16 + wslot;
      const bool is_head = kb0 == 0;
      // slab st holds the head piece of tile st, slab sk_tiles + st the tail piece (each only when needed)
      uint32_t* head_part = g.sk_ws + (size_t)st * kSkSlabWords + wslot * kSkWarpWords;
      uint32_t* tail_part = g.sk_ws + (size_t)(g.sk_tiles + st) * kSkSlabWords + wslot * kSkWarpWords;
      uint32_t* mine = is_head ? head_part : tail_part;
      const uint32_t* theirs = is_head ? tail_part : head_part;
      auto stamp = [&]() {  // everything this warp wrote is visible before the ticket counts it; returns the old count
        __threadfence();
        __syncwarp();
        int old = 0;
        if (lane == 0) old = atomicAdd(ticket, 1);
        return __shfl_sync(0xffffffffu, old, 0);
      };
      bool other_done = false;
      if (!is_head) {  // the tail comes second by design: has the head's owner been here?
        int seen = 0;
        if (lane == 0) seen = atomicAdd(ticket, 0);
        other_done = __shfl_sync(0xffffffffu, seen, 0) == 1;
        __threadfence();
      }
      const bool linear = sizeof(OutT) == 4 && g.act == 0;
      if (linear) {
        if (is_head) {
          // the whole epilogue on this piece alone: D = alpha * piece + beta * C + bias, stored
          epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, false>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u);
          epilogue_tile<KIND, OutT, OUT_M_MAJOR, 128, NBUF, true>(g, &tmD, t_addr + 128, m0, n0 + 256, my_buf, nstore, lane,
                                                               &acc_empty[h], remote);
          if (lane == 0) {
            tma_store_wait_all<0>();  // the stores have reached memory, not only left shared memory
            fence_proxy_async_all();
          }
          if (stamp() == 1) {
            // the tail's owner was here first and left its raw piece: add it to D
            __threadfence();
            sk_finish_tile<KIND, OutT, OUT_M_MAJOR, EPI_RED, NBUF>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u,
                                                             theirs, nullptr, false);
            if (lane == 0) *ticket = 0;
          }
        } else if (other_done) {
          if (lane == 0) fence_proxy_async_all();
          __syncwarp();
          sk_finish_tile<KIND, OutT, OUT_M_MAJOR, EPI_RED, NBUF>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, &acc_empty[h], remote,
                                                           nullptr, nullptr, true);
          if (lane == 0) *ticket = 0;  // ready for the next launch
        } else {
          sk_write_partial(t_addr, mine, lane, &acc_empty[h], remote);
          if (stamp() == 1) {
            // the head's owner stored D in the meantime: add this piece, read back from the workspace
            __threadfence();
            if (lane == 0) fence_proxy_async_all();
            __syncwarp();
            sk_finish_tile<KIND, OutT, OUT_M_MAJOR, EPI_RED, NBUF>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u, mine,
                                                             nullptr, false);
            if (lane == 0) *ticket = 0;
          }
        }
      } else {
        if (other_done) {
          sk_finish_tile<KIND, OutT, OUT_M_MAJOR, EPI_SUM, NBUF>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, &acc_empty[h], remote,
                                                           nullptr, theirs, true);
          if (lane == 0) *ticket = 0;
        } else {
          sk_write_partial(t_addr, mine, lane, &acc_empty[h], remote);
          if (stamp() == 1) {
            __threadfence();
            sk_finish_tile<KIND, OutT, OUT_M_MAJOR, EPI_SUM, NBUF>(g, &tmD, t_addr, m0, n0, my_buf, nstore, lane, nullptr, 0u, mine,
                                                             theirs, false);
            if (lane == 0) *ticket = 0;
          }
        }
      }
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

template <int KIND, typename OutT, bool OUT_M_MAJOR, int STAGES, int NBUF>
static int launch_wide_cfg(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmArgs& args, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (128 * 128 + 256 * 128) + 8 * NBUF * 4096 + 256 + 1024;
  auto kern = gemm_tcgen05_2cta_wide_kernel<KIND, OutT, OUT_M_MAJOR, STAGES, NBUF>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  int clusters = h->num_sms / 2;
  if (clusters > tiles && args.sk_tiles == 0) clusters = tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(320, 1, 1);
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
  if (args.sk_tiles > 0) {  // the tail's scratch is shared by every launch of the handle
    if (int rc = order_scratch_use(h, &h->tail_order, stream)) return rc;
  }
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, td, args));
  if (args.sk_tiles > 0) return scratch_used(&h->tail_order, stream);
  return MOYE_OK;
}

template <int KIND, typename OutT, bool OUT_M_MAJOR>
static int launch_wide_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                            const GemmArgs& args, cudaStream_t stream) {
  // 4 stages of 48 KB and one 4 KB staging buffer per epilogue warp.  3 stages with two staging buffers measured
  // slower: the main loop then runs at 0.61 instead of 0.55 us per K block, which costs more than the staging wait.
  return launch_wide_cfg<KIND, OutT, OUT_M_MAJOR, 4, 1>(h, ta, tb, td, args, stream);
}

template <int KIND, typename OutT>
static int launch_wide_major(bool m_major, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                             const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream) {
  return m_major ? launch_wide_inst<KIND, OutT, true>(h, ta, tb, td, args, stream)
                 : launch_wide_inst<KIND, OutT, false>(h, ta, tb, td, args, stream);
}

int launch_dense_wide(int kind, int out, bool m_major, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                      const CUtensorMap& td, const GemmArgs& a, cudaStream_t stream) {
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

}  // namespace moye
