#include "gemm_common.cuh"

namespace moye {

// ------------------------------------------------------------------------------------------
// Split-K on thread-block clusters, for products whose output has far fewer tiles than the GPU has SMs
// (a few hundred rows against a mid-sized weight matrix): a cluster of S CTAs owns one 128 x BN tile, CTA r
// accumulates K blocks [r*KB/S, (r+1)*KB/S) in tensor memory.  The partial tiles are summed through the L2 cache:
// CTA r owns columns [r*BN/S, (r+1)*BN/S) of the tile; every CTA writes the columns of its raw fp32 / s32
// accumulator that others own into its image in the handle's scratch (coalesced 512-byte stores straight from the
// registers tcgen05.ld fills) and keeps its own columns in shared memory, the cluster meets at one barrier, and
// CTA r fetches its column range of the S - 1 other images into its shared memory (the pipeline stages are free by
// then) with one bulk copy per image, sums the S parts -- always in rank order, so the result does not depend on
// timing -- applies the epilogue and stores D.  Distributed shared memory carried this exchange before and took
// 3-5 us for 96 KB per CTA (about 25 GB/s per SM, whether the peers pushed or the owner pulled); the same bytes
// through L2 take about half of that (all SMs writing at once: about 6 TB/s; staging the image and writing it with
// bulk stores was slower than the plain stores).  No atomics, no waiting on other clusters; the only wait
// besides the pipeline's is the cluster barrier.  The kernel is launched with the programmatic dependent-launch
// attribute: its set-up (barriers, tensor memory) may overlap the end of the previous grid of the stream, and it
// waits for that grid before its first access to global memory.  The reference has no split-K form; the arithmetic
// is the same `gemm!` tower (src/algorithm/blas.jl:39-88) with the K loop cut into S consecutive pieces.
enum : int { SITES_PROD_EMPTY = 131, SITES_MMA_FULL = 133, SITES_EPI_ACC = 134, SITES_RED = 135 };

// Image of one CTA's accumulator in the scratch, in 16-byte words: [half-chunk of 16 columns][quarter q of the rows]
// [j = 0..3][lane].  Thread `lane` of an epilogue warp with q = warp % 4 holds row 32 q + lane; word j of half-chunk
// hc are its columns 16 hc + 4 j .. + 3.  A warp's store of one word index is 512 contiguous bytes, and the column
// range an owner needs is one contiguous block of every image.
__host__ __device__ constexpr int splitk_image_words(int bn) { return bn * 128; }  // 32-bit words per CTA

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
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  constexpr bool INT_OUT = (KIND == KIND_I8);
  constexpr int HC = BN / 16;            // half-chunks (16 columns) of the tile
  constexpr int HC_BYTES = 4 * 4 * 32 * 16;  // one half-chunk of an image: 8 KB
  static_assert(BN * 512 <= STAGES * STAGE_BYTES, "the S column ranges must fit into the pipeline stages");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* red_full = bars + 2 * STAGES + 1;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = (int)cluster_nctarank();
  const int rank = (int)cluster_ctarank();
  const int tile = blockIdx.x / S;
  const int mi = tile % g.m_tiles, ni = tile / g.m_tiles;
  const int kb0 = (int)((long long)g.k_blocks * rank / S);
  const int kb1 = (int)((long long)g.k_blocks * (rank + 1) / S);
  const bool have = kb1 > kb0;

  // The producer thread sets the barriers up and requests the first stages at once: those loads are in flight while
  // warp 1 allocates tensor memory and the CTA meets at the barrier below.
  const int pre = kb1 - kb0 < STAGES ? kb1 - kb0 : STAGES;
  if (warp == 0 && lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(red_full, 1);
    fence_mbar_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    griddep_wait();
    for (int i = 0; i < pre; ++i) {
      mbar_arrive_expect_tx(&full[i], STAGE_BYTES);
      uint8_t* sa = smem + i * STAGE_BYTES;
      load_operand<ELEM, BK, true>(sa, &tmA, &full[i], g.a_mn, mi * BM, BM, kb0 + i, g.status);
      load_operand<ELEM, BK, true>(sa + A_BYTES, &tmB, &full[i], g.b_mn, ni * BN, BN, kb0 + i, g.status);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  griddep_wait();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);
  uint4* const image0 = reinterpret_cast<uint4*>(g.sk_ws) + (size_t)tile * S * (splitk_image_words(BN) / 4);  // the cluster's S images

  if (warp == 0) {
    if (lane == 0) {
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int kb = kb0 + pre; kb < kb1; ++kb) {
        if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITES_PROD_EMPTY)) break;
        mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
        uint8_t* sa = smem + stage * STAGE_BYTES;
        load_operand<ELEM, BK, true>(sa, &tmA, &full[stage], g.a_mn, mi * BM, BM, kb, g.status);
        load_operand<ELEM, BK, true>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, ni * BN, BN, kb, g.status);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && have) {
      int stage = 0;
      uint32_t phase = 0;
      bool fed = true;
      const OperandDesc da = make_operand_desc<BK, UMMA_K>(g.a_mn), db = make_operand_desc<BK, UMMA_K>(g.b_mn);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full[stage], phase, g.status, SITES_MMA_FULL)) { fed = false; break; }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
        const uint64_t ad = da.base + (sa >> 4), bd = db.base + ((sa + A_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          tc_mma_ss<KIND>(tmem_base, ad + k * da.kstep, bd + k * db.kstep, g.idesc, (kb > kb0 || k != 0) ? 1u : 0u);
        tc_commit(&empty[stage]);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
      if (fed) tc_commit(acc_full);  // arrives once every MMA above has completed, i.e. has read its stage
    }
  } else {
    // epilogue warps: this CTA's raw accumulator (zeros if it had no K block) goes to its image in the scratch
    const int q = warp & 3;
    bool ok = true;
    if (have) ok = mbar_wait(acc_full, 0, g.status, SITES_EPI_ACC);
    tc_fence_after_sync();
    // The part of the tile this CTA owns itself stays in its shared memory (the pipeline stages are free: the
    // accumulator is complete), in the place the peers' parts will take around it; the rest goes to the image.
    const int HPO = HC / S;  // half-chunks per owner
    uint4* const img = image0 + (size_t)rank * (splitk_image_words(BN) / 4) + q * 128 + lane;
    uint4* const own = reinterpret_cast<uint4*>(smem) + q * 128 + lane;
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
      for (int hh = 0; hh < 2; ++hh) {
        const int hc = 2 * c + hh;
        uint4* const dst = (hc / HPO == rank ? own : img) + hc * 512;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          dst[j * 32] = make_uint4(v[16 * hh + 4 * j], v[16 * hh + 4 * j + 1], v[16 * hh + 4 * j + 2], v[16 * hh + 4 * j + 3]);
      }
    }
    fence_proxy_async_all();  // the images are read by bulk copies
  }

  // The cluster barrier (release / acquire at cluster scope): all S images are complete, and every CTA's accumulator
  // is, hence its pipeline stages are free.  Every thread of every CTA passes here, whatever happened above.
  __syncwarp();
  tc_fence_before_sync();
  cluster_arrive();
  cluster_wait();
  griddep_launch();

  // CTA `rank` owns half-chunks [rank * HPO, (rank + 1) * HPO) of the tile: that block of every peer's image, to
  // shared memory slot p (slot `rank` holds this CTA's own part already)
  const int HPO = HC / S;
  if (warp == 0 && lane == 0) {
    fence_proxy_async_all();
    mbar_arrive_expect_tx(red_full, (uint32_t)((S - 1) * HPO * HC_BYTES));
    for (int p = 0; p < S; ++p)
      if (p != rank)
        bulk_load_1d(smem + p * HPO * HC_BYTES,
                   reinterpret_cast<const uint8_t*>(image0 + (size_t)p * (splitk_image_words(BN) / 4)) + (size_t)rank * HPO * HC_BYTES,
                   (uint32_t)(HPO * HC_BYTES), red_full);
  }
  const bool summed = mbar_wait(red_full, 0, g.status, SITES_RED);
  if (summed) {
    // One task = the 32 rows of quarter q x the 16 columns of one owned half-chunk, one row per lane; the six warps
    // share the 4 HPO tasks.  Shared memory holds [image p][owned half-chunk][q][j][lane] 16-byte words.
    const bool plain = g.beta == 0.f && g.act == 0 && g.bias_mode == 0;
    // debug build: the largest element offset that belongs to D (and to C)
    [[maybe_unused]] const long long d_last = (long long)(g.M - 1) * g.d_sm + (long long)(g.N - 1) * g.d_sn;
    [[maybe_unused]] const long long c_last = (long long)(g.M - 1) * g.c_sm + (long long)(g.N - 1) * g.c_sn;
    auto reduce = [&](auto s_tag) {
      constexpr int SS = decltype(s_tag)::value;
#pragma unroll 1
      for (int task = warp; task < 4 * HPO; task += 6) {
        const int hl = task >> 2, q = task & 3;
        const uint4* src = reinterpret_cast<const uint4*>(smem) + ((hl * 4 + q) * 4) * 32 + lane;
        uint4 part[SS][4];
#pragma unroll
        for (int p = 0; p < SS; ++p) {
#pragma unroll
          for (int j = 0; j < 4; ++j) part[p][j] = src[p * HPO * (HC_BYTES / 16) + j * 32];
        }
        const int gm = mi * BM + q * 32 + lane;
        const int gn = ni * BN + (rank * HPO + hl) * 16;
        const int count = g.N - gn < 16 ? g.N - gn : 16;  // columns of this half-chunk inside D (<= 0: none)
        if (gm >= g.M || count <= 0) continue;
        const long long off = (long long)gm * g.d_sm + (long long)gn * g.d_sn;
        if (!MOYE_DBG_OK(off >= 0 && off + (long long)(count - 1) * g.d_sn <= d_last, g.status, 951)) continue;
        if (!MOYE_DBG_OK(g.beta == 0.f || (g.C != nullptr && (long long)gm * g.c_sm + (long long)(gn + count - 1) * g.c_sn <= c_last),
                         g.status, 952))
          continue;
        OutT* d = reinterpret_cast<OutT*>(g.D) + off;
        const bool vec = g.d_sn == 1 && count == 16 && (reinterpret_cast<uintptr_t>(d) & 15) == 0;
        if constexpr (INT_OUT) {
          int acc[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            int4 a = make_int4(0, 0, 0, 0);
#pragma unroll
            for (int p = 0; p < SS; ++p) {
              a.x += (int)part[p][j].x; a.y += (int)part[p][j].y; a.z += (int)part[p][j].z; a.w += (int)part[p][j].w;
            }
            acc[4 * j] = a.x; acc[4 * j + 1] = a.y; acc[4 * j + 2] = a.z; acc[4 * j + 3] = a.w;
          }
          if (g.beta != 0.f) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (e < count) acc[e] += reinterpret_cast<const int*>(g.C)[(long long)gm * g.c_sm + (long long)(gn + e) * g.c_sn];
          }
          if (vec) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              reinterpret_cast<int4*>(d)[j] = make_int4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (e < count) d[e * g.d_sn] = acc[e];
          }
        } else {
          float acc[16];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int p = 0; p < SS; ++p) {  // rank order: the sum does not depend on timing
              a.x += __uint_as_float(part[p][j].x); a.y += __uint_as_float(part[p][j].y);
              a.z += __uint_as_float(part[p][j].z); a.w += __uint_as_float(part[p][j].w);
            }
            acc[4 * j] = a.x; acc[4 * j + 1] = a.y; acc[4 * j + 2] = a.z; acc[4 * j + 3] = a.w;
          }
          if (plain) {
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] *= g.alpha;
          } else {
            const float brow = g.bias_mode == 2 ? __ldg(g.bias + gm) : 0.f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              float x = acc[e] * g.alpha + brow;
              if (g.bias_mode == 1 && e < count) x += __ldg(g.bias + gn + e);
              if (g.beta != 0.f && e < count)
                x += g.beta * load_c_as_float<OutT>(g.C, (long long)gm * g.c_sm + (long long)(gn + e) * g.c_sn);
              acc[e] = apply_act(x, g.act);
            }
          }
          if (vec) {
            if constexpr (sizeof(OutT) == 4) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<float4*>(d)[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
            } else {
              uint32_t w[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const OutT lo = cvt_out<OutT>(acc[2 * e]), hi = cvt_out<OutT>(acc[2 * e + 1]);
                w[e] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&lo)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&hi)) << 16);
              }
              reinterpret_cast<uint4*>(d)[0] = make_uint4(w[0], w[1], w[2], w[3]);
              reinterpret_cast<uint4*>(d)[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (e < count) d[e * g.d_sn] = cvt_out<OutT>(acc[e]);
          }
        }
      }
    };
    if (S == 2) reduce(std::integral_constant<int, 2>{});
    else if (S == 4) reduce(std::integral_constant<int, 4>{});
    else reduce(std::integral_constant<int, 8>{});
  }

  // nothing reads another CTA's data after the barrier: the CTAs of a cluster leave independently
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


template <int KIND, typename OutT, int BN>
static int launch_splitk_inst(moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                              int split, cudaStream_t stream) {
  constexpr int STAGES = (227 * 1024 - 1024 - 256) / (128 * 128 + BN * 128);
  constexpr int SMEM = STAGES * (128 * 128 + BN * 128) + 256 + 1024;
  static_assert(2 * STAGES * 8 + 16 + 4 <= 256, "barriers and the tensor-memory address must fit behind the stages");
  auto kern = gemm_tcgen05_splitk_kernel<KIND, OutT, BN, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int tiles = args.m_tiles * args.n_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // the kernel waits for the stream's previous grid itself (griddepcontrol.wait), after its set-up
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_without_pdl() ? 1 : 2;
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
  // one image per CTA in the handle's scratch, which the K-split tail of the 256 x 512 kernel uses too
  const size_t need = (size_t)tiles * split * splitk_image_words(BN) * sizeof(uint32_t);
  if (need > h->tail_ws_bytes - kTailTicketBytes)
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "the split-K path holds one %d KB image per CTA in %zu MB of scratch; %d tiles x %d CTAs do not fit "
              "(it is meant for products with fewer tiles than the GPU has SMs)", splitk_image_words(BN) * 4 / 1024,
              (h->tail_ws_bytes - kTailTicketBytes) >> 20, tiles, split);
  if (int rc = order_scratch_use(h, &h->tail_order, stream)) return rc;
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, args));
  return scratch_used(&h->tail_order, stream);
}

template <int KIND, typename OutT>
static int launch_splitk_bn(int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& args,
                            int split, cudaStream_t stream) {
  if (bn == 256) return launch_splitk_inst<KIND, OutT, 256>(h, ta, tb, args, split, stream);
  if (bn == 128) return launch_splitk_inst<KIND, OutT, 128>(h, ta, tb, args, split, stream);
  MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the split-K path takes tile_n 128 or 256 (got %d)", bn);
}

int launch_dense_splitk(int kind, int out, int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                        const GemmArgs& a, int split, cudaStream_t stream) {
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

}  // namespace moye
