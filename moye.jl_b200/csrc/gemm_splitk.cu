#include "gemm_common.cuh"

namespace moye {

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
        load_operand<ELEM, BK, true>(sa, &tmA, &full[stage], g.a_mn, mi * BM, BM, kb, g.status);
        load_operand<ELEM, BK, true>(sa + A_BYTES, &tmB, &full[stage], g.b_mn, ni * BN, BN, kb, g.status);
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
    // debug build: the largest element offset that belongs to D (and to C)
    [[maybe_unused]] const long long d_last = (long long)(g.M - 1) * g.d_sm + (long long)(g.N - 1) * g.d_sn;
    [[maybe_unused]] const long long c_last = (long long)(g.M - 1) * g.c_sm + (long long)(g.N - 1) * g.c_sn;
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
          if (!MOYE_DBG_OK(off >= 0 && off + (long long)(count - 1) * g.d_sn <= d_last, g.status, 951)) continue;
          if (!MOYE_DBG_OK(g.beta == 0.f || (g.C != nullptr && (long long)gm * g.c_sm + (long long)(gn + count - 1) * g.c_sn <= c_last),
                           g.status, 952))
            continue;
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
