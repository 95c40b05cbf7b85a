// Shared pieces of the dense tcgen05 GEMM kernels: the argument block, operand loads, shared-memory descriptors
// and the epilogue (TMEM -> registers -> alpha/beta/bias/activation -> staging tile -> TMA store) that all of them use.
// Reference counterpart of the whole family: `matmul_kernel`, examples/gemm.jl:4-64.
#pragma once
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
  // stream-K tail of the 256 x 512 pair kernel (all zero / null when it is off)
  int sk_tiles;          // the last `sk_tiles` tiles of the schedule are cut in two along K (see gemm_wide.cu)
  int sk_chains;         // they form `sk_chains` chains of sk_tiles / sk_chains (+1) tiles, each worked by one pair more
  int sk_t_long, sk_t_short;  // K blocks a pair of a long / short chain is busy for
  int sk_lead;           // K blocks by which a head ends before the tail that is added to it
  uint32_t* sk_ws;       // raw fp32 / s32 partial accumulators: 2 * sk_tiles slabs of kSkSlabWords
  int* sk_tickets;       // [sk_tiles][2 CTAs][8 epilogue warps], zero between launches
};

// One partial accumulator of a CTA pair in the stream-K workspace: [2 CTAs][8 epilogue warps][8 chunks of 32
// columns][32 columns][32 rows] 32-bit words.  A warp's 32 KB are contiguous, and both the warp that writes a chunk
// and the warp that later reads it touch 32 consecutive words per instruction.
constexpr int kSkWarpWords = 8 * 1024;
constexpr int kSkSlabWords = 2 * 8 * kSkWarpWords;

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
                                             int rows, int kb, [[maybe_unused]] int* dbg_status = nullptr) {
#ifdef MOYE_DEBUG
  // x (the coordinate along the contiguous mode) times the element size must be a multiple of 16 bytes, the
  // destination 1024-byte aligned inside the stage (the 128-byte swizzle's atom), coordinates not negative
  if (dbg_status != nullptr &&
      (kb < 0 || row0 < 0 || ((mn ? row0 : kb * BK) * ELEM) % 16 != 0 || (smem_u32(dst) & (mn ? 127u : 1023u)) != 0)) {
    atomicCAS(dbg_status, 0, 982);
    return;  // the load is skipped: the consumer's bounded wait ends the kernel
  }
#endif
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

// A K-split tile (gemm_wide.cu) is computed in two pieces by two CTA pairs.  How the second to arrive puts them
// together depends on the epilogue:
//   EPI_SUM  the first left its raw accumulator in the workspace; the second adds it to its own (from tensor memory
//            if it is still there, else from the workspace too) and runs the whole epilogue.  Any epilogue.
//   EPI_RED  the first ran the epilogue on its piece alone and stored D; the second scales its piece by alpha and
//            ADDS it to D with a TMA reduction.  Only where the epilogue is linear and D has 32-bit elements.
// Either way the value is first piece + second piece, a sum of two terms, so it does not depend on who came first.
enum : int { EPI_PLAIN = 0, EPI_SUM = 1, EPI_RED = 2 };
struct FixUp {
  const uint32_t* own;     // this warp's slab of its own pair's raw accumulator in the workspace (read when !own_in_tmem)
  const uint32_t* other;   // this warp's slab of the other pair's raw accumulator (EPI_SUM)
  bool own_in_tmem;
  bool release;            // hand the accumulator back after the last tensor-memory read
  int chunk0;              // the warp's slab holds 8 chunks of 32 columns; this call starts at chunk `chunk0`
};

// Epilogue of one accumulator tile for one warp: its 32 TMEM lanes x BN columns go
// TMEM -> registers -> (alpha, beta, convert) -> staging tile in shared memory -> TMA store.
// After the last TMEM read the accumulator is handed back: an arrive on `acc_empty_local`, or,
// when `acc_empty_remote` is non-zero, on that shared::cluster address (the pair leader's barrier).
// BETA (plain epilogue only): compiled for beta != 0, where C is prefetched a chunk ahead, or for beta == 0, where
// the tensor-memory read is started early instead; the two never hold their look-ahead registers at the same time.
template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN, int NBUF, bool RELEASE, int MODE, bool BETA>
__device__ __forceinline__ void epilogue_tile_impl(const GemmArgs& g, const CUtensorMap* tmD, uint32_t t_addr, int m0,
                                                   int n0, uint8_t* my_buf, int& nstore, int lane,
                                                   uint64_t* acc_empty_local, uint32_t acc_empty_remote,
                                                   const FixUp* fx) {
  constexpr int EPI_BUF = 4096;
  constexpr bool INT_OUT = (KIND == KIND_I8);
  // columns handled per TMA store: a 128-byte row for N-major output, 32 for M-major
  constexpr int SC = OUT_M_MAJOR ? 32 : (128 / (int)sizeof(OutT));
  constexpr int SUB = SC / 32;
  constexpr bool FIX = MODE == EPI_SUM, RED = MODE == EPI_RED;
  // EPI_SUM: the other pair's part of the NEXT chunk is requested while this chunk is converted and stored, so
  // the L2 round trip is paid once per call and not once per chunk
  uint32_t ta[FIX ? 32 : 1];
  auto request_others = [&](int q) {
    if constexpr (FIX) {
      const uint32_t* p = fx->other + (fx->chunk0 + q) * 1024 + lane;
#pragma unroll
      for (int j = 0; j < 32; ++j) ta[j] = __ldcg(p + j * 32);
    }
  };
  request_others(0);
  // beta != 0: the 32 values of C a thread needs for a chunk are requested one chunk ahead, so that their way from
  // memory overlaps the tensor-memory read and the stores of the chunk before (the tensor cores wait for this loop)
  constexpr bool CPRE = MODE == EPI_PLAIN && BETA;
  uint32_t cpre[CPRE ? 32 : 1];
  auto request_c = [&](int q) {
    if constexpr (CPRE) {
      const int row = m0 + lane;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = n0 + q * 32 + j;
        cpre[j] = 0u;
        if (row < g.M && col < g.N) {
          const long long off = (long long)row * g.c_sm + (long long)col * g.c_sn;
          if constexpr (INT_OUT) cpre[j] = (uint32_t)reinterpret_cast<const int*>(g.C)[off];
          else cpre[j] = __float_as_uint(load_c_as_float<OutT>(g.C, off));
        }
      }
    }
  };
  request_c(0);
#pragma unroll 1
  for (int c = 0; c < BN / SC; ++c) {
    uint8_t* sb = my_buf + (nstore % NBUF) * EPI_BUF;
    // plain epilogue: the tensor-memory read of this chunk is in flight while the warp waits for its staging buffer
    constexpr bool EARLY_LD = MODE == EPI_PLAIN && !BETA;
    uint32_t v0[EARLY_LD ? 32 : 1];
    if constexpr (EARLY_LD) tmem_ld_x32(t_addr + c * SC, v0);
    if (lane == 0) tma_store_wait_read<NBUF - 1>();  // the store that last used `sb` has drained
    __syncwarp();
#pragma unroll
    for (int s = 0; s < SUB; ++s) {
      uint32_t v[32];
      const int col0 = c * SC + s * 32;
      if constexpr (FIX || RED) {
        const int q = c * SUB + s;
        if (fx->own_in_tmem) {
          tmem_ld_x32(t_addr + col0, v);
          tmem_ld_wait();
        } else {
          const uint32_t* p = fx->own + (fx->chunk0 + q) * 1024 + lane;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __ldcg(p + j * 32);
        }
      }
      if constexpr (FIX) {
        const int q = c * SUB + s;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if constexpr (INT_OUT) v[j] = (uint32_t)((int)v[j] + (int)ta[j]);
          else v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(ta[j]));
        }
        if (q + 1 < BN / 32) request_others(q + 1);
      } else if constexpr (!RED) {
        if (EARLY_LD && s == 0) {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = v0[j];
        } else {
          tmem_ld_x32(t_addr + col0, v);
          tmem_ld_wait();
        }
      }
      if (((FIX || RED) ? (fx->release && fx->own_in_tmem) : RELEASE) && c == BN / SC - 1 && s == SUB - 1) {
        // last read of this accumulator: hand it back to the MMA warp
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (acc_empty_remote != 0u) mbar_arrive_remote(acc_empty_remote);
          else mbar_arrive(acc_empty_local);
        }
      }
      if constexpr (CPRE) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if constexpr (INT_OUT) v[j] = (uint32_t)((int)v[j] + (int)cpre[j]);
          else v[j] = __float_as_uint(__uint_as_float(v[j]) * g.alpha + g.beta * __uint_as_float(cpre[j]));
        }
        if (c * SUB + s + 1 < BN / 32) request_c(c * SUB + s + 1);
      } else if (MODE == EPI_SUM && g.beta != 0.f) {
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
      if constexpr (!INT_OUT && !RED) {
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
    // debug build: a store or reduce must not start at a negative coordinate, its x must sit on a 16-byte boundary,
    // the staging buffer must be one of this warp's, and the tile must lie in the accumulator's columns
    if (!MOYE_DBG_OK(m0 >= 0 && n0 + c * SC >= 0 && (((OUT_M_MAJOR ? m0 : n0 + c * SC) * (int)sizeof(OutT)) & 15) == 0 &&
                         sb >= my_buf && sb < my_buf + NBUF * EPI_BUF && (t_addr & 0xFFFFu) + BN <= 512u,
                     g.status, 981)) {
      ++nstore;
      continue;
    }
    if (lane == 0) {
      if constexpr (RED) {
        if constexpr (OUT_M_MAJOR) tma_reduce_add_2d(tmD, sb, m0, n0 + c * SC);
        else tma_reduce_add_2d(tmD, sb, n0 + c * SC, m0);
      } else {
        if constexpr (OUT_M_MAJOR) tma_store_2d(tmD, sb, m0, n0 + c * SC);
        else tma_store_2d(tmD, sb, n0 + c * SC, m0);
      }
      tma_store_commit();
    }
    ++nstore;
  }
}

template <int KIND, typename OutT, bool OUT_M_MAJOR, int BN, int NBUF = 2, bool RELEASE = true, int MODE = EPI_PLAIN>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& g, const CUtensorMap* tmD, uint32_t t_addr, int m0,
                                              int n0, uint8_t* my_buf, int& nstore, int lane,
                                              uint64_t* acc_empty_local, uint32_t acc_empty_remote,
                                              const FixUp* fx = nullptr) {
  if constexpr (MODE == EPI_PLAIN) {
    if (g.beta != 0.f)
      epilogue_tile_impl<KIND, OutT, OUT_M_MAJOR, BN, NBUF, RELEASE, MODE, true>(g, tmD, t_addr, m0, n0, my_buf, nstore, lane,
                                                                                  acc_empty_local, acc_empty_remote, fx);
    else
      epilogue_tile_impl<KIND, OutT, OUT_M_MAJOR, BN, NBUF, RELEASE, MODE, false>(g, tmD, t_addr, m0, n0, my_buf, nstore, lane,
                                                                                   acc_empty_local, acc_empty_remote, fx);
  } else {
    epilogue_tile_impl<KIND, OutT, OUT_M_MAJOR, BN, NBUF, RELEASE, MODE, false>(g, tmD, t_addr, m0, n0, my_buf, nstore, lane,
                                                                                 acc_empty_local, acc_empty_remote, fx);
  }
}

// Entry points of the per-kernel translation units (each instantiates one kernel family): `kind` is an MmaKind,
// `out` the moye_dtype_t of D.
int launch_dense_single(int kind, int out, bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta,
                        const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream);
int launch_dense_pair(int kind, int out, bool m_major, int bn, moye_b200_ctx* h, const CUtensorMap& ta,
                      const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream);
int launch_dense_wide(int kind, int out, bool m_major, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                      const CUtensorMap& td, const GemmArgs& args, cudaStream_t stream);
int launch_dense_splitk(int kind, int out, int bn, moye_b200_ctx* h, const CUtensorMap& ta, const CUtensorMap& tb,
                        const GemmArgs& args, int split, cudaStream_t stream);

}  // namespace moye
