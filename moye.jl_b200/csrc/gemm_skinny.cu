// Skinny (decode-shaped) GEMM for sm_100a: D(M,N) = alpha * X(M,K) . W(N,K)^T with M <= 128.
//
// The product is bound by reading W once from HBM, so the kernel is organised around keeping
// as many W bytes in flight as possible:
//   - operands are swapped for the tensor core: 128 rows of W are the tcgen05 "M" side, the
//     (zero-padded) rows of X the "N" side, so no MMA lanes are wasted on padding of W;
//   - stream-K: the (W row-block, K-block) units are dealt out to one persistent CTA per SM in
//     equal shares, so every SM streams the same number of bytes whatever N is.  With T row-blocks
//     on G CTAs every CTA owns T div G whole row-blocks; the other T mod G row-blocks are cut along
//     K into G equal contiguous runs.  A CTA works through its run of the cut row-blocks FIRST and
//     its whole row-blocks last: the exchange of partial sums then overlaps the streaming of the
//     whole row-blocks, and the kernel ends with a plain store (16 x 28672 x 8192: the tail after
//     the last K block was 4.6 us with the cut row-blocks last);
//   - a 12-deep TMA ring (about 200 KB of loads in flight per SM);
//   - a CTA whose run covers only part of a row-block's K range writes an fp32 partial to a
//     workspace; the CTA that arrives last at that row-block (an atomic ticket, no spinning)
//     sums the partials in CTA order, which makes the result independent of timing.
//
// Reference counterpart: the same `matmul_kernel` as the dense path (examples/gemm.jl:4-64);
// MoYe has no split-K form.  The `gemm!` rank tower it follows is src/algorithm/blas.jl:39-88.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "ptx.cuh"

namespace moye {

struct SkinnyArgs {
  int M, N, K;
  int n_tiles, k_blocks;
  int split_tiles;      // row-blocks 0 .. split_tiles-1 are cut along K and shared by all CTAs
  int whole;            // whole row-blocks per CTA: split_tiles + c, split_tiles + c + grid, ...
  long long units;      // split_tiles * k_blocks: the units of the cut row-blocks
  uint32_t idesc;
  float alpha;
  void* D;
  long long d_sm, d_sn;  // element strides of D
  const float* bias;     // fused epilogue D = act(alpha * acc + bias); see moye_gemm_params_t.flags
  int bias_mode;         // 0 none, 1 bias[n], 2 bias[m]
  int act;               // 0 none, 1 relu, 2 gelu, 3 silu
  int* tickets;          // [n_tiles], zero between launches
  float* partials;       // [grid][2][NX][128] fp32
  int* status;
};

constexpr long long kMinRun = 8;  // shortest run of (row-block, K-block) units given to a CTA

enum : int { SITE_SK_PROD = 201, SITE_SK_ACC = 202, SITE_SK_FULL = 203, SITE_SK_EPI = 204 };

// AND-reduction of `pred` over the 128 epilogue threads (named barrier 1), so that all four
// epilogue warps take the same branch after a bounded wait.
__device__ __forceinline__ bool epi_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n.reg .pred p, q;\nsetp.ne.u32 q, %1, 0;\nbar.red.and.pred p, 1, 128, q;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// First unit of CTA c's run of the cut row-blocks' units: equal contiguous runs; with fewer units than CTAs the first
// `units` CTAs get one unit each (never an empty run BETWEEN two owners of a row-block: the exchange counts on every CTA
// from a row-block's first owner to its last arriving).
__device__ __forceinline__ long long run_start(long long c, long long units, int grid) {
  return units >= grid ? c * units / grid : (c < units ? c : units);
}

// The CTA whose run contains unit u.
__device__ __forceinline__ int owner_of(long long u, long long units, int grid) {
  if (units < grid) return (int)u;
  long long c = u * grid / units;
  while (c + 1 < grid && run_start(c + 1, units, grid) <= u) ++c;
  while (c > 0 && run_start(c, units, grid) > u) --c;
  return (int)c;
}

template <typename OutT>
__device__ __forceinline__ void store_out(void* D, long long off, float f) {
  if constexpr (sizeof(OutT) == 4) reinterpret_cast<float*>(D)[off] = f;
  else if constexpr (std::is_same<OutT, __half>::value) reinterpret_cast<__half*>(D)[off] = __float2half_rn(f);
  else reinterpret_cast<__nv_bfloat16*>(D)[off] = __float2bfloat16_rn(f);
}

template <typename OutT, int NX, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const SkinnyArgs g) {
  constexpr int BK = 64;
  constexpr int W_BYTES = 128 * 128;
  constexpr int X_BYTES = NX * 128;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr uint32_t TMEM_COLS = (2 * NX < 32) ? 32 : 2 * NX;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = bars + 2 * STAGES + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  int* ticket_bcast = reinterpret_cast<int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int grid = gridDim.x;
  // This CTA's work as one sequence v = 0 .. nv-1: first its run [u_begin, u_end) of the cut row-blocks' units, then
  // its whole row-blocks.  A segment is a maximal stretch of one row-block: one accumulator.
  const int kbn = g.k_blocks;
  const long long u_begin = run_start(blockIdx.x, g.units, grid);
  const long long u_end = run_start(blockIdx.x + 1, g.units, grid);
  const int ns = (int)(u_end - u_begin);
  const int nv = ns + g.whole * kbn;
  auto locate = [&](int v, int& tile, int& kb) {
    if (v < ns) {
      const long long u = u_begin + v;
      tile = (int)(u / kbn);
      kb = (int)(u - (long long)tile * kbn);
    } else {
      const int j = (v - ns) / kbn;
      tile = g.split_tiles + (int)blockIdx.x + j * grid;
      kb = (v - ns) - j * kbn;
    }
  };
  auto segment_end = [&](int v, int tile) {  // one past the last v of the segment that holds v
    if (v < ns) {
      const long long te = (long long)(tile + 1) * kbn - u_begin;
      return te < ns ? (int)te : ns;
    }
    return ns + ((v - ns) / kbn + 1) * kbn;
  };
  const int pre = nv < STAGES ? nv : STAGES;

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
    prefetch_tensormap(&tmW);
    prefetch_tensormap(&tmX);
    // the first ring of loads is requested at once: it is in flight while warp 1 allocates tensor memory and the
    // CTA meets at the barrier below
    griddep_wait();
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_x = l2_policy_evict_last();
    for (int i = 0; i < pre; ++i) {
      int tile, kb;
      locate(i, tile, kb);
      mbar_arrive_expect_tx(&full[i], STAGE_BYTES);
      uint8_t* sw = smem + i * STAGE_BYTES;
      tma_load_2d_hint(sw, &tmW, &full[i], kb * BK, tile * 128, pol_w);
      tma_load_2d_hint(sw + W_BYTES, &tmX, &full[i], kb * BK, 0, pol_x);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  // programmatic dependent launch (handle-based launches carry the attribute; without it both are no-ops): the next
  // grid of the stream may set itself up on this SM as soon as this CTA leaves; nothing above touched global memory
  // except the loads behind the producer's own wait
  griddep_launch();
  griddep_wait();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_holder);

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      int stage = pre == STAGES ? 0 : pre;
      uint32_t phase = pre == STAGES ? 1 : 0;
      for (int v = pre; v < nv; ++v) {
        int tile, kb;
        locate(v, tile, kb);
        if (!mbar_wait(&empty[stage], phase ^ 1, g.status, SITE_SK_PROD)) break;
        mbar_arrive_expect_tx(&full[stage], STAGE_BYTES);
        uint8_t* sw = smem + stage * STAGE_BYTES;
        tma_load_2d_hint(sw, &tmW, &full[stage], kb * BK, tile * 128, pol_w);
        tma_load_2d_hint(sw + W_BYTES, &tmX, &full[stage], kb * BK, 0, pol_x);
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int seg = 0;
      bool ok = true;
      int v = 0;
      while (v < nv && ok) {
        int tile, kb_first;
        locate(v, tile, kb_first);
        const int seg_end = segment_end(v, tile);
        const int buf = seg & 1;
        const uint32_t aphase = (seg >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], aphase ^ 1, g.status, SITE_SK_ACC)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * NX;
        bool first = true;
        for (; v < seg_end; ++v) {
          if (!mbar_wait(&full[stage], phase, g.status, SITE_SK_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sw = smem_u32(smem + stage * STAGE_BYTES);
          const uint64_t wdesc = umma_desc_k_sw128(sw);
          const uint64_t xdesc = umma_desc_k_sw128(sw + W_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            tc_mma_ss<KIND_F16>(d_tmem, wdesc + 2 * k, xdesc + 2 * k, g.idesc, (first && k == 0) ? 0u : 1u);
          }
          first = false;
          tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[buf]);
        ++seg;
      }
    }
  } else {
    const int q = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    int seg = 0;
    int v = 0;
    while (v < nv) {
      int tile, kb_first;
      locate(v, tile, kb_first);
      const int seg_end = segment_end(v, tile);
      const long long tile_begin = (long long)tile * kbn;  // in the units of the cut row-blocks (used for those only)
      const long long tile_end = tile_begin + kbn;
      const bool whole = kb_first == 0 && seg_end - v == kbn;
      const int buf = seg & 1;
      const uint32_t aphase = (seg >> 1) & 1;
      if (!epi_all(mbar_wait(&acc_full[buf], aphase, g.status, SITE_SK_EPI))) break;
      tc_fence_after_sync();
      // The accumulator is drained in chunks of CH columns (= rows of X) so that NX up to 128 needs no more
      // registers than NX = 32; the accumulator buffer is handed back after the last chunk has been read.
      constexpr int CH = NX < 32 ? NX : 32;
      const int last_c0 = ((g.M - 1) / CH) * CH;  // chunks past the M rows of X hold padding and are not read
      const int n_local = q * 32 + lane;
      const int n = tile * 128 + n_local;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * NX;
      auto load_chunk = [&](int c0, float (&acc)[CH]) {
        if constexpr (CH == 16) {
          uint32_t v[16];
          tmem_ld_x16(t_addr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = __uint_as_float(v[j]);
        } else {
          uint32_t v[32];
          tmem_ld_x32(t_addr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[j] = __uint_as_float(v[j]);
        }
        if (c0 == last_c0) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
      };
      // D(m, n) = act(alpha * x + bias): bias per output column n (one value per thread) or per row m
      const float bias_n = (g.bias_mode == 1 && n < g.N) ? __ldg(g.bias + n) : 0.f;
      auto finish_at = [&](int m, int col, float x, float bias_col) {
        float v = x * g.alpha + bias_col;
        if (g.bias_mode == 2) v += __ldg(g.bias + m);
        if (g.act == 1) v = fmaxf(v, 0.f);
        else if (g.act == 2) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
        else if (g.act == 3) v = v / (1.f + __expf(-v));
        store_out<OutT>(g.D, (long long)m * g.d_sm + (long long)col * g.d_sn, v);
      };
      auto finish = [&](int m, float x) { finish_at(m, n, x, bias_n); };
      // four consecutive columns of one row with one store, when D's rows are contiguous and aligned for it
      const bool vec_ok = g.d_sn == 1 && (g.d_sm & 3) == 0 && (reinterpret_cast<uintptr_t>(g.D) & (4 * sizeof(OutT) - 1)) == 0;
      auto finish4 = [&](int m, int col, const float (&x)[4], const float (&bcol)[4]) {
        if (vec_ok && col + 3 < g.N) {
          float v[4];
          const float brow = g.bias_mode == 2 ? __ldg(g.bias + m) : 0.f;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float t = x[e] * g.alpha + bcol[e] + brow;
            if (g.act == 1) t = fmaxf(t, 0.f);
            else if (g.act == 2) t = 0.5f * t * (1.f + erff(t * 0.70710678118654752f));
            else if (g.act == 3) t = t / (1.f + __expf(-t));
            v[e] = t;
          }
          OutT* dst = reinterpret_cast<OutT*>(g.D) + (long long)m * g.d_sm + col;
          if constexpr (sizeof(OutT) == 4) {
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          } else {
            OutT h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              if constexpr (std::is_same<OutT, __half>::value) h[e] = __float2half_rn(v[e]);
              else h[e] = __float2bfloat16_rn(v[e]);
            }
            uint2 w;
            w.x = (uint32_t)(*reinterpret_cast<uint16_t*>(&h[0])) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&h[1])) << 16);
            w.y = (uint32_t)(*reinterpret_cast<uint16_t*>(&h[2])) | ((uint32_t)(*reinterpret_cast<uint16_t*>(&h[3])) << 16);
            *reinterpret_cast<uint2*>(dst) = w;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col + e < g.N) finish_at(m, col + e, x[e], bcol[e]);
        }
      };
      if (whole) {
        // These warps run alone on their schedulers, so every instruction costs its full latency: the common case
        // (no activation, no per-row bias) is a multiply-add, a conversion, a store and a pointer step per row.
        const bool plain = g.act == 0 && g.bias_mode != 2;
        OutT* drow = reinterpret_cast<OutT*>(g.D) + (long long)n * g.d_sn;
        const long long dstep = g.d_sm;
        const float alpha = g.alpha;
#pragma unroll 1
        for (int c0 = 0; c0 <= last_c0; c0 += CH) {
          float acc[CH];
          load_chunk(c0, acc);
          if (n < g.N) {
            if (plain) {
              OutT* p = drow + (long long)c0 * dstep;
              const int left = g.M - c0;
#pragma unroll
              for (int j = 0; j < CH; ++j) {
                if (j < left) {
                  if constexpr (sizeof(OutT) == 4) *reinterpret_cast<float*>(p) = fmaf(acc[j], alpha, bias_n);
                  else if constexpr (std::is_same<OutT, __half>::value) *p = __float2half_rn(fmaf(acc[j], alpha, bias_n));
                  else *p = __float2bfloat16_rn(fmaf(acc[j], alpha, bias_n));
                }
                p += dstep;
              }
            } else {
#pragma unroll
              for (int j = 0; j < CH; ++j)
                if (c0 + j < g.M) finish(c0 + j, acc[j]);
            }
          }
        }
      } else {
        // partial sum: slot 0 for the first row-block of this CTA's run, slot 1 for the last
        const int slot = (tile == (int)(u_begin / kbn)) ? 0 : 1;
        float* mine = g.partials + ((long long)blockIdx.x * 2 + slot) * (NX * 128);
#pragma unroll 1
        for (int c0 = 0; c0 <= last_c0; c0 += CH) {
          float acc[CH];
          load_chunk(c0, acc);
#pragma unroll
          for (int j = 0; j < CH; ++j)
            if (c0 + j < g.M) __stcg(&mine[(c0 + j) * 128 + n_local], acc[j]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int c_first = owner_of(tile_begin, g.units, grid);
        const int c_last = owner_of(tile_end - 1, g.units, grid);
        if (et == 0) {
          const int old = atomicAdd(&g.tickets[tile], 1);
          *ticket_bcast = old;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int ticket = *reinterpret_cast<volatile int*>(ticket_bcast);
        if (ticket == c_last - c_first) {
          // last to arrive: every partial of this row-block is in memory; sum in CTA order.  Every CTA after
          // the first starts its run inside this row-block, so its partial is in slot 0; only the first one may
          // have come here from an earlier row-block (slot 1).  Thread (r, l) of the 4 x 32 epilogue threads sums
          // columns 4l .. 4l+3 of the rows r, r+4, ...: 128-bit loads, the partials of 8 CTAs in flight at once
          // (measured: the cost is per load instruction, about 26 ns each, plus one L2 round trip per batch).
          __threadfence();
          const int slot_first = run_start(c_first, g.units, grid) >= tile_begin ? 0 : 1;
          const int l4 = (et & 31) * 4;
          const int n4 = tile * 128 + l4;
          auto partial_of = [&](int c) {
            return g.partials + ((long long)c * 2 + (c == c_first ? slot_first : 0)) * (NX * 128) + l4;
          };
          float bias4[4] = {0.f, 0.f, 0.f, 0.f};
          if (g.bias_mode == 1) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (n4 + k < g.N) bias4[k] = __ldg(g.bias + n4 + k);
          }
#pragma unroll 1
          for (int m0 = et >> 5; m0 < g.M; m0 += 16) {  // rows m0, m0+4, m0+8, m0+12
            float4 sum[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) sum[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
            for (int c = c_first; c <= c_last; c += 8) {
              float4 v[8][4];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float* theirs = partial_of(c + i <= c_last ? c + i : c_last);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const int m = m0 + 4 * k;
                  v[i][k] = (m < g.M) ? __ldcg(reinterpret_cast<const float4*>(theirs + m * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (c + i <= c_last) {
#pragma unroll
                  for (int k = 0; k < 4; ++k) {
                    sum[k].x += v[i][k].x; sum[k].y += v[i][k].y; sum[k].z += v[i][k].z; sum[k].w += v[i][k].w;
                  }
                }
              }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int m = m0 + 4 * k;
              if (m < g.M) {
                const float x[4] = {sum[k].x, sum[k].y, sum[k].z, sum[k].w};
                finish4(m, n4, x, bias4);
              }
            }
          }
          if (et == 0) g.tickets[tile] = 0;  // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // ticket_bcast may be reused
      }
      v = seg_end;
      ++seg;
    }
  }

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

// Grid size and the split into cut and whole row-blocks (see the file comment).  One CTA per SM, but never runs
// shorter than 8 units (144 KB of W) when every row-block is cut: below that the partial-sum exchange costs more than
// the extra CTAs bring (4096 x 512 weights: 10.6 us against 16 with 148 CTAs).  With at least as many row-blocks as
// CTAs every CTA owns whole row-blocks and the left-over ones are cut over all CTAs; otherwise every row-block is
// cut and a CTA's run is one contiguous stretch of units.
static int plan_runs(SkinnyArgs& a, int num_sms) {
  const long long all = (long long)a.n_tiles * a.k_blocks;
  long long grid = num_sms;
  if (grid > all / kMinRun) grid = all / kMinRun > 0 ? all / kMinRun : 1;
  if (grid == num_sms && stream_k_whole_grid(a.n_tiles, a.k_blocks, num_sms)) grid = a.n_tiles;  // one whole row-block each
  const long long q = a.n_tiles / grid, r = a.n_tiles % grid;
  // Short runs and many partial sums per cut row-block are fine here: the exchange is hidden behind the whole
  // row-blocks (20480 x 8192: 55.7-56.9 -> 51.8-52.7 us with 12 cut row-blocks shared by 12-13 CTAs each; 19200 x 8192:
  // 54.0-55.4 -> 50.2-50.7 with 2 shared by 74 each)
  if (q >= 1) {
    a.whole = (int)q;
    a.split_tiles = (int)r;
  } else {
    a.whole = 0;
    a.split_tiles = a.n_tiles;
  }
  a.units = (long long)a.split_tiles * a.k_blocks;
  return (int)grid;
}

template <typename OutT, int NX>
static int launch_skinny_inst(moye_b200_ctx* h, const CUtensorMap& tw, const CUtensorMap& tx, SkinnyArgs a,
                              cudaStream_t stream) {
  constexpr int STAGE = 128 * 128 + NX * 128;
  constexpr int STAGES = (227 * 1024 - 1024 - 512) / STAGE;
  constexpr int SMEM = STAGES * STAGE + 512 + 1024;
  auto kern = gemm_skinny_kernel<OutT, NX, STAGES>;
  if (int rc = configure_once(h, kern, (int)SMEM)) return rc;
  const int grid = plan_runs(a, h->num_sms);
  // workspace: a fixed ticket area (zero at rest: the kernel restores it, moye_b200_status() clears it after a
  // time-out) then the partial slots.  It is allocated once, sized for the widest X tile, so no launch ever frees
  // or re-allocates it.
  if ((size_t)a.n_tiles * sizeof(int) > kSkinnyTicketBytes)
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "N = %d exceeds the %zu row-blocks the ticket area holds", a.N,
              kSkinnyTicketBytes / sizeof(int));
  if (!h->workspace) {
    if (int rc = ensure_workspace(h, kSkinnyTicketBytes + (size_t)h->num_sms * 2 * 128 * 128 * sizeof(float))) return rc;
  }
  a.tickets = reinterpret_cast<int*>(h->workspace);
  a.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(h->workspace) + kSkinnyTicketBytes);
  // every stream-K launch of a handle shares that scratch: a launch on another stream than the last one waits for it
  if (int rc = order_scratch_use(h, &h->sk_order, stream)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the kernel waits for the previous grid itself
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_without_pdl() ? 0 : 1;
  MOYE_CUDA(cudaLaunchKernelEx(&cfg, kern, tw, tx, a));
  return scratch_used(&h->sk_order, stream);
}

template <int NX>
static int launch_skinny_out(int out, moye_b200_ctx* h, const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyArgs& a,
                             cudaStream_t stream) {
  if (out == MOYE_F32) return launch_skinny_inst<float, NX>(h, tw, tx, a, stream);
  if (out == MOYE_F16) return launch_skinny_inst<__half, NX>(h, tw, tx, a, stream);
  return launch_skinny_inst<__nv_bfloat16, NX>(h, tw, tx, a, stream);
}

int launch_gemm_skinny(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                       const moye_gemm_params_t* p, cudaStream_t stream) {
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (A->dtype != MOYE_F16 && A->dtype != MOYE_BF16)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "the skinny path takes f16 or bf16 operands");
  if (M > 128) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "the skinny path needs M <= 128 (got %lld)", (long long)M);
  if (p->beta != 0.f) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the skinny path does not read C (beta must be 0)");
  const int out = D->dtype;
  if (!(out == MOYE_F32 || (out == MOYE_F16 && A->dtype == MOYE_F16) || (out == MOYE_BF16 && A->dtype == MOYE_BF16)))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "output dtype %d not supported for operand dtype %d", out, A->dtype);
  const int nx = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  CUtensorMap tw, tx;
  if (int rc = make_tmap_2d(h, &tw, B->ptr, B->dtype, K, N, (uint64_t)B->stride[0] * 2, 64, 128, true)) return rc;
  if (int rc = make_tmap_2d(h, &tx, A->ptr, A->dtype, K, M, (uint64_t)A->stride[0] * 2, 64, nx, true)) return rc;
  SkinnyArgs a;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.n_tiles = (int)((N + 127) / 128);
  a.k_blocks = (int)((K + 63) / 64);
  const uint32_t fmt = A->dtype == MOYE_BF16 ? 1u : 0u;
  a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(nx >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.alpha = p->alpha * p->scale_a * p->scale_b;
  a.D = D->ptr;
  a.d_sm = D->stride[0];
  a.d_sn = D->stride[1];
  a.partials = nullptr;
  a.tickets = nullptr;
  a.status = h->d_status;
  a.act = p->flags & MOYE_EPI_ACT_MASK;
  a.bias_mode = (p->flags & MOYE_EPI_BIAS_MASK) >> 4;
  a.bias = a.bias_mode ? p->bias : nullptr;
  switch (nx) {
    case 16: return launch_skinny_out<16>(out, h, tw, tx, a, stream);
    case 32: return launch_skinny_out<32>(out, h, tw, tx, a, stream);
    case 64: return launch_skinny_out<64>(out, h, tw, tx, a, stream);
    default: return launch_skinny_out<128>(out, h, tw, tx, a, stream);
  }
}

// ------------------------------------------------------------------------------------------
// The same stream-K kernel for callers that are not allowed to allocate device memory.
//
// Who that is: code running where cudaMalloc is off limits -- a host thread inside a
// latency-critical serving loop whose memory was carved up at start-up, a plugin that a host
// application loads under a "no allocations after initialisation" rule, or a caller that
// never created a handle (moye_b200_create allocates the status word and, later, the
// workspace).  For them the stream-K scratch (tickets + fp32 partial tiles + a status word)
// lives in this file-scope device array instead of the handle's workspace.  Every GPU that
// loads the library carries these bytes until the process exits.
constexpr int kStaticMaxSms = 160;          // CTAs the partial area is sized for (B200 has 148)
constexpr int kStaticMaxNx = 32;            // padded rows of X
constexpr int kStaticMaxRowBlocks = 4096;   // row blocks of W, i.e. N <= 524288
constexpr size_t kStaticStatusBytes = 256;
constexpr size_t kStaticTicketBytes = kStaticMaxRowBlocks * sizeof(int);
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxSms * 2 * kStaticMaxNx * 128 * sizeof(float);
constexpr size_t kStaticScratchBytes = kStaticStatusBytes + kStaticTicketBytes + kStaticPartialBytes;  // 5.02 MiB

static __device__ __align__(256) unsigned char g_skinny_scratch[kStaticScratchBytes];

// In host code `g_skinny_scratch` is only a stand-in for the symbol, not an address the GPU
// understands; the device address is looked up once per device and kept here.
struct StaticSetup {
  bool ready = false;
  unsigned char* base = nullptr;
  int num_sms = 0;
};
static StaticSetup g_static_setup[64];
static std::mutex g_static_mu;

template <typename OutT, int NX>
static int configure_skinny_kernel() {
  constexpr int STAGE = 128 * 128 + NX * 128;
  constexpr int STAGES = (227 * 1024 - 1024 - 512) / STAGE;
  constexpr int SMEM = STAGES * STAGE + 512 + 1024;
  MOYE_CUDA(cudaFuncSetAttribute(gemm_skinny_kernel<OutT, NX, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 SMEM));
  return MOYE_OK;
}

// First use on a device (that device being current): resolve the scratch address, size the grid,
// raise the kernels' shared-memory limit.  Nothing here allocates.
static int static_setup_for_current_device(StaticSetup** out) {
  int dev = -1;
  MOYE_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_static_mu);
  StaticSetup& s = g_static_setup[dev];
  if (!s.ready) {
    int major = 0, sms = 0;
    MOYE_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) MOYE_FAIL(MOYE_ERR_NO_DEVICE, "device %d is not sm_100", dev);
    MOYE_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    void* p = nullptr;
    MOYE_CUDA(cudaGetSymbolAddress(&p, g_skinny_scratch));
    if (int rc = configure_skinny_kernel<float, 16>()) return rc;
    if (int rc = configure_skinny_kernel<__half, 16>()) return rc;
    if (int rc = configure_skinny_kernel<__nv_bfloat16, 16>()) return rc;
    if (int rc = configure_skinny_kernel<float, 32>()) return rc;
    if (int rc = configure_skinny_kernel<__half, 32>()) return rc;
    if (int rc = configure_skinny_kernel<__nv_bfloat16, 32>()) return rc;
    s.base = static_cast<unsigned char*>(p);
    s.num_sms = sms;
    s.ready = true;
  }
  *out = &s;
  return MOYE_OK;
}

template <typename OutT, int NX>
static void launch_skinny_static(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyArgs& a, int grid,
                                 cudaStream_t stream) {
  constexpr int STAGE = 128 * 128 + NX * 128;
  constexpr int STAGES = (227 * 1024 - 1024 - 512) / STAGE;
  constexpr int SMEM = STAGES * STAGE + 512 + 1024;
  gemm_skinny_kernel<OutT, NX, STAGES><<<grid, 192, SMEM, stream>>>(tw, tx, a);
}

}  // namespace moye

extern "C" int moye_b200_gemm_skinny_static(const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                                            float alpha, int32_t* device_status, void* stream_) {
  using namespace moye;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!D || !A || !B) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "D, A and B must be non-null");
  if (A->rank != 2 || B->rank != 2 || D->rank != 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "A, B, D must be rank 2");
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K || D->shape[0] != M || D->shape[1] != N) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "shape mismatch");
  if (M <= 0 || N <= 0 || K <= 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "empty GEMM");
  if (!A->ptr || !B->ptr || !D->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null data pointer");
  if (A->dtype != B->dtype || (A->dtype != MOYE_F16 && A->dtype != MOYE_BF16))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "operands must both be f16 or both bf16");
  const int out = D->dtype;
  if (!(out == MOYE_F32 || (out == MOYE_F16 && A->dtype == MOYE_F16) || (out == MOYE_BF16 && A->dtype == MOYE_BF16)))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "output dtype %d not supported for operand dtype %d", out, A->dtype);
  if (A->stride[1] != 1 || B->stride[1] != 1)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "A and B must be K-major (stride 1 along K)");
  if (M > kStaticMaxNx)
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "M = %lld exceeds the %d rows the static scratch is sized for", (long long)M,
              kStaticMaxNx);
  if (K > INT32_MAX / 2) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "K = %lld is too large", (long long)K);
  if (N > (int64_t)kStaticMaxRowBlocks * 128)
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "N = %lld exceeds the %lld rows of W the static scratch is sized for (%d row blocks)",
              (long long)N, (long long)kStaticMaxRowBlocks * 128, kStaticMaxRowBlocks);
  StaticSetup* su = nullptr;
  if (int rc = static_setup_for_current_device(&su)) return rc;
  if (su->num_sms > kStaticMaxSms)
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "%d SMs exceed the %d the static scratch is sized for", su->num_sms, kStaticMaxSms);

  const int nx = M <= 16 ? 16 : 32;  // M <= kStaticMaxNx was checked above
  CUtensorMap tw, tx;
  if (int rc = encode_tmap_2d_uncached(&tw, B->ptr, B->dtype, K, N, (uint64_t)B->stride[0] * 2, 64, 128, true)) return rc;
  if (int rc = encode_tmap_2d_uncached(&tx, A->ptr, A->dtype, K, M, (uint64_t)A->stride[0] * 2, 64, nx, true)) return rc;

  SkinnyArgs a;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.n_tiles = (int)((N + 127) / 128);
  a.k_blocks = (int)((K + 63) / 64);
  const uint32_t fmt = A->dtype == MOYE_BF16 ? 1u : 0u;
  a.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(nx >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  a.alpha = alpha;
  a.bias = nullptr;
  a.bias_mode = 0;
  a.act = 0;
  a.D = D->ptr;
  a.d_sm = D->stride[0];
  a.d_sn = D->stride[1];
  a.status = device_status ? device_status : reinterpret_cast<int*>(su->base);
  a.tickets = reinterpret_cast<int*>(su->base + kStaticStatusBytes);
  a.partials = reinterpret_cast<float*>(su->base + kStaticStatusBytes + kStaticTicketBytes);
  // The array keeps whatever the previous call left: the tickets (and the built-in status word)
  // must read zero when the kernel starts, the partial tiles are always written before they are read.
  MOYE_CUDA(cudaMemsetAsync(su->base, 0, kStaticStatusBytes + (size_t)a.n_tiles * sizeof(int), stream));
  const int grid = plan_runs(a, su->num_sms);
  if (nx == 16) {
    if (out == MOYE_F32) launch_skinny_static<float, 16>(tw, tx, a, (int)grid, stream);
    else if (out == MOYE_F16) launch_skinny_static<__half, 16>(tw, tx, a, (int)grid, stream);
    else launch_skinny_static<__nv_bfloat16, 16>(tw, tx, a, (int)grid, stream);
  } else {
    if (out == MOYE_F32) launch_skinny_static<float, 32>(tw, tx, a, (int)grid, stream);
    else if (out == MOYE_F16) launch_skinny_static<__half, 32>(tw, tx, a, (int)grid, stream);
    else launch_skinny_static<__nv_bfloat16, 32>(tw, tx, a, (int)grid, stream);
  }
  MOYE_CUDA(cudaGetLastError());
  return MOYE_OK;
}

extern "C" int moye_b200_gemm_skinny_static_status(void* stream_, int32_t* site) {
  using namespace moye;
  StaticSetup* su = nullptr;
  if (int rc = static_setup_for_current_device(&su)) return rc;
  MOYE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)));
  int v = 0;
  MOYE_CUDA(cudaMemcpy(&v, su->base, sizeof(int), cudaMemcpyDeviceToHost));
  if (site) *site = v;
  if (v != 0) MOYE_FAIL(MOYE_ERR_TIMEOUT, "a bounded wait inside the static skinny GEMM ran out (site code %d)", v);
  return MOYE_OK;
}
