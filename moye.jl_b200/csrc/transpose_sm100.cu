// Transposing tiled copy for sm_100a: dst(i, j) = src(i, j) for rank-2 tensors of equal shape (m, n) where src is
// contiguous along n and dst along m, i.e. `copyto!(dest, transpose(src))`.
//
// Reference counterpart: `transpose_kernel` (test/host/copy_async.jl:51-74: @tile of both arrays, copyto!
// gmem->smem through a (32,32):(1,33) padded tile, `MoYe.transpose` of the shared tile, copyto! smem->gmem).
//
// Here a stage of 8V rows x 8V*NB columns (V = 16 / sizeof(T) elements per 128-bit vector; 8 KB, 16 KB for
// 1-byte elements) arrives by TMA in the 128-byte swizzle, 64 threads each turn V x V element blocks in registers
// (V 128-bit reads along the source rows, V 128-bit writes along the destination rows) into a second swizzled
// tile, and TMA stores it.  The thread -> block map walks diagonals, which makes every 8-lane phase of both the
// reads and the writes touch 8 distinct 16-byte bank groups: no padding, no bank conflicts.  Loads run one
// stage ahead of the stores, four CTAs per SM.  Ragged edges need no code: TMA zero-fills loads and clips stores.
// HBM-bound: algorithmic traffic is one read plus one write of the tensor.
#include "common.h"
#include "ptx.cuh"

namespace moye {

enum : int { SITE_TRANSPOSE_FULL = 311 };

struct TransposeArgs {
  int m;        // extent along the destination's contiguous mode
  int tiles_m;  // stages along m
  long long tiles;
  int* status;
};

// Tile order: m fastest.  A banded two-dimensional order (contiguous spans in both the source and the destination
// rows for the CTAs running together) was measured and made no difference (8192^2, fp16 and fp32).
__device__ __forceinline__ void transpose_tile_coord(long long t, const TransposeArgs& a, int& tm, int& tn) {
  tm = (int)(t % a.tiles_m);
  tn = (int)(t / a.tiles_m);
}

__device__ __forceinline__ uint4 lds_v4(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// out[c] = column c of the V x V block whose rows are in[0..V): element q of out[c] is element c of in[q].
template <int E>
__device__ __forceinline__ void transpose_block(const uint4 (&in)[16 / E], uint4 (&out)[16 / E]) {
  constexpr int V = 16 / E;
  uint32_t w[V][4];
#pragma unroll
  for (int q = 0; q < V; ++q) {
    w[q][0] = in[q].x; w[q][1] = in[q].y; w[q][2] = in[q].z; w[q][3] = in[q].w;
  }
#pragma unroll
  for (int c = 0; c < V; ++c) {
    uint32_t o[4];
    if constexpr (E == 8) {
      o[0] = w[0][2 * c]; o[1] = w[0][2 * c + 1]; o[2] = w[1][2 * c]; o[3] = w[1][2 * c + 1];
    } else if constexpr (E == 4) {
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = w[k][c];
    } else if constexpr (E == 2) {
#pragma unroll
      for (int k = 0; k < 4; ++k) o[k] = __byte_perm(w[2 * k][c >> 1], w[2 * k + 1][c >> 1], (c & 1) ? 0x7632 : 0x5410);
    } else {
      const uint32_t sel = (uint32_t)(((4 + (c & 3)) << 4) | (c & 3));  // byte c&3 of each of the two words
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t lo = __byte_perm(w[4 * k][c >> 2], w[4 * k + 1][c >> 2], sel);
        const uint32_t hi = __byte_perm(w[4 * k + 2][c >> 2], w[4 * k + 3][c >> 2], sel);
        o[k] = __byte_perm(lo, hi, 0x5410);
      }
    }
    out[c] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <int E, int SLOTS_ = 2, int NB_ = 0, int RM_ = 1>
struct TransposeCfg {
  static constexpr int RM = RM_;                       // square 8V x 8V sub-tiles along m per stage (1 or 2)
  static constexpr int V = 16 / E;                     // elements per 128-bit vector = block edge
  static constexpr int NB = NB_ ? NB_ : ((8 / V) > 0 ? (8 / V) : 1); // input boxes per stage: 8 KB stages (16 KB for 1-byte elements)
  static constexpr int ROWS = 8 * V * RM_;             // source rows (m) per stage
  static constexpr int COLS = 8 * V * NB;              // source columns (n) per stage
  static constexpr int IN_BOX = ROWS * 128;            // bytes of one input box {8V columns, 8V*RM rows}
  static constexpr int STAGE = IN_BOX * NB;
  static constexpr int OUT_HALF = STAGE / RM_;         // bytes of one output box {8V, 8V*NB}
  static constexpr int SLOTS = SLOTS_, LOOK = SLOTS_ - 1;
  static constexpr int SMEM = (SLOTS + 2) * STAGE + SLOTS * 8 + 1024;
};

template <int E, int SLOTS_ = 2, int NB_ = 0, int RM_ = 1>
__global__ void __launch_bounds__(64 * RM_) transpose_tma_kernel(const __grid_constant__ CUtensorMap tmS,
                                                            const __grid_constant__ CUtensorMap tmD,
                                                            const TransposeArgs a) {
  using Cfg = TransposeCfg<E, SLOTS_, NB_, RM_>;
  constexpr int V = Cfg::V, NB = Cfg::NB, STAGE = Cfg::STAGE, SLOTS = Cfg::SLOTS, LOOK = Cfg::LOOK;
  static_assert(SLOTS == LOOK + 1, "the slot refilled in iteration i is the one consumed in iteration i - 1");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* in = smem;
  uint8_t* out = smem + SLOTS * STAGE;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (SLOTS + 2) * STAGE);
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int s = 0; s < SLOTS; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
    prefetch_tensormap(&tmS);
    prefetch_tensormap(&tmD);
  }
  __syncthreads();
  griddep_launch();  // programmatic dependent launch: see launch_dependent()
  griddep_wait();

  const long long first = blockIdx.x, stride = gridDim.x;
  const long long mine = first < a.tiles ? (a.tiles - first + stride - 1) / stride : 0;
  auto issue_load = [&](long long i) {
    int tm, tn;
    transpose_tile_coord(first + i * stride, a, tm, tn);
    const int m0 = tm * Cfg::ROWS, n0 = tn * Cfg::COLS;
    const int slot = (int)(i % SLOTS);
    mbar_arrive_expect_tx(&full[slot], STAGE);
#pragma unroll
    for (int b = 0; b < NB; ++b) tma_load_2d(in + slot * STAGE + b * Cfg::IN_BOX, &tmS, &full[slot], n0 + b * 8 * V, m0);
  };
  if (tid == 0)
    for (long long i = 0; i < LOOK && i < mine; ++i) issue_load(i);

  // diagonal thread -> block map: row group i (rows V*i .. V*i+V-1), 16-byte column chunk j
  const int lane = tid & 31, warp = tid >> 5;
  const int t8 = lane & 7;
  const int bi = t8 + (RM_ == 2 ? 8 * (warp & 1) : 0);
  const int bj = (t8 + (lane >> 3) + 4 * (RM_ == 2 ? (warp >> 1) : warp)) & 7;
  bool failed = false;
  for (long long i = 0; i < mine; ++i) {
    const int slot = (int)(i % SLOTS);
    if (tid == 0) tma_store_wait_read<1>();  // the store that last read output buffer i & 1 has drained
    __syncthreads();                         // everyone is done with iteration i - 1
    if (tid == 0 && i + LOOK < mine) issue_load(i + LOOK);
    int ok = 1;
    if (tid == 0) ok = mbar_wait(&full[slot], (uint32_t)((i / SLOTS) & 1), a.status, SITE_TRANSPOSE_FULL) ? 1 : 0;
    if (__syncthreads_or(!ok)) {
      failed = true;
      break;
    }
    uint8_t* ob = out + (int)(i & 1) * STAGE + (bi >> 3) * Cfg::OUT_HALF;
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const uint8_t* ib = in + slot * STAGE + b * Cfg::IN_BOX;
      uint4 rin[V], rout[V];
#pragma unroll
      for (int q = 0; q < V; ++q) {
        const int r = V * bi + q;
        rin[q] = lds_v4(ib + r * 128 + ((bj ^ (r & 7)) << 4));
      }
      transpose_block<E>(rin, rout);
#pragma unroll
      for (int c = 0; c < V; ++c) {
        const int R = b * 8 * V + V * bj + c;  // destination row = source column inside the stage
        *reinterpret_cast<uint4*>(ob + R * 128 + (((bi & 7) ^ (R & 7)) << 4)) = rout[c];
      }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      int tm, tn;
      transpose_tile_coord(first + i * stride, a, tm, tn);
      const int m0 = tm * Cfg::ROWS, n0 = tn * Cfg::COLS;
      uint8_t* o = out + (int)(i & 1) * STAGE;
      tma_store_2d(&tmD, o, m0, n0);
      if (RM_ == 2 && m0 + 8 * V < a.m) tma_store_2d(&tmD, o + Cfg::OUT_HALF, m0 + 8 * V, n0);
      tma_store_commit();
    }
  }
  if (tid == 0) {
    tma_store_wait_all<0>();
    if (failed) {
      // a bounded wait gave up: loads may still be in flight into this CTA's shared memory; give them time
      for (int k = 0; k < 64; ++k) __nanosleep(1000);
    }
  }
}

template <int E, int SLOTS_ = 2, int NB_ = 0, int RM_ = 1>
static int launch_transpose_inst(moye_b200_ctx* h, const CUtensorMap& ts, const CUtensorMap& td, int64_t m, int64_t n,
                                 cudaStream_t stream) {
  using Cfg = TransposeCfg<E, SLOTS_, NB_, RM_>;
  TransposeArgs a;
  a.m = (int)m;
  a.tiles_m = (int)((m + Cfg::ROWS - 1) / Cfg::ROWS);
  a.tiles = (long long)a.tiles_m * ((n + Cfg::COLS - 1) / Cfg::COLS);
  a.status = h->d_status;
  auto kern = transpose_tma_kernel<E, SLOTS_, NB_, RM_>;
  if (int rc = configure_once(h, kern, Cfg::SMEM)) return rc;
  // Measured on 8192^2 (fp16 / fp32): 2 slots of 8 KB with 4 CTAs per SM reach 5.7 / 6.0 TB/s; deeper rings, larger
  // stages or more CTAs per SM all lose 5-20 % (more requests in flight scatter over more DRAM pages).
  int per_sm = 225 * 1024 / Cfg::SMEM;
  if (per_sm > 4) per_sm = 4;
  if (per_sm < 1) per_sm = 1;
  long long grid = a.tiles < (long long)h->num_sms * per_sm ? a.tiles : (long long)h->num_sms * per_sm;
  MOYE_CUDA(launch_dependent(kern, dim3((unsigned)grid), dim3(64 * RM_), Cfg::SMEM, stream, ts, td, a));
  return MOYE_OK;
}

// dst and src have shape (m, n); src has stride 1 along n, dst stride 1 along m (the caller swaps modes for the
// mirrored case).  Pitches are in elements.
int launch_transpose(moye_b200_ctx* h, void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int dtype,
                     int64_t m, int64_t n, cudaStream_t stream) {
  const int eb = dtype_bytes(dtype);
  if (eb != 1 && eb != 2 && eb != 4 && eb != 8)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "the transposing copy takes elements of 1, 2, 4 or 8 bytes");
  if (m > INT32_MAX / 4 || n > INT32_MAX / 4) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "extent too large");
  if (((uintptr_t)src & 15) || ((uintptr_t)dst & 15))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "the transposing copy needs 16-byte aligned base pointers");
  if ((m > 1 && (src_pitch * eb) % 16 != 0) || (n > 1 && (dst_pitch * eb) % 16 != 0))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "pitches must be multiples of 16 bytes");
  const int V = 16 / eb;
  const int nb = (8 / V) > 0 ? (8 / V) : 1;
  const int rm = 1;  // rows of 8V x 8V sub-tiles per stage (TransposeCfg::RM)
  CUtensorMap ts, td;
  if (int rc = make_tmap_2d(h, &ts, src, dtype, n, m, (uint64_t)src_pitch * eb, 8 * V, 8 * V * rm, TMAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tmap_2d(h, &td, dst, dtype, m, n, (uint64_t)dst_pitch * eb, 8 * V, 8 * V * nb, TMAP_SWIZZLE_128B)) return rc;
  switch (eb) {
    case 1: return launch_transpose_inst<1>(h, ts, td, m, n, stream);
    case 2: return launch_transpose_inst<2>(h, ts, td, m, n, stream);
    case 4: return launch_transpose_inst<4>(h, ts, td, m, n, stream);
    default: return launch_transpose_inst<8>(h, ts, td, m, n, stream);
  }
}

}  // namespace moye
