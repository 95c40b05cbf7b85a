// Tiled copy kernels for sm_100a: dst = src for rank-2 tensors whose first mode is contiguous
// (MoYe's column-major default), moved tile by tile through shared memory.
//
// Reference counterparts: `copy_kernel` (test/host/copy_async.jl:3-25: @tile, @parallelize,
// copyto! gmem->smem, cp_async_wait, sync_threads, copyto! smem->gmem) and the atom path
// `copyto!(tiled_copy, dst, src)` (src/algorithm/copy.jl:106-130) with
// `UniversalCopy{UInt128}` atoms (src/arch/copy/copy.jl:26-51).
//
// Two forms:
//   1. UNIVERSAL128 -- 256 threads laid out (tile_m/8, 256/(tile_m/8)) over the tile, each
//      moving 128-bit values: ld.global.nc.v4 -> st.shared.v4 -> bar -> ld.shared.v4 ->
//      st.global.v4.  All of a thread's loads are issued before the first store so that
//      16 KB per CTA (x 8 CTAs per SM) are in flight.
//   2. TMA -- one elected thread per CTA drives a ring of shared-memory tiles:
//      cp.async.bulk.tensor load (mbarrier completion) then cp.async.bulk.tensor store
//      straight out of the same tile; loads run LOOKAHEAD tiles ahead of stores (3 slots, 1 ahead,
//      two to four CTAs per SM).
// Both are HBM-bound: algorithmic traffic is one read plus one write of the tensor.
#include <utility>

#include "common.h"
#include "ptx.cuh"

namespace moye {

enum : int { SITE_COPY_FULL = 301 };

__device__ __forceinline__ uint4 ld_nc_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_v4(uint4* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

struct CopyArgs {
  const uint4* src;
  uint4* dst;
  long long src_pitch;  // uint4 units between consecutive columns
  long long dst_pitch;
  int m_vecs;           // extent of the contiguous mode in uint4
  int n;                // extent of the strided mode
  int tmv_log2;         // log2(tile extent along m in uint4)
  int tn;               // tile extent along n
  int tiles_m;
  long long tiles;
};

template <int ITEMS>
__global__ void __launch_bounds__(256) copy_u128_kernel(const CopyArgs a) {
  extern __shared__ uint4 tile[];
  griddep_launch();  // programmatic dependent launch: see launch_dependent()
  griddep_wait();
  const int tmv = 1 << a.tmv_log2;
  const int tile_items = tmv * a.tn;
  for (long long t = blockIdx.x; t < a.tiles; t += gridDim.x) {
    const int tm = (int)(t % a.tiles_m);
    const long long tn_i = t / a.tiles_m;
    uint4 r[ITEMS];
    bool ok[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int item = threadIdx.x + i * 256;
      const int vec = item & (tmv - 1);
      const int col = item >> a.tmv_log2;
      const int gm = tm * tmv + vec;
      const long long gn = tn_i * a.tn + col;
      ok[i] = item < tile_items && gm < a.m_vecs && gn < a.n;
      if (ok[i]) r[i] = ld_nc_v4(a.src + gn * a.src_pitch + gm);
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
      if (ok[i]) tile[threadIdx.x + i * 256] = r[i];
    __syncthreads();
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
      const int item = threadIdx.x + i * 256;
      if (ok[i]) {
        const int vec = item & (tmv - 1);
        const int col = item >> a.tmv_log2;
        const uint4 v = tile[item];
        st_v4(a.dst + (tn_i * a.tn + col) * a.dst_pitch + tm * tmv + vec, v);
      }
    }
    __syncthreads();
  }
}

struct TmaCopyArgs {
  int tiles_m;
  long long tiles;
  int box_m, box_n;
  int tile_bytes;
  int* status;
};

template <int SLOTS, int LOOKAHEAD>
__global__ void __launch_bounds__(32) copy_tma_kernel(const __grid_constant__ CUtensorMap tmS,
                                                      const __grid_constant__ CUtensorMap tmD, const TmaCopyArgs a) {
  static_assert(SLOTS - LOOKAHEAD - 1 >= 0, "ring too small for the lookahead");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)SLOTS * a.tile_bytes);
  if (threadIdx.x == 0) {
    for (int s = 0; s < SLOTS; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
    prefetch_tensormap(&tmS);
    prefetch_tensormap(&tmD);
  }
  __syncwarp();
  griddep_launch();  // programmatic dependent launch: see launch_dependent()
  griddep_wait();
  if (threadIdx.x == 0) {
    const long long first = blockIdx.x;
    const long long stride = gridDim.x;
    const long long mine = first < a.tiles ? (a.tiles - first + stride - 1) / stride : 0;
    for (long long i = 0; i < mine + LOOKAHEAD; ++i) {
      if (i < mine) {
        const int slot = (int)(i % SLOTS);
        // the store that last read this slot (tile i - SLOTS) must have drained
        tma_store_wait_read<SLOTS - LOOKAHEAD - 1>();
        const long long t = first + i * stride;
        const int x = (int)(t % a.tiles_m) * a.box_m;
        const int y = (int)(t / a.tiles_m) * a.box_n;
        mbar_arrive_expect_tx(&full[slot], a.tile_bytes);
        tma_load_2d(smem + (size_t)slot * a.tile_bytes, &tmS, &full[slot], x, y);
      }
      if (i >= LOOKAHEAD) {
        const long long j = i - LOOKAHEAD;
        const int slot = (int)(j % SLOTS);
        const uint32_t parity = (uint32_t)((j / SLOTS) & 1);
        if (!mbar_wait(&full[slot], parity, a.status, SITE_COPY_FULL)) break;
        const long long t = first + j * stride;
        const int x = (int)(t % a.tiles_m) * a.box_m;
        const int y = (int)(t / a.tiles_m) * a.box_n;
        tma_store_2d(&tmD, smem + (size_t)slot * a.tile_bytes, x, y);
        tma_store_commit();
      }
    }
    tma_store_wait_all<0>();
    if (*reinterpret_cast<volatile int*>(a.status) != 0) {
      for (int k = 0; k < 64; ++k) __nanosleep(1000);
    }
  }
}

static int ilog2_exact(long long v) {
  int l = 0;
  while ((1ll << l) < v) ++l;
  return (1ll << l) == v ? l : -1;
}

int launch_copy(moye_b200_ctx* h, const moye_tensor_t* dst_in, const moye_tensor_t* src_in, const moye_copy_params_t* pp,
                cudaStream_t stream) {
  moye_copy_params_t p = {MOYE_COPY_AUTO, 0, 0, 0};
  if (pp) p = *pp;
  if (p.flags != 0) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "flags must be 0");
  if (dst_in->rank != 2 || src_in->rank != 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "tiled copy takes rank-2 tensors");
  moye_tensor_t dst_v = *dst_in, src_v = *src_in;
  if (src_v.stride[1] == 1 && dst_v.stride[1] == 1 && !(src_v.stride[0] == 1 && dst_v.stride[0] == 1)) {
    // both row-major: the same copy with the modes of both views (and of the tile) swapped
    for (moye_tensor_t* t : {&dst_v, &src_v}) {
      std::swap(t->shape[0], t->shape[1]);
      std::swap(t->stride[0], t->stride[1]);
    }
    std::swap(p.tile_m, p.tile_n);
  }
  const moye_tensor_t *dst = &dst_v, *src = &src_v;
  if (dst->dtype != src->dtype) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "dst and src dtypes differ");
  const int eb = dtype_bytes(src->dtype);
  if (eb == 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "unknown dtype %d", src->dtype);
  const int64_t m = src->shape[0], n = src->shape[1];
  if (dst->shape[0] != m || dst->shape[1] != n) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "dst and src shapes differ");
  if (m == 0 || n == 0) return MOYE_OK;  // nothing to move
  if (m < 0 || n < 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "negative extent");
  if (!dst->ptr || !src->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null data pointer");
  // operands of different majorness: the transposing kernel (`copyto!(dest, transpose(src))`)
  const bool s0 = src->stride[0] == 1 || m == 1, s1 = src->stride[1] == 1 || n == 1;
  const bool d0 = dst->stride[0] == 1 || m == 1, d1 = dst->stride[1] == 1 || n == 1;
  if (p.mode == MOYE_COPY_TRANSPOSE || (p.mode == MOYE_COPY_AUTO && !(s0 && d0) && ((s1 && d0) || (s0 && d1)))) {
    if (p.tile_m != 0 || p.tile_n != 0) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the transposing copy chooses its own tiles");
    log_line("copy %lld x %lld, %d-byte elements -> transposing kernel", (long long)m, (long long)n, eb);
    if (src->stride[1] == 1 && dst->stride[0] == 1)
      return launch_transpose(h, dst->ptr, dst->stride[1], src->ptr, src->stride[0], src->dtype, m, n, stream);
    if (src->stride[0] == 1 && dst->stride[1] == 1)  // the mirrored case: swap the modes of both views
      return launch_transpose(h, dst->ptr, dst->stride[0], src->ptr, src->stride[1], src->dtype, n, m, stream);
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT,
              "the transposing copy needs src with stride 1 along one mode and dst with stride 1 along the other");
  }
  if (src->stride[0] != 1 || dst->stride[0] != 1)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "tiled copy needs stride 1 along the first mode of both tensors");
  if (m > INT32_MAX / 4 || n > INT32_MAX / 4) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "extent too large");
  // default tile: 256-byte columns x 64 columns = 16 KB (128 x 64 for 2-byte elements)
  const int tile_m = p.tile_m ? p.tile_m : (256 / eb > 0 ? 256 / eb : 1);
  const int tile_n = p.tile_n ? p.tile_n : 64;
  if (tile_m <= 0 || tile_n <= 0) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "bad tile");
  if (((uintptr_t)src->ptr & 15) || ((uintptr_t)dst->ptr & 15))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "tiled copy needs 16-byte aligned base pointers");
  if ((m * eb) % 16 != 0 || (n > 1 && ((src->stride[1] * eb) % 16 != 0 || (dst->stride[1] * eb) % 16 != 0)))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "column length and pitches must be multiples of 16 bytes for 128-bit atoms");
  int mode = p.mode;
  if (mode == MOYE_COPY_AUTO) mode = (eb <= 8 && tile_m <= 256) ? MOYE_COPY_TMA : MOYE_COPY_UNIVERSAL128;
  log_line("copy %lld x %lld, %d-byte elements, tile %d x %d -> %s", (long long)m, (long long)n, eb, tile_m, tile_n,
           mode == MOYE_COPY_TMA ? "TMA ring" : "128-bit universal copy");

  if (mode == MOYE_COPY_UNIVERSAL128) {
    const long long tile_m_bytes = (long long)tile_m * eb;
    const int lg = ilog2_exact(tile_m_bytes / 16);
    if (tile_m_bytes % 16 != 0 || lg < 0)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile_m * sizeof(T) must be 16 * 2^k bytes (got %lld)", tile_m_bytes);
    const int tmv = 1 << lg;
    const long long items = (long long)tmv * tile_n;
    if (items > 256 * 8) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile of %lld bytes exceeds 32 KB", items * 16);
    CopyArgs a;
    a.src = reinterpret_cast<const uint4*>(src->ptr);
    a.dst = reinterpret_cast<uint4*>(dst->ptr);
    a.src_pitch = src->stride[1] * eb / 16;
    a.dst_pitch = dst->stride[1] * eb / 16;
    a.m_vecs = (int)(m * eb / 16);
    a.n = (int)n;
    a.tmv_log2 = lg;
    a.tn = tile_n;
    a.tiles_m = (a.m_vecs + tmv - 1) / tmv;
    a.tiles = (long long)a.tiles_m * ((n + tile_n - 1) / tile_n);
    const int per_thread = (int)((items + 255) / 256);
    const size_t smem = (size_t)per_thread * 256 * 16;
    long long grid = a.tiles < (long long)h->num_sms * 8 ? a.tiles : (long long)h->num_sms * 8;
    const dim3 g((unsigned)grid), b(256);
    if (per_thread <= 1) MOYE_CUDA(launch_dependent(copy_u128_kernel<1>, g, b, smem, stream, a));
    else if (per_thread <= 2) MOYE_CUDA(launch_dependent(copy_u128_kernel<2>, g, b, smem, stream, a));
    else if (per_thread <= 4) MOYE_CUDA(launch_dependent(copy_u128_kernel<4>, g, b, smem, stream, a));
    else MOYE_CUDA(launch_dependent(copy_u128_kernel<8>, g, b, smem, stream, a));
    return MOYE_OK;
  }
  if (mode == MOYE_COPY_TMA) {
    if (eb > 8) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "TMA copy takes elements of at most 8 bytes");
    if (tile_m > 256 || tile_n > 256) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "TMA box extents are limited to 256");
    if (((long long)tile_m * eb) % 16 != 0) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile_m * sizeof(T) must be a multiple of 16");
    const long long tile_bytes = (long long)tile_m * tile_n * eb;
    if (tile_bytes % 128 != 0) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile bytes (%lld) must be a multiple of 128", tile_bytes);
    // Measured on 8192^2 fp16 (128 x 64 tiles): 3 slots, loads one tile ahead, 2 CTAs per SM: 5.98 TB/s; the first
    // configuration (6 slots, two ahead) 5.57; 8 KB tiles (256 x 16) with 4 CTAs per SM 5.96-6.04.  As in the
    // transposing kernel, fewer requests in flight per SM is faster, not slower.
    constexpr int SLOTS = 3, LOOK = 1;
    if (tile_bytes * SLOTS + 1024 > 110 * 1024)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "tile of %lld bytes is too large for the %d-slot ring", tile_bytes, SLOTS);
    CUtensorMap ts, td;
    if (int rc = make_tmap_2d(h, &ts, src->ptr, src->dtype, m, n, (uint64_t)src->stride[1] * eb, tile_m, tile_n, false))
      return rc;
    if (int rc = make_tmap_2d(h, &td, dst->ptr, dst->dtype, m, n, (uint64_t)dst->stride[1] * eb, tile_m, tile_n, false))
      return rc;
    TmaCopyArgs a;
    a.tiles_m = (int)((m + tile_m - 1) / tile_m);
    a.tiles = (long long)a.tiles_m * ((n + tile_n - 1) / tile_n);
    a.box_m = tile_m;
    a.box_n = tile_n;
    a.tile_bytes = (int)tile_bytes;
    a.status = h->d_status;
    const size_t smem = (size_t)tile_bytes * SLOTS + 128 + SLOTS * 8;
    auto kern = copy_tma_kernel<SLOTS, LOOK>;
    // the limit is raised once per handle, so it must cover every tile the checks above admit, not just this one
    if (int rc = configure_once(h, kern, 110 * 1024 + 128 + SLOTS * 8)) return rc;
    long long per_sm = (96 * 1024) / (tile_bytes * SLOTS);  // 2 CTAs per SM with 16 KB tiles, 4 with 8 KB ones
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    long long grid = a.tiles < (long long)h->num_sms * per_sm ? a.tiles : (long long)h->num_sms * per_sm;
    MOYE_CUDA(launch_dependent(kern, dim3((unsigned)grid), dim3(32), smem, stream, ts, td, a));
    return MOYE_OK;
  }
  MOYE_FAIL(MOYE_ERR_INVALID_ARG, "unknown copy mode %d", mode);
}

}  // namespace moye
