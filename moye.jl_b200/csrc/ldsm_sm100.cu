// `copyto!(tiled_copy, dst, src)` for a TiledCopy built on an ldmatrix atom (`LDSM_U32x1_N` ... `LDSM_U16x8_T`,
// reference src/arch/copy/ldmatrix.jl:18-96, traits src/traits/ldmatrix.jl:1-41): the kernel of the reference's
// own device test (test/device/tiled_copy.jl:2-23).  One tile of 16-bit elements goes global -> shared memory
// through its layout, every thread loads its fragments with `ldmatrix` from the shared-memory addresses that
// `partition_S` gives it, and stores the values it received to the global addresses that `partition_D` gives it.
// With a consistent TiledCopy the output equals the input; that is the test.
//
// The partitions are MoYe's host-side layout algebra: the caller evaluates them once and passes two tables of
// element offsets (the first element of every source fragment; every destination value).  The dense GEMM kernels
// do not use ldmatrix -- tcgen05.mma reads shared memory through descriptors -- so this path exists for the
// TiledCopy API surface, not for speed: one CTA, a tile of at most 48 KB.
#include "common.h"
#include "ptx.cuh"

namespace moye {

template <int X, bool TRANS>
__device__ __forceinline__ void ldmatrix_b16(uint32_t addr, uint32_t (&r)[4]) {
  if constexpr (X == 1) {
    if constexpr (TRANS) asm volatile("ldmatrix.sync.aligned.m8n8.x1.trans.shared.b16 {%0}, [%1];" : "=r"(r[0]) : "r"(addr));
    else asm volatile("ldmatrix.sync.aligned.m8n8.x1.shared.b16 {%0}, [%1];" : "=r"(r[0]) : "r"(addr));
  } else if constexpr (X == 2) {
    if constexpr (TRANS) asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
    else asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
  } else {
    if constexpr (TRANS)
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
    else
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
  }
}

// src_off[t * iters + i]: element offset in the tile of the first value of thread t's i-th source fragment (8
// contiguous 16-bit values, 16-byte aligned); dst_off[(t * iters + i) * 2X + v]: element offset of the v-th value the
// thread receives.  `span` elements are staged (the cosize of the tile's layout).
template <int X, bool TRANS>
__global__ void ldsm_tiled_copy_kernel(uint16_t* out, const uint16_t* in, int span, int iters, const int* src_off,
                                       const int* dst_off, int* status) {
  extern __shared__ __align__(16) uint16_t tile[];
  for (int i = threadIdx.x; i < span; i += blockDim.x) tile[i] = in[i];
  __syncthreads();
  for (int it = 0; it < iters; ++it) {
    const int so = src_off[threadIdx.x * iters + it];
    uint32_t r[4] = {0u, 0u, 0u, 0u};
    // the instruction is warp-wide: every lane executes it, with an address inside the tile
    const bool ok = MOYE_DBG_OK(so >= 0 && so + 8 <= span && (so & 7) == 0, status, 971);
    ldmatrix_b16<X, TRANS>(smem_u32(tile + (ok ? so : 0)), r);
    const int* d = dst_off + (size_t)(threadIdx.x * iters + it) * (2 * X);
#pragma unroll
    for (int v = 0; v < 2 * X; ++v) {
      const int o = d[v];
      if (MOYE_DBG_OK(o >= 0 && o < span, status, 972)) out[o] = (uint16_t)(r[v >> 1] >> (16 * (v & 1)));
    }
  }
}

}  // namespace moye

using namespace moye;

extern "C" int moye_b200_ldsm_copy(moye_handle_t h, void* dst, const void* src, int32_t span, int32_t matrices,
                                   int32_t transposed, int32_t threads, int32_t iters, const int32_t* src_offsets,
                                   const int32_t* dst_offsets, void* stream_) {
  if (!h) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null handle");
  int dev = -1;
  MOYE_CUDA(cudaGetDevice(&dev));
  if (dev != h->device) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "handle belongs to device %d but device %d is current", h->device, dev);
  if (!dst || !src || !src_offsets || !dst_offsets) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null argument");
  if (matrices != 1 && matrices != 2 && matrices != 4) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "ldmatrix moves 1, 2 or 4 matrices (got %d)", matrices);
  if (threads < 32 || threads > 1024 || threads % 32) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "threads must be a multiple of 32 up to 1024 (got %d)", threads);
  if (iters < 1 || span < 8) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "empty tile");
  if ((size_t)span * 2 > 48 * 1024) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "the tile spans %d elements; one CTA stages at most 24576", span);
  if ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 1) MOYE_FAIL(MOYE_ERR_MISALIGNED, "16-bit elements need 2-byte alignment");
  // every source fragment: 8 contiguous values inside the tile on a 16-byte boundary; every destination inside it
  const size_t n_src = (size_t)threads * iters, n_dst = n_src * 2 * matrices;
  for (size_t i = 0; i < n_src; ++i)
    if (src_offsets[i] < 0 || src_offsets[i] + 8 > span || (src_offsets[i] & 7))
      MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "source fragment %zu starts at element %d: ldmatrix rows are 8 contiguous 16-bit "
                "values on a 16-byte boundary inside the tile", i, src_offsets[i]);
  for (size_t i = 0; i < n_dst; ++i)
    if (dst_offsets[i] < 0 || dst_offsets[i] >= span) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "destination offset %d outside the tile", dst_offsets[i]);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t bytes = (n_src + n_dst) * sizeof(int);
  if (bytes > h->table_bytes) {
    if (h->table) {
      MOYE_CUDA(cudaDeviceSynchronize());
      MOYE_CUDA(cudaFree(h->table));
      h->table = nullptr;
      h->table_bytes = 0;
    }
    const size_t want = bytes < (64u << 10) ? (64u << 10) : bytes;
    MOYE_CUDA(cudaMalloc(&h->table, want));
    h->table_bytes = want;
  }
  if (int rc = order_scratch_use(h, &h->table_order, stream)) return rc;
  int* d_src = reinterpret_cast<int*>(h->table);
  int* d_dst = d_src + n_src;
  MOYE_CUDA(cudaMemcpyAsync(d_src, src_offsets, n_src * sizeof(int), cudaMemcpyHostToDevice, stream));
  MOYE_CUDA(cudaMemcpyAsync(d_dst, dst_offsets, n_dst * sizeof(int), cudaMemcpyHostToDevice, stream));
  const size_t smem = ((size_t)span * 2 + 15) & ~size_t(15);
  uint16_t* o = static_cast<uint16_t*>(dst);
  const uint16_t* in = static_cast<const uint16_t*>(src);
#define MOYE_LDSM(XX, TT) ldsm_tiled_copy_kernel<XX, TT><<<1, threads, smem, stream>>>(o, in, span, iters, d_src, d_dst, h->d_status)
  if (transposed) {
    if (matrices == 1) MOYE_LDSM(1, true); else if (matrices == 2) MOYE_LDSM(2, true); else MOYE_LDSM(4, true);
  } else {
    if (matrices == 1) MOYE_LDSM(1, false); else if (matrices == 2) MOYE_LDSM(2, false); else MOYE_LDSM(4, false);
  }
#undef MOYE_LDSM
  MOYE_CUDA(cudaGetLastError());
  return scratch_used(&h->table_order, stream);
}
