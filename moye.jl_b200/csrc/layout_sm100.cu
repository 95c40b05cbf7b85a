// Layout-function evaluation on the device, and the elementwise copy through two layouts.
//
// A MoYe `Layout` maps a 1-based linear index to a 1-based offset:
//   layout(i) = 1 + sum_k ((i-1) / prod(shape[0..k-1]) % shape[k]) * stride[k]
// over the flattened modes in colexicographic order; the last mode wraps like the others
// and a layout with a single mode does not wrap at all
// (reference src/stride.jl:20-31 `coord_to_index0` applied to an integer coordinate, reached
// from the call operator in src/layout.jl).  `copyto!(dst, src)` walks i = 1:size(src) through
// both layouts (reference src/algorithm/copy.jl:4-16,42-64).
#include "common.h"

namespace moye {

struct FlatLayout {
  int rank;
  long long shape[MOYE_MAX_FLAT_RANK];
  long long stride[MOYE_MAX_FLAT_RANK];
};

__device__ __forceinline__ long long layout_offset0(const FlatLayout& l, long long idx0) {
  if (l.rank == 1) return idx0 * l.stride[0];  // a single mode does not wrap
  long long off = 0;
#pragma unroll 1
  for (int k = 0; k < l.rank; ++k) {
    const long long s = l.shape[k];
    const long long q = idx0 / s;
    off += (idx0 - q * s) * l.stride[k];
    idx0 = q;
  }
  return off;
}

__global__ void __launch_bounds__(256) layout_eval_kernel(const FlatLayout l, long long first, long long n,
                                                          long long* out) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = 1 + layout_offset0(l, first + i - 1);
}

template <typename T>
__global__ void __launch_bounds__(256) layout_copy_kernel(T* dst, const FlatLayout dl, const T* src,
                                                          const FlatLayout sl, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[layout_offset0(dl, i)] = src[layout_offset0(sl, i)];
}

static int flatten_arg(const moye_layout_t* in, FlatLayout* out, long long* size) {
  if (in->rank < 1 || in->rank > MOYE_MAX_FLAT_RANK)
    MOYE_FAIL(MOYE_ERR_INVALID_ARG, "layout rank %d outside 1..%d", in->rank, MOYE_MAX_FLAT_RANK);
  long long sz = 1;
  out->rank = in->rank;
  for (int k = 0; k < in->rank; ++k) {
    if (in->shape[k] < 1) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "layout extent %lld in mode %d", (long long)in->shape[k], k);
    if (sz > INT64_MAX / in->shape[k]) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "layout size overflows 63 bits");
    sz *= in->shape[k];
    out->shape[k] = in->shape[k];
    out->stride[k] = in->stride[k];
  }
  *size = sz;
  return MOYE_OK;
}

int launch_layout_eval(moye_b200_ctx* h, const moye_layout_t* l, int64_t first, int64_t n, int64_t* out,
                       cudaStream_t stream) {
  FlatLayout fl;
  long long sz;
  if (int rc = flatten_arg(l, &fl, &sz)) return rc;
  if (n < 0 || first < 1) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "need n >= 0 and a 1-based first index");
  if (n == 0) return MOYE_OK;
  long long blocks = (n + 255) / 256;
  const long long cap = (long long)h->num_sms * 8;
  if (blocks > cap) blocks = cap;
  layout_eval_kernel<<<(int)blocks, 256, 0, stream>>>(fl, first, n, reinterpret_cast<long long*>(out));
  MOYE_CUDA(cudaGetLastError());
  return MOYE_OK;
}

int launch_layout_copy(moye_b200_ctx* h, void* dst, const moye_layout_t* dl, const void* src,
                       const moye_layout_t* sl, int elem_bytes, cudaStream_t stream) {
  FlatLayout fd, fs;
  long long nd, ns;
  if (int rc = flatten_arg(dl, &fd, &nd)) return rc;
  if (int rc = flatten_arg(sl, &fs, &ns)) return rc;
  if (nd != ns) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "layout sizes differ: dst %lld, src %lld", nd, ns);
  if (((uintptr_t)dst % elem_bytes) || ((uintptr_t)src % elem_bytes))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "pointers must be aligned to the element size");
  long long blocks = (ns + 255) / 256;
  const long long cap = (long long)h->num_sms * 8;
  if (blocks > cap) blocks = cap;
  switch (elem_bytes) {
    case 1: layout_copy_kernel<uint8_t><<<(int)blocks, 256, 0, stream>>>((uint8_t*)dst, fd, (const uint8_t*)src, fs, ns); break;
    case 2: layout_copy_kernel<uint16_t><<<(int)blocks, 256, 0, stream>>>((uint16_t*)dst, fd, (const uint16_t*)src, fs, ns); break;
    case 4: layout_copy_kernel<uint32_t><<<(int)blocks, 256, 0, stream>>>((uint32_t*)dst, fd, (const uint32_t*)src, fs, ns); break;
    case 8: layout_copy_kernel<uint64_t><<<(int)blocks, 256, 0, stream>>>((uint64_t*)dst, fd, (const uint64_t*)src, fs, ns); break;
    case 16: layout_copy_kernel<uint4><<<(int)blocks, 256, 0, stream>>>((uint4*)dst, fd, (const uint4*)src, fs, ns); break;
    default: MOYE_FAIL(MOYE_ERR_INVALID_ARG, "elem_bytes must be 1, 2, 4, 8 or 16 (got %d)", elem_bytes);
  }
  MOYE_CUDA(cudaGetLastError());
  return MOYE_OK;
}

}  // namespace moye
