// Y = a*X + b*Y over two arrays of equal layout: MoYe's `axpby!` (reference src/algorithm/blas.jl:1-9) as a
// stand-alone device operation.  The reference walks the two engines in memory order, one element per iteration,
// and skips the read of Y when b == 0; so does this kernel, 16 bytes per thread and access.
//
// Arithmetic follows the host path literally: the two products are rounded separately and then added (Julia does
// not contract `a*x + b*y` into a fused multiply-add), in fp32 for f32 / f16 / bf16 elements, with one rounding to
// the element type on the store.  HBM-bound: 2 (b == 0) or 3 accesses of `elem` bytes per element.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "ptx.cuh"

namespace moye {

template <typename T>
__device__ __forceinline__ float elem_to_float(T v);
template <>
__device__ __forceinline__ float elem_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float elem_to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float elem_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T float_to_elem(float f);
template <>
__device__ __forceinline__ float float_to_elem<float>(float f) { return f; }
template <>
__device__ __forceinline__ __half float_to_elem<__half>(float f) { return __float2half_rn(f); }
template <>
__device__ __forceinline__ __nv_bfloat16 float_to_elem<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }

template <typename T>
__device__ __forceinline__ T axpby_one(float a, T x, float b, T y, bool read_y) {
  const float ax = __fmul_rn(a, elem_to_float<T>(x));
  return float_to_elem<T>(read_y ? __fadd_rn(ax, __fmul_rn(b, elem_to_float<T>(y))) : ax);
}

// rows x cols elements, `cols` contiguous, rows `pitch` elements apart (the same pitch in X and Y is not required).
// VEC elements (16 bytes) per access when both rows allow it, else element by element.
template <typename T, bool VECTOR>
__global__ void __launch_bounds__(256)
axpby_kernel(T* y, const T* x, long long rows, long long cols, long long pitch_y,
             long long pitch_x, float a, float b) {
  constexpr int VEC = 16 / (int)sizeof(T);
  griddep_launch();  // programmatic dependent launch: see launch_dependent()
  griddep_wait();
  const bool read_y = b != 0.f;
  const long long per_row = VECTOR ? cols / VEC : cols;
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row, c = i - r * per_row;
    if constexpr (VECTOR) {
      const uint4 xv = __ldcs(reinterpret_cast<const uint4*>(x + r * pitch_x) + c);
      uint4* yp = reinterpret_cast<uint4*>(y + r * pitch_y) + c;
      uint4 yv = make_uint4(0u, 0u, 0u, 0u);
      if (read_y) yv = *yp;
      T xe[VEC], ye[VEC];
      *reinterpret_cast<uint4*>(xe) = xv;
      *reinterpret_cast<uint4*>(ye) = yv;
#pragma unroll
      for (int e = 0; e < VEC; ++e) ye[e] = axpby_one<T>(a, xe[e], b, ye[e], read_y);
      *yp = *reinterpret_cast<uint4*>(ye);
    } else {
      T* yp = y + r * pitch_y + c;
      *yp = axpby_one<T>(a, x[r * pitch_x + c], b, read_y ? *yp : float_to_elem<T>(0.f), read_y);
    }
  }
}

template <typename T>
static int launch_axpby_t(moye_b200_ctx* h, void* y, const void* x, long long rows, long long cols, long long pitch_y,
                          long long pitch_x, float a, float b, cudaStream_t stream) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec = cols % VEC == 0 && pitch_y % VEC == 0 && pitch_x % VEC == 0 &&
                   (reinterpret_cast<uintptr_t>(y) & 15) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const long long items = rows * (vec ? cols / VEC : cols);
  long long blocks = (items + 255) / 256;
  const long long cap = (long long)h->num_sms * 8;  // grid-stride beyond 8 CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const dim3 g((unsigned)blocks), blk(256);
  if (vec)
    MOYE_CUDA(launch_dependent(axpby_kernel<T, true>, g, blk, 0, stream, static_cast<T*>(y), static_cast<const T*>(x), rows, cols,
                               pitch_y, pitch_x, a, b));
  else
    MOYE_CUDA(launch_dependent(axpby_kernel<T, false>, g, blk, 0, stream, static_cast<T*>(y), static_cast<const T*>(x), rows, cols,
                               pitch_y, pitch_x, a, b));
  return MOYE_OK;
}

int launch_axpby(moye_b200_ctx* h, const moye_tensor_t* Y, const moye_tensor_t* X, float a, float b, cudaStream_t stream) {
  if (X->dtype != Y->dtype) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "axpby!: X and Y must have the same element type");
  if (X->rank != Y->rank || X->rank < 1 || X->rank > 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "axpby!: rank 1 or 2, equal in X and Y");
  long long shape[2] = {X->shape[0], X->rank == 2 ? X->shape[1] : 1};
  long long sx[2] = {X->stride[0], X->rank == 2 ? X->stride[1] : shape[0]};
  long long sy[2] = {Y->stride[0], Y->rank == 2 ? Y->stride[1] : shape[0]};
  for (int i = 0; i < X->rank; ++i)
    if (X->shape[i] != Y->shape[i]) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "axpby!: shapes differ");
  if (shape[0] <= 0 || shape[1] <= 0) return MOYE_OK;  // nothing to do, as the reference's empty loop
  if (!X->ptr || !Y->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null data pointer");
  // both arrays contiguous along the same mode; the other mode may be pitched
  long long rows, cols, py, px;
  if ((sx[0] == 1 || shape[0] == 1) && (sy[0] == 1 || shape[0] == 1)) {
    cols = shape[0]; rows = shape[1]; px = sx[1]; py = sy[1];
  } else if ((sx[1] == 1 || shape[1] == 1) && (sy[1] == 1 || shape[1] == 1)) {
    cols = shape[1]; rows = shape[0]; px = sx[0]; py = sy[0];
  } else {
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "axpby!: X and Y must be contiguous along the same mode");
  }
  if (rows > 1 && (px < cols || py < cols)) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "axpby!: rows overlap");
  switch (X->dtype) {
    case MOYE_F32: return launch_axpby_t<float>(h, Y->ptr, X->ptr, rows, cols, py, px, a, b, stream);
    case MOYE_F16: return launch_axpby_t<__half>(h, Y->ptr, X->ptr, rows, cols, py, px, a, b, stream);
    case MOYE_BF16: return launch_axpby_t<__nv_bfloat16>(h, Y->ptr, X->ptr, rows, cols, py, px, a, b, stream);
    default: MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "axpby!: element type %d is not supported (f32, f16, bf16)", X->dtype);
  }
}

}  // namespace moye
