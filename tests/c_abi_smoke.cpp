// A C++ caller of the C ABI, with nothing but the header, the CUDA runtime and the shared library: what a
// non-Python, non-Julia user of libmoye_b200 writes.  Built and run by tests/test_abi.py (without a device it must
// report MOYE_ERR_NO_DEVICE and exit 3) and tests/test_gpu_gemm.py (on a B200 it must print C_ABI_SMOKE_OK).
//
// The product mirrors the reference's `matmul(A, B, C)` (examples/gemm.jl:66-89, checked there with C == A * B'):
// fp16 operands holding small integers, so every dot product is exact in fp32 and the comparison is `==`.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "moye_b200.h"

#define CHECK_CUDA(x)                                                       \
  do {                                                                      \
    cudaError_t e_ = (x);                                                   \
    if (e_ != cudaSuccess) {                                                \
      std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));         \
      return 2;                                                             \
    }                                                                       \
  } while (0)
#define CHECK_MOYE(x)                                                       \
  do {                                                                      \
    int rc_ = (x);                                                          \
    if (rc_ != MOYE_OK) {                                                   \
      std::fprintf(stderr, "%s -> %d: %s\n", #x, rc_, moye_b200_last_error()); \
      return 2;                                                             \
    }                                                                       \
  } while (0)

static moye_tensor_t matrix(void* p, moye_dtype_t dt, long long rows, long long cols, long long s0, long long s1) {
  moye_tensor_t t = {};
  t.ptr = p;
  t.dtype = dt;
  t.rank = 2;
  t.shape[0] = rows;
  t.shape[1] = cols;
  t.stride[0] = s0;
  t.stride[1] = s1;
  return t;
}

int main() {
  if (moye_b200_version() != MOYE_B200_VERSION) {
    std::fprintf(stderr, "header and library versions differ\n");
    return 2;
  }
  moye_handle_t h = nullptr;
  int rc = moye_b200_create(&h);
  if (rc == MOYE_ERR_NO_DEVICE) {
    std::printf("no device: %s\n", moye_b200_last_error());
    return 3;
  }
  if (rc != MOYE_OK) {
    std::fprintf(stderr, "moye_b200_create -> %d: %s\n", rc, moye_b200_last_error());
    return 2;
  }
  const int M = 384, N = 520, K = 1000, LDK = 1008;  // ragged edges; row pitch a multiple of 16 bytes
  std::vector<__half> a((size_t)M * LDK, __float2half(0.f)), b((size_t)N * LDK, __float2half(0.f));
  for (int m = 0; m < M; ++m)
    for (int k = 0; k < K; ++k) a[(size_t)m * LDK + k] = __float2half((float)((m + 2 * k) % 7 - 3));
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) b[(size_t)n * LDK + k] = __float2half((float)((3 * n + k) % 5 - 2));
  __half *dA = nullptr, *dB = nullptr;
  float *dC = nullptr, *dT = nullptr;
  CHECK_CUDA(cudaMalloc(&dA, a.size() * sizeof(__half)));
  CHECK_CUDA(cudaMalloc(&dB, b.size() * sizeof(__half)));
  CHECK_CUDA(cudaMalloc(&dC, (size_t)M * N * sizeof(float)));
  CHECK_CUDA(cudaMalloc(&dT, (size_t)M * N * sizeof(float)));
  CHECK_CUDA(cudaMemcpy(dA, a.data(), a.size() * sizeof(__half), cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dB, b.data(), b.size() * sizeof(__half), cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemset(dC, 0xFF, (size_t)M * N * sizeof(float)));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));

  // D (M, N) row-major = A (M, K) . B (N, K)^T, then the same result transposed with the copy entry point
  const moye_tensor_t A = matrix(dA, MOYE_F16, M, K, LDK, 1), B = matrix(dB, MOYE_F16, N, K, LDK, 1);
  const moye_tensor_t D = matrix(dC, MOYE_F32, M, N, N, 1);
  CHECK_MOYE(moye_b200_gemm(h, &D, &A, &B, nullptr, nullptr, stream));
  const moye_tensor_t Tdst = matrix(dT, MOYE_F32, M, N, 1, M);  // column-major view of a second buffer
  CHECK_MOYE(moye_b200_copy(h, &Tdst, &D, nullptr, stream));
  int32_t site = 0;
  CHECK_MOYE(moye_b200_status(h, stream, &site));  // synchronises the stream and reads the device-side status

  std::vector<float> c((size_t)M * N), t((size_t)M * N);
  CHECK_CUDA(cudaMemcpy(c.data(), dC, c.size() * sizeof(float), cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(t.data(), dT, t.size() * sizeof(float), cudaMemcpyDeviceToHost));
  long long bad = 0;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += (float)((m + 2 * k) % 7 - 3) * (float)((3 * n + k) % 5 - 2);
      if (c[(size_t)m * N + n] != acc || t[(size_t)n * M + m] != acc) ++bad;
    }
  // an argument the kernels cannot serve is an error with a message, never a slower path
  const moye_tensor_t odd = matrix(dA, MOYE_F16, M, K, LDK + 1, 1);
  const int refused = moye_b200_gemm(h, &D, &odd, &B, nullptr, nullptr, stream);
  CHECK_MOYE(moye_b200_destroy(h));
  cudaFree(dA);
  cudaFree(dB);
  cudaFree(dC);
  cudaFree(dT);
  if (bad != 0 || refused != MOYE_ERR_MISALIGNED) {
    std::fprintf(stderr, "%lld wrong elements, misaligned operand -> %d\n", bad, refused);
    return 1;
  }
  std::printf("C_ABI_SMOKE_OK\n");
  return 0;
}
