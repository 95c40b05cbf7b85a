// Host-side plumbing shared by the entry points: the handle, error reporting, dtype
// helpers and tensor-map (TMA descriptor) construction.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <utility>

#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>

#include "../../include/moye_b200.h"

namespace moye {

void set_error(const char* fmt, ...);
const char* get_error();
// MOYE_B200_LOG=1: one line per entry-point call on stderr (shape, types, the kernel and tile chosen);
// MOYE_B200_LOG=2: also every error message as it is set.  Read once per process.
int log_level();
void log_line(const char* fmt, ...);

// Stream-K decode kernel: with slightly fewer 128-row blocks of W than SMs, one whole row-block per CTA on n_tiles
// CTAs (no partial sums to exchange, the other SMs idle) is faster than cutting every row-block over all SMs, as long
// as the idle SMs would not have streamed much: measured on 148 SMs, bf16, M = 1 and 16 (us, whole / cut):
// 14336 x 2048 14.4 / 18.7, 14336 x 4096 23.8 / 25.4-26.5, 16384 x 4096 24.6 / 28.0-29.3, 18432 x 4096 26.3 / 30.3-31.4,
// 14336 x 5120 28.7 / 31.1-32.6, 16384 x 6144 34.3 / 36.9-38.3, 17920 x 8192 46.1 / 49.8-51.0, but 14336 x 8192
// 44.2 / 42.8 and 12288 x 4096 23.4 / 23.1-24.3.
inline bool stream_k_whole_grid(long long n_tiles, long long k_blocks, int num_sms) {
  return n_tiles < num_sms && n_tiles * 2 >= num_sms && (num_sms - n_tiles) * k_blocks <= 3000;
}

// MOYE_B200_NO_PDL=1: launch without the programmatic dependent-launch attribute (to compare with and without).
// Read once per process.
bool launch_without_pdl();

// Launches `kern` with the programmatic dependent-launch attribute (unless MOYE_B200_NO_PDL=1): the grid may set
// itself up while the stream's previous grid finishes.  Only for kernels that execute griddepcontrol.wait before
// their first access to global memory.
template <typename... Params, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = launch_without_pdl() ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}

// NVTX range around an entry point (shows up in Nsight timelines); a no-op costing one branch when no tool is attached.
struct NvtxRange {
  explicit NvtxRange(const char* name);
  ~NvtxRange();
};

#define MOYE_FAIL(code, ...)     \
  do {                           \
    ::moye::set_error(__VA_ARGS__); \
    return (code);               \
  } while (0)

#define MOYE_CUDA(call)                                                                  \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess) {                                                            \
      ::moye::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return MOYE_ERR_CUDA;                                                              \
    }                                                                                    \
  } while (0)

inline int dtype_bytes(int dt) {
  switch (dt) {
    case MOYE_F32: case MOYE_S32: case MOYE_U32: return 4;
    case MOYE_F16: case MOYE_BF16: case MOYE_U16: return 2;
    case MOYE_S8: case MOYE_U8: case MOYE_E4M3: return 1;
    case MOYE_U64: return 8;
    case MOYE_U128: return 16;
    default: return 0;
  }
}

struct TmapKey {
  const void* ptr;
  int dtype;
  uint64_t d0, d1, s1;
  uint32_t b0, b1;
  int swizzle;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && dtype == o.dtype && d0 == o.d0 && d1 == o.d1 && s1 == o.s1 && b0 == o.b0 &&
           b1 == o.b1 && swizzle == o.swizzle;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    auto mix = [&h](uint64_t v) { h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2); };
    mix(k.dtype); mix(k.d0); mix(k.d1); mix(k.s1); mix(k.b0); mix(k.b1); mix(k.swizzle);
    return h;
  }
};

}  // namespace moye

// Orders the launches that share one scratch buffer of a handle when they come on different streams.
struct ScratchOrder {
  cudaEvent_t done = nullptr;       // recorded after the last launch that used the buffer
  cudaStream_t last = nullptr;
  bool used = false;
};

// The handle.  One per (host thread, device).
struct moye_b200_ctx {
  int device = -1;
  int num_sms = 0;
  int smem_optin = 0;
  int* d_status = nullptr;          // device status word (0 = OK, else wait-site code)
  void* workspace = nullptr;        // stream-K scratch of the skinny kernel: tickets, then partial sums
  size_t workspace_bytes = 0;
  void* tail_ws = nullptr;          // stream-K tail of the dense 256 x 512 kernel: tickets, then partial accumulators
  size_t tail_ws_bytes = 0;
  void* split_ws = nullptr;         // lo(A), lo(B) of the Float32 GEMM's three-product split
  size_t split_ws_bytes = 0;
  void* table = nullptr;            // offset tables of the ldmatrix tiled copy
  size_t table_bytes = 0;
  ScratchOrder sk_order, tail_order, split_order, table_order;
  void* comm = nullptr;             // ncclComm_t of this rank (comm_nccl.cu), null until moye_b200_comm_init
  int comm_rank = 0, comm_world = 0;
  std::mutex mu;
  std::unordered_map<moye::TmapKey, CUtensorMap, moye::TmapKeyHash> tmaps;
  std::unordered_set<const void*> configured;   // kernels whose dynamic-smem limit is already raised
  std::unordered_map<uint64_t, int> cluster_fit; // (kernel, cluster size) -> clusters the device can hold at once
};

namespace moye {

// Encodes (or fetches from the handle's cache) a rank-2 tiled tensor map.
//   dims  = {extent along the contiguous mode, extent along the strided mode}  (elements)
//   stride1_bytes = byte stride of the strided mode (multiple of 16)
//   box   = {box extent contiguous, box extent strided}
//   swizzle = 0 none, 1 (or true) the 128-byte swizzle with 16-byte atoms, TMAP_SWIZZLE_128B_ATOM_32B the
//   128-byte swizzle with 32-byte atoms (box[0]*elem must be <= 128 bytes when swizzled)
enum { TMAP_SWIZZLE_NONE = 0, TMAP_SWIZZLE_128B = 1, TMAP_SWIZZLE_128B_ATOM_32B = 2 };
int make_tmap_2d(moye_b200_ctx* h, CUtensorMap* out, const void* ptr, int dtype, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle);

int encode_tmap_2d_uncached(CUtensorMap* out, const void* ptr, int dtype, uint64_t dim0, uint64_t dim1,
                            uint64_t stride1_bytes, uint32_t box0, uint32_t box1, bool swizzle128);

// Raises a kernel's dynamic shared-memory limit the first time this handle launches it.
template <typename K>
inline int configure_once(moye_b200_ctx* h, K kernel, int smem_bytes) {
  const void* key = reinterpret_cast<const void*>(kernel);
  {
    std::lock_guard<std::mutex> lk(h->mu);
    if (h->configured.count(key)) return MOYE_OK;
  }
  MOYE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  std::lock_guard<std::mutex> lk(h->mu);
  h->configured.insert(key);
  return MOYE_OK;
}

// Grows the handle-owned workspace to at least `bytes` (never shrinks).
int ensure_workspace(moye_b200_ctx* h, size_t bytes);
// Ticket areas at the front of both stream-K scratch buffers (zero whenever no kernel is running).
constexpr size_t kSkinnyTicketBytes = 64 * 1024;
constexpr size_t kTailTicketBytes = 64 * 1024;
int ensure_tail_workspace(moye_b200_ctx* h);
// Before a launch that uses a shared scratch buffer: if the previous user ran on another stream, make `stream`
// wait for it.  After the launch: remember it.  Launches on one stream pay an event record and nothing else.
int order_scratch_use(moye_b200_ctx* h, ScratchOrder* o, cudaStream_t stream);
int scratch_used(ScratchOrder* o, cudaStream_t stream);

int launch_gemm(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                const moye_tensor_t* C, const moye_gemm_params_t* p, cudaStream_t stream);
int launch_copy(moye_b200_ctx* h, const moye_tensor_t* dst, const moye_tensor_t* src, const moye_copy_params_t* p,
                cudaStream_t stream);
int launch_transpose(moye_b200_ctx* h, void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int dtype,
                     int64_t m, int64_t n, cudaStream_t stream);
int launch_axpby(moye_b200_ctx* h, const moye_tensor_t* Y, const moye_tensor_t* X, float a, float b, cudaStream_t stream);
int launch_layout_copy(moye_b200_ctx* h, void* dst, const moye_layout_t* dl, const void* src,
                       const moye_layout_t* sl, int elem_bytes, cudaStream_t stream);
int launch_layout_eval(moye_b200_ctx* h, const moye_layout_t* l, int64_t first, int64_t n, int64_t* out,
                       cudaStream_t stream);

}  // namespace moye
