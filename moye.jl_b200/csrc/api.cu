// extern "C" entry points of libmoye_b200 plus the handle, the error string and tensor-map
// construction.  Argument checking lives here and in the per-kernel launchers: a request the
// kernels cannot serve is an error, never a slower fallback.
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "common.h"
#include "ptx.cuh"

namespace moye {

static thread_local char g_err[512] = "";

int log_level() {
  static const int level = [] {
    const char* e = std::getenv("MOYE_B200_LOG");
    return e ? std::atoi(e) : 0;
  }();
  return level;
}

bool launch_without_pdl() {
  static const bool off = [] {
    const char* e = std::getenv("MOYE_B200_NO_PDL");
    return e && e[0] == '1';
  }();
  return off;
}

void log_line(const char* fmt, ...) {
  if (log_level() < 1) return;
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  fprintf(stderr, "[moye_b200] %s\n", buf);
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  if (log_level() >= 2) fprintf(stderr, "[moye_b200] error: %s\n", g_err);
}

NvtxRange::NvtxRange(const char* name) { nvtxRangePushA(name); }
NvtxRange::~NvtxRange() { nvtxRangePop(); }
const char* get_error() { return g_err; }

// cuTensorMapEncodeTiled is fetched through the runtime so the library has no link-time
// dependency on the driver library (it must load on a machine without a GPU).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

static bool tmap_dtype(int dt, CUtensorMapDataType* out) {
  switch (dt) {
    case MOYE_F32: *out = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; return true;
    case MOYE_F16: *out = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; return true;
    case MOYE_BF16: *out = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; return true;
    case MOYE_S8: case MOYE_U8: case MOYE_E4M3: *out = CU_TENSOR_MAP_DATA_TYPE_UINT8; return true;
    case MOYE_S32: *out = CU_TENSOR_MAP_DATA_TYPE_INT32; return true;
    case MOYE_U16: *out = CU_TENSOR_MAP_DATA_TYPE_UINT16; return true;
    case MOYE_U32: *out = CU_TENSOR_MAP_DATA_TYPE_UINT32; return true;
    case MOYE_U64: *out = CU_TENSOR_MAP_DATA_TYPE_UINT64; return true;
    default: return false;
  }
}

int make_tmap_2d(moye_b200_ctx* h, CUtensorMap* out, const void* ptr, int dtype, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, int swizzle) {
  TmapKey key{ptr, dtype, dim0, dim1, stride1_bytes, box0, box1, swizzle};
  {
    std::lock_guard<std::mutex> lk(h->mu);
    auto it = h->tmaps.find(key);
    if (it != h->tmaps.end()) {
      *out = it->second;
      return MOYE_OK;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) MOYE_FAIL(MOYE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType tdt;
  if (!tmap_dtype(dtype, &tdt)) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "dtype %d has no tensor-map type", dtype);
  const int eb = dtype_bytes(dtype);
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "tensor base %p is not 16-byte aligned", ptr);
  if (dim1 > 1 && (stride1_bytes & 15) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "row pitch of %llu bytes is not a multiple of 16",
              (unsigned long long)stride1_bytes);
  if (box0 > 256 || box1 > 256 || ((uint64_t)box0 * eb) % 16 != 0)
    MOYE_FAIL(MOYE_ERR_INVALID_ARG, "bad TMA box %u x %u", box0, box1);
  if (swizzle && (uint64_t)box0 * eb > 128) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "swizzled box wider than 128 bytes");
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {dim1 > 1 ? stride1_bytes : (cuuint64_t)((dim0 * eb + 15) / 16 * 16)};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUtensorMapSwizzle sw = swizzle == TMAP_SWIZZLE_128B_ATOM_32B ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                : (swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
  CUresult r = enc(&m, tdt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    MOYE_FAIL(MOYE_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (dims %llu x %llu, pitch %llu, box %u x %u)",
              (int)r, (unsigned long long)dim0, (unsigned long long)dim1, (unsigned long long)stride1_bytes, box0,
              box1);
  {
    std::lock_guard<std::mutex> lk(h->mu);
    if (h->tmaps.size() > 4096) h->tmaps.clear();
    h->tmaps.emplace(key, m);
  }
  *out = m;
  return MOYE_OK;
}

// Encodes a rank-2 tiled tensor map straight into `out`: no handle, no cache, no heap.
int encode_tmap_2d_uncached(CUtensorMap* out, const void* ptr, int dtype, uint64_t dim0, uint64_t dim1,
                            uint64_t stride1_bytes, uint32_t box0, uint32_t box1, bool swizzle128) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) MOYE_FAIL(MOYE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMapDataType tdt;
  if (!tmap_dtype(dtype, &tdt)) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "dtype %d has no tensor-map type", dtype);
  const int eb = dtype_bytes(dtype);
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "tensor base %p is not 16-byte aligned", ptr);
  if (dim1 > 1 && (stride1_bytes & 15) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "row pitch of %llu bytes is not a multiple of 16",
              (unsigned long long)stride1_bytes);
  cuuint64_t dims[2] = {dim0, dim1};
  cuuint64_t strides[1] = {dim1 > 1 ? stride1_bytes : (cuuint64_t)((dim0 * eb + 15) / 16 * 16)};
  cuuint32_t box[2] = {box0, box1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, tdt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) MOYE_FAIL(MOYE_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  return MOYE_OK;
}

// The skinny kernel's scratch is allocated once, at the size its widest instantiation needs, so that no launch
// ever has to synchronise the device to free and re-allocate it.
int ensure_workspace(moye_b200_ctx* h, size_t bytes) {
  if (h->workspace) {
    if (bytes <= h->workspace_bytes) return MOYE_OK;
    MOYE_FAIL(MOYE_ERR_TOO_LARGE, "the stream-K scratch holds %zu bytes, %zu were asked for", h->workspace_bytes, bytes);
  }
  size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
  void* p = nullptr;
  MOYE_CUDA(cudaMalloc(&p, want));
  cudaError_t e = cudaMemset(p, 0, kSkinnyTicketBytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    MOYE_FAIL(MOYE_ERR_CUDA, "clearing the stream-K tickets failed: %s", cudaGetErrorString(e));
  }
  h->workspace_bytes = want;
  h->workspace = p;
  return MOYE_OK;
}

int order_scratch_use(moye_b200_ctx* h, ScratchOrder* o, cudaStream_t stream) {
  (void)h;
  if (!o->done) MOYE_CUDA(cudaEventCreateWithFlags(&o->done, cudaEventDisableTiming));
  if (o->used && o->last != stream) MOYE_CUDA(cudaStreamWaitEvent(stream, o->done, 0));
  return MOYE_OK;
}

int scratch_used(ScratchOrder* o, cudaStream_t stream) {
  MOYE_CUDA(cudaEventRecord(o->done, stream));
  o->last = stream;
  o->used = true;
  return MOYE_OK;
}

static int check_handle(moye_b200_ctx* h) {
  if (!h) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null handle");
  int dev = -1;
  MOYE_CUDA(cudaGetDevice(&dev));
  if (dev != h->device)
    MOYE_FAIL(MOYE_ERR_INVALID_ARG, "handle belongs to device %d but device %d is current", h->device, dev);
  return MOYE_OK;
}

}  // namespace moye

using namespace moye;

namespace moye {
// One warp waits, with the same bounded wait every kernel of the library uses, on an mbarrier that nothing ever
// arrives at.  The wait gives up after its poll limit, records the site code and the kernel returns normally.
__global__ void bounded_wait_probe_kernel(int* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, status, 901);
}
}  // namespace moye

extern "C" {

int moye_b200_version(void) { return MOYE_B200_VERSION; }

const char* moye_b200_last_error(void) { return get_error(); }

int moye_b200_create(moye_handle_t* out) {
  if (!out) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null output pointer");
  *out = nullptr;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    MOYE_FAIL(MOYE_ERR_NO_DEVICE, "no CUDA device is visible; libmoye_b200 has no CPU path");
  }
  int dev = 0;
  MOYE_CUDA(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  MOYE_CUDA(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10)
    MOYE_FAIL(MOYE_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major,
              prop.minor);
  moye_b200_ctx* h = new moye_b200_ctx();
  h->device = dev;
  h->num_sms = prop.multiProcessorCount;
  h->smem_optin = (int)prop.sharedMemPerBlockOptin;
  cudaError_t e = cudaMalloc(&h->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    set_error("allocating the status word failed: %s", cudaGetErrorString(e));
    delete h;
    return MOYE_ERR_CUDA;
  }
  *out = h;
  return MOYE_OK;
}

int moye_b200_destroy(moye_handle_t h) {
  if (!h) return MOYE_OK;
  cudaSetDevice(h->device);
  cudaDeviceSynchronize();
  if (h->d_status) cudaFree(h->d_status);
  if (h->workspace) cudaFree(h->workspace);
  if (h->tail_ws) cudaFree(h->tail_ws);
  if (h->split_ws) cudaFree(h->split_ws);
  if (h->table) cudaFree(h->table);
  if (h->table_order.done) cudaEventDestroy(h->table_order.done);
  if (h->split_order.done) cudaEventDestroy(h->split_order.done);
  if (h->sk_order.done) cudaEventDestroy(h->sk_order.done);
  if (h->tail_order.done) cudaEventDestroy(h->tail_order.done);
  delete h;
  return MOYE_OK;
}

int moye_b200_status(moye_handle_t h, void* stream, int32_t* site) {
  if (int rc = check_handle(h)) return rc;
  MOYE_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int v = 0;
  MOYE_CUDA(cudaMemcpy(&v, h->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (site) *site = v;
  if (v != 0) {
    // A kernel that gave up may have left stream-K tickets half counted: whoever would have restored them never
    // arrived.  Nothing of this handle is running any more on `stream`; wait for its other streams too, then put
    // both ticket areas back to zero so that the next product starts clean.
    MOYE_CUDA(cudaDeviceSynchronize());
    MOYE_CUDA(cudaMemset(h->d_status, 0, sizeof(int)));
    if (h->workspace) MOYE_CUDA(cudaMemset(h->workspace, 0, kSkinnyTicketBytes));
    if (h->tail_ws) MOYE_CUDA(cudaMemset(h->tail_ws, 0, kTailTicketBytes));
    MOYE_FAIL(MOYE_ERR_TIMEOUT, "a bounded device-side wait ran out (site code %d)", v);
  }
  return MOYE_OK;
}

int moye_b200_selftest_bounded_wait(moye_handle_t h, void* stream) {
  if (int rc = check_handle(h)) return rc;
  moye::bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(h->d_status);
  MOYE_CUDA(cudaGetLastError());
  return MOYE_OK;
}

int moye_b200_selftest_dirty_tickets(moye_handle_t h, void* stream) {
  if (int rc = check_handle(h)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (h->workspace) MOYE_CUDA(cudaMemsetAsync(h->workspace, 0x01, kSkinnyTicketBytes, s));
  if (h->tail_ws) MOYE_CUDA(cudaMemsetAsync(h->tail_ws, 0x01, kTailTicketBytes, s));
  return MOYE_OK;
}

int moye_b200_gemm(moye_handle_t h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                   const moye_tensor_t* C, const moye_gemm_params_t* params, void* stream) {
  NvtxRange range("moye_b200_gemm");
  if (int rc = check_handle(h)) return rc;
  if (!D || !A || !B) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "D, A and B must be non-null");
  return launch_gemm(h, D, A, B, C, params, static_cast<cudaStream_t>(stream));
}

int moye_b200_copy(moye_handle_t h, const moye_tensor_t* dst, const moye_tensor_t* src,
                   const moye_copy_params_t* params, void* stream) {
  NvtxRange range("moye_b200_copy");
  if (int rc = check_handle(h)) return rc;
  if (!dst || !src) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "dst and src must be non-null");
  return launch_copy(h, dst, src, params, static_cast<cudaStream_t>(stream));
}

int moye_b200_axpby(moye_handle_t h, const moye_tensor_t* Y, const moye_tensor_t* X, float a, float b, void* stream) {
  NvtxRange range("moye_b200_axpby");
  if (int rc = check_handle(h)) return rc;
  if (!Y || !X) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "Y and X must be non-null");
  return launch_axpby(h, Y, X, a, b, static_cast<cudaStream_t>(stream));
}

int moye_b200_layout_copy(moye_handle_t h, void* dst, const moye_layout_t* dl, const void* src,
                          const moye_layout_t* sl, int32_t elem_bytes, void* stream) {
  NvtxRange range("moye_b200_layout_copy");
  if (int rc = check_handle(h)) return rc;
  if (!dst || !src || !dl || !sl) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null argument");
  return launch_layout_copy(h, dst, dl, src, sl, elem_bytes, static_cast<cudaStream_t>(stream));
}

int moye_b200_layout_eval(moye_handle_t h, const moye_layout_t* l, int64_t first, int64_t n, int64_t* out,
                          void* stream) {
  NvtxRange range("moye_b200_layout_eval");
  if (int rc = check_handle(h)) return rc;
  if (!l || (!out && n > 0)) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null argument");
  return launch_layout_eval(h, l, first, n, out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
