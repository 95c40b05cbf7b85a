// Reassembling sharded results over NVLink: all-gather of the row / column blocks of a matrix, and broadcast of a
// replicated operand, on NCCL.  The reference has no multi-GPU code; these entry points exist because the GEMM and
// the copy shard along M (or N for weight-bound shapes) over the GPUs of one box, one process per GPU, and a
// caller that wants the whole of C on every rank needs the gather behind the same C ABI as the kernels.
//
// NCCL is looked up at run time (`libnccl.so.2`, already in the process when the caller is a PyTorch program), so
// the library loads, and everything else in it works, on a machine without NCCL.  No kernel of this library is ever
// handed another GPU's memory: the only code that touches a peer is NCCL's own.
#include <dlfcn.h>

#include <cstring>

#include "common.h"

namespace moye {

typedef struct ncclComm* nccl_comm_t;
struct nccl_unique_id { char internal[128]; };
enum { kNcclInt8 = 0 };

struct NcclApi {
  int (*GetUniqueId)(nccl_unique_id*) = nullptr;
  int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
  int (*CommDestroy)(nccl_comm_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};

static NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return;
    auto sym = [&](const char* n) { return dlsym(lib, n); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.Broadcast = reinterpret_cast<decltype(api.Broadcast)>(sym("ncclBroadcast"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.Broadcast &&
             api.GroupStart && api.GroupEnd && api.GetErrorString;
  });
  return &api;
}

#define MOYE_NCCL(api, call)                                                                         \
  do {                                                                                               \
    int r__ = (call);                                                                                \
    if (r__ != 0) {                                                                                  \
      ::moye::set_error("%s failed: %s", #call, (api)->GetErrorString ? (api)->GetErrorString(r__) : "?"); \
      return MOYE_ERR_NCCL;                                                                          \
    }                                                                                                \
  } while (0)

static int need_api(NcclApi** out) {
  NcclApi* a = nccl_api();
  if (!a->ok) MOYE_FAIL(MOYE_ERR_NCCL, "libnccl.so.2 could not be loaded (or lacks a needed symbol)");
  *out = a;
  return MOYE_OK;
}

// [begin, end) of rank r's block of `extent` items cut into `world` blocks that are multiples of `align`
// (the last block takes the ragged remainder).  The same arithmetic as `shard_range` of the host package.
void comm_shard_range(int64_t extent, int world, int rank, int64_t align, int64_t* lo, int64_t* hi) {
  const int64_t units = (extent + align - 1) / align;
  int64_t b = (units * rank / world) * align, e = (units * (rank + 1) / world) * align;
  *lo = b < extent ? b : extent;
  *hi = e < extent ? e : extent;
}

}  // namespace moye

using namespace moye;

extern "C" {

int moye_b200_comm_unique_id(char* id128) {
  if (!id128) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null id buffer");
  NcclApi* a;
  if (int rc = need_api(&a)) return rc;
  nccl_unique_id id;
  MOYE_NCCL(a, a->GetUniqueId(&id));
  std::memcpy(id128, id.internal, sizeof(id.internal));
  return MOYE_OK;
}

int moye_b200_comm_init(moye_handle_t h, int32_t rank, int32_t world, const char* id128) {
  if (!h || !id128) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null handle or id");
  if (world < 1 || rank < 0 || rank >= world) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "bad rank %d of %d", rank, world);
  if (h->comm) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "this handle already has a communicator");
  int dev = -1;
  MOYE_CUDA(cudaGetDevice(&dev));
  if (dev != h->device) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "handle belongs to device %d but device %d is current", h->device, dev);
  NcclApi* a;
  if (int rc = need_api(&a)) return rc;
  nccl_unique_id id;
  std::memcpy(id.internal, id128, sizeof(id.internal));
  nccl_comm_t c = nullptr;
  MOYE_NCCL(a, a->CommInitRank(&c, world, id, rank));
  h->comm = c;
  h->comm_rank = rank;
  h->comm_world = world;
  return MOYE_OK;
}

int moye_b200_comm_destroy(moye_handle_t h) {
  if (!h) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null handle");
  if (!h->comm) return MOYE_OK;
  NcclApi* a;
  if (int rc = need_api(&a)) return rc;
  MOYE_NCCL(a, a->CommDestroy(static_cast<nccl_comm_t>(h->comm)));
  h->comm = nullptr;
  h->comm_world = 0;
  return MOYE_OK;
}

int moye_b200_allgather(moye_handle_t h, const moye_tensor_t* shard, const moye_tensor_t* full, int32_t mode,
                        int64_t align, void* stream_) {
  if (!h || !shard || !full) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null argument");
  if (!h->comm) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "no communicator: call moye_b200_comm_init first");
  if (shard->rank != 2 || full->rank != 2 || (mode != 0 && mode != 1))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "all-gather takes rank-2 tensors split along mode 0 or 1");
  if (shard->dtype != full->dtype) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "shard and full differ in element type");
  if (align < 1) align = 1;
  const int world = h->comm_world, rank = h->comm_rank;
  const int other = 1 - mode;
  int64_t lo, hi;
  comm_shard_range(full->shape[mode], world, rank, align, &lo, &hi);
  if (shard->shape[mode] != hi - lo || shard->shape[other] != full->shape[other])
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "rank %d owns [%lld, %lld) of mode %d, but the shard is %lld x %lld", rank,
              (long long)lo, (long long)hi, mode, (long long)shard->shape[0], (long long)shard->shape[1]);
  // a block must be one contiguous byte range: the split mode is the outer one in memory, in both tensors
  const int64_t inner = full->shape[other];
  auto compact = [&](const moye_tensor_t* t) {
    return (t->stride[other] == 1 || inner == 1) && (t->stride[mode] == inner || t->shape[mode] == 1);
  };
  if (!compact(full) || !compact(shard))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT,
              "the blocks of mode %d are not contiguous in memory (strides full (%lld,%lld), shard (%lld,%lld)): split the "
              "mode that is outermost in memory (rows of a row-major matrix, columns of a column-major one)",
              mode, (long long)full->stride[0], (long long)full->stride[1], (long long)shard->stride[0],
              (long long)shard->stride[1]);
  const size_t eb = (size_t)dtype_bytes(full->dtype);
  if (eb == 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "unknown element type %d", full->dtype);
  NcclApi* a;
  if (int rc = need_api(&a)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  nccl_comm_t comm = static_cast<nccl_comm_t>(h->comm);
  bool equal = true;
  for (int r = 0; r < world; ++r) {
    int64_t l, e;
    comm_shard_range(full->shape[mode], world, r, align, &l, &e);
    if (e - l != hi - lo) equal = false;
  }
  uint8_t* base = static_cast<uint8_t*>(full->ptr);
  if (equal) {
    MOYE_NCCL(a, a->AllGather(shard->ptr, base, (size_t)(hi - lo) * inner * eb, kNcclInt8, comm, stream));
  } else {
    // ragged blocks: one broadcast per owner, fused into one NCCL group
    MOYE_NCCL(a, a->GroupStart());
    for (int r = 0; r < world; ++r) {
      int64_t l, e;
      comm_shard_range(full->shape[mode], world, r, align, &l, &e);
      void* dst = base + (size_t)l * inner * eb;
      const void* src = r == rank ? shard->ptr : dst;
      if (e > l) {
        int rc = a->Broadcast(src, dst, (size_t)(e - l) * inner * eb, kNcclInt8, r, comm, stream);
        if (rc != 0) {
          a->GroupEnd();
          set_error("ncclBroadcast failed: %s", a->GetErrorString(rc));
          return MOYE_ERR_NCCL;
        }
      }
    }
    MOYE_NCCL(a, a->GroupEnd());
  }
  return MOYE_OK;
}

int moye_b200_bcast(moye_handle_t h, const moye_tensor_t* t, int32_t root, void* stream_) {
  if (!h || !t) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null argument");
  if (!h->comm) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "no communicator: call moye_b200_comm_init first");
  if (root < 0 || root >= h->comm_world) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "bad root %d", root);
  if (t->rank < 1 || t->rank > 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "broadcast takes rank-1 or rank-2 tensors");
  // compact in memory, either mode outermost
  const int64_t s0 = t->shape[0], s1 = t->rank == 2 ? t->shape[1] : 1;
  const int64_t d0 = t->stride[0], d1 = t->rank == 2 ? t->stride[1] : s0;
  const bool ok = ((d0 == 1 || s0 == 1) && (d1 == s0 || s1 == 1)) || ((d1 == 1 || s1 == 1) && (d0 == s1 || s0 == 1));
  if (!ok) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "broadcast needs a tensor that is compact in memory");
  const size_t eb = (size_t)dtype_bytes(t->dtype);
  if (eb == 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "unknown element type %d", t->dtype);
  NcclApi* a;
  if (int rc = need_api(&a)) return rc;
  MOYE_NCCL(a, a->Broadcast(t->ptr, t->ptr, (size_t)s0 * s1 * eb, kNcclInt8, root, static_cast<nccl_comm_t>(h->comm),
                            static_cast<cudaStream_t>(stream_)));
  return MOYE_OK;
}

}  // extern "C"
