/*
 * moye_b200.h -- C ABI of libmoye_b200: the Blackwell (sm_100a) implementation of the tiled
 * GEMM / TiledCopy hot path of MoYe.jl.
 *
 * MoYe.jl itself has no FFI: its `gemm!` / `copyto!` are per-thread device functions that
 * CUDA.jl compiles into a user kernel (reference examples/gemm.jl:4-64, launched at :86).
 * The entry points below are what host-level `gemm!(tiled_mma, D, A, B, C)` and
 * `copyto!(tiled_copy, dst, src)` methods on global-memory MoYeArrays bind to with `ccall`;
 * every declaration names the reference interface whose work it takes over.
 *
 * Conventions
 *   - All pointers inside a moye_tensor_t are DEVICE pointers owned by the caller, except
 *     where an entry point says "host".  The library never frees caller memory.
 *   - Shapes and strides are in ELEMENTS, 0-based arithmetic (offset = sum coord[i]*stride[i]),
 *     i.e. MoYe's `layout(coord) - 1`.
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*), like the
 *     `@cuda` launch it replaces.  Return value: 0 on success, a negative moye_status_t
 *     otherwise; `moye_b200_last_error()` gives a thread-local message.  Nothing aborts,
 *     traps or throws across this boundary, and there is no CPU fallback.
 *   - One handle per (host thread, device).  A handle may be used with several streams: the kernels that keep
 *     scratch in the handle (the stream-K decode GEMM, the K-split tail of the dense kernel and the split-K cluster
 *     kernel, the Float32 split, the ldmatrix copy) are ordered by the library with an event whenever two of them that share a scratch
 *     buffer come on different streams; everything else runs concurrently.  Scratch buffers are allocated once,
 *     on first use, at their final size; only the Float32 split buffer grows with the operands.
 *   - Environment: MOYE_B200_LOG=1 prints one line per product / copy on stderr with the kernel the dispatch
 *     chose; =2 also prints every error message as it is set.  Launching entry points open an NVTX range.
 *     MOYE_B200_NO_PDL=1 launches every kernel without the programmatic dependent-launch attribute (to compare
 *     with and without).
 */
#ifndef MOYE_B200_H
#define MOYE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOYE_B200_VERSION 100
#define MOYE_MAX_RANK 4
#define MOYE_MAX_FLAT_RANK 12

typedef struct moye_b200_ctx* moye_handle_t;

typedef enum {
  MOYE_OK = 0,
  MOYE_ERR_INVALID_ARG = -1,
  MOYE_ERR_UNSUPPORTED_DTYPE = -2,
  MOYE_ERR_UNSUPPORTED_LAYOUT = -3,
  MOYE_ERR_UNSUPPORTED_SHAPE = -4,
  MOYE_ERR_MISALIGNED = -5,
  MOYE_ERR_CUDA = -6,
  MOYE_ERR_TIMEOUT = -7,   /* a bounded device-side wait ran out (see moye_b200_status) */
  MOYE_ERR_NO_DEVICE = -8,
  MOYE_ERR_TOO_LARGE = -9,
  MOYE_ERR_NCCL = -10      /* NCCL is missing or one of its calls failed (multi-GPU entry points only) */
} moye_status_t;

/* Element types.  MoYe spells them Float32, Float16, BFloat16, Int8, UInt8, Int32; e4m3 is
 * new (the reference has no fp8 type). */
typedef enum {
  MOYE_F32 = 0,
  MOYE_F16 = 1,
  MOYE_BF16 = 2,
  MOYE_S8 = 3,
  MOYE_U8 = 4,
  MOYE_E4M3 = 5,
  MOYE_S32 = 6,
  MOYE_U16 = 7,
  MOYE_U32 = 8,
  MOYE_U64 = 9,
  MOYE_U128 = 10
} moye_dtype_t;

/* A MoYeArray over global memory, flattened: engine pointer + layout (reference
 * src/array.jl:53-59 `MoYeArray{T,N,E,L}`, src/engine.jl:6-48 `ViewEngine`). */
typedef struct {
  void* ptr;
  int32_t dtype;                 /* moye_dtype_t */
  int32_t rank;                  /* 1..MOYE_MAX_RANK */
  int64_t shape[MOYE_MAX_RANK];
  int64_t stride[MOYE_MAX_RANK]; /* elements */
} moye_tensor_t;

/* A flattened Layout (reference src/layout.jl:1-60): `rank` leaf modes in colexicographic
 * order, as produced by `flatten(layout)`. */
typedef struct {
  int32_t rank;                  /* 1..MOYE_MAX_FLAT_RANK */
  int32_t reserved;
  int64_t shape[MOYE_MAX_FLAT_RANK];
  int64_t stride[MOYE_MAX_FLAT_RANK];
} moye_layout_t;

/* Fused epilogue, selected in moye_gemm_params_t.flags: one activation OR-ed with one bias mode.
 * D = act(alpha*scale_a*scale_b*(A.B^T) + beta*C + bias), evaluated in fp32 before the output
 * conversion.  The reference has no counterpart beyond `axpby!` (its README lists epilogue fusion
 * as missing); the s8 -> s32 path takes neither. */
enum {
  MOYE_EPI_NONE = 0,
  MOYE_EPI_RELU = 1,             /* max(x, 0) */
  MOYE_EPI_GELU = 2,             /* x/2 * (1 + erf(x / sqrt 2)) */
  MOYE_EPI_SILU = 3,             /* x / (1 + exp(-x)) */
  MOYE_EPI_ACT_MASK = 0xF,
  MOYE_EPI_BIAS_COL = 0x10,      /* bias[n], N floats: one value per column of D */
  MOYE_EPI_BIAS_ROW = 0x20,      /* bias[m], M floats: one value per row of D */
  MOYE_EPI_BIAS_MASK = 0x30,
  /* Stream-K tail of the dense kernel on 256 x 512 tiles (path 0 or 4): when the last wave of tiles would leave
   * CTA pairs idle, its tiles are cut along K into one run per pair and the pieces are added in K order (the
   * result does not depend on timing; s8 stays exact).  The library decides from the shape; these bits overrule it. */
  MOYE_GEMM_TAIL_OFF = 0x100,
  MOYE_GEMM_TAIL_ON = 0x200,
  /* Float32 operands.  Without this bit they are multiplied to Float32 accuracy (three tf32 tensor-core products of
   * the operands' high and low parts, see moye_b200_gemm).  With it the caller accepts ONE tf32 product: operands are
   * read with a 10-bit mantissa (the low 13 bits dropped), about 1e-3 relative, at three times the speed. */
  MOYE_GEMM_ALLOW_TF32 = 0x400
};

/* Parameters of the tiled GEMM.  alpha/beta follow `axpby!` (reference
 * src/algorithm/blas.jl:1-9): D = alpha*scale_a*scale_b*(A.B^T) + beta*C, and C is not read
 * when beta == 0.  Zero in a tiling field means "library default". */
typedef struct {
  float alpha;
  float beta;
  float scale_a;                 /* per-tensor dequantisation scales (fp8 path); 1 otherwise */
  float scale_b;
  int32_t tile_n;                /* CTA tile N: 0 (auto), 64, 128 or 256; tile M is 128.  Widened to 128 (256 on
                                    CTA pairs) when B is MN-major with 8-bit elements */
  int32_t split_k;               /* path 5: CTAs per output tile (2, 4 or 8; 0 = auto); ignored elsewhere */
  int32_t path;                  /* 0 auto, 1 dense kernel (single CTAs), 2 skinny stream-K kernel (M <= 128),
                                    3 dense kernel on CTA pairs (cta_group::2), 256 x tile_n tiles,
                                    4 CTA pairs on 256 x 512 tiles,
                                    5 split-K on thread-block clusters: 128 x tile_n tiles, the `split_k` CTAs of a tile
                                    sum their parts through the handle's scratch (for outputs with few tiles; at most
                                    591 CTAs with tile_n 256, else MOYE_ERR_TOO_LARGE) */
  int32_t flags;                 /* fused epilogue: MOYE_EPI_* activation | MOYE_EPI_BIAS_*; 0 = plain GEMM */
  const float* bias;             /* device pointer, fp32, read only when a bias mode is set */
} moye_gemm_params_t;

typedef enum {
  MOYE_COPY_AUTO = 0,
  MOYE_COPY_UNIVERSAL128 = 1,    /* 128-bit UniversalCopy atoms, gmem -> smem -> gmem */
  MOYE_COPY_TMA = 2,             /* cp.async.bulk.tensor load + store through an smem ring */
  MOYE_COPY_TRANSPOSE = 3        /* src and dst contiguous along different modes: TMA load, 128-bit register
                                    transposition between two swizzled smem tiles, TMA store (the automatic choice
                                    for such operands; takes over `transpose_kernel`, reference
                                    test/host/copy_async.jl:51-74) */
} moye_copy_mode_t;

typedef struct {
  int32_t mode;                  /* moye_copy_mode_t */
  int32_t tile_m;                /* tile extent along the contiguous mode; 0 = default (256 bytes) */
  int32_t tile_n;                /* tile extent along the strided mode;    0 = default (64)  */
  int32_t flags;                 /* reserved, must be 0 */
} moye_copy_params_t;

/* Library lifetime.  A handle is bound to the CUDA device current at creation; it owns a
 * small device status word, the stream-K workspace and a tensor-map cache.  Replaces nothing
 * in the reference (CUDA.jl owns the context there). */
int moye_b200_create(moye_handle_t* out);
int moye_b200_destroy(moye_handle_t h);
int moye_b200_version(void);
const char* moye_b200_last_error(void);

/* Synchronises `stream` and returns the device-side status word: MOYE_OK, or
 * MOYE_ERR_TIMEOUT if a bounded mbarrier wait inside a kernel gave up (the kernel then tears
 * down cleanly and the context stays usable: on such a report the call also waits for the whole
 * device and puts the stream-K ticket areas of the handle back to zero, which a kernel that gave
 * up may have left half counted).  `site` (may be NULL) receives the code of the wait that ran
 * out (in the debug build also the code of a failed device-side address check, 951-982).  The reference's counterpart is `CUDA.synchronize()` after the launch
 * (reference test/device/matmul.jl:80). */
int moye_b200_status(moye_handle_t h, void* stream, int32_t* site);

/* Integration test of the error path: launches a one-warp kernel that waits, with the bounded wait every
 * kernel of the library uses, on an mbarrier nothing arrives at.  The wait gives up after its poll limit
 * (about two seconds), the kernel returns normally, and the next moye_b200_status() on the stream
 * reports MOYE_ERR_TIMEOUT with site code 901; the context stays usable.  No counterpart in the reference
 * (its kernels have no waits that can fail). */
int moye_b200_selftest_bounded_wait(moye_handle_t h, void* stream);

/* Second half of that integration test: overwrites the ticket areas of both stream-K scratch buffers of the handle
 * (those that exist) with non-zero counts on `stream`, which is the state a kernel that gave up half-way would
 * leave behind.  A following time-out report through moye_b200_status() must put them back to zero.  Never call
 * this outside a test: the next stream-K product on the handle is wrong until moye_b200_status() has seen a
 * time-out.  No counterpart in the reference. */
int moye_b200_selftest_dirty_tickets(moye_handle_t h, void* stream);

/* D = alpha*scale_a*scale_b * A.B^T + beta*C with A:(M,K), B:(N,K), C,D:(M,N).
 * Takes over the whole `matmul_kernel` of reference examples/gemm.jl:4-64 (the gemm!-based
 * form is test/device/matmul.jl:3-53): local_tile of A/B/C, the gmem->smem `copyto!`
 * (src/algorithm/copy.jl:42-64), the `gemm!` tower (src/algorithm/blas.jl:11-131) and the
 * epilogue `copyto!(gC, rC)` (examples/gemm.jl:62), on tcgen05 tensor cores.
 * Supported (A,B -> accum -> D): f16,f16 -> f32 -> f32|f16; bf16,bf16 -> f32 -> f32|bf16;
 * s8|u8,s8|u8 -> s32 -> s32 (bit-exact; signed and unsigned may be mixed, reference S32U8S8S32 ... ops,
 * src/arch/mma/make_mma_ops.jl:143-160); e4m3,e4m3 -> f32 -> bf16|f32 with scale_a*scale_b;
 * f32,f32 -> f32 -> f32 on the tf32 tensor-core kind: by default to Float32 accuracy (three products of the
 * operands' high and low parts, D = lo(A).B + A.lo(B) + A.B, as accurate as the host's fp32 gemm!; rows of A and
 * B must be 16-byte multiples; a handle-owned buffer of the operands' size holds the low parts), with
 * MOYE_GEMM_ALLOW_TF32 one product (operands read with a 10-bit mantissa, about 1e-3 relative, three times faster).
 * The Float32 arrays of examples/gemm.jl run as they are.
 * A and B may each be K-major (stride 1 along K) or MN-major (stride 1 along M / N: MoYe's
 * column-major arrays, the storage of examples/gemm.jl:92-93), for every operand type.
 * D may be M-major or N-major.  The strided mode's pitch must be a multiple of 16 bytes.
 * C may be NULL when beta == 0.  Violations are errors, never fallbacks. */
int moye_b200_gemm(moye_handle_t h, const moye_tensor_t* D, const moye_tensor_t* A,
                   const moye_tensor_t* B, const moye_tensor_t* C,
                   const moye_gemm_params_t* params, void* stream);

/* dst = src for two rank-2 tensors of equal shape and dtype, each contiguous along one mode,
 * tile by tile through shared memory.  Both contiguous along the same mode: takes over
 * `copy_kernel` (reference test/host/copy_async.jl:3-25) and `copyto!(tiled_copy, dst, src)`
 * with 128-bit atoms (src/algorithm/copy.jl:106-130, src/arch/copy/copy.jl:26-51).  Contiguous
 * along different modes (`copyto!(dest, transpose(src))`; elements of 1, 2, 4 or 8 bytes): takes
 * over `transpose_kernel` (test/host/copy_async.jl:51-74). */
int moye_b200_copy(moye_handle_t h, const moye_tensor_t* dst, const moye_tensor_t* src,
                   const moye_copy_params_t* params, void* stream);

/* `copyto!(tiled_copy, dst, src)` for a TiledCopy on an ldmatrix atom (`LDSM_U32x{1,2,4}_N`, `LDSM_U16x{2,4,8}_T`;
 * reference src/arch/copy/ldmatrix.jl:18-96, src/traits/ldmatrix.jl:1-41), as in the kernel of the reference's
 * device test (test/device/tiled_copy.jl:2-23): one tile of 16-bit elements, `span` elements long in memory
 * (at most 24576), is staged in shared memory; each of `threads` threads (a multiple of 32) loads `iters`
 * fragments with `ldmatrix` (`matrices` = 1, 2 or 4, `transposed` = .trans) and stores the 2 * matrices values of
 * every fragment to global memory.  The two tables are HOST arrays of element offsets inside the tile, evaluated
 * by the caller from `partition_S` / `partition_D`: src_offsets[t * iters + i] is the first of the 8 contiguous
 * values of thread t's i-th source fragment (16-byte aligned), dst_offsets[(t * iters + i) * 2 * matrices + v]
 * where its v-th received value goes.  dst and src are device pointers to the tile's first element. */
int moye_b200_ldsm_copy(moye_handle_t h, void* dst, const void* src, int32_t span, int32_t matrices,
                        int32_t transposed, int32_t threads, int32_t iters, const int32_t* src_offsets,
                        const int32_t* dst_offsets, void* stream);

/* dst[Ld(i)] = src[Ls(i)] for i in 1:size(Ls), any two layouts of equal size: the
 * elementwise `copyto!(dst, src)` of reference src/algorithm/copy.jl:4-16,42-64 evaluated
 * on the device.  elem_bytes in {1,2,4,8,16}. */
int moye_b200_layout_copy(moye_handle_t h, void* dst, const moye_layout_t* dst_layout,
                          const void* src, const moye_layout_t* src_layout,
                          int32_t elem_bytes, void* stream);

/* out[i] = layout(i + first) for i in 0:n-1, with MoYe's 1-based linear indexing
 * (reference src/layout.jl call operator -> src/stride.jl:20-31 `coord_to_index0`): the
 * layout function evaluated on the device.  `out` is a device array of n int64. */
int moye_b200_layout_eval(moye_handle_t h, const moye_layout_t* layout, int64_t first,
                          int64_t n, int64_t* out, void* stream);

/* D(M,N) = alpha * A(M,K) . B(N,K)^T for M <= 32 (the decode shape), for callers that must
 * not allocate.  It has no counterpart in the reference.
 *
 * The other GEMM entry point keeps its stream-K scratch in memory the handle obtains with
 * cudaMalloc (and creating a handle allocates too).  Some callers cannot do that: a serving
 * loop whose device memory was fully handed out at start-up, a plugin bound by a "no
 * allocation after initialisation" rule, or code that simply has no handle.  This entry point
 * takes no handle and calls no cudaMalloc / cudaFree or any other allocating routine: its
 * scratch (tickets, fp32 partial tiles, a status word; 5.02 MiB) is a static device array
 * inside the library, which every GPU that loads the library holds until the process exits.
 *
 * Limits (errors, with a message, beyond them): M <= 32, N <= 524288 (4096 row blocks of W),
 * at most 160 SMs.  A, B f16 or bf16, K-major, 16-byte-aligned rows; D f32 or the operand type,
 * any strides.  beta is 0 (C is not read).
 *
 * The first call on a device (with that device current) looks up the array's device address
 * and raises the kernels' shared-memory limit; make that first call before any stream capture.
 * All calls share the one array and it keeps the previous call's contents: each call clears
 * the part that must start at zero on `stream` before its kernel.  Two calls that overlap on
 * the GPU (different streams, or different host threads without ordering) race on it; order
 * them on one stream or with events.
 *
 * device_status: optional device int32 that receives a wait-site code if a bounded wait in
 * the kernel gives up (0 otherwise; the caller clears it); NULL keeps that word inside the array,
 * where moye_b200_gemm_skinny_static_status() reads it. */
int moye_b200_gemm_skinny_static(const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                                 float alpha, int32_t* device_status, void* stream);

/* Reads back what the most recent moye_b200_gemm_skinny_static() calls on this device recorded when they were
 * given device_status == NULL: synchronises `stream`, copies the status word out of the static array (no
 * allocation: a plain 4-byte cudaMemcpy) and returns MOYE_OK, or MOYE_ERR_TIMEOUT with the wait-site code in
 * `site` (may be NULL).  The word is cleared by the next static GEMM call, so ask before launching another.
 * No counterpart in the reference. */
int moye_b200_gemm_skinny_static_status(void* stream, int32_t* site);

/* Y = a*X + b*Y, elementwise over two rank-1 or rank-2 arrays of equal shape and element type (f32, f16, bf16) that
 * are contiguous along the same mode: `axpby!` of reference src/algorithm/blas.jl:1-9 on global-memory arrays.  As
 * there, Y is not read when b == 0.  Arithmetic as on the host: both products rounded to fp32, then added, one
 * rounding to the element type.  X may be Y. */
int moye_b200_axpby(moye_handle_t h, const moye_tensor_t* Y, const moye_tensor_t* X, float a, float b, void* stream);

/* ---- several GPUs: one process (or thread) per GPU, each with its own handle ------------------------------------
 * The reference has no multi-GPU code.  The hot path shards without any exchange: GEMM along M (rows of A and D, B
 * replicated), weight-bound products along N (rows of W, columns of Y), copies along row blocks; every rank calls
 * moye_b200_gemm / moye_b200_copy on its own block.  What needs the other GPUs is putting a result back together,
 * or handing the replicated operand round; those two run on NCCL (looked up at run time as libnccl.so.2).
 *
 *   moye_b200_comm_unique_id   rank 0 makes a 128-byte id and hands it to the others by any host channel
 *   moye_b200_comm_init        every rank, with its device current: joins (collective; blocks until all have)
 *   moye_b200_allgather        every rank contributes its block of `full`; afterwards all hold all of it
 *   moye_b200_bcast            `t` of rank `root` is copied into `t` of every rank
 *   moye_b200_comm_destroy     leaves; moye_b200_destroy does not do this for you
 *
 * Blocks follow one rule everywhere: extent E along the split mode, cut into `world` blocks whose borders are
 * multiples of `align` (units = ceil(E / align); rank r owns [units*r/world, units*(r+1)/world) * align, clipped
 * to E).  `mode` is the split mode of `full` (0 or 1); it must be the OUTER mode in memory in both tensors, so
 * that a block is one contiguous byte range (rows of a row-major matrix, columns of a column-major one);
 * anything else is MOYE_ERR_UNSUPPORTED_LAYOUT.  `shard` may point into `full` (in place) or elsewhere.  Both
 * collectives are asynchronous on `stream` like every other call. */
int moye_b200_comm_unique_id(char* id128);
int moye_b200_comm_init(moye_handle_t h, int32_t rank, int32_t world, const char* id128);
int moye_b200_comm_destroy(moye_handle_t h);
int moye_b200_allgather(moye_handle_t h, const moye_tensor_t* shard, const moye_tensor_t* full, int32_t mode,
                        int64_t align, void* stream);
int moye_b200_bcast(moye_handle_t h, const moye_tensor_t* t, int32_t root, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOYE_B200_H */
