// Dense tiled GEMM for sm_100a: D = alpha * A.B^T (+ beta*C), A:(M,K) and B:(N,K) K-major.
//
// This kernel is the Blackwell re-design of MoYe's `matmul_kernel` (reference
// examples/gemm.jl:4-64).  The roles of the reference's steps map as follows:
//   @tile mA (bM,bK) (blockIdx.x, :)           -> TMA tensor-map box + tile coordinates
//   copyto!(sA, gA) ; cp_async_wait ; sync     -> cp.async.bulk.tensor into a 128B-swizzled
//                                                 smem ring, mbarrier full/empty pipeline
//   gemm!(rC, sA, sB, rC) / FMA triple loop    -> tcgen05.mma, accumulator in tensor memory
//   copyto!(gC, rC)                            -> tcgen05.ld -> registers -> smem -> TMA store
//
// One persistent CTA per SM, 6 warps: warp 0 = TMA producer, warp 1 = MMA issuer (also owns
// the TMEM allocation), warps 2-5 = epilogue.  The accumulator is double-buffered in TMEM
// so the epilogue of tile i overlaps the main loop of tile i+1.
//
// This file is the host-side dispatch: argument checks, the choice of kernel and tile, tensor maps.  The kernels
// are in gemm_single.cu, gemm_pair.cu, gemm_wide.cu, gemm_splitk.cu (dense) and gemm_skinny.cu (decode shapes).
#include "gemm_common.cuh"

namespace moye {

int launch_gemm_skinny(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                       const moye_gemm_params_t* p, cudaStream_t stream);

// The stream-K tail's scratch: a ticket area (zero at rest; the warp that finishes a tile restores its ticket,
// moye_b200_status() clears the area after a time-out) and two partial-accumulator slabs per CTA pair.  Allocated
// once, at its final size, the first time a product takes the tail.
int ensure_tail_workspace(moye_b200_ctx* h) {
  std::lock_guard<std::mutex> lk(h->mu);
  if (h->tail_ws) return MOYE_OK;
  const size_t bytes = kTailTicketBytes + (size_t)(h->num_sms / 2) * 2 * kSkSlabWords * sizeof(uint32_t);
  void* p = nullptr;
  MOYE_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, kTailTicketBytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    MOYE_FAIL(MOYE_ERR_CUDA, "clearing the stream-K tickets failed: %s", cudaGetErrorString(e));
  }
  h->tail_ws = p;
  h->tail_ws_bytes = bytes;
  return MOYE_OK;
}

// ------------------------------------------------------------------------------------------
// Float32 operands at Float32 accuracy on the tf32 tensor-core kind ("3 x TF32").  The tensor core reads a Float32
// with its low 13 mantissa bits dropped, i.e. it multiplies hi(a) * hi(b).  With lo(x) = x - hi(x) (exact in fp32)
//   a * b = hi(a) hi(b) + lo(a) hi(b) + hi(a) lo(b) + lo(a) lo(b),
// and the last term is below 2^-22 of the product.  Three products with fp32 accumulation give the rest:
//   D  = alpha * lo(A) . B^T + beta * C        (the tensor core takes hi(B) and the top 11 bits of lo(A))
//   D += alpha * A . lo(B)^T
//   D  = act(alpha * A . B^T + D + bias)
// small terms first.  lo(A) and lo(B) live in a handle-owned buffer that grows on demand (the first product at a
// larger size synchronises the device to re-allocate it).  The reference multiplies Float32 in Float32
// (examples/gemm.jl:51-57 through UniversalFMA); this keeps its accuracy, not its bit pattern.
__global__ void __launch_bounds__(256) split_lo_kernel(float* lo, const float* x, long long rows, long long cols,
                                                      long long pitch, long long elems, int* status) {
  const long long per_row = cols / 4;  // cols is a multiple of 4 and rows are 16-byte aligned: checked by the caller
  const long long total = rows * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_row, c = i - r * per_row;
    if (!MOYE_DBG_OK(r * pitch + 4 * c + 3 < elems, status, 961)) continue;
    const float4 v = *(reinterpret_cast<const float4*>(x + r * pitch) + c);
    float4 o;
    o.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
    o.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
    o.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
    o.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
    *(reinterpret_cast<float4*>(lo + r * pitch) + c) = o;
  }
}

int launch_gemm(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                const moye_tensor_t* C, const moye_gemm_params_t* pp, cudaStream_t stream);

static int launch_gemm_f32x3(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                             const moye_tensor_t* C, const moye_gemm_params_t& p, cudaStream_t stream) {
  if (D->dtype != MOYE_F32) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "Float32 operands give a Float32 result");
  // the operand as (rows of contiguous elements) x pitch: either mode may be the contiguous one
  struct Span { long long rows, cols, pitch, elems; };
  auto span_of = [](const moye_tensor_t* t, Span* s) {
    const long long s0 = t->shape[0], s1 = t->shape[1];
    if (t->stride[1] == 1 && (t->stride[0] != 1 || s1 > 1 || s0 == 1)) { s->rows = s0; s->cols = s1; s->pitch = t->stride[0]; }
    else if (t->stride[0] == 1) { s->rows = s1; s->cols = s0; s->pitch = t->stride[1]; }
    else return false;
    if (s->rows == 1) s->pitch = s->cols;
    s->elems = (s->rows - 1) * s->pitch + s->cols;
    return s->pitch >= s->cols;
  };
  Span sa, sb;
  if (!span_of(A, &sa) || !span_of(B, &sb))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "A and B need a unit stride along K or along M / N");
  auto aligned = [](const moye_tensor_t* t, const Span& s) {
    return (reinterpret_cast<uintptr_t>(t->ptr) & 15) == 0 && s.cols % 4 == 0 && (s.rows == 1 || s.pitch % 4 == 0);
  };
  if (!aligned(A, sa) || !aligned(B, sb))
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "Float32 operands need 16-byte aligned rows whose length is a multiple of 4 elements");
  const size_t a_bytes = ((size_t)sa.elems * 4 + 255) & ~size_t(255), b_bytes = ((size_t)sb.elems * 4 + 255) & ~size_t(255);
  if (a_bytes + b_bytes > h->split_ws_bytes) {
    if (h->split_ws) {
      MOYE_CUDA(cudaDeviceSynchronize());
      MOYE_CUDA(cudaFree(h->split_ws));
      h->split_ws = nullptr;
      h->split_ws_bytes = 0;
    }
    MOYE_CUDA(cudaMalloc(&h->split_ws, a_bytes + b_bytes));
    h->split_ws_bytes = a_bytes + b_bytes;
  }
  if (int rc = order_scratch_use(h, &h->split_order, stream)) return rc;
  float* a_lo = reinterpret_cast<float*>(h->split_ws);
  float* b_lo = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(h->split_ws) + a_bytes);
  auto split = [&](float* lo, const moye_tensor_t* t, const Span& s) {
    long long blocks = (s.rows * (s.cols / 4) + 255) / 256;
    if (blocks > (long long)h->num_sms * 8) blocks = (long long)h->num_sms * 8;
    split_lo_kernel<<<(unsigned)(blocks < 1 ? 1 : blocks), 256, 0, stream>>>(lo, static_cast<const float*>(t->ptr), s.rows,
                                                                             s.cols, s.pitch, s.elems, h->d_status);
  };
  split(a_lo, A, sa);
  split(b_lo, B, sb);
  MOYE_CUDA(cudaGetLastError());
  moye_tensor_t Al = *A, Bl = *B;
  Al.ptr = a_lo;
  Bl.ptr = b_lo;
  moye_gemm_params_t q = p;
  q.flags = (p.flags & (MOYE_GEMM_TAIL_OFF | MOYE_GEMM_TAIL_ON)) | MOYE_GEMM_ALLOW_TF32;  // no bias / activation yet
  q.bias = nullptr;
  if (int rc = launch_gemm(h, D, &Al, B, C, &q, stream)) return rc;   // D  = alpha lo(A) B^T + beta C
  q.beta = 1.f;
  if (int rc = launch_gemm(h, D, A, &Bl, D, &q, stream)) return rc;   // D += alpha A lo(B)^T
  q.flags = p.flags | MOYE_GEMM_ALLOW_TF32;
  q.bias = p.bias;
  if (int rc = launch_gemm(h, D, A, B, D, &q, stream)) return rc;     // D  = act(alpha A B^T + D + bias)
  return scratch_used(&h->split_order, stream);
}

int launch_gemm(moye_b200_ctx* h, const moye_tensor_t* D, const moye_tensor_t* A, const moye_tensor_t* B,
                const moye_tensor_t* C, const moye_gemm_params_t* pp, cudaStream_t stream) {
  moye_gemm_params_t p = {1.f, 0.f, 1.f, 1.f, 0, 0, 0, 0, nullptr};
  if (pp) p = *pp;
  const int act = p.flags & MOYE_EPI_ACT_MASK, bias_mode = (p.flags & MOYE_EPI_BIAS_MASK) >> 4;
  if ((p.flags & ~(MOYE_EPI_ACT_MASK | MOYE_EPI_BIAS_MASK | MOYE_GEMM_TAIL_OFF | MOYE_GEMM_TAIL_ON | MOYE_GEMM_ALLOW_TF32)) != 0 ||
      act > MOYE_EPI_SILU || bias_mode > 2 || (p.flags & (MOYE_GEMM_TAIL_OFF | MOYE_GEMM_TAIL_ON)) == (MOYE_GEMM_TAIL_OFF | MOYE_GEMM_TAIL_ON))
    MOYE_FAIL(MOYE_ERR_INVALID_ARG, "unknown or contradictory bits in flags (0x%x)", p.flags);
  if (p.path < 0 || p.path > 5) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "path must be 0..5 (got %d)", p.path);
  if (bias_mode != 0 && !p.bias) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "a bias mode is set but bias is NULL");
  if (bias_mode != 0 && (reinterpret_cast<uintptr_t>(p.bias) & 3) != 0)
    MOYE_FAIL(MOYE_ERR_MISALIGNED, "bias must be 4-byte aligned");
  if (A->rank != 2 || B->rank != 2 || D->rank != 2) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "A, B, D must be rank 2");
  const int64_t M = A->shape[0], K = A->shape[1], N = B->shape[0];
  if (B->shape[1] != K || D->shape[0] != M || D->shape[1] != N)
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "shape mismatch: A (%lld,%lld) B (%lld,%lld) D (%lld,%lld)", (long long)M,
              (long long)K, (long long)N, (long long)B->shape[1], (long long)D->shape[0], (long long)D->shape[1]);
  if (M <= 0 || N <= 0 || K <= 0) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "empty GEMM");
  if (M > INT32_MAX / 2 || N > INT32_MAX / 2 || K > INT32_MAX / 2) MOYE_FAIL(MOYE_ERR_TOO_LARGE, "extent too large");
  if (!A->ptr || !B->ptr || !D->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "null data pointer");
  // 8-bit integers may be mixed (the reference has S32U8S8S32 / S32S8U8S32 ops, src/arch/mma/make_mma_ops.jl:143-160)
  const bool a_int8 = A->dtype == MOYE_S8 || A->dtype == MOYE_U8, b_int8 = B->dtype == MOYE_S8 || B->dtype == MOYE_U8;
  if (A->dtype != B->dtype && !(a_int8 && b_int8))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "A and B must have the same dtype (s8 and u8 may be mixed)");

  if (A->dtype == MOYE_F32 && B->dtype == MOYE_F32 && !(p.flags & MOYE_GEMM_ALLOW_TF32))
    return launch_gemm_f32x3(h, D, A, B, C, p, stream);

  int kind;
  uint32_t ab_fmt, b_fmt, c_fmt;
  switch (A->dtype) {
    case MOYE_F16: kind = KIND_F16; ab_fmt = 0; c_fmt = 1; break;
    case MOYE_BF16: kind = KIND_F16; ab_fmt = 1; c_fmt = 1; break;
    case MOYE_S8: kind = KIND_I8; ab_fmt = 1; c_fmt = 2; break;
    case MOYE_U8: kind = KIND_I8; ab_fmt = 0; c_fmt = 2; break;
    case MOYE_E4M3: kind = KIND_F8; ab_fmt = 0; c_fmt = 1; break;
    case MOYE_F32: kind = KIND_TF32; ab_fmt = 2; c_fmt = 1; break;  // operands are read as tf32 (10-bit mantissa)
    default: MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "operand dtype %d is not supported by the tcgen05 path", A->dtype);
  }
  b_fmt = kind == KIND_I8 ? (B->dtype == MOYE_S8 ? 1u : 0u) : ab_fmt;
  const int out = D->dtype;
  const bool out_ok = (A->dtype == MOYE_F16 && (out == MOYE_F32 || out == MOYE_F16)) ||
                      (A->dtype == MOYE_BF16 && (out == MOYE_F32 || out == MOYE_BF16)) ||
                      (kind == KIND_I8 && out == MOYE_S32) ||
                      (A->dtype == MOYE_E4M3 && (out == MOYE_BF16 || out == MOYE_F32)) ||
                      (A->dtype == MOYE_F32 && out == MOYE_F32);
  if (!out_ok) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_DTYPE, "output dtype %d not supported for operand dtype %d", out, A->dtype);
  // K-major (stride 1 along K) or MN-major (stride 1 along M / N, MoYe's column-major default)
  const bool a_mn = A->stride[1] != 1 || (K == 1 && A->stride[0] == 1 && M > 1);
  const bool b_mn = B->stride[1] != 1 || (K == 1 && B->stride[0] == 1 && N > 1);
  if ((a_mn && A->stride[0] != 1) || (b_mn && B->stride[0] != 1))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "A and B need a unit stride along K or along M / N; got A (%lld,%lld), B (%lld,%lld)",
              (long long)A->stride[0], (long long)A->stride[1], (long long)B->stride[0], (long long)B->stride[1]);
  bool m_major;
  if (D->stride[0] == 1 && (D->stride[1] != 1 || N == 1)) m_major = true;
  else if (D->stride[1] == 1) m_major = false;
  else MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "D must have a unit stride in one mode");

  float alpha = p.alpha * p.scale_a * p.scale_b;
  if (kind == KIND_I8) {
    if (alpha != 1.f || (p.beta != 0.f && p.beta != 1.f))
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the s8 -> s32 path is exact integer arithmetic: alpha must be 1, beta 0 or 1");
    if (act != 0 || bias_mode != 0)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the s8 -> s32 path takes no bias or activation (its epilogue is exact integer arithmetic)");
  }
  if (p.beta != 0.f) {
    if (!C || !C->ptr) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "beta != 0 needs C");
    if (C->rank != 2 || C->shape[0] != M || C->shape[1] != N || C->dtype != D->dtype)
      MOYE_FAIL(MOYE_ERR_UNSUPPORTED_SHAPE, "C must match D in shape and dtype");
  }

  if (p.path == 2 && (a_mn || b_mn)) MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "the skinny path takes K-major operands");
  // Automatic choice for decode shapes, from measurements at M = 1 .. 128 (bf16, weights from 1024 x 4096 to
  // 28672 x 8192).  The stream-K kernel deals equal runs of (row-block, K-block) units to all SMs; it is the fastest
  // form on large weights, where the other kernels' tile counts do not divide the SMs (16 x 28672 x 8192: 70-73 us
  // against 93 for split-K on clusters and 85 for single CTAs; 8192 x 8192 and 14336 x 4096 weights with 1-4 rows:
  // 30.4 / 28.6 us against 31.1 / 29.7).  On mid-sized weights the cluster split-K kernel (below) is faster at every M
  // (4096 x 4096: 12.5-14.0 us against 16.6-17.1; 8192 x 2048: 13.8 against 16.5-17; 2048 x 8192: 15.9-16.3 against
  // 16.5-18.6; 4096 x 1024: 8.9 against 12.4), and from 17 rows the stream-K kernel's X tiles and epilogue grow with M
  // (8192 x 8192, M = 32: 33.2 us against 30.7), unless it streams whole row-blocks (below).
  bool use_skinny = p.path == 2;
  if (p.path == 0 && p.tile_n == 0 && p.beta == 0.f && kind == KIND_F16 && M <= 128 && !a_mn && !b_mn && N >= 128 && K >= 512 &&
      (size_t)((N + 127) / 128) * sizeof(int) <= kSkinnyTicketBytes) {
    const long long nk = (long long)N * K;
    const long long row_blocks = (N + 127) / 128, k_blocks = (K + 63) / 64;
    // At least as many row-blocks as SMs (every CTA streams whole row-blocks and the exchange of the cut ones is hidden
    // behind them; the dense kernel would run in waves), or slightly fewer (one whole row-block per CTA, nothing to
    // exchange): the stream-K kernel up to 128 rows.  M = 17 ... 128, stream-K / dense kernel [cuBLAS]: 20480 x 8192
    // 56.5-62.4 / 89.3-90.7 us [56.6-66.0], 16384 x 4096 24.9-26.9 / 30.1-31.5 [25.0-27.1], 28672 x 8192 75.3-85.2 /
    // 79.9-84.7 [75.4-94.6], 37888 x 4096 51.7-55.9 / 54.6-56.7 [55.9-60.0]; 20480 x 2048 with 1-16 rows 17.9-19.5 / 29.9.
    const bool streams_whole = row_blocks >= h->num_sms || stream_k_whole_grid(row_blocks, k_blocks, h->num_sms);
    use_skinny = streams_whole || (M <= 16 && nk >= (64ll << 20)) || (M <= 4 && nk >= (48ll << 20));
  }
  if (use_skinny) {
    log_line("gemm %lld x %lld x %lld  in %d  -> stream-K decode kernel", (long long)M, (long long)N, (long long)K, A->dtype);
    return launch_gemm_skinny(h, D, A, B, &p, stream);
  }

  int bn = p.tile_n;
  if (bn == 0) {
    bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
    // one row of tiles (M <= 128): 256-wide tiles only if there are enough of them to occupy most SMs; otherwise
    // 128-wide tiles double the CTAs that stream B (14336 x 4096 weights, M = 64: 29 us against 35.5)
    if (M <= 128 && bn == 256 && (N + 255) / 256 < (long long)h->num_sms * 2 / 3) bn = 128;
  }
  // path 4 = CTA pairs on 256 x 512 tiles.  Chosen automatically when it fills the SM pairs at least as well as
  // 256 x 256 tiles do: it needs less operand traffic per flop and measured about 8 % faster on full waves.
  bool wide = p.path == 4;
  const int kb_all = (int)((K + 128 / dtype_bytes(A->dtype) - 1) / (128 / dtype_bytes(A->dtype)));
  // The K-split tail of the 256 x 512 kernel (gemm_wide.cu): the R tiles of the last, partly filled wave are shared
  // by all pairs in chains of L tiles on L + 1 pairs, every pair busy for t = ceil((L kb + lead) / (L + 1)) K blocks.
  // `last_wave` is the length of the last wave in K-block times.
  constexpr int kTailLead = 6;    // K blocks by which a head ends before the tail it is added to: time to drain,
                                  // store and publish an accumulator
  constexpr int kTailFixup = 10;  // K-block times a split tile costs extra: every pair of a chain drains its
                                  // accumulator once more, and the tensor cores wait while it does (measured: 5.6-6 us
                                  // per drain of a 256 x 512 fp32 tile against 0.55-0.62 us per K block)
  struct TailPlan { int sk_tiles, sk_chains, t_long, t_short, lead; double last_wave; };
  auto tail_plan = [&](bool force) {
    TailPlan tp = {0, 0, 0, 0, 0, 0.0};
    const long long pairs = h->num_sms / 2;
    const long long tiles = ((M + 255) / 256) * ((N + 511) / 512);
    const long long rest = tiles % pairs;
    if (rest == 0) return tp;
    tp.last_wave = kb_all;
    if ((p.flags & MOYE_GEMM_TAIL_OFF) || kb_all < 2) return tp;
    const long long chains = pairs - rest < rest ? pairs - rest : rest;
    const long long base = rest / chains;
    const long long lead = kTailLead < kb_all / 4 ? kTailLead : kb_all / 4;
    // every head h(i) = (i+1) t - i kb - lead and every tail must keep at least one K block
    auto busy = [&](long long len) { return (len * kb_all + lead + len) / (len + 1); };  // ceil((len kb + lead) / (len + 1))
    auto fits = [&](long long len) {
      const long long t = busy(len);
      if (t > kb_all - 1 || t - lead < 1) return false;
      for (long long i = 0; i < len; ++i) {
        const long long hd = (i + 1) * t - i * kb_all - lead;
        if (hd < 1 || hd > kb_all - 1) return false;
      }
      return true;
    };
    if (!fits(base) || (rest % chains && !fits(base + 1))) return tp;  // K too short to cut that often
    const long long t_long = busy(base + 1), t_short = busy(base), t_max = rest % chains ? t_long : t_short;
    // worth it when the chains, the extra drain included, end clearly before a whole tile would
    if (force || (double)(t_max + kTailFixup) <= 0.92 * kb_all) {
      tp.sk_tiles = (int)rest;
      tp.sk_chains = (int)chains;
      tp.t_long = (int)t_long;
      tp.t_short = (int)t_short;
      tp.lead = (int)lead;
      tp.last_wave = (double)(t_max + kTailFixup);
    }
    return tp;
  };
  if (p.path == 0 && M > 128 && bn == 256 && N >= 512) {
    const long long clusters = h->num_sms / 2;
    auto fill = [&](long long tm, long long tn, bool tail) {
      const long long tiles = ((M + tm - 1) / tm) * ((N + tn - 1) / tn);
      double waves = (double)((tiles + clusters - 1) / clusters);
      if (tail && tiles % clusters != 0) waves = (double)(tiles / clusters) + tail_plan(false).last_wave / kb_all;
      return (double)M * (double)N / (waves * clusters * tm * tn);
    };
    wide = fill(256, 512, true) * 1.08 >= fill(256, 256, false);
  }
  if (wide) bn = 256;
  const TailPlan tail = wide ? tail_plan((p.flags & MOYE_GEMM_TAIL_ON) != 0) : TailPlan{0, 0, 0, 0, 0, 0.0};
  // path 5 = split-K on clusters (128 x tile_n tiles, `split_k` CTAs per tile).  Chosen automatically when the
  // output has so few tiles that the other kernels would leave most SMs idle and K is long enough to cut (at least
  // 8 blocks per CTA): the tile width (256, 128) and split (4, 2) that put the most CTAs on the SMs without
  // exceeding them (4096 x 4096 weights, M = 128: 13.2 us with 32 tiles x 4 against 25-29 unsplit; M = 512: 22
  // against 30).  Clusters of 8 measured slower than clusters of 4 with the same number of CTAs (4096 x 4096, M = 128:
  // 24.2 us with 16 tiles x 8 against 13.2 with 32 x 4).
  const int kb_total = (int)((K + 128 / dtype_bytes(A->dtype) - 1) / (128 / dtype_bytes(A->dtype)));
  int split = 0;
  if (p.path == 5) {
    if (p.split_k != 0 && p.split_k != 2 && p.split_k != 4 && p.split_k != 8)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "split_k must be 0, 2, 4 or 8 (got %d)", p.split_k);
    if (p.tile_n != 0 && p.tile_n != 128 && p.tile_n != 256)
      MOYE_FAIL(MOYE_ERR_INVALID_ARG, "the split-K path takes tile_n 0, 128 or 256 (got %d)", p.tile_n);
  }
  // The cluster kernel takes K-major operands only: with MN-major (column-major) operands it raised an illegal
  // memory access on the device (256 x 512 x 1024 tf32, clusters of 4), the cause is not found yet, so such
  // products stay on the other kernels and an explicit request is refused.
  if (p.path == 5 && (a_mn || b_mn))
    MOYE_FAIL(MOYE_ERR_UNSUPPORTED_LAYOUT, "the split-K path takes K-major operands");
  if (p.path == 5 || (p.path == 0 && !wide && p.tile_n == 0 && !a_mn && !b_mn)) {
    long long best_ctas = 0;
    for (int bn_c = 256; bn_c >= 128; bn_c /= 2) {
      if (p.tile_n != 0 && bn_c != p.tile_n) continue;
      if (bn_c == 256 && N <= 128) continue;
      const long long tiles_c = ((M + 127) / 128) * ((N + bn_c - 1) / bn_c);
      for (int sp = 4; sp >= 2; sp /= 2) {
        if (p.split_k != 0 && sp != p.split_k) continue;
        if (tiles_c * sp <= h->num_sms && kb_total >= 8 * sp) {
          if (tiles_c * sp > best_ctas) { best_ctas = tiles_c * sp; split = sp; bn = bn_c; }
          break;
        }
      }
    }
    // clusters of 8 only where they put strictly more CTAs to work (128 x 1024 x 8192: 12.3 us with 8 tiles x 8
    // against 16.0 with 8 x 4)
    for (int bn_c = 256; bn_c >= 128; bn_c /= 2) {
      if ((p.tile_n != 0 && bn_c != p.tile_n) || (bn_c == 256 && N <= 128) || (p.split_k != 0 && p.split_k != 8)) continue;
      const long long tiles_c = ((M + 127) / 128) * ((N + bn_c - 1) / bn_c);
      if (tiles_c * 8 <= h->num_sms && kb_total >= 64 && tiles_c * 8 > best_ctas) { best_ctas = tiles_c * 8; split = 8; bn = bn_c; }
    }
    if (p.path == 5 && split == 0) {  // asked for explicitly: honour it even where it is not the fast choice
      split = p.split_k ? p.split_k : 2;
      bn = p.tile_n ? p.tile_n : (N > 128 ? 256 : 128);
    }
  }
  const bool pair = !split && (wide || p.path == 3 || (p.path == 0 && M > 128 && bn >= 128));
  if (pair && bn < 128) MOYE_FAIL(MOYE_ERR_INVALID_ARG, "CTA pairs take tile_n 128 or 256 (got %d)", bn);
  const int eb = dtype_bytes(A->dtype);
  if (b_mn && eb == 1) {
    // an MN-major tile is loaded in chunks of 128 bytes along N = 128 8-bit elements: a CTA's share of B must be
    // at least that wide (single CTAs: tile_n >= 128; pairs: tile_n 256, i.e. 128 columns per CTA); a narrower
    // request is widened
    const int need = pair ? 256 : 128;
    if (bn < need) bn = need;
  }
  const int bk = 128 / eb;
  CUtensorMap ta, tb, td;
  const int ch = 128 / eb;  // elements in one 128-byte chunk
  // MN-major 32-bit tiles have one legal shared-memory form: the 128-byte swizzle with 32-byte atoms
  const int mn_swizzle = eb == 4 ? TMAP_SWIZZLE_128B_ATOM_32B : TMAP_SWIZZLE_128B;
  if (a_mn) {
    if (int rc = make_tmap_2d(h, &ta, A->ptr, A->dtype, M, K, (uint64_t)A->stride[1] * eb, ch, bk, mn_swizzle)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &ta, A->ptr, A->dtype, K, M, (uint64_t)A->stride[0] * eb, bk, 128, true)) return rc;
  }
  if (b_mn) {
    if (int rc = make_tmap_2d(h, &tb, B->ptr, B->dtype, N, K, (uint64_t)B->stride[1] * eb, ch, bk, mn_swizzle)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &tb, B->ptr, B->dtype, K, N, (uint64_t)B->stride[0] * eb, bk,
                              wide ? 256 : (pair ? bn / 2 : bn), true))
      return rc;
  }
  const int ob = dtype_bytes(out);
  if (m_major) {
    if (int rc = make_tmap_2d(h, &td, D->ptr, out, M, N, (uint64_t)D->stride[1] * ob, 32, 32, false)) return rc;
  } else {
    if (int rc = make_tmap_2d(h, &td, D->ptr, out, N, M, (uint64_t)D->stride[0] * ob, 128 / ob, 32, true)) return rc;
  }

  GemmArgs a;
  a.M = (int)M; a.N = (int)N; a.K = (int)K;
  a.m_tiles = pair ? (int)((M + 255) / 256) : (int)((M + 127) / 128);
  a.n_tiles = wide ? (int)((N + 511) / 512) : (int)((N + bn - 1) / bn);
  a.k_blocks = (int)((K + bk - 1) / bk);
  // Tile groups: all column tiles of `group_m` row tiles run before the next group, so the group's A panel
  // (rows x K) is re-used from L2 while B streams through.  Size the panel at about 32 MB: the 126 MB L2 is two 63 MB halves, and a 67 MB panel measurably thrashes (DRAM reads 1.1 GB -> 1.3-1.4 GB at 8192^3).
  {
    const long long rows_per_tile = pair ? 256 : 128;
    long long gm = (32ll << 20) / ((long long)K * eb * rows_per_tile);
    if (gm < 4) gm = 4;
    if (gm > a.m_tiles) gm = a.m_tiles;
    a.group_m = (int)gm;
  }
  a.idesc = (c_fmt << 4) | (ab_fmt << 7) | (b_fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
            ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((pair ? 256 : 128) >> 4) << 24);
  a.a_mn = a_mn ? 1 : 0;
  a.b_mn = b_mn ? 1 : 0;
  a.bias = bias_mode ? p.bias : nullptr;
  a.bias_mode = bias_mode;
  a.act = act;
  a.alpha = alpha;
  a.beta = p.beta;
  a.C = (p.beta != 0.f) ? C->ptr : nullptr;
  a.c_sm = (p.beta != 0.f) ? C->stride[0] : 0;
  a.c_sn = (p.beta != 0.f) ? C->stride[1] : 0;
  a.status = h->d_status;
  a.D = D->ptr;
  a.d_sm = D->stride[0];
  a.d_sn = D->stride[1];
  a.sk_tiles = 0;
  a.sk_chains = 1;
  a.sk_t_long = a.sk_t_short = a.sk_lead = 0;
  a.sk_ws = nullptr;
  a.sk_tickets = nullptr;
  if (wide && tail.sk_tiles > 0) {
    if (int rc = ensure_tail_workspace(h)) return rc;
    a.sk_tiles = tail.sk_tiles;
    a.sk_chains = tail.sk_chains;
    a.sk_t_long = tail.t_long;
    a.sk_t_short = tail.t_short;
    a.sk_lead = tail.lead;
    a.sk_tickets = reinterpret_cast<int*>(h->tail_ws);
    a.sk_ws = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(h->tail_ws) + kTailTicketBytes);
  }

  if (split) {  // the partial tiles of a cluster meet in the same scratch
    if (int rc = ensure_tail_workspace(h)) return rc;
    a.sk_ws = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(h->tail_ws) + kTailTicketBytes);
  }

  if (log_level() >= 1)
    log_line("gemm %lld x %lld x %lld  in %d out %d  A %s B %s D %s  -> %s, tile_n %d%s%s", (long long)M, (long long)N, (long long)K,
             A->dtype, out, a_mn ? "MN-major" : "K-major", b_mn ? "MN-major" : "K-major", m_major ? "M-major" : "N-major",
             split ? "split-K clusters" : (wide ? "CTA pairs, 256 x 512 tiles" : (pair ? "CTA pairs" : "single CTAs")), wide ? 512 : bn,
             split ? (split == 2 ? ", 2 CTAs per tile" : (split == 4 ? ", 4 CTAs per tile" : ", 8 CTAs per tile")) : "",
             a.sk_tiles > 0 ? ", K-split tail" : "");
  if (split) return launch_dense_splitk(kind, out, bn, h, ta, tb, a, split, stream);
  if (wide) return launch_dense_wide(kind, out, m_major, h, ta, tb, td, a, stream);
  if (pair) return launch_dense_pair(kind, out, m_major, bn, h, ta, tb, td, a, stream);
  return launch_dense_single(kind, out, m_major, bn, h, ta, tb, td, a, stream);
}

}  // namespace moye
