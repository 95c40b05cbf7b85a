# MoYeB200 -- host-level `gemm!` / `copyto!` methods for MoYe arrays in global memory, bound to
# libmoye_b200 (include/moye_b200.h) with ccall.  Additive: nothing in MoYe changes.
#
# This file has never been executed: the image this library is built in has no Julia.  It is the
# binding a MoYe maintainer would add; the same calls are exercised from Python (ctypes) by the tests.
module MoYeB200

using MoYe, CUDA, Libdl
using MoYe: MoYeArray, ViewEngine, Layout, TiledMMA, TiledCopy, AbstractMMAOP, AbstractCopyOp,
            flatten, coalesce, shape, stride, layout, rank

const libmoye_b200 = Ref{String}(get(ENV, "MOYE_B200_LIB", "libmoye_b200.so"))
__init__() = atexit(destroy_handles)

# ---- C structs (include/moye_b200.h)
struct MoyeTensor
    ptr::Ptr{Cvoid}
    dtype::Int32
    rank::Int32
    shape::NTuple{4, Int64}
    stride::NTuple{4, Int64}
end
struct MoyeGemmParams
    alpha::Float32; beta::Float32; scale_a::Float32; scale_b::Float32
    tile_n::Int32; split_k::Int32; path::Int32; flags::Int32
    bias::Ptr{Cvoid}   # Float32 device vector of the fused epilogue, C_NULL without one
end
const EPI_ACT = Dict(nothing => 0, :relu => 1, :gelu => 2, :silu => 3)   # MOYE_EPI_* of the header
const EPI_BIAS_COL, EPI_BIAS_ROW = 0x10, 0x20
const GEMM_TAIL_OFF, GEMM_TAIL_ON, GEMM_ALLOW_TF32 = 0x100, 0x200, 0x400     # MOYE_GEMM_* of the header
struct MoyeCopyParams
    mode::Int32; tile_m::Int32; tile_n::Int32; flags::Int32
end

primitive type E4M3 8 end   # MoYe has no fp8 type; bits only

moye_dtype(::Type{Float32}) = Int32(0); moye_dtype(::Type{Float16}) = Int32(1)
moye_dtype(::Type{MoYe.BFloat16}) = Int32(2); moye_dtype(::Type{Int8}) = Int32(3)
moye_dtype(::Type{UInt8}) = Int32(4); moye_dtype(::Type{E4M3}) = Int32(5); moye_dtype(::Type{Int32}) = Int32(6)

# ---- the gap MoYe leaves on the host side: arrays over device pointers (src/engine.jl:10-15 only
# wraps Ptr and LLVMPtr; src/pointer.jl:1 only recognises LLVMPtr{..., AS.Global} as global memory)
MoYe.ViewEngine(p::CuPtr{T}) where {T} = ViewEngine{T, CuPtr{T}}(p, 0)          # hypothetical ctor
MoYe.MoYeArray(A::CuArray{T}, l::Layout) where {T} = MoYeArray(ViewEngine(pointer(A)), l)
MoYe.MoYeArray(A::CuArray{T}, s::Tuple) where {T} = MoYeArray(A, MoYe.make_layout(s))
MoYe.isgmem(::MoYeArray{T, N, ViewEngine{T, CuPtr{T}}}) where {T, N} = true

# ---- new ops (MoYe's naming: src/arch/mma/make_mma_ops.jl:368, src/arch/copy/copy_async.jl:8)
abstract type AbstractSM100MMAOP{D, A, B, C} <: AbstractMMAOP{D, A, B, C} end
struct MMAOP_SM100_128x256x16_F32F16F16F32_SS <: AbstractSM100MMAOP{Float32, Float16, Float16, Float32} end
struct MMAOP_SM100_128x256x16_F32BF16BF16F32_SS <: AbstractSM100MMAOP{Float32, MoYe.BFloat16, MoYe.BFloat16, Float32} end
struct MMAOP_SM100_128x256x32_S32S8S8S32_SS <: AbstractSM100MMAOP{Int32, Int8, Int8, Int32} end
struct MMAOP_SM100_128x256x32_S32U8U8S32_SS <: AbstractSM100MMAOP{Int32, UInt8, UInt8, Int32} end
struct MMAOP_SM100_128x256x32_F32E4M3E4M3F32_SS <: AbstractSM100MMAOP{Float32, E4M3, E4M3, Float32} end
# Float32 storage on the tf32 kind.  gemm! keeps Float32 accuracy (three tf32 products of the operands' high and low
# parts) unless `allow_tf32 = true` asks for one product (operands read with the low 13 mantissa bits dropped)
struct MMAOP_SM100_128x256x8_F32TF32TF32F32_SS <: AbstractSM100MMAOP{Float32, Float32, Float32, Float32} end
struct CPOP_TMA_LOAD_SW128 <: AbstractCopyOp{Registers{UInt128, 1}, Registers{UInt128, 1}} end
struct CPOP_TMA_STORE <: AbstractCopyOp{Registers{UInt128, 1}, Registers{UInt128, 1}} end
# one thread issues a tcgen05 instruction for the whole CTA tile; the accumulator lives in tensor memory
MoYe.thr_id(::MoYe.MMATraits{<:AbstractSM100MMAOP}) = MoYe.@Layout 1
MoYe.shape_mnk(::MMAOP_SM100_128x256x16_F32F16F16F32_SS) = MoYe.static((128, 256, 16))
MoYe.shape_mnk(::MMAOP_SM100_128x256x16_F32BF16BF16F32_SS) = MoYe.static((128, 256, 16))
MoYe.shape_mnk(::MMAOP_SM100_128x256x32_S32S8S8S32_SS) = MoYe.static((128, 256, 32))
MoYe.shape_mnk(::MMAOP_SM100_128x256x32_S32U8U8S32_SS) = MoYe.static((128, 256, 32))
MoYe.shape_mnk(::MMAOP_SM100_128x256x32_F32E4M3E4M3F32_SS) = MoYe.static((128, 256, 32))
MoYe.shape_mnk(::MMAOP_SM100_128x256x8_F32TF32TF32F32_SS) = MoYe.static((128, 256, 8))

# ---- descriptor flattening: layout(x) -> (shape, stride) of a rank-2 view, 0-based element strides
function moye_tensor(x::MoYeArray{T}) where {T}
    l = layout(x)
    rank(l) == 2 || error("libmoye_b200 takes rank-2 arrays")
    m1, m2 = coalesce(l[1]), coalesce(l[2])
    (rank(m1) == 1 && rank(m2) == 1) || error("each mode must be describable by one stride")
    MoyeTensor(Ptr{Cvoid}(UInt(pointer(x))), moye_dtype(T), Int32(2),
               (Int64(shape(m1)), Int64(shape(m2)), 0, 0), (Int64(stride(m1)), Int64(stride(m2)), 0, 0))
end

const MOYE_B200_VERSION = 100   # MOYE_B200_VERSION of the header this file was written against
const handles = Dict{Tuple{Int, Int}, Ptr{Cvoid}}()
function handle()
    key = (Threads.threadid(), CUDA.deviceid(CUDA.device()))
    get!(handles, key) do
        v = ccall((:moye_b200_version, libmoye_b200[]), Cint, ())
        v == MOYE_B200_VERSION || error("libmoye_b200 is version $v, this binding expects $MOYE_B200_VERSION")
        h = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:moye_b200_create, libmoye_b200[]), Cint, (Ref{Ptr{Cvoid}},), h))
        h[]
    end
end
# one handle per (thread, device) for the life of the process; released at exit (scratch buffers, events, tensor-map cache)
function destroy_handles()
    for (_, h) in handles
        ccall((:moye_b200_destroy, libmoye_b200[]), Cint, (Ptr{Cvoid},), h)
    end
    empty!(handles)
end
check(rc) = rc == 0 ? nothing :
    error("libmoye_b200 ($rc): " * unsafe_string(ccall((:moye_b200_last_error, libmoye_b200[]), Cstring, ())))

# ---- gemm!(tiled_mma, D, A, B, C): replaces the whole matmul_kernel of examples/gemm.jl:4-64
# `tile_n = 0` leaves the tile width and the kernel (single CTAs, CTA pairs, 256 x 512 pair tiles with a K-split
# tail, split-K clusters, stream-K for decode shapes) to the library; pass the atom's N (`tile_size(mma, _2)`) to
# pin the tile.  `tail = true / false` overrules the library's choice of the K-split tail.
function MoYe.gemm!(mma::TiledMMA{<:MoYe.MMAAtom{<:MoYe.MMATraits{<:AbstractSM100MMAOP}}},
                    D::MoYeArray, A::MoYeArray, B::MoYeArray, C::Union{MoYeArray, Nothing} = nothing;
                    alpha = 1, beta = 0, scale_a = 1f0, scale_b = 1f0, stream = CUDA.stream(),
                    bias::Union{CuVector{Float32}, Nothing} = nothing, bias_along = :col, activation = nothing,
                    tile_n = 0, path = 0, split_k = 0, allow_tf32 = false, tail = nothing)
    all(MoYe.isgmem, (D, A, B)) || error("host-level gemm! needs global-memory arrays (no CPU fallback)")
    # fused epilogue D = act(alpha*A*B' + beta*C + bias): bias[n] (:col) or bias[m] (:row)
    flags = EPI_ACT[activation] | (bias === nothing ? 0 : (bias_along === :col ? EPI_BIAS_COL : EPI_BIAS_ROW))
    flags |= allow_tf32 ? GEMM_ALLOW_TF32 : 0
    flags |= tail === nothing ? 0 : (tail ? GEMM_TAIL_ON : GEMM_TAIL_OFF)
    bptr = bias === nothing ? C_NULL : Ptr{Cvoid}(UInt(pointer(bias)))
    p = Ref(MoyeGemmParams(alpha, beta, scale_a, scale_b, Int32(tile_n), Int32(split_k), Int32(path), Int32(flags), bptr))
    tD, tA, tB = Ref(moye_tensor(D)), Ref(moye_tensor(A)), Ref(moye_tensor(B))
    tC = (C === nothing || iszero(beta)) ? C_NULL : Ref(moye_tensor(C))
    check(ccall((:moye_b200_gemm, libmoye_b200[]), Cint,
                (Ptr{Cvoid}, Ref{MoyeTensor}, Ref{MoyeTensor}, Ref{MoyeTensor}, Ptr{Cvoid}, Ref{MoyeGemmParams}, Ptr{Cvoid}),
                handle(), tD, tA, tB, tC, p, stream.handle))
    return D
end

# ---- axpby!(a, X, b, Y) on global-memory arrays (src/algorithm/blas.jl:1-9): Y = a*X + b*Y
function MoYe.axpby!(a::Number, X::MoYeArray{T, N, ViewEngine{T, CuPtr{T}}}, b::Number,
                     Y::MoYeArray{T, N, ViewEngine{T, CuPtr{T}}}; stream = CUDA.stream()) where {T, N}
    check(ccall((:moye_b200_axpby, libmoye_b200[]), Cint,
                (Ptr{Cvoid}, Ref{MoyeTensor}, Ref{MoyeTensor}, Cfloat, Cfloat, Ptr{Cvoid}),
                handle(), Ref(moye_tensor(Y)), Ref(moye_tensor(X)), Float32(a), Float32(b), stream.handle))
    return Y
end

# ---- Swizzle{B,M,S}: the XOR functor MoYe's README lists as missing (README.md:14-17); composes with a layout
struct Swizzle{B, M, S} end
Swizzle(b::Int, m::Int, s::Int) = Swizzle{b, m, s}()
function (::Swizzle{B, M, S})(offset0::Integer) where {B, M, S}
    mask = ((1 << B) - 1) << (M + S)
    return offset0 ⊻ ((offset0 & mask) >> S)
end
struct ComposedLayout{SW <: Swizzle, L <: Layout}
    swizzle::SW
    offset::Int
    layout::L
end
Base.:∘(sw::Swizzle, l::Layout) = ComposedLayout(sw, 0, l)
MoYe.composition(sw::Swizzle, l::Layout) = ComposedLayout(sw, 0, l)
(c::ComposedLayout)(coord...) = c.swizzle(c.layout(coord...) - 1 + c.offset) + 1     # 1-based like Layout
MoYe.shape(c::ComposedLayout) = shape(c.layout)
Base.size(c::ComposedLayout) = size(c.layout)
"The shared-memory operand stage TMA writes and tcgen05.mma reads: (row, k) -> byte offset, 128-byte swizzle."
umma_smem_layout(::Type{T}, rows::Int) where {T} =
    Swizzle(3, 4, 3) ∘ MoYe.make_layout((rows, 128 ÷ sizeof(T)), (128, sizeof(T)))

# ---- several GPUs, one process (or task) per GPU: NCCL behind the same C ABI
"128-byte NCCL id made by rank 0; hand it to the other ranks over any host channel (MPI.bcast, a file, a socket)."
function comm_unique_id()
    id = Vector{UInt8}(undef, 128)
    check(ccall((:moye_b200_comm_unique_id, libmoye_b200[]), Cint, (Ptr{UInt8},), id))
    return id
end
comm_init(rank::Integer, world::Integer, id::Vector{UInt8}) =
    check(ccall((:moye_b200_comm_init, libmoye_b200[]), Cint, (Ptr{Cvoid}, Int32, Int32, Ptr{UInt8}), handle(), rank, world, id))
comm_destroy() = check(ccall((:moye_b200_comm_destroy, libmoye_b200[]), Cint, (Ptr{Cvoid},), handle()))
"Every rank's block of `full` along `mode` (1 or 2, MoYe counts from 1) ends up in every rank's `full`."
function allgather!(full::MoYeArray, shard::MoYeArray; mode = 2, align = 1, stream = CUDA.stream())
    check(ccall((:moye_b200_allgather, libmoye_b200[]), Cint,
                (Ptr{Cvoid}, Ref{MoyeTensor}, Ref{MoyeTensor}, Int32, Int64, Ptr{Cvoid}),
                handle(), Ref(moye_tensor(shard)), Ref(moye_tensor(full)), Int32(mode - 1), Int64(align), stream.handle))
    return full
end
function bcast!(x::MoYeArray, root::Integer = 0; stream = CUDA.stream())
    check(ccall((:moye_b200_bcast, libmoye_b200[]), Cint, (Ptr{Cvoid}, Ref{MoyeTensor}, Int32, Ptr{Cvoid}),
                handle(), Ref(moye_tensor(x)), Int32(root), stream.handle))
    return x
end
"Rows (or columns) [lo, hi) of rank `rank` (0-based) when `extent` is cut into `world` blocks of multiples of `align`."
function shard_range(extent::Integer, world::Integer, rank::Integer, align::Integer = 1)
    units = cld(extent, align)
    return min(units * rank ÷ world * align, extent) + 1, min(units * (rank + 1) ÷ world * align, extent)
end

# ---- copyto!(tiled_copy, dst, src): replaces copy_kernel of test/host/copy_async.jl:3-25
function Base.copyto!(tc::TiledCopy, dst::MoYeArray{T, 2, ViewEngine{T, CuPtr{T}}},
                      src::MoYeArray{T, 2, ViewEngine{T, CuPtr{T}}}; stream = CUDA.stream()) where {T}
    tiler = MoYe.tile_size(tc)
    mode = MoYe.get_traits(tc).copy_op isa CPOP_TMA_LOAD_SW128 ? Int32(2) : Int32(1)
    p = Ref(MoyeCopyParams(mode, Int32(tiler[1]), Int32(max(tiler[2], 64)), 0))
    check(ccall((:moye_b200_copy, libmoye_b200[]), Cint,
                (Ptr{Cvoid}, Ref{MoyeTensor}, Ref{MoyeTensor}, Ref{MoyeCopyParams}, Ptr{Cvoid}),
                handle(), Ref(moye_tensor(dst)), Ref(moye_tensor(src)), p, stream.handle))
    return dst
end

# ---- copyto!(dst, src) on global-memory arrays, each contiguous along one mode.  `copyto!(a, MoYe.transpose(b))`
# replaces transpose_kernel of test/host/copy_async.jl:51-95 (the library picks the transposing kernel).
function Base.copyto!(dst::MoYeArray{T, 2, ViewEngine{T, CuPtr{T}}}, src::MoYeArray{T, 2, ViewEngine{T, CuPtr{T}}};
                      stream = CUDA.stream()) where {T}
    check(ccall((:moye_b200_copy, libmoye_b200[]), Cint,
                (Ptr{Cvoid}, Ref{MoyeTensor}, Ref{MoyeTensor}, Ptr{Cvoid}, Ptr{Cvoid}),
                handle(), Ref(moye_tensor(dst)), Ref(moye_tensor(src)), C_NULL, stream.handle))
    return dst
end

# ---- matmul(A, B, C) of examples/gemm.jl:66-89, on the tcgen05 atom for eltype(A)
function matmul(A::CuMatrix{Float16}, B::CuMatrix{Float16}, C::CuMatrix{Float32})
    # K-major views of row-major storage: pass transposed CuArrays, e.g. A = CuArray(A_host')'
    mma = MoYe.make_tiled_mma(MMAOP_SM100_128x256x16_F32F16F16F32_SS())
    MoYe.gemm!(mma, MoYeArray(C, size(C)), MoYeArray(A, size(A)), MoYeArray(B, size(B)))
end
# the literal examples/gemm.jl:91-96 call: column-major Float32 A (M,K), B (N,K), C (M,N)
function matmul(A::CuMatrix{Float32}, B::CuMatrix{Float32}, C::CuMatrix{Float32}; allow_tf32 = false)
    mma = MoYe.make_tiled_mma(MMAOP_SM100_128x256x8_F32TF32TF32F32_SS())
    MoYe.gemm!(mma, MoYeArray(C, size(C)), MoYeArray(A, size(A)), MoYeArray(B, size(B)); allow_tf32)
end

"Synchronise and surface a device-side bounded-wait failure (moye_b200_status)."
function status(stream = CUDA.stream())
    site = Ref{Int32}(0)
    check(ccall((:moye_b200_status, libmoye_b200[]), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Ref{Int32}), handle(), stream.handle, site))
end

end # module
