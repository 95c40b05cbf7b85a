"""Ops, traits, atoms and tiled atoms: MoYe's L3/L4 layers, extended with Blackwell ops.

Mirrors the reference's naming:
  ops      `MMAOP_<M>x<N>x<K>_<D><A><B><C>_<TN>`  (src/arch/mma/make_mma_ops.jl:355-424),
           `UniversalFMA` (src/arch/mma/mma.jl:53-64), `UniversalCopy{S,D}`
           (src/arch/copy/copy.jl:26-51), `CPOP_ASYNC_CACHEALWAYS` (src/arch/copy/copy_async.jl:8-24)
  traits   thread-id layout and (thread, value) -> coordinate layouts per op
           (src/traits/mma.jl:23-42, src/traits/mma_sm80.jl, src/traits/copy.jl:3-21)
  atoms    `MMAAtom`, `TiledMMA`, `ThrMMA` (src/atom/mma.jl), `CopyAtom`, `TiledCopy`,
           `ThrCopy` (src/atom/copy.jl)

New for sm_100a (what the hot path actually runs on):
  `MMAOP_SM100_128xNx16_F32F16F16F32_SS`, `..._F32BF16BF16F32_SS`  tcgen05.mma kind::f16
  `MMAOP_SM100_128xNx32_S32S8S8S32_SS`                             tcgen05.mma kind::i8
  `MMAOP_SM100_128xNx32_F32E4M3E4M3F32_SS`                         tcgen05.mma kind::f8f6f4
  `MMAOP_SM100_128xNx8_F32TF32TF32F32_SS`                          tcgen05.mma kind::tf32 (Float32 storage)
  `CPOP_TMA_LOAD_SW128`, `CPOP_TMA_STORE`                          cp.async.bulk.tensor
A tcgen05 instruction is issued by ONE thread for the whole CTA tile and accumulates in
tensor memory, so its thread-id layout is `1:0` and its "fragments" are whole tiles.
"""
from . import _lib
from .array import MoYeArray
from .layout import (COLON, Layout, _tup, append_layout, coalesce, composition, cosize, get_congr_coord, logical_divide,
                     make_layout, product_each, raked_product, right_inverse, size, tiled_product, upcast,
                     zipped_divide)

__all__ = [
    "MMAOp", "CopyOp", "UniversalFMA", "UniversalCopy", "CPOP_ASYNC_CACHEALWAYS", "CPOP_TMA_LOAD_SW128",
    "CPOP_TMA_STORE", "MMAAtom", "TiledMMA", "ThrMMA", "make_tiled_mma", "CopyAtom", "TiledCopy", "ThrCopy",
    "make_tiled_copy", "make_tma_tiled_copy", "make_tiled_copy_A", "make_tiled_copy_B", "make_tiled_copy_C", "MMA_OPS", "mma_op",
    "sm100_mma_op", "DTYPE_BITS", "LDSM_OPS", "ldsm_op", "ldsm_tiled_copy_tables",
]

DTYPE_BITS = {_lib.F32: 32, _lib.F16: 16, _lib.BF16: 16, _lib.S8: 8, _lib.U8: 8, _lib.E4M3: 8, _lib.S32: 32,
              _lib.U16: 16, _lib.U32: 32, _lib.U64: 64, _lib.U128: 128}
_TAG = {"F32": _lib.F32, "F16": _lib.F16, "BF16": _lib.BF16, "S8": _lib.S8, "U8": _lib.U8, "S32": _lib.S32,
        "E4M3": _lib.E4M3, "TF32": _lib.F32}


def L(shape, stride=None):
    return Layout(shape, stride)


# ------------------------------------------------------------------------------ MMA ops + traits
class MMAOp:
    """One matrix-multiply instruction: shape, operand types, and its traits
    (`thr_id`, `layout_a/b/c`: (thread, value) -> linear coordinate in the (M,K)/(N,K)/(M,N) tile)."""

    def __init__(self, name, mnk, d, a, b, c, thr_id, layout_a, layout_b, layout_c, arch, kind=None):
        self.name, self.shape_mnk = name, tuple(mnk)
        self.valtype_d, self.valtype_a, self.valtype_b, self.valtype_c = d, a, b, c
        self.thr_id, self.layout_a, self.layout_b, self.layout_c = thr_id, layout_a, layout_b, layout_c
        self.arch, self.kind = arch, kind

    def __repr__(self):
        return self.name


def UniversalFMA(d, a=None, b=None, c=None):
    """The 1x1x1 scalar "atom" `d = a*b + c` (reference src/arch/mma/mma.jl:53-64,
    traits src/traits/mma.jl:38-42)."""
    a, b, c = a if a is not None else d, b if b is not None else d, c if c is not None else d
    one = L((1, 1))
    return MMAOp("UniversalFMA", (1, 1, 1), d, a, b, c, L(1), one, one, one, "any")


def _sm80_layouts(mnk, float_ab):
    """(thread, value) layouts of the warp-level mma.sync shapes (reference src/traits/mma_sm80.jl:1-43)."""
    if mnk == (16, 8, 8):
        a = L(((4, 8), (2, 2)), ((32, 1), (16, 8)))
        return a, L(((4, 8), 2), ((16, 1), 8)), a
    if mnk == (16, 8, 16) and float_ab:
        return (L(((4, 8), (2, 2, 2)), ((32, 1), (16, 8, 128))), L(((4, 8), (2, 2)), ((16, 1), (8, 64))),
                L(((4, 8), (2, 2)), ((32, 1), (16, 8))))
    if mnk in ((16, 8, 16), (16, 8, 32)):
        return (L(((4, 8), (4, 2, 2)), ((64, 1), (16, 8, 256))), L(((4, 8), (4, 2)), ((32, 1), (8, 128))),
                L(((4, 8), (2, 2)), ((32, 1), (16, 8))))
    if mnk == (8, 8, 16):
        a = L(((4, 8), 4), ((32, 1), 8))
        return a, a, L(((4, 8), 2), ((16, 1), 8))
    raise KeyError(mnk)


MMA_OPS = {}


def _register_sm80():
    names = [
        ("MMAOP_16x8x8_F16F16F16F16_TN", (16, 8, 8), "F16", "F16", "F16", "F16"),
        ("MMAOP_16x8x8_F32F16F16F32_TN", (16, 8, 8), "F32", "F16", "F16", "F32"),
        ("MMAOP_16x8x8_F32BF16BF16F32_TN", (16, 8, 8), "F32", "BF16", "BF16", "F32"),
        ("MMAOP_16x8x16_F16F16F16F16_TN", (16, 8, 16), "F16", "F16", "F16", "F16"),
        ("MMAOP_16x8x16_F32F16F16F32_TN", (16, 8, 16), "F32", "F16", "F16", "F32"),
        ("MMAOP_16x8x16_F32BF16BF16F32_TN", (16, 8, 16), "F32", "BF16", "BF16", "F32"),
        ("MMAOP_16x8x16_S32S8S8S32_TN", (16, 8, 16), "S32", "S8", "S8", "S32"),
        ("MMAOP_16x8x32_S32S8S8S32_TN", (16, 8, 32), "S32", "S8", "S8", "S32"),
        ("MMAOP_8x8x16_S32S8S8S32_TN", (8, 8, 16), "S32", "S8", "S8", "S32"),
    ]
    for name, mnk, d, a, b, c in names:
        la, lb, lc = _sm80_layouts(mnk, a in ("F16", "BF16"))
        if name == "MMAOP_8x8x16_S32S8S8S32_TN":
            lb = L(((4, 8), 2), ((32, 1), 8))  # reference src/traits/mma_sm80.jl:104-111 special case
        MMA_OPS[name] = MMAOp(name, mnk, _TAG[d], _TAG[a], _TAG[b], _TAG[c], L(32), la, lb, lc, "sm_80")
    # the tf32 warp ops of the tensor-core manual (reference src/traits/mma_sm80.jl:104-111): Float32 storage
    f32 = _lib.F32
    MMA_OPS["MMAOP_16x8x8_F32TF32TF32F32_TN"] = MMAOp(
        "MMAOP_16x8x8_F32TF32TF32F32_TN", (16, 8, 8), f32, f32, f32, f32, L(32),
        L(((4, 8), (2, 2)), ((16, 1), (8, 64))), L(((4, 8), 2), ((8, 1), 32)), L(((4, 8), (2, 2)), ((32, 1), (16, 8))), "sm_80")
    MMA_OPS["MMAOP_16x8x4_F32TF32TF32F32_TN"] = MMAOp(
        "MMAOP_16x8x4_F32TF32TF32F32_TN", (16, 8, 4), f32, f32, f32, f32, L(32),
        L(((4, 8), 2), ((16, 1), 8)), L(((4, 8), 1), ((8, 1), 8)), L(((4, 8), (2, 2)), ((32, 1), (16, 8))), "sm_80")


_register_sm80()


def sm100_mma_op(ab, n=256):
    """The tcgen05 op for operand type `ab` ("F16", "BF16", "S8", "U8", "E4M3", or "TF32" for Float32
    storage read with a 10-bit mantissa) and tile N.
    One instruction covers 128 x n x K (K = 32 bytes of the operand type); one thread issues
    it and the accumulator lives in tensor memory, hence thr_id = 1:0 and value layouts that
    span the whole tile."""
    acc = "S32" if ab in ("S8", "U8") else "F32"
    k = 16 if ab in ("F16", "BF16") else (8 if ab == "TF32" else 32)
    kind = {"F16": "kind::f16", "BF16": "kind::f16", "S8": "kind::i8", "U8": "kind::i8", "E4M3": "kind::f8f6f4",
            "TF32": "kind::tf32"}[ab]
    name = f"MMAOP_SM100_128x{n}x{k}_{acc}{ab}{ab}{acc}_SS"
    if name not in MMA_OPS:
        MMA_OPS[name] = MMAOp(name, (128, n, k), _TAG[acc], _TAG[ab], _TAG[ab], _TAG[acc], L(1),
                              L((1, (128, k))), L((1, (n, k))), L((1, (128, n))), "sm_100a", kind)
    return MMA_OPS[name]


for _ab in ("F16", "BF16", "S8", "U8", "E4M3", "TF32"):
    for _n in (64, 128, 256):
        sm100_mma_op(_ab, _n)


def mma_op(name):
    return MMA_OPS[name]


class MMAAtom:
    """reference src/atom/mma.jl:26-47."""

    def __init__(self, op):
        self.op = op

    def __getattr__(self, k):
        return getattr(self.op, k)


class TiledMMA:
    """`TiledMMA{Atom, AtomLayoutMNK, PermutationMNK}` (reference src/atom/mma.jl:80-107)."""

    def __init__(self, atom, atom_layout_mnk, permutation_mnk):
        self.atom, self.atom_layout_mnk, self.permutation_mnk = atom, atom_layout_mnk, permutation_mnk

    @property
    def thr_layout_vmnk(self):
        """(thr_id, atom_M, atom_N, atom_K) -> thread index (reference src/atom/mma.jl:115-118)."""
        return tiled_product(self.atom.thr_id, self.atom_layout_mnk)

    def __len__(self):
        return size(self.thr_layout_vmnk)

    def tile_size(self, i):
        """Extent of the CTA tile along mode i (0 = M, 1 = N, 2 = K) (reference src/atom/mma.jl:178-189)."""
        core = self.atom.shape_mnk[i] * size(self.thr_layout_vmnk, i + 1)
        p = self.permutation_mnk[i]
        if p == COLON:
            return core
        return max(core, size(p) if isinstance(p, Layout) else p)

    def tile_shape(self):
        return tuple(self.tile_size(i) for i in range(3))

    def _thrfrg(self, x, m0, m1, tv_layout):
        a_mnk, t_vmnk = self.atom.shape_mnk, self.thr_layout_vmnk
        perm = (self.permutation_mnk[m0], self.permutation_mnk[m1])
        t = logical_divide(x, perm)
        a = zipped_divide(t, (make_layout(a_mnk[m0]), make_layout(a_mnk[m1])))
        tv = composition(a, (tv_layout, COLON))
        thr_tile = (COLON, (make_layout(size(t_vmnk, m0 + 1)), make_layout(size(t_vmnk, m1 + 1))))
        return zipped_divide(tv, thr_tile)

    def thrfrg_C(self, c):
        """((thr, (atom_M, atom_N)), (val, (rest_M, rest_N))) (reference src/atom/mma.jl:120-137)."""
        return self._thrfrg(c, 0, 1, self.atom.layout_c)

    def thrfrg_A(self, a):
        return self._thrfrg(a, 0, 2, self.atom.layout_a)

    def thrfrg_B(self, b):
        return self._thrfrg(b, 1, 2, self.atom.layout_b)

    def get_slice(self, thr_idx):
        return ThrMMA(self, get_congr_coord(self.thr_layout_vmnk, thr_idx))

    def _layout_tv(self, which):
        ts = self.tile_shape()
        thr = self.thr_layout_vmnk
        inv = right_inverse(thr)
        if which == "C":
            tv = self.thrfrg_C(make_layout((ts[0], ts[1])))
            return composition(tv, (inv, COLON))
        if which == "A":
            tv = self.thrfrg_A(make_layout((ts[0], ts[2])))
            tile = (COLON, (make_layout((size(thr, 1), size(thr, 2)), (1, 0)), COLON))
        else:
            tv = self.thrfrg_B(make_layout((ts[1], ts[2])))
            tile = (COLON, (make_layout((size(thr, 1), size(thr, 2)), (0, 1)), COLON))
        return composition(composition(tv, (tile, COLON)), (inv, COLON))

    def _layout_mn(self, which):
        """(layout over the tile -> index into (thr, val), thread-id layout) (reference src/atom/mma.jl:236-262)."""
        ts, thr = self.tile_shape(), self.thr_layout_vmnk
        if which == "C":
            ref, tv, thrid = make_layout((ts[0], ts[1])), self.thrfrg_C, thr(COLON, COLON, COLON, 1)
        elif which == "A":
            ref, tv, thrid = make_layout((ts[0], ts[2])), self.thrfrg_A, thr(COLON, COLON, 1, COLON)
        else:
            ref, tv, thrid = make_layout((ts[1], ts[2])), self.thrfrg_B, thr(COLON, 1, COLON, COLON)
        return composition(right_inverse(tv(ref)), make_layout(ref.shape)), thrid

    def get_layoutC_MN(self):
        return self._layout_mn("C")

    def get_layoutA_MK(self):
        return self._layout_mn("A")

    def get_layoutB_NK(self):
        return self._layout_mn("B")

    def get_layoutA_TV(self):
        return self._layout_tv("A")

    def get_layoutB_TV(self):
        return self._layout_tv("B")

    def get_layoutC_TV(self):
        return self._layout_tv("C")

    def __repr__(self):
        return f"TiledMMA({self.atom.op.name}, thr_vmnk={self.thr_layout_vmnk}, perm={self.permutation_mnk})"


class ThrMMA:
    """One thread's slice of a TiledMMA (reference src/atom/mma.jl:100-107,292-304)."""

    def __init__(self, tiled_mma, thr_vmnk):
        self.tiled_mma, self.thr_vmnk = tiled_mma, _tup(thr_vmnk)

    def _partition(self, x, frg, i0, i1):
        arr = MoYeArray(x, frg(x.layout))
        coord = (self.thr_vmnk[0], (self.thr_vmnk[i0], self.thr_vmnk[i1]))
        rest = len(arr.layout[1][1])
        return arr.view((coord, (COLON, (COLON,) * rest)))

    def partition_C(self, c):
        return self._partition(c, self.tiled_mma.thrfrg_C, 1, 2)

    def partition_A(self, a):
        return self._partition(a, self.tiled_mma.thrfrg_A, 1, 3)

    def partition_B(self, b):
        return self._partition(b, self.tiled_mma.thrfrg_B, 2, 3)


def make_tiled_mma(op, atom_layout=None, permutations=(COLON, COLON, COLON)):
    """reference src/atom/mma.jl:193-199,229-233: the K mode of the atom layout is padded with 1:0."""
    atom = op if isinstance(op, MMAAtom) else MMAAtom(op)
    atom_layout = atom_layout if atom_layout is not None else make_layout((1, 1, 1))
    perms = tuple(permutations) + (COLON,) * (3 - len(permutations))
    return TiledMMA(atom, append_layout(atom_layout, 3), perms)


# ------------------------------------------------------------------------------ copy ops + atoms
class CopyOp:
    """A copy instruction with its traits in BITS: `thr_id`, and (thread, bit) layouts of
    source, destination and reference (reference src/traits/copy.jl:3-21)."""

    def __init__(self, name, thr_id, src_bits, dst_bits, ref_bits=None, mode=None):
        self.name, self.thr_id = name, thr_id
        self.src_bits, self.dst_bits, self.ref_bits = src_bits, dst_bits, ref_bits or src_bits
        self.mode = mode  # the moye_copy_mode_t a device-level copyto! runs this op with

    def __repr__(self):
        return self.name


def UniversalCopy(src_bits, dst_bits=None):
    """`UniversalCopy{S,D}`: one thread moves sizeof(S) bytes with one load and one store
    (reference src/arch/copy/copy.jl:26-51, traits src/traits/copy.jl:16-21).  128 bits is
    the widest: `UniversalCopy(128)` is MoYe's `UniversalCopy{UInt128}`."""
    dst_bits = dst_bits or src_bits
    return CopyOp(f"UniversalCopy{{{src_bits}b,{dst_bits}b}}", L(1), L((1, src_bits)), L((1, dst_bits)),
                  mode=_lib.COPY_UNIVERSAL128 if src_bits == 128 else None)


def CPOP_ASYNC_CACHEALWAYS(bits):
    """`cp.async.ca` of 4/8/16 bytes (reference src/arch/copy/copy_async.jl:8-24, traits
    src/traits/cp_async.jl:2-7).  On sm_100a a device-level copy through this op is served by the
    128-bit kernel when it moves 16 bytes."""
    if bits not in (32, 64, 128):
        raise ValueError("cp.async moves 4, 8 or 16 bytes")
    return CopyOp(f"CPOP_ASYNC_CACHEALWAYS{{{bits}b}}", L(1), L((1, bits)), L((1, bits)),
                  mode=_lib.COPY_UNIVERSAL128 if bits == 128 else None)


def _ldsm(name, src, dst):
    op = CopyOp(name, L(32), src, dst, dst, mode=_lib.COPY_LDSM)
    op.matrices = int(name[name.index("x") + 1]) // (2 if name.endswith("_T") else 1)   # x1 / x2 / x4 of the instruction
    op.transposed = name.endswith("_T")
    return op


# ldmatrix ops: 32 threads move 1 / 2 / 4 8x8 b16 matrices from shared memory to registers, optionally
# transposed.  Bit-level (thread, bit) layouts as in reference src/traits/ldmatrix.jl:1-41 (ops:
# src/arch/copy/ldmatrix.jl:18-48).  tcgen05 reads its operands straight from shared-memory descriptors,
# so the GEMM kernels do not issue ldmatrix; a TiledCopy built on these ops (reference test/copy.jl:152-157,
# docs/src/manual/tensor_core.md) partitions exactly as in MoYe, and `copyto_(tiled_copy, dst, src)` runs it on
# the device as the reference's test kernel does (test/device/tiled_copy.jl:2-23, `ldsm_tiled_copy_tables`).
LDSM_OPS = {
    "LDSM_U32x1_N": _ldsm("LDSM_U32x1_N", L(((8, 4), 128), ((128, 0), 1)), L((32, 32), (32, 1))),
    "LDSM_U32x2_N": _ldsm("LDSM_U32x2_N", L(((16, 2), 128), ((128, 0), 1)), L((32, (32, 2)), (32, (1, 1024)))),
    "LDSM_U32x4_N": _ldsm("LDSM_U32x4_N", L((32, 128), (128, 1)), L((32, (32, 4)), (32, (1, 1024)))),
    "LDSM_U16x2_T": _ldsm("LDSM_U16x2_T", L(((8, 4), 128), ((128, 0), 1)),
                          L(((4, 8), (16, 2)), ((256, 16), (1, 128)))),
    "LDSM_U16x4_T": _ldsm("LDSM_U16x4_T", L(((16, 2), 128), ((128, 0), 1)),
                          L(((4, 8), (16, 2, 2)), ((256, 16), (1, 128, 1024)))),
    "LDSM_U16x8_T": _ldsm("LDSM_U16x8_T", L((32, 128), (128, 1)),
                          L(((4, 8), (16, 2, 4)), ((256, 16), (1, 128, 1024)))),
}


def ldsm_op(name):
    return LDSM_OPS[name]


def CPOP_TMA_LOAD_SW128(tile_bits):
    """cp.async.bulk.tensor load of a whole tile by one thread into 128B-swizzled smem."""
    return CopyOp("CPOP_TMA_LOAD_SW128", L(1), L((1, tile_bits)), L((1, tile_bits)), mode=_lib.COPY_TMA)


def CPOP_TMA_STORE(tile_bits):
    """cp.async.bulk.tensor store of a whole smem tile by one thread."""
    return CopyOp("CPOP_TMA_STORE", L(1), L((1, tile_bits)), L((1, tile_bits)), mode=_lib.COPY_TMA)


class CopyAtom:
    """`CopyAtom{Traits,T}`: the op's bit layouts upcast to values of T
    (reference src/atom/copy.jl:31-53)."""

    def __init__(self, op, dtype):
        bits = DTYPE_BITS[dtype]
        self.op, self.dtype = op, dtype
        self.thr_id = op.thr_id
        self.val_layout_src = upcast(op.src_bits, bits)
        self.val_layout_dst = upcast(op.dst_bits, bits)
        self.val_layout_ref = upcast(op.ref_bits, bits)
        for l in (self.val_layout_src, self.val_layout_dst, self.val_layout_ref):
            if size(l, 0) != size(self.thr_id):
                raise ValueError("thread counts of the op's layouts disagree")
        self.num_val_src = size(self.val_layout_src, 1)
        self.num_val_dst = size(self.val_layout_dst, 1)


class TiledCopy:
    """`TiledCopy(atom, layout_TV, tiler_MN)` (reference src/atom/copy.jl:86-125)."""

    def __init__(self, atom, tiled_layout_tv, tiler_mn):
        if size(tiled_layout_tv, 0) % size(atom.val_layout_ref, 0) or \
           size(tiled_layout_tv, 1) % size(atom.val_layout_ref, 1):
            raise ValueError("the tiled (thr, val) layout is not a multiple of the atom's")
        self.copy_atom, self.tiled_layout_tv, self.tiler_mn = atom, tiled_layout_tv, tuple(tiler_mn)

    def __len__(self):
        return size(self.tiled_layout_tv, 0)

    def tile_size(self):
        return self.tiler_mn

    def _tile2thrfrg(self, x, ref2trg):
        """reference src/atom/copy.jl:127-135."""
        atom = self.copy_atom
        nthr, nval = size(atom.val_layout_ref, 0), size(atom.val_layout_ref, 1)
        atom_tv = zipped_divide(self.tiled_layout_tv, (nthr, nval))
        trg_tv = composition(atom_tv, (ref2trg, COLON))
        zipped = Layout(tuple(zip(_tup(trg_tv.shape[0]), _tup(trg_tv.shape[1]))),
                        tuple(zip(_tup(trg_tv.stride[0]), _tup(trg_tv.stride[1]))))
        thrval2mn = coalesce(zipped, (1, (1, 1)))
        tv = composition(x, (thrval2mn, COLON))
        return Layout(_tup(tv.shape[0]) + (tv.shape[1],), _tup(tv.stride[0]) + (tv.stride[1],))

    def tidfrg_S(self, src):
        a = self.copy_atom
        return self._tile2thrfrg(zipped_divide(src, self.tiler_mn),
                                 composition(right_inverse(a.val_layout_ref), a.val_layout_src))

    def tidfrg_D(self, dst):
        a = self.copy_atom
        return self._tile2thrfrg(zipped_divide(dst, self.tiler_mn),
                                 composition(right_inverse(a.val_layout_ref), a.val_layout_dst))

    def _layout_tv_of(self, val_layout):
        """(thr, val) -> offset in the tile (reference src/atom/copy.jl:168-174,184-190)."""
        ref = make_layout((self.tiler_mn, 1))
        tv = self._tile2thrfrg(ref, composition(right_inverse(self.copy_atom.val_layout_ref), val_layout))
        return tv(COLON, COLON, 1)

    def get_layoutS_TV(self):
        return self._layout_tv_of(self.copy_atom.val_layout_src)

    def get_layoutD_TV(self):
        return self._layout_tv_of(self.copy_atom.val_layout_dst)

    def _layout_mn_of(self, tv):
        return composition(right_inverse(tv), make_layout(self.tiler_mn)), make_layout(size(self.tiled_layout_tv, 0))

    def get_layoutS_MN(self):
        """(layout over the tile -> index into (thr, val), thread-id layout) (reference src/atom/copy.jl:176-182)."""
        return self._layout_mn_of(self.get_layoutS_TV())

    def get_layoutD_MN(self):
        return self._layout_mn_of(self.get_layoutD_TV())

    def get_slice(self, thr_idx):
        return ThrCopy(self, thr_idx)

    def __repr__(self):
        return f"TiledCopy({self.copy_atom.op.name}, tv={self.tiled_layout_tv}, tiler={self.tiler_mn})"


class ThrCopy:
    """reference src/atom/copy.jl:198-214."""

    def __init__(self, tiled_copy, thr_idx):
        self.tiled_copy, self.thr_idx = tiled_copy, thr_idx

    def _partition(self, x, frg):
        arr = MoYeArray(x, frg(x.layout))
        n = len(x.layout)
        return arr.view((self.thr_idx, COLON, (COLON,) * n))

    def partition_S(self, s):
        return self._partition(s, self.tiled_copy.tidfrg_S)

    def partition_D(self, d):
        return self._partition(d, self.tiled_copy.tidfrg_D)


def ldsm_tiled_copy_tables(tiled_copy, tile_layout):
    """What every thread of an ldmatrix TiledCopy does to a tile with layout `tile_layout` (16-bit elements), as
    two tables of 0-based element offsets: `src[t][i]`, the first value of thread t's i-th source fragment in
    `partition_S(thr_copy, tile)`, and `dst[t][i][v]`, where the v-th value it receives lands in
    `partition_D(thr_copy, tile)` -- the `copyto!(tiled_copy, tXrX, tXsX); copyto!(tXgX, tXrX)` of the reference's
    test kernel (test/device/tiled_copy.jl:13-20).  Returns (span, iters, src, dst) with lists of ints."""
    import torch
    atom = tiled_copy.copy_atom
    nsrc, ndst = atom.num_val_src, atom.num_val_dst
    span = int(cosize(tile_layout))
    tile = MoYeArray(torch.zeros(1, dtype=torch.int16), tile_layout)
    src, dst, iters = [], [], None
    for t in range(1, len(tiled_copy) + 1):
        thr = tiled_copy.get_slice(t)
        s, d = thr.partition_S(tile), thr.partition_D(tile)
        n_s, n_d = size(s.layout), size(d.layout)
        if n_s % nsrc or n_d % ndst or n_s // nsrc != n_d // ndst:
            raise ValueError("source and destination partitions disagree on the number of atoms")
        iters = n_s // nsrc
        for i in range(iters):
            first = s.offset + s.layout(i * nsrc + 1) - 1
            if any(s.offset + s.layout(i * nsrc + v + 1) - 1 != first + v for v in range(nsrc)):
                raise ValueError(f"thread {t}: the {nsrc} values of a source fragment are not contiguous in the tile")
            src.append(first)
            dst.extend(d.offset + d.layout(i * ndst + v + 1) - 1 for v in range(ndst))
    return span, iters, src, dst


def make_tiled_copy(copy_atom, thr_layout, val_layout=None):
    """reference src/atom/copy.jl:249-258: `layout_mn = raked_product(thr, val)`, its right
    inverse gives (thr, val) -> (m, n); the tiler is the per-mode extent of layout_mn."""
    val_layout = val_layout if val_layout is not None else make_layout(1)
    layout_mn = raked_product(thr_layout, val_layout, True)
    layout_tv = composition(right_inverse(layout_mn), make_layout((size(thr_layout), size(val_layout))))
    return TiledCopy(copy_atom, layout_tv, product_each(_tup(layout_mn.shape)))


def make_tma_tiled_copy(dtype, tile=(128, 64), store=False):
    """A TiledCopy whose single thread moves one whole `tile` with one TMA instruction:
    thread layout 1, value layout = the tile."""
    bits = DTYPE_BITS[dtype] * tile[0] * tile[1]
    op = CPOP_TMA_STORE(bits) if store else CPOP_TMA_LOAD_SW128(bits)
    return make_tiled_copy(CopyAtom(op, dtype), make_layout(1), make_layout(tuple(tile)))


def make_tiled_copy_A(copy_atom, tiled_mma):
    return TiledCopy(copy_atom, tiled_mma.get_layoutA_TV(), (tiled_mma.tile_size(0), tiled_mma.tile_size(2)))


def make_tiled_copy_B(copy_atom, tiled_mma):
    return TiledCopy(copy_atom, tiled_mma.get_layoutB_TV(), (tiled_mma.tile_size(1), tiled_mma.tile_size(2)))


def make_tiled_copy_C(copy_atom, tiled_mma):
    return TiledCopy(copy_atom, tiled_mma.get_layoutC_TV(), (tiled_mma.tile_size(0), tiled_mma.tile_size(1)))
