"""Host-side logic of the product package against the oracle and the reference's goldens:
layout algebra (structure on static layouts, values everywhere), MoYeArray tiling views,
TiledCopy / TiledMMA partitioning (reference test/copy.jl:102-145, test/tiled_mma.jl:12-39)."""
import json
import os

import numpy as np
import pytest
import torch

import layout_oracle as lo

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def tt(x):
    return tuple(tt(e) for e in x) if isinstance(x, (list, tuple)) else int(x)


def same(pl, ol):
    """product layout == oracle layout, structurally."""
    return tt(pl.shape) == tt(lo.dynamic(ol.shape)) and tt(pl.stride) == tt(lo.dynamic(ol.stride))


SHAPES = [
    ((2, (1, 6)), (1, (6, 2))), ((4, 3), (3, 1)), ((8, 8), (8, 1)), (((2, 2, 2), (2, 2, 2)), ((1, 16, 4), (8, 2, 32))),
    ((2, 4, 6), (4, 1, 8)), ((4, 8, 2), (2, 8, 1)), (12, 2), ((3, 7), (0, 0)), ((2, 4, 4, 6), (4, 1, 0, 8)),
    ((8, (4, 2), 16), (3, (100, 7), 1000)), ((2, 1, 6), (1, 6, 2)), (((4, 2),), ((1, 16),)),
]


@pytest.mark.parametrize("shape,stride", SHAPES)
def test_unary_ops_match_oracle(mb, shape, stride):
    P, O = mb.make_layout(shape, stride), lo.SL(shape, stride)
    n = int(lo.size(O))
    assert mb.size(P) == n and mb.cosize(P) == int(lo.cosize(O))
    assert [P(i) for i in range(1, n + 1)] == [int(O(i)) for i in range(1, n + 1)]
    assert same(mb.coalesce(P), lo.coalesce(O))
    assert same(mb.filter_layout(P), lo.lfilter(O))
    assert same(mb.right_inverse(P), lo.right_inverse(O))
    try:
        oc = lo.complement(O)
    except AssertionError:
        oc = None
    if oc is not None:
        assert same(mb.complement(P), oc)
        assert same(mb.complement(P, 4 * int(lo.cosize(O))), lo.complement(O, lo.S(4 * int(lo.cosize(O)))))


BINARY = [
    (((4, 3), (3, 1)), ((6, 2), (2, 1))), (((8, 8), (8, 1)), (((2, 2, 2), (2, 2, 2)), ((1, 16, 4), (8, 2, 32)))),
    (((4, 8, 2), (2, 8, 1)), ((2, 2, 2), (1, 8, 2))), ((20, 2), ((4, 5), (1, 4))), ((20, 2), ((4, 5), (5, 1))),
    (((12,), (2,)), ((4, 3), (3, 1))), (((4, 3), (1, 4)), ((2, 3), (2, 4))),
    (((128, 24, 5), (1, 128, 3072)), (64, 2)), (((128, 24, 5), (1, 128, 3072)), (480, 32)),
]


@pytest.mark.parametrize("a,b", BINARY)
def test_composition_matches_oracle(mb, a, b):
    PA, PB = mb.make_layout(*a), mb.make_layout(*b)
    OA, OB = lo.SL(*a), lo.SL(*b)
    pc, oc = mb.composition(PA, PB), lo.composition(OA, OB)
    assert same(pc, oc)
    assert all(pc(i) == PA(PB(i)) for i in range(1, mb.size(pc) + 1))
    assert (PA @ PB) == pc


def test_products_and_divides_match_oracle_and_goldens(mb):
    tile, mot = mb.make_layout((2, 2), (1, 2)), mb.make_layout((3, 4), (4, 1))
    otile, omot = lo.SL((2, 2), (1, 2)), lo.SL((3, 4), (4, 1))
    for name in ("logical_product", "zipped_product", "tiled_product"):
        assert same(getattr(mb, name)(tile, mot), getattr(lo, name)(otile, omot))
    for name in ("blocked_product", "raked_product"):
        for co in (False, True):
            assert same(getattr(mb, name)(tile, mot, co), getattr(lo, name)(otile, omot, co))
    # reference test/layout.jl:485-495 goldens, directly
    assert mb.blocked_product(tile, mot, True) == mb.make_layout(((2, 3), 8), ((1, 16), 2))
    assert mb.raked_product(tile, mot, True) == mb.make_layout(((3, 2), (4, 2)), ((16, 1), (4, 2)))
    raked = mb.raked_product(tile, mot)
    sub = (mb.make_layout(2, 3), mb.make_layout(2, 4))
    # reference test/layout.jl:524-531,610-617
    assert mb.logical_divide(mb.make_layout(16, 3), mb.make_layout(4, 2)) == mb.make_layout((4, (2, 2)), (6, (3, 24)))
    assert mb.logical_divide(raked, sub) == mb.make_layout(((2, 3), (2, 4)), ((1, 16), (2, 4)))
    assert mb.zipped_divide(raked, sub) == mb.make_layout(((2, 2), (3, 4)), ((1, 2), (16, 4)))
    assert mb.tiled_divide(raked, sub) == mb.make_layout(((2, 2), 3, 4), ((1, 2), 16, 4))
    assert mb.zipped_divide(mb.make_layout((256, 256)), (128, 8)) == \
        mb.make_layout(((128, 8), (2, 32)), ((1, 256), (128, 2048)))
    assert same(mb.tile_to_shape(mb.make_layout((2, 2)), (4, 6)), lo.tile_to_shape(lo.SL((2, 2)), lo.static((4, 6))))


def test_recast_and_fragment_match_oracle(mb):
    for shape, stride in [((4, 3), (1, 4)), ((8, 8), (1, 8)), ((1, 128), (0, 1)), ((4, 3), (3, 1))]:
        P, O = mb.make_layout(shape, stride), lo.SL(shape, stride)
        assert same(mb.downcast(P, 2), lo.downcast(O, 2))
        if stride[0] == 1 or stride[0] == 0:
            assert same(mb.upcast(P, 2), lo.upcast(O, 2))
    for shape, stride in [((2, 3, 4), (1, 8, 2)), ((8, 8), (16, 4096)), ((4,), (3,))]:
        assert same(mb.make_fragment_like(mb.make_layout(shape, stride)), lo.make_fragment_like(lo.SL(shape, stride)))
    assert same(mb.make_ordered_layout((2, 3, 4), (2, 0, 1)), lo.make_ordered_layout(lo.static((2, 3, 4)), lo.static((2, 0, 1))))


def test_config1_layout_fixture(mb):
    """Layout evaluation, coalesce, composition and logical_divide of shape (8,(4,2),16) with
    random strides agree bit-for-bit with the committed oracle fixture."""
    with open(os.path.join(GOLD, "cfg1_layouts.json")) as f:
        cases = json.load(f)["cases"]
    for c in cases:
        L = mb.make_layout(tt(c["shape"]), tt(c["stride"]))
        assert [L(i) for i in range(1, 1025)] == c["values"]
        co = mb.coalesce(L)
        assert tt(co.shape) == tt(c["coalesce"]["shape"]) and tt(co.stride) == tt(c["coalesce"]["stride"])
        comp = mb.composition(L, mb.make_layout((32, 2), (2, 64)))
        assert tt(comp.shape) == tt(c["composition"]["shape"]) and tt(comp.stride) == tt(c["composition"]["stride"])
        assert [comp(i) for i in range(1, 65)] == c["composition"]["values"]
        div = mb.logical_divide(L, (mb.make_layout(2), mb.make_layout(4), mb.make_layout(4)))
        assert tt(div.shape) == tt(c["logical_divide"]["shape"])
        assert [div(i) for i in range(1, 1025)] == c["logical_divide"]["values"]


def test_coordinates_and_int_tuples(mb):
    # reference test/stride.jl:5-59, test/int_tuple.jl:24-41
    assert [mb.coord_to_index(c, (3, 4), (2, 8)) for c in (5, 7, 12)] == [11, 17, 29]
    assert [mb.coord_to_index(c, (3, (2, 2)), (2, (16, 8))) for c in ((2, 3), (1, 2), (3, 4))] == [11, 17, 29]
    assert [mb.coord_to_index(c, (3, 4)) for c in ((1, 2), (2, 3), (3, 4))] == [4, 8, 12]
    assert mb.index_to_coord(9, (3, 4), (1, 3)) == (3, 3) and mb.index_to_coord(10, (3, 4), (1, 3)) == (1, 4)
    with pytest.raises(ValueError):
        mb.index_to_coord(9, (3, 4), (1, 3, 5))
    assert mb.compact_col_major((3, 4, 5)) == (1, 3, 12) and mb.compact_row_major((3, 4, 5)) == (20, 5, 1)
    assert mb.shape_div((12, 3), (2, 3)) == (6, 1) and mb.shape_div((12, 3), 3) == (4, 3)
    assert mb.shape_div(12, (3, 4)) == 1
    assert mb.slice_tuple((3, (4, 5)), (":", (2, ":"))) == (3, 5)
    assert mb.Swizzle(3, 4, 3)(0x0090) == 0x0090 ^ 0x10


def test_tiling_views_match_oracle(mb):
    M = N = K = 256
    data = torch.arange(1, M * K + 1, dtype=torch.float32)
    npdata = data.numpy()
    mA = mb.MoYeArray(data, mb.make_layout((M, K)))
    oA = lo.make_view(npdata, lo.make_layout((M, K), (lo.S(1), M)))
    # examples/gemm.jl:22-36
    for bx in (1, 2):
        pt = mb.local_tile(mA, (128, 8), (bx, mb.COLON))
        ot = lo.local_tile(oA, lo.static((128, 8)), (bx, lo.COLON))
        assert pt.offset == ot.offset and tt(pt.shape) == tt(lo.dynamic(ot.layout.shape))
        assert tt(pt.stride) == tt(lo.dynamic(ot.layout.stride))
        for tid in (1, 5, 77, 256):
            pp = mb.local_partition(pt, mb.make_layout((32, 8)), tid)
            op = lo.local_partition(ot, lo.SL((32, 8)), tid)
            assert pp.offset == op.offset and tt(pp.shape) == tt(lo.dynamic(op.layout.shape))
            assert pp[1, 1, 3] == op.get((1, 1, 3))
    ct = mb.local_tile(mA, (128, 128), (2, 1))
    oc = lo.local_tile(oA, lo.static((128, 128)), (2, 1))
    for tid in (1, 18, 255):
        a = mb.local_partition(ct, mb.make_layout((16, 16)), tid)
        b = lo.local_partition(oc, lo.SL((16, 16)), tid)
        assert a.offset == b.offset and tt(a.stride) == tt(lo.dynamic(b.layout.stride)) == (16, 16 * M)
        # projections (X, :) and (:, X) of examples/gemm.jl:33-34
        ax = mb.local_partition(ct, mb.make_layout((16, 16)), tid, (1, mb.COLON))
        bx = lo.local_partition(oc, lo.SL((16, 16)), tid, (lo.S(1), lo.COLON))
        assert ax.offset == bx.offset and tt(ax.shape) == tt(lo.dynamic(bx.layout.shape)) == (8, 128)
        ay = mb.local_partition(ct, mb.make_layout((16, 16)), tid, (mb.COLON, 1))
        by = lo.local_partition(oc, lo.SL((16, 16)), tid, (lo.COLON, lo.S(1)))
        # (:, X) keeps thread-layout mode 2 and applies it to the FIRST mode of x (as for sB in the example)
        assert ay.offset == by.offset and tt(ay.shape) == tt(lo.dynamic(by.layout.shape)) == (8, 128)


def test_moyearray_basics(mb):
    # reference test/array.jl:12-60 style: construction, indexing through the layout, view
    t = torch.arange(24, dtype=torch.int32)
    x = mb.MoYeArray(t, mb.make_layout((2, 3, 4)))
    assert x[2, 3, 4] == 23 and x[1] == 0 and x[24] == 23 and len(x) == 24
    v = x.view(mb.COLON, 2, mb.COLON)
    assert v.shape == (2, 4) and v.stride == (1, 6) and v[1, 1] == 2
    x[2, 1, 1] = 99
    assert t[1] == 99
    r = mb.recast(mb.MoYeArray(torch.zeros(12, dtype=torch.int64), mb.make_layout((4, 3))), torch.int32)
    assert r.shape == (8, 3) and r.stride == (1, 8)  # reference test/array.jl:84-95
    m = mb.MoYeArray(torch.zeros(3, 5))
    assert m.shape == (3, 5) and m.stride == (5, 1)
    assert not mb.isgmem(m)
    f = mb.make_fragment_like_array(mb.MoYeArray(torch.zeros(64), mb.make_layout((8, 8), (1, 8))))
    assert f.shape == (8, 8) and len(f) == 64


def test_tiled_mma_goldens(mb):
    # reference test/tiled_mma.jl:12-39
    A = mb.MoYeArray(torch.arange(1, 48 * 8 * 7 + 1), mb.make_layout((48 * 7, 8)))
    B = mb.MoYeArray(torch.arange(1, 40 * 9 * 8 + 1), mb.make_layout((40 * 9, 8)))
    C = mb.MoYeArray(torch.arange(1, 48 * 7 * 40 * 9 + 1), mb.make_layout((48 * 7, 40 * 9)))
    tm = mb.make_tiled_mma(mb.mma_op("MMAOP_16x8x8_F16F16F16F16_TN"), mb.make_layout((3, 5)))
    assert tm.tile_shape() == (48, 40, 8) and len(tm) == 480
    assert tm.thr_layout_vmnk == mb.make_layout((32, 3, 5, 1), (1, 32, 96, 0))
    thr = tm.get_slice(1)
    tC, tA, tB = thr.partition_C(C), thr.partition_A(A), thr.partition_B(B)
    assert (mb.size(tC.layout, 1), mb.size(tC.layout, 2)) == (7, 9)
    assert (mb.size(tA.layout, 1), mb.size(tA.layout, 2)) == (7, 1)
    assert (mb.size(tB.layout, 1), mb.size(tB.layout, 2)) == (9, 1)
    # every element of C is owned by exactly one (thread, value) pair
    seen = torch.zeros(48 * 7 * 40 * 9, dtype=torch.int32)
    small = mb.MoYeArray(torch.arange(1, 48 * 40 + 1), mb.make_layout((48, 40)))
    owned = torch.zeros(48 * 40, dtype=torch.int32)
    for tid in range(1, 481):
        p = tm.get_slice(tid).partition_C(small)
        for i in range(1, len(p) + 1):
            owned[p[i] - 1] += 1
    assert bool((owned == 1).all()) and seen.sum() == 0
    # docs/src/manual/tensor_core.md:358-391 configuration
    tm2 = mb.make_tiled_mma(mb.mma_op("MMAOP_16x8x16_F32F16F16F32_TN"), mb.make_layout((2, 2, 1)), (32, 32, 16))
    assert tm2.tile_shape() == (32, 32, 16) and len(tm2) == 128
    sm = mb.make_tiled_mma(mb.sm100_mma_op("F16", 256))
    assert sm.tile_shape() == (128, 256, 16) and len(sm) == 1


def run_tiled_copy_kernel(mb, tiled_copy, smem_layout):
    """The host emulation `tiled_copy_kernel` of reference test/copy.jl:102-121."""
    n = mb.size(smem_layout)
    g_in = torch.arange(1, n + 1, dtype=torch.int16)
    g_out = torch.zeros_like(g_in)
    smem = torch.zeros_like(g_in)
    t_in, t_out, t_s = (mb.MoYeArray(x, smem_layout) for x in (g_in, g_out, smem))
    for i in range(1, n + 1):
        t_s[i] = t_in[i]
    for tid in range(1, len(tiled_copy) + 1):
        thr = tiled_copy.get_slice(tid)
        src, dst = thr.partition_S(t_s), thr.partition_D(t_out)
        assert len(src) == len(dst)
        for i in range(1, len(src) + 1):
            dst[i] = src[i]
    return g_in, g_out


def test_tiled_copy_goldens(mb):
    atom = mb.CopyAtom(mb.UniversalCopy(16), mb._lib.U16)
    # reference test/copy.jl:125-134
    tc = mb.make_tiled_copy(atom, mb.make_layout((16, 2)), mb.make_layout((2, 4)))
    assert tc.tiler_mn == (32, 8) and len(tc) == 32
    g_in, g_out = run_tiled_copy_kernel(mb, tc, mb.make_layout((32, 32), (1, 32)))
    assert torch.equal(g_in, g_out)
    # reference test/copy.jl:136-145
    tc = mb.make_tiled_copy(atom, mb.make_layout((32, 1)), mb.make_layout((1, 8)))
    g_in, g_out = run_tiled_copy_kernel(mb, tc, mb.make_layout((32, (2, 4)), (2, (1, 64))))
    assert torch.equal(g_in, g_out)
    # docs/src/manual/tiled_matmul.md:9-16 thread map, and the 128-bit configurations
    tc = mb.make_tiled_copy(atom, mb.make_layout((2, 3), (3, 1)), mb.make_layout((2, 3), (1, 2)))
    assert tc.tiled_layout_tv == mb.make_layout(((3, 2), (2, 3)), ((12, 2), (1, 4))) and tc.tiler_mn == (4, 9)
    tc = mb.make_tiled_copy(mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F32), mb.make_layout((32, 8)), mb.make_layout((4, 1)))
    assert tc.tiled_layout_tv == mb.make_layout((256, 4), (4, 1)) and tc.tiler_mn == (128, 8)
    tc = mb.make_tiled_copy(mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F16), mb.make_layout((16, 16)), mb.make_layout((8, 1)))
    assert tc.tiled_layout_tv == mb.make_layout((256, 8), (8, 1)) and tc.tiler_mn == (128, 16)
    with pytest.raises(ValueError):
        mb.TiledCopy(mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F16), mb.make_layout((256, 4)), (128, 8))


def test_ldmatrix_atoms_construct_and_tile(mb):
    # reference test/copy.jl:152-157: the three non-transposed ldmatrix atoms tile (16,2) x (2,4) threads/values;
    # reference test/device/tiled_copy.jl:60-89 uses the transposed ones on u16
    for name, nsrc, ndst in (("LDSM_U32x1_N", 8, 2), ("LDSM_U32x2_N", 8, 4), ("LDSM_U32x4_N", 8, 8),
                             ("LDSM_U16x2_T", 8, 2), ("LDSM_U16x4_T", 8, 4), ("LDSM_U16x8_T", 8, 8)):
        atom = mb.CopyAtom(mb.ldsm_op(name), mb._lib.U16)
        assert mb.size(atom.thr_id) == 32
        assert atom.num_val_src == nsrc and atom.num_val_dst == ndst
    for name in ("LDSM_U32x1_N", "LDSM_U32x2_N", "LDSM_U32x4_N"):
        tc = mb.make_tiled_copy(mb.CopyAtom(mb.ldsm_op(name), mb._lib.U16), mb.make_layout((16, 2)), mb.make_layout((2, 4)))
        assert len(tc) == 32 and tc.tiler_mn == (32, 8)
    # every destination value of a 32x8 u16 tile is produced exactly once by an x4 atom over 32 threads
    tc = mb.make_tiled_copy(mb.CopyAtom(mb.ldsm_op("LDSM_U32x4_N"), mb._lib.U16), mb.make_layout((32, 1)), mb.make_layout((1, 8)))
    tile = mb.MoYeArray(torch.arange(1, 257, dtype=torch.int16), mb.make_layout((32, 8)))
    seen = torch.zeros(256, dtype=torch.int32)
    for tid in range(1, 33):
        d = tc.get_slice(tid).partition_D(tile)
        for i in range(1, len(d) + 1):
            seen[d[i] - 1] += 1
    assert bool((seen == 1).all())


def test_host_operands_are_rejected(mb):
    a = mb.MoYeArray(torch.zeros(64, 64, dtype=torch.float16))
    c = mb.MoYeArray(torch.zeros(64, 64))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.gemm_(c, a, a, None)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mb.copyto_(a, a)


def test_print_layout_table(mb):
    """Same table as the reference's print_layout (src/print.jl:7-44): header, rulers of ndigits(cosize)+3
    characters per cell, 1-based indices right-aligned."""
    import io
    buf = io.StringIO()
    text = mb.print_layout(mb.make_layout((2, 3), (3, 1)), file=buf)
    want = "\n".join(["(2, 3):(3, 1)",
                      "      1   2   3 ",
                      "    +---+---+---+",
                      " 1  | 1 | 2 | 3 |",
                      "    +---+---+---+",
                      " 2  | 4 | 5 | 6 |",
                      "    +---+---+---+"])
    assert text == want and buf.getvalue() == want + "\n"
    wide = mb.print_layout(mb.make_layout(((2, 2), 4), ((1, 8), 2)), file=io.StringIO()).splitlines()
    assert wide[2] == "    +----+----+----+----+" and wide[3] == " 1  |  1 |  3 |  5 |  7 |"
