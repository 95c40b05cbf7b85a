"""Host-side logic of the product package against the oracle and the reference's goldens:
layout algebra (structure on static layouts, values everywhere), MoYeArray tiling views,
TiledCopy / TiledMMA partitioning (reference test/copy.jl:102-145, test/tiled_mma.jl:12-39)."""
import json
import os

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


def test_swizzle_composes_with_layouts(mb):
    """`Swizzle ∘ Layout` as part of the algebra (the gap reference README.md:14-17 names): the composed layout
    reproduces, offset for offset, the XOR the kernels' epilogue and TMA's SWIZZLE_128B mode use."""
    sw = mb.Swizzle(3, 4, 3)
    rows = mb.make_layout((32, 128), (128, 1))              # 32 staging rows of 128 bytes, byte offsets
    tile = sw @ rows
    assert isinstance(tile, mb.ComposedLayout) and tile == mb.composition(sw, rows)
    assert mb.size(tile) == 4096 and mb.cosize(tile) == 4096 and len(tile) == 2 and tile.shape == (32, 128)
    # the 1024 16-byte stores of the GEMM epilogue: row `lane`, 16-byte group j -> rowp + ((j ^ (lane & 7)) << 4)
    for lane in range(32):
        for j in range(8):
            for b in range(4):   # four bytes inside the group, so 1024 offsets in all
                assert tile(lane + 1, 16 * j + 4 * b + 1) - 1 == lane * 128 + ((j ^ (lane & 7)) << 4) + 4 * b
    assert tile.offset0(5 * 1 + 0) == sw(rows.offset0(5))   # 0-based form
    # a swizzle permutes offsets inside aligned 1024-byte blocks: the image of the tile is the tile
    assert sorted(tile(i) for i in range(1, 4097)) == list(range(1, 4097))
    # slicing keeps the swizzle and folds the fixed coordinate into the offset; composing on the right reaches inside
    col = tile(mb.COLON, 17)
    assert [col(r) for r in (1, 2, 9)] == [tile(r, 17) for r in (1, 2, 9)]
    sub = tile @ mb.make_layout((8, 8), (1, 512))           # rows 0..7 x every 16th byte
    assert all(sub(r, c) == tile(r, 16 * (c - 1) + 1) for r in range(1, 9) for c in range(1, 9))
    assert tile[1] == mb.ComposedLayout(sw, mb.make_layout(128, 1))
    # the K-major operand stage of the tensor-core kernels is the same function over (row, k) of 16-bit elements
    stage = mb.umma_smem_layout(mb._lib.F16, 128, "K")
    assert stage(9, 1) - 1 == 8 * 128 and stage(2, 1) - 1 == 128 + 16 and stage(2, 9) - 1 == 128
    mn = mb.umma_smem_layout(mb._lib.F16, 128, "MN")         # chunks of 64 elements along M, K rows 128 bytes apart
    assert mn((1, 2), 1) - 1 == 64 * 128 and mn((9, 1), 2) - 1 == 128 + (16 ^ 16)
    text = mb.print_layout(mb.Swizzle(2, 0, 3) @ mb.make_layout((8, 8), (8, 1)), file=open(os.devnull, "w"))
    assert "| 10 |  9 | 12 | 11 |" in text and text.startswith("Swizzle(2,0,3) o (8, 8):(8, 1)")
    with pytest.raises(ValueError):
        mb.Swizzle(3, 4, 2)
    with pytest.raises(TypeError):
        mb.ComposedLayout(rows, rows)


def test_ownership_pictures(mb):
    """`print_typst` for a TiledCopy / TiledMMA (reference src/print.jl:317-345) and the tcgen05 views."""
    import io
    # the thread map the manual draws (docs/src/manual/tiled_matmul.md:9-16): thr (32,8) x val (4,1) on a (128,8) tile
    tc = mb.make_tiled_copy(mb.CopyAtom(mb.UniversalCopy(128), mb._lib.F32), mb.make_layout((32, 8)), mb.make_layout((4, 1)))
    lay, thr = tc.get_layoutS_MN()
    n = len(tc)
    for m in range(128):
        for c in range(8):
            idx0 = lay(m + 1, c + 1) - 1
            assert (idx0 % n, idx0 // n) == (m // 4 + 32 * c, m % 4)
    assert tc.get_layoutD_MN()[0] == lay and mb.size(thr) == 256
    text = mb.print_typst(tc, file=io.StringIO())
    assert text.count("owner(") == 2 * 128 * 8 + 1 and "owner(33, 2)," in text
    # the tf32 configuration of the tensor-core manual (docs/src/manual/tensor_core.md:358-366)
    mma = mb.make_tiled_mma(mb.mma_op("MMAOP_16x8x8_F32TF32TF32F32_TN"), mb.make_layout((2, 2, 1), (2, 1, 1)), (32, 32, 8))
    assert len(mma) == 128 and mma.tile_shape() == (32, 32, 8)
    c_mn, c_thr = mma.get_layoutC_MN()
    owners = {}
    for m in range(1, 33):
        for nn in range(1, 33):
            idx0 = c_mn(m, nn) - 1
            owners.setdefault(c_thr(idx0 % mb.size(c_thr) + 1) - 1, []).append(idx0 // mb.size(c_thr))
    assert sorted(owners) == list(range(128)) and all(sorted(v) == list(range(8)) for v in owners.values())
    text = mb.print_typst(mma, file=io.StringIO())
    assert text.count("owner(") == 32 * 32 + 2 * 32 * 8 + 1
    # a tcgen05 atom: one issuing thread owns everything; the informative pictures are where the data lives
    op = mb.sm100_mma_op("F16", 128)
    text = mb.print_typst(mb.make_tiled_mma(op), file=io.StringIO())
    assert text.count("owner(0, ") == 128 * 128 + 2 * 128 * 16
    text = mb.print_tmem_layout(op, cta_pair=True, file=io.StringIO())
    assert "128 x 2 CTAs lanes x 128 columns" in text and "warp%4=3" in text
    assert mb.tmem_accumulator_layout(128, cta_pair=True)(130, 5) == (1, 1, 4)
    text = mb.print_umma_smem_layout(mb._lib.F16, 8, "K", file=io.StringIO())
    assert "    1     c1      c0      c3      c2      c5      c4      c7      c6" in text
    with pytest.raises(ValueError):
        mb.print_tmem_layout(mb.mma_op("MMAOP_16x8x16_F32F16F16F32_TN"))


def test_copy_dispatch_is_decided_on_the_host(mb):
    """`copyto_` never tries one kernel and falls back to another: shapes, strides and alignment decide up front."""
    base = torch.zeros(64 * 1024 + 64, dtype=torch.float16)
    full = mb.MoYeArray(base[:64 * 1024], mb.make_layout((256, 256)))
    assert mb.copy_dispatch(full, full) == ("tiled", None)
    rowm = mb.MoYeArray(base[:64 * 1024], mb.make_layout((256, 256), (256, 1)))
    assert mb.copy_dispatch(full, rowm) == ("tiled", None)                           # contiguous along different modes: transpose
    odd = mb.MoYeArray(base[1:64 * 1024 + 1], mb.make_layout((256, 256)))
    assert mb.copy_dispatch(full, odd) == ("elementwise", "a base address is not 16-byte aligned")
    pitched = mb.MoYeArray(base, mb.make_layout((250, 256), (1, 257)))
    path, why = mb.copy_dispatch(mb.MoYeArray(base, mb.make_layout((250, 256), (1, 256))), pitched)
    assert path == "elementwise" and "pitch" in why
    hier = mb.MoYeArray(base[:64 * 1024], mb.make_layout(((16, 16), 256), ((1, 4096), 16)))
    assert mb.copy_dispatch(full, hier) == ("elementwise", None)                     # not a rank-2 strided matrix at all
    diff = mb.MoYeArray(base[:32 * 1024], mb.make_layout((128, 256)))
    assert mb.copy_dispatch(full, diff)[0] == "elementwise"


def test_manual_kernel_variants_host_side(mb):
    """The objects the reference manual builds for its pipelined and tensor-core kernels, evaluated on the host:
    the partition shapes are the ones its comments state (docs/src/manual/pipeline.md:105-128,
    tensor_core.md:283-312,352-381)."""
    import importlib.util
    ex = {}
    for name in ("pipeline", "tensor_core"):
        spec = importlib.util.spec_from_file_location("example_" + name, os.path.join(os.path.dirname(__file__), "..", "examples", name + ".py"))
        ex[name] = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ex[name])
    p = ex["pipeline"].host_side()
    assert p["threads"] == 256 and p["blocks"] == (16, 16) and p["mma_tile"] == (32, 8, 1)
    assert p["gA"] == (128, 8, 32) and p["gC"] == (128, 128)                       # (bM, bK, k), (bM, bN)
    assert p["tAgA"] == ((2, 1), 2, 1, 32) and p["tAsA"] == ((2, 1), 2, 1, 2)      # (CPY, CPY_M, CPY_K, k | 2)
    assert p["tCsA"] == (1, 4, 8, 2) and p["tCsB"] == (1, 16, 8, 2) and p["tCgC"] == (1, 4, 16)   # (MMA, MMA_M|N, MMA_K, 2)
    assert p["tCrA"] == (1, 4, 8) and p["tCrC"] == (1, 4, 16) and p["k_tile_max"] == 32 and p["k_block_max"] == 8
    assert p["smem_floats"] == 2 * ((128 + 2) * 8 * 2 - 2)                          # two padded (bM, bK, 2) buffers
    t = ex["tensor_core"].host_side()
    assert t["threads"] == 128 and t["mma_tile"] == (32, 32, 8)
    assert t["gmem_copy_A_tiler"] == (64, 8) and t["gmem_copy_B_tiler"] == (32, 16)
    assert t["smem_copy_A_tiler"] == (32, 8) and t["smem_copy_B_tiler"] == (32, 8) and t["smem_copy_threads"] == (128, 128)
    assert t["tCsA"] == ((2, 2), 4, 2, 2) and t["tCsB"] == (2, 8, 2, 2)
    assert mb.size(mb.make_layout(t["tCsA_retiled"])) == mb.size(mb.make_layout(t["tCsA"]))
