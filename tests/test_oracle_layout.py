"""Pins the layout-algebra oracle (oracle/layout_oracle.py) to the reference's own golden
vectors.  Every case is transcribed from a test or docstring of MoYe.jl; the comment on each
block gives the reference file and lines it comes from."""

import pytest

from layout_oracle import (COLON, GenColMajor, GenRowMajor, S, SL, blocked_product, capacity, coalesce, colex_less,
                           complement, composition, coord_to_index, cosize, depth, downcast, elem_less, escan,
                           flatten, increment, index_to_coord, insert, iscompatible, lflatten, logical_divide,
                           logical_product, make_layout, make_ordered_layout, prepend, append, raked_product,
                           recast, remove, repeat_like, replace, right_inverse, left_inverse, shape_div, size,
                           slice_, static, tiled_divide, tiled_product, unflatten, unwrap, upcast, zip2_by,
                           zipped_divide, zipped_product, compact_col_major, compact_row_major, front, back,
                           tuple_cat, lfilter, is_static, make_fragment_like, max_common_vector, tile_to_shape)


def dyn(shape, stride=None):
    return make_layout(shape) if stride is None else make_layout(shape, stride)


# ---- test/tuple_alg.jl:4-9
@pytest.mark.parametrize("flat,profile,want", [
    ((1, 2, 3), (0, 0, 0), (1, 2, 3)),
    ((1, 2, 3, 4), (0, (0, (0, 0))), (1, (2, (3, 4)))),
    ((1, 2, 3, 4), ((0, 0), (0, 0)), ((1, 2), (3, 4))),
    ((1, 2, 3, 4, 5), (0, (0, 0), 0), (1, (2, 3), 4)),
    ((1, 2, 3, 4, 5, 6), (0, (0, (0, (0, (0, 0))))), (1, (2, (3, (4, (5, 6)))))),
    ((), (), ()),
])
def test_unflatten(flat, profile, want):
    assert unflatten(flat, profile) == want


def test_tuple_helpers():
    # test/tuple_alg.jl:13-59
    assert front(((2, 3), 4)) == (2, 3) or front(flatten(((2, 3), 4))) == 2
    assert back(flatten((2, (3, 4)))) == 4
    assert tuple_cat([(1, 2), (3, 4)]) == (1, 2, 3, 4)
    assert insert((1, 2, 3), 10, 2) == (1, 10, 2, 3)
    assert remove((1, 2, 3), 2) == (1, 3)
    assert replace((1, 2, 3), 10, 2) == (1, 10, 3)
    assert unwrap(((1,),)) == 1
    assert append((1, 2), 3) == (1, 2, 3)
    assert append((1, 2), 3, 4) == (1, 2, 3, 3)
    assert prepend((1, 2), 3) == (3, 1, 2)
    assert prepend((1, 2), 3, 4) == (3, 3, 1, 2)
    assert escan(lambda a, b: a * b, (1, 2, 3, 4, 5), 10) == (10, 10, 20, 60, 240)
    # test/tuple_alg.jl:69-70
    assert zip2_by((("A", "a"), (("B", "b"), ("C", "c")), "d"), (0, (0, 0))) == \
        (("A", ("B", "C")), ("a", ("b", "c"), "d"))


def test_int_tuple():
    # test/int_tuple.jl:7
    assert capacity(((2, 3, (1, 1)), 4)) == 24
    # :11-15
    assert repeat_like((2, 3, 4), 1) == (1, 1, 1)
    assert repeat_like(((2, 3), (4, 5)), 1) == ((1, 1), (1, 1))
    # :24-30
    assert shape_div((12, 3), (2, 3)) == (6, 1)
    assert shape_div((12, 3), 3) == (4, 3)
    assert shape_div(12, (3, 4)) == 1
    # :35-41
    assert slice_((3, 4), (2, COLON)) == (4,)
    assert slice_((3, (4, 5)), (COLON, (2, COLON))) == (3, 5)
    assert slice_(((2, 4), (4, 2)), (COLON, (COLON, COLON))) == ((2, 4), 4, 2)


@pytest.mark.parametrize("a,b,want", [  # test/int_tuple.jl:46-62
    ((1, 2, 3), (1, 2, 4), True), ((1, 2, 3), (1, 2, 3), False), ((1, 2, 3), (1, 2, 3, 1), True),
    ((1, 2, 3, 1), (1, 2, 3), False), (((1, 2, 3),), ((1, 2, 3),), False), (((1, 2, 3),), ((1, 2, 4),), True),
    (((1, 2, 3),), ((1, 2, 3), 1), True), (((1, 2, 3), 1), ((1, 2, 3), 2), True),
    (((1, 2, 3), 2), ((1, 2, 4), 1), False), (((1, 2), (3, 4)), ((5, 6), (7, 8)), True),
    (((1, 2), (3, 4)), ((1, 2), (7, 8)), True), (((1, 2), (3, 4)), ((1, 2), (1, 8)), False),
    (((1, 2), (3, 4)), ((3, 4), (3, 4)), False), (((1, 2), (3, 4)), ((3, 4), (3, 4, 1)), True),
    (((1, 2), (3, 4)), ((3, 4), (3, 4), 1), True),
])
def test_elem_less(a, b, want):
    assert elem_less(a, b) == want


@pytest.mark.parametrize("a,b,want", [  # test/int_tuple.jl:68-83
    ((1, 2, 3), (1, 2, 4), True), ((1, 2, 3), (1, 2, 3), False), ((1, 2, 3), (1, 1, 2, 3), True),
    ((1, 1, 2, 3), (1, 2, 3), False), (((1, 2, 3),), ((1, 2, 3),), False), (((0, 2, 3),), ((1, 2, 3),), True),
    (((1, 2, 3),), (1, (1, 2, 3)), True), ((1, (1, 2, 3)), (2, (1, 2, 3)), True),
    ((2, (1, 2, 3)), (1, (2, 2, 3)), True), (((1, 2), (3, 4)), ((5, 6), (7, 8)), True),
    (((1, 2), (3, 4)), ((2, 3), (3, 4)), True), (((1, 2), (3, 4)), ((1, 3), (3, 4)), True),
    (((5, 4), (3, 4)), ((3, 4), (3, 4)), False), (((1, 2), (3, 4)), ((1, 1, 2), (3, 4)), True),
])
def test_colex_less(a, b, want):
    assert colex_less(a, b) == want


@pytest.mark.parametrize("c,s,want", [  # test/int_tuple.jl:89-96
    ((1, 1), (3, 4), (2, 1)), ((3, 1), (3, 4), (1, 2)), ((3, 4), (3, 4), (1, 1)),
    ((2, (2, 1), 1), (2, (2, 3), 3), (1, (1, 2), 1)), ((2, (2, 2), 1), (2, (2, 3), 3), (1, (1, 3), 1)),
    ((2, (2, 3), 1), (2, (2, 3), 3), (1, (1, 1), 2)), ((2, (2, 3), 3), (2, (2, 3), 3), (1, (1, 1), 1)),
])
def test_increment(c, s, want):
    assert increment(c, s) == want


def test_coord_to_index():
    # test/stride.jl:5-7 (1-D), :15-17 (h-D), :25-27 (R-D), :37-39 (default stride)
    assert [coord_to_index(c, (3, 4), (2, 8)) for c in (5, 7, 12)] == [11, 17, 29]
    assert [coord_to_index(c, (3, 4), (2, 8)) for c in ((2, 2), (1, 3), (3, 4))] == [11, 17, 29]
    assert [coord_to_index(c, (3, (2, 2)), (2, (16, 8))) for c in ((2, 3), (1, 2), (3, 4))] == [11, 17, 29]
    assert [coord_to_index(c, (3, 4)) for c in ((1, 2), (2, 3), (3, 4))] == [4, 8, 12]
    # test/stride.jl:48-49
    assert index_to_coord(9, (3, 4), (1, 3)) == (3, 3)
    assert index_to_coord(10, (3, 4), (1, 3)) == (1, 4)
    # test/stride.jl:58-59
    assert compact_col_major(static((3, 4, 5))) == (1, 3, 12)
    assert compact_row_major(static((3, 4, 5))) == (20, 5, 1)
    assert is_static(compact_col_major(static((3, 4, 5))))


def test_make_layout_docstrings():
    # src/stride.jl:150-165 docstrings: a dynamic extent 1 keeps a stride, the first stride is static 1
    l = make_layout(((1, (2, 4)), 1), GenColMajor)
    assert l.stride == ((1, (1, 2)), 8)
    l = make_layout(((1, (2, 4)), 1), GenRowMajor)
    assert l.stride == ((8, (4, 1)), 1)
    # test/layout.jl:29-30
    assert lflatten(make_layout(((4, 3), 1), ((3, 1), 0))) == make_layout((4, 3, 1), (3, 1, 0))
    # static extent 1 gets stride 0 (src/stride.jl:173-174)
    assert SL((1, 4)).stride == (0, 1)


def check_coalesce(l):
    c = coalesce(l)
    assert depth(c.shape) <= 1
    assert size(c) == size(l)
    for i in range(1, int(size(l)) + 1):
        assert c(i) == l(i)


def test_coalesce():
    # test/layout.jl:35
    assert coalesce(SL((2, (1, 6)), (1, (6, 2)))) == SL(12, 1)
    # test/layout.jl:39-130: coalescing preserves the function and the size
    two, four, six, one = S(2), S(4), S(6), S(1)
    cases = [
        make_layout(one, 0), make_layout(one, one), make_layout((two, four)), make_layout((two, four, six)),
        make_layout((two, one, six), (one, six, two)), make_layout((two, one, six), (one, 7, two)),
        make_layout((two, one, six), (four, 7, S(8))), make_layout((2, four, six)), make_layout((two, 4, six)),
        make_layout((two, four, 6)), make_layout((two, four), GenRowMajor),
        make_layout((two, four, six), GenRowMajor), make_layout((2, four, six), GenRowMajor),
        make_layout((two, 4, six), GenRowMajor), make_layout((two, four, 6), GenRowMajor),
        make_layout((two, one, S(3)), GenRowMajor), make_layout((two, 1, S(3)), GenRowMajor),
        make_layout((two, 1, S(3)), (two, 4, four)), make_layout((two, 1, S(3)), (two, 0, four)),
        SL(((2, 2), (2, 2)), ((1, 4), (8, 32))),
    ]
    for l in cases:
        check_coalesce(l)
    # dynamic modes never merge, a dynamic 1 is not dropped (src/layout.jl:441-479)
    assert coalesce(make_layout((2, 4), (1, 2))) == make_layout((2, 4), (1, 2))
    assert coalesce(SL((2, 4), (1, 2))) == SL(8, 1)


def check_composition(a, b):
    c = composition(a, b)
    assert iscompatible(b.shape, c.shape)
    for i in range(1, int(size(c)) + 1):
        assert c(i) == a(b(i)), (a, b, c, i)


COMPOSITION_STATIC = [  # test/layout.jl:149-282
    (SL(1, 0), SL(1, 0)), (SL(1, 0), SL(1, 1)), (SL(1, 1), SL(1, 0)), (SL(1, 1), SL(1, 1)),
    (SL((4,)), SL((4,))), (SL((4,), (2,)), SL((4,))), (SL((4,)), SL((4,), (2,))), (SL((4,), (0,)), SL((4,))),
    (SL((4,)), SL((4,), (0,))), (SL((1,), (0,)), SL((4,))), (SL((4,)), SL((1,), (0,))), (SL((4,)), SL((2,))),
    (SL((4,), (2,)), SL((2,))), (SL((4,)), SL((2,), (2,))), (SL((4,), (2,)), SL((2,), (2,))),
    (SL((4, 3)), SL((12,))), (SL((12,)), SL((4, 3))), (SL((12,), (2,)), SL((4, 3))),
    (SL((12,)), SL((4, 3), (3, 1))), (SL((12,), (2,)), SL((4, 3), (3, 1))), (SL((12,)), SL((2, 3), (2, 4))),
    (SL((4, 3)), SL((4, 3))), (SL((4, 3)), SL((12,))), (SL((4, 3)), SL((6,), (2,))),
    (SL((4, 3)), SL((6, 2), (2, 1))), (SL((4, 3), (3, 1)), SL((4, 3))), (SL((4, 3), (3, 1)), SL((12,))),
    (SL((4, 3), (3, 1)), SL((6,), (2,))), (SL((4, 3), (3, 1)), SL((6, 2), (2, 1))),
    (SL((8, 8)), SL(((2, 2, 2), (2, 2, 2)), ((1, 16, 4), (8, 2, 32)))),
    (SL((8, 8), (8, 1)), SL(((2, 2, 2), (2, 2, 2)), ((1, 16, 4), (8, 2, 32)))),
    (SL(((2, 2, 2), (2, 2, 2)), ((1, 16, 4), (8, 2, 32))), SL(8, 4)),
    (SL(((4, 2),), ((1, 16),)), SL((4, 2), (2, 1))), (SL((2, 2), (2, 1)), SL((2, 2), (2, 1))),
    (SL((4, 8, 2)), SL((2, 2, 2), (2, 8, 1))), (SL((4, 8, 2), (2, 8, 1)), SL((2, 2, 2), (1, 8, 2))),
    (SL((4, 8, 2), (2, 8, 1)), SL((4, 2, 2), (2, 8, 1))),
]


@pytest.mark.parametrize("a,b", COMPOSITION_STATIC)
def test_composition_static(a, b):
    check_composition(a, b)


def test_composition_goldens_and_dynamic():
    # test/layout.jl:134-135
    assert composition(dyn(20, 2), dyn((4, 5), (1, 4))) == dyn((4, 5), (2, 8))
    assert composition(dyn(20, 2), dyn((4, 5), (5, 1))) == dyn((4, 5), (10, 2))
    # test/layout.jl:284-313 (dynamic operands)
    for a, b in [(dyn(12, 1), dyn(4, 1)), (dyn((12, 3), (1, 24)), dyn(4, 1)), (dyn(16, 2), dyn(4, 2)),
                 (dyn((128, 24, 5), (1, 128, 3072)), dyn(64, 2)),
                 (dyn((128, 24, 5), (1, 128, 3072)), make_layout(480, S(32)))]:
        check_composition(a, b)


def check_complement(l, cotarget=None):
    cot = cosize(l) if cotarget is None else cotarget
    r = complement(l, cot)
    fl = lfilter(l)
    assert size(r) >= int(cot) // int(size(fl))
    assert cosize(r) <= -(-int(cot) // int(cosize(l))) * int(cosize(l))
    completed = make_layout(l, r)
    assert cosize(completed) >= cot
    for i in range(2, int(size(r)) + 1):
        assert r(i - 1) < r(i)
        for j in range(1, int(size(l)) + 1):
            assert r(i) != l(j)
    assert size(r) <= cosize(r)
    assert cosize(r) >= int(cot) // int(size(fl))
    assert cosize(completed) <= cosize(r) + cosize(l)


def test_complement():
    # test/layout.jl:317-318
    assert complement(SL(4, 1), S(24)) == SL(6, 4)
    assert complement(SL(6, 4), S(24)) == SL(4, 1)
    assert complement(SL(4, 2), S(24)) == SL((2, 3), (1, 8))
    # test/layout.jl:351-414
    for l, cot in [(SL(1, 0), None), (SL(1, 0), S(2)), (SL(1, 1), None), (SL(1, 1), S(2)), (SL(1, 2), S(1)),
                   (SL(1, 2), S(2)), (SL(1, 2), S(8)), (SL(4, 0), S(1)), (SL(4, 0), S(2)), (SL(4, 0), S(8)),
                   (SL(4, 1), S(1)), (SL(4, 1), S(2)), (SL(4, 1), S(8)), (SL(4, 2), S(1)), (SL(4, 2), S(2)),
                   (SL(4, 2), S(16)), (SL(4, 4), S(1)), (SL(4, 4), S(2)), (SL(4, 4), S(17)), (SL((2, 4)), None),
                   (SL((2, 3)), None), (SL((2, 4), (1, 4)), None), (SL((2, 4, 8), (8, 1, 64)), None),
                   (SL(((2, 2), (2, 2)), ((1, 4), (8, 32))), None), (SL((2, (3, 4)), (3, (1, 6))), None),
                   (SL((4, 6), (1, 6)), None), (SL((4, 10), (1, 10)), None)]:
        check_complement(l, cot)


TILE = SL((2, 2), (1, 2))
MOT = SL((3, 4), (4, 1))


def test_products():
    # test/layout.jl:421-424
    r = logical_product(TILE, MOT)
    assert r.shape == ((2, 2), (3, 4)) and r.stride == ((1, 2), (16, 4))
    # :427
    assert logical_product(SL(1), SL((2, 2))) == SL((1, (2, 2)))
    # :485-488
    r = blocked_product(TILE, MOT, True)
    assert r.shape == ((2, 3), 8) and r.stride == ((1, 16), 2)
    # :492-495
    r = raked_product(TILE, MOT, True)
    assert r.shape == ((3, 2), (4, 2)) and r.stride == ((16, 1), (4, 2))
    # :500-503
    r = zipped_product(TILE, MOT)
    assert r.shape == ((2, 2), (3, 4)) and r.stride == ((1, 2), (16, 4))
    # :508-511
    r = tiled_product(TILE, MOT)
    assert r.shape == ((2, 2), 3, 4) and r.stride == ((1, 2), 16, 4)
    # :430-480: rank and compatibility of the first mode
    for a, b in [(SL(1, 0), SL(1, 0)), (SL(1, 0), SL(1, 1)), (SL(1, 1), SL(1, 1)), (SL(4, 0), SL(3, 1)),
                 (SL(3, 0), SL(4, 0)), (SL(3, 2), SL(4, 1)), (SL((3,)), SL((2, 4))), (SL((8, (2, 2))), SL(4, 2)),
                 (SL((2, 2)), SL((3, 3), (3, 1))), (SL(3, 32), SL((8, 8))),
                 (SL(((2, 2), (2, 2)), ((1, 4), (8, 32))), SL((2, 2), (1, 2))),
                 (SL(((2, 2), (2, 2)), ((1, 4), (8, 32))), SL((2, 2), (2, 1)))]:
        c = logical_product(a, b)
        assert len(c.shape) == 2
        assert iscompatible(a.shape, c.shape[0])


def test_product_docstring_tables():
    # src/layout.jl:783-823: value table of logical_product((2,2):(1,2), (3,4):(4,1))
    r = logical_product(TILE, MOT)
    row1 = [int(r((1, j))) for j in range(1, 13)]
    assert row1 == [1, 17, 33, 5, 21, 37, 9, 25, 41, 13, 29, 45]
    # src/layout.jl:855-878 blocked product table, first column and first row
    b = blocked_product(TILE, MOT)
    assert [int(b((i, 1))) for i in range(1, 7)] == [1, 2, 17, 18, 33, 34]
    assert [int(b((1, j))) for j in range(1, 9)] == [1, 3, 5, 7, 9, 11, 13, 15]
    # src/layout.jl:894-917 raked product table
    k = raked_product(TILE, MOT)
    assert [int(k((i, 1))) for i in range(1, 7)] == [1, 17, 33, 2, 18, 34]
    assert [int(k((1, j))) for j in range(1, 9)] == [1, 5, 9, 13, 3, 7, 11, 15]


def test_divides():
    raked = raked_product(TILE, MOT)
    subtile = (SL(2, 3), SL(2, 4))
    # test/layout.jl:524-531
    assert logical_divide(SL(16, 3), SL(4, 1)) == SL((4, 4), (3, 12))
    assert logical_divide(SL(16, 3), SL(4, 4)) == SL((4, 4), (12, 3))
    assert logical_divide(SL(16, 3), SL(4, 2)) == SL((4, (2, 2)), (6, (3, 24)))
    assert logical_divide(SL(16, 3), SL((2, 2), (4, 1))) == SL(((2, 2), (2, 2)), ((12, 3), (6, 24)))
    assert logical_divide(raked, subtile) == SL(((2, 3), (2, 4)), ((1, 16), (2, 4)))
    # :610-611, :616-617
    assert zipped_divide(raked, subtile) == SL(((2, 2), (3, 4)), ((1, 2), (16, 4)))
    assert tiled_divide(raked, subtile) == SL(((2, 2), 3, 4), ((1, 2), 16, 4))
    # :535-606
    for l, t in [(SL(1, 0), SL(1, 0)), (SL(1, 0), SL(1, 1)), (SL(1, 1), SL(1, 0)), (SL(1, 1), SL(1, 1)),
                 (SL(6, 1), SL(2, 1)), (SL(6, 1), SL(2, 3)), (SL((6, 6), (1, 12)), SL((6, 3), (3, 1))),
                 (SL((6, 6), (12, 1)), SL((6, 3), (3, 1))), (SL(32), SL((2, 8))), (SL((4, 1), (1, 1)), SL(2, 1)),
                 (SL((4, 1), (1, 1)), SL(2, 2)), (SL((8, 8), (1, 8)), SL((32, 2))),
                 (SL((8, 8), (8, 1)), SL((32, 2)))]:
        c = logical_divide(l, t)
        assert len(c.shape) == 2
        assert iscompatible(t.shape, c.shape[0])
    # the tile derivation of examples/gemm.jl:22 on a dynamic (M,K):(_1,M) array
    z = zipped_divide(make_layout((256, 256), (S(1), 256)), static((128, 8)))
    assert z == make_layout(((128, 8), (2, 32)), ((1, 256), (128, 2048)))


@pytest.mark.parametrize("l", [  # test/layout.jl:634-651
    SL(1, 0), SL(1, 1), SL((4,), (0,)), SL((4,), (1,)), SL((4,), (2,)), SL((1, 1), (0, 0)), SL((3, 7), (0, 0)),
    SL((1,), (1,)), SL((2, 4), (0, 2)), SL((8, 4)), SL((8, 4), (4, 1)), SL((2, 4, 6)), SL((2, 4, 6), (4, 1, 8)),
    SL((2, 4, 4, 6), (4, 1, 0, 8)), SL((4, 2), (1, 16)), SL((4, 2), (1, 5)),
])
def test_right_inverse(l):
    inv = right_inverse(l)
    for i in range(1, int(size(inv)) + 1):
        assert l(inv(i)) == i


def test_left_inverse():
    for l in [SL((8, 4)), SL((8, 4), (4, 1)), SL((4, 2), (1, 16)), SL((2, 4, 6), (4, 1, 8))]:
        inv = left_inverse(l)
        for i in range(1, int(size(l)) + 1):
            assert inv(l(i)) == i


def test_recast():
    # test/array.jl:84-106: (4,3) Int64 -> Int32 (8,3) -> UInt128 (2,3); layouts only
    l = SL((4, 3))
    assert downcast(l, 2) == SL((8, 3), (1, 8))
    assert upcast(l, 2) == SL((2, 3), (1, 2))
    assert recast(l, 4, 8) == SL((8, 3), (1, 8))
    assert recast(l, 16, 8) == SL((2, 3), (1, 2))
    # dynamic (test/array.jl:127-143): dynamic strides divide, shapes stay
    d = make_layout((4, 3), (S(1), 4))
    assert upcast(d, 2) == make_layout((2, 3), (1, 2))
    # bit layouts of copy traits upcast to values (src/atom/copy.jl:35-37)
    assert upcast(SL((1, 128)), 16) == SL((1, 8))


def test_make_fragment_like_and_misc():
    # src/layout.jl:1143-1149: first mode col-major, the rest ordered like the source strides
    assert make_fragment_like(SL((2, 3, 4), (1, 8, 2))) == SL((2, 3, 4), (1, 8, 2))
    assert make_fragment_like(SL((8, 8), (16, 4096))) == SL((8, 8))
    assert make_fragment_like(make_layout((8, 8), (16, 4096))) == make_layout((8, 8))
    assert max_common_vector(SL((8, 4)), SL((8, 4))) == 32
    assert max_common_vector(SL((8, 4)), SL((8, 4), (4, 1))) == 1
    assert make_ordered_layout(static((2, 3, 4)), static((2, 0, 1))) == SL((2, 3, 4), (12, 1, 3))
    assert tile_to_shape(SL((2, 2)), static((4, 6))) == blocked_product(SL((2, 2)), SL((2, 3)), True)


def test_index_periodicity():
    # docs/src/manual/array.md:15-22: linear indexing wraps in every mode, including the last
    l = SL((2, 3))
    assert [int(l(i)) for i in range(1, 13)] == [1, 2, 3, 4, 5, 6] * 2
    # a rank-1 layout does not wrap (src/stride.jl:1-9)
    assert int(SL(4, 2)(7)) == 13
