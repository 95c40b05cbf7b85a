"""TEST INFRASTRUCTURE -- CPU restatement of MoYe.jl's host-side layout algebra.

This file is the *checker* for the layout / tiling part of the hot path; it is imported only
by tests, by the smoke check and by the CPU-baseline leg of the benchmark, never by the
product package.  It restates, in plain Python over nested tuples, the algorithms of the
reference (all citations are paths inside the MoYe.jl project):

  src/utilities.jl, src/algorithm/tuple_algorithms.jl, src/int_tuple.jl   IntTuple helpers
  src/stride.jl                                                           coordinates, compact strides
  src/layout.jl                                                           Layout algebra
  src/algorithm/array_algorithms.jl                                       local_tile / local_partition

Data model.  An IntTuple is an int or a tuple of IntTuples.  A leaf is *static* (class `S`,
MoYe's `StaticInt`, written `_4` / `@Layout`) or *dynamic* (plain `int`).  The flag never
changes what a layout computes, only how results are structured (dynamic modes are never
merged by `coalesce`, a dynamic 1 is not dropped, ...), exactly as in the reference.
A Layout is the pair (shape, stride).  All public indices and coordinates are 1-based.

Parity pin: every golden vector of the reference's own tests for this algebra
(test/layout.jl, test/stride.jl, test/int_tuple.jl, test/tuple_alg.jl, test/tiled_mma.jl and
the docstrings) is asserted against this file by tests/test_oracle_layout.py.
"""
from collections import namedtuple

COLON = ":"  # MoYe's `:` / Colon()


# --------------------------------------------------------------------------- static ints
class S(int):
    """A static integer (Static.jl `StaticInt{N}`).  S op S -> S, S op int -> int."""

    __slots__ = ()

    def _w(self, other, v):
        return S(v) if isinstance(other, S) else int(v)

    def __add__(self, o): return self._w(o, int(self) + int(o))
    def __radd__(self, o): return self._w(o, int(o) + int(self))
    def __sub__(self, o): return self._w(o, int(self) - int(o))
    def __rsub__(self, o): return self._w(o, int(o) - int(self))
    def __mul__(self, o): return self._w(o, int(self) * int(o))
    def __rmul__(self, o): return self._w(o, int(o) * int(self))
    def __floordiv__(self, o): return self._w(o, _tdiv(int(self), int(o)))
    def __rfloordiv__(self, o): return self._w(o, _tdiv(int(o), int(self)))
    def __mod__(self, o): return self._w(o, _trem(int(self), int(o)))
    def __rmod__(self, o): return self._w(o, _trem(int(o), int(self)))
    def __neg__(self): return S(-int(self))
    def __abs__(self): return S(abs(int(self)))
    def __repr__(self): return f"_{int(self)}"


def _tdiv(a, b):
    """Julia `div` / `÷`: truncates toward zero."""
    q = abs(a) // abs(b)
    return q if (a >= 0) == (b >= 0) else -q


def _trem(a, b):
    """Julia `rem` / `%`: sign of the dividend."""
    return a - b * _tdiv(a, b)


def idiv(a, b):
    if isinstance(a, S):
        return a // b
    if isinstance(b, S):
        return b.__rfloordiv__(a)
    return _tdiv(a, b)


def irem(a, b):
    if isinstance(a, S):
        return a % b
    if isinstance(b, S):
        return b.__rmod__(a)
    return _trem(a, b)


def is_tuple(x):
    return isinstance(x, tuple)


def is_static(x):
    """Static.jl `is_static` on an IntTuple: every leaf is static."""
    if is_tuple(x):
        return all(is_static(e) for e in x)
    return isinstance(x, S)


def static(x):
    """`static(x)`: make every leaf static (src/utilities.jl)."""
    if is_tuple(x):
        return tuple(static(e) for e in x)
    return x if x == COLON else S(x)


def dynamic(x):
    if is_tuple(x):
        return tuple(dynamic(e) for e in x)
    return int(x)


def imin(a, b):
    return a if a <= b else b  # keeps the static flag of the chosen operand, as `min` does


def sign(a):
    v = (a > 0) - (a < 0)
    return S(v) if isinstance(a, S) else v


ONE, ZERO = S(1), S(0)


def is_static_value(x, v):
    return isinstance(x, S) and int(x) == v


# --------------------------------------------------------------------------- tuple helpers
def flatten(x):
    """src/algorithm/tuple_algorithms.jl `flatten`: leaves in order; an int stays an int."""
    if not is_tuple(x):
        return x
    out = ()
    for e in x:
        f = flatten(e)
        out += f if is_tuple(f) else (f,)
    return out


def flatten_to_tuple(x):
    f = flatten(x)
    return f if is_tuple(f) else (f,)


def unflatten(flat, profile):
    """Inverse of flatten against a nesting profile (tuple_algorithms.jl `unflatten`)."""
    if not is_tuple(profile):
        return flat[0] if is_tuple(flat) else flat
    it = iter(flat)

    def build(p):
        if is_tuple(p):
            return tuple(build(e) for e in p)
        return next(it)

    return build(profile)


def product(x):
    """src/int_tuple.jl `product`."""
    if not is_tuple(x):
        return x
    p = ONE
    for e in x:
        p = p * product(e)
    return p


def product_each(x):
    return tuple(product(e) for e in x)


def rank(x):
    return len(x) if is_tuple(x) else 1


def depth(x):
    if not is_tuple(x):
        return 0
    return 1 + max((depth(e) for e in x), default=0)


def capacity(x):
    return product(x)


def front(x):
    """First leaf-or-mode of a tuple, the value itself for an int."""
    return x[0] if is_tuple(x) else x


def back(x):
    return x[-1] if is_tuple(x) else x


def as_tuple(x):
    return x if is_tuple(x) else (x,)


def unwrap(x):
    """tuple_algorithms.jl `unwrap`: a 1-tuple decays to its element."""
    while is_tuple(x) and len(x) == 1:
        x = x[0]
    return x


def append(t, v, n=None):
    """`append(t, v)` or `append(t, v, N)`: pad with v up to rank N."""
    t = as_tuple(t)
    if n is None:
        return t + (v,)
    return t + (v,) * max(0, int(n) - len(t))


def prepend(t, v, n=None):
    t = as_tuple(t)
    if n is None:
        return (v,) + t
    return (v,) * max(0, int(n) - len(t)) + t


def replace_front(t, v):
    return (v,) + t[1:] if is_tuple(t) else v


def repeat_like(t, v):
    if is_tuple(t):
        return tuple(repeat_like(e, v) for e in t)
    return v


def shape_div(a, b):
    """src/int_tuple.jl:84-101."""
    if is_tuple(a):
        if is_tuple(b):
            assert len(a) == len(b)
            return tuple(shape_div(x, y) for x, y in zip(a, b))
        res = []
        for ai in a:
            res.append(shape_div(ai, b))
            b = shape_div(b, product(ai))
        return tuple(res)
    if is_tuple(b):
        return shape_div(a, product(b))
    if isinstance(a, S) and isinstance(b, S):
        assert int(a) % int(b) == 0 or int(b) % int(a) == 0, f"Cannot divide {a} by {b} or vice versa"
    q = idiv(a, b)
    if q != 0:
        return q
    return sign(a) * sign(b)


def elem_scale(x, y):
    """src/int_tuple.jl:103-109."""
    if is_tuple(x):
        return tuple(elem_scale(a, b) for a, b in zip(x, y))
    return x * capacity(y)


def iscompatible(a, b):
    """src/int_tuple.jl:116-120: any coordinate into a is a coordinate into b."""
    if is_tuple(a):
        return is_tuple(b) and len(a) == len(b) and all(iscompatible(x, y) for x, y in zip(a, b))
    return a == capacity(b)


def iscongruent(a, b):
    return repeat_like(a, 0) == repeat_like(b, 0)


def filter_zeros(stride, shape):
    """Extents paired with a *static* zero stride become static 1 (int_tuple.jl:123-128)."""
    if is_tuple(stride):
        return tuple(filter_zeros(d, s) for d, s in zip(stride, shape))
    return ONE if is_static_value(stride, 0) else shape


def tuple_cat(parts):
    out = ()
    for p in parts:
        out += p
    return out


def slice_(a, idx):
    """Keep the modes whose coordinate is `:` (int_tuple.jl:130-143)."""
    if is_tuple(idx):
        assert is_tuple(a) and len(a) == len(idx)
        return tuple_cat(slice_(x, i) for x, i in zip(a, idx))
    return (a,) if idx == COLON else ()


def dice(a, idx):
    """Keep the modes whose coordinate is an integer (int_tuple.jl:145-156)."""
    if is_tuple(idx):
        assert is_tuple(a) and len(a) == len(idx)
        return tuple_cat(dice(x, i) for x, i in zip(a, idx))
    return () if idx == COLON else (a,)


def has_colon(c):
    if is_tuple(c):
        return any(has_colon(e) for e in c)
    return c == COLON


def elem_less(a, b):
    """src/int_tuple.jl:196-211 (an exhausted left tuple is "less")."""
    if not is_tuple(a) and not is_tuple(b):
        return a < b
    if len(a) == 0:
        return True
    if len(b) == 0:
        return False
    x, y = a[0], b[0]
    if len(a) == 1 and len(b) == 1:
        return x < y
    if not (x == y or elem_less(x, y)):
        return False
    return elem_less(a[1:], b[1:])


def colex_less(a, b):
    """src/int_tuple.jl:184-194: the last element is the most significant."""
    if not is_tuple(a) and not is_tuple(b):
        return a < b
    if len(a) == 0:
        return len(b) != 0
    if len(b) == 0:
        return False
    x, y = a[-1], b[-1]
    if x != y:
        return colex_less(x, y)
    return colex_less(a[:-1], b[:-1])


def increment(coord, shape):
    """Next 1-based hierarchical coordinate in colexicographic order (src/int_tuple.jl:218-231)."""
    if not is_tuple(coord):
        return coord + 1 if coord < shape else 1
    c, s = coord[0], shape[0]
    if len(coord) == 1 and len(shape) == 1:
        return increment(c, s)
    if c != s:
        return (increment(c, s),) + tuple(coord[1:])
    rest = increment(coord[1:], shape[1:])
    return (repeat_like(s, 1),) + (rest if is_tuple(rest) else (rest,))


def insert(t, v, i):
    """tuple_algorithms.jl `insert` (1-based position)."""
    return t[: i - 1] + (v,) + t[i - 1:]


def remove(t, i):
    return t[: i - 1] + t[i:]


def replace(t, v, i):
    return t[: i - 1] + (v,) + t[i:]


def escan(f, t, init):
    """Exclusive scan (tuple_algorithms.jl `escan`)."""
    out, acc = [], init
    for e in t:
        out.append(acc)
        acc = f(acc, e)
    return tuple(out)


def zip2_by(t, guide):
    """tuple_algorithms.jl:213-224: split every mode that `guide` marks into (tile, rest)."""
    if is_tuple(guide):
        gr = len(guide)
        assert len(t) >= gr
        split = [zip2_by(t[i], guide[i]) for i in range(gr)]
        return (tuple(s[0] for s in split), tuple(s[1] for s in split) + tuple(t[gr:]))
    assert len(t) == 2
    return (t[0], t[1])


def tzip(*ts):
    """tuple_algorithms.jl `_zip`: transpose a tuple of tuples."""
    if len(ts) == 1:
        (t,) = ts
        if is_tuple(t) and t and is_tuple(t[0]):
            return tuple(tuple(e[i] for e in t) for i in range(len(t[0])))
        return t
    return tuple(tuple(t[i] for t in ts) for i in range(len(ts[0])))


# --------------------------------------------------------------------------- coordinates
def coord_to_index0(coord, shape, stride):
    """0-based coordinate -> 0-based offset (src/stride.jl:1-54)."""
    if is_tuple(coord):
        assert is_tuple(shape) and len(coord) == len(shape) == len(stride)
        return sum((coord_to_index0(c, s, d) for c, s, d in zip(coord, shape, stride)), ZERO)
    if not is_tuple(shape):
        return coord * stride
    # integer coordinate into a tuple shape: colexicographic split (src/stride.jl:1-31)
    n = len(shape)
    if n == 1:
        if is_tuple(shape[0]):
            return coord_to_index0(coord, shape[0], stride[0])
        return coord * stride[0]
    result = ZERO
    c = coord
    for s, d in zip(shape, stride):
        if is_tuple(s):
            result = result + coord_to_index0(irem(c, product(s)), s, d)
        else:
            result = result + irem(c, s) * d
        c = idiv(c, product(s))
    return result


def _offset(c):
    """1-based -> 0-based, `:` -> 0 (src/stride.jl:73-80)."""
    if is_tuple(c):
        return tuple(_offset(e) for e in c)
    if c == COLON:
        return ZERO
    return c - ONE


def coord_to_index(coord, shape, stride=None):
    """1-based coordinate -> 1-based index (src/stride.jl:82-89)."""
    if stride is None:
        stride = compact_col_major(shape)
    return coord_to_index0(_offset(coord), shape, stride) + ONE


def index_to_coord(index, shape, stride=None):
    """1-based index -> 1-based (hierarchical) coordinate (src/stride.jl:91-128)."""
    if stride is None:
        if not is_tuple(shape):
            return index
        if is_tuple(index):
            return tuple(index_to_coord(i, s) for i, s in zip(index, shape))
        stride = compact_col_major(shape, ONE)
    if is_tuple(index):
        return tuple(index_to_coord(i, s, d) for i, s, d in zip(index, shape, stride))
    if is_tuple(shape):
        if not is_tuple(stride):
            stride = compact_col_major(shape, stride)
        return tuple(index_to_coord(index, s, d) for s, d in zip(shape, stride))
    if is_static_value(shape, 1):
        return ZERO
    return irem(idiv(index - ONE, stride), shape) + ONE


def coord_to_coord(coord, src_shape, dst_shape):
    """src/stride.jl:133-141."""
    if is_tuple(coord) and is_tuple(src_shape) and is_tuple(dst_shape):
        return tuple(coord_to_coord(c, s, d) for c, s, d in zip(coord, src_shape, dst_shape))
    return index_to_coord(coord_to_index(coord, src_shape), dst_shape)


def _compact(shape, current, left):
    """Returns (strides, next) -- src/stride.jl:168-251."""
    if is_tuple(shape):
        out = []
        seq = shape if left else tuple(reversed(shape))
        for s in seq:
            r, current = _compact(s, current, left)
            out.append(r)
        if not left:
            out.reverse()
        return tuple(out), current
    if is_static_value(shape, 1):
        return ZERO, current
    return current, current * shape


def compact_col_major(shape, current=ONE):
    return _compact(shape, current, True)[0]


def compact_row_major(shape, current=ONE):
    return _compact(shape, current, False)[0]


def compact_order(shape, order):
    """src/stride.jl:253-276: stride of a leaf = product of the extents ordered before it."""
    old_shape = flatten_to_tuple(product_like(shape, order))
    flat_order = flatten_to_tuple(order)
    max_order = ZERO
    for o in flat_order:
        if isinstance(o, S) and isinstance(max_order, S) and max_order <= o:
            max_order = o
    old_order = tuple(o if isinstance(o, S) else S(i + 1) + max_order for i, o in enumerate(flat_order))
    new_order = unflatten(old_order, order)

    def rec(s, o):
        if is_tuple(o):
            return tuple(rec(x, y) for x, y in zip(s, o))
        d = ONE
        for os_, oo in zip(old_shape, old_order):
            if oo < o:
                d = d * product(os_)
        return compact_col_major(s, d)

    return rec(shape, new_order)


def product_like(x, guide):
    """src/int_tuple.jl:55-60: products of x taken at the nesting of guide."""
    if is_tuple(guide):
        return tuple(product_like(a, g) for a, g in zip(x, guide))
    return product(x)


# --------------------------------------------------------------------------- Layout
class Layout:
    """`Layout{N,Shape,Stride}` of src/layout.jl:1-60.  Calling it is the layout function."""

    __slots__ = ("shape", "stride")

    def __init__(self, shape, stride):
        self.shape = shape
        self.stride = stride

    def __call__(self, *coord):
        if len(coord) == 1:
            coord = coord[0]
        if has_colon(coord):
            return slice_layout(self, coord)
        return coord_to_index(coord, self.shape, self.stride)

    def __getitem__(self, i):  # 0-based mode access for Python callers
        return mode(self, i + 1)

    def __eq__(self, other):
        return isinstance(other, Layout) and self.shape == other.shape and self.stride == other.stride

    def __ne__(self, other):
        return not self.__eq__(other)

    def __hash__(self):
        return hash((self.shape, self.stride))

    def __repr__(self):
        return f"{self.shape}:{self.stride}"


GenColMajor = "GenColMajor"
GenRowMajor = "GenRowMajor"


def make_layout(*args):
    """src/layout.jl:120-180.  make_layout(shape[, stride|order tag]) or make_layout(layouts...)."""
    if args and all(isinstance(a, Layout) for a in args):
        return Layout(tuple(a.shape for a in args), tuple(a.stride for a in args))
    if len(args) == 1:
        return Layout(args[0], compact_col_major(args[0]))
    shape, second = args
    if second == GenColMajor:
        return Layout(shape, compact_col_major(shape))
    if second == GenRowMajor:
        return Layout(shape, compact_row_major(shape))
    assert iscongruent(shape, second), f"shape {shape} and stride {second} are not congruent"
    return Layout(shape, second)


def SL(shape, stride=None):
    """`@Layout shape stride`: every leaf static."""
    if stride is None:
        return make_layout(static(shape))
    if stride in (GenColMajor, GenRowMajor):
        return make_layout(static(shape), stride)
    return make_layout(static(shape), static(stride))


def make_ordered_layout(shape, order=None):
    """src/layout.jl:182-221: compact layout whose stride order follows `order`."""
    if isinstance(shape, Layout) and order is None:
        return make_ordered_layout(shape.shape, shape.stride)
    if order in (GenColMajor, GenRowMajor):
        return make_layout(shape, order)
    return Layout(shape, compact_order(shape, order))


def make_layout_like(layout):
    """src/layout.jl:223-225."""
    return make_ordered_layout(layout.shape, filter_zeros(layout.stride, layout.stride))


def shape(l, *idx):
    s = l.shape
    for i in idx:
        s = s[i - 1]
    return s


def stride(l, *idx):
    s = l.stride
    for i in idx:
        s = s[i - 1]
    return s


def mode(l, i):
    """`layout[i]` (1-based)."""
    if not is_tuple(l.shape):
        assert i == 1
        return l
    return Layout(l.shape[i - 1], l.stride[i - 1])


def lrank(l):
    return rank(l.shape)


def ldepth(l):
    return depth(l.shape)


def size(l, *idx):
    return capacity(shape(l, *idx)) if isinstance(l, Layout) else capacity(l)


def cosize(l):
    """src/layout.jl:330-340: `layout(size(layout))`."""
    return l(size(l))


def lflatten(l):
    return Layout(flatten(l.shape), flatten(l.stride))


def lappend(l, n):
    """`append(layout, N)`: pad with `1:0` modes up to rank N (src/layout.jl:262-275)."""
    s, d = as_tuple(l.shape), as_tuple(l.stride)
    if not is_tuple(l.shape) and int(n) == 1:
        return l
    k = max(0, int(n) - len(s))
    return Layout(s + (ONE,) * k, d + (ZERO,) * k)


def lprepend(l, n):
    s, d = as_tuple(l.shape), as_tuple(l.stride)
    k = max(0, int(n) - len(s))
    return Layout((ONE,) * k + s, (ZERO,) * k + d)


def group(l, b, e):
    """`group(layout, B, E)`: fold modes B..E (1-based, inclusive) into one (tuple_algorithms.jl:179-190)."""
    def g(t):
        t = as_tuple(t)
        return t[: b - 1] + (t[b - 1:e],) + t[e:]
    return Layout(g(l.shape), g(l.stride))


def slice_layout(l, coord):
    """`layout(coord)` with colons: the sub-layout of the `:` modes (src/layout.jl:364-367)."""
    return make_layout(unwrap_keep(slice_(l.shape, coord)), unwrap_keep(slice_(l.stride, coord)))


def unwrap_keep(t):
    # a sliced layout keeps tuple form unless exactly one leaf remains
    if is_tuple(t) and len(t) == 1 and not is_tuple(t[0]):
        return t[0]
    if is_tuple(t) and len(t) == 1:
        return t[0]
    return t


def slice_and_offset(l, coord):
    """src/layout.jl:368-371: sliced layout and the 0-based offset of its origin."""
    return slice_layout(l, coord), coord_to_index0(_offset(coord), l.shape, l.stride)


def dice_layout(l, coord):
    return make_layout(unwrap_keep(dice(l.shape, coord)), unwrap_keep(dice(l.stride, coord)))


def get_congr_coord(l, index):
    """src/layout.jl:115-119: hierarchical coordinate of a 1-based index under l's own strides."""
    return index_to_coord(index, l.shape, l.stride)


# --------------------------------------------------------------------------- coalesce
def bw_coalesce(old_shape, old_stride, new_shape, new_stride):
    """src/layout.jl:441-479, walking old modes from last to first."""
    for i in range(len(old_shape) - 1, -1, -1):
        s, d = old_shape[i], old_stride[i]
        if is_static_value(s, 1):
            continue
        if is_static_value(new_shape, 1):
            new_shape, new_stride = s, d
        elif (isinstance(front(new_shape), S) and isinstance(s, S) and isinstance(d, S)
              and isinstance(front(new_stride), S) and s * d == front(new_stride)):
            new_shape = replace_front(new_shape, s * front(new_shape))
            new_stride = replace_front(new_stride, d)
        else:
            new_shape = prepend(new_shape, s)
            new_stride = prepend(new_stride, d)
    if is_static_value(new_shape, 1):
        return Layout(ONE, ZERO)
    return Layout(new_shape, new_stride)


def coalesce(l, profile=None):
    """src/layout.jl:497-506."""
    if profile is not None and is_tuple(profile):
        assert len(profile) <= lrank(l)
        modes = [coalesce(mode(l, i + 1), profile[i]) for i in range(len(profile))]
        modes += [mode(l, i + 1) for i in range(len(profile), lrank(l))]
        return make_layout(*modes)
    fs, fd = flatten_to_tuple(l.shape), flatten_to_tuple(l.stride)
    return bw_coalesce(fs[:-1], fd[:-1], fs[-1], fd[-1])


def lfilter_zeros(l):
    return make_layout(filter_zeros(l.stride, l.shape), l.stride)


def lfilter(l):
    """`filter(layout)` (src/layout.jl:511-517)."""
    return coalesce(lfilter_zeros(l))


# --------------------------------------------------------------------------- composition
def _composition_leaf(ls, ld, rs, rd):
    """LHS (flattened shape/stride) against one RHS leaf rs:rd (src/layout.jl:520-565)."""
    if is_static_value(rd, 0):
        return Layout(rs, rd)
    if not is_tuple(ls):
        return Layout(rs, ld * rd)
    s0, d0 = ls[:-1], ld[:-1]
    if is_static_value(rd, 1):
        s1, d1, rest_stride = s0, d0, None
    else:
        s1, rest = [], rd
        for si in s0:
            s1.append(shape_div(si, rest))
            rest = shape_div(rest, si)
        s1 = tuple(s1)
        d1 = elem_scale(d0, shape_div(s0, s1))
        rest_stride = rest
    s2, rem = [], rs
    for si in s1:
        s2.append(imin(abs(si), rem))
        rem = shape_div(rem, abs(si))
    last = ld[-1] if rest_stride is None else rest_stride * ld[-1]
    return bw_coalesce(tuple(s2), d1 if rest_stride is not None else d0, rem, last)


def _composition_sd(ls, ld, rs, rd):
    if is_tuple(rs):
        parts = [_composition_sd(ls, ld, a, b) for a, b in zip(rs, rd)]
        return make_layout(*parts)
    return _composition_leaf(ls, ld, rs, rd)


def composition(lhs, rhs):
    """`lhs ∘ rhs` (src/layout.jl:567-608)."""
    if rhs == COLON:
        return lhs
    if isinstance(rhs, Layout):
        return _composition_sd(flatten(lhs.shape), flatten(lhs.stride), rhs.shape, rhs.stride)
    if is_tuple(rhs) and any(isinstance(r, Layout) or r == COLON for r in rhs):
        assert len(rhs) <= lrank(lhs)
        modes = [composition(mode(lhs, i + 1), rhs[i]) for i in range(len(rhs))]
        modes += [mode(lhs, i + 1) for i in range(len(rhs), lrank(lhs))]
        return make_layout(*modes)
    return composition(lhs, make_layout(rhs))


def withshape(l, shp):
    return composition(l, make_layout(shp))


# --------------------------------------------------------------------------- complement
def _complement(shp, strd, cotarget):
    """src/layout.jl:621-652.  Strides must be static."""
    if not is_tuple(shp):
        if is_static_value(strd, 0):
            return make_layout(cotarget)
        shp, strd = (shp,), (strd,)
    assert is_static(strd), "complement needs static strides"
    shp, strd = list(shp), list(strd)
    r_shape, r_stride = [], [ONE]
    for i in range(len(shp) - 1):
        m = strd[0]
        for d in strd:
            m = imin(m, d)
        k = strd.index(m)
        ns = idiv(m, r_stride[i])
        assert ns != 0
        r_shape.append(ns)
        r_stride.append(m * shp[k])
        del shp[k], strd[k]
    ns = idiv(strd[0], r_stride[-1])
    assert ns != 0
    r_shape.append(ns)
    new_stride = shp[0] * strd[0]
    rest_shape = _cld(cotarget, new_stride)
    rest_stride = compact_col_major(rest_shape, new_stride)
    return coalesce(make_layout((tuple(r_shape), rest_shape), (tuple(r_stride), rest_stride)))


def _cld(a, b):
    v = -((-int(a)) // int(b))
    return S(v) if isinstance(a, S) and isinstance(b, S) else v


def complement(l, cotarget=None):
    """src/layout.jl:654-668."""
    f = lfilter(l)
    if cotarget is None:
        cotarget = cosize(f)
    return _complement(f.shape, f.stride, cotarget)


# --------------------------------------------------------------------------- inverses
def right_inverse(l):
    """src/layout.jl:670-730."""
    if l == COLON:
        return l
    f = coalesce(l)
    fs, fd = as_tuple(f.shape), as_tuple(f.stride)
    astride = tuple(abs(d) for d in fd)
    nxt = None
    for i, d in enumerate(astride):
        if is_static_value(d, 1):
            nxt = i
            break
    if nxt is None:
        return Layout(ONE, ZERO)
    seq = []
    while nxt is not None and nxt not in seq:
        seq.append(nxt)
        ns = astride[nxt] * fs[nxt]
        if not isinstance(ns, S):
            break
        nxt = next((j for j, d in enumerate(astride) if isinstance(d, S) and d == ns), None)
    rstride = as_tuple(compact_col_major(f.shape))
    rs = tuple(fs[i] for i in seq)
    rd = tuple(sign(fd[i]) * rstride[i] for i in seq)
    return make_layout(unwrap(rs), unwrap(rd))


def left_inverse(l):
    """src/layout.jl:738."""
    if l == COLON:
        return l
    return right_inverse(make_layout(l, complement(l)))


def max_common_vector(a, b):
    """src/layout.jl:752-761."""
    inv_b = right_inverse(b)
    common = coalesce(composition(a, inv_b))
    s1, d1 = front(common.shape), front(common.stride)
    if isinstance(s1, S) and d1 == 1:
        return s1
    return ONE


# --------------------------------------------------------------------------- products
def tile_unzip(l, tile):
    """src/layout.jl:776-778."""
    guide = _tile_guide(tile)
    return make_layout(zip2_by(l.shape, guide), zip2_by(l.stride, guide))


def _tile_guide(tile):
    if is_tuple(tile):
        return tuple(_tile_guide(t) for t in tile)
    return 0


def logical_product(l, tile):
    """src/layout.jl:826-838."""
    if tile == COLON:
        return l
    if is_tuple(tile):
        modes = [logical_product(mode(l, i + 1), tile[i]) for i in range(len(tile))]
        modes += [mode(l, i + 1) for i in range(len(tile), lrank(l))]
        return make_layout(*modes)
    if not isinstance(tile, Layout):
        tile = make_layout(tile)
    return make_layout(l, composition(complement(l, size(l) * cosize(tile)), tile))


def zipped_product(l, tile):
    return tile_unzip(logical_product(l, tile), tile)


def _unpack_second(d):
    """`d(:, repeat(:, R))`: mode 1 kept, the modes of mode 2 spliced in."""
    s2, d2 = as_tuple(d.shape[1]), as_tuple(d.stride[1])
    return Layout((d.shape[0],) + s2, (d.stride[0],) + d2)


def tiled_product(l, tile):
    """src/layout.jl:843-846."""
    if isinstance(tile, Layout) or not is_tuple(tile):
        lp = logical_product(l, tile)
        return _unpack_second(lp)
    return _unpack_second(zipped_product(l, tile))


def _lzip(a, b):
    return make_layout(tzip(as_tuple(a.shape), as_tuple(b.shape)), tzip(as_tuple(a.stride), as_tuple(b.stride)))


def blocked_product(block, l, coalesce_result=False):
    """src/layout.jl:880-889."""
    r = max(lrank(block), lrank(l))
    res = logical_product(lappend(block, r), lappend(l, r))
    res = _lzip(mode(res, 1), mode(res, 2))
    return coalesce(res, (ONE,) * r) if coalesce_result else res


def raked_product(block, l, coalesce_result=False):
    """src/layout.jl:919-928."""
    r = max(lrank(block), lrank(l))
    res = logical_product(lappend(block, r), lappend(l, r))
    res = _lzip(mode(res, 2), mode(res, 1))
    return coalesce(res, (ONE,) * r) if coalesce_result else res


def tile_to_shape(l, trg_shape, ord_shape=GenColMajor):
    """src/layout.jl:930-935."""
    r = rank(trg_shape)
    padded = lappend(l, r)
    product_shape = shape_div(product_each(trg_shape), product_each(padded.shape))
    return coalesce(blocked_product(padded, make_ordered_layout(product_shape, ord_shape)), product_shape)


# --------------------------------------------------------------------------- recast
def upcast(l, m):
    """src/layout.jl:945-970."""
    m = S(m)

    def f(s, d):
        if is_tuple(s):
            return make_layout(*[f(a, b) for a, b in zip(s, d)])
        if is_static_value(d, 0):
            return Layout(s, d)
        if isinstance(d, S):
            return Layout(shape_div(s, shape_div(m, abs(d))), shape_div(d, m))
        assert d % int(m) == 0, "Safe division failed"
        return Layout(s, d // int(m))

    return f(l.shape, l.stride)


def downcast(l, m):
    """src/layout.jl:972-1000."""
    m = S(m)

    def f(s, d):
        if is_tuple(s):
            return make_layout(*[f(a, b) for a, b in zip(s, d)])
        if d == 1 or (isinstance(d, S) and d == -1):
            return Layout(s * m, d)
        return Layout(s, d * m)

    return f(l.shape, l.stride)


def recast(l, new_bytes, old_bytes):
    """src/layout.jl:1002-1010."""
    if new_bytes == old_bytes:
        return l
    if new_bytes > old_bytes:
        assert new_bytes % old_bytes == 0
        return upcast(l, new_bytes // old_bytes)
    assert old_bytes % new_bytes == 0
    return downcast(l, old_bytes // new_bytes)


# --------------------------------------------------------------------------- divides
def logical_divide(l, tile):
    """src/layout.jl:1058-1070."""
    if tile == COLON:
        return l
    if is_tuple(tile):
        assert len(tile) <= lrank(l), "too many modes in tile"
        modes = [logical_divide(mode(l, i + 1), tile[i]) for i in range(len(tile))]
        modes += [mode(l, i + 1) for i in range(len(tile), lrank(l))]
        return make_layout(*modes)
    if not isinstance(tile, Layout):
        tile = make_layout(tile)
    return composition(l, make_layout(tile, complement(tile, size(l))))


def zipped_divide(l, tile):
    """src/layout.jl:1114-1116."""
    return tile_unzip(logical_divide(l, tile), tile)


def tiled_divide(l, tile):
    """src/layout.jl:1123-1127."""
    return _unpack_second(zipped_divide(l, tile))


def make_fragment_like(l):
    """src/layout.jl:1143-1149."""
    if isinstance(l, Layout):
        if is_static(l.shape) and is_static(l.stride):
            if lrank(l) == 1:
                return make_layout(l.shape)
            rest = make_layout(*[mode(l, i) for i in range(2, lrank(l) + 1)])
            return tiled_product(make_layout(l.shape[0]), make_ordered_layout(rest))
        return make_layout(l.shape)
    return make_layout(l)


# --------------------------------------------------------------------------- tensors (views)
class View(namedtuple("View", ["data", "offset", "layout"])):
    """A non-owning MoYeArray over a flat numpy buffer: engine pointer = (data, offset)
    (src/array.jl:53-59, src/engine.jl:6-48).  Indexing is 1-based through the layout."""

    __slots__ = ()

    def at(self, *coord):
        if len(coord) == 1:
            coord = coord[0]
        return self.offset + int(self.layout(coord)) - 1

    def get(self, *coord):
        return self.data[self.at(*coord)]

    def set(self, value, *coord):
        self.data[self.at(*coord)] = value

    def view(self, *coord):
        """`view(x, coord...)` = slice_and_offset (src/array.jl:221-237)."""
        if len(coord) == 1 and is_tuple(coord[0]):
            coord = coord[0]
        sl, off = slice_and_offset(self.layout, tuple(coord))
        return View(self.data, self.offset + int(off), sl)


def make_view(data, layout, offset=0):
    return View(data, offset, layout)


def vzipped_divide(x, tile):
    return View(x.data, x.offset, zipped_divide(x.layout, tile))


def local_tile(x, tile, coord, proj=None):
    """`@tile x tile coord` (src/algorithm/array_algorithms.jl:113-120)."""
    if proj is not None:
        return local_tile(x, dice(tile, proj), dice(coord, proj))
    r1, r2 = len(tile), lrank(x.layout)
    z = vzipped_divide(x, tile)
    return z.view(((COLON,) * r1, append(coord, COLON, r2)))


def local_partition(x, tile, coord, proj=None):
    """`@parallelize x threadlayout idx [proj]` (array_algorithms.jl:36-47)."""
    if isinstance(tile, Layout):
        if proj is not None:
            shp = tuple(capacity(s) for s in as_tuple(tile.shape))
            return local_partition(x, dice(shp, proj), as_tuple(get_congr_coord(dice_layout(tile, proj), coord)))
        shp = tuple(capacity(s) for s in as_tuple(tile.shape))
        return local_partition(x, shp, as_tuple(get_congr_coord(tile, coord)))
    if proj is not None:
        return local_partition(x, dice(tile, proj), dice(coord, proj))
    n = lrank(x.layout)
    z = vzipped_divide(x, tile)
    return z.view((tuple(coord), (COLON,) * n))


def copyto(dst, src):
    """Elementwise `copyto!(dst, src)`: 1-D index through both layouts
    (src/algorithm/copy.jl:4-16,42-64)."""
    n = int(size(src.layout))
    assert int(size(dst.layout)) == n
    for i in range(1, n + 1):
        dst.data[dst.at(i)] = src.data[src.at(i)]
