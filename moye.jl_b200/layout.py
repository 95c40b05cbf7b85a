"""Host-side layout algebra of the B200 path: MoYe's `Layout` and its operations.

This mirrors the public names of MoYe.jl's layout layer (reference src/layout.jl,
src/stride.jl, src/int_tuple.jl) so that tile shapes, thread-value maps, swizzles and TMA
descriptors are derived on the host exactly as MoYe derives them.  Conventions kept from the
reference: shapes and strides are nested tuples of ints; public indices and coordinates are
1-based; `layout(i)` walks the shape colexicographically.

Unlike the reference there is no static/dynamic distinction: every extent is a known Python
int at the time a kernel is configured, which corresponds to MoYe's all-static (`@Layout`)
behaviour.  Function values are identical either way (reference docs/src/manual/layout.md:43-56).
"""
from functools import reduce

__all__ = [
    "Layout", "make_layout", "make_ordered_layout", "GenColMajor", "GenRowMajor", "COLON",
    "flatten", "unflatten", "product", "product_each", "rank", "depth", "capacity", "shape_div", "elem_scale",
    "iscompatible", "slice_tuple", "dice_tuple", "coord_to_index", "index_to_coord", "coord_to_coord",
    "compact_col_major", "compact_row_major", "compact_order", "size", "cosize", "coalesce", "filter_layout",
    "composition", "complement", "right_inverse", "left_inverse", "logical_product", "zipped_product",
    "tiled_product", "blocked_product", "raked_product", "tile_to_shape", "logical_divide", "zipped_divide",
    "tiled_divide", "upcast", "downcast", "recast_layout", "make_fragment_like", "max_common_vector",
    "get_congr_coord", "append_layout", "prepend_layout", "group_modes", "Swizzle", "ComposedLayout", "print_layout",
]

COLON = ":"
GenColMajor = "GenColMajor"
GenRowMajor = "GenRowMajor"


def _is_t(x):
    return isinstance(x, tuple)


def _tup(x):
    return x if _is_t(x) else (x,)


def _tdiv(a, b):
    q = abs(a) // abs(b)
    return q if (a >= 0) == (b >= 0) else -q


def _sgn(a):
    return (a > 0) - (a < 0)


# ------------------------------------------------------------------------------ IntTuple
def flatten(x):
    """Leaves of a nested tuple in order (reference src/algorithm/tuple_algorithms.jl `flatten`)."""
    if not _is_t(x):
        return x
    out = []
    stack = [x]
    while stack:
        cur = stack.pop()
        if _is_t(cur):
            stack.extend(reversed(cur))
        else:
            out.append(cur)
    return tuple(out)


def _flat(x):
    f = flatten(x)
    return f if _is_t(f) else (f,)


def unflatten(flat, profile):
    it = iter(_tup(flat))

    def build(p):
        return tuple(build(e) for e in p) if _is_t(p) else next(it)

    return build(profile)


def product(x):
    return reduce(lambda a, b: a * b, _flat(x), 1) if _is_t(x) else x


def product_each(x):
    return tuple(product(e) for e in x)


def rank(x):
    return len(x) if _is_t(x) else 1


def depth(x):
    return 1 + max((depth(e) for e in x), default=0) if _is_t(x) else 0


capacity = product


def shape_div(a, b):
    """reference src/int_tuple.jl:84-101."""
    if _is_t(a):
        if _is_t(b):
            if len(a) != len(b):
                raise ValueError("shape_div: rank mismatch")
            return tuple(shape_div(x, y) for x, y in zip(a, b))
        out = []
        for ai in a:
            out.append(shape_div(ai, b))
            b = shape_div(b, product(ai))
        return tuple(out)
    if _is_t(b):
        return shape_div(a, product(b))
    if a % b != 0 and b % a != 0:
        raise ValueError(f"cannot divide {a} by {b} or vice versa")
    q = _tdiv(a, b)
    return q if q != 0 else _sgn(a) * _sgn(b)


def elem_scale(x, y):
    if _is_t(x):
        return tuple(elem_scale(a, b) for a, b in zip(x, y))
    return x * product(y)


def iscompatible(a, b):
    if _is_t(a):
        return _is_t(b) and len(a) == len(b) and all(iscompatible(x, y) for x, y in zip(a, b))
    return a == product(b)


def slice_tuple(a, idx):
    """Keep what sits under a `:` (reference src/int_tuple.jl:130-143)."""
    if _is_t(idx):
        out = ()
        for x, i in zip(a, idx):
            out += slice_tuple(x, i)
        return out
    return (a,) if idx == COLON else ()


def dice_tuple(a, idx):
    """Keep what sits under an integer (reference src/int_tuple.jl:145-156)."""
    if _is_t(idx):
        out = ()
        for x, i in zip(a, idx):
            out += dice_tuple(x, i)
        return out
    return () if idx == COLON else (a,)


def _has_colon(c):
    return any(_has_colon(e) for e in c) if _is_t(c) else c == COLON


# ------------------------------------------------------------------------------ coordinates
def _c2i0(coord, shape, stride):
    if _is_t(coord):
        return sum(_c2i0(c, s, d) for c, s, d in zip(coord, shape, stride))
    if not _is_t(shape):
        return coord * stride
    if len(shape) == 1:
        return _c2i0(coord, shape[0], stride[0]) if _is_t(shape[0]) else coord * stride[0]
    total = 0
    for s, d in zip(shape, stride):
        ext = product(s)
        q = _tdiv(coord, ext)
        r = coord - q * ext
        total += _c2i0(r, s, d) if _is_t(s) else r * d
        coord = q
    return total


def _off(c):
    if _is_t(c):
        return tuple(_off(e) for e in c)
    return 0 if c == COLON else c - 1


def coord_to_index(coord, shape, stride=None):
    """1-based (possibly hierarchical) coordinate -> 1-based index (reference src/stride.jl:82-89)."""
    if stride is None:
        stride = compact_col_major(shape)
    return _c2i0(_off(coord), shape, stride) + 1


def index_to_coord(index, shape, stride=None):
    """reference src/stride.jl:91-128."""
    if stride is None:
        if not _is_t(shape):
            return index
        if _is_t(index):
            return tuple(index_to_coord(i, s) for i, s in zip(index, shape))
        stride = compact_col_major(shape)
    if _is_t(index):
        if not (len(index) == len(shape) == len(stride)):
            raise ValueError("index, shape, and stride must have the same rank")
        return tuple(index_to_coord(i, s, d) for i, s, d in zip(index, shape, stride))
    if _is_t(shape):
        if not _is_t(stride):
            stride = compact_col_major(shape, stride)
        if len(shape) != len(stride):
            raise ValueError("shape, and stride must have the same rank")
        return tuple(index_to_coord(index, s, d) for s, d in zip(shape, stride))
    if shape == 1:
        return 0
    q = _tdiv(index - 1, stride)
    return q - _tdiv(q, shape) * shape + 1


def coord_to_coord(coord, src_shape, dst_shape):
    if _is_t(coord) and _is_t(src_shape) and _is_t(dst_shape):
        return tuple(coord_to_coord(c, s, d) for c, s, d in zip(coord, src_shape, dst_shape))
    return index_to_coord(coord_to_index(coord, src_shape), dst_shape)


def _compact(shape, cur, left):
    if _is_t(shape):
        seq = shape if left else shape[::-1]
        out = []
        for s in seq:
            r, cur = _compact(s, cur, left)
            out.append(r)
        return (tuple(out) if left else tuple(out[::-1])), cur
    if shape == 1:
        return 0, cur
    return cur, cur * shape


def compact_col_major(shape, current=1):
    """Column-major compact strides; an extent of 1 gets stride 0 (reference src/stride.jl:168-251)."""
    return _compact(shape, current, True)[0]


def compact_row_major(shape, current=1):
    return _compact(shape, current, False)[0]


def compact_order(shape, order):
    """Strides such that a leaf's stride is the product of all extents ordered before it
    (reference src/stride.jl:253-276)."""
    flat_shape = tuple(product(s) for s in _leaves_like(shape, order))
    flat_order = _flat(order)

    def rec(s, o):
        if _is_t(o):
            return tuple(rec(a, b) for a, b in zip(s, o))
        d = 1
        for fs, fo in zip(flat_shape, flat_order):
            if fo < o:
                d *= fs
        return compact_col_major(s, d)

    return rec(shape, order)


def _leaves_like(shape, guide):
    if _is_t(guide):
        out = []
        for s, g in zip(shape, guide):
            out.extend(_leaves_like(s, g))
        return out
    return [shape]


# ------------------------------------------------------------------------------ Layout
class Layout:
    """`Layout(shape, stride)`: a function from (hierarchical) coordinates to offsets
    (reference src/layout.jl:1-60).  `layout(i)` / `layout(coord)` are 1-based like MoYe;
    `layout.offset0(i0)` is the 0-based form the kernels use."""

    __slots__ = ("shape", "stride")

    def __init__(self, shape, stride=None):
        if stride is None:
            stride = compact_col_major(shape)
        if _shape_profile(shape) != _shape_profile(stride):
            raise ValueError(f"shape {shape} and stride {stride} are not congruent")
        self.shape = shape
        self.stride = stride

    def __call__(self, *coord):
        if len(coord) == 1:
            coord = coord[0]
        if _has_colon(coord):
            return Layout(_unwrap1(slice_tuple(self.shape, coord)), _unwrap1(slice_tuple(self.stride, coord)))
        return coord_to_index(coord, self.shape, self.stride)

    def offset0(self, idx0):
        return _c2i0(idx0, self.shape, self.stride)

    def __getitem__(self, i):
        """Mode `i` (0-based here; MoYe's `layout[i]` is 1-based)."""
        if not _is_t(self.shape):
            if i != 0:
                raise IndexError(i)
            return self
        return Layout(self.shape[i], self.stride[i])

    def __len__(self):
        return rank(self.shape)

    def __eq__(self, other):
        return isinstance(other, Layout) and self.shape == other.shape and self.stride == other.stride

    def __hash__(self):
        return hash((self.shape, self.stride))

    def __repr__(self):
        return f"{self.shape}:{self.stride}"

    def __matmul__(self, other):
        """`A @ B` is MoYe's `A ∘ B`."""
        return composition(self, other)

    def flat(self):
        """(shape, stride) as flat tuples of leaves: what the C ABI takes."""
        return _flat(self.shape), _flat(self.stride)


def _shape_profile(x):
    return tuple(_shape_profile(e) for e in x) if _is_t(x) else 0


def _unwrap1(t):
    return t[0] if _is_t(t) and len(t) == 1 else t


def make_layout(*args):
    """`make_layout(shape[, stride | GenColMajor | GenRowMajor])` or `make_layout(layouts...)`
    (reference src/layout.jl:120-180)."""
    if args and all(isinstance(a, Layout) for a in args):
        return Layout(tuple(a.shape for a in args), tuple(a.stride for a in args))
    if len(args) == 1:
        return Layout(args[0])
    shape, second = args
    if second == GenColMajor:
        return Layout(shape, compact_col_major(shape))
    if second == GenRowMajor:
        return Layout(shape, compact_row_major(shape))
    return Layout(shape, second)


def make_ordered_layout(shape, order=None):
    """reference src/layout.jl:182-221."""
    if isinstance(shape, Layout) and order is None:
        return make_ordered_layout(shape.shape, shape.stride)
    if order in (GenColMajor, GenRowMajor):
        return make_layout(shape, order)
    return Layout(shape, compact_order(shape, order))


def size(l, *modes):
    s = l.shape if isinstance(l, (Layout, ComposedLayout)) else l
    for m in modes:
        s = s[m]
    return product(s)


def cosize(l):
    if isinstance(l, ComposedLayout):
        block = 1 << (l.swizzle.bits + l.swizzle.base + abs(l.swizzle.shift))
        return -(-(cosize(l.layout) + l.offset) // block) * block
    return l(size(l))


def append_layout(l, n):
    """Pad with `1:0` modes up to rank n (reference src/layout.jl:262-275)."""
    if not _is_t(l.shape) and n == 1:
        return l
    s, d = _tup(l.shape), _tup(l.stride)
    k = max(0, n - len(s))
    return Layout(s + (1,) * k, d + (0,) * k)


def prepend_layout(l, n):
    s, d = _tup(l.shape), _tup(l.stride)
    k = max(0, n - len(s))
    return Layout((1,) * k + s, (0,) * k + d)


def group_modes(l, begin, end):
    """Fold modes [begin, end) (0-based) into one mode (reference tuple_algorithms.jl:179-190)."""
    s, d = _tup(l.shape), _tup(l.stride)
    return Layout(s[:begin] + (s[begin:end],) + s[end:], d[:begin] + (d[begin:end],) + d[end:])


def get_congr_coord(l, index):
    """Coordinate of a 1-based index under the layout's own strides (reference src/layout.jl:115-119)."""
    return index_to_coord(index, l.shape, l.stride)


# ------------------------------------------------------------------------------ coalesce
def _bw_coalesce(old_shape, old_stride, new_shape, new_stride):
    """reference src/layout.jl:441-479, all-static case."""
    ns, nd = list(_tup(new_shape)), list(_tup(new_stride))
    scalar_one = not _is_t(new_shape) and new_shape == 1
    for s, d in zip(reversed(old_shape), reversed(old_stride)):
        if s == 1:
            continue
        if scalar_one:
            ns, nd, scalar_one = [s], [d], False
        elif s * d == nd[0]:
            ns[0] *= s
            nd[0] = d
        else:
            ns.insert(0, s)
            nd.insert(0, d)
    if scalar_one or (len(ns) == 1 and ns[0] == 1):
        return Layout(1, 0)
    if len(ns) == 1:
        return Layout(ns[0], nd[0])
    return Layout(tuple(ns), tuple(nd))


def coalesce(l, profile=None):
    """Merge modes that one stride can describe (reference src/layout.jl:497-506)."""
    if profile is not None and _is_t(profile):
        modes = [coalesce(l[i], profile[i]) for i in range(len(profile))]
        modes += [l[i] for i in range(len(profile), len(l))]
        return make_layout(*modes)
    fs, fd = l.flat()
    return _bw_coalesce(fs[:-1], fd[:-1], fs[-1], fd[-1])


def filter_layout(l):
    """`filter(layout)`: drop stride-0 modes, then coalesce (reference src/layout.jl:511-517)."""
    def fz(d, s):
        return tuple(fz(a, b) for a, b in zip(d, s)) if _is_t(d) else (1 if d == 0 else s)
    return coalesce(Layout(fz(l.stride, l.shape), l.stride))


# ------------------------------------------------------------------------------ composition
def _compose_leaf(ls, ld, rs, rd):
    if rd == 0:
        return Layout(rs, 0)
    if not _is_t(ls):
        return Layout(rs, ld * rd)
    head_s, head_d = ls[:-1], ld[:-1]
    rest = rd
    s1 = []
    for si in head_s:
        s1.append(shape_div(si, rest))
        rest = shape_div(rest, si)
    d1 = tuple(d * product(shape_div(a, b)) for d, a, b in zip(head_d, head_s, s1))
    rem = rs
    s2 = []
    for si in s1:
        s2.append(min(abs(si), rem))
        rem = shape_div(rem, abs(si))
    return _bw_coalesce(tuple(s2), d1, rem, rest * ld[-1])


def _compose(ls, ld, rs, rd):
    if _is_t(rs):
        return make_layout(*[_compose(ls, ld, a, b) for a, b in zip(rs, rd)])
    return _compose_leaf(ls, ld, rs, rd)


def composition(lhs, rhs):
    """`lhs ∘ rhs`: R(c) = lhs(rhs(c)) (reference src/layout.jl:520-608).  `lhs` may be a `Swizzle` (the result is a
    `ComposedLayout`) or a `ComposedLayout` (the right-hand side composes with its inner layout)."""
    if isinstance(lhs, Swizzle):
        if not isinstance(rhs, Layout):
            rhs = make_layout(rhs)
        return ComposedLayout(lhs, rhs)
    if isinstance(lhs, ComposedLayout):
        return ComposedLayout(lhs.swizzle, composition(lhs.layout, rhs), lhs.offset)
    if rhs == COLON:
        return lhs
    if isinstance(rhs, Layout):
        fs, fd = lhs.flat()
        if len(fs) == 1:
            fs, fd = fs[0], fd[0]
        return _compose(fs, fd, rhs.shape, rhs.stride)
    if _is_t(rhs) and any(isinstance(r, Layout) or r == COLON for r in rhs):
        if len(rhs) > len(lhs):
            raise ValueError("too many modes in the tiler")
        modes = [composition(lhs[i], rhs[i]) for i in range(len(rhs))]
        modes += [lhs[i] for i in range(len(rhs), len(lhs))]
        return make_layout(*modes)
    return composition(lhs, make_layout(rhs))


# ------------------------------------------------------------------------------ complement
def complement(l, cotarget=None):
    """A layout that, with `l`, tiles [0, cotarget) (reference src/layout.jl:621-668)."""
    f = filter_layout(l)
    if cotarget is None:
        cotarget = cosize(f)
    if not _is_t(f.shape):
        if f.stride == 0:
            return make_layout(cotarget)
        shp, strd = [f.shape], [f.stride]
    else:
        shp, strd = list(f.shape), list(f.stride)
    rs, rd = [], [1]
    while len(shp) > 1:
        m = min(strd)
        k = strd.index(m)
        ext = _tdiv(m, rd[-1])
        if ext == 0:
            raise ValueError("complement: overlapping strides")
        rs.append(ext)
        rd.append(m * shp[k])
        del shp[k], strd[k]
    ext = _tdiv(strd[0], rd[-1])
    if ext == 0:
        raise ValueError("complement: overlapping strides")
    rs.append(ext)
    last = shp[0] * strd[0]
    rest = -((-cotarget) // last)
    return coalesce(Layout((tuple(rs), rest), (tuple(rd), compact_col_major(rest, last))))


# ------------------------------------------------------------------------------ inverses
def right_inverse(l):
    """`l(right_inverse(l)(i)) == i` (reference src/layout.jl:717-730)."""
    f = coalesce(l)
    fs, fd = _tup(f.shape), _tup(f.stride)
    mag = [abs(d) for d in fd]
    if 1 not in mag:
        return Layout(1, 0)
    seq = []
    i = mag.index(1)
    while i is not None and i not in seq:
        seq.append(i)
        nxt = mag[i] * fs[i]
        i = mag.index(nxt) if nxt in mag else None
    col = _tup(compact_col_major(f.shape))
    rs = tuple(fs[k] for k in seq)
    rd = tuple(_sgn(fd[k]) * col[k] for k in seq)
    return Layout(_unwrap1(rs), _unwrap1(rd))


def left_inverse(l):
    return right_inverse(make_layout(l, complement(l)))


def max_common_vector(a, b):
    """Number of contiguous elements both layouts agree on (reference src/layout.jl:752-761)."""
    common = coalesce(composition(a, right_inverse(b)))
    s1 = common.shape[0] if _is_t(common.shape) else common.shape
    d1 = common.stride[0] if _is_t(common.stride) else common.stride
    return s1 if d1 == 1 else 1


# ------------------------------------------------------------------------------ products / divides
def _guide(tile):
    return tuple(_guide(t) for t in tile) if _is_t(tile) else 0


def _zip2_by(t, guide):
    if _is_t(guide):
        parts = [_zip2_by(t[i], guide[i]) for i in range(len(guide))]
        return tuple(p[0] for p in parts), tuple(p[1] for p in parts) + tuple(t[len(guide):])
    return t[0], t[1]


def _tile_unzip(l, tile):
    g = _guide(tile)
    return Layout(_zip2_by(l.shape, g), _zip2_by(l.stride, g))


def _splice_second(l):
    return Layout((l.shape[0],) + _tup(l.shape[1]), (l.stride[0],) + _tup(l.stride[1]))


def _per_mode(fn, l, tile):
    if len(tile) > len(l):
        raise ValueError("too many modes in tile")
    modes = [fn(l[i], tile[i]) for i in range(len(tile))] + [l[i] for i in range(len(tile), len(l))]
    return make_layout(*modes)


def logical_product(l, tile):
    """reference src/layout.jl:826-838."""
    if tile == COLON:
        return l
    if _is_t(tile):
        return _per_mode(logical_product, l, tile)
    if not isinstance(tile, Layout):
        tile = make_layout(tile)
    return make_layout(l, composition(complement(l, size(l) * cosize(tile)), tile))


def zipped_product(l, tile):
    return _tile_unzip(logical_product(l, tile), tile)


def tiled_product(l, tile):
    if _is_t(tile):
        return _splice_second(zipped_product(l, tile))
    return _splice_second(logical_product(l, tile))


def _zip_modes(a, b):
    return Layout(tuple(zip(_tup(a.shape), _tup(b.shape))), tuple(zip(_tup(a.stride), _tup(b.stride))))


def blocked_product(block, l, coalesce_result=False):
    """reference src/layout.jl:880-889."""
    r = max(len(block), len(l))
    res = logical_product(append_layout(block, r), append_layout(l, r))
    res = _zip_modes(res[0], res[1])
    return coalesce(res, (1,) * r) if coalesce_result else res


def raked_product(block, l, coalesce_result=False):
    """reference src/layout.jl:919-928."""
    r = max(len(block), len(l))
    res = logical_product(append_layout(block, r), append_layout(l, r))
    res = _zip_modes(res[1], res[0])
    return coalesce(res, (1,) * r) if coalesce_result else res


def tile_to_shape(l, trg_shape, order=GenColMajor):
    """reference src/layout.jl:930-935."""
    r = rank(trg_shape)
    padded = append_layout(l, r)
    pshape = shape_div(product_each(trg_shape), product_each(_tup(padded.shape)))
    return coalesce(blocked_product(padded, make_ordered_layout(pshape, order)), pshape)


def logical_divide(l, tile):
    """`l ∘ (tile, complement(tile, size(l)))` (reference src/layout.jl:1058-1070)."""
    if tile == COLON:
        return l
    if _is_t(tile):
        return _per_mode(logical_divide, l, tile)
    if not isinstance(tile, Layout):
        tile = make_layout(tile)
    return composition(l, make_layout(tile, complement(tile, size(l))))


def zipped_divide(l, tile):
    """((tile modes), (rest modes)) (reference src/layout.jl:1114-1116)."""
    return _tile_unzip(logical_divide(l, tile), tile)


def tiled_divide(l, tile):
    return _splice_second(zipped_divide(l, tile))


# ------------------------------------------------------------------------------ recast
def upcast(l, m):
    """Layout of the same memory seen as elements m times wider (reference src/layout.jl:945-970)."""
    def f(s, d):
        if _is_t(s):
            return make_layout(*[f(a, b) for a, b in zip(s, d)])
        if d == 0:
            return Layout(s, 0)
        return Layout(shape_div(s, shape_div(m, abs(d))), shape_div(d, m))
    return f(l.shape, l.stride)


def downcast(l, m):
    """reference src/layout.jl:972-1000."""
    def f(s, d):
        if _is_t(s):
            return make_layout(*[f(a, b) for a, b in zip(s, d)])
        return Layout(s * m, d) if abs(d) == 1 else Layout(s, d * m)
    return f(l.shape, l.stride)


def recast_layout(l, new_bytes, old_bytes):
    if new_bytes == old_bytes:
        return l
    if new_bytes > old_bytes:
        if new_bytes % old_bytes:
            raise ValueError("cannot recast")
        return upcast(l, new_bytes // old_bytes)
    if old_bytes % new_bytes:
        raise ValueError("cannot recast")
    return downcast(l, old_bytes // new_bytes)


def make_fragment_like(l):
    """Compact layout of the same shape: first mode column-major, the rest in the source's
    stride order (reference src/layout.jl:1143-1149)."""
    if not isinstance(l, Layout):
        return make_layout(l)
    if len(l) == 1:
        return make_layout(l.shape)
    rest = make_layout(*[l[i] for i in range(1, len(l))])
    return tiled_product(make_layout(l.shape[0]), make_ordered_layout(rest))


# ------------------------------------------------------------------------------ swizzle
class Swizzle:
    """The XOR swizzle functor `Swizzle{B,M,S}`: bits [M+S, M+S+B) of a 0-based offset are XOR-ed into bits
    [M, M+B).  MoYe lists bank-conflict swizzling as missing (reference README.md:14-17); the B200 kernels need
    it because TMA and tcgen05 agree on the 128-byte pattern `Swizzle(3, 4, 3)` over byte offsets.  A swizzle
    composes with a layout: `Swizzle(3, 4, 3) @ layout` (or `composition(swizzle, layout)`) is the layout
    function followed by the XOR, a `ComposedLayout`."""

    __slots__ = ("bits", "base", "shift")

    def __init__(self, bits, base, shift):
        if bits < 0 or base < 0 or abs(shift) < bits:
            raise ValueError("invalid swizzle")
        self.bits, self.base, self.shift = bits, base, shift

    def __call__(self, offset0):
        mask = ((1 << self.bits) - 1) << (self.base + self.shift)
        return offset0 ^ ((offset0 & mask) >> self.shift)

    def __matmul__(self, other):
        return composition(self, other)

    def __eq__(self, other):
        return isinstance(other, Swizzle) and (self.bits, self.base, self.shift) == (other.bits, other.base, other.shift)

    def __hash__(self):
        return hash((self.bits, self.base, self.shift))

    def __repr__(self):
        return f"Swizzle({self.bits},{self.base},{self.shift})"


class ComposedLayout:
    """`swizzle ∘ offset ∘ layout`: the offset of `layout`, shifted by a constant, then XOR-swizzled.  Everything
    about the domain (shape, rank, size, slicing a mode, composing with another layout on the right) is the inner
    layout's; only the value changes.  Evaluation is 1-based like `Layout`: `(S ∘ L)(i) = S(L(i) - 1 + offset) + 1`.
    The image of a swizzle is a permutation of aligned blocks of 2^(M+S+B) offsets, so `cosize` is the inner
    layout's rounded up to such a block."""

    __slots__ = ("swizzle", "offset", "layout")

    def __init__(self, swizzle, layout, offset=0):
        if not isinstance(swizzle, Swizzle) or not isinstance(layout, Layout):
            raise TypeError("ComposedLayout(Swizzle, Layout[, offset])")
        self.swizzle, self.layout, self.offset = swizzle, layout, int(offset)

    shape = property(lambda self: self.layout.shape)
    stride = property(lambda self: self.layout.stride)

    def __call__(self, *coord):
        if len(coord) == 1:
            coord = coord[0]
        inner = self.layout(coord)
        if isinstance(inner, Layout):  # a slice: the kept modes, the fixed ones folded into the offset
            return ComposedLayout(self.swizzle, inner, self.offset + self.layout(_first_coord(coord, self.layout.shape)) - 1)
        return self.swizzle(inner - 1 + self.offset) + 1

    def offset0(self, idx0):
        return self.swizzle(self.layout.offset0(idx0) + self.offset)

    def __getitem__(self, i):
        return ComposedLayout(self.swizzle, self.layout[i], self.offset)

    def __len__(self):
        return len(self.layout)

    def __eq__(self, other):
        return (isinstance(other, ComposedLayout) and self.swizzle == other.swizzle and self.layout == other.layout
                and self.offset == other.offset)

    def __hash__(self):
        return hash((self.swizzle, self.layout, self.offset))

    def __matmul__(self, other):
        return composition(self, other)

    def __repr__(self):
        off = f" o {self.offset}" if self.offset else ""
        return f"{self.swizzle!r}{off} o {self.layout!r}"


def _first_coord(coord, shape):
    """`coord` with every colon replaced by the first coordinate of its mode (all ones)."""
    if coord == COLON:
        return tuple(_first_coord(COLON, s) for s in shape) if _is_t(shape) else 1
    if _is_t(coord):
        return tuple(_first_coord(c, s) for c, s in zip(coord, shape))
    return coord


def print_layout(layout, file=None):
    """`print_layout(layout)` for a rank-2 layout: the table of 1-based indices, rows = mode 1, columns = mode 2
    (reference src/print.jl:7-44, same cell widths and rulers).  Returns the text as well."""
    if len(layout) != 2:
        raise ValueError("print_layout takes a rank-2 layout (a swizzled one is fine)")
    rows, cols = size(layout[0]), size(layout[1])
    w = len(str(cosize(layout))) + 2
    rule = "    " + ("+-----------------"[:w + 1]) * cols + "+"
    out = [repr(layout), "    " + "".join("  " + str(n).rjust(w - 2) + " " for n in range(1, cols + 1))]
    for m in range(1, rows + 1):
        out.append(rule)
        out.append(str(m).rjust(2) + "  " + "".join("| " + str(layout(m, n)).rjust(w - 2) + " " for n in range(1, cols + 1)) + "|")
    out.append(rule)
    text = "\n".join(out)
    print(text, file=file)
    return text
