"""`MoYeArray`: a tensor = engine (pointer) + layout, and the tiling views built on it.

Mirrors reference src/array.jl:53-59 (`MoYeArray{T,N,E,L}`), src/engine.jl:6-48
(`ViewEngine`), src/pointer.jl:1-20 (`isgmem`) and src/algorithm/array_algorithms.jl:36-47,
113-120 (`local_partition` / `@parallelize`, `local_tile` / `@tile`).  The engine here is a
torch tensor used purely as a typed pointer into device (or host) memory; all indexing goes
through the layout, 1-based like MoYe.
"""
import torch

from . import _lib
from .layout import (COLON, Layout, _c2i0, _off, _tup, _unwrap1, dice_tuple, get_congr_coord, make_layout,
                     make_fragment_like as _fragment_layout, product, rank, recast_layout, size, slice_tuple,
                     zipped_divide)

__all__ = ["MoYeArray", "isgmem", "local_tile", "local_partition", "tile", "parallelize", "zeros_",
           "make_fragment_like_array", "recast", "transpose", "TORCH_TO_MOYE"]

TORCH_TO_MOYE = {
    torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.int8: _lib.S8,
    torch.uint8: _lib.U8, torch.int32: _lib.S32, torch.int16: _lib.U16, torch.int64: _lib.U64,
}
if hasattr(torch, "float8_e4m3fn"):
    TORCH_TO_MOYE[torch.float8_e4m3fn] = _lib.E4M3
if hasattr(torch, "uint16"):
    TORCH_TO_MOYE[torch.uint16] = _lib.U16


class MoYeArray:
    """A non-owning view: `storage` (a 1-D torch tensor standing for the engine's pointer),
    an element `offset` into it, and a `Layout`.

    `MoYeArray(tensor, layout)` views `tensor`'s memory through `layout` (the tensor's own
    shape is ignored, as `MoYeArray(pointer(A), layout)` does in the reference);
    `MoYeArray(tensor)` with no layout takes the tensor's shape and strides.
    """

    __slots__ = ("storage", "offset", "layout", "_abi")

    def __init__(self, data, layout=None, offset=0):
        if isinstance(data, MoYeArray):
            storage, offset = data.storage, data.offset + offset
        elif isinstance(data, torch.Tensor):
            if layout is None:
                if data.dim() == 0:
                    layout = Layout(1, 0)
                elif data.dim() == 1:
                    layout = Layout(data.shape[0], data.stride(0))
                else:
                    layout = Layout(tuple(data.shape), tuple(data.stride()))
            storage = data.as_strided((_span(data),), (1,)) if data.numel() else data.reshape(-1)
        else:
            raise TypeError("MoYeArray wraps a torch.Tensor (used as a typed pointer) or another MoYeArray")
        if not isinstance(layout, Layout):
            layout = make_layout(layout)
        if storage.dtype not in TORCH_TO_MOYE:
            raise TypeError(f"unsupported element type {storage.dtype}")
        self.storage, self.offset, self.layout = storage, int(offset), layout
        self._abi = None  # cached C-ABI descriptor (the view is immutable)

    # -- engine
    @property
    def dtype(self):
        return TORCH_TO_MOYE[self.storage.dtype]

    @property
    def elem_bytes(self):
        return self.storage.element_size()

    @property
    def ptr(self):
        """Address of element 1 (`pointer(x)`)."""
        return self.storage.data_ptr() + self.offset * self.elem_bytes

    @property
    def device(self):
        return self.storage.device

    # -- layout
    @property
    def shape(self):
        return self.layout.shape

    @property
    def stride(self):
        return self.layout.stride

    def size(self, *modes):
        return size(self.layout, *modes)

    def __len__(self):
        return size(self.layout)

    def rank(self):
        return rank(self.layout.shape)

    # -- element access (host-side convenience; the kernels never go through this)
    def _index0(self, coord):
        if len(coord) == 1:
            coord = coord[0]
        return self.offset + _c2i0(_off(coord), self.layout.shape, self.layout.stride)

    def __getitem__(self, coord):
        coord = coord if isinstance(coord, tuple) else (coord,)
        if any(_colon_in(c) for c in coord):
            return self.view(*coord)
        return self.storage[self._index0(coord)].item()

    def __setitem__(self, coord, value):
        coord = coord if isinstance(coord, tuple) else (coord,)
        self.storage[self._index0(coord)] = value

    def view(self, *coord):
        """`view(x, coord...)`: fix the integer coordinates, keep the `:` modes
        (reference src/array.jl:221-237 -> `slice_and_offset`, src/layout.jl:364-371)."""
        if len(coord) == 1:
            coord = coord[0]
        sl = Layout(_unwrap1(slice_tuple(self.layout.shape, coord)), _unwrap1(slice_tuple(self.layout.stride, coord)))
        off = _c2i0(_off(coord), self.layout.shape, self.layout.stride)
        return MoYeArray(self, sl, off)

    def with_layout(self, layout):
        return MoYeArray(self, layout)

    def to_torch(self):
        """The elements in colexicographic order as a new 1-D tensor (gathers through the layout)."""
        fs, fd = self.layout.flat()
        idx = torch.zeros(1, dtype=torch.int64, device=self.device)
        for s, d in zip(fs, fd):
            step = torch.arange(s, device=self.device, dtype=torch.int64) * d
            idx = (step.unsqueeze(1) + idx.unsqueeze(0)).reshape(-1)
        return self.storage[idx + self.offset]

    def __repr__(self):
        return f"MoYeArray({self.storage.dtype}, {self.layout}, offset={self.offset}, {self.device})"


def _colon_in(c):
    return any(_colon_in(e) for e in c) if isinstance(c, tuple) else c == COLON


def _span(t):
    """Number of storage elements a strided tensor reaches from its first element."""
    return 1 + sum((s - 1) * abs(d) for s, d in zip(t.shape, t.stride())) if t.numel() else 0


def isgmem(x):
    """True when the array lives in device global memory (reference src/pointer.jl:1-2)."""
    return x.storage.is_cuda


def zeros_(x):
    """`zeros!(x)` (reference src/algorithm/array_algorithms.jl:182)."""
    if x.layout == make_layout(x.layout.shape):
        x.storage[x.offset:x.offset + size(x.layout)] = 0
    else:
        for i in range(1, size(x.layout) + 1):
            x[i] = 0
    return x


def make_fragment_like_array(x, dtype=None):
    """`make_fragment_like(x)`: a new owning array with a compact layout of x's shape
    (reference src/algorithm/array_algorithms.jl:1-9)."""
    l = _fragment_layout(x.layout)
    buf = torch.empty(size(l), dtype=dtype or x.storage.dtype, device=x.device)
    return MoYeArray(buf, l)


def transpose(x):
    """`MoYe.transpose(x)`: the same memory seen with its two modes swapped; of a rank-2 `Layout`, the layout
    `make_layout(l[2], l[1])` (reference src/array.jl:247-249, src/layout.jl:772-774)."""
    if isinstance(x, Layout):
        if len(x) != 2:
            raise ValueError("transpose takes a rank-2 layout")
        return make_layout(x[1], x[0])
    return MoYeArray(x, transpose(x.layout))


def recast(x, new_dtype):
    """Reinterpret the element type, rescaling the layout (reference src/array.jl:294-314)."""
    new_bytes = torch.empty(0, dtype=new_dtype).element_size()
    l = recast_layout(x.layout, new_bytes, x.elem_bytes)
    byte_off = x.offset * x.elem_bytes
    if byte_off % new_bytes:
        raise ValueError("recast: misaligned view")
    return MoYeArray(x.storage.view(torch.uint8).view(new_dtype), l, byte_off // new_bytes)


def local_tile(x, tile_shape, coord, proj=None):
    """`@tile x tile coord`: the tile at `coord` of x divided by `tile_shape`; a `:` in
    `coord` keeps every tile along that mode (reference array_algorithms.jl:113-120)."""
    if proj is not None:
        return local_tile(x, dice_tuple(tuple(tile_shape), proj), dice_tuple(tuple(coord), proj))
    tile_shape, coord = tuple(tile_shape), tuple(coord)
    r1, r2 = len(tile_shape), rank(x.layout.shape)
    z = MoYeArray(x, zipped_divide(x.layout, tile_shape))
    rest = coord + (COLON,) * (r2 - len(coord))
    return z.view(((COLON,) * r1, rest))


def local_partition(x, tile_or_layout, coord, proj=None):
    """`@parallelize x threadlayout idx [proj]`: the elements of x that thread `idx` of the
    thread layout owns, interleaved (reference array_algorithms.jl:36-47,101-111)."""
    if isinstance(tile_or_layout, Layout):
        tl = tile_or_layout
        shp = tuple(product(s) for s in _tup(tl.shape))
        if proj is not None:
            kept = Layout(_unwrap1(dice_tuple(tl.shape, proj)), _unwrap1(dice_tuple(tl.stride, proj)))
            return local_partition(x, dice_tuple(shp, proj), _tup(get_congr_coord(kept, coord)))
        return local_partition(x, shp, _tup(get_congr_coord(tl, coord)))
    if proj is not None:
        return local_partition(x, dice_tuple(tuple(tile_or_layout), proj), dice_tuple(tuple(coord), proj))
    n = rank(x.layout.shape)
    z = MoYeArray(x, zipped_divide(x.layout, tuple(tile_or_layout)))
    return z.view((tuple(coord), (COLON,) * n))


tile = local_tile          # the `@tile` macro
parallelize = local_partition  # the `@parallelize` macro
