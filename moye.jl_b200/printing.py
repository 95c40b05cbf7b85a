"""Pictures of who owns what: `print_typst` for a TiledMMA / TiledCopy (MoYe's teaching tool, reference
src/print.jl:46-345) and, for the Blackwell atoms where "who" is not a thread of a warp, text views of where the
data lives: tensor-memory lanes and columns, and the swizzled shared-memory operand tile.

`print_typst` writes Typst source: one table per matrix, every cell labelled with the thread that owns the element
and the position of the element among that thread's values, coloured by thread.  The reference emits a table of
`cell(thread, value)` calls over a fixed colour list; this module emits the same information with a palette
computed from the thread index.  Compile the output with `typst compile file.typ` (no renderer is needed here).
"""
import sys

from .atom import DTYPE_BITS, TiledCopy, TiledMMA
from .layout import Swizzle, composition, make_layout, size

__all__ = ["print_typst", "print_tmem_layout", "print_umma_smem_layout", "umma_smem_layout", "tmem_accumulator_layout"]


def _owner(layout_mn, thr_id, i, j):
    """(thread index, 1-based value index) of element (i, j) of a tile: `fldmod1(layout(i, j), size(thr_id))` and
    the thread-id layout applied to the remainder (reference src/print.jl:67-71)."""
    nthr = size(thr_id)
    idx0 = layout_mn(i, j) - 1
    return thr_id(idx0 % nthr + 1) - 1, idx0 // nthr + 1


_PREAMBLE = """#set page(width: auto, height: auto, margin: 6pt)
#set text(size: 6pt)
#let owner(t, v) = box(width: 2.1em, height: 2.1em, inset: 1pt, stroke: 0.3pt + black,
  fill: color.hsl(calc.rem(t * 47, 360) * 1deg, 55%, 82%), align(center + horizon)[T#t \\ V#v])
#let label(s) = box(width: 2.1em, height: 2.1em, align(center + horizon, text(fill: gray)[#s]))
"""


def _table(title, rows, cols, cell, row_label, col_label):
    out = [f"== {title}", f"#grid(columns: {cols + 1}, gutter: 0pt,", "  label[],"]
    out.append("  " + " ".join(f"label[{col_label}{c}]," for c in range(1, cols + 1)))
    for r in range(1, rows + 1):
        cells = " ".join("owner({}, {}),".format(*cell(r, c)) for c in range(1, cols + 1))
        out.append(f"  label[{row_label}{r}], {cells}")
    out.append(")")
    return "\n".join(out)


def print_typst(x, file=None):
    """`print_typst(tiled_mma)` / `print_typst(tiled_copy)`: Typst source of the ownership tables (C, A, B of one
    CTA tile; source and destination of one copy tile).  Returns the text and prints it to `file` (stdout)."""
    parts = [_PREAMBLE]
    if isinstance(x, TiledMMA):
        m, n, k = x.tile_shape()
        parts.append(f"= {x.atom.op.name}: tile {m} x {n} x {k}, {len(x)} thread(s)")
        for name, (lay, thr), rows, cols, rl, cl in (("C (M x N)", x.get_layoutC_MN(), m, n, "m", "n"),
                                                      ("A (M x K)", x.get_layoutA_MK(), m, k, "m", "k"),
                                                      ("B (N x K)", x.get_layoutB_NK(), n, k, "n", "k")):
            parts.append(_table(name, rows, cols, lambda r, c, lay=lay, thr=thr: _owner(lay, thr, r, c), rl, cl))
    elif isinstance(x, TiledCopy):
        m, n = x.tiler_mn[0], x.tiler_mn[1] if len(x.tiler_mn) > 1 else 1
        parts.append(f"= {x.copy_atom.op.name}: tile {m} x {n}, {len(x)} thread(s)")
        for name, (lay, thr) in (("source", x.get_layoutS_MN()), ("destination", x.get_layoutD_MN())):
            parts.append(_table(name, m, n, lambda r, c, lay=lay, thr=thr: _owner(lay, thr, r, c), "m", "n"))
    else:
        raise TypeError("print_typst takes a TiledMMA or a TiledCopy")
    text = "\n\n".join(parts) + "\n"
    print(text, file=file if file is not None else sys.stdout, end="")
    return text


# ------------------------------------------------------------------------------ tcgen05: where the data lives
def tmem_accumulator_layout(tile_n, cta_pair=False):
    """(m, n) of the accumulator tile -> (CTA of the pair, tensor-memory lane, column), as a function.  One CTA holds
    128 rows of the tile in its 128 lanes; with `cta_group::2` the second CTA holds rows 128..255.  Column j of the
    accumulator is tensor-memory column j (fp32 / s32: one 32-bit column per element)."""
    rows = 256 if cta_pair else 128

    def where(m, n):
        if not (1 <= m <= rows and 1 <= n <= tile_n):
            raise IndexError((m, n))
        return (m - 1) // 128, (m - 1) % 128, n - 1

    return where


def print_tmem_layout(op, cta_pair=False, file=None):
    """Text view of an `MMAOP_SM100_*` accumulator in tensor memory and of who reads it in the epilogue: the
    tcgen05.ld 32x32b shape gives thread t of epilogue warp w the lane 32 * (w mod 4) + t, register j the column
    j of the chunk, so a warp's chunk of 32 columns is a 32 x 32 block with one ROW of D per thread."""
    if op.arch != "sm_100a":
        raise ValueError("print_tmem_layout takes an MMAOP_SM100_* op")
    n = op.shape_mnk[1]
    out = [f"{op.name}: accumulator 128{' x 2 CTAs' if cta_pair else ''} lanes x {n} columns (32-bit) of tensor memory",
           "  row m of the CTA tile -> lane (m - 1) mod 128" + (" of CTA (m - 1) div 128" if cta_pair else ""),
           "  column n -> tensor-memory column n - 1 (+ the accumulator buffer's base column)",
           "  epilogue warp w may read lanes 32 (w mod 4) .. 32 (w mod 4) + 31 only:", ""]
    out.append("  lanes      " + "".join(f"cols {c:3d}-{min(c + 31, n - 1):3d}  " for c in range(0, min(n, 128), 32)) + ("..." if n > 128 else ""))
    for q in range(4):
        out.append(f"  {32 * q:3d}-{32 * q + 31:3d}    " + "".join(f"warp%4={q} ld#{c // 32:<2d}   " for c in range(0, min(n, 128), 32)))
    out += ["", "  inside one tcgen05.ld.32x32b.x32 (a 32 x 32 block): thread t <- lane base + t; register j <- column base + j"]
    text = "\n".join(out)
    print(text, file=file if file is not None else sys.stdout)
    return text


def umma_smem_layout(dtype, rows, major="K"):
    """The shared-memory layout of one pipeline stage of an operand as TMA writes it and tcgen05.mma reads it:
    (row, k) -> BYTE offset, a `ComposedLayout` with the 128-byte swizzle `Swizzle(3, 4, 3)`.

    K-major (stride 1 along K): rows of 128 bytes (one K block), 8 rows per 1024-byte swizzle atom.
    MN-major (stride 1 along M / N, MoYe's column-major arrays): chunks of 128 bytes along MN; inside a chunk the K
    rows are 128 bytes apart, successive chunks `K block x 128` bytes apart.  16- and 8-bit elements; 32-bit
    MN-major tiles use 32-byte swizzle atoms and are not drawn here."""
    eb = DTYPE_BITS[dtype] // 8
    bk = 128 // eb
    sw = Swizzle(3, 4, 3)
    if major == "K":
        return composition(sw, make_layout((rows, bk), (128, eb)))
    if eb == 4:
        raise ValueError("MN-major 32-bit tiles use the 32-byte-atom swizzle")
    ch = 128 // eb                        # elements of one 128-byte chunk along MN
    if rows % ch:
        raise ValueError(f"rows must be a multiple of {ch}")
    return composition(sw, make_layout(((ch, rows // ch), bk), ((eb, bk * 128), 128)))


def print_umma_smem_layout(dtype, rows=8, major="K", file=None):
    """Text view of `umma_smem_layout`: for the first `rows` rows, the 16-byte column (0..7) inside the 128-byte
    row where each 16-byte group of K lands.  The XOR pattern is what removes the bank conflicts MoYe's README
    lists as missing (reference README.md:14-17)."""
    lay = umma_smem_layout(dtype, max(rows, 8) if major == "K" else 128 // (DTYPE_BITS[dtype] // 8), major)
    eb = DTYPE_BITS[dtype] // 8
    per16 = 16 // eb
    out = [f"{'K' if major == 'K' else 'MN'}-major operand stage, {DTYPE_BITS[dtype]}-bit elements: {lay!r}  (byte offsets)",
           "  row   " + " ".join(f"{'k' if major == 'K' else 'm'}{g * per16:3d}.." for g in range(8)) +
           ("    <- 16-byte groups of one 128-byte K block" if major == "K" else "    <- 16-byte groups of one 128-byte chunk along M / N")]
    if major == "K":
        for r in range(1, rows + 1):
            cols = [(lay(r, g * per16 + 1) - 1 - (r - 1) * 128) // 16 for g in range(8)]
            out.append(f"  {r - 1:3d}   " + " ".join(f"  c{c}   " for c in cols))
        out.append("  (cN = 16-byte column N of the row in shared memory: group g of row r sits in column g xor (r mod 8))")
    else:
        for k in range(1, rows + 1):
            cols = [(lay((g * per16 + 1, 1), k) - 1 - (k - 1) * 128) // 16 for g in range(8)]
            out.append(f"  k{k - 1:2d}   " + " ".join(f"  c{c}   " for c in cols))
        out.append("  (rows are K indices here; the 128 bytes of a row hold 128 / element-size consecutive M / N indices)")
    text = "\n".join(out)
    print(text, file=file if file is not None else sys.stdout)
    return text
