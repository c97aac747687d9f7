"""GGUF tensors under tensor parallelism: the v-head order of converted checkpoints and per-rank windows on quantised blocks.

Two facts make GGUF sharding different from slicing a rectangle out of a dense matrix:

* **atoms**: a quantised tensor can only be cut between blocks (32 or 256 elements along a row), so a column window is a
  window of blocks and must start and end on block boundaries;
* **v-head order**: the llama.cpp converter writes the gated-delta-net's value heads in a *tiled* order: grouped head ``h`` (the
  model's order: the ``vpr = nv / nk`` value heads of key head 0, then those of key head 1, ...) sits at file position
  ``(h % vpr) * nk + h // vpr``. A rank that took "its half of the file" would get value heads of every key head instead of the
  contiguous grouped window its key heads need, so heads are gathered in grouped order when the tensor is read.

The invariant every role keeps (and ``tests/test_formats.py`` checks): **what rank r loads equals a contiguous block of the
fully loaded tensor in grouped order** -- a row window, a column window of atoms, or (for the packed q / k / v tensors) one window
per segment, concatenated. Anything that cannot be cut exactly is refused loudly: a dimension the world does not divide, a column
cut inside a block, a head width that is not a whole number of blocks.

Role table (GGUF key -> how it is cut):

    ffn_gate, ffn_up, attn_q (per head [q | gate] rows), attn_k, attn_v   rows
    output (only with ``head_split``)                                      rows
    attn_qkv, ssm_conv1d (q | k | v channels)                               one row window per segment, the v segment in grouped head order
    attn_gate, ssm_alpha, ssm_beta, ssm_a, ssm_dt                          rows by grouped v head
    ffn_down, attn_output                                                  block-aligned column window of every row
    ssm_out                                                                columns by grouped v head (head width must be whole blocks)
    norms, embeddings, q / k norms, ssm_norm                               replicated

Reference counterpart: ``crates/models/src/formats/gguf/shard.rs:1-80`` (roles, invariant, refusals) and the tiled / grouped
head formula of ``formats/gguf/transform.rs``.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

ROWS, SEGS, ROWS_HEAD, COLS, COLS_HEAD, REPLICATE = "rows", "segs", "rows_head", "cols", "cols_head", "replicate"

_ROLES = {
    "ffn_gate": ROWS, "ffn_up": ROWS, "attn_q": ROWS, "attn_k": ROWS, "attn_v": ROWS,
    "attn_qkv": SEGS, "ssm_conv1d": SEGS,
    "attn_gate": ROWS_HEAD, "ssm_alpha": ROWS_HEAD, "ssm_beta": ROWS_HEAD, "ssm_a": ROWS_HEAD, "ssm_dt": ROWS_HEAD,
    "ffn_down": COLS, "attn_output": COLS, "ssm_out": COLS_HEAD,
}


class ShardError(ValueError):
    pass


@dataclass(frozen=True)
class GdnDims:
    """Head geometry of the gated-delta-net layers: ``nk`` key heads of width ``kd``, ``nv`` value heads of width ``vd``."""
    nk: int
    nv: int
    kd: int
    vd: int

    @property
    def vpr(self) -> int:
        return self.nv // self.nk


@dataclass(frozen=True)
class ShardSel:
    rank: int
    world: int
    head_split: bool = False       # cut the lm_head's vocabulary rows too

    def window(self, total: int, what: str, key: str) -> tuple[int, int]:
        if total % self.world:
            raise ShardError(f"{key}: {what} = {total} is not divisible by the tensor-parallel world {self.world}")
        n = total // self.world
        return self.rank * n, n


def role(key: str, sel: ShardSel | None = None) -> str:
    """How the GGUF tensor ``key`` (``blk.<i>.<name>.weight`` / ``.bias`` / bare) is cut."""
    parts = key.split(".")
    name = parts[2] if parts[0] == "blk" and len(parts) > 2 else parts[0]
    if name == "output" and len(parts) > 1 and parts[1] == "weight":
        return ROWS if sel is not None and sel.head_split else REPLICATE
    return _ROLES.get(name, REPLICATE)


def file_pos_of_grouped(h, dims: GdnDims):
    """File (tiled) position of grouped value head ``h`` (scalar or array)."""
    return (h % dims.vpr) * dims.nk + h // dims.vpr


def grouped_head_order(dims: GdnDims) -> np.ndarray:
    """``order[h]`` = file position of grouped head h: ``tensor_in_file[order]`` is the tensor in grouped order."""
    return file_pos_of_grouped(np.arange(dims.nv), dims)


def head_rows(heads: np.ndarray, width: int) -> np.ndarray:
    """Row (or column) indices of the given heads, ``width`` rows each, in the given head order."""
    return (heads[:, None] * width + np.arange(width)[None]).reshape(-1)


@dataclass
class Plan:
    """What to read of one tensor: ``rows`` (indices into the file's rows, None = all) and ``col_atoms`` (indices of the
    column atoms of every row, None = all); an atom is ``atom`` elements wide."""
    rows: np.ndarray | None
    col_atoms: np.ndarray | None
    atom: int
    shape: tuple          # resulting (rows, columns) in elements


def plan(key: str, shape: tuple, block_elems: int, dims: GdnDims, sel: ShardSel | None) -> Plan:
    """The read plan of GGUF tensor ``key`` with logical ``shape`` (rows, columns) -- 1-D tensors are (n, 1) -- whose rows are
    stored as blocks of ``block_elems`` elements (1 for native float types). ``sel = None`` loads the whole tensor; value heads
    come out in grouped order either way."""
    r = role(key, sel)
    n_rows, n_cols = shape
    one_d = n_cols == 1
    w = sel if sel is not None else ShardSel(0, 1)

    def v_heads() -> np.ndarray:
        lo, n = w.window(dims.nv, "value heads", key)
        return grouped_head_order(dims)[lo:lo + n]

    if r == REPLICATE:
        return Plan(None, None, block_elems, shape)
    if r == ROWS:
        lo, n = w.window(n_rows, "rows", key)
        return Plan(np.arange(lo, lo + n), None, block_elems, (n, n_cols))
    if r == ROWS_HEAD:
        if n_rows % dims.nv:
            raise ShardError(f"{key}: {n_rows} rows are not a whole number of rows per value head ({dims.nv} heads)")
        rows = head_rows(v_heads(), n_rows // dims.nv)
        return Plan(rows, None, block_elems, (len(rows), n_cols))
    if r == SEGS:
        kq, vv = dims.nk * dims.kd, dims.nv * dims.vd
        if n_rows != 2 * kq + vv:
            raise ShardError(f"{key}: {n_rows} rows, expected q | k | v = {2 * kq + vv}")
        klo, kn = w.window(dims.nk, "key heads", key)
        krows = head_rows(np.arange(klo, klo + kn), dims.kd)
        rows = np.concatenate([krows, kq + krows, 2 * kq + head_rows(v_heads(), dims.vd)])
        return Plan(rows, None, block_elems, (len(rows), n_cols))
    if one_d:
        raise ShardError(f"{key}: a 1-D tensor cannot be cut along columns")
    if n_cols % block_elems:
        raise ShardError(f"{key}: {n_cols} columns are not whole blocks of {block_elems}")
    atoms = n_cols // block_elems
    if r == COLS:
        lo, n = w.window(n_cols, "columns", key)
        if lo % block_elems or n % block_elems:
            raise ShardError(f"{key}: the column cut at {lo} (+{n}) falls inside a block of {block_elems} elements")
        return Plan(None, np.arange(lo // block_elems, (lo + n) // block_elems), block_elems, (n_rows, n))
    # COLS_HEAD: columns are the value heads' output dims, vd each
    if n_cols != dims.nv * dims.vd:
        raise ShardError(f"{key}: {n_cols} columns, expected nv * vd = {dims.nv * dims.vd}")
    if dims.vd % block_elems:
        raise ShardError(f"{key}: the head width {dims.vd} is not a whole number of blocks of {block_elems} elements: a block "
                         "holds columns of two heads that the tiled order separates")
    per = dims.vd // block_elems
    col_atoms = head_rows(v_heads(), per)
    assert atoms == dims.nv * per
    return Plan(None, col_atoms, block_elems, (n_rows, len(col_atoms) * block_elems))


def apply_raw(raw: np.ndarray, shape: tuple, block_elems: int, block_bytes: int, p: Plan) -> np.ndarray:
    """Cut the raw bytes of a block-quantised tensor (rows of ``columns / block_elems`` blocks of ``block_bytes`` bytes)
    according to ``p``; returns uint8 ``[rows, blocks * block_bytes]``."""
    n_rows, n_cols = shape
    blocks = n_cols // block_elems
    t = np.ascontiguousarray(raw).view(np.uint8).reshape(n_rows, blocks, block_bytes)
    if p.rows is not None:
        t = t[p.rows]
    if p.col_atoms is not None:
        t = t[:, p.col_atoms]
    return np.ascontiguousarray(t).reshape(t.shape[0], -1)


def apply_dense(x, p: Plan):
    """The same cut on a dense (dequantised or native) tensor of shape (rows, columns) or (rows,)."""
    if p.rows is not None:
        x = x[p.rows]
    if p.col_atoms is not None:
        cols = head_rows(np.asarray(p.col_atoms), p.atom)
        x = x[:, cols]
    return x
