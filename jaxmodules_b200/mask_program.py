"""Tracing a Python ``mask_fn(b, h, q, k)`` into a mask program for the device.

The reference evaluates ``mask_fn`` by vmapping it over index grids
(jaxmodules/attention.py:70-73, jaxmodules/vectorize.py:407-527): the function is traced once
with abstract integers.  ``trace`` does the same with symbolic integers that record every
arithmetic, comparison and bit operation into straight-line three-address code — the
``bma_mask_program`` of include/bma.h — which ``bma_mask_table_build`` then evaluates on the GPU
for the whole index box.  Functions that branch on their arguments (``if q > k``), or call NumPy
functions on them, cannot be traced; the caller falls back to evaluating them on the host.

``where`` / ``minimum`` / ``maximum`` / ``absolute`` work on symbols and on plain numbers or
arrays alike, and ``Table`` wraps an integer array that the mask indexes with its arguments
(``seg[b, q] == seg[b, k]``).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Callable, List, Tuple

import numpy as np
import torch

from . import _native as nat

__all__ = ["Program", "Table", "TraceError", "trace", "where", "minimum", "maximum", "absolute", "run_on_host"]


class TraceError(Exception):
    """The function cannot be expressed as a mask program."""


@dataclass
class Program:
    code: List[Tuple[int, int, int, int]] = field(default_factory=list)   # (op, x, y, z)
    tables: List[torch.Tensor] = field(default_factory=list)              # int32, 1-D or 2-D
    uses_b: bool = False
    uses_h: bool = False

    @property
    def result(self) -> int:
        return 3 + len(self.code)


class Table:
    """An integer lookup table a traced mask may index: ``t[i]`` (1-D) or ``t[i, j]`` (2-D).
    Indices outside the table clamp to its edge (as gathers do under JAX)."""

    def __init__(self, values):
        arr = np.asarray(values.cpu() if isinstance(values, torch.Tensor) else values)
        if arr.ndim not in (1, 2) or not np.issubdtype(arr.dtype, np.integer) and arr.dtype != bool:
            raise TypeError("Table takes a 1-D or 2-D integer array")
        self.values = torch.from_numpy(np.ascontiguousarray(arr.astype(np.int32)))

    def __getitem__(self, idx):
        idx = idx if isinstance(idx, tuple) else (idx,)
        if len(idx) != self.values.ndim:
            raise IndexError("Table needs one index per dimension")
        syms = [i for i in idx if isinstance(i, Sym)]
        if not syms:
            return int(self.values[tuple(int(i) for i in idx)]) if all(np.ndim(i) == 0 for i in idx) else \
                self.values.numpy()[tuple(np.clip(np.asarray(i), 0, n - 1) for i, n in zip(idx, self.values.shape))]
        tr = syms[0].tr
        slot = tr.table_slot(self)
        ops = [tr.lift(i) for i in idx]
        if len(ops) == 1:
            return tr.emit("LOAD1", slot, ops[0].ix, 0, boolean=False, raw_x=True)
        return tr.emit("LOAD2", slot, ops[0].ix, ops[1].ix, boolean=False, raw_x=True)


class _Tracer:
    def __init__(self):
        self.prog = Program()
        self.consts = {}
        self._tables = {}

    def emit(self, op, x, y=0, z=0, *, boolean, raw_x=False) -> "Sym":
        """Append one instruction; ``raw_x`` marks x as an immediate / table slot, not a value."""
        if len(self.prog.code) >= nat.PROGRAM_MAX_INSTR:
            raise TraceError("mask program longer than %d instructions" % nat.PROGRAM_MAX_INSTR)
        self.prog.code.append((nat.OP[op], int(x), int(y), int(z)))
        return Sym(self, 3 + len(self.prog.code), boolean)

    def lift(self, v) -> "Sym":
        if isinstance(v, Sym):
            return v
        if isinstance(v, (bool, np.bool_)):
            v = int(v)
        if isinstance(v, (int, np.integer)):
            v = int(v)
            if not -(1 << 31) <= v < (1 << 31):
                raise TraceError("constant does not fit 32 bits")
            if v not in self.consts:
                self.consts[v] = self.emit("CONST", v, boolean=False)
            return self.consts[v]
        raise TraceError(f"cannot use a value of type {type(v).__name__} in a mask program")

    def table_slot(self, t: Table) -> int:
        if id(t) not in self._tables:
            if len(self.prog.tables) >= nat.PROGRAM_MAX_TABLES:
                raise TraceError("too many tables")
            self._tables[id(t)] = len(self.prog.tables)
            self.prog.tables.append(t.values)
        return self._tables[id(t)]


def operands(op: int, x: int, y: int, z: int) -> Tuple[int, ...]:
    """Value indices an instruction reads."""
    name = nat.OPS[op]
    if name == "CONST":
        return ()
    if name == "LOAD1":
        return (y,)
    if name == "LOAD2":
        return (y, z)
    if name == "SELECT":
        return (x, y, z)
    if op < nat.OP["ADD"]:
        return (x,)
    return (x, y)


class Sym:
    """A traced 32-bit integer (or boolean) value."""
    __array_ufunc__ = None      # NumPy scalars defer to the reflected operators below
    __hash__ = None

    def __init__(self, tr: _Tracer, ix: int, boolean: bool):
        self.tr, self.ix, self.boolean = tr, ix, boolean

    def _bin(self, op, other, boolean=False, swap=False):
        o = self.tr.lift(other)
        a, b = (o, self) if swap else (self, o)
        return self.tr.emit(op, a.ix, b.ix, boolean=boolean)

    def __add__(self, o): return self._bin("ADD", o)
    def __radd__(self, o): return self._bin("ADD", o, swap=True)
    def __sub__(self, o): return self._bin("SUB", o)
    def __rsub__(self, o): return self._bin("SUB", o, swap=True)
    def __mul__(self, o): return self._bin("MUL", o)
    def __rmul__(self, o): return self._bin("MUL", o, swap=True)
    def __floordiv__(self, o): return self._bin("FLOORDIV", o)
    def __rfloordiv__(self, o): return self._bin("FLOORDIV", o, swap=True)
    def __mod__(self, o): return self._bin("MOD", o)
    def __rmod__(self, o): return self._bin("MOD", o, swap=True)
    def __lshift__(self, o): return self._bin("SHL", o)
    def __rshift__(self, o): return self._bin("SHR", o)
    def __lt__(self, o): return self._bin("LT", o, True)
    def __le__(self, o): return self._bin("LE", o, True)
    def __gt__(self, o): return self._bin("GT", o, True)
    def __ge__(self, o): return self._bin("GE", o, True)
    def __eq__(self, o): return self._bin("EQ", o, True)
    def __ne__(self, o): return self._bin("NE", o, True)

    def _logic(self, op, other, swap=False):
        o = self.tr.lift(other)
        return self._bin(op, o, boolean=self.boolean and (o.boolean or isinstance(other, (bool, np.bool_))), swap=swap)

    def __and__(self, o): return self._logic("AND", o)
    def __rand__(self, o): return self._logic("AND", o, True)
    def __or__(self, o): return self._logic("OR", o)
    def __ror__(self, o): return self._logic("OR", o, True)
    def __xor__(self, o): return self._logic("XOR", o)
    def __rxor__(self, o): return self._logic("XOR", o, True)

    def __neg__(self): return self.tr.emit("NEG", self.ix, boolean=False)
    def __pos__(self): return self
    def __abs__(self): return self.tr.emit("ABS", self.ix, boolean=False)

    def __invert__(self):   # ~ on a comparison result is logical not (NumPy / JAX booleans), on an integer bitwise
        return self.tr.emit("NOT" if self.boolean else "INV", self.ix, boolean=self.boolean)

    def __bool__(self):
        raise TraceError("the mask branches on its arguments (use where(cond, a, b) and & | ~ instead of if / and / or / not)")

    def __index__(self):
        raise TraceError("a traced value cannot index a Python or NumPy container (wrap the array in Table)")

    __int__ = __index__


def where(cond, a, b):
    """``a if cond else b`` element by element, for traced values and for numbers / arrays."""
    syms = [v for v in (cond, a, b) if isinstance(v, Sym)]
    if not syms:
        return np.where(cond, a, b)
    tr = syms[0].tr
    c, x, y = tr.lift(cond), tr.lift(a), tr.lift(b)
    both_bool = all(isinstance(v, (bool, np.bool_)) or (isinstance(v, Sym) and v.boolean) for v in (a, b))
    return tr.emit("SELECT", c.ix, x.ix, y.ix, boolean=both_bool)


def _two(op, np_fn, a, b):
    syms = [v for v in (a, b) if isinstance(v, Sym)]
    if not syms:
        return np_fn(a, b)
    tr = syms[0].tr
    return tr.emit(op, tr.lift(a).ix, tr.lift(b).ix, boolean=False)


def minimum(a, b):
    return _two("MIN", np.minimum, a, b)


def maximum(a, b):
    return _two("MAX", np.maximum, a, b)


def absolute(a):
    return abs(a) if isinstance(a, Sym) else np.abs(a)


def trace(mask_fn: Callable, nargs: int = 4) -> Program:
    """Run ``mask_fn`` on symbolic (b, h, q, k) — or (h, q, k) for three-argument masks, the
    reference's ``co_argcount == 3`` rule (jaxmodules/attention.py:405-407) — and return its program.
    Raises TraceError when the function cannot be traced."""
    tr = _Tracer()
    b, h, q, k = (Sym(tr, i, False) for i in range(4))
    try:
        out = mask_fn(b, h, q, k) if nargs == 4 else mask_fn(h, q, k)
    except TraceError:
        raise
    except Exception as e:   # NumPy functions, float arithmetic, container indexing ...
        raise TraceError(f"{type(e).__name__}: {e}") from e
    if isinstance(out, (bool, np.bool_, int, np.integer)):
        out = tr.lift(int(bool(out)))
    if not isinstance(out, Sym):
        raise TraceError("mask_fn did not return a traced value")
    if out.ix != tr.prog.result:      # the predicate must be the last value: copy it there
        out = tr.emit("OR", out.ix, out.ix, boolean=out.boolean)
    used = {r for ins in tr.prog.code for r in operands(*ins)}
    tr.prog.uses_b, tr.prog.uses_h = 0 in used, 1 in used
    return tr.prog


def run_on_host(prog: Program, b, h, q, k):
    """The program on NumPy int32 arrays (broadcast together): the statement of what the device
    kernel computes, used by the tests as its oracle-side twin."""
    b, h, q, k = np.broadcast_arrays(*(np.asarray(v, dtype=np.int64) for v in (b, h, q, k)))
    wrap = lambda v: ((np.asarray(v, dtype=np.int64) + (1 << 31)) % (1 << 32) - (1 << 31))
    v = [b, h, q, k]
    for op, x, y, z in prog.code:
        name = nat.OPS[op]
        if name == "CONST":
            r = np.full(b.shape, x, dtype=np.int64)
        elif name == "NEG": r = -v[x]
        elif name == "ABS": r = np.abs(v[x])
        elif name == "NOT": r = (v[x] == 0).astype(np.int64)
        elif name == "INV": r = ~v[x]
        elif name == "ADD": r = v[x] + v[y]
        elif name == "SUB": r = v[x] - v[y]
        elif name == "MUL": r = v[x] * v[y]
        elif name in ("FLOORDIV", "MOD"):
            d = np.where(v[y] == 0, 1, v[y])
            r = np.where(v[y] == 0, 0, v[x] // d if name == "FLOORDIV" else v[x] % d)
        elif name == "MIN": r = np.minimum(v[x], v[y])
        elif name == "MAX": r = np.maximum(v[x], v[y])
        elif name in ("LT", "LE", "GT", "GE", "EQ", "NE"):
            f = {"LT": np.less, "LE": np.less_equal, "GT": np.greater, "GE": np.greater_equal, "EQ": np.equal, "NE": np.not_equal}[name]
            r = f(v[x], v[y]).astype(np.int64)
        elif name == "AND": r = v[x] & v[y]
        elif name == "OR": r = v[x] | v[y]
        elif name == "XOR": r = v[x] ^ v[y]
        elif name == "SHL": r = v[x] << (v[y] & 31)
        elif name == "SHR": r = v[x] >> (v[y] & 31)
        elif name == "SELECT": r = np.where(v[x] != 0, v[y], v[z])
        elif name == "LOAD1":
            t = prog.tables[x].numpy().reshape(-1)
            r = t[np.clip(v[y], 0, t.shape[0] - 1)].astype(np.int64)
        elif name == "LOAD2":
            t = prog.tables[x].numpy()
            r = t[np.clip(v[y], 0, t.shape[0] - 1), np.clip(v[z], 0, t.shape[1] - 1)].astype(np.int64)
        else:
            raise ValueError(name)
        v.append(wrap(r))
    return v[-1] != 0


def _c_program(prog: Program, device):
    """(bma_mask_program struct, device tensors it points at)."""
    if not prog.code:
        raise ValueError("empty program")
    c = nat.MaskProgram()
    c.n_instr, c.n_tables = len(prog.code), len(prog.tables)
    flat = [w for ins in prog.code for w in ins]
    c.code[:len(flat)] = flat
    keep = []
    for i, t in enumerate(prog.tables):
        dt = t.to(device=device, dtype=torch.int32).contiguous()
        keep.append(dt)
        c.tables[i] = dt.data_ptr()
        c.table_rows[i] = dt.shape[0] if dt.ndim == 2 else 1
        c.table_cols[i] = dt.shape[-1]
        c.table_stride[i] = dt.stride(0) if dt.ndim == 2 else 0
    return c, keep


def build_table(prog: Program, B: int, H: int, N: int, L: int, device, q_offset: int = 0, k_offset: int = 0) -> torch.Tensor:
    """``bma_mask_table_build``: the program evaluated over the box, packed into the bit table
    ``[Bm, Hm, N, ceil(L/32)]`` int32 on ``device`` (Bm / Hm are 1 when b / h are not read)."""
    Bm, Hm = (B if prog.uses_b else 1), (H if prog.uses_h else 1)
    words = (L + 31) // 32
    c, keep = _c_program(prog, device)
    bits = torch.empty((Bm, Hm, N, words), dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        nat.check(nat.lib().bma_mask_table_build(C.byref(c), Bm, Hm, N, L, q_offset, k_offset, bits.data_ptr(),
                                                 torch.cuda.current_stream(device).cuda_stream), "bma_mask_table_build")
    bits._bma_keep = keep   # the tables must outlive the launch
    return bits


def build_tiles(prog: Program, B: int, H: int, N: int, L: int, device):
    """``bma_mask_tiles_build``: the program evaluated over the box into the TILES form of the mask description —
    (tile_class uint8 ``[Bm, Hm, TQ, TK]``, tile_slot int32 of the same shape, tile_bits int32 ``[cut tiles, 2, 128, 4]``:
    every cut tile by query row and by key row).  Memory grows with the tiles the mask cuts (4 KB each), not with N * L.  Two passes: the first only counts the cut
    tiles (one host synchronisation, once per mask), the second stores them."""
    Bm, Hm = (B if prog.uses_b else 1), (H if prog.uses_h else 1)
    TQ, TK = (N + 127) // 128, (L + 127) // 128
    c, keep = _c_program(prog, device)
    cls = torch.empty((Bm, Hm, TQ, TK), dtype=torch.uint8, device=device)
    slot = torch.empty((Bm, Hm, TQ, TK), dtype=torch.int32, device=device)
    counter = torch.zeros((1,), dtype=torch.int32, device=device)
    lib = nat.lib()
    with torch.cuda.device(device):
        st = torch.cuda.current_stream(device).cuda_stream
        nat.check(lib.bma_mask_tiles_build(C.byref(c), Bm, Hm, N, L, 0, 0, cls.data_ptr(), slot.data_ptr(), None, 0,
                                           counter.data_ptr(), st), "bma_mask_tiles_build")
        cut = int(counter.item())
        bits = torch.empty((max(cut, 1), 2, 128, 4), dtype=torch.int32, device=device)
        if cut:
            counter.zero_()
            nat.check(lib.bma_mask_tiles_build(C.byref(c), Bm, Hm, N, L, 0, 0, cls.data_ptr(), slot.data_ptr(), bits.data_ptr(),
                                               cut, counter.data_ptr(), st), "bma_mask_tiles_build")
    bits._bma_keep = keep   # the program's tables must outlive the launch
    return cls, slot, bits
