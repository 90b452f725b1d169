"""Fusion planner behind the plain backend trait: an unmodified stream of trait calls, fewer launches.

`FusingBackend` has the method set of `weta_core::Backend` (crates/weta-core/src/backend.rs:65-106) and wraps a
`B200Backend`.  f32 `unary` / `binary` calls are not launched when they are made: each returns a handle on a node of an
expression graph.  The graph is evaluated when a value is really needed (another kind of op consumes it, the host
reads it, or a storage it reads is about to be overwritten), and then a whole tree of element-wise nodes that share
one index space runs as ONE launch of `wb_ew_fused` (include/weta_b200.h): BatchNorm's element-wise passes between two
reductions, dropout's four calls, the cross-entropy chains, Adam's thirteen calls per parameter.  Nodes whose handle
the caller has already dropped and that nothing else consumes are never computed or stored at all.

Nothing changes for the caller: same calls, same shapes, and bit-identical values (the fused kernel applies the same
ops in the same order with the same roundings).  The reference launches one kernel per trait call, about 400 per
training step (README.md:123-124; crates/weta-cuda/src/lib.rs:482-521).
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, List, Optional, Tuple

from .backend import B200Backend, DeviceStorage
from .core import DType, Layout, WbView

MAX_INPUTS, MAX_INSTRS, MAX_OUTPUTS = 8, 48, 4


class WbEwInstr(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("op", ctypes.c_int32), ("a", ctypes.c_int32), ("b", ctypes.c_int32),
                ("p1", ctypes.c_double), ("p2", ctypes.c_double)]


class _Node:
    """One pending element-wise op.  `inputs` are (source, layout) pairs, a source being another node or a concrete
    DeviceStorage.  `concrete` is set once the node's value has been stored."""

    __slots__ = ("kind", "op", "p1", "p2", "inputs", "n", "concrete", "handle_ref", "consumers", "__weakref__")

    def __init__(self, kind, op, p1, p2, inputs, n):
        self.kind, self.op, self.p1, self.p2, self.inputs, self.n = kind, op, p1, p2, inputs, n
        self.concrete: Optional[DeviceStorage] = None
        self.handle_ref = None
        self.consumers = weakref.WeakSet()


class LazyStorage:
    """What the caller holds in place of a device storage: the value exists at the latest when `.ptr` is read."""

    __slots__ = ("node", "backend", "__weakref__")

    def __init__(self, node: _Node, backend: "FusingBackend"):
        self.node, self.backend = node, backend
        node.handle_ref = weakref.ref(self)

    def concrete(self) -> DeviceStorage:
        if self.node.concrete is None:
            self.backend._materialise(self.node)
        return self.node.concrete

    @property
    def ptr(self) -> int:
        return self.concrete().ptr

    @property
    def length(self) -> int:
        return self.node.n


def _identity(layout: Layout, n: int) -> bool:
    return layout.offset == 0 and layout.numel() == n and layout.is_contiguous()


class FusingBackend:
    name = "b200"

    def __init__(self, inner: B200Backend):
        self.inner = inner
        self.lib = inner.lib
        self.handle = inner.handle
        self.ordinal = inner.ordinal
        P, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        self.lib.wb_ew_fused.argtypes = [P, ctypes.POINTER(WbView), i32, ctypes.POINTER(WbEwInstr), i32, ctypes.POINTER(ctypes.c_int32),
                                         ctypes.POINTER(P), i32, i64]
        self.lib.wb_ew_fused.restype = i32
        self._readers: Dict[int, "weakref.WeakSet[_Node]"] = {}  # storage handle -> pending nodes that read it
        self._aliases: Dict[int, "weakref.WeakSet[_Node]"] = {}  # storage handle -> nodes whose value was written straight into it
        self.ops_deferred = 0  # f32 unary / binary trait calls taken into the graph
        self.programs = 0      # fused launches issued
        self.ops_fused = 0     # trait calls those launches stood for (deferred calls never counted here were dropped unread)

    # -- plumbing shared with B200Backend ---------------------------------------------------
    def check(self, status):
        self.inner.check(status)

    def synchronize(self):
        self.inner.synchronize()

    def stream(self):
        return self.inner.stream()

    def launch_count(self):
        return self.inner.launch_count()

    def gemm_check(self):
        self.inner.gemm_check()

    def set_matmul_mode(self, mode):
        self.inner.set_matmul_mode(mode)

    def alloc(self, n, dt):
        return self.inner.alloc(n, dt)

    def _c(self, s):
        return s.concrete() if isinstance(s, LazyStorage) else s

    # -- the lazy ops ----------------------------------------------------------------------
    def _source(self, s, layout: Layout):
        """A node input: the node itself when it can be inlined (read through the identity view), else a storage."""
        if isinstance(s, LazyStorage):
            if s.node.concrete is None and _identity(layout, s.node.n):
                return s.node
            return s.concrete()
        return s

    def _new_node(self, kind, op, p1, p2, pairs, n) -> LazyStorage:
        node = _Node(kind, op, p1, p2, pairs, n)
        self.ops_deferred += 1
        for src, _ in pairs:
            if isinstance(src, _Node):
                src.consumers.add(node)
            else:
                self._readers.setdefault(src.handle, weakref.WeakSet()).add(node)
        return LazyStorage(node, self)

    def unary(self, op, p1, p2, s, l: Layout, dt):
        if dt != DType.F32 or l.numel() == 0:
            return self.inner.unary(op, p1, p2, self._c(s), l, dt)
        return self._new_node(1, op, float(p1), float(p2), [(self._source(s, l), l)], l.numel())

    def binary(self, op, sa, la: Layout, sb, lb: Layout, dt):
        if dt != DType.F32 or la.numel() == 0:
            return self.inner.binary(op, self._c(sa), la, self._c(sb), lb, dt)
        return self._new_node(2, op, 0.0, 0.0, [(self._source(sa, la), la), (self._source(sb, lb), lb)], la.numel())

    # -- evaluation ------------------------------------------------------------------------
    def _wanted(self, node: _Node, inside) -> bool:
        """Does anything outside the program being built still need this node's value?"""
        if node.handle_ref is not None and node.handle_ref() is not None:
            return True
        return any(c.concrete is None and c not in inside for c in node.consumers)

    def _tree(self, root: _Node):
        """Nodes of the pending tree under root, children before parents."""
        order, seen = [], set()
        stack = [(root, False)]
        while stack:
            node, done = stack.pop()
            if done:
                order.append(node)
                continue
            if id(node) in seen:
                continue
            seen.add(id(node))
            stack.append((node, True))
            for src, _ in node.inputs:
                if isinstance(src, _Node) and src.concrete is None:
                    stack.append((src, False))
        return order

    def _materialise(self, root: _Node, into: Optional[Tuple[DeviceStorage, int]] = None):
        """Stores root's value (into a fresh storage, or at element offset `into[1]` of storage `into[0]`)."""
        if root.concrete is not None:
            return
        while True:
            order = self._tree(root)
            inside = set(order)
            inputs: List[Tuple[DeviceStorage, Layout]] = []
            keys = {}
            for node in order:
                for src, lay in node.inputs:
                    if not (isinstance(src, _Node) and src.concrete is None):
                        st = src.concrete if isinstance(src, _Node) else src
                        k = (st.handle, lay.shape, lay.strides, lay.offset)
                        if k not in keys:
                            keys[k] = len(inputs)
                            inputs.append((st, lay))
            extra = [nd for nd in order if nd is not root and self._wanted(nd, inside)]
            n_instr = len(order) + len(inputs)
            if n_instr <= MAX_INSTRS and len(inputs) <= MAX_INPUTS and 1 + len(extra) <= MAX_OUTPUTS:
                break
            # Too large for one launch: store a sub-tree of its own first (it then enters as an input).  Too many values
            # wanted outside: store one of those.  Too many ops or operands: store the largest sub-tree that fits by
            # itself (upper bounds: shared nodes are counted once per use), so a long chain splits into few launches.
            if 1 + len(extra) > MAX_OUTPUTS:
                victim = extra[0]
            else:
                size = {}
                victim, best = None, -1
                for nd in order:
                    ops, leaves = 1, 0
                    for src, _ in nd.inputs:
                        if isinstance(src, _Node) and src.concrete is None:
                            ops += size[id(src)][0]
                            leaves += size[id(src)][1]
                        else:
                            leaves += 1
                    size[id(nd)] = (ops, leaves)
                    if nd is not root and ops + leaves <= MAX_INSTRS and leaves <= MAX_INPUTS and ops > best:
                        victim, best = nd, ops
            if victim is None:  # cannot happen: a single op has at most two operands
                raise RuntimeError("element-wise program does not fit and cannot be split")
            self._materialise(victim)
        # emit: loads first, then the ops in dependency order
        prog = (WbEwInstr * n_instr)()
        reg_of_input = {}
        k = 0
        for key, idx in keys.items():
            prog[k] = WbEwInstr(0, 0, idx, 0, 0.0, 0.0)
            reg_of_input[idx] = k
            k += 1
        reg = {}

        def operand(src, lay):
            if isinstance(src, _Node) and src.concrete is None:
                return reg[id(src)]
            st = src.concrete if isinstance(src, _Node) else src
            return reg_of_input[keys[(st.handle, lay.shape, lay.strides, lay.offset)]]

        for node in order:
            a = operand(*node.inputs[0])
            b = operand(*node.inputs[1]) if node.kind == 2 else 0
            prog[k] = WbEwInstr(node.kind, node.op, a, b, node.p1, node.p2)
            reg[id(node)] = k
            k += 1
        views = (WbView * max(len(inputs), 1))(*[lay.view(st.ptr, DType.F32) for st, lay in inputs])
        outs_nodes = [root] + extra
        storages = []
        out_ptrs = (ctypes.c_void_p * len(outs_nodes))()
        out_regs = (ctypes.c_int32 * len(outs_nodes))()
        for i, nd in enumerate(outs_nodes):
            if nd is root and into is not None:
                st = None
                out_ptrs[i] = into[0].ptr + 4 * into[1]
            else:
                st = self.inner.alloc(nd.n, DType.F32)
                out_ptrs[i] = st.ptr
            storages.append(st)
            out_regs[i] = reg[id(nd)]
        self.inner.check(self.lib.wb_ew_fused(self.inner.handle, views, len(inputs), prog, n_instr, out_regs, out_ptrs, len(outs_nodes), root.n))
        self.programs += 1
        self.ops_fused += len(order)
        for nd, st in zip(outs_nodes, storages):
            nd.concrete = st if st is not None else into[0]
            nd.inputs = []  # the value exists: let go of the operands

    def _flush_readers(self, storage: DeviceStorage):
        """Called before `storage` is overwritten in place: evaluates every pending node that reads it, and gives every
        live handle whose value was written straight into it (see copy_strided) a storage of its own."""
        for node in list(self._aliases.pop(storage.handle, ())):
            if node.concrete is storage and node.handle_ref is not None and node.handle_ref() is not None:
                node.concrete = self._copy_out(storage, Layout.contiguous([node.n]), node.n)
        readers = self._readers.pop(storage.handle, None)
        if not readers:
            return
        for node in list(readers):
            if node.concrete is None and (self._wanted(node, ()) or len(node.consumers) > 0):
                self._materialise(node)

    # -- everything else evaluates its operands and goes straight through -------------------
    def from_host(self, flat):
        return self.inner.from_host(flat)

    def to_host(self, s, l, dt):
        return self.inner.to_host(self._c(s), l, dt)

    def zeros(self, n, dt):
        return self.inner.zeros(n, dt)

    def copy_strided(self, src, ls: Layout, dt, dst, ld: Layout):
        dst_c = self._c(dst)
        self._flush_readers(dst_c)
        if (isinstance(src, LazyStorage) and src.node.concrete is None and dt == DType.F32 and _identity(ls, src.node.n) and _identity(ld, src.node.n)
                and dst_c.length == src.node.n and not self._reads(src.node, dst_c)):
            # The pending expression is written straight into the destination (an in-place `assign` over a whole storage,
            # e.g. theta -= step).  The source handle then shares the destination's storage until that is next overwritten.
            node = src.node
            self._materialise(node, into=(dst_c, 0))
            self._aliases.setdefault(dst_c.handle, weakref.WeakSet()).add(node)
            return
        self.inner.copy_strided(self._c(src), ls, dt, dst_c, ld)

    def _copy_out(self, storage, layout, n):
        out = self.inner.alloc(n, DType.F32)
        self.inner.copy_strided(storage, layout, DType.F32, out, Layout.contiguous([n]))
        return out

    def _reads(self, root: _Node, storage: DeviceStorage) -> bool:
        """True if the pending tree under root reads `storage` through anything but the identity view (writing the
        result over such an operand element by element would not be safe)."""
        for node in self._tree(root):
            for src, lay in node.inputs:
                st = src.concrete if isinstance(src, _Node) else src
                if st is not None and st.handle == storage.handle and not (lay.is_contiguous() and lay.numel() == root.n):
                    return True
        return False

    def reduce(self, op, s, l, dt, axis):
        return self.inner.reduce(op, self._c(s), l, dt, axis)

    def matmul(self, sa, la, sb, lb, dt):
        return self.inner.matmul(self._c(sa), la, self._c(sb), lb, dt)

    def im2col(self, s, l, dt, p):
        return self.inner.im2col(self._c(s), l, dt, p)

    def col2im(self, s, l, dt, p, chw):
        return self.inner.col2im(self._c(s), l, dt, p, chw)

    def cast(self, s, l, dt, to):
        return self.inner.cast(self._c(s), l, dt, to)

    def random(self, n, dt, dist, seed):
        return self.inner.random(n, dt, dist, seed)
