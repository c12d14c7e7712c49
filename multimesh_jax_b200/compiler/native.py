"""Lowering of task templates to native kernel programs.

A :class:`~multimesh_jax_b200.compiler.lower.TemplateProgram` is an instruction list that Python
interprets: per instruction it materialises arguments, allocates results and calls into the
kernel library. For templates whose instructions all map onto entry points of the kernel
library - the transformer stages of the models in this package when they hold no collective -
this module builds the same computation as a ``_mm_C.KernelProgram``: a flat list of
``(entry point address, packed arguments)`` records that the C++ launcher replays in one call
(the role of ``RunExecutable`` binding tile pointers and scalars to a compiled task,
``src/pjrt_client/hlo_executor.cc:75-174``).

Memory is planned here, once per template, instead of being requested from an allocator per
instruction (``src/pjrt_client/mm_pjrt_executable.cc:549-590``, ``src/pjrt_client/allocator.h:10-24``):

* every task output gets a fixed offset inside one *output block* that the executable
  allocates per launch and carves the output tiles from;
* every intermediate gets an offset inside the per-device *scratch tile* of the runtime
  context, assigned by a liveness-based first-fit allocator, so the scratch a template needs
  is the peak of its live intermediates, not their sum;
* operators that may overwrite a dead operand do so (the rules of ``FAST_OPS`` /
  ``INPLACE_OPERANDS``).

Pointer arguments are recorded as ``(slot, byte offset)``; the slots of a launch are its input
tiles, the output block, the scratch tile and the gradient accumulators it adds into. A
template that contains anything else (a collective, an operator without an emitter, a strided
view) raises :class:`NativeUnsupported` and keeps its interpreted program.
"""
from __future__ import annotations

import ctypes
import json
from ctypes import c_float
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import _lib
from ..ops import attention as _attention  # noqa: F401  (declares the attention entry points)
from .capture import DTYPE_FROM_NAME
from .lower import Instr, TemplateProgram, _tensor_ids_in_order, _V

ALIGN = 256


class NativeUnsupported(Exception):
    """The template cannot be expressed as a list of kernel-library calls."""


def _round(n: int, a: int = ALIGN) -> int:
    return (n + a - 1) // a * a


class Sym:
    """A contiguous tensor at ``offset`` bytes inside slot ``slot``."""
    __slots__ = ("slot", "off", "shape", "dtype", "root")

    def __init__(self, slot: int, off: int, shape: Sequence[int], dtype: torch.dtype, root: Optional[int] = None):
        self.slot, self.off, self.shape, self.dtype = slot, off, tuple(int(s) for s in shape), dtype
        self.root = root            # id of the allocation this symbol lives in (for liveness)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * self.dtype.itemsize

    def view(self, shape: Sequence[int]) -> "Sym":
        shape = list(shape)
        if -1 in shape:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.numel // max(known, 1)
        out = Sym(self.slot, self.off, shape, self.dtype, self.root)
        if out.numel != self.numel:
            raise NativeUnsupported(f"view of {self.shape} as {shape}")
        return out


STREAM = object()


class _Scratch:
    """First-fit allocator over the scratch tile with explicit frees (offsets are planned once)."""

    def __init__(self):
        self.free: List[Tuple[int, int]] = []     # (offset, size), sorted by offset
        self.top = 0
        self.peak = 0
        self.live: Dict[int, Tuple[int, int]] = {}
        self._next = 0

    def alloc(self, nbytes: int) -> Tuple[int, int]:
        size = _round(max(nbytes, 1))
        for i, (off, sz) in enumerate(self.free):
            if sz >= size:
                if sz == size:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + size, sz - size)
                break
        else:
            off = self.top
            self.top += size
            self.peak = max(self.peak, self.top)
        self._next += 1
        self.live[self._next] = (off, size)
        return self._next, off

    def release(self, ident: int) -> None:
        off, size = self.live.pop(ident)
        self.free.append((off, size))
        self.free.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        if merged and merged[-1][0] + merged[-1][1] == self.top:
            self.top = merged[-1][0]
            merged.pop()
        self.free = merged


class NativeProgram:
    """One variant (first write / accumulate) of a template as a kernel program."""

    def __init__(self):
        from .. import _mm_C
        self.kernel = _mm_C.KernelProgram()
        self.out_block_bytes = 0                # all chunks together
        self.out_chunks: List[int] = []         # bytes of each allocation the launch's fresh outputs are carved from
        self.scratch_bytes = 0
        # per template output: ("block", chunk, offset, shape, dtype) | ("input", index, shape) | ("acc", position)
        # | ("slice", index, shape): rows [scalar, scalar + shape[0]) of input `index`
        # | ("ext", j, shape, dtype): the whole of external tile j, a slot of its own that the caller
        #   points at memory of its choosing (the peer-mapped tile a cross-submesh reshard reads)
        self.outputs: List[tuple] = []
        self.external: List[int] = []           # output positions with an external tile, in slot order
        self.acc_positions: List[int] = []      # output positions whose accumulator tile is a slot of the launch
        self.num_calls = 0


class _Builder:
    def __init__(self, cap, template: dict, prog: TemplateProgram, accumulate: Sequence[int], have_acc: bool):
        self.cap, self.g, self.template, self.prog = cap, cap.graph, template, prog
        self.lib = _lib.load()
        self.n_in = len(prog.inputs)
        self.SLOT_OUT = self.n_in
        self.SLOT_SCRATCH = self.n_in + 1
        self.accumulate = list(accumulate)
        self.have_acc = have_acc
        self.np = NativeProgram()
        self.scratch = _Scratch()
        self.env: Dict[int, Sym] = {}
        self.out_pos = {v: k for k, v in enumerate(prog.outputs)}
        self.out_chunks: List[int] = []
        self.out_base = None                    # first slot of output chunks 1, 2, ... (chunk 0 is SLOT_OUT)
        self.acc_slot: Dict[int, int] = {}
        self.refs: Dict[int, int] = {}          # scratch allocation id -> number of live values in it
        self.scaled: Dict[int, int] = {}        # microbatch slices: value -> bytes per unit of the launch's scalar

    # ---------------------------------------------------------------- memory
    def new_value(self, vid: int, shape, dtype) -> Sym:
        """Storage for IR value ``vid``: inside the output block when it is a (non-accumulated)
        task output, else in the scratch tile."""
        j = self.reaches_ext.get(vid)
        if j is not None and j not in self.ext_taken:
            probe = Sym(self.ext_slot[j], 0, shape, dtype)
            if probe.nbytes == self.ext_bytes[j]:
                self.ext_taken.add(j)
                return probe
        if vid in self.reaches_output:
            return self.out_region(shape, dtype)
        return self.temp(shape, dtype)

    def temp(self, shape, dtype) -> Sym:
        probe = Sym(0, 0, shape, dtype)
        ident, off = self.scratch.alloc(probe.nbytes)
        self.refs[ident] = 0
        return Sym(self.SLOT_SCRATCH, off, shape, dtype, root=ident)

    # Fresh outputs are carved from a few allocations of at most OUT_CHUNK bytes each (one of its
    # own for anything larger) instead of one block: a task that saves tens of GB of activations
    # would otherwise need that much contiguous free memory.
    OUT_CHUNK = 256 << 20

    def out_region(self, shape, dtype) -> Sym:
        nb = _round(Sym(0, 0, shape, dtype).nbytes)
        if self.out_chunks and self.out_chunks[-1] + nb <= self.OUT_CHUNK:
            off = self.out_chunks[-1]
            self.out_chunks[-1] += nb
        else:
            self.out_chunks.append(nb)
            off = 0
        c = len(self.out_chunks) - 1
        return Sym(self.SLOT_OUT if c == 0 else self.out_base + c - 1, off, shape, dtype)

    def out_chunk_of(self, slot: int):
        """Index of the output chunk that ``slot`` names, or None."""
        if slot == self.SLOT_OUT:
            return 0
        if self.out_base is not None and slot >= self.out_base:
            return slot - self.out_base + 1
        return None

    def bind(self, vid: int, sym: Sym) -> None:
        self.env[vid] = sym
        if sym.root is not None:
            self.refs[sym.root] = self.refs.get(sym.root, 0) + 1

    def drop(self, vid: int) -> None:
        sym = self.env.pop(vid, None)
        if sym is not None and sym.root is not None:
            self.refs[sym.root] -= 1
            if self.refs[sym.root] == 0:
                self.scratch.release(sym.root)
                del self.refs[sym.root]

    def free_temp(self, sym: Sym) -> None:
        if sym.root is not None and self.refs.get(sym.root, 0) == 0:
            self.scratch.release(sym.root)
            self.refs.pop(sym.root, None)

    # ---------------------------------------------------------------- calls
    def call(self, name: str, *args) -> None:
        sig = _lib._SIGS.get(name)
        fn = getattr(self.lib, name, None)
        if sig is None or fn is None:
            raise NativeUnsupported(f"kernel library has no entry point {name}")
        if len(sig[1]) != len(args):
            raise NativeUnsupported(f"{name}: expected {len(sig[1])} arguments, got {len(args)}")
        packed = []
        for a, ctype in zip(args, sig[1]):
            if a is STREAM:
                packed.append(("s",))
            elif a is None:
                packed.append(("p", -1, 0))
            elif isinstance(a, Sym):
                packed.append(("p", a.slot, a.off))
            elif isinstance(a, tuple) and a and a[0] == "scaled":        # (tag, Sym, scalar index, bytes per unit)
                packed.append(("p", a[1].slot, a[1].off, a[2], a[3]))
            elif ctype is c_float:
                packed.append(("f", float(a)))
            else:
                packed.append(("i", int(a)))
        addr = ctypes.cast(fn, ctypes.c_void_p).value
        self.np.kernel.add_call(addr, name, packed)
        self.np.num_calls += 1

    # ---------------------------------------------------------------- helpers
    def sym_of(self, vid: int) -> Sym:
        if vid in self.scaled:
            raise NativeUnsupported("a microbatch slice is read by an operator without an offset-aware emitter")
        try:
            return self.env[vid]
        except KeyError:
            raise NativeUnsupported(f"value {vid} is not available")

    def slice_sym(self, vid: int) -> Sym:
        """Shape and base of a value that may be a microbatch slice (its address also depends on
        the launch's scalar; pass ``ptr(vid)`` to the kernel)."""
        try:
            return self.env[vid]
        except KeyError:
            raise NativeUnsupported(f"value {vid} is not available")

    def ptr(self, vid: int):
        sym = self.slice_sym(vid)
        row = self.scaled.get(vid)
        return sym if row is None else ("scaled", sym, 0, row)

    def copy(self, dst: Sym, src: Sym) -> None:
        self.call("mm_memcpy_d2d", dst, src, src.nbytes, STREAM)

    def gemm(self, a: Sym, a_mn: bool, b: Sym, b_mn: bool, out: Sym, mode: int) -> None:
        from ..ops import kernels as K
        M, Kd = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
        N = b.shape[1] if b_mn else b.shape[0]
        pair = K.PAIR_MIN_M > 0 and M >= K.PAIR_MIN_M
        self.call("mm_gemm_pair_bf16" if pair else "mm_gemm_bf16", a, int(a_mn), a.shape[1], b, int(b_mn), b.shape[1],
                  out, mode, out.shape[1], M, N, Kd, STREAM)


# ------------------------------------------------------------------------------------------------
# emitters: one per operator; each binds the instruction's outputs in b.env
# ------------------------------------------------------------------------------------------------
def _flat2(s: Sym) -> Sym:
    return s.view((-1, s.shape[-1]))


def _const_args(ins: Instr) -> list:
    """Non-tensor positional arguments of a captured operator, in order."""
    return [a for a in ins.args if not isinstance(a, _V)]


def _emit_linear(b: _Builder, ins: Instr, ids, op):
    x, w = b.sym_of(ids[0]), b.sym_of(ids[1])
    if x.dtype != torch.bfloat16:
        raise NativeUnsupported("linear in a dtype other than bf16")
    Kd = x.shape[-1]
    out_shape = x.shape[:-1] + w.shape[:-1]
    out = b.new_value(ins.outs[0], out_shape, x.dtype)
    b.gemm(x.view((-1, Kd)), False, w.view((-1, Kd)), False, out.view((-1, out.numel // (x.numel // Kd))), 0)
    b.bind(ins.outs[0], out)


def _emit_linear_dgrad(b: _Builder, ins: Instr, ids, op):
    dy, w = b.sym_of(ids[0]), b.sym_of(ids[1])
    Kd = w.shape[-1]
    w2 = w.view((-1, Kd))
    nb = len(dy.shape) - (len(w.shape) - 1)
    out = b.new_value(ins.outs[0], dy.shape[:nb] + (Kd,), dy.dtype)
    b.gemm(dy.view((-1, w2.shape[0])), False, w2, True, out.view((-1, Kd)), 0)
    b.bind(ins.outs[0], out)


def _emit_linear_wgrad(b: _Builder, ins: Instr, ids, op):
    dy, x = b.sym_of(ids[0]), b.sym_of(ids[1])
    Kd = x.shape[-1]
    nb = len(x.shape) - 1
    x2 = x.view((-1, Kd))
    dy2 = dy.view((x2.shape[0], -1))
    out_shape = dy.shape[nb:] + (Kd,)
    if ins.kind == 6:           # writes / adds straight into the gradient accumulator
        pos, dtype = ins.extra
        if dtype != torch.float32:
            raise NativeUnsupported("fused accumulation into a non-fp32 accumulator")
        if b.have_acc:
            acc = Sym(b.acc_slot_for(pos), 0, out_shape, dtype)
            b.gemm(dy2, True, x2, True, acc.view((-1, Kd)), 2)
            b.bind(ins.outs[0], acc)
        else:
            out = b.out_region(out_shape, dtype)
            b.gemm(dy2, True, x2, True, out.view((-1, Kd)), 1)
            b.bind(ins.outs[0], out)
            b.fresh_acc[pos] = out
        return
    out = b.new_value(ins.outs[0], out_shape, dy.dtype)
    b.gemm(dy2, True, x2, True, out.view((-1, Kd)), 0)
    b.bind(ins.outs[0], out)


def _emit_rmsnorm(b: _Builder, ins: Instr, ids, op):
    x, w = b.sym_of(ids[0]), b.sym_of(ids[1])
    eps = _const_args(ins)[0]
    D = x.shape[-1]
    rows = x.numel // D
    y = b.new_value(ins.outs[0], x.shape, x.dtype)
    rstd = b.new_value(ins.outs[1], x.shape[:-1], torch.float32)
    b.call("mm_rmsnorm_fwd", x, w, y, rstd, rows, D, eps, STREAM)
    b.bind(ins.outs[0], y)
    b.bind(ins.outs[1], rstd)


def _emit_add_rmsnorm(b: _Builder, ins: Instr, ids, op):
    x, delta, w = (b.sym_of(v) for v in ids[:3])
    eps = _const_args(ins)[0]
    D = x.shape[-1]
    rows = x.numel // D
    if x.numel % 8:
        raise NativeUnsupported("add of a tensor whose size is not a multiple of 8")
    xn = b.new_value(ins.outs[0], x.shape, x.dtype)
    b.call("mm_add_bf16", x, delta, xn, x.numel, STREAM)
    y = b.new_value(ins.outs[1], x.shape, x.dtype)
    rstd = b.new_value(ins.outs[2], x.shape[:-1], torch.float32)
    b.call("mm_rmsnorm_fwd", xn, w, y, rstd, rows, D, eps, STREAM)
    b.bind(ins.outs[0], xn)
    b.bind(ins.outs[1], y)
    b.bind(ins.outs[2], rstd)


def _norm_bwd(b: _Builder, x: Sym, w: Sym, dy: Sym, rstd: Sym, dx: Sym, add_to_dx: bool, dw_vid: int):
    D = x.shape[-1]
    rows = x.numel // D
    parts = b.lib.mm_rmsnorm_bwd_parts(rows)
    part = b.temp((parts, D), torch.float32)
    dw32 = b.temp((D,), torch.float32)
    b.call("mm_rmsnorm_bwd", x, w, dy, rstd, dx, dw32, part, rows, D, 0, int(add_to_dx), STREAM)
    b.free_temp(part)
    dw = b.new_value(dw_vid, (D,), w.dtype)
    if w.dtype == torch.float32:
        b.copy(dw, dw32)
    else:
        b.call("mm_f32_to_bf16", dw32, dw, D, STREAM)
    b.free_temp(dw32)
    b.bind(dw_vid, dw)


def _emit_rmsnorm_bwd(b: _Builder, ins: Instr, ids, op):
    x, w, dy, rstd = (b.sym_of(v) for v in ids[:4])
    dx = b.new_value(ins.outs[0], x.shape, x.dtype)
    _norm_bwd(b, x, w, dy, rstd, dx, False, ins.outs[1])
    b.bind(ins.outs[0], dx)


def _emit_add_rmsnorm_bwd(b: _Builder, ins: Instr, ids, op):
    xn, w, dxn, dy, rstd = (b.sym_of(v) for v in ids[:5])
    if b.may_overwrite(ins, ids[2]):
        acc = Sym(dxn.slot, dxn.off, dxn.shape, dxn.dtype, dxn.root)     # the dead operand becomes the result
    else:
        acc = b.new_value(ins.outs[0], dxn.shape, dxn.dtype)
        b.copy(acc, dxn)
    _norm_bwd(b, xn, w, dy, rstd, acc, True, ins.outs[1])
    b.bind(ins.outs[0], acc)


def _emit_swiglu(b: _Builder, ins: Instr, ids, op):
    gu = b.sym_of(ids[0])
    F = gu.shape[-1]
    T = gu.numel // (2 * F)
    h = b.new_value(ins.outs[0], gu.shape[:-2] + (F,), gu.dtype)
    b.call("mm_swiglu_fwd", gu, h, T, F, STREAM)
    b.bind(ins.outs[0], h)


def _emit_swiglu_bwd(b: _Builder, ins: Instr, ids, op):
    gu, dh = b.sym_of(ids[0]), b.sym_of(ids[1])
    F = gu.shape[-1]
    T = gu.numel // (2 * F)
    dgu = b.new_value(ins.outs[0], gu.shape, gu.dtype)
    b.call("mm_swiglu_bwd", gu, dh, dgu, T, F, STREAM)
    b.bind(ins.outs[0], dgu)


def _emit_attention(b: _Builder, ins: Instr, ids, op):
    qkv, cos, sin = (b.sym_of(v) for v in ids[:3])
    rep = _const_args(ins)[0]
    B, S, H, D = qkv.shape
    if not b.lib.mm_flash_attn_supported(S, D) or qkv.dtype != torch.bfloat16:
        raise NativeUnsupported("attention shape outside the tcgen05 kernels")
    if b.may_overwrite(ins, ids[0]):
        qkv_r = Sym(qkv.slot, qkv.off, qkv.shape, qkv.dtype, qkv.root)
    else:
        qkv_r = b.new_value(ins.outs[2], qkv.shape, qkv.dtype)
        b.copy(qkv_r, qkv)
    n_rot = H // (rep + 2) * (rep + 1)
    b.call("mm_rope", qkv_r, cos, sin, B * S, cos.shape[0], n_rot, D, H * D, 0, rep + 1, rep + 2, STREAM)
    hkv = H // (rep + 2)
    out = b.new_value(ins.outs[0], (B, S, hkv * rep, D), qkv.dtype)
    lse = b.new_value(ins.outs[1], (B, hkv * rep, S), torch.float32)
    b.call("mm_flash_attn_fwd", qkv_r, out, lse, B, S, hkv, rep, D, STREAM)
    b.bind(ins.outs[0], out)
    b.bind(ins.outs[1], lse)
    b.bind(ins.outs[2], qkv_r)


def _emit_attention_bwd(b: _Builder, ins: Instr, ids, op):
    dout, qkv_r, out, lse, cos, sin = (b.sym_of(v) for v in ids[:6])
    rep = _const_args(ins)[0]
    B, S, H, D = qkv_r.shape
    if not b.lib.mm_flash_attn_supported(S, D) or dout.dtype != torch.bfloat16:
        raise NativeUnsupported("attention shape outside the tcgen05 kernels")
    hkv = H // (rep + 2)
    hq = hkv * rep
    dqkv = b.new_value(ins.outs[0], qkv_r.shape, qkv_r.dtype)
    dq_acc = b.temp((B, S, hq, D), torch.float32)
    delta = b.temp((B, hq, S), torch.float32)
    b.call("mm_flash_attn_bwd", qkv_r, out, dout, lse, dqkv, dq_acc, delta, B, S, hkv, rep, D, STREAM)
    b.free_temp(dq_acc)
    b.free_temp(delta)
    n_rot = hkv * (rep + 1)
    b.call("mm_rope", dqkv, cos, sin, B * S, cos.shape[0], n_rot, D, H * D, 1, rep + 1, rep + 2, STREAM)
    b.bind(ins.outs[0], dqkv)


def _emit_cross_entropy(b: _Builder, ins: Instr, ids, op):
    logits, targets = b.sym_of(ids[0]), b.ptr(ids[1])
    scale = _const_args(ins)[0]
    V = logits.shape[-1]
    rows = logits.numel // V
    if V % 8 or logits.dtype != torch.bfloat16:
        raise NativeUnsupported("cross-entropy layout")
    if b.may_overwrite(ins, ids[0]):
        buf = Sym(logits.slot, logits.off, logits.shape, logits.dtype, logits.root)
    else:
        buf = b.new_value(ins.outs[1], logits.shape, logits.dtype)
        b.copy(buf, logits)
    loss_rows = b.temp((rows,), torch.float32)
    b.call("mm_cross_entropy", buf, targets, loss_rows, None, None, rows, V, V, 0, scale, 1, STREAM)
    loss = b.new_value(ins.outs[0], (), torch.float32)
    b.call("mm_sum_scale_f32", loss_rows, rows, scale, loss, STREAM)
    b.free_temp(loss_rows)
    b.bind(ins.outs[0], loss)
    b.bind(ins.outs[1], buf)


def _emit_embedding(b: _Builder, ins: Instr, ids, op):
    table, tok = b.sym_of(ids[0]), b.slice_sym(ids[1])
    V, D = table.shape
    out = b.new_value(ins.outs[0], tok.shape + (D,), table.dtype)
    b.call("mm_embedding_fwd", table, b.ptr(ids[1]), out, tok.numel, D, 0, V, STREAM)
    b.bind(ins.outs[0], out)


def _emit_embedding_bwd(b: _Builder, ins: Instr, ids, op):
    dout, tok = b.sym_of(ids[0]), b.slice_sym(ids[1])
    vocab = _const_args(ins)[0]
    D = dout.shape[-1]
    if ins.kind != 6:
        raise NativeUnsupported("embedding gradient outside an accumulator")
    pos, dtype = ins.extra
    if dtype != torch.float32:
        raise NativeUnsupported("embedding gradient into a non-fp32 accumulator")
    if b.have_acc:
        acc = Sym(b.acc_slot_for(pos), 0, (vocab, D), dtype)
    else:
        acc = b.out_region((vocab, D), dtype)
        b.call("mm_zero", acc, acc.nbytes, STREAM)
        b.fresh_acc[pos] = acc
    b.call("mm_embedding_bwd", dout, b.ptr(ids[1]), acc, tok.numel, D, 0, vocab, STREAM)
    b.bind(ins.outs[0], acc)


def _emit_adamw(b: _Builder, ins: Instr, ids, op):
    param, master, m, v, grad, step = (b.sym_of(x) for x in ids[:6])
    lr, beta1, beta2, eps, wd, gs = _const_args(ins)[:6]
    if param.dtype != torch.bfloat16 or grad.dtype != torch.float32 or master.numel % 4:
        raise NativeUnsupported("AdamW layout")
    outs = []
    for k, (src, vid) in enumerate(zip((param, master, m, v), ins.outs)):
        if b.may_overwrite(ins, ids[k]):
            outs.append(Sym(src.slot, src.off, src.shape, src.dtype, src.root))
        else:
            dst = b.new_value(vid, src.shape, src.dtype)
            if k > 0:
                b.copy(dst, src)
            outs.append(dst)
    p2, a2, m2, v2 = outs
    b.call("mm_adamw", a2, p2, m2, v2, grad, master.numel, lr, beta1, beta2, eps, wd, 1, gs, step, STREAM)
    for vid, s in zip(ins.outs, outs):
        b.bind(vid, s)


def _emit_view(b: _Builder, ins: Instr, ids, op):
    src = b.slice_sym(ids[0])
    out_shape = b.g.value(ins.outs[0])["shape"]
    b.bind(ins.outs[0], src.view(out_shape))
    if ids[0] in b.scaled:
        b.scaled[ins.outs[0]] = b.scaled[ids[0]]


def _emit_alias(b: _Builder, ins: Instr, ids, op):
    src = b.slice_sym(ids[0])
    b.bind(ins.outs[0], Sym(src.slot, src.off, src.shape, src.dtype, src.root))
    if ids[0] in b.scaled:
        b.scaled[ins.outs[0]] = b.scaled[ids[0]]


def _emit_ones_like(b: _Builder, ins: Instr, ids, op):
    src = b.sym_of(ids[0])
    if src.dtype != torch.float32:
        raise NativeUnsupported("ones_like of a non-fp32 value")
    out = b.new_value(ins.outs[0], src.shape, src.dtype)
    b.call("mm_fill_f32", out, 1.0, out.numel, STREAM)
    b.bind(ins.outs[0], out)


def _emit_zeros(b: _Builder, ins: Instr, ids, op):
    v = b.g.value(ins.outs[0])
    out = b.new_value(ins.outs[0], v["shape"], DTYPE_FROM_NAME[v["dtype"]])
    b.call("mm_zero", out, out.nbytes, STREAM)
    b.bind(ins.outs[0], out)


def _emit_to_copy(b: _Builder, ins: Instr, ids, op):
    src = b.sym_of(ids[0])
    v = b.g.value(ins.outs[0])
    dt = DTYPE_FROM_NAME[v["dtype"]]
    out = b.new_value(ins.outs[0], src.shape, dt)
    if src.dtype == torch.float32 and dt == torch.bfloat16:
        b.call("mm_f32_to_bf16", src, out, src.numel, STREAM)
    elif src.dtype == torch.bfloat16 and dt == torch.float32:
        b.call("mm_bf16_to_f32", src, out, src.numel, 0, STREAM)
    elif src.dtype == dt:
        b.copy(out, src)
    else:
        raise NativeUnsupported(f"conversion {src.dtype} -> {dt}")
    b.bind(ins.outs[0], out)


def _emit_mul(b: _Builder, ins: Instr, ids, op):
    if len(ids) != 2:
        raise NativeUnsupported("multiplication by a constant")
    x, s = b.sym_of(ids[0]), b.sym_of(ids[1])
    if s.numel != 1 or x.dtype != torch.bfloat16 or s.dtype != torch.bfloat16:
        raise NativeUnsupported("general element-wise product")
    out = b.new_value(ins.outs[0], x.shape, x.dtype)
    b.call("mm_scale_bf16", x, s, out, x.numel, STREAM)
    b.bind(ins.outs[0], out)


def _emit_add(b: _Builder, ins: Instr, ids, op):
    if len(ids) == 1:           # tensor + python constant: the optimizer's step counter
        x = b.sym_of(ids[0])
        const = _const_args(ins)
        if x.dtype != torch.int64 or len(const) != 1 or not isinstance(const[0], int):
            raise NativeUnsupported("addition of a constant")
        out = b.new_value(ins.outs[0], x.shape, x.dtype)
        b.call("mm_add_i64", x, const[0], out, x.numel, STREAM)
        b.bind(ins.outs[0], out)
        return
    x, y = b.sym_of(ids[0]), b.sym_of(ids[1])
    if x.shape != y.shape or x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16 or x.numel % 8 or ins.kwargs:
        raise NativeUnsupported("general addition")
    out = b.new_value(ins.outs[0], x.shape, x.dtype)
    b.call("mm_add_bf16", x, y, out, x.numel, STREAM)
    b.bind(ins.outs[0], out)


EMITTERS = {
    "mm_ops.linear.default": _emit_linear,
    "mm_ops.linear_dgrad.default": _emit_linear_dgrad,
    "mm_ops.linear_wgrad.default": _emit_linear_wgrad,
    "mm_ops.rmsnorm.default": _emit_rmsnorm,
    "mm_ops.add_rmsnorm.default": _emit_add_rmsnorm,
    "mm_ops.rmsnorm_bwd.default": _emit_rmsnorm_bwd,
    "mm_ops.add_rmsnorm_bwd.default": _emit_add_rmsnorm_bwd,
    "mm_ops.swiglu.default": _emit_swiglu,
    "mm_ops.swiglu_bwd.default": _emit_swiglu_bwd,
    "mm_ops.attention.default": _emit_attention,
    "mm_ops.attention_bwd.default": _emit_attention_bwd,
    "mm_ops.cross_entropy.default": _emit_cross_entropy,
    "mm_ops.embedding.default": _emit_embedding,
    "mm_ops.embedding_bwd.default": _emit_embedding_bwd,
    "mm_ops.adamw.default": _emit_adamw,
    "aten.view.default": _emit_view,
    "aten._unsafe_view.default": _emit_view,
    "aten.reshape.default": _emit_view,
    "aten.detach.default": _emit_alias,
    "aten.alias.default": _emit_alias,
    "aten.ones_like.default": _emit_ones_like,
    "aten.zeros.default": _emit_zeros,
    "aten._to_copy.default": _emit_to_copy,
    "aten.mul.Tensor": _emit_mul,
    "aten.add.Tensor": _emit_add,
}


# operators that may write a result over a dead operand: (tensor operand position, result position)
_MAY_WRITE_OVER = {
    "mm_ops.attention.default": ((0, 2),),
    "mm_ops.add_rmsnorm_bwd.default": ((2, 0),),
    "mm_ops.cross_entropy.default": ((0, 1),),
    "mm_ops.adamw.default": ((0, 0), (1, 1), (2, 2), (3, 3)),
}


def build_native(cap, plan: dict, template: dict, prog: TemplateProgram, accumulate: Sequence[int], have_acc: bool,
                 external: Sequence[int] = (), protected_inputs: Sequence[int] = ()) -> NativeProgram:
    """The kernel program of one variant of ``template``: ``accumulate[k]`` is the accumulate
    mode class of output ``k`` (0 plain, else accumulated) and ``have_acc`` says whether the
    accumulator tiles already exist (they then are slots of the launch) or are created by this
    launch. ``external``: positions of plain outputs that are written into a tile the caller
    supplies per launch (slots after the accumulators, in the order given).
    ``protected_inputs``: positions of inputs whose storage must never take a result (someone
    outside the task graph of this device - a pull from another GPU - may still read them).
    Raises :class:`NativeUnsupported`."""
    if template["num_devices"] != 1:
        raise NativeUnsupported("templates on more than one device run collectives")
    g = cap.graph
    b = _Builder(cap, template, prog, accumulate, have_acc)
    b.fresh_acc = {}
    acc_positions = [k for k, m in enumerate(accumulate) if m]
    b.np.acc_positions = acc_positions if have_acc else []
    slot_of_acc = {pos: b.n_in + 2 + j for j, pos in enumerate(acc_positions)}
    b.acc_slot_for = lambda pos: slot_of_acc[pos]
    external = [k for k in external if accumulate[k] == 0]
    b.np.external = list(external)
    b.ext_slot = {j: b.n_in + 2 + len(b.np.acc_positions) + j for j in range(len(external))}
    b.out_base = b.n_in + 2 + len(b.np.acc_positions) + len(external)
    b.ext_bytes, b.ext_taken, b.reaches_ext = {}, set(), {}
    for j, k in enumerate(external):
        val = g.value(prog.outputs[k])
        sh = val.get("sharding")
        b.ext_bytes[j] = Sym(0, 0, sh["shard_size"] if sh else val["shape"], DTYPE_FROM_NAME[val["dtype"]]).nbytes
        b.reaches_ext[prog.outputs[k]] = j
    input_index = {v: i for i, v in enumerate(prog.inputs)}
    for v, i in input_index.items():
        val = g.value(v)
        sh = val.get("sharding")
        shape = sh["shard_size"] if sh else val["shape"]
        b.env[v] = Sym(i, 0, shape, DTYPE_FROM_NAME[val["dtype"]])
    # Values whose storage a task output ends up naming - directly, through view-like operators
    # (autograd hands saved tensors on as detached aliases) or because an operator may write its
    # result over them - are placed in the output block from the start, so no output is copied.
    alias_parent: Dict[int, int] = {}
    for ins in prog.instrs:
        if ins.kind == 1 and isinstance(ins.args, int):
            alias_parent[ins.outs[0]] = ins.args
        elif ins.kind in (0, 6):
            opn = g.node(ins.node_id)["op"]
            ids_ = _tensor_ids_in_order(ins.args, ins.kwargs)
            if EMITTERS.get(opn) in (_emit_view, _emit_alias) and ids_:
                alias_parent[ins.outs[0]] = ids_[0]
            for operand, result in _MAY_WRITE_OVER.get(opn, ()):
                if operand < len(ids_) and result < len(ins.outs):
                    alias_parent[ins.outs[result]] = ids_[operand]
    b.reaches_output = {v for k, v in enumerate(prog.outputs) if accumulate[k] == 0}
    for ins in reversed(prog.instrs):
        for o in ins.outs or ():
            if o in b.reaches_output and o in alias_parent:
                b.reaches_output.add(alias_parent[o])
                if o in b.reaches_ext:
                    b.reaches_ext.setdefault(alias_parent[o], b.reaches_ext[o])
    # operand liveness inside the program, and operands other tasks still need
    last: Dict[int, int] = {}
    for idx, ins in enumerate(prog.instrs):
        for v in _reads_of(ins):
            last[v] = idx
    keep = set(prog.outputs)
    mine = set(prog.inputs)
    shared_inputs = {v for t in plan["templates"] if t is not template and t["name"] != template["name"]
                     for v in t["inputs"] if v in mine}
    shared_inputs |= {prog.inputs[i] for i in protected_inputs}

    def may_overwrite(ins: Instr, vid: int) -> bool:
        """The operand dies with this instruction and its storage may take the result (the rule
        of the interpreted program's in-place operator variants)."""
        idx = b.cur
        if last.get(vid, -1) > idx or vid in keep or vid in shared_inputs:
            return False
        if vid in b.scaled:
            return False
        return True       # input tiles are private to the step (non-donated arguments are cloned when bound)
    b.may_overwrite = may_overwrite

    for idx, ins in enumerate(prog.instrs):
        b.cur = idx
        kind = ins.kind
        if kind in (0, 6):
            op = g.node(ins.node_id)["op"]
            emit = EMITTERS.get(op)
            if emit is None or ins.kwargs and any(isinstance(v, _V) for v in ins.kwargs.values()):
                raise NativeUnsupported(f"no native emitter for {op}")
            emit(b, ins, _tensor_ids_in_order(ins.args, ins.kwargs), op)
        elif kind == 1:         # identity (accumulate marker, layout marker)
            src = b.sym_of(ins.args)
            b.bind(ins.outs[0], Sym(src.slot, src.off, src.shape, src.dtype, src.root))
        elif kind == 2:
            src = b.sym_of(ins.args)
            out = b.new_value(ins.outs[0], src.shape, src.dtype)
            b.copy(out, src)
            b.bind(ins.outs[0], out)
        elif kind == 3:         # microbatch slice of dimension 0: a pointer offset taken from the launch's scalars
            dim, size, shards = ins.extra
            src = b.sym_of(ins.args)
            if dim != 0 or shards != 1:
                raise NativeUnsupported("microbatch slice of an inner or sharded dimension")
            row = src.nbytes // src.shape[0]
            out = Sym(src.slot, src.off, (size,) + src.shape[1:], src.dtype, src.root)
            b.bind(ins.outs[0], out)
            b.scaled[ins.outs[0]] = row
        else:
            raise NativeUnsupported(f"instruction kind {kind} (a collective or an exchanging operator)")
        for v in prog._last_use.get(idx, ()):
            b.drop(v)
    # outputs
    for k, v in enumerate(prog.outputs):
        if v in b.scaled:          # a microbatch slice of an input handed on as it is (token ids kept for the backward task)
            sym = b.slice_sym(v)
            if sym.slot >= b.n_in or sym.off != 0 or accumulate[k]:
                raise NativeUnsupported("a microbatch slice of an intermediate is a task output")
            b.np.outputs.append(("slice", sym.slot, sym.shape))
            continue
        sym = b.sym_of(v)
        mode = accumulate[k]
        if k in external:
            j = external.index(k)
            if not (sym.slot == b.ext_slot[j] and sym.off == 0):
                dst = Sym(b.ext_slot[j], 0, sym.shape, sym.dtype)
                b.copy(dst, sym)
            b.np.outputs.append(("ext", j, sym.shape, sym.dtype))
            continue
        if mode:
            fused = prog.fused_acc.get(k)
            if fused:
                if have_acc:
                    b.np.outputs.append(("acc", k))
                else:
                    fr = b.fresh_acc[k]
                    b.np.outputs.append(("block", b.out_chunk_of(fr.slot), fr.off, fr.shape, fr.dtype))
                continue
            acc_dtype = DTYPE_FROM_NAME[plan_store_dtype(plan, template, k)]
            if acc_dtype != torch.float32:
                raise NativeUnsupported("accumulator in a dtype other than fp32")
            if have_acc:
                acc = Sym(slot_of_acc[k], 0, sym.shape, acc_dtype)
                if sym.dtype == torch.bfloat16:
                    b.call("mm_bf16_to_f32", sym, acc, sym.numel, 1, STREAM)
                elif sym.dtype == torch.float32:
                    b.call("mm_accumulate_f32", acc, sym, sym.numel, STREAM)
                else:
                    raise NativeUnsupported("accumulation of this dtype")
                b.np.outputs.append(("acc", k))
            else:
                dst = b.out_region(sym.shape, acc_dtype)
                if sym.dtype == torch.bfloat16:
                    b.call("mm_bf16_to_f32", sym, dst, sym.numel, 0, STREAM)
                elif sym.dtype == torch.float32:
                    b.copy(dst, sym)
                else:
                    raise NativeUnsupported("accumulation of this dtype")
                b.np.outputs.append(("block", b.out_chunk_of(dst.slot), dst.off, dst.shape, dst.dtype))
            continue
        if b.out_chunk_of(sym.slot) is not None:
            b.np.outputs.append(("block", b.out_chunk_of(sym.slot), sym.off, sym.shape, sym.dtype))
        elif sym.slot < b.n_in:
            if sym.off != 0:
                raise NativeUnsupported("task output is a slice of a task input")
            b.np.outputs.append(("input", sym.slot, sym.shape))
        else:
            # an output that ended up in scratch (it aliases an intermediate): give it its own region
            dst = b.out_region(sym.shape, sym.dtype)
            b.copy(dst, sym)
            b.np.outputs.append(("block", b.out_chunk_of(dst.slot), dst.off, dst.shape, dst.dtype))
    b.np.out_chunks = list(b.out_chunks)
    b.np.out_block_bytes = sum(b.out_chunks)
    b.np.scratch_bytes = b.scratch.peak
    return b.np


def _reads_of(ins: Instr) -> List[int]:
    if ins.kind in (0, 6):
        return _tensor_ids_in_order(ins.args, ins.kwargs)
    return [ins.args] if isinstance(ins.args, int) else []


def plan_store_dtype(plan: dict, template: dict, out_pos: int) -> str:
    """dtype of the store that output ``out_pos`` of ``template`` is written to."""
    for op in plan["ops"]:
        if op["kind"] == "task" and op["template"] == template["id"]:
            return plan["stores"][op["outputs"][out_pos]]["shape"]["dtype"]
    raise NativeUnsupported("template is never launched")
