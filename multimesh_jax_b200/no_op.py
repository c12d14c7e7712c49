"""Marker operations that carry front-end annotations into the captured graph.

The reference builds JAX primitives that lower to side-effect-free custom
calls and transpose to themselves so that they survive ``grad``
(``multimesh/jax/no_op.py:27-97``). Here a single ``torch.library`` operator
``mm::marker(x, kind, payload)`` plays that role: it is the identity on ``x``,
shows up as one node in the ``torch.fx`` capture, and its autograd formula
applies the same marker to the incoming gradient (for kinds that are linear
annotations, e.g. sharding hints) or passes the gradient through unchanged.
"""
from __future__ import annotations

import json
from typing import Any, Callable

import torch

_LIB = torch.library.Library("mm", "DEF")
_LIB.define("marker(Tensor x, str kind, str payload) -> Tensor")


def _marker_impl(x, kind, payload):
    return x.clone()


def _marker_fake(x, kind, payload):
    return torch.empty_like(x)


torch.library.impl(_LIB, "marker", "CompositeExplicitAutograd")(_marker_impl)
torch.library.register_fake("mm::marker")(_marker_fake)

# Marker kinds whose annotation also applies to the cotangent.
_SELF_TRANSPOSING = {"AutoSharding"}


def _marker_setup_context(ctx, inputs, output):
    _, kind, payload = inputs
    ctx.kind = kind
    ctx.payload = payload


def _marker_backward(ctx, grad):
    if ctx.kind in _SELF_TRANSPOSING:
        return torch.ops.mm.marker(grad, ctx.kind, ctx.payload), None, None
    if ctx.kind == "Relayout" and ctx.payload:
        # a layout change point with a stated cotangent layout is mirrored in the backward pass
        p = json.loads(ctx.payload)
        if "grad_axes" in p:
            back = {"axes": p["grad_axes"], "logical": p.get("logical", True), "grad_axes": p["axes"]}
            return torch.ops.mm.marker(grad, "Relayout", json.dumps(back)), None, None
    return grad, None, None


torch.library.register_autograd("mm::marker", _marker_backward, setup_context=_marker_setup_context)

# Names understood by the graph compiler (the wire format between front end and passes).
MICROBATCH = "Microbatch"
MICROBATCH_SLICE = "MicrobatchSlice"
MICROBATCH_INIT = "MicrobatchInit"
MICROBATCH_OUT = "MicrobatchOut"
AUTO_SHARDING = "AutoSharding"
MARKING = "Marking"


def no_op(name: str) -> Callable[..., torch.Tensor]:
    """Returns ``f(x, config)`` that tags ``x`` with a marker called ``name``.

    ``config`` may be any JSON-serialisable object (or a string, passed as is).
    Outside a capture the function is the identity.
    """

    def apply(x: torch.Tensor, config: Any = "") -> torch.Tensor:
        from . import state
        if not state.trace.active:
            return x
        payload = config if isinstance(config, str) else json.dumps(config)
        return torch.ops.mm.marker(x, name, payload)

    apply.__name__ = f"no_op_{name}"
    return apply


_marking = no_op(MARKING)


def mark_gradient(x: torch.Tensor) -> torch.Tensor:
    """Tags ``x`` as a gradient (informational; no pass depends on it)."""
    return _marking(x, "gradient")


def mark_loss(x: torch.Tensor) -> torch.Tensor:
    """Tags ``x`` as the loss (informational; no pass depends on it)."""
    return _marking(x, "loss")
