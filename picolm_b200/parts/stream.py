"""The residual stream of a step: fp32 `x` [T, d] and the delta that the last
part produced and that has not been added yet.  The add is folded into the next
norm (one pass over the stream instead of two)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class PostNormed:
    """A sublayer's float32 result that is still to be normalised (by `norm`, an RMSNorm part) before it is added to
    the stream: the next norm over the stream may do both in one kernel; anything else calls `compute()`."""
    __slots__ = ("delta", "norm")

    def __init__(self, delta: torch.Tensor, norm):
        self.delta, self.norm = delta, norm

    @property
    def shape(self):
        return self.delta.shape

    def compute(self) -> torch.Tensor:
        return self.norm.normalize(self.delta)

    def adds_in_place(self, x: torch.Tensor) -> bool:
        return False


class BiasedDelta:
    """A sublayer's result whose last projection has a bias that no product's epilogue adds: `delta` (float32 rows,
    or a product that has not run) plus `bias` (float32 [d]).  A norm that reads the stream next may add both in its
    own pass; anything else calls `compute()`."""
    __slots__ = ("delta", "bias")

    def __init__(self, delta, bias: torch.Tensor):
        self.delta, self.bias = delta, bias

    @property
    def shape(self):
        return self.delta.shape

    def compute(self) -> torch.Tensor:
        from .. import ops
        rows = self.delta.compute() if hasattr(self.delta, "compute") else self.delta
        return ops.add_bias(rows, self.bias)

    def adds_in_place(self, x: torch.Tensor) -> bool:
        return False


@dataclass
class ResidualStream:
    x: torch.Tensor                              # fp32 [T, d]
    pending: Optional[torch.Tensor] = None       # fp32 [T, d], to be added to x
    narrowed: bool = False                       # `narrow` has run: the rows are the wanted rows, in their order

    def narrow(self, rows: torch.Tensor) -> None:
        """Keep the rows `rows` (int32, on the device) only, in that order: what is left of a step's last layer
        once its mixer has seen all tokens is needed at the wanted rows alone.  A product that has not run yet
        (`ops.PendingLinear`) is narrowed at its left operand: it then runs on those rows."""
        from .. import ops
        self.x = ops.gather_rows(self.x, rows)
        if self.pending is not None:
            self.pending = _narrowed(self.pending, rows)
        self.narrowed = True


def pending_addends(p):
    """A pending delta as the addends a kernel that folds it into the stream takes: (rows or a product that has not
    run, bias vector or None, weight of the delta's own RMS norm or None, that norm's eps)."""
    if isinstance(p, PostNormed):
        return p.delta, None, p.norm.weight_f32(), float(p.norm.params["eps"])
    if isinstance(p, BiasedDelta):
        return p.delta, p.bias, None, 0.0
    return p, None, None, 0.0


def settle(stream: "ResidualStream", dtype, vec: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None):
    """Add what is pending (and, if given, the float32 vector `vec` [d] and the float32 rows `extra` [T, d]) to the
    stream; returns the sum in `dtype` (None: returns nothing).  For parts that read the stream itself, not a norm
    of it."""
    from .. import ops
    p = stream.pending
    if vec is not None and isinstance(p, BiasedDelta):
        p = p.compute()                       # one vector a pass
    delta, bias, post_w, post_eps = pending_addends(p)
    stream.pending = None
    return ops.dyt_norm(stream.x, dtype, delta=delta, delta_bias=bias if vec is None else vec, post_weight=post_w,
                        post_eps=post_eps, extra=extra)


def _narrowed(p, rows):
    """The pending delta `p` at the rows `rows` only."""
    from .. import ops
    if isinstance(p, PostNormed):
        return PostNormed(ops.gather_rows(p.delta, rows), p.norm)
    if isinstance(p, BiasedDelta):
        return BiasedDelta(_narrowed(p.delta, rows), p.bias)
    if isinstance(p, ops.PendingLinear):
        a = p.a.materialize() if isinstance(p.a, ops.LazyRows) else p.a
        return ops.PendingLinear(ops.gather_rows(a, rows), p.w)
    return ops.gather_rows(p, rows)
