"""Norms.  RMSNorm as the reference computes it: `ss = sum x^2;
r = 1/sqrtf(ss/size + eps); out = (x*r)*w` (picolm/tensor.c:2942-3064), the
weight used as stored (the reference's safetensors loader adds 1.0 to it,
picolm/model_core.c:993-995, which suits another model family, not this one)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import Part, WeightSpec, register_part
from .stream import BiasedDelta, PostNormed, ResidualStream, pending_addends


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    """params: size, eps, name (the weight's tensor name relative to the part's prefix; default "weight", ""
    for a tensor that is called by the prefix alone), one_plus (True: the weight is stored around zero and the row
    is multiplied by 1 + w; the sum is made once, in float32, when the weights are loaded).  Weight: [size]."""

    @property
    def _name(self) -> str:
        return self.params.get("name", "weight")

    @property
    def one_plus(self) -> bool:
        return bool(self.params.get("one_plus", False))

    def weight_specs(self):
        return {self._name: WeightSpec((self.params["size"],), init="normal" if self.one_plus else "ones_normal")}

    def load(self, tensors):
        self.weight = tensors[self._name]
        if self.one_plus:
            # 1 + w has more digits than the stored type holds: kept in float32 (the norm kernels take either)
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def weight_f32(self) -> torch.Tensor:
        """The weight in float32 (made once), for kernels that apply this norm to a float32 delta on the way."""
        w = getattr(self, "_weight_f32", None)
        if w is None:
            w = self._weight_f32 = self.weight.to(torch.float32).contiguous()
        return w

    @property
    def can_defer_scale(self) -> bool:
        """Whether the scale may be left to the products that take the result (their epilogues apply a weight of the
        run's type, which 1 + w is not)."""
        return not self.one_plus

    graph_safe = True
    graph_safe_prompts = True

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, defer_scale: bool = False):
        """Normalise `x + pending`.  Without `rows` the sum is written back to the
        stream and the delta is consumed; with `rows` only those rows are
        normalised and the stream is left as it is.

        With `defer_scale` (the caller hands the result to products only) a pending product runs
        with the add, this norm's weight and the sums of squares in its epilogue, and the result is
        `ops.ScaledRows`: the product that takes it applies the scale."""
        p = stream.pending
        if isinstance(p, PostNormed):
            # a sublayer's result that wants a norm of its own before the add: both norms and the add in one kernel
            if rows is None and ops.post_pre_norm_supported(stream.x, p.delta, p.norm.weight, self.weight):
                stream.pending = None
                return ops.post_pre_norm(stream.x, p.delta, p.norm.weight, p.norm.params["eps"], self.weight,
                                         self.params["eps"], self.runtime.dtype)
            stream.pending = p.compute()
        if isinstance(stream.pending, BiasedDelta):
            stream.pending = stream.pending.compute()
        if (defer_scale and rows is None
                and ops.residual_norm_supported(stream.pending, stream.x, self.weight)):
            h = ops.linear_residual_norm(stream.pending, stream.x, self.weight, self.params["eps"])
            stream.pending = None
            return h
        h = ops.rmsnorm(stream.x, self.weight, self.params["eps"], self.runtime.dtype,
                        delta=stream.pending, rows=rows)
        if rows is None:
            stream.pending = None
        return h

    def normalize(self, rows: torch.Tensor) -> torch.Tensor:
        """The norm of float32 rows that are not the stream (a sublayer's result, normalised before it is added);
        float32 [T, size]."""
        return ops.rmsnorm(rows, self.weight, self.params["eps"], torch.float32)


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """Layer norm with a weight and no bias: `(x - mean) / sqrt(var + eps) * w`, var the mean squared deviation.
    params: size, eps, name (the weight's tensor name relative to the part's prefix; default "weight", "" for a
    tensor that is called by the prefix alone).  Weight: [size].  Statistics and the stream in float32."""

    graph_safe = True
    graph_safe_prompts = True

    @property
    def _name(self) -> str:
        return self.params.get("name", "weight")

    def weight_specs(self):
        return {self._name: WeightSpec((self.params["size"],), init="ones_normal")}

    def load(self, tensors):
        self.weight = tensors[self._name]

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, defer_scale: bool = False):
        """Normalise `x + pending` (the pending delta with its bias, if it has one, added in the same pass).  Without
        `rows` the sum is written back to the stream and the delta is consumed; with `rows` only those rows are
        normalised and the stream is left as it is."""
        p, bias = stream.pending, None
        if isinstance(p, PostNormed):
            p = p.compute()
        if isinstance(p, BiasedDelta):
            p, bias = p.delta, p.bias
        h = ops.layernorm(stream.x, self.weight, self.params["eps"], self.runtime.dtype, delta=p, bias=bias, rows=rows)
        if rows is None:
            stream.pending = None
        return h


@register_part("norm", "dyt")
class DynamicTanh(Part):
    """A norm that computes no mean and no variance: `tanh(alpha * x) * w + b` elementwise, alpha one learned number.
    params: size, name (the weight's tensor name relative to the part's prefix, "" for the prefix alone; default
    "weight"), alpha_name and bias_name (default: the weight's name with ".alpha" / ".b" added).  Tensors: weight and
    bias [size], alpha [].  Everything in float32 on the float32 stream."""

    graph_safe = True
    graph_safe_prompts = True

    def _names(self):
        base = self.params.get("name", "weight")
        sub = (lambda s: (base + "." + s) if base else s)
        return base, self.params.get("alpha_name", sub("alpha")), self.params.get("bias_name", sub("b"))

    def weight_specs(self):
        w, a, b = self._names()
        n = self.params["size"]
        return {w: WeightSpec((n,), init="ones_normal"), a: WeightSpec((), init="uniform", lo=0.4, hi=1.2),
                b: WeightSpec((n,), init="normal")}

    def load(self, tensors):
        w, a, b = self._names()
        self.weight = tensors[w].to(torch.float32).contiguous()
        self.alpha = tensors[a].to(torch.float32).reshape(1).contiguous()
        self.bias = tensors[b].to(torch.float32).contiguous()

    def weight_bytes(self):
        return 4 * (self.weight.numel() + self.bias.numel() + 1)

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None, defer_scale: bool = False):
        """The norm of `x + pending`: a pending delta, its bias or its own RMS norm are added in the same pass.
        Without `rows` the sum is written back to the stream and the delta is consumed; with `rows` only those rows
        are normalised and the stream is left as it is."""
        delta, bias, post_w, post_eps = pending_addends(stream.pending)
        h = ops.dyt_norm(stream.x, self.runtime.dtype, alpha=self.alpha, weight=self.weight, bias=self.bias, delta=delta,
                         delta_bias=bias, post_weight=post_w, post_eps=post_eps, rows=rows)
        if rows is None:
            stream.pending = None
        return h
