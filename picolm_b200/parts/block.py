"""Arrangements: how one layer's norms, mixers and feed-forwards are wired around
the residual stream.  Interface of the family: built from `(layer_spec,
runtime)`; the arrangement alone reads `layer_spec.parts` (which parts a layer has
and what they are called is its business, not the model's);
`parts()` lists `(relative prefix, part)` for the weights; `cache_specs()` lists
what the layer wants of the cache, one `CacheSpec` per part that keeps something;
`prepare(max_seq_tokens)` runs once before the first step;
`forward(stream, step, caches)` runs the layer on the stream in place, `caches`
holding one entry per entry of `cache_specs()`, in that order.  An arrangement
with `narrows_rows = True` also takes `keep_rows=`: the rows that anything after the
layer will read (the model says so to the last layer of a step), so that it may
narrow the stream to them as soon as its parts no longer need the others.

`pre_norm` is the reference's Llama layer: `x += mixer(norm(x));
x += feed_forward(norm(x))` (picolm/model_core.c:1797-2210).
"""
from __future__ import annotations

from typing import List

import torch

from .. import ops
from ..cache.spec import CacheSpec
from ..config.spec import LayerSpec, PartSpec
from .base import Part, WeightSpec, build_part, register_part
from .stream import PostNormed, settle


class Arrangement(Part):
    """Base of the arrangements: builds every part the layer's spec names and answers the model's
    questions from them.  A subclass says which names it needs (`wants`) and how they are wired
    (`forward`)."""

    wants: tuple = ()
    narrows_rows = False

    def __init__(self, layer_spec: LayerSpec, runtime):
        super().__init__(dict(getattr(layer_spec, "params", None) or {}), runtime)
        self.spec = layer_spec
        missing = [n for n in self.wants if n not in layer_spec.parts]
        if missing:
            raise ValueError(f"layer {layer_spec.prefix!r}: the {self.kind} arrangement needs the parts "
                             f"{', '.join(missing)}; the spec has {', '.join(sorted(layer_spec.parts))}")
        self.named = {name: build_part(family, spec, runtime) for name, (family, spec) in layer_spec.parts.items()}
        for name, part in self.named.items():
            setattr(self, name, part)

    def parts(self):
        return [(self.spec.parts[name][1].prefix, part) for name, part in self.named.items()]

    def cache_owners(self) -> List[str]:
        """Names of the parts that keep something in the cache, in the order of `cache_specs()`."""
        return [name for name, part in self.named.items()
                if getattr(part, "cache_spec", None) is not None and part.cache_spec() is not None]

    def cache_specs(self):
        """One entry per thing kept; a part that keeps several (`cache_specs()` of its own) has them side by side."""
        out = []
        for name in self.cache_owners():
            part = self.named[name]
            out.extend(part.cache_specs() if hasattr(part, "cache_specs") else [part.cache_spec()])
        return out

    def _mixer_cache(self, caches):
        """What the mixer is handed of the layer's caches: its one cache, or all of them if it keeps several."""
        if hasattr(self.mixer, "cache_specs"):
            return caches
        return caches[0] if caches else None

    def prepare(self, max_seq_tokens: int) -> None:
        for part in self.named.values():
            prep = getattr(part, "prepare", None)
            if prep is not None:
                prep(max_seq_tokens)

    @staticmethod
    def _norm(norm, consumer, stream):
        """A norm may leave its scale to the products of the part that takes its result, when both
        say that they can (`can_defer_scale`, `takes_scaled_rows`)."""
        if getattr(norm, "can_defer_scale", False) and getattr(consumer, "takes_scaled_rows", False):
            return norm.forward(stream, defer_scale=True)
        return norm.forward(stream)


@register_part("arrangement", "pre_norm")
class PreNormBlock(Arrangement):
    """`x += mixer(norm(x)); x += feed_forward(norm'(x))`; the feed-forward and its norm are optional (a layer that
    only mixes).  Optional too: `token_input` with `token_input_norm`, a last step `x += norm''(input(x, token))`."""
    wants = ("mixer_norm", "mixer")

    narrows_rows = True

    def forward(self, stream, step, caches, keep_rows=None):
        """`keep_rows` (the model gives it to the last layer of a step when few rows are wanted): once the mixer
        has seen all tokens, the stream is narrowed to those rows and the feed-forward runs on them alone; with
        no row to keep, nothing runs after the mixer."""
        h = self._norm(self.mixer_norm, self.mixer, stream)
        stream.pending = self.mixer.forward(h, step, self._mixer_cache(caches))
        if keep_rows is not None:
            if keep_rows.numel() == 0:
                stream.pending = None
                return
            stream.narrow(keep_rows)
        if "feed_forward" in self.named:
            h = self._norm(self.feed_forward_norm, self.feed_forward, stream)
            stream.pending = self.feed_forward.forward(h, step)
        if "token_input" in self.named:
            # an input from the token itself, gated by the stream as the sublayers leave it; its result passes a norm
            # of its own before it is added, which is left to whatever reads the stream next
            x = settle(stream, self.runtime.dtype)
            stream.pending = PostNormed(self.token_input.forward(x, step, rows=keep_rows), self.token_input_norm)


def pre_norm_layer(prefix: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                   feed_forward_norm: PartSpec, cache_of=None, token_input: PartSpec = None,
                   token_input_norm: PartSpec = None) -> LayerSpec:
    """The spec of a `pre_norm` layer from its four parts; without `feed_forward` the layer only mixes.  With
    `token_input` (family "token_input") and `token_input_norm` (an RMS norm) the layer ends with `x += norm(input(x,
    token))`."""
    parts = {"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer)}
    if feed_forward is not None:
        parts.update({"feed_forward_norm": ("norm", feed_forward_norm), "feed_forward": ("feed_forward", feed_forward)})
    if token_input is not None:
        parts.update({"token_input": ("token_input", token_input), "token_input_norm": ("norm", token_input_norm)})
    return LayerSpec(prefix, "pre_norm", parts, cache_of=cache_of)


@register_part("arrangement", "sandwich_norm")
class SandwichNormBlock(Arrangement):
    """A norm before and a norm after each sublayer: `x += post(mixer(pre(x))); x += post'(feed_forward(pre'(x)))`.
    The norms after the sublayers work on the sublayer's float32 result, before it is added to the stream.  The
    feed-forward and its two norms are optional (a layer that only mixes)."""

    wants = ("mixer_norm", "mixer", "mixer_post_norm")
    narrows_rows = True

    @staticmethod
    def _rows(delta):
        return delta.compute() if hasattr(delta, "compute") else delta

    def forward(self, stream, step, caches, keep_rows=None):
        h = self.mixer_norm.forward(stream)
        delta = self._rows(self.mixer.forward(h, step, self._mixer_cache(caches)))
        if keep_rows is not None:
            # the last layer of a step: only these rows are read afterwards, and the norms go row by row
            if keep_rows.numel() == 0:
                stream.pending = None
                return
            stream.pending = delta
            stream.narrow(keep_rows)
            delta = stream.pending
        # the closing norms are left to the norm that reads the stream next: it does them with the add and its own work
        stream.pending = PostNormed(delta, self.mixer_post_norm)
        if "feed_forward" not in self.named:
            return
        h = self.feed_forward_norm.forward(stream)
        stream.pending = PostNormed(self._rows(self.feed_forward.forward(h, step)), self.feed_forward_post_norm)


def sandwich_norm_layer(prefix: str, mixer: PartSpec, mixer_norm: PartSpec, mixer_post_norm: PartSpec,
                        feed_forward: PartSpec = None, feed_forward_norm: PartSpec = None,
                        feed_forward_post_norm: PartSpec = None, cache_of=None) -> LayerSpec:
    """The spec of a `sandwich_norm` layer; without `feed_forward` the layer only mixes."""
    parts = {"mixer_norm": ("norm", mixer_norm), "mixer": ("mixer", mixer), "mixer_post_norm": ("norm", mixer_post_norm)}
    if feed_forward is not None:
        parts.update({"feed_forward_norm": ("norm", feed_forward_norm), "feed_forward": ("feed_forward", feed_forward),
                      "feed_forward_post_norm": ("norm", feed_forward_post_norm)})
    return LayerSpec(prefix, "sandwich_norm", parts, cache_of=cache_of)


@register_part("row_filter", "token_shift")
class TokenShift(Part):
    """What a mixer reads is moved towards the token before, element by element: `h_t + (h_(t-1) - h_t) * mu` with a
    learned `mu` [size], h_(t-1) as it was before this step was applied to it, zeros before a sequence's first token.
    The row before is part of the sequence's state.  params: size, name (the tensor of mu; default "shift", "" for
    the prefix alone).

    As a kernel this is a causal convolution over time with two taps (mu for the token before, 1 - mu for the
    token itself); a norm that can do it on the way (`ops.norm_pair_shift`) is handed `mu` and the state instead."""

    graph_safe = True
    graph_safe_prompts = True

    @property
    def _name(self) -> str:
        return self.params.get("name", "shift")

    def weight_specs(self):
        return {self._name: WeightSpec((self.params["size"],), init="uniform", lo=0.0, hi=1.0)}

    def load(self, tensors):
        self.mu = tensors[self._name].to(torch.float32).contiguous()
        self.taps = torch.stack([self.mu, 1.0 - self.mu]).contiguous()          # [2, size]: the token before, the token

    def weight_bytes(self):
        return 4 * self.mu.numel()

    def cache_spec(self):
        return CacheSpec.state((self.params["size"],), private=True)

    def forward(self, h, step, cache):
        return ops.causal_conv(h, self.taps, None, cache.state, step, activation=None)


@register_part("arrangement", "parallel_norm")
class ParallelNormBlock(Arrangement):
    """Mixer and feed-forward side by side, each behind a norm of its own of the same x:
    `x += scale * (mixer(filter(norm_a(x))) + feed_forward(norm_b(x)))`.  The feed-forward with its norm and the
    filter (family "row_filter": something done to the mixer's input alone) are optional; `scale` is the layer's
    `params["residual_scale"]` (default 1).

    Both norms are RMS norms here, so that one pass over a row serves both (and a `token_shift` filter with them:
    `ops.norm_pair_shift`); other norms run one after the other.  A feed-forward that can (`adds_to_stream`) puts
    `scale * (its own result + the mixer's)` into the stream itself."""

    wants = ("mixer_norm", "mixer")
    narrows_rows = True

    def __init__(self, layer_spec, runtime):
        super().__init__(layer_spec, runtime)
        self.scale = float(self.params.get("residual_scale", 1.0))

    def _caches(self, caches):
        """(the filter's cache, what the mixer is handed) of the layer's caches, which come in the order of the parts."""
        caches = list(caches or [])
        owners = self.cache_owners()
        filt = caches.pop(0) if owners and owners[0] == "mixer_filter" else None
        if hasattr(self.mixer, "cache_specs"):
            return filt, caches
        return filt, (caches[0] if caches else None)

    def _fused_norms(self) -> bool:
        from .norm import RMSNorm
        norms = [self.mixer_norm] + ([self.feed_forward_norm] if "feed_forward" in self.named else [])
        filt = self.named.get("mixer_filter")
        return (all(isinstance(n, RMSNorm) and n.weight.dtype == torch.float32 for n in norms)
                and len({float(n.params["eps"]) for n in norms}) == 1 and (filt is None or isinstance(filt, TokenShift)))

    def forward(self, stream, step, caches, keep_rows=None):
        dt = self.runtime.dtype
        filt_cache, mixer_cache = self._caches(caches)
        filt = self.named.get("mixer_filter")
        has_ff = "feed_forward" in self.named
        if keep_rows is not None and keep_rows.numel() == 0:
            has_ff = False                                            # nothing reads what this layer adds to the stream
        h_ff = None
        if self._fused_norms():
            settle(stream, None)                                      # x += what the layer before left
            h, h_ff = ops.norm_pair_shift(
                stream.x, self.mixer_norm.weight, float(self.mixer_norm.params["eps"]), dt,
                w_b=self.feed_forward_norm.weight if has_ff and keep_rows is None else None,
                mix=filt.mu if filt is not None else None, state=filt_cache.state if filt is not None else None, step=step)
        else:
            h = self.mixer_norm.forward(stream)
            if has_ff and keep_rows is None:
                h_ff = self.feed_forward_norm.forward(stream)
            if filt is not None:
                h = filt.forward(h, step, filt_cache)
        delta = self.mixer.forward(h, step, mixer_cache)
        if keep_rows is not None:
            # the last layer of a step: once the mixer has seen all tokens only these rows matter
            if keep_rows.numel() == 0:
                stream.pending = None
                return
            stream.pending = delta
            stream.narrow(keep_rows)
            delta, stream.pending = stream.pending, None
            if has_ff:
                h_ff = self.feed_forward_norm.forward(stream)
        if hasattr(delta, "compute"):
            delta = delta.compute()
        if not has_ff:
            stream.pending = delta if self.scale == 1.0 else ops.scaled_sum(delta, self.scale, delta, 0.0)
            return
        if getattr(self.feed_forward, "adds_to_stream", False):
            self.feed_forward.forward(h_ff, step, add=delta, out_scale=self.scale, into=stream.x)
            return
        other = self.feed_forward.forward(h_ff, step)
        if hasattr(other, "compute"):
            other = other.compute()
        stream.pending = ops.scaled_sum(delta, self.scale, other, self.scale)


def parallel_norm_layer(prefix: str, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: PartSpec = None,
                        feed_forward_norm: PartSpec = None, mixer_filter: PartSpec = None, residual_scale: float = 1.0,
                        cache_of=None) -> LayerSpec:
    """The spec of a `parallel_norm` layer; without `feed_forward` the layer only mixes.  `mixer_filter`: a part of
    the "row_filter" family between the mixer's norm and the mixer."""
    parts = {"mixer_norm": ("norm", mixer_norm)}
    if mixer_filter is not None:
        parts["mixer_filter"] = ("row_filter", mixer_filter)          # (in front of the mixer: the order of the layer's caches)
    parts["mixer"] = ("mixer", mixer)
    if feed_forward is not None:
        parts.update({"feed_forward_norm": ("norm", feed_forward_norm), "feed_forward": ("feed_forward", feed_forward)})
    return LayerSpec(prefix, "parallel_norm", parts, cache_of=cache_of, params={"residual_scale": float(residual_scale)})
