"""Mixers: the part of a layer that lets tokens see other tokens.

Interface of the family: `cache_spec()` says what the layer needs of the cache
(`CacheSpec.kv`, `CacheSpec.state` or None); `prepare(max_seq_tokens)` runs once
before the first step; `forward(h, step, cache)` takes the normed activations
[T, d] of the step's tokens and returns the residual delta [T, d] in fp32.

Attention as the reference computes it: q/k/v projections without bias, RoPE on
q and k, keys and values appended to the cache, causal softmax(q.K * scale) . V
with consecutive query heads sharing a KV head (`g = h / (H/G)`), then the output
projection (picolm/model_core.c:1849-2151, picolm/model_attention.c:43-140).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.spec import CacheSpec
from ..config.spec import PartSpec
from .base import Part, WeightSpec, build_part, register_part
from .stream import BiasedDelta


def _stack_rows(tensors):
    """Concatenate weight matrices along the output features.  If their stored
    types differ, all are widened to float32 (exact)."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(list(tensors), dim=0).contiguous()


@register_part("mixer", "attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale (None:
    1/sqrt(head_dim)), window (None: all keys), position (a PartSpec of the
    position family), q_name/k_name/v_name/o_name (relative tensor names).

    Optional, for designs that have them (absent: the reference's attention):
      value_dim     width of a value head where it differs from head_dim (the keys' and queries')
      chunk         a mask of chunks: a query sees the earlier keys of its own chunk of that many positions, chunks
                    counted from position 0 of the sequence
      bias          True: q, k, v and o have biases, tensors `<name><bias_suffix>` (default ".b")
      qk_norm       {"eps", "q_name", "k_name"}: queries and keys are divided by their root mean square over ALL heads
                    at once and multiplied by those weights ([H * head_dim], [G * head_dim]), after the bias and
                    before the rotation; with "per_head": True the root mean square is each head's own and the
                    weights are [head_dim], shared by the heads
      values_from_keys  True: there is no value projection; the keys as projected (bias added, before norm and
                    rotation) serve as values
      sink_name     a tensor [num_heads]: the softmax's denominator of head h also holds exp(sink[h]), a term with no
                    key and no value that the scale does not touch
      own_kv        False: the layer has no key and value tensors (projections, biases, key norm); it attends over
                    what the layer it borrows its cache from wrote
      sink_value    a number instead of a tensor: every head's denominator also holds exp(sink_value) (0: one more 1)
      gate_name     a tensor [num_heads * value_dim, hidden]: the concatenated heads are multiplied element by element
                    by sigmoid(W_g h) before the output projection (W_g rides in the QKV product)
      conv          {"taps", "suffix"}: a short causal convolution over time on every channel of q, k and v straight
                    after the projection (before norm and rotation), no bias, no activation; tensors
                    `<q_name|k_name|v_name><suffix>` [channels, taps], the last tap the token's own.  The last taps - 1
                    projected rows of a sequence are kept beside the keys and values (a cache of the layer's own
                    even where keys and values are borrowed)
      head_scale_name  a tensor [num_heads]: head h's scores are multiplied by it (its queries are, after the rotation)
    With any of value_dim, bias, qk_norm or own_kv=False, what stands between the QKV product and attention is one
    kernel (`ops.qk_norm_rope_store`: bias, norm and rotation in float32 on the product's float32 result) and the
    cache keeps heads of one width, max(head_dim, value_dim) rounded up to 16, the narrower of keys and values padded
    with zeros (the output projection's columns are padded likewise, once, when the weights are loaded)."""

    @property
    def graph_safe(self) -> bool:
        """forward() launches kernels whose dependence on the step goes through device buffers only (apart
        from sizes fixed per batch size); the position encoding has to say the same of itself."""
        return bool(getattr(self.position, "graph_safe", False))

    @property
    def graph_safe_prompts(self) -> bool:
        return bool(getattr(self.position, "graph_safe_prompts", False))

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.H, self.G, self.hd, self.d = p["num_heads"], p["num_kv_heads"], p["head_dim"], p["hidden_size"]
        if self.H % self.G:
            raise ValueError(f"num_heads={self.H} is not a multiple of num_kv_heads={self.G}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.window = p.get("window")
        self.chunk = p.get("chunk")
        if self.chunk is not None and (self.window is not None or int(self.chunk) <= 0):
            raise ValueError("a mask of chunks needs a positive size and excludes a sliding window")
        self.vd = int(p.get("value_dim") or self.hd)
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.per_head_norm = bool(self.qk_norm and self.qk_norm.get("per_head", False))
        self.own_kv = bool(p.get("own_kv", True))
        self.v_from_k = bool(p.get("values_from_keys", False))
        if self.v_from_k and (self.vd != self.hd or not self.own_kv):
            raise ValueError("keys that serve as values need value_dim == head_dim and keys of the layer's own")
        self.sink_name = p.get("sink_name")
        self.sink_value = p.get("sink_value")
        if self.sink_name is not None and self.sink_value is not None:
            raise ValueError("attention: a learned sink and a constant one at once")
        self.gate_name, self.head_scale_name = p.get("gate_name"), p.get("head_scale_name")
        self.conv = p.get("conv")
        if self.conv is not None and (int(self.conv["taps"]) < 1 or self.v_from_k or self.bias):
            raise ValueError("attention: a convolution needs at least one tap, values of their own and projections without bias")
        # the general form: its own kernel between the product and attention, a cache of padded heads
        self.general = (self.vd != self.hd or self.bias or self.qk_norm is not None or not self.own_kv or self.v_from_k
                        or self.sink_name is not None or self.sink_value is not None or self.gate_name is not None
                        or self.conv is not None or self.head_scale_name is not None)
        self.hd_c = -(-max(self.hd, self.vd) // 16) * 16 if self.general else self.hd
        pos = p.get("position") or PartSpec("none")
        self.position = build_part("position", pos, runtime)
        if self.general and not hasattr(self.position, "rotation") and pos.kind != "none":
            raise ValueError(f"attention with a bias, a norm of q and k or values of another width needs a position "
                             f"encoding that is a rotation (or none), not {pos.kind!r}")

    def _names(self):
        """(tensor names of the projections that feed attention, in the order of their rows in the one product)."""
        p = self.params
        return [p["q_name"]] + (([p["k_name"]] if self.v_from_k else [p["k_name"], p["v_name"]]) if self.own_kv else [])

    def weight_specs(self):
        p, H, G, hd, vd, d = self.params, self.H, self.G, self.hd, self.vd, self.d
        specs = {p["q_name"]: WeightSpec((H * hd, d)), p["o_name"]: WeightSpec((d, H * vd))}
        if self.own_kv:
            specs[p["k_name"]] = WeightSpec((G * hd, d))
            if not self.v_from_k:
                specs[p["v_name"]] = WeightSpec((G * vd, d))
        if self.sink_name is not None:
            specs[self.sink_name] = WeightSpec((H,), init="normal_scaled", scale=1.0)
        if self.gate_name is not None:
            specs[self.gate_name] = WeightSpec((H * vd, d))
        if self.head_scale_name is not None:
            specs[self.head_scale_name] = WeightSpec((H,), init="uniform", lo=0.5, hi=1.5)
        if self.conv is not None:
            for name in self._names():
                specs[name + self.conv.get("suffix", ".conv")] = WeightSpec((specs[name].shape[0], int(self.conv["taps"])),
                                                                            init="normal_scaled", scale=0.5)
        if self.bias:
            sfx = p.get("bias_suffix", ".b")
            for name in self._names() + [p["o_name"]]:
                specs[name + sfx] = WeightSpec((specs[name].shape[0],), init="normal")
        if self.qk_norm is not None:
            specs[self.qk_norm["q_name"]] = WeightSpec((hd if self.per_head_norm else H * hd,), init="ones_normal")
            if self.own_kv:
                specs[self.qk_norm["k_name"]] = WeightSpec((hd if self.per_head_norm else G * hd,), init="ones_normal")
        return specs

    def load(self, tensors):
        p = self.params
        # one projection for q, k and v: rows [q heads | k heads | v heads], and behind them the gate's rows
        rows = [tensors[n] for n in self._names()]
        self.n_qkv = sum(t.shape[0] for t in rows)
        if self.gate_name is not None:
            g = tensors[self.gate_name]
            if self.hd_c != self.vd:
                # the gate meets heads of the cache's width: rows of zeros where attention hands back zeros
                wide = torch.zeros((self.H, self.hd_c, self.d), dtype=g.dtype, device=g.device)
                wide[:, :self.vd] = g.view(self.H, self.vd, self.d)
                g = wide.view(self.H * self.hd_c, self.d)
            rows.append(g)
        self.w_qkv = _stack_rows(rows)
        self.w_o = tensors[p["o_name"]]
        self.b_qkv = self.b_o = self.w_qn = self.w_kn = None
        self.sink = None if self.sink_name is None else tensors[self.sink_name].to(torch.float32).contiguous()
        if self.sink_value is not None:
            self.sink = torch.full((self.H,), float(self.sink_value), dtype=torch.float32, device=self.w_o.device)
        self.head_scale = (None if self.head_scale_name is None
                           else tensors[self.head_scale_name].to(torch.float32).contiguous())
        self.w_conv = None
        if self.conv is not None:
            # tap-major [taps, channels] in float32, the channels in the order of the product's columns
            sfx = self.conv.get("suffix", ".conv")
            self.w_conv = torch.cat([tensors[n + sfx].to(torch.float32) for n in self._names()]).t().contiguous()
        if self.bias:
            sfx = p.get("bias_suffix", ".b")
            self.b_qkv = torch.cat([tensors[n + sfx].to(torch.float32) for n in self._names()]).contiguous()
            self.b_o = tensors[p["o_name"] + sfx].to(torch.float32).contiguous()
        if self.qk_norm is not None:
            self.w_qn = tensors[self.qk_norm["q_name"]].to(self.runtime.dtype).contiguous()
            if self.own_kv:
                self.w_kn = tensors[self.qk_norm["k_name"]].to(self.runtime.dtype).contiguous()
        if self.general and self.hd_c != self.vd:
            # attention hands back heads of the cache's width: the columns beyond a value head's own meet zeros
            w = torch.zeros((self.d, self.H, self.hd_c), dtype=self.w_o.dtype, device=self.w_o.device)
            w[:, :, :self.vd] = self.w_o.view(self.d, self.H, self.vd)
            self.w_o = w.view(self.d, self.H * self.hd_c).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def cache_spec(self):
        # (chunks: pages are kept; a layer that borrows this cache may cut its chunks elsewhere)
        return CacheSpec.kv(self.G, self.hd_c, self.window)

    def cache_specs(self):
        """The keys and values, and for a convolution the last taps - 1 projected rows of every sequence (the layer's
        own even where it borrows keys and values).  `forward` takes them in this order, or the first alone."""
        specs = [self.cache_spec()]
        if self.conv is not None and int(self.conv["taps"]) > 1:
            cols = self.H * self.hd + ((self.G * self.hd + self.G * self.vd) if self.own_kv else 0)
            specs.append(CacheSpec.state(((int(self.conv["taps"]) - 1) * cols,), private=True))
        return specs

    def prepare(self, max_seq_tokens: int) -> None:
        self.position.prepare(max_seq_tokens)

    takes_scaled_rows = True          # h goes into a product and nowhere else

    def _forward_general(self, h, step, cache, conv_state=None):
        dt = self.runtime.dtype
        if self.own_kv and not cache.writable:
            raise RuntimeError("a layer that reads another layer's cache must be built with own_kv=False")
        proj = ops.linear(h, self.w_qkv, torch.float32)      # bias, norm and rotation work on the float32 sums
        qkv = proj[:, :self.n_qkv] if self.gate_name is not None else proj
        if self.w_conv is not None and self.w_conv.shape[0] > 1 and conv_state is None:
            raise RuntimeError("attention with a convolution was handed no state for it")
        q = torch.empty((h.shape[0], self.H, self.hd_c), dtype=dt, device=h.device)
        rotation = self.position.rotation() if hasattr(self.position, "rotation") else None
        ops.qk_norm_rope_store(qkv, self.b_qkv, self.w_qn, self.w_kn, self.qk_norm["eps"] if self.qk_norm else 0.0, q,
                               cache, rotation, step, self.H, self.G, self.hd, self.vd, own_kv=self.own_kv,
                               per_head=self.per_head_norm, values_from_keys=self.v_from_k, q_scale=self.head_scale,
                               conv=self.w_conv, conv_state=conv_state.state if conv_state is not None else None)
        ctx = ops.attention(q, cache, step, self.G, self.scale, chunk=self.chunk, sink=self.sink)
        if self.gate_name is not None:
            ctx = ops.gated_norm(ctx, dt, group=self.hd_c, gate=proj[:, self.n_qkv:], gate_mode=ops.GATE_AFTER_NORM,
                                 activation="sigmoid", norm=False)
        delta = ops.linear(ctx, self.w_o, torch.float32, defer=True)
        return BiasedDelta(delta, self.b_o) if self.b_o is not None else delta

    def forward(self, h, step, cache):
        conv_state = None
        if isinstance(cache, (list, tuple)):                 # all of `cache_specs()`, in their order
            conv_state = cache[1] if len(cache) > 1 else None
            cache = cache[0]
        if self.general:
            return self._forward_general(h, step, cache, conv_state)
        dt = self.runtime.dtype
        qkv = ops.linear(h, self.w_qkv, dt)
        # a position encoding that can describe itself as a rotation (`rotation()`) may be applied, and the
        # cache written, by the decode attention kernel itself
        rotation = (self.position.rotation() if step.is_decode and not self.chunk and hasattr(self.position, "rotation")
                    else None)
        if rotation is not None and ops.attention_decode_rope_supported(qkv, cache, rotation, self.hd):
            ctx = ops.attention_decode_rope(qkv, cache, step, self.H, self.G, self.hd, self.scale, rotation)
        else:
            q = torch.empty((h.shape[0], self.H, self.hd), dtype=dt, device=h.device)
            self.position.apply(qkv, q, cache, step, self.H, self.G, self.hd)
            ctx = ops.attention(q, cache, step, self.G, self.scale, chunk=self.chunk)
        return ops.linear(ctx, self.w_o, torch.float32, defer=True)


def _rows(delta):
    """(float32 rows, bias vector or None) of a mixer's result, whatever form it was handed back in."""
    bias = None
    if isinstance(delta, BiasedDelta):
        delta, bias = delta.delta, delta.bias
    if hasattr(delta, "compute"):
        delta = delta.compute()
    return delta, bias


@register_part("mixer", "parallel")
class ParallelMixers(Part):
    """Two mixers side by side that read the same normed rows; the result is `left_scale * left + right_scale *
    right`.  params: left, right (`PartSpec`s of the mixer family; their `prefix` is where their tensors live below
    this part's), left_scale, right_scale.  Each half keeps what it keeps in the cache: the layer's caches are the
    left's, then the right's (`cache_specs`), and `forward` takes them as a list."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        self.halves = [(self.params[side].prefix, build_part("mixer", self.params[side], runtime)) for side in ("left", "right")]
        self.scales = (float(self.params["left_scale"]), float(self.params["right_scale"]))

    @property
    def graph_safe(self) -> bool:
        return all(bool(getattr(part, "graph_safe", False)) for _, part in self.halves)

    @property
    def graph_safe_prompts(self) -> bool:
        return all(bool(getattr(part, "graph_safe_prompts", False)) for _, part in self.halves)

    def weight_specs(self):
        return {(f"{prefix}.{name}" if prefix else name): ws for prefix, part in self.halves
                for name, ws in part.weight_specs().items()}

    def load(self, tensors):
        for prefix, part in self.halves:
            part.load({name: tensors[f"{prefix}.{name}" if prefix else name] for name in part.weight_specs()})

    def weight_bytes(self):
        return sum(part.weight_bytes() for _, part in self.halves)

    def cache_specs(self):
        return [s for _, part in self.halves for s in ([part.cache_spec()] if part.cache_spec() is not None else [])]

    def cache_spec(self):
        specs = self.cache_specs()
        return specs[0] if specs else None

    def prepare(self, max_seq_tokens: int) -> None:
        for _, part in self.halves:
            prep = getattr(part, "prepare", None)
            if prep is not None:
                prep(max_seq_tokens)

    def forward(self, h, step, caches):
        caches = list(caches)
        results = []
        for _, part in self.halves:
            cache = caches.pop(0) if part.cache_spec() is not None else None
            results.append(_rows(part.forward(h, step, cache)))
        (left, left_bias), (right, right_bias) = results
        if right_bias is not None:
            right = ops.add_bias(right, right_bias)
        return ops.scaled_sum(left, self.scales[0], right, self.scales[1], bias_a=left_bias)
