"""Feed-forwards.  Interface of the family: `forward(h, step)` takes the normed
activations [T, d] and returns the residual delta [T, d] in fp32.

The gated MLP as the reference computes it: `g = Wg x`, `u = Wu x`,
`h = g / (1 + expf(-g)) * u`, `delta = Wd h`, no bias
(picolm/model_core.c:2182-2204, picolm/tensor.c:3306-3315).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, WeightSpec, register_part
from .mixer import _stack_rows


@register_part("feed_forward", "gated_mlp")
class GatedMLP(Part):
    """params: hidden_size, intermediate_size, activation ("silu", or "gelu_tanh": the reference's gelu,
    picolm/tensor.c:3317-3323; or "swish_clamped" with its constants `limit` and `slope`: g' = min(g, limit),
    u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1)), gate_name/up_name/down_name (relative tensor names).  The product whose
    epilogue applies the activation exists for both (a build variant of the kernels for gelu_tanh); operands the
    tensor cores do not take run a plain product and the activation as a kernel of its own."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        if self.params["activation"] not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"activation {self.params['activation']!r} has no kernel; known: "
                             + ", ".join(ops.GATE_ACTIVATIONS))

    def weight_specs(self):
        p = self.params
        d, F = p["hidden_size"], p["intermediate_size"]
        return {
            p["gate_name"]: WeightSpec((F, d)),
            p["up_name"]: WeightSpec((F, d)),
            p["down_name"]: WeightSpec((d, F)),
        }

    def load(self, tensors):
        p = self.params
        gate, up = tensors[p["gate_name"]], tensors[p["up_name"]]
        # One projection for both branches.  Where the tensor-core product can apply the activation
        # in its epilogue, the rows are laid out in tiles of 64 gate rows and their 64 up rows;
        # otherwise plainly [gate | up] with the activation as a kernel of its own.
        self.fused = (p["activation"] in ("silu", "gelu_tanh", "swish_clamped") and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 and gate.shape[0] % 64 == 0
                      and gate.shape[1] % 8 == 0 and gate.shape[1] >= 64)
        self.w_gate_up = ops.interleave_gate_up(gate, up) if self.fused else _stack_rows([gate, up])
        self.w_down = tensors[p["down_name"]]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    takes_scaled_rows = True          # h goes into a product and nowhere else
    graph_safe = True
    graph_safe_prompts = True

    def forward(self, h, step):
        if self.fused:
            # handed to the next product and nowhere else
            act = ops.linear_swiglu(h, self.w_gate_up, defer=True, activation=self.params["activation"],
                                    limit=float(self.params.get("limit", 0.0)), slope=float(self.params.get("slope", 1.0)))
        else:
            act = ops.swiglu(ops.linear(h, self.w_gate_up, self.runtime.dtype), activation=self.params["activation"],
                             limit=float(self.params.get("limit", 0.0)), slope=float(self.params.get("slope", 1.0)))
        return ops.linear(act, self.w_down, torch.float32, defer=True)


@register_part("feed_forward", "routed_mlp")
class RoutedMLP(Part):
    """A mixture of experts: every token uses `top` of `experts` small gated MLPs (`W_down(silu(W_gate h) * W_up h)`,
    no biases), chosen by a router, and optionally one shared expert that every token uses.

    params: hidden_size, experts, top, expert_size (an expert's inner width), route_scale, groups (None, or
    {"count", "keep"}: the experts form `count` equal groups of neighbours, and only experts of the `keep` groups with
    the largest sums of their two best choice scores can be chosen), correction_name (None, or a tensor [experts]
    added to the scores for the choice only), router_name, expert_prefix (expert e's tensors are
    `<expert_prefix><e>.<gate_name|up_name|down_name>`), gate_name/up_name/down_name, shared (None, or
    {"size", "prefix", "gate"}: the shared expert's inner width, its tensors' prefix, and the name under that prefix of
    the [1, hidden] row whose sigmoid multiplies the shared expert's result per token; None: no such gate).

    Optional: scores ("sigmoid", or "softmax": over all router outputs), group_score ("top2", or "max": a group's
    score is its best choice score), normalize (False: the weights are the chosen scores as they are, times
    `route_scale`), identity (a number: the router has that many outputs more, behind the experts', for experts
    without tensors whose output is their input; they take part in scores, groups and choice like the others).

    The router's logits are a float32 product; scores are `sigmoid(logit)`; the weights of the chosen experts are
    their scores (without the correction) divided by their sum (+ 1e-20), times `route_scale`.  The choice stays on
    the device: the chosen (token, expert) pairs are sorted by expert into tiles, and the experts' products run over
    those tiles (`ops/routed.py`).

    `forward(h, step, add=, out_scale=, into=)`: the weighted sum can take a sublayer's float32 rows beside it, a
    factor on the sum of both, and the residual stream to add the result to (`adds_to_stream`)."""

    graph_safe = True
    graph_safe_prompts = True
    adds_to_stream = True

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.E, self.top, self.F, self.d = int(p["experts"]), int(p["top"]), int(p["expert_size"]), int(p["hidden_size"])
        g = p.get("groups")
        self.n_groups, self.keep = (int(g["count"]), int(g["keep"])) if g else (1, 1)
        self.identity = int(p.get("identity") or 0)
        self.n_out = self.E + self.identity                  # the router's outputs: experts, then identity experts
        self.scores, self.group_score = p.get("scores", "sigmoid"), p.get("group_score", "top2")
        self.normalize = bool(p.get("normalize", True))
        if self.scores not in ("sigmoid", "softmax") or self.group_score not in ("top2", "max"):
            raise ValueError(f"routed_mlp: scores={self.scores!r} (sigmoid, softmax) or group_score={self.group_score!r} "
                             f"(top2, max) is not known")
        if not 0 < self.top <= self.n_out or self.n_out % self.n_groups or not 0 < self.keep <= self.n_groups or self.identity < 0:
            raise ValueError(f"routed_mlp: top={self.top}, router outputs={self.n_out}, groups={self.n_groups}, "
                             f"kept={self.keep} do not fit together")
        if self.top > self.keep * (self.n_out // self.n_groups):
            raise ValueError(f"routed_mlp: {self.keep} groups of {self.n_out // self.n_groups} experts cannot give {self.top} choices")
        self.shared = None
        sh = p.get("shared")
        if sh:
            self.shared = GatedMLP({"hidden_size": self.d, "intermediate_size": int(sh["size"]), "activation": "silu",
                                    "gate_name": p["gate_name"], "up_name": p["up_name"], "down_name": p["down_name"]}, runtime)

    def _expert(self, e: int, which: str) -> str:
        return f"{self.params['expert_prefix']}{e}.{self.params[which]}"

    def weight_specs(self):
        p = self.params
        specs = {p["router_name"]: WeightSpec((self.n_out, self.d))}
        if p.get("correction_name"):
            specs[p["correction_name"]] = WeightSpec((self.n_out,), init="normal")
        for e in range(self.E):
            specs[self._expert(e, "gate_name")] = WeightSpec((self.F, self.d))
            specs[self._expert(e, "up_name")] = WeightSpec((self.F, self.d))
            specs[self._expert(e, "down_name")] = WeightSpec((self.d, self.F))
        if self.shared is not None:
            sh = p["shared"]
            for rel, ws in self.shared.weight_specs().items():
                specs[f"{sh['prefix']}.{rel}"] = ws
            if sh.get("gate"):
                specs[f"{sh['prefix']}.{sh['gate']}"] = WeightSpec((1, self.d))
        return specs

    def load(self, tensors):
        p = self.params
        rows = [tensors[p["router_name"]]]
        self.gate_col = None
        if self.shared is not None:
            sh = p["shared"]
            self.shared.load({rel: tensors[f"{sh['prefix']}.{rel}"] for rel in self.shared.weight_specs()})
            if sh.get("gate"):
                rows.append(tensors[f"{sh['prefix']}.{sh['gate']}"])
                self.gate_col = self.n_out
        # the router and the shared expert's gate as one float32 product: [experts (+ 1), hidden]
        self.w_router = _stack_rows(rows)
        self.correction = (tensors[p["correction_name"]].to(torch.float32).contiguous() if p.get("correction_name") else None)
        # [E, 2F, d]: an expert's gate rows, then its up rows (in turns of 64 where the inner width allows it: the
        # layout of the tensor-core product with the activation in its epilogue, which every kernel here reads); [E, d, F]
        gates, ups = [tensors[self._expert(e, "gate_name")] for e in range(self.E)], [tensors[self._expert(e, "up_name")] for e in range(self.E)]
        self.interleaved = self.F % 64 == 0
        self.w_gate_up = torch.stack([ops.interleave_gate_up(g, u) if self.interleaved else torch.cat([g, u])
                                      for g, u in zip(gates, ups)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert(e, "down_name")] for e in range(self.E)]).contiguous()

    def weight_bytes(self):
        """What a decode step of one token reads: the router, `top` experts, the shared expert."""
        return self.weight_bytes_for(1)

    def weight_bytes_for(self, tokens: int) -> int:
        """What a decode step of `tokens` tokens reads at most: each token's `top` experts, all different until all
        experts are in use."""
        per = (self.w_gate_up.numel() + self.w_down.numel()) // self.E * self.w_down.element_size()
        return (self.w_router.numel() * self.w_router.element_size() + min(self.E, tokens * self.top) * per
                + (self.shared.weight_bytes() if self.shared is not None else 0))

    def forward(self, h, step, add=None, out_scale: float = 1.0, into=None):
        if hasattr(h, "materialize"):
            h = h.materialize()
        T = h.shape[0]
        logits = ops.router_logits(h, self.w_router)
        ids, weights, gate = ops.route_topk(logits, self.n_out, self.top, self.correction, self.n_groups, self.keep,
                                            float(self.params["route_scale"]), self.gate_col, scores=self.scores,
                                            group_score=self.group_score, normalize=self.normalize)
        skip = self.identity
        if self.interleaved and T * self.top >= 64 * self.E and ops.moe_tc_supported(h, self.w_gate_up, self.w_down):
            # many pairs an expert (prompts): tiles of 128 rows on tcgen05, the tokens' rows laid out in sorted order first
            pairs = ops.moe_align(ids, self.E, 128, skip)
            act = ops.moe_gate_up_tc(ops.moe_gather(h, pairs), self.w_gate_up, pairs)
            y = ops.moe_down_tc(act, self.w_down, pairs)
        else:
            # few pairs an expert (decode steps): small tiles, so that a tile's padding costs little; bfloat16 on
            # mma.sync, float32 on the CUDA cores (which take tiles of 64 rows where experts have many)
            bm = 16 if (h.dtype == torch.bfloat16 or T * self.top <= 16 * self.E) else 64
            pairs = ops.moe_align(ids, self.E, bm, skip)
            act = ops.moe_gate_up(h, self.w_gate_up, pairs, interleaved=self.interleaved)
            y = ops.moe_down(act, self.w_down, pairs)
        shared = None
        if self.shared is not None:
            shared = self.shared.forward(h, step)
            shared = shared.compute() if hasattr(shared, "compute") else shared
        return ops.moe_combine(y, pairs, weights, shared, gate, ident=h if skip else None, add=add, out_scale=out_scale,
                               into=into)
