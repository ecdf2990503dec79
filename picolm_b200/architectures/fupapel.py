"""Fupapel as a layout of parts: every layer is a `parallel_norm` arrangement (mixer and feed-forward side by side
behind RMS norms of their own whose weights are stored around zero, the sum of both times one constant) with a
`token_shift` in front of the mixer, one of three mixers, and a `routed_mlp` or no feed-forward.  This file only fills
`PartSpec`s from `FupapelConfig` and names the tensors (`l<i>.norm1`, `l<i>.norm2`, `l<i>.shift`, `l<i>.mix.*`,
`l<i>.mlp.*`, `embed`, `final.norm`, `head`); the parts know nothing of the design.

The mixers: `attention` is the library's attention part with a norm over the whole of q and of k, a rotation in
half-split pairs, a mask of chunks, a sink of score 0 and a sigmoid gate on the heads; `attention_2` the same part
with short convolutions behind the projections, the three-band frequency rule, a factor per head on the scores and
a learned sink, and with `kv_from: j` the keys and values of layer j (`LayerSpec.cache_of`; the convolution's tail
and the shift's row stay the layer's own); `latent_attention` the latent part with a rotated part beside the
latent, a learned sink and a gate per head.  The feed-forward routes by softmax scores over experts and identity
experts together, groups by their best choice score, and does not renormalise the weights.

Constants the design fixes: the sink of score 0; experts' tensors `e<k>.*`.
"""
from __future__ import annotations

from ..config.fupapel import ARCHITECTURE, FupapelConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec
from ..parts.block import parallel_norm_layer

ZERO_SINK = 0.0                  # `attention`: one more exp(0) in every head's denominator


def _rope(rot, head_dim: int) -> PartSpec:
    if rot is None or rot["dims"] == 0:
        return PartSpec("none")
    scaling = None
    if rot["scaling"] is not None:
        sc = rot["scaling"]
        scaling = {"rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
                   "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]}
    return PartSpec("rope", {"head_dim": head_dim, "rotary_dim": rot["dims"], "theta": rot["base"], "scaling": scaling,
                             "pairing": "half", "max_positions": 1 << 30})


def _mixer_spec(cfg: FupapelConfig, layer) -> PartSpec:
    m, d = layer.mixer, cfg.width
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": d, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
            "q_rank": m["q_rank"], "scale": m["scale"], "window": None, "chunk": m["mask_size"], "eps": cfg.norm_eps,
            "rot_dim": m["rot_dim"],
            "position": _rope(m["rot"], m["rot_dim"]), "sink_name": "sink", "gate_per_head": True}, prefix="mix")
    params = {
        "hidden_size": d, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "scale": m["scale"], "window": None, "chunk": m["mask_size"],
        "position": _rope(m["rot"], m["dim"]),
        "qk_norm": {"eps": cfg.norm_eps, "q_name": "q.norm", "k_name": "k.norm"},
        "q_name": "q", "k_name": "k", "v_name": "v", "o_name": "o"}
    if layer.type == "attention":
        params.update({"sink_value": ZERO_SINK, "gate_name": "g"})
    else:
        params.update({"sink_name": "sink", "head_scale_name": "temp", "conv": {"taps": m["conv"], "suffix": ".conv"},
                       "own_kv": m["kv_from"] is None})
    return PartSpec("attention", params, prefix="mix")


def _mlp_spec(cfg: FupapelConfig, mlp) -> PartSpec:
    r = mlp["router"]
    return PartSpec("routed_mlp", {
        "hidden_size": cfg.width, "experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"],
        "route_scale": 1.0, "groups": r.get("groups"), "correction_name": "correction", "router_name": "router",
        "expert_prefix": "e", "shared": None, "gate_name": "gate", "up_name": "up", "down_name": "down",
        "scores": "softmax", "group_score": "max", "normalize": False, "identity": r["identity"]}, prefix="mlp")


def fupapel_spec(cfg: FupapelConfig) -> ModelSpec:
    d = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"size": d, "eps": cfg.norm_eps, "name": "", "one_plus": True}, prefix=name)

    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        ff = _mlp_spec(cfg, layer.mlp) if layer.mlp is not None else None
        if ff is None:
            ignored.append(rf"^l{i}\.norm2$")                       # a layer that only mixes has no use for it
        layers.append(parallel_norm_layer(
            prefix=f"l{i}", mixer=_mixer_spec(cfg, layer), mixer_norm=norm("norm1"), feed_forward=ff,
            feed_forward_norm=norm("norm2") if ff is not None else None,
            mixer_filter=PartSpec("token_shift", {"size": d, "name": ""}, prefix="shift"),
            residual_scale=cfg.residual_mult, cache_of=layer.mixer.get("kv_from")))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed"}),
        layers=tuple(layers), schedule=tuple(range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": d, "eps": cfg.norm_eps, "name": "norm", "one_plus": True}, prefix="final"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "head"}),
        max_positions=1 << 20,
        ignored_tensors=tuple(ignored),
    )


register_architecture(ARCHITECTURE, FupapelConfig.from_dict, fupapel_spec)
