"""Tebasun as a layout of parts: every layer is a `pre_norm` arrangement whose norms compute no statistics (`dyt`),
around one of two mixers (`rglru`, or `parallel`: attention with a sink beside a gated delta rule), an optional
dense feed-forward with SiLU, and a last step that adds a gated input from the token itself through an RMS norm.
A range of layers runs several times in a row with the same weights: the schedule names those layers once per
pass (each run of the schedule has its own cache and state), and every pass starts with a `run_input`.
This file only fills `PartSpec`s from `TebasunConfig` and names the tensors (`l<i>.norm1`, `l<i>.mix.*`,
`l<i>.mlp.*`, `l<i>.side.*`, `embed`, `side.embed`, `loop.step`, `final.norm`); the parts know nothing of the design.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec
from ..config.tebasun import ARCHITECTURE, TebasunConfig
from ..parts.block import pre_norm_layer

RGLRU_RATE = 8.0                 # the constant of the diagonal recurrence's decay
UNIT_NORM_EPS = 1e-6             # inside the root where the delta rule's queries and keys are made unit vectors


def _attention_spec(cfg: TebasunConfig, m) -> PartSpec:
    position = PartSpec("none")
    rot = m["rot"]
    if rot is not None:
        scaling = None
        if rot["scaling"] is not None:
            scaling = dict(rot["scaling"], rope_type="yarn")
        position = PartSpec("rope", {"head_dim": m["dim"], "rotary_dim": rot["dims"], "theta": rot["base"],
                                     "scaling": scaling, "pairing": "half", "max_positions": 1 << 30})
    return PartSpec("attention", {
        "hidden_size": cfg.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "value_dim": m["vdim"], "scale": m["scale"], "window": None, "position": position, "bias": True,
        "bias_suffix": ".b", "qk_norm": {"eps": cfg.norm_eps, "q_name": "q.norm", "k_name": "k.norm", "per_head": True},
        "values_from_keys": True, "sink_name": "sink", "q_name": "q", "k_name": "k", "v_name": None, "o_name": "o"},
        prefix="left")


def _mixer_spec(cfg: TebasunConfig, layer) -> PartSpec:
    m, d = layer.mixer, cfg.width
    if layer.type == "rglru":
        return PartSpec("rglru", {"hidden_size": d, "width": m["width"], "blocks": m["blocks"], "conv": m["conv"],
                                  "rate": RGLRU_RATE}, prefix="mix")
    if layer.type == "parallel":
        r = m["right"]
        right = PartSpec("gated_delta", {
            "hidden_size": d, "heads": r["heads"], "kv_heads": r["kv_heads"], "dim": r["dim"], "vdim": r["vdim"],
            "conv": r["conv"], "rank": r.get("rank"), "eps": cfg.norm_eps, "l2_eps": UNIT_NORM_EPS}, prefix="right")
        return PartSpec("parallel", {"left": _attention_spec(cfg, m["left"]), "right": right,
                                     "left_scale": m["left_scale"], "right_scale": m["right_scale"]}, prefix="mix")
    raise ValueError(f"no mixer of type {layer.type!r}")


def tebasun_spec(cfg: TebasunConfig) -> ModelSpec:
    d, n = cfg.width, len(cfg.layers)

    def norm(name):
        return PartSpec("dyt", {"size": d, "name": ""}, prefix=name)

    layers, ignored = [], []
    for i, layer in enumerate(cfg.layers):
        ff = None
        if layer.mlp is not None:
            ff = PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": layer.mlp["ff"], "activation": "silu",
                                        "gate_name": "gate", "up_name": "up", "down_name": "down"}, prefix="mlp")
        else:
            ignored.append(rf"^l{i}\.norm2(\.b|\.alpha)?$")          # a layer that only mixes has no use for them
        side = side_norm = None
        if cfg.side_dim is not None:
            side = PartSpec("gated_token_rows", {
                "hidden_size": d, "dim": cfg.side_dim, "vocab_size": cfg.vocab, "table_columns": n * cfg.side_dim,
                "first_column": i * cfg.side_dim, "table_name": "/side.embed", "gate_name": "gate", "proj_name": "proj"},
                prefix="side")
            side_norm = PartSpec("rmsnorm", {"size": d, "eps": cfg.norm_eps, "name": "norm"}, prefix="side")
        layers.append(pre_norm_layer(prefix=f"l{i}", mixer=_mixer_spec(cfg, layer), feed_forward=ff,
                                     mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ff else None,
                                     token_input=side, token_input_norm=side_norm))
    schedule, run_input, run_input_at = list(range(n)), None, []
    if cfg.loop is not None:
        start, stop, times = cfg.loop
        schedule = list(range(start))
        for t in range(times):
            # every pass starts with its own entry of the table; every pass but the first also with the embedding's output
            run_input_at.append((len(schedule), t, t > 0))
            schedule += list(range(start, stop))
        schedule += list(range(stop, n))
        run_input = PartSpec("step_vector", {"hidden_size": d, "entries": times, "name": "step"}, prefix="loop")
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed",
                                               "scale": cfg.embedding_scale}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=PartSpec("dyt", {"size": d, "name": "norm"}, prefix="final"),
        lm_head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": d, "name": "embed"}),
        max_positions=1 << 30,
        ignored_tensors=tuple(ignored),
        run_input=run_input, run_input_at=tuple(run_input_at),
    )


register_architecture(ARCHITECTURE, TebasunConfig.from_dict, tebasun_spec)
