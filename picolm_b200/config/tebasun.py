"""Typed configuration of the Tebasun design: a decoder whose layers are listed one by one in config.json, each
with one of two mixers (`rglru`: a gated diagonal linear recurrence behind a short convolution; `parallel`: softmax
attention with a sink beside a gated delta rule, their results added with two constants), an optional dense
feed-forward, a norm without statistics, a per-layer input from the token itself, and a range of layers that runs
several times in a row with the same weights.

config.json keys: `architecture` ("Tebasun"), `vocab`, `width`, `norm.eps`, `embedding.scale`,
`token_side.dim` (optional: no per-layer token input without it), `loop: {start, stop, times}` (optional), and
`layers`: a list of `{"type", "mixer": {...}, "mlp": null | {"kind": "dense", "ff"}}` with
  rglru     mixer {width, blocks, conv}
  parallel  mixer {left: {heads, kv_heads, dim, vdim, scale, rot?: {base, dims, scaling?: {factor, original, fast,
            slow}}}, right: {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale}
Every size and constant is read from there, per layer; nothing is assumed equal between layers.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .llama import ConfigError

ARCHITECTURE = "Tebasun"
MIXER_TYPES = ("rglru", "parallel")
MLP_KINDS = ("dense",)


def _need(d, key: str, where: str):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks the key {key!r}")
    return d[key]


def _positive(v, what: str, kind=int):
    try:
        out = kind(v)
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: {what} must be a number, not {v!r}") from None
    if not out > 0:
        raise ConfigError(f"config.json: {what} must be positive")
    return out


def _number(v, what: str) -> float:
    try:
        return float(v)
    except (TypeError, ValueError):
        raise ConfigError(f"config.json: {what} must be a number, not {v!r}") from None


def _plain(v):
    if isinstance(v, Mapping):
        return {k: _plain(x) for k, x in v.items()}
    return v


def _read_rot(rot, where: str) -> Optional[Dict[str, Any]]:
    if rot is None:
        return None
    dims = int(_need(rot, "dims", where))
    if dims == 0:
        return None
    out: Dict[str, Any] = {"base": _positive(_need(rot, "base", where), f"{where}.base", float), "dims": dims, "scaling": None}
    sc = rot.get("scaling")
    if sc is not None:
        out["scaling"] = {k: _positive(_need(sc, k, f"{where}.scaling"), f"{where}.scaling.{k}", float)
                          for k in ("factor", "original", "fast", "slow")}
    return out


def _read_left(m, where: str) -> Dict[str, Any]:
    out = {k: _positive(_need(m, k, where), f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim")}
    out["scale"] = _positive(_need(m, "scale", where), f"{where}.scale", float)
    out["rot"] = _read_rot(m.get("rot"), f"{where}.rot")
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    if out["vdim"] != out["dim"]:
        raise ConfigError(f"config.json: {where}: the keys serve as values, so vdim must equal dim")
    r = out["rot"]
    if r is not None and (r["dims"] < 0 or r["dims"] % 2 or r["dims"] > out["dim"]):
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim")
    return out


def _read_right(m, where: str) -> Dict[str, Any]:
    out = {k: _positive(_need(m, k, where), f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    if m.get("rank") is not None:
        out["rank"] = _positive(m["rank"], f"{where}.rank")        # optional: the tensors' shapes give it otherwise
    return out


@dataclass(frozen=True)
class TebasunLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": _plain(self.mixer), "mlp": _plain(self.mlp)}


@dataclass(frozen=True)
class TebasunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    side_dim: Optional[int]                    # None: no per-layer token input
    loop: Optional[Tuple[int, int, int]]       # (start, stop, times) or None
    layers: Tuple[TebasunLayer, ...]
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "TebasunConfig":
        vocab = _positive(_need(raw, "vocab", "the model"), "vocab")
        width = _positive(_need(raw, "width", "the model"), "width")
        eps = _number(_need(_need(raw, "norm", "the model"), "eps", "norm"), "norm.eps")
        if eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        scale = _number(_need(_need(raw, "embedding", "the model"), "scale", "embedding"), "embedding.scale")
        side = raw.get("token_side")
        side_dim = None if side is None else _positive(_need(side, "dim", "token_side"), "token_side.dim")
        entries = _need(raw, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(e, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type={kind!r} is not known ({', '.join(MIXER_TYPES)})")
            m = _need(e, "mixer", where)
            if kind == "rglru":
                mixer = {k: _positive(_need(m, k, f"{where}.mixer"), f"{where}.mixer.{k}") for k in ("width", "blocks", "conv")}
                if mixer["width"] % mixer["blocks"]:
                    raise ConfigError(f"config.json: {where}.mixer.width is not a multiple of blocks")
            else:
                mixer = {"left": _read_left(_need(m, "left", f"{where}.mixer"), f"{where}.mixer.left"),
                         "right": _read_right(_need(m, "right", f"{where}.mixer"), f"{where}.mixer.right"),
                         "left_scale": _number(_need(m, "left_scale", f"{where}.mixer"), f"{where}.mixer.left_scale"),
                         "right_scale": _number(_need(m, "right_scale", f"{where}.mixer"), f"{where}.mixer.right_scale")}
            mlp = e.get("mlp")
            if mlp is not None:
                mk = _need(mlp, "kind", f"{where}.mlp")
                if mk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind={mk!r} is not known ({', '.join(MLP_KINDS)})")
                mlp = {"kind": mk, "ff": _positive(_need(mlp, "ff", f"{where}.mlp"), f"{where}.mlp.ff")}
            layers.append(TebasunLayer(kind, mixer, mlp))
        loop = raw.get("loop")
        if loop is not None:
            start, stop = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop"))
            times = _positive(_need(loop, "times", "loop"), "loop.times")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop.start={start}, loop.stop={stop} do not name a range of the {len(layers)} layers")
            loop = (start, stop, times)
        return TebasunConfig(vocab, width, eps, scale, side_dim, loop, tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                               "layers": [layer.to_dict() for layer in self.layers]}
        if self.side_dim is not None:
            out["token_side"] = {"dim": self.side_dim}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def replace(self, **kw) -> "TebasunConfig":
        return dataclasses.replace(self, **kw)
