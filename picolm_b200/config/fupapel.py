"""Typed configuration of the Fupapel design: a decoder whose layers are listed one by one in config.json, each with
one of three attention mixers and a routed feed-forward (or none), both reading the same x through norms of their
own; the mixer's input is shifted towards the token before.

config.json keys: `architecture` ("Fupapel"), `vocab`, `width`, `norm.eps`, `residual_mult`, and `layers`: a list of
`{"type", "mixer": {...}, "mlp": null | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "identity"?,
"groups"?: {"count", "keep"}}}}` with
  attention         mixer {heads, kv_heads, dim, vdim, scale, mask?: {size}, rot?: {base, dims, scaling?}}
  attention_2       the same and conv (taps), kv_from? (the layer whose keys and values it uses)
  latent_attention  mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot: {base, dims}, mask?: {size}}
`rot.scaling` is {factor, low, high, original}.  Every size and constant is read from there, per layer; nothing is
assumed equal between layers.  A mixer without `mask` sees every earlier key, one without `rot` rotates nothing.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .llama import ConfigError

ARCHITECTURE = "Fupapel"
MIXER_TYPES = ("attention", "attention_2", "latent_attention")
MLP_KINDS = ("moe",)


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


def _read_rot(rot, where: str, limit: int) -> Optional[Dict[str, Any]]:
    if rot is None:
        return None
    dims = int(_need(rot, "dims", where))
    if dims < 0 or dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.dims must be even and at most {limit}")
    out: Dict[str, Any] = {"base": _positive(_need(rot, "base", where), f"{where}.base", float), "dims": dims, "scaling": None}
    if rot.get("scaling") is not None:
        sc = rot["scaling"]
        out["scaling"] = {k: _positive(_need(sc, k, where + ".scaling"), f"{where}.scaling.{k}", float)
                          for k in ("factor", "low", "high", "original")}
        if out["scaling"]["high"] == out["scaling"]["low"]:
            raise ConfigError(f"config.json: {where}.scaling.high must differ from low")
    return out


def _read_mask(m, where: str) -> Optional[int]:
    if m.get("mask") is None:
        return None
    return _positive(_need(m["mask"], "size", where + ".mask"), f"{where}.mask.size")


def _read_attention(m, where: str, second: bool) -> Dict[str, Any]:
    out: Dict[str, Any] = {k: _positive(_need(m, k, where), f"{where}.{k}") for k in ("heads", "kv_heads", "dim", "vdim")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is not a multiple of kv_heads")
    out["scale"] = _number(_need(m, "scale", where), f"{where}.scale")
    out["mask_size"] = _read_mask(m, where)
    out["rot"] = _read_rot(m.get("rot"), where + ".rot", out["dim"])
    out["conv"] = out["kv_from"] = None
    if second:
        out["conv"] = _positive(_need(m, "conv", where), f"{where}.conv")
        out["kv_from"] = None if m.get("kv_from") is None else int(m["kv_from"])
    return out


def _read_latent(m, where: str) -> Dict[str, Any]:
    out: Dict[str, Any] = {k: _positive(_need(m, k, where), f"{where}.{k}")
                           for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")}
    out["scale"] = _number(_need(m, "scale", where), f"{where}.scale")
    out["mask_size"] = _read_mask(m, where)
    out["rot"] = _read_rot(_need(m, "rot", where), where + ".rot", out["rot_dim"])
    if out["rot"]["dims"] != out["rot_dim"]:
        raise ConfigError(f"config.json: {where}.rot.dims must equal rot_dim: the rotated part is rotated whole")
    return out


def _read_mlp(mlp, where: str) -> Optional[Dict[str, Any]]:
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}.kind={kind!r} is not known ({', '.join(MLP_KINDS)})")
    r = _need(mlp, "router", where)
    router: Dict[str, Any] = {"experts": _positive(_need(r, "experts", where + ".router"), f"{where}.router.experts"),
                              "top": _positive(_need(r, "top", where + ".router"), f"{where}.router.top"),
                              "identity": int(r.get("identity") or 0), "groups": None}
    if router["identity"] < 0:
        raise ConfigError(f"config.json: {where}.router.identity must not be negative")
    n_out = router["experts"] + router["identity"]
    if router["top"] > n_out:
        raise ConfigError(f"config.json: {where}.router.top exceeds the number of experts")
    if r.get("groups") is not None:
        g = r["groups"]
        count = _positive(_need(g, "count", where + ".router.groups"), f"{where}.router.groups.count")
        keep = _positive(_need(g, "keep", where + ".router.groups"), f"{where}.router.groups.keep")
        if n_out % count or keep > count:
            raise ConfigError(f"config.json: {where}.router.groups: the router's {n_out} outputs do not form {count} equal "
                              f"groups of which {keep} are kept")
        if router["top"] > keep * (n_out // count):
            raise ConfigError(f"config.json: {where}.router: the kept groups hold fewer experts than 'top'")
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "router": router,
            "expert": {"ff": _positive(_need(_need(mlp, "expert", where), "ff", where + ".expert"), f"{where}.expert.ff")}}


@dataclass(frozen=True)
class FupapelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]

    def to_dict(self) -> Dict[str, Any]:
        m = self.mixer
        keys = ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale") if self.type == "latent_attention" \
            else ("heads", "kv_heads", "dim", "vdim", "scale")
        mixer: Dict[str, Any] = {k: m[k] for k in keys}
        if m["mask_size"] is not None:
            mixer["mask"] = {"size": m["mask_size"]}
        if m["rot"] is not None:
            mixer["rot"] = {"base": m["rot"]["base"], "dims": m["rot"]["dims"]}
            if m["rot"]["scaling"] is not None:
                mixer["rot"]["scaling"] = dict(m["rot"]["scaling"])
        if m.get("conv") is not None:
            mixer["conv"] = m["conv"]
        if m.get("kv_from") is not None:
            mixer["kv_from"] = m["kv_from"]
        mlp = _plain(self.mlp)
        if mlp is not None:
            router = {k: v for k, v in mlp["router"].items() if not (k == "groups" and v is None)}
            mlp = {"kind": mlp["kind"], "expert": mlp["expert"], "router": router}
        return {"type": self.type, "mixer": mixer, "mlp": mlp}


@dataclass(frozen=True)
class FupapelConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[FupapelLayer, ...]
    architecture: str = ARCHITECTURE

    @staticmethod
    def from_dict(raw: Mapping[str, Any]) -> "FupapelConfig":
        vocab = _positive(_need(raw, "vocab", "the model"), "'vocab'")
        width = _positive(_need(raw, "width", "the model"), "'width'")
        eps = _number(_need(_need(raw, "norm", "the model"), "eps", "norm"), "'norm.eps'")
        if eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        mult = _number(raw.get("residual_mult", 1.0), "'residual_mult'")          # (absent: the sum is added as it is)
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
            if kind == "latent_attention":
                mixer = _read_latent(m, where + ".mixer")
            else:
                mixer = _read_attention(m, where + ".mixer", second=kind == "attention_2")
            layers.append(FupapelLayer(kind, mixer, _read_mlp(e.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(layers):
            j = layer.mixer.get("kv_from")
            if j is None:
                continue
            if not 0 <= j < i or layers[j].type != "attention_2" or layers[j].mixer["kv_from"] is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from={j} does not name an earlier layer of its kind "
                                  f"with keys and values of its own")
            a, b = layer.mixer, layers[j].mixer
            for key in ("kv_heads", "dim", "vdim"):           # what the cache's rows are made of
                if a[key] != b[key]:
                    raise ConfigError(f"config.json: layers[{i}] uses the keys and values of layers[{j}] but its {key} differs")
        return FupapelConfig(vocab, width, eps, mult, tuple(layers))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "layers": [layer.to_dict() for layer in self.layers]}

    def replace(self, **kw) -> "FupapelConfig":
        return dataclasses.replace(self, **kw)
