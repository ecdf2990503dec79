"""Throughput of another design (Potuzen, Kunulorn, Tebasun, Fupapel) beside the Llama decoder (Tebasun: beside Potuzen, the
other design whose layers are recurrences and attention in turn; Fupapel: beside Kunulorn, the other design of chunked
attention and routed feed-forwards) at equal layer sizes (random weights): prefill
tokens/s of one prompt and decode tokens/s of a batch, at a few sizes that resemble a real model's layers,
and, with `kernels=True`, the device time of every kind of launch with the fraction of the memory's or the
tensor cores' measured rate that it reaches.  `bench.py --design potuzen|kunulorn|tebasun|fupapel` calls this."""
from __future__ import annotations

import json
import os
import statistics
import sys
import tempfile
import time

# name -> (width, feed-forward, layers, vocabulary, the Llama twin's (heads, kv heads, head size))
SIZES = {
    "w2048": (2048, 8192, 8, 32000, (32, 8, 64)),
    "w4096": (4096, 14336, 4, 32000, (32, 8, 128)),
}


def potuzen_config(width: int, ff: int, layers: int, vocab: int) -> dict:
    """Layers in turn: latent attention behind a window, a state-space mixer, two of gated linear attention."""
    latent = {"type": "latent_attention",
              "mixer": {"heads": width // 128, "dim": 128, "vdim": 128, "kv_rank": 256, "q_rank": width // 2,
                        "scale": 128 ** -0.5, "mask": {"size": 4096}}}
    mamba = {"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8, "conv": 4,
                                         "norm_groups": 8}}
    gla = {"type": "gla", "mixer": {"heads": width // 256, "dim": 128, "vdim": 256, "tau": 16.0, "decay_rank": 16}}
    turn = [latent, mamba, gla, gla]
    mlp = {"kind": "dense", "ff": ff}
    return {"architecture": "Potuzen", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "layers": [dict(turn[i % 4], mlp=mlp) for i in range(layers)]}


def kunulorn_config(width: int, ff: int, layers: int, vocab: int, heads) -> dict:
    """Attention with the Llama twin's head counts under chunks of 8,192 positions; feed-forwards in turn dense (the
    twin's width) and routed (experts a quarter as wide: three chosen of 32, or of 16 at the larger size, and one
    shared, so that a token's arithmetic equals the dense layer's); the last quarter of the layers reads the keys and
    values of the layer two before."""
    H, G, hd = heads
    experts = 32 if width <= 2048 else 16
    out = []
    for i in range(layers):
        m = {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "mask": {"size": 8192},
             "rot": {"base": 500000.0, "dims": hd}}
        if i >= layers - max(1, layers // 4):
            m["kv_from"] = i - 2
        mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
        if i % 2:
            mlp = {"kind": "moe", "expert": {"ff": ff // 4}, "shared": {"ff": ff // 4},
                   "router": {"experts": experts, "top": 3, "scale": 2.5, "groups": {"count": 4, "keep": 2}}}
        out.append({"type": "attention", "mixer": m, "mlp": mlp})
    return {"architecture": "Kunulorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(width) ** 0.5}, "layers": out}


def tebasun_config(width: int, ff: int, layers: int, vocab: int) -> dict:
    """`layers` runs of the schedule: a gated diagonal recurrence as wide as the model first and last, and between
    them layers of attention (heads of 128, a sink, half of each head rotated with stretched frequencies) beside a
    gated delta rule (heads of 128 x 128); a dense feed-forward in every layer; the second and third layer (the second alone of fewer than six) run twice."""
    rglru = {"type": "rglru", "mixer": {"width": width, "blocks": width // 256, "conv": 4}, "mlp": {"kind": "dense", "ff": ff}}
    left = {"heads": width // 128, "kv_heads": width // 512, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "rot": {"base": 500000.0, "dims": 64, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    right = {"heads": width // 256, "kv_heads": width // 512, "dim": 128, "vdim": 128, "conv": 4, "rank": 16}
    parallel = {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.5},
                "mlp": {"kind": "dense", "ff": ff}}
    looped = 2 if layers >= 6 else 1                           # these layers are counted twice
    n = layers - looped
    return {"architecture": "Tebasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
            "token_side": {"dim": 64}, "loop": {"start": 1, "stop": 1 + looped, "times": 2},
            "layers": [rglru if i in (0, n - 1) else parallel for i in range(n)]}


def fupapel_config(width: int, ff: int, layers: int, vocab: int, heads) -> dict:
    """Layers in turn: gated attention with the twin's head counts (half of each head rotated), attention behind short
    convolutions (whole heads rotated with stretched frequencies), attention through a latent (a row of 192 + 64 a
    position), and a convolved layer that reads the keys and values of the one two before; chunks of 8,192 positions;
    every layer routes to 4 of 30 experts (14 at the larger size) and 2 identity experts, the experts a quarter of
    the dense width, so that a token's arithmetic is at most a dense layer's."""
    H, G, hd = heads
    n_out = 32 if width <= 2048 else 16
    mlp = {"kind": "moe", "expert": {"ff": ff // 4},
           "router": {"experts": n_out - 2, "identity": 2, "top": 4, "groups": {"count": 4, "keep": 2}}}
    gated = {"type": "attention", "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                                            "mask": {"size": 8192}, "rot": {"base": 500000.0, "dims": hd // 2}}}
    conv = {"type": "attention_2", "mixer": {"heads": H, "kv_heads": G, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "conv": 4,
                                             "mask": {"size": 8192},
                                             "rot": {"base": 500000.0, "dims": hd, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0,
                                                                                             "original": 8192}}}}
    latent = {"type": "latent_attention", "mixer": {"heads": width // 128, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 192,
                                                    "q_rank": width // 2, "scale": 128 ** -0.5, "rot": {"base": 10000.0, "dims": 64}}}
    out = []
    for i in range(layers):
        layer = json.loads(json.dumps([gated, conv, latent, conv][i % 4]))
        if i % 4 == 3:
            layer["mixer"]["kv_from"] = i - 2
        layer["mlp"] = mlp
        out.append(layer)
    return {"architecture": "Fupapel", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": out}


def llama_config(width: int, ff: int, layers: int, vocab: int, heads) -> dict:
    H, G, hd = heads
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": layers, "hidden_size": width,
            "num_attention_heads": H, "num_key_value_heads": G, "head_dim": hd, "intermediate_size": ff, "vocab_size": vocab,
            "rope_theta": 500000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "max_position_embeddings": 8192,
            "tie_word_embeddings": False, "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2}


def _measure(cfg_dict: dict, prompt_tokens: int, batch: int, steps: int, warmup: int, kernels: bool) -> dict:
    import torch
    from picolm_b200 import ops
    from picolm_b200.config import config_from_dict
    from picolm_b200.engine import Engine
    from picolm_b200.weights import write_random_model
    cfg = config_from_dict(cfg_dict)
    vocab = cfg_dict.get("vocab", cfg_dict.get("vocab_size"))
    g = torch.Generator().manual_seed(1)
    with tempfile.TemporaryDirectory() as tmp:
        write_random_model(cfg, 1, tmp, norm_std=0.0)
        per_seq = (max(prompt_tokens, 512) + steps + 2 * warmup + 80) // 64 * 64 + 64
        engine = Engine.from_folder(tmp, dtype="bfloat16", max_tokens=(batch + 1) * per_seq, max_seqs=batch + 1)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def prompt(n):
        return torch.randint(0, vocab, (n,), generator=g).tolist()

    times = []
    for i in range(warmup + 8):
        s = engine.new_sequence()
        p = prompt(prompt_tokens)
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        engine.step([(s, p)])
        b.record()
        torch.cuda.synchronize()
        engine.end_sequence(s)
        if i >= warmup:
            times.append(a.elapsed_time(b))
        elif kernels and i == warmup - 1:
            ops.trace_report(file=open(os.devnull, "w"))       # what a kernel's first launches cost is not its time
    out = {"prefill_tokens_per_s": round(prompt_tokens / statistics.median(times) * 1e3, 1),
           "prefill_ms": round(statistics.median(times), 3)}
    if kernels:
        out["prefill_kernels"] = _table(ops.trace_report(file=open(os.devnull, "w")))
    slots = [engine.new_sequence() for _ in range(batch)]
    engine.step([(s, prompt(512)) for s in slots])
    toks = [[int(t)] for t in torch.randint(0, vocab, (batch,), generator=g)]
    for _ in range(warmup):
        engine.step([(s, t) for s, t in zip(slots, toks)])
    if kernels:
        ops.trace_report(file=open(os.devnull, "w"))
    a, b = ev(), ev()
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        engine.step([(s, t) for s, t in zip(slots, toks)])
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    out.update(decode_tokens_per_s=round(batch / ms * 1e3, 1), decode_ms_per_step=round(ms, 4), decode_batch=batch,
               decode_from_graph=bool(engine._graphs), weight_gb=round(engine.model.weight_bytes_per_step(batch) / 1e9, 3))
    # (a routed feed-forward counts min(experts, batch x top) experts a layer: what the batch reads at most)
    out["decode_hbm_frac"] = round(engine.model.weight_bytes_per_step(batch) / (ms * 1e-3) / (ops._lib.PEAK_GBS * 1e9), 3)
    if kernels:
        out["decode_kernels"] = _table(ops.trace_report(file=open(os.devnull, "w")))
    for s in slots:
        engine.end_sequence(s)
    return out


def _table(rows, top=14):
    """The rows of `ops.trace_report` as dictionaries: share of the time, and the larger of the two roofline fractions."""
    from picolm_b200.ops import _lib
    total = sum(r[1] for _, r in rows) or 1.0
    out = []
    for what, (n, ms, nbytes, flops) in rows[:top]:
        gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
        tf = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        out.append({"launch": what, "count": n, "ms": round(ms, 3), "share": round(ms / total, 3),
                    "hbm_frac": round(gbs / _lib.PEAK_GBS, 3), "tensor_frac": round(tf / _lib.PEAK_TFLOPS, 3)})
    return out


def run(design: str, sizes, prompt_tokens: int, batch: int, steps: int, warmup: int, kernels: bool) -> dict:
    if design not in ("potuzen", "kunulorn", "tebasun", "fupapel"):
        raise ValueError(f"no design {design!r} to compare (known: potuzen, kunulorn, tebasun, fupapel)")
    beside = {"tebasun": "potuzen", "fupapel": "kunulorn"}.get(design, "llama")
    result = {"design": design, "beside": {"potuzen": "Potuzen", "kunulorn": "Kunulorn"}.get(beside, "LlamaForCausalLM"), "dtype": "bf16",
              "data": "synthetic (random weights and tokens)",
              "prompt_tokens": prompt_tokens, "decode_batch": batch, "steps": steps, "warmup": warmup, "sizes": {}}
    for name in sizes:
        width, ff, layers, vocab, heads = SIZES[name]
        t0 = time.time()
        config = {"potuzen": lambda: potuzen_config(width, ff, layers, vocab),
                  "kunulorn": lambda: kunulorn_config(width, ff, layers, vocab, heads),
                  "tebasun": lambda: tebasun_config(width, ff, layers, vocab),
                  "fupapel": lambda: fupapel_config(width, ff, layers, vocab, heads)}[design]()
        ours = _measure(config, prompt_tokens, batch, steps, warmup, kernels)
        twin_config = {"potuzen": lambda: potuzen_config(width, ff, layers, vocab),
                       "kunulorn": lambda: kunulorn_config(width, ff, layers, vocab, heads),
                       "llama": lambda: llama_config(width, ff, layers, vocab, heads)}[beside]()
        twin = _measure(twin_config, prompt_tokens, batch, steps, warmup, kernels)
        result["sizes"][name] = {
            "width": width, "ff": ff, "layers": layers, design: ours, beside: twin,
            "prefill_ratio": round(ours["prefill_tokens_per_s"] / twin["prefill_tokens_per_s"], 3),
            "decode_ratio": round(ours["decode_tokens_per_s"] / twin["decode_tokens_per_s"], 3)}
        print(f"[bench] {name}: {time.time() - t0:.0f} s", file=sys.stderr)
    return result


def main(args) -> int:
    from picolm_b200.ops import _lib
    if args.design_kernels and not _lib.TRACED:
        print("the per-launch table needs PICOLM_B200_TRACE=1 in the environment before the package is imported")
        return 2
    sizes = [s for s in args.design_sizes.split(",") if s]
    for s in sizes:
        if s not in SIZES:
            print(f"unknown size {s!r}; known: {', '.join(SIZES)}")
            return 2
    result = run(args.design, sizes, args.design_prompt, args.batch, min(args.steps, 64), max(args.warmup, 3),
                 args.design_kernels)
    print(json.dumps(result))
    return 0
