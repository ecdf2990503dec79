"""The Tebasun design through the library, against the plain implementation in
`tests/plain/tebasun_plain.py`: each mechanism alone (kernels against plain functions, then models of one
kind of layer), prompts against token-by-token decoding, portions, batches, pages and slots used again,
far keys and page borders, the first tokens, long decoding, sizes that make special cases (one block,
one head, one tap, no rotation, a full rotation, no feed-forward, no token input, a loop from the first
layer or to the last), and greedy generation through the library's entry point.

Weights are random; where random weights would hide a fault they are reshaped: the attention's scale is
large so that the softmax is peaked (one far key, or the extra term of the denominator, then decides a row
of logits), and decays are drawn close to 1 so that the first tokens stay in a state for hundreds of steps.
"""
import json
import math
import os

import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import tebasun_plain as P
from util import random_tokens

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-4          # of the logits' spread; two float32 computations in different orders of summation
VOCAB = 97


def _rglru(width=48, blocks=3, conv=3, mlp=None):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}, "mlp": mlp}


def _rot(dims=8, base=10000.0, scaling=True):
    return {"base": base, "dims": dims,
            "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0} if scaling else None}


def _parallel(heads=4, kv_heads=2, dim=16, rot=None, scale=0.9, rheads=4, rkv=2, rdim=8, rvdim=12, conv=4,
              left_scale=0.7, right_scale=1.3, ff=56, rank=5):
    rot = _rot() if rot is None else (rot or None)
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot:
        left["rot"] = rot
    return {"type": "parallel",
            "mixer": {"left": left,
                      "right": {"heads": rheads, "kv_heads": rkv, "dim": rdim, "vdim": rvdim, "conv": conv, "rank": rank},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _config(layers, width=40, loop=None, side=6, eps=1e-5, emb_scale=1.7):
    out = {"architecture": "Tebasun", "vocab": VOCAB, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": emb_scale}, "layers": [json.loads(json.dumps(layer)) for layer in layers]}
    if side:
        out["token_side"] = {"dim": side}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


def _make(tmp_path, name, config, seed, slow=False, sink=None):
    """A model folder with random weights for `config`; returns (folder, plain tensors, config).  `slow`: the decays
    of both recurrences are drawn close to 1.  `sink`: every head's sink is this number (else drawn from N(0, 2))."""
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors, save_safetensors
    cfg = config_from_dict(config)
    tensors = random_tensors(cfg, seed, std=0.12, norm_std=0.2)
    g = torch.Generator().manual_seed(seed + 1000)
    for n in list(tensors):
        t = tensors[n]
        if n.endswith(".sink"):
            tensors[n] = (torch.full(t.shape, float(sink)) if sink is not None else 2.0 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif slow and n.endswith(".mix.lam"):
            tensors[n] = (-9.0 + 2.0 * torch.rand(t.shape, generator=g)).to(t.dtype)
        elif slow and n.endswith(".A_log"):
            tensors[n] = (-4.0 + torch.rand(t.shape, generator=g)).to(t.dtype)
    d = str(tmp_path / name)
    os.makedirs(d, exist_ok=True)
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    return d, P.read_safetensors(os.path.join(d, "model.safetensors")), cfg.to_dict()


def _plain(tensors, config, tokens, dtype=torch.float64):
    return P.forward(config, tensors, tokens, dtype).to(torch.float32)


def _close(got, want, tol=FP32_TOL, what=""):
    err = (got.double() - want.double()).abs().max().item()
    spread = want.double().std().item()
    assert err <= tol * spread, f"{what}: max |diff| {err:.3e} is {err / spread:.2e} of the logits' spread (limit {tol})"


def _engine(d, dtype="float32", max_tokens=64 * 40, **kw):
    from picolm_b200.engine import Engine
    return Engine.from_folder(d, dtype=dtype, max_tokens=max_tokens, **kw)


class _Step:
    """What the kernels read of a step, for sequences that bring `lens` tokens each."""

    def __init__(self, lens, slots, dev, starts=None):
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + n)
        i32 = dict(dtype=torch.int32, device=dev)
        self.n_seqs, self.n_tokens, self.max_new = len(lens), offs[-1], max(lens)
        self.is_decode = all(n == 1 for n in lens)
        self.seq_start = torch.tensor(offs, **i32)
        self.seq_slot = torch.tensor(slots, **i32)
        self.tok_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], **i32)
        starts = starts or [0] * len(lens)
        self.tok_pos = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], **i32)


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("d", [40, 42, 256])
def test_norm_without_statistics_kernel(d):
    """tanh(alpha v) w + b on v = x + what is pending: plain rows, rows with a bias vector, rows that pass an RMS
    norm of their own first, further rows; the sum goes back to the stream unless rows are gathered."""
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(d)
    T = 11
    x, delta, extra = (torch.randn(T, d, generator=g) * 3 for _ in range(3))
    w, b, vec, pw = (torch.randn(d, generator=g) for _ in range(4))
    alpha = torch.tensor([0.37])
    cu = lambda t: t.to(dev).contiguous()
    D = torch.float64

    def want(v):
        return P.tanh_norm(v, w.to(D), b.to(D), alpha.to(D))

    xs = cu(x)
    out = ops.dyt_norm(xs, torch.float32, alpha=cu(alpha), weight=cu(w), bias=cu(b))
    assert torch.allclose(out.cpu().double(), want(x.to(D)), atol=1e-6) and torch.equal(xs.cpu(), x)
    out = ops.dyt_norm(xs, torch.float32, alpha=cu(alpha), weight=cu(w), bias=cu(b), delta=cu(delta), delta_bias=cu(vec))
    v = x.to(D) + delta.to(D) + vec.to(D)
    assert torch.allclose(out.cpu().double(), want(v), atol=1e-5) and torch.allclose(xs.cpu().double(), v, atol=1e-5)
    xs = cu(x)
    out = ops.dyt_norm(xs, torch.bfloat16, alpha=cu(alpha), weight=cu(w), bias=cu(b), delta=cu(delta), post_weight=cu(pw),
                       post_eps=1e-3, extra=cu(extra))
    v = x.to(D) + P.rms_norm(delta.to(D), pw.to(D), 1e-3) + extra.to(D)
    assert torch.allclose(xs.cpu().double(), v, atol=1e-5)
    assert torch.allclose(out.float().cpu().double(), want(v), atol=2e-2, rtol=2e-2)
    xs = cu(x)
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32, device=dev)
    out = ops.dyt_norm(xs, torch.float32, alpha=cu(alpha), weight=cu(w), bias=cu(b), delta=cu(delta), rows=rows)
    assert torch.allclose(out.cpu().double(), want((x + delta).to(D))[rows.cpu().long()], atol=1e-5) and torch.equal(xs.cpu(), x)
    xs = cu(x)
    assert ops.dyt_norm(xs, None, delta_bias=cu(vec), extra=cu(extra)) is None
    assert torch.allclose(xs.cpu().double(), x.to(D) + vec.to(D) + extra.to(D), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,blocks", [(48, 3), (40, 1), (70, 2), (36, 36)])
def test_gated_diagonal_recurrence_kernels(dtype, W, blocks):
    """Gates and scan of the diagonal recurrence over ragged prompts, then portions and single tokens, with the state
    carried in rows of a wider buffer; decays close to 1 among the channels (the state lasts)."""
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(W + blocks)
    n = W // blocks
    total = [75, 9, 40]
    u = [torch.randn(t, W + 8, generator=g).to(dtype) for t in total]
    y = [torch.randn(t, W + 8, generator=g).to(dtype) for t in total]
    wr, wi = (torch.randn(blocks, n, n, generator=g) * 0.4).to(dtype), (torch.randn(blocks, n, n, generator=g) * 0.4).to(dtype)
    br, bi, yb = torch.randn(W, generator=g), torch.randn(W, generator=g), torch.randn(W, generator=g)
    lam = -9.0 + 9.0 * torch.rand(W, generator=g)
    rate = 8.0 * P.softplus(lam.double())
    D = torch.float64
    want = []
    for us, ys in zip(u, y):
        ub = us[:, 4:4 + W].to(D).view(-1, blocks, n)
        r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wr.to(D)).reshape(-1, W) + br.to(D))
        i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, wi.to(D)).reshape(-1, W) + bi.to(D))
        a = torch.exp(-r * rate)
        S = P.diagonal_recurrence(a, torch.sqrt(1 - a * a) * i * us[:, 4:4 + W].to(D))
        want.append(S * P.gelu_tanh(ys[:, 4:4 + W].to(D) + yb.to(D)))
    state = torch.zeros(6, W + 5, device=dev)
    slots = [4, 1, 2]
    got, at = [[] for _ in total], [0, 0, 0]
    cu = lambda t: t.to(dev).contiguous()
    for cut in ([40, 3, 30], [1, 1, 1], [2, 2, 2], [1, 1, 1], [31, 2, 6]):
        step = _Step(cut, slots, dev)
        ur = torch.cat([u[k][at[k]:at[k] + c] for k, c in enumerate(cut)]).to(dev)
        yr = torch.cat([y[k][at[k]:at[k] + c] for k, c in enumerate(cut)]).to(dev)
        log_a, x = ops.rglru_gates(ur[:, 4:4 + W], cu(wr), cu(wi), cu(br), cu(bi), cu(rate.float()), blocks)
        out = ops.diag_scan(log_a, x, yr[:, 4:4 + W], cu(yb), state[:, :W], step)
        o = 0
        for k, c in enumerate(cut):
            got[k].append(out[o:o + c].float().cpu())
            o, at[k] = o + c, at[k] + c
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for k in range(3):
        err = (torch.cat(got[k]).double() - want[k]).abs().max().item()
        assert err <= tol * max(1.0, want[k].abs().max().item()), f"sequence {k}: {err:.3e}"
    assert state[:, W:].abs().max() == 0 and state[0].abs().max() == 0 and state[3].abs().max() == 0


def test_a_decay_next_to_one_keeps_its_digits():
    """log a = -1e-5: a float32 a has lost half the digits of 1 - a, and a state that has run for 4000 tokens shows it;
    the kernels carry log a and stay at float32 rounding of the exact state."""
    from picolm_b200 import ops
    dev = "cuda:0"
    T, W = 4000, 32
    g = torch.Generator().manual_seed(5)
    log_a = torch.full((T, W), -1e-5) * (1 + torch.rand(T, W, generator=g))
    x = torch.randn(T, W, generator=g).abs()
    want = P.diagonal_recurrence(torch.exp(log_a.double()), x.double())
    state = torch.zeros(1, W, device=dev)
    zero = torch.zeros(T, W, device=dev)            # gelu_tanh(0 + 3) is the same known factor everywhere
    out = ops.diag_scan(log_a.to(dev), x.to(dev), zero, torch.full((W,), 3.0, device=dev), state, _Step([T], [0], dev))
    got = out.cpu().double() / P.gelu_tanh(torch.tensor(3.0, dtype=torch.float64))
    assert ((got - want).abs() / want).max().item() < 1e-6
    assert ((state.cpu().double()[0] - want[-1]).abs() / want[-1]).max().item() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N,Pv,H,hpg", [(8, 12, 4, 2), (32, 32, 2, 1), (5, 33, 3, 3), (20, 70, 1, 1), (130, 8, 2, 1)])
def test_delta_rule_kernels(dtype, N, Pv, H, hpg):
    """What the delta rule takes (unit q and k, decays, write strengths) and its recurrence, head by head against the
    plain loop: ragged prompts, portions, single tokens, the state carried in rows of a wider buffer."""
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(N * 7 + Pv)
    G = H // hpg
    total = [37 + 96, 6, 20 + 64]        # the first portion runs chunk by chunk (several chunks, the last ragged)
    mk = lambda t, c: torch.randn(t, c + 8, generator=g).to(dtype)
    q, k, v = [mk(t, G * N) for t in total], [mk(t, G * N) for t in total], [mk(t, H * Pv) for t in total]
    z, braw = [mk(t, H * N) for t in total], [mk(t, H) for t in total]
    a_log, dt_bias = -3.0 + 3.5 * torch.rand(H, generator=g), -4.0 + 4.0 * torch.rand(H * N, generator=g)
    D = torch.float64
    want = []
    for s in range(3):
        T = total[s]
        qq, kk = q[s][:, 4:4 + G * N].to(D).view(T, G, N), k[s][:, 4:4 + G * N].to(D).view(T, G, N)
        qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + 1e-6) * N ** -0.5
        kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
        dec = torch.exp(-torch.exp(a_log.to(D))[None, :, None]
                        * P.softplus(z[s][:, 4:4 + H * N].to(D) + dt_bias.to(D)).view(T, H, N))
        beta = torch.sigmoid(braw[s][:, 4:4 + H].to(D))
        vv = v[s][:, 4:4 + H * Pv].to(D).view(T, H, Pv)
        want.append(torch.cat([P.delta_rule(qq[:, h // hpg], kk[:, h // hpg], vv[:, h], dec[:, h], beta[:, h])
                               for h in range(H)], dim=1))
    state = torch.zeros(5, H * N * Pv + 3, device=dev)
    slots = [3, 0, 1]
    got, at = [[] for _ in total], [0, 0, 0]
    cu = lambda t: t.to(dev).contiguous()
    for cut in ([20 + 96, 2, 9 + 64], [1, 1, 1], [2, 2, 2], [1, 1, 1], [13, 0, 7]):
        live = [i for i, c in enumerate(cut) if c]
        step = _Step([cut[i] for i in live], [slots[i] for i in live], dev)
        rows = lambda src: torch.cat([src[i][at[i]:at[i] + cut[i]] for i in live]).to(dev)
        qr, kr, vr, zr, br_ = rows(q), rows(k), rows(v), rows(z), rows(braw)
        qn, kn, qk, dec, beta = ops.delta_prep(qr[:, 4:4 + G * N], kr[:, 4:4 + G * N], zr[:, 4:4 + H * N], br_[:, 4:4 + H],
                                               cu(a_log), cu(dt_bias), 1e-6, N ** -0.5, H, N, heads_per_group=hpg)
        out = ops.delta_scan(qn, kn, qk, dec, beta, vr[:, 4:4 + H * Pv], state[:, :H * N * Pv], step, H, N, Pv,
                             heads_per_group=hpg)
        o = 0
        for i in live:
            got[i].append(out[o:o + cut[i]].float().cpu())
            o, at[i] = o + cut[i], at[i] + cut[i]
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for s in range(3):
        err = (torch.cat(got[s]).double() - want[s]).abs().max().item()
        assert err <= tol * max(1.0, want[s].abs().max().item()), f"sequence {s}: {err:.3e}"
    assert state[:, H * N * Pv:].abs().max() == 0 and state[2].abs().max() == 0 and state[4].abs().max() == 0


def test_token_gate_and_scaled_sum_kernels():
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(1)
    R, dim, cols = 9, 6, 30
    for dtype, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2)):
        gate, table = torch.randn(R, dim, generator=g).to(dtype), torch.randn(VOCAB, cols, generator=g).to(dtype)
        toks = torch.randint(0, VOCAB, (R,), generator=g).to(torch.int32)
        out = ops.token_gate(gate.to(dev), table.to(dev), 12, toks.to(dev))
        want = P.gelu_tanh(gate.double()) * table.double()[toks.long(), 12:18]
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
        rows = torch.tensor([8, 2, 2], dtype=torch.int32)
        out = ops.token_gate(gate[:3].contiguous().to(dev), table.to(dev), 24, toks.to(dev), rows.to(dev))
        want = P.gelu_tanh(gate[:3].double()) * table.double()[toks.long()[rows.long()], 24:30]
        assert torch.allclose(out.cpu().double(), want, atol=tol, rtol=tol)
    a, b, vec = torch.randn(7, 40, generator=g), torch.randn(7, 40, generator=g), torch.randn(40, generator=g)
    out = ops.scaled_sum(a.to(dev), 0.7, b.to(dev), -1.3, bias_a=vec.to(dev))
    assert torch.allclose(out.cpu(), 0.7 * (a + vec) - 1.3 * b, atol=1e-6)


# ------------------------------------------------------------------------------------ models of few layers
ALONE = {
    "rglru": [_rglru(), _rglru(width=40, blocks=1, conv=1, mlp={"kind": "dense", "ff": 24})],
    "rglru_many_blocks": [_rglru(width=64, blocks=16, conv=2), _rglru(width=36, blocks=36, conv=5)],
    "parallel": [_parallel(), _parallel(heads=3, kv_heads=1, dim=24, rot=_rot(dims=24, scaling=False), rheads=2, rkv=1, rdim=12,
                                        rvdim=8, conv=2, ff=None)],
    "parallel_no_rotation": [_parallel(heads=1, kv_heads=1, dim=8, rot=False, rheads=1, rkv=1, rdim=16, rvdim=16, conv=1)],
    "parallel_equal_heads": [_parallel(heads=2, kv_heads=2, dim=32, rot=_rot(dims=4, base=50.0), rheads=3, rkv=3, rdim=20, rvdim=5)],
    "mixed": [_rglru(), _parallel(), _rglru(width=32, blocks=2, conv=4), _parallel(heads=2, kv_heads=1, dim=8, rot=_rot(dims=2))],
    # a width that is no multiple of 4 or 8: the kernels that take vectors of four and the tensor maps refuse it
    "odd_width": [_rglru(width=35, blocks=5), _parallel()],
}
LOOPS = {"rglru": None, "mixed": (1, 3, 3), "parallel": (0, 2, 2), "odd_width": (1, 2, 2)}
SIDES = {"rglru_many_blocks": None, "parallel_equal_heads": 1, "odd_width": 3}
WIDTHS = {"odd_width": 42}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_float32_model_matches_plain_in_every_cut(tmp_path, name):
    config = _config(ALONE[name], width=WIDTHS.get(name, 40), loop=LOOPS.get(name), side=SIDES.get(name, 6))
    d, tensors, config = _make(tmp_path, name, config, seed=len(name))
    eng = _engine(d)
    a, b, c = random_tokens(150, VOCAB, 1), random_tokens(67, VOCAB, 2), random_tokens(1, VOCAB, 3)
    want = {id(t): _plain(tensors, config, t) for t in (a, b, c)}
    for t in (a, b, c):
        _close(run_whole(eng, t), want[id(t)], what="whole")
    _close(run_tail(eng, a, tail=90), want[id(a)], what="prompt, then 90 single tokens")       # over a page border
    _close(run_tail(eng, b, tail=len(b)), want[id(b)], what="token by token from the first")
    for sizes in ([64, 64, 22], [3, 2, 61, 2, 2, 80], [149, 1], [2] * 33 + [1]):
        t = a if sum(sizes) == 150 else b
        _close(run_chunks(eng, t, sizes), want[id(t)], what=f"portions {sizes[:6]}")
    outs = run_batch(eng, [b, c, a], [40, 1, 129])
    for got, t in zip(outs, (b, c, a)):
        _close(got, want[id(t)], what="batch of unequal requests")
    # slots and pages that were used are used again, and give the same
    _close(run_whole(eng, a), want[id(a)], what="whole, again")
    # few rows wanted: the last layer narrows the stream after its mixer, and the token input finds the rows' tokens
    s = eng.new_sequence()
    got = eng.step([(s, a)], [[149, 3]]).float().cpu()
    eng.end_sequence(s)
    _close(got, want[id(a)][[149, 3]], what="two rows of a prompt")
    eng.cache.check()
    assert eng.cache.slots.used == 0 and all(g.pool.used == 0 for g in eng.cache.kv_groups)


def test_every_pass_of_a_loop_has_its_own_cache_and_start(tmp_path):
    """The looped layers are named once per pass in the schedule, every pass owns what it keeps, and a pass starts
    with its own vector (and, from the second on, the embedding's output): without either the logits move."""
    layers = [_rglru(), _parallel(), _rglru(width=32, blocks=4), _parallel(heads=2, kv_heads=2, dim=8, rot=_rot(dims=8))]
    d, tensors, config = _make(tmp_path, "loop", _config(layers, loop=(1, 3, 3)), seed=4)
    eng = _engine(d)
    assert eng.model.spec.schedule == (0, 1, 2, 1, 2, 1, 2, 3)
    assert eng.model.spec.run_input_at == ((1, 0, False), (3, 1, True), (5, 2, True))
    assert len(eng.cache.state) == 8 and sum(len(g.layers) for g in eng.cache.kv_groups) == 4
    t = random_tokens(90, VOCAB, 4)
    want = _plain(tensors, config, t)
    zeroed = dict(tensors, **{"loop.step": torch.zeros_like(tensors["loop.step"])})
    assert (_plain(zeroed, config, t) - want).abs().max() > 100 * FP32_TOL * want.std()
    once = json.loads(json.dumps(config))
    once["loop"]["times"] = 1
    assert (_plain(dict(tensors, **{"loop.step": tensors["loop.step"][:1]}), once, t) - want).abs().max() > 100 * FP32_TOL * want.std()
    _close(run_tail(eng, t, tail=30), want, what="looped layers")
    _close(run_chunks(eng, t, [2, 50, 38]), want, what="looped layers in portions")


# ----------------------------------------------------------------------------- far keys, sinks, page borders
def test_a_far_key_decides_logits_through_attention(tmp_path):
    """Attention alone carries the first tokens to the end here (the delta rule beside it forgets within tens of
    tokens): with a peaked softmax, changing token 3 of 600 moves the last rows of logits, in a prompt, in portions
    that cut pages and in 200 single tokens."""
    layers = [_parallel(scale=1.6, right_scale=0.4), _parallel(heads=2, kv_heads=1, dim=16, scale=1.2, rot=_rot(dims=16))]
    d, tensors, config = _make(tmp_path, "far_key", _config(layers), seed=12)
    t = random_tokens(600, VOCAB, 8)
    want = _plain(tensors, config, t)
    changed = list(t)
    changed[3] = (changed[3] + 1) % VOCAB
    moved = (_plain(tensors, config, changed)[400:] - want[400:]).abs().amax(dim=1) / want.std()
    assert (moved > 50 * FP32_TOL).sum() >= 10, "the weights do not let a far key show"
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=200), want, what="200 single tokens")
    _close(run_chunks(eng, t, [333, 67, 2, 198]), want, what="portions")


def test_the_sink_takes_its_share_of_every_softmax(tmp_path):
    """One more term in the denominator and nothing in the numerator: without it (a sink far below every score)
    the logits differ by far more than the tolerance, from the very first token on, where the sink stands against
    a single key."""
    layers = [_parallel(scale=0.5, right_scale=0.2, left_scale=1.5)]
    d, tensors, config = _make(tmp_path, "sink", _config(layers, side=None), seed=2)
    t = random_tokens(140, VOCAB, 9)
    want = _plain(tensors, config, t)
    none = dict(tensors, **{"l0.mix.left.sink": torch.full_like(tensors["l0.mix.left.sink"], -60.0)})
    moved = (_plain(none, config, t) - want).abs().amax(dim=1) / want.std()
    assert moved[0] > 100 * FP32_TOL and (moved > 100 * FP32_TOL).sum() > 100, "the weights do not let the sink show"
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=len(t)), want, what="token by token")
    outs = run_batch(eng, [t, t[:5]], [70, 1])
    _close(outs[0], want, what="batch")
    _close(outs[1], want[:5], what="batch, the short request")


def test_first_tokens_stay_in_the_states(tmp_path):
    """Decays close to 1 in both recurrences (attention switched off by its constant): the first tokens of a
    300-token prompt still move the last logits, through prompts, portions and 150 single tokens alike.  (A slow
    channel takes little of each token, sqrt(1 - a^2) of it, so five tokens are changed, and the bar is lower than
    for a key that a peaked softmax picks.)"""
    layers = [_rglru(), _parallel(left_scale=0.0, right_scale=1.5), _rglru(width=32, blocks=2, conv=2)]
    d, tensors, config = _make(tmp_path, "far_state", _config(layers), seed=21, slow=True)
    t = random_tokens(300, VOCAB, 8)
    want = _plain(tensors, config, t)
    changed = [(tok + 1) % VOCAB if i < 5 else tok for i, tok in enumerate(t)]
    assert (_plain(tensors, config, changed)[-1] - want[-1]).abs().max() > 30 * FP32_TOL * want.std()
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=150), want, what="150 single tokens")
    _close(run_chunks(eng, t, [133, 67, 100]), want, what="portions")


def test_requests_that_end_at_page_borders_in_one_batch(tmp_path):
    layers = [_parallel(scale=1.1), _rglru()]
    d, tensors, config = _make(tmp_path, "borders", _config(layers), seed=6)
    lens = [63, 64, 65, 128, 129, 1]
    reqs = [random_tokens(n + 4, VOCAB, 30 + n) for n in lens]
    eng = _engine(d)
    for _ in range(2):                                # the second time takes the pages and slots the first gave back
        outs = run_batch(eng, reqs, lens)
        for got, r in zip(outs, reqs):
            _close(got, _plain(tensors, config, r), what=f"a request of {len(r)} tokens")
    eng.cache.check()
    assert eng.cache.slots.used == 0 and all(g.pool.used == 0 for g in eng.cache.kv_groups)


def test_stretched_rotation_tables():
    """The frequencies and the amplitude that the position part makes, against the plain rule, for ramps that are
    cut at either end and for a rotation without stretching."""
    from picolm_b200.parts.position import rope_inverse_frequencies, rope_magnitude
    for dims, base, sc in ((8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}),
                           (32, 500000.0, {"factor": 16.0, "original": 4096, "fast": 32.0, "slow": 0.5}),
                           (6, 30.0, {"factor": 2.0, "original": 16, "fast": 1.5, "slow": 1.0}), (12, 100.0, None)):
        want, amp = P.stretched_frequencies(dims, base, sc)
        got = rope_inverse_frequencies(dims, base, dict(sc, rope_type="yarn") if sc else None)
        assert torch.allclose(torch.tensor(got, dtype=torch.float64), want, rtol=1e-12)
        assert math.isclose(rope_magnitude(dict(sc, rope_type="yarn") if sc else None), amp, rel_tol=1e-12)


# ------------------------------------------------------------------------------------------------ bfloat16
def test_bfloat16_follows_the_plain_implementation(tmp_path):
    """The serving precision stays within rounding of the exact logits, and its own cuts agree with each other far
    more closely than that."""
    layers = [_rglru(width=64, blocks=4), _parallel(dim=32, rot=_rot(dims=16), rdim=16, rvdim=16, ff=128), _rglru(width=96, blocks=2)]
    d, tensors, config = _make(tmp_path, "bf16", _config(layers, width=64, loop=(1, 2, 2), side=8), seed=3)
    t, u = random_tokens(200, VOCAB, 5), random_tokens(31, VOCAB, 6)
    want = _plain(tensors, config, t)
    eng = _engine(d, dtype="bfloat16")
    whole = run_whole(eng, t)
    rel = ((whole - want).double().pow(2).mean().sqrt() / want.double().std()).item()
    assert rel < 0.05, f"bfloat16 logits are {rel:.3f} of the spread away from the exact ones"
    for got in (run_tail(eng, t, tail=70), run_chunks(eng, t, [64, 2, 134]), run_batch(eng, [u, t], [11, 130])[1]):
        rel = ((got - whole).double().pow(2).mean().sqrt() / want.double().std()).item()
        assert rel < 0.03, f"two cuts of the same request differ by {rel:.3f} of the spread"
    eng.cache.check()


@pytest.mark.parametrize("dim,heads,kv", [(64, 4, 2), (128, 2, 1), (96, 3, 3), (40, 2, 1)])
def test_bfloat16_sink_attention_on_the_tensor_cores(tmp_path, dim, heads, kv):
    """Head sizes that the bfloat16 attention kernels take on the tensor cores (tcgen05 prompts at 64 and 128, mma.sync
    prompts and decode steps at the other multiples of 16, heads padded to the next one at 40), with the sink and with
    keys that serve as values: without the sink the exact logits differ by several times what bfloat16 costs, so a
    kernel that forgot it would show; prompts, portions and single tokens agree."""
    layers = [_parallel(heads=heads, kv_heads=kv, dim=dim, rot=_rot(dims=dim // 2), scale=1.5 * dim ** -0.5, right_scale=0.3,
                        left_scale=1.5, ff=None)]
    d, tensors, config = _make(tmp_path, f"tc{dim}", _config(layers, width=64, side=None), seed=dim, sink=5.0)
    t = random_tokens(200, VOCAB, dim)
    want = _plain(tensors, config, t)
    none = dict(tensors, **{"l0.mix.left.sink": torch.full_like(tensors["l0.mix.left.sink"], -60.0)})
    gap = ((_plain(none, config, t) - want).double().pow(2).mean().sqrt() / want.double().std()).item()
    assert gap > 0.15, f"the weights do not let the sink show ({gap:.3f})"
    eng = _engine(d, dtype="bfloat16")
    whole = run_whole(eng, t)
    rel = ((whole - want).double().pow(2).mean().sqrt() / want.double().std()).item()
    assert rel < 0.05, f"bfloat16 logits are {rel:.3f} of the spread away from the exact ones"
    for got in (run_tail(eng, t, tail=70), run_chunks(eng, t, [64, 2, 134]), run_batch(eng, [t[:9], t], [5, 130])[1]):
        rel = ((got - whole).double().pow(2).mean().sqrt() / want.double().std()).item()
        assert rel < 0.03, f"two cuts of the same request differ by {rel:.3f} of the spread"


# ---------------------------------------------------------------------------------------------- generation
def test_greedy_generation_through_the_entry_point(tmp_path):
    """`generate` (the scheduler, batching, sampling at temperature 0) gives the tokens that the plain implementation
    chooses one by one, for requests of unequal lengths that run together."""
    from picolm_b200.api import generate, model_load
    layers = [_rglru(), _parallel(scale=1.0), _parallel(heads=2, kv_heads=1, dim=8, rot=False, ff=None)]
    d, tensors, config = _make(tmp_path, "gen", _config(layers, loop=(0, 2, 2)), seed=17)
    prompts = [random_tokens(70, VOCAB, 1), random_tokens(3, VOCAB, 2), random_tokens(1, VOCAB, 3)]
    n_new = 12
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(n_new):
            seq.append(int(_plain(tensors, config, seq)[-1].argmax()))
        want.append(seq[len(p):])
    eng = model_load(d, dtype="float32", context=256, max_batch=4)
    got = generate(eng, prompts, max_tokens=n_new, temperature=0.0)
    for g_, w_, p in zip(got, want, prompts):
        if g_ != w_:
            # a tie within the tolerance may be broken either way: then the plain logits at the first difference must be tied
            k = next(i for i, (x, y) in enumerate(zip(g_, w_)) if x != y)
            row = _plain(tensors, config, list(p) + w_[:k])[-1]
            assert abs(row[g_[k]] - row[w_[k]]) <= FP32_TOL * row.std(), f"token {k} differs: {g_[k]} for {w_[k]}"
