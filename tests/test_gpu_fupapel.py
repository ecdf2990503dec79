"""The Fupapel design through the library, against the plain implementation in
`tests/plain/fupapel_plain.py`: each mechanism alone (kernels against plain functions, then models of one
kind of layer), prompts against token-by-token decoding, portions down to two tokens, batches of unequal
requests, pages and slots used again, keys far away, at page borders and on either side of a chunk's edge,
the first tokens, long decoding, sizes that make special cases (one key head or as many as query heads,
keys and values of different widths, no rotation, a whole and a part rotation, stretched or not, one tap,
no groups, one choice, no identity expert, no feed-forward, a layer that borrows keys and values), and
greedy generation through the library's entry point.

Weights are random; where random weights would hide a fault they are reshaped: the attention's scale is
large so that the softmax is peaked (one far key, a chunk's edge or the sink then decides a row of logits),
and the token shift is drawn over all of [0, 1] so that the row before matters.
"""
import json
import math
import os

import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import fupapel_plain as P
from util import random_tokens

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-4          # of the logits' spread; two float32 computations in different orders of summation
VOCAB = 97


def _moe(experts=6, top=2, ff=20, identity=2, groups=(4, 2)):
    router = {"experts": experts, "top": top, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _rot(dims=8, base=300.0, scaling=False):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    return out


def _attn(heads=4, kv_heads=2, dim=16, vdim=24, chunk=7, scale=0.9, rot=8, base=300.0, mlp="moe"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = _rot(rot, base)
    return {"type": "attention", "mixer": m, "mlp": _moe() if mlp == "moe" else mlp}


def _attn2(heads=4, kv_heads=2, dim=16, vdim=8, chunk=9, scale=0.8, rot=16, base=1000.0, scaling=True, conv=3,
           kv_from=None, mlp="moe"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = _rot(rot, base, scaling)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": _moe() if mlp == "moe" else mlp}


def _latent(heads=3, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=28, scale=0.7, base=5000.0, mlp="moe", chunk=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": _rot(rot_dim, base)}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "latent_attention", "mixer": m, "mlp": _moe() if mlp == "moe" else mlp}


def _config(layers, width=40, eps=1e-5, mult=0.7):
    return {"architecture": "Fupapel", "vocab": VOCAB, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": [json.loads(json.dumps(layer)) for layer in layers]}


def _make(tmp_path, name, config, seed, std=0.12, sink=None):
    """A model folder with random weights for `config`; returns (folder, plain tensors, config).  `sink`: every learned
    sink is this number (else drawn from N(0, 2))."""
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors, save_safetensors
    cfg = config_from_dict(config)
    tensors = random_tensors(cfg, seed, std=std, norm_std=0.2)
    g = torch.Generator().manual_seed(seed + 1000)
    for n in list(tensors):
        t = tensors[n]
        if n.endswith(".sink"):
            tensors[n] = (torch.full(t.shape, float(sink)) if sink is not None else 2.0 * torch.randn(t.shape, generator=g)).to(t.dtype)
        elif n.endswith(".correction"):
            tensors[n] = (0.3 * torch.randn(t.shape, generator=g)).to(t.dtype)      # of the scores' own size: it decides choices
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
    """What the kernels read of a step, for sequences that bring `lens` tokens each from position `starts`."""

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
        self.max_position = max(s + n - 1 for s, n in zip(starts, lens))


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("d", [40, 42, 256])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_two_norms_and_the_shift_in_one_pass(d, out_dtype):
    """Both norms of the same rows and the mixer's rows shifted towards the token before, over ragged steps whose
    sequences go on from a state: the whole of three sequences in one step equals their pieces in three."""
    from picolm_b200 import ops
    dev = "cuda"
    g = torch.Generator().manual_seed(d)
    lens = [9, 1, 14]
    xs = [torch.randn(n, d, generator=g) for n in lens]
    w_a, w_b, mu = 1 + 0.2 * torch.randn(d, generator=g), 1 + 0.2 * torch.randn(d, generator=g), torch.rand(d, generator=g)
    eps = 1e-5
    want_a = [P.token_shift(P.rms_norm(x.double(), w_a.double(), eps), mu.double()) for x in xs]
    want_b = [P.rms_norm(x.double(), w_b.double(), eps) for x in xs]
    state = torch.full((5, d + 3), 7.0, device=dev)
    slots = [3, 0, 1]
    state[slots] = 0.0
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    cuts = [[(0, 4), (0, 1), (0, 2)], [(4, 5), None, (2, 13)], [(5, 9), None, (13, 14)]]
    got_a = [torch.zeros(n, d) for n in lens]
    got_b = [torch.zeros(n, d) for n in lens]
    for cut in cuts:
        live = [i for i, c in enumerate(cut) if c is not None]
        step = _Step([cut[i][1] - cut[i][0] for i in live], [slots[i] for i in live], dev)
        x = torch.cat([xs[i][cut[i][0]:cut[i][1]] for i in live]).to(dev)
        a, b = ops.norm_pair_shift(x, w_a.to(dev), eps, out_dtype, w_b=w_b.to(dev), mix=mu.to(dev), state=state, step=step)
        o = 0
        for i in live:
            n = cut[i][1] - cut[i][0]
            got_a[i][cut[i][0]:cut[i][1]] = a[o:o + n].float().cpu()
            got_b[i][cut[i][0]:cut[i][1]] = b[o:o + n].float().cpu()
            o += n
    for i in range(3):
        assert (got_a[i].double() - want_a[i]).abs().max() < tol * 4, f"shifted rows of sequence {i}"
        assert (got_b[i].double() - want_b[i]).abs().max() < tol * 4, f"second norm of sequence {i}"
    assert (state[2] == 7.0).all() and (state[:, d:] != 0).any(), "rows of other slots and columns beyond the state were touched"
    # without a shift and a second norm it is a plain norm
    a, b = ops.norm_pair_shift(xs[0].to(dev), w_a.to(dev), eps, out_dtype)
    assert b is None and (a.float().cpu().double() - P.rms_norm(xs[0].double(), w_a.double(), eps)).abs().max() < tol * 4


def test_shift_as_a_convolution_of_two_taps(tmp_path):
    """The part's own forward (for norms that cannot do the shift on the way): a causal convolution with the taps
    (mu, 1 - mu) and the row before as its state."""
    from picolm_b200.parts import build_part
    from picolm_b200.config.spec import PartSpec
    from picolm_b200.runtime import Runtime
    from picolm_b200.cache.sequence_cache import StateLayerCache
    dev = "cuda"
    g = torch.Generator().manual_seed(4)
    part = build_part("row_filter", PartSpec("token_shift", {"size": 24, "name": ""}), Runtime(torch.device(dev), torch.float32))
    mu = torch.rand(24, generator=g)
    part.load({"": mu.to(dev)})
    h = torch.randn(11, 24, generator=g)
    want = P.token_shift(h.double(), mu.double())
    state = torch.zeros(3, 24, device=dev)
    a = part.forward(h[:6].to(dev).contiguous(), _Step([6], [1], dev), StateLayerCache(state))
    b = part.forward(h[6:].to(dev).contiguous(), _Step([5], [1], dev, starts=[6]), StateLayerCache(state))
    assert (torch.cat([a, b]).cpu().double() - want).abs().max() < 1e-5
    assert part.cache_spec().private and part.cache_spec().shape == (24,)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rot,hd,pairing", [(8, 16, "half"), (16, 16, "half"), (6, 32, "adjacent")])
def test_rotation_of_rows_in_place(dtype, rot, hd, pairing):
    from picolm_b200 import ops
    from picolm_b200.parts.position import rope_inverse_frequencies
    dev = "cuda"
    g = torch.Generator().manual_seed(rot)
    T, H = 13, 3
    pos = torch.randint(0, 500, (T,), generator=g)
    x = torch.randn(T, H * hd + 5, generator=g).to(dtype)
    inv = torch.tensor(rope_inverse_frequencies(rot, 700.0, None), dtype=torch.float64)
    ang = torch.arange(512, dtype=torch.float64)[:, None] * inv[None, :]
    rotation = ops.Rotation(ang.cos().float().to(dev), ang.sin().float().to(dev), rot, pairing)
    xd = x.to(dev)
    view = xd[:, :H * hd]
    ops.rope_rows(view, rotation, pos.to(torch.int32).to(dev), H, hd)
    src = x[:, :H * hd].double().reshape(T, H, hd)
    if pairing == "half":
        want = P.rotate_halves(src, pos.tolist(), rot, 700.0)
    else:
        a = ang[pos]
        want = src.clone()
        u, v = src[..., 0:rot:2], src[..., 1:rot:2]
        want[..., 0:rot:2] = u * a.cos()[:, None] - v * a.sin()[:, None]
        want[..., 1:rot:2] = v * a.cos()[:, None] + u * a.sin()[:, None]
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert (xd[:, :H * hd].float().cpu().double().reshape(T, H, hd) - want).abs().max() < tol
    assert torch.equal(xd[:, H * hd:].cpu(), x[:, H * hd:]), "columns beyond the heads were touched"


def test_stretched_frequencies_follow_the_three_band_rule():
    """The library's table builder against the plain rule, with parameters under which all three bands occur."""
    from picolm_b200.parts.position import rope_inverse_frequencies
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    want = P.stretched_frequencies(32, 1000.0, sc)
    plain = P.stretched_frequencies(32, 1000.0, None)
    kinds = {("kept" if w == p else "divided" if abs(w - p / 8.0) < 1e-15 else "blended") for w, p in zip(want, plain)}
    assert kinds == {"kept", "divided", "blended"}
    got = rope_inverse_frequencies(32, 1000.0, {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                                "high_freq_factor": 4.0, "original_max_position_embeddings": 64})
    assert max(abs(a - b) for a, b in zip(got, want)) < 1e-12


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("n_rot,n_norm,R", [(8, 24, 32), (0, 20, 32), (16, 40, 64)])
def test_latent_row_into_the_pages(in_dtype, out_dtype, n_rot, n_norm, R):
    """[rotated shared key part | normed latent | zeros] at every token's place in the pages, pages out of order."""
    from picolm_b200 import ops
    from picolm_b200.parts.position import rope_inverse_frequencies
    dev = "cuda"
    g = torch.Generator().manual_seed(n_rot + n_norm)
    lens, starts = [70, 3], [60, 127]
    step = _Step(lens, [0, 1], dev, starts=starts)
    table = torch.tensor([[5, 2, 7], [1, 6, 3]], dtype=torch.int32, device=dev)
    pages = torch.full((8, 1, 64, R), 9.0, dtype=out_dtype, device=dev)
    rows = torch.randn(sum(lens), n_rot + n_norm + 6, generator=g).to(in_dtype)
    w = 1 + 0.3 * torch.randn(n_norm, generator=g)
    rotation = None
    if n_rot:
        inv = torch.tensor(rope_inverse_frequencies(n_rot, 900.0, None), dtype=torch.float64)
        ang = torch.arange(256, dtype=torch.float64)[:, None] * inv[None, :]
        rotation = ops.Rotation(ang.cos().float().to(dev), ang.sin().float().to(dev), n_rot, "half")
    wq = 1 + 0.3 * torch.randn(3, generator=g)
    rows_d = rows.to(dev)
    c_q = ops.latent_store(rows_d[:, 3:3 + n_rot + n_norm], w.to(dev), 1e-5, rotation, n_rot, pages, step, table,
                           q_rows=rows_d[:, :3], q_weight=wq.to(dev))
    src = rows[:, 3:3 + n_rot + n_norm].double()
    assert c_q.dtype == out_dtype
    assert (c_q.float().cpu().double() - P.rms_norm(rows[:, :3].double(), wq.double(), 1e-5)).abs().max() < (1e-5 if out_dtype == torch.float32 else 3e-2)
    untouched = torch.full_like(pages, 9.0)
    again = ops.latent_store(rows_d[:, 3:3 + n_rot + n_norm], w.to(dev), 1e-5, rotation, n_rot, untouched, step, table, store=False,
                             q_rows=rows_d[:, :3], q_weight=wq.to(dev))
    assert torch.equal(again, c_q) and (untouched == 9.0).all(), "a layer that only reads the cache wrote it"
    pos = step.tok_pos.cpu().tolist()
    want = torch.zeros(sum(lens), R, dtype=torch.float64)
    if n_rot:
        want[:, :n_rot] = P.rotate_halves(src[:, None, :n_rot], pos, n_rot, 900.0)[:, 0]
    want[:, n_rot:n_rot + n_norm] = P.rms_norm(src[:, n_rot:], w.double(), 1e-5)
    tol = 1e-5 if out_dtype == torch.float32 else 3e-2
    for t in range(sum(lens)):
        b = int(step.tok_seq[t])
        page = int(table[b, pos[t] // 64])
        assert (pages[page, 0, pos[t] % 64].float().cpu().double() - want[t]).abs().max() < tol, f"token {t}"
    assert (pages[4] == 9.0).all() and (pages[0] == 9.0).all()


@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("own", [True, False])
def test_convolution_norm_rotation_factor_and_cache_write_in_one_kernel(taps, own):
    """Between the QKV product and attention of a convolved layer: the short convolution over time on every column
    (from a tail of earlier steps), the norm over all heads, the rotation, the factor per head, the cache write; the
    product's row holds more columns behind q, k and v.  A prompt in two portions and single tokens against the plain
    functions over the whole sequence."""
    from picolm_b200 import ops
    from picolm_b200.cache.sequence_cache import KVLayerCache
    from picolm_b200.parts.position import rope_inverse_frequencies
    dev = "cuda"
    g = torch.Generator().manual_seed(taps)
    H, G, D, Dv, rot, hd_c, eps = 4, 2, 12, 6, 8, 16, 1e-5
    cols = H * D + ((G * D + G * Dv) if own else 0)
    T = 75
    proj = torch.randn(T, cols + 7, generator=g)
    w_conv = 0.5 * torch.randn(cols, taps, generator=g)
    wq, wk, temp = 1 + 0.2 * torch.randn(H * D, generator=g), 1 + 0.2 * torch.randn(G * D, generator=g), 0.5 + torch.rand(H, generator=g)
    conv = P.short_conv(proj[:, :cols].double(), w_conv.double())
    pos = list(range(T))
    want_q = P.rotate_halves(P.rms_norm(conv[:, :H * D], wq.double(), eps).reshape(T, H, D), pos, rot, 700.0) * temp.double()[None, :, None]
    inv = torch.tensor(rope_inverse_frequencies(rot, 700.0, None), dtype=torch.float64)
    ang = torch.arange(128, dtype=torch.float64)[:, None] * inv[None, :]
    rotation = ops.Rotation(ang.cos().float().to(dev), ang.sin().float().to(dev), rot, "half")
    table = torch.tensor([[3, 1]], dtype=torch.int32, device=dev)
    k_pages = torch.zeros(4, G, 64, hd_c, device=dev)
    v_pages = torch.zeros(4, G, 64, hd_c, device=dev)
    state = torch.zeros(3, max(1, (taps - 1) * cols) + 2, device=dev)
    got_q = torch.zeros(T, H, hd_c)
    start = 0
    for n in [40, 2, 1, 1, 30, 1]:
        step = _Step([n], [1], dev, starts=[start])
        q = torch.full((n, H, hd_c), 5.0, device=dev)
        kv = KVLayerCache(k_pages, v_pages, table, None, own)
        ops.qk_norm_rope_store(proj[start:start + n].to(dev)[:, :cols], None, wq.to(dev), wk.to(dev) if own else None, eps, q, kv,
                               rotation, step, H, G, D, Dv, own_kv=own, q_scale=temp.to(dev), conv=w_conv.t().contiguous().to(dev),
                               conv_state=state)
        got_q[start:start + n] = q.cpu()
        start += n
    assert (got_q[:, :, :D].double() - want_q).abs().max() < 2e-5 and (got_q[:, :, D:] == 0).all()
    assert (state[0] == 0).all() and (state[2] == 0).all()
    if own:
        want_k = P.rotate_halves(P.rms_norm(conv[:, H * D:H * D + G * D], wk.double(), eps).reshape(T, G, D), pos, rot, 700.0)
        want_v = conv[:, H * D + G * D:].reshape(T, G, Dv)
        for t in range(T):
            page = int(table[0, t // 64])
            assert (k_pages[page, :, t % 64, :D].cpu().double() - want_k[t]).abs().max() < 2e-5, f"key {t}"
            assert (v_pages[page, :, t % 64, :Dv].cpu().double() - want_v[t]).abs().max() < 2e-5, f"value {t}"
    else:
        assert (k_pages == 0).all() and (v_pages == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [3, 90])
def test_one_matrix_per_head_with_a_gate_per_head(dtype, T):
    from picolm_b200 import ops
    dev = "cuda"
    g = torch.Generator().manual_seed(T)
    H, O, I = 3, 20, 32
    x = torch.randn(T, H * I, generator=g).to(dtype)
    w = (0.3 * torch.randn(H, O, I, generator=g)).to(dtype)
    gate = torch.randn(T, H + 2, generator=g)
    got = ops.head_linear(x.to(dev), w.to(dev), gate=gate.to(dev)[:, 1:1 + H], gate_per_head=True).float().cpu()
    want = torch.einsum("hoi,thi->tho", w.double(), x.double().reshape(T, H, I)) * torch.sigmoid(gate[:, 1:1 + H].double())[:, :, None]
    assert (got.double().reshape(T, H, O) - want).abs().max() < (1e-5 if dtype == torch.float32 else 5e-2)


@pytest.mark.parametrize("E,ident,top,groups", [(6, 2, 2, (4, 2)), (10, 2, 3, (3, 1)), (5, 0, 1, None), (4, 4, 3, (8, 3)), (7, 1, 8, None)])
def test_router_choice_by_softmax_scores(E, ident, top, groups):
    """Softmax over experts and identity experts together, the correction for the choice only (negative choice scores
    included), groups by their best choice score, weights as the scores stand."""
    from picolm_b200 import ops
    dev = "cuda"
    g = torch.Generator().manual_seed(E * 10 + top)
    T, n_out = 50, E + ident
    logits = 2.0 * torch.randn(T, n_out + 1, generator=g)
    corr = torch.randn(n_out, generator=g) - 0.5
    r = {"experts": E, "identity": ident, "top": top}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    W = {"router": torch.eye(n_out, dtype=torch.float64), "correction": corr.double()}
    want_ids, want_w = P.route(logits[:, :n_out].double(), W, r)
    ids, weights, _ = ops.route_topk(logits.to(dev), n_out, top, corr.to(dev), groups[0] if groups else 1, groups[1] if groups else 1,
                                     1.0, None, scores="softmax", group_score="max", normalize=False)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (weights.cpu().double() - want_w).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_weighted_sum_with_identity_experts_into_the_stream(dtype):
    """Pairs of an expert without tensors enter as weight * input; the mixer's rows beside the sum, one factor on both,
    added to the stream in place."""
    from picolm_b200 import ops
    dev = "cuda"
    g = torch.Generator().manual_seed(1)
    T, top, E, ident, d = 37, 3, 4, 2, 24
    ids = torch.stack([torch.randperm(E + ident, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    weights = torch.rand(T, top, generator=g)
    h = torch.randn(T, d, generator=g).to(dtype)
    add, x = torch.randn(T, d, generator=g), torch.randn(T, d, generator=g)
    pairs = ops.moe_align(ids.to(dev), E, 16, ident)
    where = pairs.where.cpu().reshape(T, top)
    assert ((where < 0) == (ids >= E)).all()
    assert int((pairs.sorted >= 0).sum()) == int((ids < E).sum())
    y = torch.randn(pairs.rows, d, generator=g)
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            src = h[t].double() if ids[t, k] >= E else y[where[t, k]].double()
            want[t] += weights[t, k].double() * src
    out = ops.moe_combine(y.to(dev), pairs, weights.to(dev), ident=h.to(dev))
    assert (out.cpu().double() - want).abs().max() < 1e-5
    xd = x.to(dev)
    back = ops.moe_combine(y.to(dev), pairs, weights.to(dev), ident=h.to(dev), add=add.to(dev), out_scale=0.3, into=xd)
    assert back.data_ptr() == xd.data_ptr()
    assert (xd.cpu().double() - (x.double() + 0.3 * (want + add.double()))).abs().max() < 1e-5


# ------------------------------------------------------------------------------------------------- models
MODELS = {
    # each mixer alone
    "gated": ([_attn(), _attn(heads=2, kv_heads=1, dim=8, vdim=8, chunk=64, rot=8)], {}),
    "convolved": ([_attn2(), _attn2(heads=2, kv_heads=2, dim=24, vdim=24, chunk=65, rot=8, scaling=False, conv=4)], {}),
    "latent": ([_latent(), _latent(heads=2, dim=16, rot_dim=16, vdim=16, kv_rank=32, q_rank=16, chunk=11)], {}),
    # all three, a layer that borrows keys and values (and cuts its chunks elsewhere would need its own mask: the same
    # mask here, other queries), a layer without feed-forward, no groups, one choice, no identity experts
    "mixed": ([_attn(mlp=_moe(groups=None)), _attn2(kv_heads=1), _latent(mlp=None), _attn2(kv_heads=1, chunk=5, kv_from=1,
               mlp=_moe(top=1, identity=0, groups=(3, 1))), _attn(heads=4, kv_heads=4, rot=0, chunk=None)], {"mult": 0.5}),
    # an odd width, one tap, a rotation of two components, every router output kept, a factor of 1 on the residual
    "odd": ([_attn2(heads=3, kv_heads=1, dim=10, vdim=6, rot=2, conv=1, chunk=130, mlp=_moe(experts=3, top=4, ff=12, identity=1, groups=(2, 2))),
             _latent(heads=1, dim=8, rot_dim=2, vdim=8, kv_rank=16, q_rank=8), _attn2(heads=3, kv_heads=1, dim=10, vdim=6, rot=2,
             conv=2, chunk=3, kv_from=0, mlp=None)], {"width": 42, "mult": 1.0}),
}


@pytest.mark.parametrize("name", sorted(MODELS))
def test_float32_model_matches_plain_in_every_cut(tmp_path, name):
    """Whole prompts, a prompt and 90 single tokens over a page border, token by token from the first, portions down
    to two tokens, a batch of unequal requests, and the same again on slots and pages that were given back."""
    layers, kw = MODELS[name]
    d, tensors, config = _make(tmp_path, name, _config(layers, **kw), seed=len(name))
    reqs = [random_tokens(n, VOCAB, 100 + i) for i, n in enumerate([150, 40, 1, 129])]
    want = [_plain(tensors, config, t) for t in reqs]
    eng = _engine(d)
    for turn in range(2):
        _close(run_whole(eng, reqs[0]), want[0], what="whole")
        _close(run_tail(eng, reqs[0], tail=90), want[0], what="a prompt and 90 single tokens")
        _close(run_tail(eng, reqs[1], tail=40), want[1], what="token by token from the first")
        _close(run_chunks(eng, reqs[0], [2, 62, 3, 61, 2, 20]), want[0], what="portions")
        outs = run_batch(eng, reqs, [64, 7, 1, 129])
        for i, (got, ref) in enumerate(zip(outs, want)):
            _close(got, ref, what=f"batch, request {i}, turn {turn}")
    eng.cache.check()
    assert eng.cache.slots.used == 0


def test_few_wanted_rows_and_the_arrangement_without_its_fused_kernels(tmp_path, monkeypatch):
    """A step of which few rows are wanted narrows the stream in its last layer (with and without a feed-forward there);
    and the arrangement's general path (norms one after the other, the shift as the part's own convolution, the two
    sublayers' results joined by a kernel of their own and left pending) gives the same logits as the fused one."""
    from picolm_b200.parts.block import ParallelNormBlock
    from picolm_b200.parts.feed_forward import RoutedMLP
    for name in ("mixed", "odd"):
        layers, kw = MODELS[name]
        d, tensors, config = _make(tmp_path, "few" + name, _config(layers, **kw), seed=31)
        t, u = random_tokens(100, VOCAB, 12), random_tokens(9, VOCAB, 13)
        want_t, want_u = _plain(tensors, config, t), _plain(tensors, config, u)
        for general in (False, True):
            with monkeypatch.context() as m:
                if general:
                    m.setattr(ParallelNormBlock, "_fused_norms", lambda self: False)
                    m.setattr(RoutedMLP, "adds_to_stream", False)
                eng = _engine(d)
                a, b = eng.new_sequence(), eng.new_sequence()
                got = eng.step([(a, t[:70]), (b, u[:5])], [[69, 3], [4]]).float().cpu()
                _close(got, torch.stack([want_t[69], want_t[3], want_u[4]]), what=f"{name}: three rows of a batch")
                assert eng.step([(a, t[70:90]), (b, u[5:])], [[], []]) is None
                got = eng.step([(a, t[90:])], [[9]]).float().cpu()
                _close(got, want_t[99:100], what=f"{name}: after a step of which nothing was wanted")
                eng.end_sequence(a), eng.end_sequence(b)
                if general:
                    _close(run_tail(eng, t, tail=30), want_t, what=f"{name}: the general path, prompt and single tokens")


def test_layer_that_borrows_keys_and_values_keeps_its_own_tails(tmp_path):
    """A borrowing layer owns the row before its shift and its queries' convolution tail, and nothing else."""
    layers, kw = MODELS["mixed"]
    d, _, _ = _make(tmp_path, "own", _config(layers, **kw), seed=2)
    eng = _engine(d)
    specs = eng.model.cache_specs()
    kinds = [(s.kind, s.private) for s in specs]
    assert kinds.count(("kv", False)) == 4, "five layers, one of which borrows: four sets of keys and values"
    assert kinds.count(("state", True)) == 5 + 2, "a shift row a layer, a convolution tail for each of the two convolved layers"
    borrower = eng.model._run_caches[3]
    assert [w for _, w in borrower] == [True, False, True] and borrower[1][0] == eng.model._run_caches[1][1][0]
    own_tail, lender_tail = specs[borrower[2][0]], specs[eng.model._run_caches[1][2][0]]
    assert own_tail.shape == (2 * 4 * 16,) and lender_tail.shape == (2 * (4 * 16 + 16 + 8),)


# -------------------------------------------------------------------------------------------- chunk edges
@pytest.mark.parametrize("chunk", [5, 64, 65, 130])
@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_chunk_edges_decide_logits_and_are_right(tmp_path, chunk, kind):
    """With a peaked softmax one key often holds most of a row's weight: a chunk that is cut one token off changes rows'
    logits by far more than the tolerance (the test first makes sure of that with the plain implementation), in
    prompts, in portions that start inside a chunk and in single tokens, with chunks that end on a page's border and
    just beside it; the first tokens of a sequence and of every chunk see only what their chunk holds."""
    make = _attn if kind == "attention" else _attn2
    layers = [make(heads=2, kv_heads=1, dim=16, vdim=8, chunk=chunk, scale=2.5, rot=8, mlp=None),
              make(heads=2, kv_heads=2, dim=16, vdim=16, chunk=chunk + 3, scale=2.5)]
    d, tensors, config = _make(tmp_path, f"c{chunk}", _config(layers), seed=chunk, sink=-3.0)
    t = random_tokens(290, VOCAB, chunk)
    want = _plain(tensors, config, t)
    for off in (-1, 1):
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = chunk + off
        diff = (_plain(tensors, other, t) - want).abs().amax(dim=1) / want.std()
        assert (diff > 50 * FP32_TOL).sum() >= 3, "the weights do not make the chunk's edge show"
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=150), want, what="single tokens over chunk starts")
    _close(run_chunks(eng, t, [chunk - 1, 2, chunk, 3, 290 - 2 * chunk - 4]), want, what="portions around the edges")
    outs = run_batch(eng, [t, t[:chunk + 1], t[:3]], [chunk, chunk - 1, 1])
    _close(outs[0], want, what="batch")
    _close(outs[1], want[:chunk + 1], what="batch, a request that just fills a chunk")
    eng.cache.check()


def test_far_keys_and_the_first_tokens(tmp_path):
    """Chunks longer than the prompt and a latent layer that sees everything: the first tokens of a 600-token prompt
    still move the last logits, through prompts, portions and 200 single tokens alike (keys nine pages away)."""
    layers = [_attn(heads=2, kv_heads=1, dim=16, vdim=16, chunk=1000, scale=1.5, rot=16, base=50000.0, mlp=None),
              _latent(scale=1.6), _attn2(chunk=640, scale=1.2)]
    d, tensors, config = _make(tmp_path, "far", _config(layers), seed=21, sink=-2.0)
    t = random_tokens(600, VOCAB, 8)
    want = _plain(tensors, config, t)
    changed = list(t)
    changed[3] = (changed[3] + 1) % VOCAB
    assert (_plain(tensors, config, changed)[-1] - want[-1]).abs().max() > 20 * FP32_TOL * want.std()
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=200), want, what="200 single tokens")
    _close(run_chunks(eng, t, [333, 67, 200]), want, what="portions")


@pytest.mark.parametrize("which", ["zero", "learned", "latent"])
def test_the_sink_counts_once_and_unscaled(tmp_path, which):
    """The extra term of the denominator decides the first tokens' rows (one key: without the sink its weight would
    be 1).  The test first shows with the plain implementation that leaving the sink out, or scaling it with the
    scores, moves logits far beyond the tolerance."""
    layer = {"zero": _attn(scale=0.3, mlp=None), "learned": _attn2(scale=0.3, mlp=None), "latent": _latent(scale=0.3, mlp=None)}[which]
    d, tensors, config = _make(tmp_path, "sink" + which, _config([layer, layer]), seed=5, sink=1.5)
    t = random_tokens(70, VOCAB, 3)
    want = _plain(tensors, config, t)
    gone = {k: (v - 60.0 if k.endswith(".sink") else v) for k, v in tensors.items()}
    if which != "zero":
        assert (_plain(gone, config, t)[:4] - want[:4]).abs().max() > 100 * FP32_TOL * want.std()
        scaled = {k: (v * 0.3 if k.endswith(".sink") else v) for k, v in tensors.items()}
        assert (_plain(scaled, config, t)[:4] - want[:4]).abs().max() > 100 * FP32_TOL * want.std()
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=69), want, what="token by token")


def test_identity_experts_and_the_correction_decide(tmp_path):
    """A router whose corrections push the choice towards the identity experts, and groups of which one is kept: the
    plain implementation's choices change if the identity experts are left out of the groups, and the library follows
    the plain implementation."""
    layers = [_attn(mlp=_moe(experts=5, top=2, identity=3, groups=(2, 1))), _latent(mlp=_moe(experts=2, top=3, identity=4, groups=(3, 2)))]
    d, tensors, config = _make(tmp_path, "ident", _config(layers), seed=9)
    g = torch.Generator().manual_seed(77)
    for i in range(2):
        c = tensors[f"l{i}.mlp.correction"]
        c.copy_(0.04 * torch.randn(c.shape, generator=g))
        c[-2:] += 0.03                             # identity experts that are often chosen, not always
    from picolm_b200.weights import save_safetensors
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    t = random_tokens(80, VOCAB, 4)
    want = _plain(tensors, config, t)
    h = torch.randn(200, 40, dtype=torch.float64)
    ids, _ = P.route(h, {k[len("l0.mlp."):]: v.double() for k, v in tensors.items() if k.startswith("l0.mlp.")}, config["layers"][0]["mlp"]["router"])
    assert 0.2 < (ids >= 5).float().mean() < 0.8
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_batch(eng, [t, t[:9]], [30, 9])[0], want, what="batch")


# ------------------------------------------------------------------------------------------------ bfloat16
@pytest.mark.parametrize("name", ["wide_heads", "serving"])
def test_bfloat16_follows_the_plain_implementation(tmp_path, name):
    """The serving precision stays within rounding of the exact logits, and its own cuts agree with each other far
    more closely than that.  `wide_heads`: head sizes 64 and 128, also for the latent's row (the tcgen05 prompt attention); `serving`: 48, 16 and
    a latent row of 80 (the mma.sync kernels), routed layers whose sizes take the tensor-core products."""
    if name == "wide_heads":
        layers = [_attn(heads=4, kv_heads=2, dim=64, vdim=64, rot=32, chunk=100, scale=0.11, mlp=_moe(experts=6, top=2, ff=64)),
                  _attn2(heads=2, kv_heads=2, dim=128, vdim=128, rot=128, chunk=90, scale=0.09, mlp=_moe(experts=6, top=2, ff=64)),
                  _latent(heads=4, dim=48, rot_dim=32, vdim=80, kv_rank=96, q_rank=72, scale=0.12, mlp=_moe(experts=6, top=2, ff=64))]
    else:
        layers = [_attn(heads=4, kv_heads=2, dim=48, vdim=32, rot=16, chunk=70, scale=0.5, mlp=_moe(experts=6, top=2, ff=64)),
                  _attn2(heads=8, kv_heads=2, dim=16, vdim=16, chunk=33, scale=0.6, mlp=_moe(experts=6, top=2, ff=64)),
                  _latent(heads=4, dim=32, rot_dim=32, vdim=32, kv_rank=48, q_rank=40, scale=0.3, mlp=None),
                  _attn2(heads=8, kv_heads=2, dim=16, vdim=16, chunk=100, scale=0.6, kv_from=1, mlp=_moe(experts=6, top=2, ff=64))]
    d, tensors, config = _make(tmp_path, "bf16" + name, _config(layers, width=128), seed=3, std=0.08)
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


def test_bfloat16_at_sizes_the_tensor_cores_refuse(tmp_path):
    """An odd width and odd head sizes in the serving precision: other kernels, the same logits within rounding."""
    layers, kw = MODELS["odd"]
    d, tensors, config = _make(tmp_path, "bf16odd", _config(layers, **kw), seed=11, std=0.08)
    t = random_tokens(140, VOCAB, 9)
    want = _plain(tensors, config, t)
    eng = _engine(d, dtype="bfloat16")
    whole = run_whole(eng, t)
    rel = ((whole - want).double().pow(2).mean().sqrt() / want.double().std()).item()
    assert rel < 0.05, f"bfloat16 logits are {rel:.3f} of the spread away from the exact ones"
    for got in (run_tail(eng, t, tail=70), run_chunks(eng, t, [64, 2, 74])):
        rel = ((got - whole).double().pow(2).mean().sqrt() / want.double().std()).item()
        assert rel < 0.03, f"two cuts of the same request differ by {rel:.3f} of the spread"


# ---------------------------------------------------------------------------------------------- generation
GEN = [_attn(chunk=6), _attn2(heads=2, kv_heads=1, dim=8, vdim=16, rot=8, chunk=20), _latent(mlp=None),
       _attn2(heads=2, kv_heads=1, dim=8, vdim=16, rot=8, chunk=9, kv_from=1)]


def _greedy(tensors, config, p, n):
    seq, out = list(p), []
    for _ in range(n):
        out.append(int(_plain(tensors, config, seq)[-1].argmax()))
        seq.append(out[-1])
    return out


def test_greedy_generation_through_the_entry_point(tmp_path):
    """`generate` (batch planning, captured decode steps, sampled ids fed back on the device) gives the plain
    implementation's greedy tokens; more requests than fit one batch, so slots and pages are used again."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "gen", _config(GEN), seed=13)
    prompts = [random_tokens(n, VOCAB, 30 + i) for i, n in enumerate([5, 70, 1, 19, 33])]
    want = [_greedy(tensors, config, p, 8) for p in prompts]
    eng = model_load(d, dtype="float32", max_batch=2)
    got, stats = generate(eng, prompts, max_tokens=8, temperature=0.0, stop_ids=[], return_stats=True)
    assert got == want
    assert stats.batches == 3 and eng.cache.slots.used == 0
    assert eng.use_graphs, "decode steps of this design are meant to replay captured graphs"
    eng.cache.check()


def test_bfloat16_generation_with_captured_prompt_steps(tmp_path):
    """In bfloat16 `generate` replays captured graphs for the prompts' step too: every generated token is, by the logits
    of the same prompts launched kernel by kernel, the best or within rounding of it."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "pgraph", _config(GEN, width=64), seed=23, std=0.08)
    prompts = [random_tokens(n, VOCAB, 60 + i) for i, n in enumerate([70, 9, 200])]
    eng = model_load(d, dtype="bfloat16", max_batch=4)
    assert eng.prompt_graphs, "every part of the design declares itself safe for captured prompt steps"
    got = generate(eng, prompts, max_tokens=6, temperature=0.0, stop_ids=[])
    assert eng._prompt_graphs, "the prompts' step was not replayed from a graph"
    plain_eng = _engine(d, dtype="bfloat16", use_graphs=False)
    slots = [plain_eng.new_sequence() for _ in prompts]
    logits = plain_eng.step(list(zip(slots, prompts))).float().cpu()
    for step in range(6):
        for i, row in enumerate(logits):
            tok = got[i][step]
            assert row[tok] >= row.max() - 0.03 * row.std(), f"request {i}, step {step}: graph and single launches disagree"
        logits = plain_eng.step([(s, [got[i][step]]) for i, s in enumerate(slots)]).float().cpu()
    for s in slots:
        plain_eng.end_sequence(s)
    eng.cache.check()


def test_trace_replay_as_a_user_runs_it(tmp_path):
    """bin/trace_run on a Fupapel folder: a batch of unequal prompts, single tokens until the shorter requests end,
    a request alone afterwards in the slot that was given back."""
    from test_gpu_trace_run import Replay
    d, tensors, config = _make(tmp_path, "replay", _config(GEN), seed=17)
    reqs = {f"q{i}": random_tokens(n, VOCAB, 300 + i) for i, n in enumerate([70, 9, 1, 30, 3, 2])}
    ref = {k: _plain(tensors, config, t) for k, t in reqs.items()}
    rp = Replay(d, "float32", str(tmp_path / "out"), max_tokens=128)
    try:
        batch = ["q0", "q1", "q2", "q4", "q5"]
        pos = {"q0": 50, "q1": 4, "q2": 1, "q4": 2, "q5": 1}
        got = rp.send([{"id": k, "tokens": reqs[k][:pos[k]], "want": [pos[k] - 1]} for k in batch],
                      end=[k for k in batch if pos[k] == len(reqs[k])])
        for row, k in enumerate(batch):
            _close(got[row:row + 1], ref[k][pos[k] - 1:pos[k]], what=f"prompt of {k}")
        live = [k for k in batch if pos[k] < len(reqs[k])]
        while live:
            ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
            got = rp.send([{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live], end=ending)
            for row, k in enumerate(live):
                _close(got[row:row + 1], ref[k][pos[k]:pos[k] + 1], what=f"{k} at {pos[k]}")
                pos[k] += 1
            live = [k for k in live if pos[k] < len(reqs[k])]
        got = rp.send([{"id": "again", "tokens": reqs["q3"], "want": [0, 29]}], end=["again"])
        _close(got, ref["q3"][[0, 29]], what="alone, afterwards")
    finally:
        rp.close()


def test_command_line(tmp_path):
    """The library's command line on a Fupapel folder: random weights from a config.json, greedy tokens equal to the
    plain implementation's, sampling, the per-layer benchmark with a row for every layer."""
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = [sys.executable, os.path.join(root, "bin", "picolm_b200")]
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(_config(GEN), f)
    d = str(tmp_path / "model")
    r = subprocess.run(exe + ["--random-weights", cfg_path, "--out", d, "-s", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    tensors = P.read_safetensors(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json")) as f:
        config = json.load(f)
    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0", "--dtype", "float32", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [[int(t) for t in ln.split()] for ln in r.stdout.strip().splitlines()] == [_greedy(tensors, config, [5, 6, 7], 6),
                                                                                    _greedy(tensors, config, [9], 6)]
    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0.8", "-k", "40", "--top-p", "0.9", "-s", "5", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [len(ln.split()) for ln in r.stdout.strip().splitlines()] == [6, 6]
    r = subprocess.run(exe + [d, "-p", "5,6,7,8", "-n", "5", "--benchmark"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [ln.split(",") for ln in r.stderr.splitlines() if re.fullmatch(r"\d+,[0-9.]+,[0-9.]+,[0-9.]+,\d+", ln)]
    assert [int(x[0]) for x in rows] == [0, 1, 2, 3] * 3
    r = subprocess.run(exe + [d, "--list-tensors"], capture_output=True, text=True, timeout=60)
    assert "l1.mlp.correction\t[8]\tBF16" in r.stdout and "l3.mix.k" not in r.stdout and "l3.mix.q.conv" in r.stdout
