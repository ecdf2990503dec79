"""A plain, slow implementation of the Tebasun design: one function per
mechanism, written from the design's equations.  It shares no code with
picolm_b200 (it has its own safetensors reader) and runs on the CPU in float64
or float32.

The design in this file's notation.  `x = embed[token] * c`.  Layers are listed
one by one in config.json; a contiguous range of them runs several times in a
row with the same weights and a state of its own each time (before every pass
but the first the embedding's output is added to x again, and before every pass
a learned vector of that pass).  A layer is `x += mixer(N1(x))`, then, if it has
a feed-forward, `x += ff(N2(x))`, then a per-layer token input
`x += rms(P (gelu(G x) * e_token)) * w`.  N is `tanh(alpha x) * w + b`, elementwise.
Two mixers: a gated diagonal linear recurrence behind a short convolution with
a GELU branch beside it, and a pair of mixers side by side whose results are
added with two constants: softmax attention (biased projections, per-head RMS
norm of q and k, partial rotation in half-split pairs with stretched
frequencies, the unrotated keys serving as values, one extra term in the
softmax's denominator per head) and a gated delta rule (short convolutions,
unit-length q and k, a decay per key channel, a write strength per head).
Final N, logits against the embedding table.

`h` is a sublayer's input [T, width] for ONE sequence whose first row is
position 0; weights are stored [out, in] and applied as `W x`.
"""
import json
import math
import struct

import torch

_ST_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}


def read_safetensors(path):
    """name -> tensor, read with nothing but the file format: 8 bytes of length, a JSON table, the data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        table = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, ent in table.items():
        if name == "__metadata__":
            continue
        a, b = ent["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=_ST_DTYPES[ent["dtype"]])
        out[name] = t.reshape(ent["shape"]).clone()
    return out


# ----------------------------------------------------------------- small pieces
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def tanh_norm(x, w, b, alpha):
    """The design's norm: no statistics at all."""
    return torch.tanh(alpha * x) * w + b


def short_conv(u, taps, bias=None):
    """u [T, C], taps [C, K] with the last column the current token's: out[t, c] = sum_j taps[c, K-1-j] u[t-j, c],
    inputs before the first token being zero."""
    T, C = u.shape
    K = taps.shape[1]
    out = torch.zeros_like(u)
    for j in range(K):
        if j < T:
            out[j:] += u[:T - j] * taps[:, K - 1 - j]
    if bias is not None:
        out = out + bias
    return out


# ------------------------------------------------------------- rotary positions
def stretched_frequencies(dims, base, scaling, dtype=torch.float64):
    """(frequencies [dims/2], amplitude): f_i = base^(-2i/dims); with `scaling` (factor, original, fast, slow) the
    slow frequencies are divided by factor, blended over a ramp in the index i, and cos and sin are multiplied by
    0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = torch.as_tensor(float(base), dtype=dtype) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half_split(x, positions, dims, freq, amplitude):
    """x [T, heads, size]: component i < dims/2 of every head is paired with component i + dims/2 and the pair is
    turned by position * freq[i]; cos and sin carry `amplitude`; components from `dims` on stay."""
    out = x.clone()
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    c, s = (ang.cos() * amplitude)[:, None, :], (ang.sin() * amplitude)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# --------------------------------------------------------------------- mixers
def softmax_with_sink(scores, sink):
    """scores [H, T, S] (minus infinity where masked), sink [H]: exp(score) / (sum exp(score) + exp(sink))."""
    m = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def sink_attention(h, w, m, eps, prefix):
    """The softmax mixer.  m: heads, kv_heads, dim, vdim, rot{base, dims, scaling}, scale."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, D)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, D)
    v = k                                                    # the keys as projected serve as values
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    rot = m.get("rot")
    if rot and rot["dims"] > 0:
        freq, amp = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        pos = list(range(T))
        q = rotate_half_split(q, pos, rot["dims"], freq, amp)
        k = rotate_half_split(k, pos, rot["dims"], freq, amp)
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1).permute(1, 0, 2)    # [H, T, D]
    vv = v.repeat_interleave(rep, dim=1).permute(1, 0, 2)
    scores = torch.einsum("thd,hsd->hts", q, kk) * m["scale"]
    causal = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    scores = scores.masked_fill(~causal[None], float("-inf"))
    p = softmax_with_sink(scores, w[prefix + "sink"])
    ctx = torch.einsum("hts,hsd->thd", p, vv).reshape(T, H * D)
    return ctx @ w[prefix + "o"].T + w[prefix + "o.b"]


def delta_rule(q, k, v, g, beta):
    """Per head.  q, k [T, N], v [T, P], g [T, N] in (0, 1], beta [T]: S <- diag(g_t) S; u = beta_t (v_t - S^T k_t);
    S <- S + k_t u^T; o_t = S^T q_t.  Returns o [T, P]."""
    T, N = k.shape
    P = v.shape[1]
    S = torch.zeros(N, P, dtype=q.dtype)
    out = torch.zeros(T, P, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def gated_delta(h, w, m, eps, prefix):
    """The delta-rule mixer.  m: heads, kv_heads, dim, vdim, conv."""
    T = h.shape[0]
    H, G, N, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ w[prefix + "q"].T, w[prefix + "q.conv"])).view(T, G, N)
    k = silu(short_conv(h @ w[prefix + "k"].T, w[prefix + "k.conv"])).view(T, G, N)
    v = silu(short_conv(h @ w[prefix + "v"].T, w[prefix + "v.conv"])).view(T, H, P)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * N ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[prefix + "b"].T)                                                 # [T, H]
    dt = softplus((h @ w[prefix + "a1"].T) @ w[prefix + "a2"].T + w[prefix + "dt_bias"]).view(T, H, N)
    g = torch.exp(-torch.exp(w[prefix + "A_log"])[None, :, None] * dt)                           # [T, H, N]
    gate = torch.sigmoid((h @ w[prefix + "g1"].T) @ w[prefix + "g2"].T).view(T, H, P)
    rep = H // G
    heads = []
    for hh in range(H):
        o = delta_rule(q[:, hh // rep], k[:, hh // rep], v[:, hh], g[:, hh], beta[:, hh])
        heads.append(rms_norm(o, w[prefix + "norm"], eps) * gate[:, hh])
    return torch.cat(heads, dim=-1) @ w[prefix + "o"].T


def parallel_mixer(h, w, m, eps, prefix):
    return (m["left_scale"] * sink_attention(h, w, m["left"], eps, prefix + "left.")
            + m["right_scale"] * gated_delta(h, w, m["right"], eps, prefix + "right."))


def diagonal_recurrence(a, b):
    """S_t = a_t S_(t-1) + b_t from S = 0, elementwise; [T, C]."""
    S = torch.zeros_like(a[0])
    out = torch.zeros_like(a)
    for t in range(a.shape[0]):
        S = a[t] * S + b[t]
        out[t] = S
    return out


def gated_recurrent(h, w, m, prefix):
    """The recurrent mixer.  m: width, blocks, conv."""
    T = h.shape[0]
    B = m["blocks"]
    y = gelu_tanh(h @ w[prefix + "y"].T + w[prefix + "y.b"])
    u = short_conv(h @ w[prefix + "x"].T + w[prefix + "x.b"], w[prefix + "conv"], w[prefix + "conv.b"])
    ub = u.view(T, B, -1)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[prefix + "ra"]) + w[prefix + "ra.b"]).reshape(T, -1)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[prefix + "ri"]) + w[prefix + "ri.b"]).reshape(T, -1)
    log_a = -8.0 * r * softplus(w[prefix + "lam"])
    a = torch.exp(log_a)
    S = diagonal_recurrence(a, torch.sqrt(1.0 - a * a) * i * u)
    return (S * y) @ w[prefix + "o"].T


# ----------------------------------------------------------------- the rest
def dense_ff(h, w, prefix):
    return (silu(h @ w[prefix + "gate"].T) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def token_side(x, tokens, w, layer, dim, eps):
    """What a layer adds from the token itself: columns [layer dim, (layer + 1) dim) of the side table."""
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[f"l{layer}.side.gate"].T) * e) @ w[f"l{layer}.side.proj"].T
    return rms_norm(y, w[f"l{layer}.side.norm"], eps)


def layer_order(cfg):
    """[(layer, pass or None)] in the order the layers run; `pass` is set at a pass's first layer."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t if i == loop["start"] else None))
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  `layers_out`: a list that receives x after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = w["embed"][tokens] * cfg["embedding"]["scale"]
    x = x0.clone()

    def norm(name):
        return tanh_norm(x, w[name], w[name + ".b"], w[name + ".alpha"])

    for i, t in layer_order(cfg):
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        layer = cfg["layers"][i]
        p = f"l{i}.mix."
        if layer["type"] == "rglru":
            x = x + gated_recurrent(norm(f"l{i}.norm1"), w, layer["mixer"], p)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(norm(f"l{i}.norm1"), w, layer["mixer"], eps, p)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + dense_ff(norm(f"l{i}.norm2"), w, f"l{i}.mlp.")
        if cfg.get("token_side"):
            x = x + token_side(x, tokens, w, i, cfg["token_side"]["dim"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return tanh_norm(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"]) @ w["embed"].T
