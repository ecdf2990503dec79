"""A plain, slow implementation of the Fupapel design: one function per
mechanism, written from the design's equations.  It shares no code with
picolm_b200 (it has its own safetensors reader) and runs on the CPU in float64
or float32.

The design in this file's notation.  `x = embed[token]`; layers listed one by one
in config.json, each `x += m (mixer(shift(N1(x))) + ff(N2(x)))` with both norms
reading the same x, `N(x) = x / sqrt(mean(x^2) + eps) (1 + w)`, m one number for
the model, and `shift(h)_t = h_t + (h_(t-1) - h_t) * mu` elementwise (h_(-1) = 0):
only the mixer reads the shifted rows.  Three mixers.  `attention`: grouped
heads, an RMS norm over the whole of q and of k, a rotation of the leading
components of every head in half-split pairs, a mask of chunks, a softmax whose
denominator holds one more 1, the heads times `sigmoid(W_g h)` elementwise.
`attention_2`: a short causal convolution over time on q, k and v straight after
the projections, the same norm and rotation (frequencies optionally stretched by
the three-band rule), a factor per head on the scores, a learned term
`exp(sink_h)` in the denominator, optionally the keys and values of an earlier
layer.  `latent_attention`: queries through a normed latent, keys and values as
per-head maps of one normed latent row per position, one rotated key part shared
by the heads, a learned sink, each head times one sigmoid gate.  The feed-forward
routes every token to `top` of the experts by softmax scores over experts and
identity experts together (a correction added for the choice only, groups kept
by their best choice score, weights not renormalised; an identity expert hands
back its input).  Final norm of the same kind, logits against `head`.

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
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def one_plus_norm(x, w, eps):
    """The layers' norm: the weight is stored around zero."""
    return rms_norm(x, 1.0 + w, eps)


def silu(z):
    return z * torch.sigmoid(z)


def token_shift(h, mu, before=None):
    """h_t + (h_(t-1) - h_t) * mu; the row before the first is `before` (zeros at a sequence's start)."""
    prev = torch.zeros_like(h)
    prev[1:] = h[:-1]
    if before is not None:
        prev[0] = before
    return h + (prev - h) * mu


def short_conv(u, w, before=None):
    """y_t = sum_j w[:, j] u_(t - taps + 1 + j) per channel; u [T, C], w [C, taps]; `before` [taps - 1, C] are the
    inputs in front of the first row (zeros at a sequence's start)."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.zeros(taps - 1, C, dtype=u.dtype) if before is None else before
    full = torch.cat([pad, u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + full[j:j + T] * w[:, j]
    return y


def stretched_frequencies(dims, base, scaling=None):
    """base^(-2i/dims), i < dims/2, as Python floats; with `scaling` {factor, low, high, original}: a frequency
    whose wavelength is under original/high stays, over original/low is divided by factor, and between them is
    blended linearly in original/wavelength."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_halves(x, positions, dims, base, scaling=None):
    """x [T, heads, size]: component i < dims/2 of every head is paired with component i + dims/2 and the pair
    turned by position * f_i; components from `dims` on stay."""
    out = x.clone()
    half = dims // 2
    freq = torch.tensor(stretched_frequencies(dims, base, scaling), dtype=torch.float64)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * freq[None, :]
    c, s = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def visible(T, chunk=None):
    """[T, T] True where query i sees key j: j <= i and, with `chunk`, both in the same chunk of that many
    positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk is not None:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_with_sink(s, mask, sink):
    """p_j = exp(s_j) / (exp(sink) + sum over visible j of exp(s_j)) for scores s [T, T]."""
    s = s.masked_fill(~mask, float("-inf"))
    top = torch.maximum(s.max(dim=-1, keepdim=True).values, torch.as_tensor(sink, dtype=s.dtype))
    e = torch.exp(s - top)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(torch.as_tensor(sink, dtype=s.dtype) - top))


def _rot(m):
    r = m.get("rot")
    return None if r is None else (int(r["dims"]), float(r["base"]), r.get("scaling"))


def _chunk(m):
    return None if m.get("mask") is None else int(m["mask"]["size"])


# --------------------------------------------------------------------- attention
def attention_keys_values(h, W, m, eps, convolved):
    """What an attention layer keeps: keys after (convolution,) norm and rotation [T, G, dim], values after
    (convolution) [T, G, vdim]."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k, v = h @ W["k"].T, h @ W["v"].T
    if convolved:
        k, v = short_conv(k, W["k.conv"]), short_conv(v, W["v.conv"])
    k = rms_norm(k, W["k.norm"], eps).reshape(T, G, D)
    if _rot(m) is not None:
        k = rotate_halves(k, list(range(T)), *_rot(m))
    return k, v.reshape(T, G, Dv)


def _heads_over_keys(q, k, v, scale, mask, sinks, temps=None):
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * scale
        if temps is not None:
            s = s * temps[head]
        out[:, head, :] = softmax_with_sink(s, mask, sinks[head]) @ v[:, g, :]
    return out


def attention(h, W, m, eps):
    """The mixer `attention`: a sink of score 0 in every head's softmax, and an elementwise sigmoid gate on the heads."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    q = rms_norm(h @ W["q"].T, W["q.norm"], eps).reshape(T, H, D)
    if _rot(m) is not None:
        q = rotate_halves(q, list(range(T)), *_rot(m))
    k, v = attention_keys_values(h, W, m, eps, convolved=False)
    heads = _heads_over_keys(q, k, v, m["scale"], visible(T, _chunk(m)), [0.0] * H)
    return (heads.reshape(T, -1) * torch.sigmoid(h @ W["g"].T)) @ W["o"].T


def attention_2(h, W, m, eps, keys_values=None):
    """The mixer `attention_2`.  `keys_values`: another layer's (keys, values) for a layer that has none of its own."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    q = short_conv(h @ W["q"].T, W["q.conv"])
    q = rms_norm(q, W["q.norm"], eps).reshape(T, H, D)
    if _rot(m) is not None:
        q = rotate_halves(q, list(range(T)), *_rot(m))
    k, v = keys_values if keys_values is not None else attention_keys_values(h, W, m, eps, convolved=True)
    heads = _heads_over_keys(q, k, v, m["scale"], visible(T, _chunk(m)), W["sink"], W["temp"])
    return heads.reshape(T, -1) @ W["o"].T


def latent_attention(h, W, m, eps):
    """The mixer `latent_attention`, with every key and value made as the equations say."""
    T = h.shape[0]
    H, D, R, Dv, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = list(range(T))
    q = (rms_norm(h @ W["dq"].T, W["dq.norm"], eps) @ W["uq"].T).reshape(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate_halves(q[..., D:], pos, R, m["rot"]["base"], m["rot"].get("scaling"))
    down = h @ W["dkv"].T
    c = rms_norm(down[:, :L], W["dkv.norm"], eps)
    k_rot = rotate_halves(down[:, None, L:], pos, R, m["rot"]["base"], m["rot"].get("scaling"))[:, 0, :]
    k_plain = (c @ W["uk"].T).reshape(T, H, D)
    v = (c @ W["uv"].T).reshape(T, H, Dv)
    gate = torch.sigmoid(h @ W["g"].T)                               # [T, H]
    mask = visible(T, _chunk(m))
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        out[:, head] = (softmax_with_sink(s, mask, W["sink"][head]) @ v[:, head]) * gate[:, head:head + 1]
    return out.reshape(T, -1) @ W["o"].T


# ------------------------------------------------------------------ feed-forward
def route(h, W, r):
    """(ids [T, top], weights [T, top]) over experts and identity experts together (the identity experts are the
    last `identity` of the router's outputs)."""
    n_out = int(r["experts"]) + int(r.get("identity", 0))
    top = int(r["top"])
    s = torch.softmax(h @ W["router"].T, dim=-1)                      # [T, n_out]
    choice = s + W["correction"]
    if r.get("groups") is not None:
        count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
        per = n_out // count
        best = choice.reshape(-1, count, per).max(dim=-1).values      # [T, count]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    return ids, torch.gather(s, 1, ids)


def routed_feed_forward(h, W, mlp):
    r = mlp["router"]
    E = int(r["experts"])
    ids, weights = route(h, W, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t].tolist(), weights[t]):
            if e >= E:
                y = h[t]                                              # an identity expert
            else:
                y = (silu(h[t] @ W[f"e{e}.gate"].T) * (h[t] @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
            out[t] = out[t] + w * y
    return out


# ------------------------------------------------------------------------- model
def _sub(tensors, prefix, dtype):
    n = len(prefix)
    return {k[n:]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence from its first token on; with `return_layers` also the stream after
    every layer [layers, T, width]."""
    eps, mult = float(config["norm"]["eps"]), float(config["residual_mult"])
    x = tensors["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        W = _sub(tensors, f"l{i}.mix.", dtype)
        h = token_shift(one_plus_norm(x, tensors[f"l{i}.norm1"].to(dtype), eps), tensors[f"l{i}.shift"].to(dtype))
        if layer["type"] == "attention":
            delta = attention(h, W, m, eps)
        elif layer["type"] == "attention_2":
            if m.get("kv_from") is not None:
                delta = attention_2(h, W, m, eps, keys_values=kept[int(m["kv_from"])])
            else:
                kept[i] = attention_keys_values(h, W, m, eps, convolved=True)
                delta = attention_2(h, W, m, eps, keys_values=kept[i])
        elif layer["type"] == "latent_attention":
            delta = latent_attention(h, W, m, eps)
        else:
            raise ValueError(f"no mixer of type {layer['type']!r}")
        if layer.get("mlp") is not None:
            h2 = one_plus_norm(x, tensors[f"l{i}.norm2"].to(dtype), eps)
            delta = delta + routed_feed_forward(h2, _sub(tensors, f"l{i}.mlp.", dtype), layer["mlp"])
        x = x + mult * delta
        after.append(x)
    logits = one_plus_norm(x, tensors["final.norm"].to(dtype), eps) @ tensors["head"].to(dtype).T
    return (logits, torch.stack(after)) if return_layers else logits


def load_model(folder):
    with open(f"{folder}/config.json", "r", encoding="utf-8") as f:
        config = json.load(f)
    return config, read_safetensors(f"{folder}/model.safetensors")
