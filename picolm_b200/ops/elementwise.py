"""Embedding, RMSNorm, SwiGLU, rotary encoding with the cache write."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import PAGE_TOKENS, KernelError, _check, _dev, _dt, _fn, _i32, _p, _stream, set_bounds


def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = float(table[tokens[t], :]) * scale as the fp32 residual stream."""
    _i32(tokens, "tokens")
    _dev(table, "table")
    n, (vocab, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, d), dtype=torch.float32, device=table.device)
    _check(_fn("elementwise", "plm_embed")(_p(tokens), _p(table), _dt(table, "table"), _p(out), n, d, vocab, float(scale),
                                           _stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of the fp32 stream `x` [T, d].  With `delta` the sum x + delta is
    normalised and, unless `rows` gathers, written back to x.  `rows` (int32)
    picks the source rows; the output then has len(rows) rows."""
    _dev(x, "x")
    _dev(weight, "weight")
    if x.dtype != torch.float32:
        raise KernelError("the residual stream must be float32")
    T, d = x.shape
    if weight.shape != (d,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, the stream is {d} wide")
    if hasattr(delta, "compute"):                          # a product that has not run yet (gemm.PendingLinear)
        if rows is None and delta.adds_in_place(x):        # many rows: the add in the product's epilogue
            delta.add_into(x)
            delta = None
        else:
            delta = delta.compute()
    if delta is not None:
        _dev(delta, "delta")
        if delta.dtype != torch.float32 or delta.shape != x.shape:
            raise KernelError("delta must be float32 and shaped like x")
    n_rows = T
    if rows is not None:
        _i32(rows, "rows")
        n_rows = rows.numel()
    if out is None:
        out = torch.empty((n_rows, d), dtype=out_dtype, device=x.device)
    set_bounds("elementwise", n_rows=T, device=x.device)
    _check(_fn("elementwise", "plm_rmsnorm")(
        _p(x), _p(delta), _p(weight), _dt(weight, "weight"), _p(out), _dt(out, "out"), _p(rows), n_rows, d,
        float(eps), _stream()), f"rmsnorm rows={n_rows} d={d}",
        nbytes=n_rows * d * (4 + (8 if delta is not None else 0) + out.element_size()))
    return out


def post_pre_norm_supported(x: torch.Tensor, delta, w_post: torch.Tensor, w_pre: torch.Tensor) -> bool:
    """Whether `post_pre_norm` takes this case: float32 stream and delta of one shape, rows of a multiple of 4 and at
    most 16,384 columns, two norm weights of one type."""
    return (isinstance(delta, torch.Tensor) and delta.dtype == torch.float32 and x.dtype == torch.float32
            and delta.shape == x.shape and x.is_contiguous() and delta.is_contiguous() and x.shape[1] % 4 == 0
            and x.shape[1] <= 16384 and w_post.dtype == w_pre.dtype and w_post.shape == w_pre.shape == (x.shape[1],)
            and x.data_ptr() % 16 == 0 and delta.data_ptr() % 16 == 0)


def post_pre_norm(x: torch.Tensor, delta: torch.Tensor, w_post: torch.Tensor, eps_post: float, w_pre: torch.Tensor,
                  eps_pre: float, out_dtype: torch.dtype) -> torch.Tensor:
    """x += RMSNorm(delta; w_post) in place on the fp32 stream, and RMSNorm(x; w_pre) of the new x as [T, d] of
    `out_dtype`: a sublayer's closing norm, the residual add and the next sublayer's opening norm in one kernel."""
    _dev(x, "x"), _dev(delta, "delta"), _dev(w_post, "w_post"), _dev(w_pre, "w_pre")
    if not post_pre_norm_supported(x, delta, w_post, w_pre):
        raise KernelError("post_pre_norm: not a case the fused kernel takes")
    T, d = x.shape
    out = torch.empty((T, d), dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "plm_post_pre_norm")(
        _p(x), _p(delta), _p(w_post), _p(w_pre), _dt(w_pre, "w_pre"), _p(out), _dt(out, "out"), T, d, float(eps_post),
        float(eps_pre), _stream()), f"post_pre_norm rows={T} d={d}", nbytes=T * d * (12 + out.element_size()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """x[rows] for a 2-D `x` with contiguous rows and int32 `rows` on the device: [len(rows), x.shape[1]]."""
    _i32(rows, "rows")
    if not x.is_cuda:
        raise KernelError(f"x is on {x.device}; picolm_b200 kernels run on a CUDA device only")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gather_rows takes a matrix with contiguous rows")
    n, d = rows.numel(), x.shape[1]
    out = torch.empty((n, d), dtype=x.dtype, device=x.device)
    set_bounds("elementwise", n_rows=x.shape[0], device=x.device)
    _check(_fn("elementwise", "plm_gather_rows")(_p(x), _p(out), _p(rows), n, d * x.element_size(),
                                                x.stride(0) * x.element_size(), _stream()),
           f"gather_rows {n} of {x.shape[0]}", nbytes=2 * n * d * x.element_size())
    return out


# "swish_clamped": g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(slope g') (u' + 1); its two constants
# are arguments of `swiglu`
GATE_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, activation: str = "silu", limit: float = 0.0,
           slope: float = 1.0) -> torch.Tensor:
    """gate_up [T, 2F] (gate columns first) -> act(gate) * up, [T, F]; `activation` "silu" or "gelu_tanh"
    (the reference's two: picolm/tensor.c:3306-3323)."""
    _dev(gate_up, "gate_up")
    if activation not in GATE_ACTIVATIONS:
        raise KernelError(f"activation {activation!r} has no kernel; known: {', '.join(GATE_ACTIVATIONS)}")
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError("gate_up must have an even number of columns")
    if out is None:
        out = torch.empty((T, F2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    _check(_fn("elementwise", "plm_swiglu")(_p(gate_up), _p(out), _dt(gate_up, "gate_up"),
                                            GATE_ACTIVATIONS[activation], T, F2 // 2, float(limit), float(slope),
                                            _stream()), "swiglu")
    return out


def rope_store(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
               tok_pos: torch.Tensor, tok_seq: torch.Tensor, block_table: torch.Tensor,
               num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int, pairing: str,
               store: bool = True) -> None:
    """Rotate the query and key heads of `qkv` [T, (H+2G)*hd] by their tokens'
    positions; write queries to `q_out` [T, H, hd] and keys/values into the paged
    cache [pages, G, PAGE_TOKENS, hd]."""
    _dev(qkv, "qkv")
    _dev(q_out, "q_out")
    _i32(tok_pos, "tok_pos"), _i32(tok_seq, "tok_seq"), _i32(block_table, "block_table")
    T = qkv.shape[0]
    H, G, hd = num_heads, num_kv_heads, head_dim
    if qkv.shape[1] != (H + 2 * G) * hd or q_out.shape != (T, H, hd) or q_out.dtype != qkv.dtype:
        raise KernelError("rope_store: qkv / q_out shapes do not match the head counts")
    if store:
        for c, n in ((k_cache, "k_cache"), (v_cache, "v_cache")):
            _dev(c, n)
            if c.dtype != q_out.dtype or c.shape[1:] != (G, PAGE_TOKENS, hd):
                raise KernelError(f"rope_store: {n} must be [pages, {G}, {PAGE_TOKENS}, {hd}] of {q_out.dtype}")
    if cos is not None:
        _dev(cos, "cos"), _dev(sin, "sin")
        if cos.dtype != torch.float32 or cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rope_store: cos/sin tables must be float32 [positions, rotary_dim/2]")
    if pairing not in ("half", "adjacent"):
        raise KernelError(f"rope_store: unknown pairing {pairing!r}")
    set_bounds("elementwise", n_pages=k_cache.shape[0] if store else 0, n_seqs=block_table.shape[0],
               n_positions=block_table.shape[1] * PAGE_TOKENS, device=qkv.device)
    _check(_fn("elementwise", "plm_rope_store")(
        _p(qkv), _p(q_out), _p(k_cache) if store else None, _p(v_cache) if store else None, _dt(qkv, "qkv"),
        _p(cos), _p(sin), _p(tok_pos), _p(tok_seq), _p(block_table), block_table.shape[1], T, H, G, hd,
        rotary_dim, 0 if pairing == "half" else 1, 1 if store else 0, _stream()), "rope_store")


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
              delta: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Layer norm with a weight and no bias of the fp32 stream `x` [T, d]: `(v - mean) / sqrt(var + eps) * w`.  With
    `delta` (fp32 [T, d], or a product that has not run) and / or `bias` (fp32 [d], a projection's bias that its product
    left out) v = x + delta + bias, written back to x unless `rows` gathers.  `rows` (int32) picks the source rows."""
    _dev(x, "x"), _dev(weight, "weight")
    if x.dtype != torch.float32:
        raise KernelError("the residual stream must be float32")
    T, d = x.shape
    if weight.shape != (d,):
        raise KernelError(f"norm weight has shape {tuple(weight.shape)}, the stream is {d} wide")
    if hasattr(delta, "compute"):                          # a product that has not run yet (gemm.PendingLinear)
        if rows is None and delta.adds_in_place(x):        # many rows: the add in the product's epilogue
            delta.add_into(x)
            delta = None
        else:
            delta = delta.compute()
    if delta is not None:
        _dev(delta, "delta")
        if delta.dtype != torch.float32 or delta.shape != x.shape:
            raise KernelError("delta must be float32 and shaped like x")
    if bias is not None:
        _dev(bias, "bias")
        if bias.dtype != torch.float32 or bias.shape != (d,):
            raise KernelError("bias must be float32 [d]")
    n_rows = T
    if rows is not None:
        _i32(rows, "rows")
        n_rows = rows.numel()
    out = torch.empty((n_rows, d), dtype=out_dtype, device=x.device)
    set_bounds("elementwise", n_rows=T, device=x.device)
    _check(_fn("elementwise", "plm_layernorm")(
        _p(x), _p(delta), _p(bias), _p(weight), _dt(weight, "weight"), _p(out), _dt(out, "out"), _p(rows), n_rows, d,
        float(eps), _stream()), f"layernorm rows={n_rows} d={d}",
        nbytes=n_rows * d * (4 + (8 if delta is not None or bias is not None else 0) + out.element_size()))
    return out


def add_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, d] += bias [d] in place, both float32; returns x."""
    _dev(x, "x"), _dev(bias, "bias")
    if x.dtype != torch.float32 or bias.dtype != torch.float32 or x.dim() != 2 or bias.shape != (x.shape[1],):
        raise KernelError("add_bias takes float32 rows [T, d] and a float32 bias [d]")
    _check(_fn("elementwise", "plm_add_bias")(_p(x), _p(bias), x.shape[0], x.shape[1], _stream()), "add_bias",
           nbytes=2 * x.numel() * 4)
    return x


def qk_norm_rope_store(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor],
                       k_norm: Optional[torch.Tensor], eps: float, q_out: torch.Tensor, kv, rotation, step,
                       num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, own_kv: bool = True,
                       per_head: bool = False, values_from_keys: bool = False,
                       q_scale: Optional[torch.Tensor] = None, conv: Optional[torch.Tensor] = None,
                       conv_state: Optional[torch.Tensor] = None) -> None:
    """What stands between a QKV product and attention where queries and keys are normalised over all their heads at
    once: per token, in fp32, `q + bias` and `k + bias` are divided by their root mean square over ALL their columns
    and multiplied by `q_norm` / `k_norm` (None: no norm), the leading `rotation.rotary_dim` components of every head
    are rotated by the token's position, `v + bias` passes.  `qkv` [T, H*D (+ G*D + G*Dv)] float32 or the run's type;
    queries go to `q_out` [T, H, hd_c], keys and values (`own_kv`) into the pages of `kv` (a `KVLayerCache` whose
    head size hd_c >= D, Dv: what lies beyond a head's own width is written as zero).  `rotation`: `ops.Rotation` or
    None.  `per_head`: the root mean square is taken over each head's own D columns, and `q_norm` / `k_norm` are [D],
    serving every head.  `values_from_keys`: qkv holds no values; `k + bias` as projected, before norm and rotation,
    is written as the value (Dv = D).  `qkv` may be the leading columns of a wider matrix (a slice with contiguous
    rows).  `q_scale` (float32 [H]): head h's queries times q_scale[h] after norm and rotation, a factor per head on
    its scores.  `conv` (float32 [taps, columns of qkv], tap-major, the token's own tap last; no bias with it): every
    column is first convolved over time with the sequence's projected rows before; `conv_state` (float32 [slots + 1,
    >= (taps - 1) * columns], contiguous rows) holds every sequence's last taps - 1 projected rows, oldest first, and
    is brought up to date."""
    if not qkv.is_cuda or qkv.dim() != 2 or qkv.stride(1) != 1:
        raise KernelError("qk_norm_rope_store: qkv must be a matrix with contiguous rows on the device")
    _dev(q_out, "q_out")
    _i32(step.tok_pos, "tok_pos"), _i32(step.tok_seq, "tok_seq"), _i32(kv.block_table, "block_table")
    T = qkv.shape[0]
    H, G, D, Dv = num_heads, num_kv_heads, key_dim, value_dim
    hd_c = q_out.shape[2]
    if values_from_keys and (Dv != D or not own_kv):
        raise KernelError("qk_norm_rope_store: keys that serve as values need value_dim == key_dim and keys of the layer's own")
    cols = H * D + ((G * D + (0 if values_from_keys else G * Dv)) if own_kv else 0)
    if qkv.shape != (T, cols) or q_out.shape != (T, H, hd_c):
        raise KernelError("qk_norm_rope_store: qkv / q_out shapes do not match the head counts")
    if own_kv:
        for c, n in ((kv.k, "k_cache"), (kv.v, "v_cache")):
            _dev(c, n)
            if c.dtype != q_out.dtype or c.shape[1:] != (G, PAGE_TOKENS, hd_c):
                raise KernelError(f"qk_norm_rope_store: {n} must be [pages, {G}, {PAGE_TOKENS}, {hd_c}] of {q_out.dtype}")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (cols,) or not bias.is_cuda):
        raise KernelError("qk_norm_rope_store: bias must be float32, one per column of qkv")
    _f32_vec(q_scale, "q_scale", H)
    taps, lds = 0, 0
    if conv is not None:
        _dev(conv, "conv")
        taps = conv.shape[0]
        if conv.dtype != torch.float32 or conv.shape != (taps, cols) or bias is not None:
            raise KernelError(f"qk_norm_rope_store: the convolution's taps must be float32 [taps, {cols}], and no bias with them")
        if taps > 1:
            if conv_state is None or not conv_state.is_cuda or conv_state.dtype != torch.float32 or conv_state.dim() != 2 \
                    or conv_state.stride(1) != 1 or conv_state.shape[1] < (taps - 1) * cols:
                raise KernelError("qk_norm_rope_store: the convolution needs a float32 state [slots, >= (taps - 1) * columns]")
            lds = conv_state.stride(0)
            set_bounds("elementwise", n_seqs=step.n_seqs, device=qkv.device)
        else:
            conv_state = None
    for wn, n, size in ((q_norm, "q_norm", D if per_head else H * D), (k_norm if own_kv else None, "k_norm", D if per_head else G * D)):
        if wn is not None and (wn.dtype != q_out.dtype or wn.shape != (size,) or not wn.is_cuda):
            raise KernelError(f"qk_norm_rope_store: {n} must be [{size}] of {q_out.dtype}")
    cos = sin = None
    rot, pairing = 0, "half"
    if rotation is not None and rotation.cos is not None:
        cos, sin, rot, pairing = rotation.cos, rotation.sin, rotation.rotary_dim, rotation.pairing
        if cos.dtype != torch.float32 or cos.shape[1] != rot // 2 or sin.shape != cos.shape:
            raise KernelError("qk_norm_rope_store: cos/sin tables must be float32 [positions, rotary_dim/2]")
        if step.max_position >= cos.shape[0]:
            raise KernelError(f"position {step.max_position} lies beyond the rotary table")
    set_bounds("elementwise", n_pages=kv.k.shape[0] if own_kv else 0, n_seqs=kv.block_table.shape[0],
               n_positions=kv.block_table.shape[1] * PAGE_TOKENS, device=qkv.device)
    _check(_fn("elementwise", "plm_qk_norm_rope_store")(
        _p(qkv), _dt(qkv, "qkv"), _p(bias), _p(q_norm), _p(k_norm) if own_kv else None, float(eps), _p(q_out),
        _p(kv.k) if own_kv else None, _p(kv.v) if own_kv else None, _dt(q_out, "q_out"), _p(cos), _p(sin),
        _p(step.tok_pos), _p(step.tok_seq), _p(kv.block_table), kv.block_table.shape[1], T, H, G, D, Dv, hd_c, rot,
        0 if pairing == "half" else 1, 1 if own_kv else 0, 1 if per_head else 0, 1 if values_from_keys else 0,
        qkv.stride(0), _p(q_scale), _p(conv), taps, _p(conv_state) if conv is not None else None, lds,
        _p(step.seq_start) if conv is not None else None, _p(step.seq_slot) if conv is not None else None,
        step.n_seqs if conv is not None else 0, 1 if conv is not None and step.is_decode else 0, _stream()),
        f"qk_norm_rope_store T={T}", kernels=2 if conv is not None and taps > 1 and not (step.is_decode and step.n_seqs == T) else 1,
        nbytes=qkv.numel() * qkv.element_size() + T * (H + (2 * G if own_kv else 0)) * hd_c * q_out.element_size())


def _f32_vec(t: Optional[torch.Tensor], name: str, d: int) -> None:
    if t is not None and (not t.is_cuda or t.dtype != torch.float32 or t.shape != (d,) or not t.is_contiguous()):
        raise KernelError(f"{name} must be float32 [{d}] on the device")


def dyt_norm(x: torch.Tensor, out_dtype: Optional[torch.dtype], alpha: Optional[torch.Tensor] = None,
             weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, delta=None,
             delta_bias: Optional[torch.Tensor] = None, post_weight: Optional[torch.Tensor] = None, post_eps: float = 0.0,
             extra: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """The norm without statistics on the fp32 stream `x` [T, d]: `tanh(alpha v) * weight + bias` elementwise, with
    `v = x + delta' + delta_bias + extra`.  `delta` (fp32 [T, d], or a product that has not run) enters as it is, or,
    with `post_weight` (fp32 [d]), divided by its own root mean square (`post_eps` inside the root) and multiplied
    by post_weight; `delta_bias` is a vector [d], `extra` more rows [T, d], all float32.  v is written back to x
    unless `rows` (int32) gathers.  alpha [1], weight, bias [d] float32.  Without `alpha` the result is v itself in
    `out_dtype`; with `out_dtype` None nothing but the sum is made (returns None)."""
    _dev(x, "x")
    if x.dtype != torch.float32:
        raise KernelError("the residual stream must be float32")
    T, d = x.shape
    if hasattr(delta, "compute"):
        if rows is None and post_weight is None and delta.adds_in_place(x):
            delta.add_into(x)
            delta = None
        else:
            delta = delta.compute()
    for t, n in ((delta, "delta"), (extra, "extra")):
        if t is not None:
            _dev(t, n)
            if t.dtype != torch.float32 or t.shape != x.shape:
                raise KernelError(f"{n} must be float32 and shaped like x")
    _f32_vec(delta_bias, "delta_bias", d), _f32_vec(post_weight, "post_weight", d)
    if alpha is not None:
        _f32_vec(weight, "weight", d), _f32_vec(bias, "bias", d)
        if weight is None or bias is None or not alpha.is_cuda or alpha.dtype != torch.float32 or alpha.numel() != 1:
            raise KernelError("dyt_norm: alpha must be one float32 on the device, with a weight and a bias")
    if post_weight is not None and delta is None:
        raise KernelError("dyt_norm: post_weight without a delta")
    n_rows = T
    if rows is not None:
        _i32(rows, "rows")
        n_rows = rows.numel()
    out = None if out_dtype is None else torch.empty((n_rows, d), dtype=out_dtype, device=x.device)
    if out is None and (rows is not None or (delta is None and delta_bias is None and extra is None)):
        return None
    set_bounds("elementwise", n_rows=T, device=x.device)
    n_in = 1 + sum(t is not None for t in (delta, extra))
    _check(_fn("elementwise", "plm_dyt_norm")(
        _p(x), _p(delta), _p(delta_bias), _p(post_weight), float(post_eps), _p(extra), _p(alpha), _p(weight), _p(bias),
        _p(out), _dt(out, "out") if out is not None else 0, _p(rows), n_rows, d, _stream()), f"dyt_norm rows={n_rows} d={d}",
        nbytes=n_rows * d * (4 * n_in + (4 if n_in > 1 and rows is None else 0) + (out.element_size() if out is not None else 0)))
    return out


def add_rows(x: torch.Tensor, a: Optional[torch.Tensor] = None, b: Optional[torch.Tensor] = None,
             vec: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, d] += a + b + vec in place (float32; a, b rows like x, vec [d]; each may be None); returns x."""
    _dev(x, "x")
    if x.dtype != torch.float32 or x.dim() != 2:
        raise KernelError("add_rows takes float32 rows [T, d]")
    for t, n in ((a, "a"), (b, "b")):
        if t is not None:
            _dev(t, n)
            if t.dtype != torch.float32 or t.shape != x.shape:
                raise KernelError(f"add_rows: {n} must be float32 and shaped like x")
    _f32_vec(vec, "vec", x.shape[1])
    _check(_fn("elementwise", "plm_add_rows")(_p(x), _p(a), _p(b), _p(vec), x.shape[0], x.shape[1], _stream()), "add_rows",
           nbytes=x.numel() * 4 * (2 + (a is not None) + (b is not None)))
    return x


def scaled_sum(a: torch.Tensor, scale_a: float, b: torch.Tensor, scale_b: float,
               bias_a: Optional[torch.Tensor] = None) -> torch.Tensor:
    """scale_a * (a + bias_a) + scale_b * b for float32 rows a, b [T, d] and an optional float32 vector bias_a [d]."""
    _dev(a, "a"), _dev(b, "b")
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.dim() != 2 or a.shape != b.shape:
        raise KernelError("scaled_sum takes two float32 matrices of one shape")
    _f32_vec(bias_a, "bias_a", a.shape[1])
    out = torch.empty_like(a)
    _check(_fn("elementwise", "plm_scaled_sum")(_p(a), float(scale_a), _p(bias_a), _p(b), float(scale_b), _p(out), a.shape[0],
                                                a.shape[1], _stream()), "scaled_sum", nbytes=3 * a.numel() * 4)
    return out


def token_gate(gate: torch.Tensor, table: torch.Tensor, first_column: int, tokens: torch.Tensor,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r, j] = gelu_tanh(gate[r, j]) * table[tokens[row r], first_column + j] for `gate` [R, dim] and a per-token
    `table` [vocab, columns] of gate's type; row r of gate belongs to token `rows[r]` of the step (None: token r)."""
    _dev(gate, "gate"), _dev(table, "table"), _i32(tokens, "tokens")
    R, dim = gate.shape
    if table.dim() != 2 or table.dtype != gate.dtype or first_column < 0 or first_column + dim > table.shape[1]:
        raise KernelError("token_gate: the table must be [vocab, columns] of the gate's type and hold the columns asked for")
    if rows is not None:
        _i32(rows, "rows")
        if rows.numel() != R:
            raise KernelError("token_gate: one row number per row of the gate")
    elif tokens.numel() < R:
        raise KernelError("token_gate: fewer tokens than rows")
    out = torch.empty_like(gate)
    set_bounds("elementwise", n_rows=tokens.numel(), device=gate.device)
    _check(_fn("elementwise", "plm_token_gate")(
        _p(gate), _dt(gate, "gate"), _p(table), _dt(table, "table"), table.shape[1], int(first_column), _p(tokens), _p(rows),
        _p(out), R, dim, table.shape[0], _stream()), f"token_gate rows={R} dim={dim}", nbytes=3 * R * dim * gate.element_size())
    return out


def rope_rows(x: torch.Tensor, rotation, tok_pos: torch.Tensor, n_heads: int, head_dim: int) -> torch.Tensor:
    """The leading `rotation.rotary_dim` components of every head of `x` [T, n_heads * head_dim] (contiguous rows; a
    column slice will do) rotated in place by the rows' positions `tok_pos`; returns x.  For rows that reach
    attention by another way than a QKV product."""
    if not x.is_cuda or x.dim() != 2 or x.stride(1) != 1 or x.shape[1] != n_heads * head_dim:
        raise KernelError(f"rope_rows: x must be [T, {n_heads * head_dim}] with contiguous rows on the device")
    _i32(tok_pos, "tok_pos")
    if rotation is None or rotation.cos is None or rotation.rotary_dim == 0:
        return x
    cos, sin, rot = rotation.cos, rotation.sin, rotation.rotary_dim
    if cos.dtype != torch.float32 or cos.shape[1] != rot // 2 or sin.shape != cos.shape or rot > head_dim:
        raise KernelError("rope_rows: cos/sin tables must be float32 [positions, rotary_dim/2], rotary_dim at most head_dim")
    set_bounds("elementwise", n_positions=cos.shape[0], device=x.device)
    _check(_fn("elementwise", "plm_rope_rows")(_p(x), _dt(x, "x"), x.stride(0), _p(cos), _p(sin), _p(tok_pos), x.shape[0],
                                               int(n_heads), int(head_dim), int(rot), 0 if rotation.pairing == "half" else 1,
                                               _stream()), f"rope_rows T={x.shape[0]} heads={n_heads}",
           nbytes=2 * x.shape[0] * n_heads * rot * x.element_size())
    return x


def norm_pair_shift(x: torch.Tensor, w_a: torch.Tensor, eps: float, out_dtype: torch.dtype,
                    w_b: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
                    state: Optional[torch.Tensor] = None, step=None):
    """Two RMS norms of the same rows of the fp32 stream `x` [T, d] in one pass: `a = x r w_a`, `b = x r w_b` with
    `r = 1 / sqrt(mean(x^2) + eps)` (w_a, w_b float32 [d]; without w_b only a is made).  With `mix` (float32 [d]) a is
    shifted towards the sequence's token before: `a_t + (a_(t-1) - a_t) * mix`, a_(t-1) unshifted; for a step's first
    token it comes from `state` (float32 [slots + 1, >= d], contiguous rows; zeros at a sequence's start), which is
    brought up to date.  Returns (a, b) in `out_dtype` (b None without w_b)."""
    _dev(x, "x")
    if x.dtype != torch.float32 or x.dim() != 2:
        raise KernelError("the residual stream must be float32 [T, d]")
    T, d = x.shape
    _f32_vec(w_a, "w_a", d), _f32_vec(w_b, "w_b", d), _f32_vec(mix, "mix", d)
    if w_a is None:
        raise KernelError("norm_pair_shift: w_a is needed")
    lds = 0
    if mix is not None:
        if state is None or step is None or not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 \
                or state.stride(1) != 1 or state.shape[1] < d:
            raise KernelError("norm_pair_shift: a shift needs the step and a float32 state [slots, >= d] on the device")
        lds = state.stride(0)
        set_bounds("elementwise", n_seqs=step.n_seqs, device=x.device)
    out_a = torch.empty((T, d), dtype=out_dtype, device=x.device)
    out_b = torch.empty((T, d), dtype=out_dtype, device=x.device) if w_b is not None else None
    _check(_fn("elementwise", "plm_norm_pair_shift")(
        _p(x), _p(w_a), _p(w_b), _p(mix), _p(state) if mix is not None else None, lds,
        _p(step.tok_seq) if mix is not None else None, _p(step.seq_start) if mix is not None else None,
        _p(step.seq_slot) if mix is not None else None, _p(out_a), _p(out_b), _dt(out_a, "out"), T, d, float(eps), _stream()),
        f"norm_pair_shift rows={T} d={d}", nbytes=T * d * (4 + (2 if w_b is not None else 1) * out_a.element_size()))
    return out_a, out_b
