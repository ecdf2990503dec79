"""Faces of the kernels for mixers with a fixed-size state (csrc/recurrent.cu): the depthwise causal
convolution, the gated linear recurrence, the gate-and-norm step, one small matrix per head, and rows
written into the pages of a cache."""
from __future__ import annotations

from typing import Optional

import torch

from ._lib import PAGE_TOKENS, KernelError, _check, _dev, _dt, _fn, _i32, _p, _stream, set_bounds

DECAY_STEP, DECAY_SIGMOID, DECAY_GIVEN = 1, 2, 3


def _cols(t: torch.Tensor, name: str) -> int:
    """A matrix whose rows are contiguous (it may be a slice of columns of a wider one); returns its row stride."""
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; picolm_b200 kernels run on a CUDA device only")
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{name} must be a matrix with contiguous rows")
    return t.stride(0)


def _f32(t: Optional[torch.Tensor], name: str, numel: int) -> None:
    if t is None:
        return
    _dev(t, name)
    if t.dtype != torch.float32 or t.numel() != numel:
        raise KernelError(f"{name} must be float32 with {numel} elements")


def causal_conv(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, step,
                in_bias: Optional[torch.Tensor] = None, activation: Optional[str] = "silu") -> torch.Tensor:
    """Depthwise causal convolution over each sequence's tokens followed by SiLU (`activation=None`: by nothing);
    `in_bias` [C] float32 is added to the step's inputs before they are used (and kept).  `u` [T, C] (a column slice
    will do), `weight` [taps, C] float32 (tap-major: a checkpoint's [C, taps] transposed) with the current token's
    tap last, `bias` [C] float32 or None, `state`
    float32 [slots, >= (taps - 1) * C] with contiguous rows: the last taps - 1 inputs of every sequence, oldest
    first; it is read for the tokens before the step's first and brought up to date.  Returns [T, C] like u."""
    ldu = _cols(u, "u")
    T, C = u.shape
    taps = weight.shape[0]
    if weight.dim() != 2 or weight.shape[1] != C:
        raise KernelError(f"causal_conv: the weights must be [taps, {C}], got {tuple(weight.shape)}")
    _f32(weight, "weight", C * taps), _f32(bias, "bias", C), _f32(in_bias, "in_bias", C)
    if activation not in ("silu", None):
        raise KernelError(f"causal_conv: activation {activation!r} is not known (silu, None)")
    lds = _cols(state, "state")
    if state.dtype != torch.float32 or state.shape[1] < (taps - 1) * C:
        raise KernelError("causal_conv: the state must be float32 with (taps - 1) * C values a row")
    out = torch.empty((T, C), dtype=u.dtype, device=u.device)
    decode = bool(step.is_decode and step.n_tokens == step.n_seqs)
    set_bounds("recurrent", n_seqs=step.n_seqs, device=u.device)
    _check(_fn("recurrent", "plm_causal_conv")(
        _p(u), _dt(u, "u"), ldu, _p(weight), _p(bias), _p(state), lds, _p(step.tok_seq), _p(step.seq_start),
        _p(step.seq_slot), _p(out), T, step.n_seqs, C, taps, 1 if decode else 0, _p(in_bias), 0 if activation == "silu" else 1,
        _stream()),
        f"causal_conv T={T} C={C} taps={taps}", kernels=1 if decode or taps == 1 else 2,
        nbytes=2 * T * C * u.element_size())
    return out


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, raw: torch.Tensor, mode: int, p0: torch.Tensor,
                p1: Optional[torch.Tensor], skip: Optional[torch.Tensor], q_scale: float, power: float,
                state: torch.Tensor, step, heads: int, key_dim: int, value_dim: int, heads_per_group: int = 1) -> torch.Tensor:
    """The recurrence S_t = diag(d_t) S_(t-1) + k_t v_t^T, y_t = S_t^T (q_scale q_t) (+ skip[h] v_t) over each
    sequence's tokens, per head, everything in float32; returns y [T, heads * value_dim] float32.

    q, k [T, groups * key_dim] (head h reads group h // heads_per_group), v [T, heads * value_dim]; column slices
    will do.  The decay comes from `raw`:
      DECAY_STEP     raw [T, heads]: dt = softplus(raw + p0[h]), d = exp(-exp(p1[h]) dt) for the whole head, and
                     v_t enters the state times dt (the skip term takes it unscaled)
      DECAY_SIGMOID  raw [T, heads * key_dim]: d[n] = sigmoid(raw + p0[h, n]) ** power
    `state` float32 [slots, >= heads * key_dim * value_dim] with contiguous rows holds S of every sequence as
    [heads, key_dim, value_dim] and is carried on."""
    ldq, ldk, ldv, ldr = _cols(q, "q"), _cols(k, "k"), _cols(v, "v"), _cols(raw, "raw")
    T = v.shape[0]
    H, N, P = heads, key_dim, value_dim
    if H % heads_per_group:
        raise KernelError("linear_scan: heads is not a multiple of heads_per_group")
    G = H // heads_per_group
    if q.shape != (T, G * N) or k.shape != (T, G * N) or v.shape != (T, H * P) or not (q.dtype == k.dtype == v.dtype == raw.dtype):
        raise KernelError("linear_scan: q, k, v do not have the shapes the head counts imply, or differ in type")
    if mode == DECAY_STEP:
        if raw.shape != (T, H):
            raise KernelError("linear_scan: a decay per head wants raw [T, heads]")
        _f32(p0, "p0", H), _f32(p1, "p1", H)
        if p1 is None:
            raise KernelError("linear_scan: a decay per head wants p1 (the logarithm of the rate)")
    elif mode == DECAY_SIGMOID:
        if raw.shape != (T, H * N):
            raise KernelError("linear_scan: a decay per key channel wants raw [T, heads * key_dim]")
        _f32(p0, "p0", H * N)
    else:
        raise KernelError(f"linear_scan: unknown decay mode {mode}")
    _f32(skip, "skip", H)
    if N > 256:
        raise KernelError(f"linear_scan: key_dim {N} exceeds 256, the largest state a thread's registers take")
    lds = _cols(state, "state")
    if state.dtype != torch.float32 or state.shape[1] < H * N * P:
        raise KernelError("linear_scan: the state must be float32 with heads * key_dim * value_dim values a row")
    y = torch.empty((T, H * P), dtype=torch.float32, device=v.device)
    # Long prompts are cut into segments that run side by side: a first pass leaves what each segment adds to the
    # state, a small kernel chains those into the state at every segment's start, a second pass gives y.
    seg_len, n_segs = scan_plan(step.n_seqs, H, N, P, step.max_new, T)
    seg_state = seg_decay = None
    kernels, run_mode = 1, mode
    if n_segs > 1:
        seg_state = torch.empty((step.n_seqs, n_segs, H * N * P), dtype=torch.float32, device=v.device)
        seg_decay = torch.empty((step.n_seqs, n_segs, H * N), dtype=torch.float32, device=v.device)
        kernels = 3
        if mode == DECAY_SIGMOID:
            # both passes want the decays: their exponentials are taken once, by a kernel of their own
            given = torch.empty((T, H * N), dtype=torch.float32, device=v.device)
            _check(_fn("recurrent", "plm_sigmoid_decay")(_p(raw), _dt(raw, "raw"), ldr, _p(p0), float(power), _p(given), T,
                                                         H * N, _stream()), f"sigmoid_decay T={T} C={H * N}",
                   nbytes=T * H * N * (4 + raw.element_size()))
            raw, ldr, run_mode = given, H * N, DECAY_GIVEN
    _check(_fn("recurrent", "plm_linear_scan")(
        _p(q), _p(k), _p(v), _p(raw), _dt(v, "v"), ldq, ldk, ldv, ldr, run_mode, _p(p0), _p(p1), _p(skip), float(q_scale),
        float(power), _p(state), lds, _p(y), H * P, _p(step.seq_start), _p(step.seq_slot), step.n_seqs, H, N, P,
        heads_per_group, seg_len, n_segs, _p(seg_state), _p(seg_decay), _stream()),
        f"linear_scan T={T} H={H} N={N} P={P}" + (f" in {n_segs} segments" if n_segs > 1 else ""),
        kernels=kernels,
        nbytes=T * (2 * G * N + H * P) * v.element_size() + T * H * P * 4 + 2 * step.n_seqs * H * N * P * 4,
        flops=(10 if n_segs > 1 else 6) * T * H * N * P)
    return y


_plans = {}


def scan_plan(n_seqs: int, heads: int, key_dim: int, value_dim: int, max_new: int, n_tokens: int = 0):
    """(tokens per segment, segments of the longest sequence) of `linear_scan` for a step of `n_tokens` tokens (0: not
    known) whose longest sequence brings `max_new` of them; one segment means one pass from the cache's state."""
    key = (n_seqs, heads, key_dim, value_dim, max_new, n_tokens)
    plan = _plans.get(key)
    if plan is None:
        import ctypes
        out = (ctypes.c_int * 2)()
        _fn("recurrent", "plm_linear_scan_plan")(n_seqs, heads, key_dim, value_dim, int(max_new), int(n_tokens),
                                                 ctypes.cast(out, ctypes.c_void_p))
        if len(_plans) > 4096:
            _plans.clear()
        plan = _plans[key] = (out[0], out[1])
    return plan


GATE_NONE, GATE_BEFORE_NORM, GATE_AFTER_NORM = 0, 1, 2
_ACTS = {"silu": 0, "sigmoid": 1}


def gated_norm(x: torch.Tensor, out_dtype: torch.dtype, weight: Optional[torch.Tensor] = None, eps: float = 0.0,
               group: Optional[int] = None, weight_per_group: bool = False, gate: Optional[torch.Tensor] = None,
               gate_mode: int = GATE_NONE, activation: str = "silu", norm: bool = True) -> torch.Tensor:
    """Rows of `x` [T, C] (float32 or the run's type; a column slice will do), in groups of `group` columns
    (default: the whole row): optionally times act(gate) first, then each group divided by its root mean square
    (eps inside the root) and multiplied by `weight` (float32, [C], or [group] with `weight_per_group`), optionally
    times act(gate) afterwards.  With `norm=False` only the gate is applied.  Returns [T, C] of `out_dtype`."""
    ldx = _cols(x, "x")
    T, C = x.shape
    group = C if group is None else int(group)
    if group <= 0 or C % group:
        raise KernelError(f"gated_norm: {C} columns do not come in groups of {group}")
    if weight is not None:
        _f32(weight, "weight", group if weight_per_group else C)
    if activation not in _ACTS:
        raise KernelError(f"gated_norm: activation {activation!r} is not known ({', '.join(_ACTS)})")
    ldg = 0
    if gate_mode != GATE_NONE:
        if gate is None or gate.shape != x.shape:
            raise KernelError("gated_norm: the gate must be shaped like x")
        ldg = _cols(gate, "gate")
    else:
        gate = None
    out = torch.empty((T, C), dtype=out_dtype, device=x.device)
    _check(_fn("recurrent", "plm_gated_norm")(
        _p(x), _dt(x, "x"), ldx, _p(gate), _dt(gate, "gate") if gate is not None else 1, ldg, _p(weight),
        1 if weight_per_group else 0, _p(out), _dt(out, "out"), C, T, C, group, float(eps), int(gate_mode),
        _ACTS[activation], 1 if norm else 0, _stream()), f"gated_norm T={T} C={C} group={group}",
        nbytes=T * C * (x.element_size() + out.element_size() + (gate.element_size() if gate is not None else 0)))
    return out


def head_linear(x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor] = None,
                gate_per_head: bool = False) -> torch.Tensor:
    """out[t, h, :] = weight[h] @ x[t, h, :] for `weight` [H, O, I] and `x` [T, H * I] (a column slice will do), with
    float32 sums; optionally times sigmoid(gate) for `gate` [T, H * O], or with `gate_per_head` [T, H]: one gate for
    all of a head's outputs.  Returns [T, H * O] of x's type."""
    ldx = _cols(x, "x")
    _dev(weight, "weight")
    H, O, I = weight.shape
    T = x.shape[0]
    if x.shape[1] != H * I or weight.dtype != x.dtype:
        raise KernelError(f"head_linear: x is {tuple(x.shape)} of {x.dtype}, the weights are {tuple(weight.shape)} of {weight.dtype}")
    ldg = 0
    if gate is not None:
        ldg = _cols(gate, "gate")
        if gate.shape != (T, H if gate_per_head else H * O) or gate.dtype not in (x.dtype, torch.float32):
            raise KernelError("head_linear: the gate must be [T, H * O] (per head: [T, H]) of x's type or float32")
    out = torch.empty((T, H * O), dtype=x.dtype, device=x.device)
    _check(_fn("recurrent", "plm_head_linear")(
        _p(x), _dt(x, "x"), ldx, _p(weight), _p(gate), _dt(gate, "gate") if gate is not None else 0, ldg, _p(out), H * O, T, H,
        O, I, 1 if gate_per_head else 0, _stream()),
        f"head_linear T={T} H={H} {O}x{I}", nbytes=(T * H * (I + O) + H * O * I) * x.element_size(), flops=2 * T * H * O * I)
    return out


def store_rows_paged(rows: torch.Tensor, pages: torch.Tensor, step, block_table: torch.Tensor) -> None:
    """Row t of `rows` [T, R] into `pages` [n_pages, 1, PAGE_TOKENS, R] at position tok_pos[t] of sequence tok_seq[t]."""
    ld = _cols(rows, "rows")
    _dev(pages, "pages"), _i32(block_table, "block_table")
    T, R = rows.shape
    if pages.dtype != rows.dtype or tuple(pages.shape[1:]) != (1, PAGE_TOKENS, R):
        raise KernelError(f"store_rows_paged: the pages must be [n, 1, {PAGE_TOKENS}, {R}] of {rows.dtype}")
    set_bounds("recurrent", n_pages=pages.shape[0], n_seqs=block_table.shape[0],
               n_positions=block_table.shape[1] * PAGE_TOKENS, device=rows.device)
    _check(_fn("recurrent", "plm_store_rows_paged")(
        _p(rows), _dt(rows, "rows"), ld, _p(pages), _p(step.tok_pos), _p(step.tok_seq), _p(block_table),
        block_table.shape[1], T, R, _stream()), f"store_rows_paged T={T} R={R}", nbytes=2 * T * R * rows.element_size())


def latent_store(rows: torch.Tensor, weight: torch.Tensor, eps: float, rotation, n_rot: int, pages: torch.Tensor, step,
                 block_table: torch.Tensor, store: bool = True, q_rows: Optional[torch.Tensor] = None,
                 q_weight: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """A latent's row into the pages of its cache, made from the projection's columns `rows` [T, n_rot + n_norm]
    (float32 or the run's type; a column slice will do): the first `n_rot` columns rotated by the token's position
    (`rotation`: `ops.Rotation` over n_rot components), the other n_norm divided by their root mean square (`eps`
    inside the root) and multiplied by `weight` (float32 [n_norm]); `pages` [n, 1, PAGE_TOKENS, R] with R >= n_rot +
    n_norm receive [rotated | normed | zeros] at position tok_pos[t] of sequence tok_seq[t] (`store=False`: nothing
    is written, for a layer that reads another layer's cache).  On the way the kernel norms a second stretch of the
    same tokens' rows: `q_rows` [T, n_q] (of rows' type; a column slice will do) divided by its root mean square and
    multiplied by `q_weight` (float32 [n_q]), returned as [T, n_q] of the pages' type."""
    ld = _cols(rows, "rows")
    _dev(pages, "pages"), _i32(block_table, "block_table")
    T, C = rows.shape
    n_norm = C - int(n_rot)
    _f32(weight, "weight", n_norm)
    R = pages.shape[-1]
    if n_norm <= 0 or tuple(pages.shape[1:]) != (1, PAGE_TOKENS, R) or R < C:
        raise KernelError(f"latent_store: the pages must be [n, 1, {PAGE_TOKENS}, >= {C}]")
    cos = sin = None
    pairing = "half"
    if n_rot:
        if rotation is None or rotation.cos is None or rotation.rotary_dim != n_rot:
            raise KernelError(f"latent_store: {n_rot} rotated columns need a rotation over {n_rot} components")
        cos, sin, pairing = rotation.cos, rotation.sin, rotation.pairing
        if step.max_position >= cos.shape[0]:
            raise KernelError(f"position {step.max_position} lies beyond the rotary table")
    q_out, ldq, n_q = None, 0, 0
    if q_rows is not None:
        ldq = _cols(q_rows, "q_rows")
        n_q = q_rows.shape[1]
        _f32(q_weight, "q_weight", n_q)
        if q_rows.shape[0] != T or q_rows.dtype != rows.dtype or q_weight is None:
            raise KernelError("latent_store: q_rows must be [T, n_q] of rows' type, with a weight")
        q_out = torch.empty((T, n_q), dtype=pages.dtype, device=rows.device)
    set_bounds("recurrent", n_pages=pages.shape[0], n_seqs=block_table.shape[0],
               n_positions=block_table.shape[1] * PAGE_TOKENS, device=rows.device)
    _check(_fn("recurrent", "plm_latent_store")(
        _p(rows), _dt(rows, "rows"), ld, _p(weight), float(eps), _p(cos), _p(sin), _p(pages), _dt(pages, "pages"),
        _p(step.tok_pos), _p(step.tok_seq), _p(block_table), block_table.shape[1], T, int(n_rot), n_norm, R,
        0 if pairing == "half" else 1, 1 if store else 0, _p(q_rows), ldq, _p(q_weight), _p(q_out), n_q, _stream()),
        f"latent_store T={T} rot={n_rot} norm={n_norm}",
        nbytes=T * ((C + n_q) * rows.element_size() + (R + n_q) * pages.element_size()))
    return q_out


def rglru_gates(u: torch.Tensor, w_rate: torch.Tensor, w_in: torch.Tensor, b_rate: torch.Tensor, b_in: torch.Tensor,
                rate: torch.Tensor, blocks: int):
    """The two gates of a real-gated diagonal recurrence from its convolved input `u` [T, W] (a column slice will
    do): the channels come in `blocks` equal parts, each with square matrices `w_rate[b]`, `w_in[b]` ([blocks, n, n],
    [out, in], of u's type) and biases [W] float32;
      log a = -sigmoid(w_rate[b] u_b + b_rate) * rate,   x = sqrt(1 - a^2) * sigmoid(w_in[b] u_b + b_in) * u
    with `rate` [W] float32 (the constant times softplus of the learned parameter).  Sums and everything behind
    them in float32; returns (log a, x), float32 [T, W] each: the logarithm, because a float next to 1 no longer
    says how far from 1 it is."""
    ldu = _cols(u, "u")
    T, W = u.shape
    if blocks <= 0 or W % blocks:
        raise KernelError(f"rglru_gates: {W} channels do not come in {blocks} equal blocks")
    n = W // blocks
    for w, name in ((w_rate, "w_rate"), (w_in, "w_in")):
        _dev(w, name)
        if tuple(w.shape) != (blocks, n, n) or w.dtype != u.dtype:
            raise KernelError(f"rglru_gates: {name} must be [{blocks}, {n}, {n}] of {u.dtype}")
    _f32(b_rate, "b_rate", W), _f32(b_in, "b_in", W), _f32(rate, "rate", W)
    a = torch.empty((T, W), dtype=torch.float32, device=u.device)
    x = torch.empty((T, W), dtype=torch.float32, device=u.device)
    _check(_fn("recurrent", "plm_rglru_gates")(
        _p(u), _dt(u, "u"), ldu, _p(w_rate), _p(w_in), _dt(w_rate, "w_rate"), _p(b_rate), _p(b_in), _p(rate), _p(a), _p(x),
        T, W, blocks, _stream()), f"rglru_gates T={T} W={W} blocks={blocks}",
        nbytes=T * W * (u.element_size() + 8) + 2 * W * n * w_rate.element_size(), flops=4 * T * W * n)
    return a, x


def diag_scan(a: torch.Tensor, x: torch.Tensor, y_raw: torch.Tensor, y_bias: Optional[torch.Tensor], state: torch.Tensor,
              step) -> torch.Tensor:
    """S_t = a_t S_(t-1) + x_t per channel over each sequence's tokens (float32 `a`, `x` [T, W], contiguous; `a` holds
    the decays' logarithms), from and into `state` (float32 [slots, >= W], contiguous rows); returns S_t * gelu_tanh(y_raw_t + y_bias) as [T, W] of
    y_raw's type (`y_raw` may be a column slice; `y_bias` [W] float32 or None)."""
    T, W = a.shape
    for t, n in ((a, "a"), (x, "x")):
        _dev(t, n)
        if t.dtype != torch.float32 or tuple(t.shape) != (T, W):
            raise KernelError(f"diag_scan: {n} must be float32 [{T}, {W}]")
    ldy = _cols(y_raw, "y_raw")
    if tuple(y_raw.shape) != (T, W):
        raise KernelError("diag_scan: y_raw must be shaped like a")
    _f32(y_bias, "y_bias", W)
    lds = _cols(state, "state")
    if state.dtype != torch.float32 or state.shape[1] < W:
        raise KernelError("diag_scan: the state must be float32 with a value per channel")
    decode = bool(step.is_decode and step.n_tokens == step.n_seqs)
    out = torch.empty((T, W), dtype=y_raw.dtype, device=a.device)
    set_bounds("recurrent", n_seqs=step.n_seqs, device=a.device)
    _check(_fn("recurrent", "plm_diag_scan")(
        _p(a), _p(x), _p(y_raw), _dt(y_raw, "y_raw"), ldy, _p(y_bias), _p(state), lds, _p(out), _p(step.seq_start),
        _p(step.seq_slot), step.n_seqs, W, 1 if decode else 0, _stream()), f"diag_scan T={T} W={W}",
        nbytes=T * W * (8 * (1 if decode else 2) + 2 * y_raw.element_size()))
    return out


DELTA_CHUNK_FROM = 16      # tokens of a step's longest sequence from which the delta rule runs chunk by chunk


def delta_chunk_workspace(n_tokens: int, n_seqs: int, heads: int, key_dim: int) -> int:
    """Floats of workspace the chunked delta rule takes (as the kernels lay it out): per chunk and head three copies
    of the chunk's keys or queries [32, NP], two matrices [32, 32] and a row [NP], NP the key size rounded up to the
    next of 32, 64, 128, 256; a sequence's chunks start at slot seq_start // 32 + its number."""
    np_ = next(w for w in (32, 64, 128, 256) if key_dim <= w)
    return (n_tokens // 32 + n_seqs + 1) * heads * (3 * 32 * np_ + 2 * 32 * 32 + np_)


def delta_prep(q: torch.Tensor, k: torch.Tensor, z: torch.Tensor, b_raw: torch.Tensor, a_log: torch.Tensor,
               dt_bias: torch.Tensor, l2_eps: float, q_scale: float, heads: int, key_dim: int, heads_per_group: int = 1):
    """What the gated delta rule's recurrence takes, per token in float32 from the convolved projections (all of one
    type, column slices will do): q, k [T, groups * key_dim] made unit vectors per group (`x / sqrt(sum x^2 +
    l2_eps)`, q also times `q_scale`), their product q . k, the decays' logarithms `-exp(a_log[h]) softplus(z + dt_bias)`
    for z [T, heads * key_dim] (the logarithm: a decay next to 1 keeps its distance from 1), and `sigmoid(b_raw)` for b_raw [T, heads].  Returns (qn, kn, qk, decay, beta)."""
    T = q.shape[0]
    H, N = heads, key_dim
    if H % heads_per_group:
        raise KernelError("delta_prep: heads is not a multiple of heads_per_group")
    G = H // heads_per_group
    ldq, ldk, ldz, ldb = _cols(q, "q"), _cols(k, "k"), _cols(z, "z"), _cols(b_raw, "b_raw")
    if (tuple(q.shape) != (T, G * N) or tuple(k.shape) != (T, G * N) or tuple(z.shape) != (T, H * N)
            or tuple(b_raw.shape) != (T, H) or not (q.dtype == k.dtype == z.dtype == b_raw.dtype)):
        raise KernelError("delta_prep: q, k, z, b_raw do not have the shapes the head counts imply, or differ in type")
    _f32(a_log, "a_log", H), _f32(dt_bias, "dt_bias", H * N)
    dev = q.device
    qn = torch.empty((T, G * N), dtype=torch.float32, device=dev)
    kn = torch.empty((T, G * N), dtype=torch.float32, device=dev)
    qk = torch.empty((T, G), dtype=torch.float32, device=dev)
    dec = torch.empty((T, H * N), dtype=torch.float32, device=dev)
    beta = torch.empty((T, H), dtype=torch.float32, device=dev)
    _check(_fn("recurrent", "plm_delta_prep")(
        _p(q), ldq, _p(k), ldk, _p(z), ldz, _p(b_raw), ldb, _dt(q, "q"), _p(a_log), _p(dt_bias), float(l2_eps),
        float(q_scale), _p(qn), _p(kn), _p(qk), _p(dec), _p(beta), T, G, H, N, _stream()), f"delta_prep T={T} H={H} N={N}",
        nbytes=T * ((2 * G + H) * N * (q.element_size() + 4)))
    return qn, kn, qk, dec, beta


def delta_scan(qn: torch.Tensor, kn: torch.Tensor, qk: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor,
               v: torch.Tensor, state: torch.Tensor, step, heads: int, key_dim: int, value_dim: int,
               heads_per_group: int = 1) -> torch.Tensor:
    """The gated delta rule over each sequence's tokens, per head, state S [key_dim, value_dim] in float32:
      S <- diag(exp(decay_t)) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
    (the read-out sees the token's own write).  qn, kn, qk, decay (its logarithm), beta as `delta_prep` returns them; v [T, heads *
    value_dim] (a column slice will do); `state` float32 [slots, >= heads * key_dim * value_dim] with contiguous
    rows holds S as [heads, key_dim, value_dim] and is carried on.  Returns o, float32 [T, heads * value_dim].
    A step whose longest sequence brings `DELTA_CHUNK_FROM` tokens or more runs chunk by chunk (two kernels: what does
    not depend on the state for all chunks side by side, then a walk over each sequence's chunks); shorter portions
    and single tokens run token by token."""
    H, N, P = heads, key_dim, value_dim
    T = v.shape[0]
    if H % heads_per_group:
        raise KernelError("delta_scan: heads is not a multiple of heads_per_group")
    G = H // heads_per_group
    ldv = _cols(v, "v")
    for t, n, cols in ((qn, "qn", G * N), (kn, "kn", G * N), (qk, "qk", G), (decay, "decay", H * N), (beta, "beta", H)):
        _dev(t, n)
        if t.dtype != torch.float32 or tuple(t.shape) != (T, cols):
            raise KernelError(f"delta_scan: {n} must be float32 [{T}, {cols}]")
    if tuple(v.shape) != (T, H * P):
        raise KernelError("delta_scan: v must be [T, heads * value_dim]")
    if N > 256:
        raise KernelError(f"delta_scan: key_dim {N} exceeds 256, the largest state a thread's registers take")
    lds = _cols(state, "state")
    if state.dtype != torch.float32 or state.shape[1] < H * N * P:
        raise KernelError("delta_scan: the state must be float32 with heads * key_dim * value_dim values a row")
    y = torch.empty((T, H * P), dtype=torch.float32, device=v.device)
    set_bounds("recurrent", n_seqs=step.n_seqs, device=v.device)
    if step.max_new >= DELTA_CHUNK_FROM and not (step.is_decode and step.n_tokens == step.n_seqs):
        floats = delta_chunk_workspace(T, step.n_seqs, H, N)
        ws = torch.empty((floats,), dtype=torch.float32, device=v.device)
        _check(_fn("recurrent", "plm_delta_chunk_scan")(
            _p(qn), _p(kn), _p(decay), _p(beta), _p(v), _dt(v, "v"), ldv, _p(state), lds, _p(y), _p(ws), _p(step.seq_start),
            _p(step.seq_slot), step.n_seqs, int(step.max_new), H, N, P, heads_per_group, _stream()),
            f"delta_chunk_scan T={T} H={H} N={N} P={P}", kernels=2,
            nbytes=2 * floats * 4 + T * H * P * (4 + v.element_size()) + 2 * step.n_seqs * H * N * P * 4,
            flops=T * H * (6 * N * P + 6 * 32 * N + 4 * 32 * P))
        return y
    _check(_fn("recurrent", "plm_delta_scan")(
        _p(qn), _p(kn), _p(qk), _p(decay), _p(beta), _p(v), _dt(v, "v"), ldv, _p(state), lds, _p(y), _p(step.seq_start),
        _p(step.seq_slot), step.n_seqs, H, N, P, heads_per_group, _stream()), f"delta_scan T={T} H={H} N={N} P={P}",
        nbytes=T * (2 * G * N + 2 * H * N) * 4 + T * H * P * (4 + v.element_size()) + 2 * step.n_seqs * H * N * P * 4,
        flops=8 * T * H * N * P)
    return y
