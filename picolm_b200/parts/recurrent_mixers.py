"""Mixers that keep a fixed-size state per sequence instead of keys and values: the state-space mixer in
its state-space-duality form ("mamba2") and gated linear attention ("gla").  Both are the same recurrence
`S_t = diag(d_t) S_(t-1) + k_t v_t^T, y_t = S_t^T q_t` (`ops.linear_scan`); they differ in where the decay
comes from, in what stands around the recurrence, and in the order of gate and norm behind it.

Everything that enters the recurrence (decays, step sizes, state, sums) is float32 in both kinds of run;
projections, the short convolution and their activations are in the run's element type.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.spec import CacheSpec
from .base import Part, WeightSpec, register_part
from .mixer import _stack_rows


class _StateMixer(Part):
    graph_safe = True               # the step is read through device buffers only (seq_start, seq_slot, tok_seq)
    # Captured prompt steps too: padding tokens belong to a sequence that `seq_start` gives no tokens, so the
    # recurrence never visits them (their rows of y stay as they were allocated, and everything after works row by
    # row); the convolution treats them as a sequence of the null slot; sequences without tokens leave their state.
    graph_safe_prompts = True

    def _f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(torch.float32).contiguous()


@register_part("mixer", "mamba2")
class Mamba2(_StateMixer):
    """params: hidden_size, heads, vdim (value size of a head), state (N), groups (heads of a group share B and C),
    conv (taps), norm_groups, eps.  One input projection laid out [z | x | B | C | dt]; x, B and C pass a depthwise
    causal convolution with SiLU; per head `S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T` with
    `dt = softplus(dt + dt_bias)`, `y_t = S_t^T C_t + D x_t`; then `y * silu(z)`, an RMS norm in `norm_groups` equal
    parts, and the output projection.

    Tensors: in [2 inner + 2 groups N + heads, hidden], conv [inner + 2 groups N, taps], conv.b, dt_bias, A_log, D
    [heads], norm [inner], o [hidden, inner], with inner = heads * vdim."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.H, self.P, self.N, self.G = p["hidden_size"], p["heads"], p["vdim"], p["state"], p["groups"]
        self.taps, self.norm_groups, self.eps = p["conv"], p["norm_groups"], float(p["eps"])
        self.inner = self.H * self.P
        self.conv_channels = self.inner + 2 * self.G * self.N
        if self.H % self.G or self.inner % self.norm_groups:
            raise ValueError("mamba2: heads must be a multiple of groups and heads * vdim of norm_groups")
        self.n_state = self.H * self.N * self.P
        self.n_conv = (self.taps - 1) * self.conv_channels

    def weight_specs(self):
        H, C = self.H, self.conv_channels
        return {
            "in": WeightSpec((2 * self.inner + 2 * self.G * self.N + H, self.d)),
            "conv": WeightSpec((C, self.taps), init="normal_scaled", scale=0.3),
            "conv.b": WeightSpec((C,), init="normal_scaled", scale=0.1),
            "dt_bias": WeightSpec((H,), init="uniform", lo=-4.0, hi=-1.0),
            "A_log": WeightSpec((H,), init="uniform", lo=-1.0, hi=1.5),
            "D": WeightSpec((H,), init="ones_normal"),
            "norm": WeightSpec((self.inner,), init="ones_normal"),
            "o": WeightSpec((self.d, self.inner)),
        }

    def load(self, tensors):
        self.w_in, self.w_o = tensors["in"], tensors["o"]
        # the kernel wants the taps' weights tap by tap, neighbouring channels side by side
        self.conv_w, self.conv_b = self._f32(tensors["conv"].to(torch.float32).t()), self._f32(tensors["conv.b"])
        self.dt_bias, self.a_log, self.skip = self._f32(tensors["dt_bias"]), self._f32(tensors["A_log"]), self._f32(tensors["D"])
        self.norm_w = self._f32(tensors["norm"])

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def cache_spec(self):
        # one row per sequence: the recurrence's state [heads, N, vdim], then the convolution's last inputs
        return CacheSpec.state((self.n_state + self.n_conv,))

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        inner, GN = self.inner, self.G * self.N
        zxbcdt = ops.linear(h, self.w_in, dt)
        z = zxbcdt[:, :inner]
        xbc = ops.causal_conv(zxbcdt[:, inner:inner + self.conv_channels], self.conv_w, self.conv_b,
                              cache.state[:, self.n_state:], step)
        y = ops.linear_scan(q=xbc[:, inner + GN:], k=xbc[:, inner:inner + GN], v=xbc[:, :inner],
                            raw=zxbcdt[:, inner + self.conv_channels:], mode=ops.DECAY_STEP, p0=self.dt_bias, p1=self.a_log,
                            skip=self.skip, q_scale=1.0, power=1.0, state=cache.state[:, :self.n_state], step=step,
                            heads=self.H, key_dim=self.N, value_dim=self.P, heads_per_group=self.H // self.G)
        g = ops.gated_norm(y, dt, weight=self.norm_w, eps=self.eps, group=inner // self.norm_groups, gate=z,
                           gate_mode=ops.GATE_BEFORE_NORM, activation="silu")
        return ops.linear(g, self.w_o, torch.float32, defer=True)


@register_part("mixer", "gla")
class GatedLinearAttention(_StateMixer):
    """params: hidden_size, heads, dim (key size of a head), vdim, tau, decay_rank (None: as the checkpoint has it), eps.  `q = W_q h / sqrt(dim)`,
    `k = W_k h`, `v = W_v h`; a decay per key channel `alpha = sigmoid(W_a2 (W_a1 h) + b)^(1/tau)`; per head
    `S_t = diag(alpha_t) S_(t-1) + k_t v_t^T`, `o_t = S_t^T q_t`; each head's o is RMS-normed over vdim with one weight
    shared by the heads, multiplied by `silu(W_g h)` and projected.

    Tensors: q, k [heads dim, hidden], v, g [heads vdim, hidden], a1 [decay_rank, hidden], a2 [heads dim, decay_rank],
    a2.b [heads dim], norm [vdim], o [hidden, heads vdim]."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.H, self.N, self.P = p["hidden_size"], p["heads"], p["dim"], p["vdim"]
        # decay_rank None: the checkpoint's a1 says how wide the decay's bottleneck is
        self.tau, self.rank, self.eps = float(p["tau"]), p.get("decay_rank"), float(p["eps"])

    def weight_specs(self):
        HN, HP, d = self.H * self.N, self.H * self.P, self.d
        return {
            "q": WeightSpec((HN, d)), "k": WeightSpec((HN, d)), "v": WeightSpec((HP, d)), "g": WeightSpec((HP, d)),
            "a1": WeightSpec((self.rank or -1, d)), "a2": WeightSpec((HN, self.rank or -1), init="normal_scaled", scale=0.5),
            "a2.b": WeightSpec((HN,), init="uniform", lo=0.0, hi=4.0),
            "norm": WeightSpec((self.P,), init="ones_normal"),
            "o": WeightSpec((d, HP)),
        }

    def load(self, tensors):
        # one projection for everything that reads h: rows [q | k | v | g | a1]
        self.w_h = _stack_rows([tensors[n] for n in ("q", "k", "v", "g", "a1")])
        self.w_a2, self.w_o = tensors["a2"], tensors["o"]
        if tensors["a1"].shape[0] != self.w_a2.shape[1]:
            raise ValueError(f"gla: a1 has {tensors['a1'].shape[0]} rows but a2 takes {self.w_a2.shape[1]} columns")
        self.a2_bias, self.norm_w = self._f32(tensors["a2.b"]), self._f32(tensors["norm"])

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_h, self.w_a2, self.w_o))

    def cache_spec(self):
        return CacheSpec.state((self.H * self.N * self.P,))

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        HN, HP = self.H * self.N, self.H * self.P
        proj = ops.linear(h, self.w_h, dt)
        q, k, v = proj[:, :HN], proj[:, HN:2 * HN], proj[:, 2 * HN:2 * HN + HP]
        g, a1 = proj[:, 2 * HN + HP:2 * HN + 2 * HP], proj[:, 2 * HN + 2 * HP:]
        # the bottleneck is a few columns wide: the CUDA-core product reads them where they lie; a wide one is copied
        # out for the tensor cores
        z = ops.gemm_simt(a1, self.w_a2, dt) if a1.shape[1] < 64 else ops.linear(a1.contiguous(), self.w_a2, dt)
        o = ops.linear_scan(q=q, k=k, v=v, raw=z, mode=ops.DECAY_SIGMOID, p0=self.a2_bias, p1=None, skip=None,
                            q_scale=self.N ** -0.5, power=1.0 / self.tau, state=cache.state, step=step, heads=self.H,
                            key_dim=self.N, value_dim=self.P)
        gated = ops.gated_norm(o, dt, weight=self.norm_w, eps=self.eps, group=self.P, weight_per_group=True, gate=g,
                               gate_mode=ops.GATE_AFTER_NORM, activation="silu")
        return ops.linear(gated, self.w_o, torch.float32, defer=True)


@register_part("mixer", "rglru")
class GatedDiagonalRecurrence(_StateMixer):
    """A recurrent block around a real-gated diagonal linear recurrence.  params: hidden_size, width (channels of the
    recurrence), blocks (the gates' matrices are block-diagonal in that many equal parts), conv (taps), rate (the
    constant c of the decay, default 8).  Two branches read h: `y = gelu_tanh(W_y h + b_y)` and
    `u = conv(W_x h + b_x)` (depthwise, causal, with a bias and no activation).  Per block b of u:
    `r = sigmoid(ra[b] u_b + ra.b)`, `i = sigmoid(ri[b] u_b + ri.b)`; `a = exp(-c r softplus(lam))`;
    `S_t = a S_(t-1) + sqrt(1 - a^2) i u` from S = 0, the first token like every other; the result is `W_o (S y)`.

    Tensors: y, x [width, hidden] with biases y.b, x.b; conv [width, taps], conv.b; ra, ri [blocks, n, n] ([out, in],
    n = width / blocks) with ra.b, ri.b [blocks, n]; lam [width]; o [hidden, width]."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.W, self.blocks, self.taps = p["hidden_size"], p["width"], p["blocks"], p["conv"]
        self.c = float(p.get("rate", 8.0))
        if self.W % self.blocks:
            raise ValueError("rglru: width must be a multiple of blocks")
        self.n_conv = (self.taps - 1) * self.W

    def weight_specs(self):
        W, d, B = self.W, self.d, self.blocks
        n = W // B
        return {
            "y": WeightSpec((W, d)), "y.b": WeightSpec((W,), init="normal"),
            "x": WeightSpec((W, d)), "x.b": WeightSpec((W,), init="normal"),
            "conv": WeightSpec((W, self.taps), init="normal_scaled", scale=0.4),
            "conv.b": WeightSpec((W,), init="normal_scaled", scale=0.1),
            "ra": WeightSpec((B, n, n)), "ra.b": WeightSpec((B, n), init="normal"),
            "ri": WeightSpec((B, n, n)), "ri.b": WeightSpec((B, n), init="normal"),
            "lam": WeightSpec((W,), init="uniform", lo=-4.0, hi=0.0),
            "o": WeightSpec((d, W)),
        }

    def load(self, tensors):
        self.w_yx = _stack_rows([tensors["y"], tensors["x"]])       # one product for both branches: rows [y | x]
        self.w_o = tensors["o"]
        self.y_bias, self.x_bias = self._f32(tensors["y.b"]), self._f32(tensors["x.b"])
        self.conv_w, self.conv_b = self._f32(tensors["conv"].to(torch.float32).t()), self._f32(tensors["conv.b"])
        self.w_ra, self.w_ri = tensors["ra"].contiguous(), tensors["ri"].contiguous()
        self.b_ra, self.b_ri = self._f32(tensors["ra.b"]).reshape(-1), self._f32(tensors["ri.b"]).reshape(-1)
        # the decay's exponent per channel, c * softplus(lam), once in float32
        self.rate = (self.c * torch.nn.functional.softplus(tensors["lam"].to(torch.float32))).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_yx, self.w_o, self.w_ra, self.w_ri))

    def cache_spec(self):
        # one row per sequence: the recurrence's state [width], then the convolution's last inputs
        return CacheSpec.state((self.W + self.n_conv,))

    def forward(self, h, step, cache):
        dt, W = self.runtime.dtype, self.W
        yx = ops.linear(h, self.w_yx, dt)
        u = ops.causal_conv(yx[:, W:], self.conv_w, self.conv_b, cache.state[:, W:], step, in_bias=self.x_bias,
                            activation=None)
        log_a, x = ops.rglru_gates(u, self.w_ra, self.w_ri, self.b_ra, self.b_ri, self.rate, self.blocks)
        g = ops.diag_scan(log_a, x, yx[:, :W], self.y_bias, cache.state[:, :W], step)
        return ops.linear(g, self.w_o, torch.float32, defer=True)


@register_part("mixer", "gated_delta")
class GatedDeltaRule(_StateMixer):
    """The delta rule with a decay per key channel.  params: hidden_size, heads, kv_heads (query/key heads; head h
    uses q/k head h // (heads / kv_heads)), dim (key size), vdim, conv (taps), rank (None: as the checkpoint's a1 and
    g1 have it), eps (of the read-out's norm), l2_eps (inside the root of the unit norm, default 1e-6).
    q, k, v each pass a depthwise causal convolution (no bias) and SiLU; q and k are made unit vectors per head and q
    is multiplied by dim^(-1/2); `beta = sigmoid(W_b h)` per head; the decay per head and key channel is
    `exp(-exp(A_log_h) softplus(W_a2 (W_a1 h) + dt_bias))`.  Per head, S [dim, vdim] from zero:
    `S <- diag(decay) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`.  Each head's o is divided by its root
    mean square over vdim, times `norm` [vdim] (shared), times `sigmoid(W_g2 (W_g1 h))`, then projected.

    Tensors: q, k [kv_heads dim, hidden], v [heads vdim, hidden], q.conv, k.conv, v.conv [channels, taps], b [heads,
    hidden], A_log [heads], a1 [rank, hidden], a2 [heads dim, rank], dt_bias [heads dim], g1 [rank', hidden], g2
    [heads vdim, rank'], norm [vdim], o [hidden, heads vdim]."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.H, self.G, self.N, self.P = p["hidden_size"], p["heads"], p["kv_heads"], p["dim"], p["vdim"]
        self.taps, self.rank, self.eps = p["conv"], p.get("rank"), float(p["eps"])
        self.l2_eps = float(p.get("l2_eps", 1e-6))
        if self.H % self.G:
            raise ValueError("gated_delta: heads must be a multiple of kv_heads")
        self.conv_channels = 2 * self.G * self.N + self.H * self.P
        self.n_state = self.H * self.N * self.P
        self.n_conv = (self.taps - 1) * self.conv_channels

    def weight_specs(self):
        GN, HN, HP, d, r = self.G * self.N, self.H * self.N, self.H * self.P, self.d, self.rank or -1
        conv = dict(init="normal_scaled", scale=0.4)
        return {
            "q": WeightSpec((GN, d)), "k": WeightSpec((GN, d)), "v": WeightSpec((HP, d)),
            "q.conv": WeightSpec((GN, self.taps), **conv), "k.conv": WeightSpec((GN, self.taps), **conv),
            "v.conv": WeightSpec((HP, self.taps), **conv),
            "b": WeightSpec((self.H, d)), "A_log": WeightSpec((self.H,), init="uniform", lo=-2.0, hi=0.5),
            "a1": WeightSpec((r, d)), "a2": WeightSpec((HN, r), init="normal_scaled", scale=0.5),
            "dt_bias": WeightSpec((HN,), init="uniform", lo=-3.0, hi=0.0),
            "g1": WeightSpec((r, d)), "g2": WeightSpec((HP, r), init="normal_scaled", scale=0.5),
            "norm": WeightSpec((self.P,), init="ones_normal"),
            "o": WeightSpec((d, HP)),
        }

    def load(self, tensors):
        # one projection for everything that reads h: rows [q | k | v | b | a1 | g1]
        self.w_h = _stack_rows([tensors[n] for n in ("q", "k", "v", "b", "a1", "g1")])
        self.r_a, self.r_g = tensors["a1"].shape[0], tensors["g1"].shape[0]
        self.w_a2, self.w_g2, self.w_o = tensors["a2"], tensors["g2"], tensors["o"]
        if self.w_a2.shape[1] != self.r_a or self.w_g2.shape[1] != self.r_g:
            raise ValueError("gated_delta: a2 / g2 do not take as many columns as a1 / g1 have rows")
        self.conv_w = self._f32(torch.cat([tensors[n].to(torch.float32) for n in ("q.conv", "k.conv", "v.conv")]).t())
        self.a_log, self.dt_bias = self._f32(tensors["A_log"]), self._f32(tensors["dt_bias"])
        self.norm_w = self._f32(tensors["norm"])

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_h, self.w_a2, self.w_g2, self.w_o))

    def cache_spec(self):
        # one row per sequence: S as [heads, dim, vdim], then the convolution's last inputs
        return CacheSpec.state((self.n_state + self.n_conv,))

    def _narrow_product(self, cols, w, dt):
        # a bottleneck of a few columns: the CUDA-core product reads them where they lie; a wide one is copied out
        return ops.gemm_simt(cols, w, dt) if cols.shape[1] < 64 else ops.linear(cols.contiguous(), w, dt)

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        GN, HP, H, C = self.G * self.N, self.H * self.P, self.H, self.conv_channels
        proj = ops.linear(h, self.w_h, dt)
        qkv = ops.causal_conv(proj[:, :C], self.conv_w, None, cache.state[:, self.n_state:], step)
        b_raw = proj[:, C:C + H]
        a1, g1 = proj[:, C + H:C + H + self.r_a], proj[:, C + H + self.r_a:]
        z = self._narrow_product(a1, self.w_a2, dt)
        gate = self._narrow_product(g1, self.w_g2, dt)
        qn, kn, qk, decay, beta = ops.delta_prep(qkv[:, :GN], qkv[:, GN:2 * GN], z, b_raw, self.a_log, self.dt_bias,
                                                 self.l2_eps, self.N ** -0.5, H, self.N, heads_per_group=H // self.G)
        o = ops.delta_scan(qn, kn, qk, decay, beta, qkv[:, 2 * GN:], cache.state[:, :self.n_state], step, H, self.N,
                           self.P, heads_per_group=H // self.G)
        gated = ops.gated_norm(o, dt, weight=self.norm_w, eps=self.eps, group=self.P, weight_per_group=True, gate=gate,
                               gate_mode=ops.GATE_AFTER_NORM, activation="sigmoid")
        return ops.linear(gated, self.w_o, torch.float32, defer=True)
