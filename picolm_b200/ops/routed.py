"""A routed feed-forward's kernels: the router's choice, the sort of the chosen (token, expert) pairs by expert, the
experts' products over the sorted pairs, the weighted sum per token.  Nothing of the choice is read on the host: the
products run over a number of tiles that the sizes alone bound, so a step through them can be captured in a graph."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._lib import KernelError, _check, _dev, _dt, _fn, _i32, _p, _stream, status_word


def router_logits(h: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """h [T, K] times the few rows of w [E, K] (the experts' router rows, a gate's) as float32 [T, E]: float32 sums in an
    order that depends on K only."""
    _dev(h, "h"), _dev(w, "w")
    T, K = h.shape
    E = w.shape[0]
    if w.shape != (E, K):
        raise KernelError(f"router_logits: h is [{T}, {K}] but w is {tuple(w.shape)}")
    out = torch.empty((T, E), dtype=torch.float32, device=h.device)
    _check(_fn("routed", "plm_router_logits")(_p(h), _dt(h, "h"), _p(w), _dt(w, "w"), _p(out), T, E, K, _stream()),
           f"router_logits {T}x{E}x{K}", flops=2 * T * E * K, nbytes=h.numel() * h.element_size())
    return out


def route_topk(logits: torch.Tensor, n_experts: int, top: int, correction: Optional[torch.Tensor] = None,
               n_groups: int = 1, keep_groups: int = 1, scale: float = 1.0,
               gate_col: Optional[int] = None, scores: str = "sigmoid", group_score: str = "top2",
               normalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """The choice of `top` experts per token from router logits [T, >= n_experts] (float32): scores are
    `sigmoid(logit)` (`scores="softmax"`: the softmax over the n_experts logits); the choice goes by score +
    `correction` (float32 [n_experts]), among the experts of the
    `keep_groups` best of `n_groups` equal groups of neighbours (a group's score: the sum of its two largest choice
    scores, or with `group_score="max"` its largest); the weights are the chosen scores without the correction,
    divided by their sum (+ 1e-20) unless `normalize` is False, times `scale`.
    Returns (ids int32 [T, top], weights float32 [T, top], gate float32 [T] = sigmoid(logits[:, gate_col]) or None)."""
    _dev(logits, "logits")
    if logits.dtype != torch.float32 or logits.dim() != 2:
        raise KernelError("route_topk: the router's logits must be float32 [T, columns]")
    T, ld = logits.shape
    E = int(n_experts)
    if not (0 < top <= E <= ld) or n_groups <= 0 or E % n_groups or not 0 < keep_groups <= n_groups:
        raise KernelError(f"route_topk: top={top}, experts={E}, groups={n_groups}, kept={keep_groups} do not fit together")
    if correction is not None:
        _dev(correction, "correction")
        if correction.dtype != torch.float32 or correction.shape != (E,):
            raise KernelError("route_topk: correction must be float32 [experts]")
    if scores not in ("sigmoid", "softmax") or group_score not in ("top2", "max"):
        raise KernelError(f"route_topk: scores {scores!r} (sigmoid, softmax) or group_score {group_score!r} (top2, max) is not known")
    ids = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    gate = torch.empty((T,), dtype=torch.float32, device=logits.device) if gate_col is not None else None
    _check(_fn("routed", "plm_route_topk")(
        _p(logits), ld, _p(correction), E, int(top), int(n_groups), int(keep_groups), float(scale), _p(ids), _p(weights),
        _p(gate), int(gate_col or 0), T, 1 if scores == "softmax" else 0, 1 if group_score == "max" else 0,
        1 if normalize else 0, _stream()), f"route_topk T={T} E={E}")
    return ids, weights, gate


class SortedPairs:
    """The chosen (token, expert) pairs sorted into tiles of `bm` rows of one expert each: `sorted` int32
    [max_tiles * bm] (pair = token * top + k, or -1), `tile_expert` int32 [max_tiles] (or -1), `where` int32
    [T * top] (the row of `sorted` that holds the pair)."""
    __slots__ = ("sorted", "tile_expert", "where", "bm", "max_tiles", "top", "n_tokens")

    def __init__(self, sorted_, tile_expert, where, bm, max_tiles, top, n_tokens):
        self.sorted, self.tile_expert, self.where = sorted_, tile_expert, where
        self.bm, self.max_tiles, self.top, self.n_tokens = bm, max_tiles, top, n_tokens

    @property
    def rows(self) -> int:
        return self.max_tiles * self.bm


def moe_max_tiles(n_entries: int, n_experts: int, bm: int) -> int:
    """The most tiles of `bm` rows that `n_entries` pairs over `n_experts` experts fill."""
    return min(n_entries, (n_entries + n_experts * (bm - 1)) // bm)


def moe_align(ids: torch.Tensor, n_experts: int, bm: int, n_skip: int = 0) -> SortedPairs:
    """The chosen pairs `ids` [T, top] sorted by expert into tiles of `bm` rows.  Ids in [n_experts, n_experts + n_skip)
    (experts without tensors, whose output is their input) are left out of the sort: `where` holds -1 for them."""
    _i32(ids, "ids")
    T, top = ids.shape
    n = T * top
    max_tiles = moe_max_tiles(n, n_experts, bm)
    dev = ids.device
    sorted_ = torch.empty((max_tiles * bm,), dtype=torch.int32, device=dev)
    tile_expert = torch.empty((max_tiles,), dtype=torch.int32, device=dev)
    where = torch.empty((n,), dtype=torch.int32, device=dev)
    _check(_fn("routed", "plm_moe_align")(_p(ids), n, int(n_experts), int(bm), _p(tile_expert), _p(sorted_), _p(where),
                                          max_tiles, int(n_skip), _stream()), f"moe_align pairs={n} E={n_experts}")
    return SortedPairs(sorted_, tile_expert, where, bm, max_tiles, top, T)


def moe_gate_up(h: torch.Tensor, w_gate_up: torch.Tensor, pairs: SortedPairs, interleaved: bool = False) -> torch.Tensor:
    """silu(W_gate[e] h) * (W_up[e] h) for every sorted pair: `h` [T, d], `w_gate_up` [E, 2F, d] (an expert's F gate
    rows, then its F up rows; `interleaved`: 64 gate rows, their 64 up rows, and so on, as `interleave_gate_up` lays
    them out), both of one type; [rows, F] of that type, in sorted order.  bfloat16 with tiles of 16 rows runs on
    `mma.sync` (F a multiple of 8, d of 32), everything else on the CUDA cores."""
    _dev(h, "h"), _dev(w_gate_up, "w_gate_up")
    E, F2, d = w_gate_up.shape
    if h.dtype != w_gate_up.dtype or h.shape != (pairs.n_tokens, d) or F2 % 2:
        raise KernelError("moe_gate_up: h [T, d] and w_gate_up [E, 2F, d] of one type are expected")
    F = F2 // 2
    out = torch.empty((pairs.rows, F), dtype=h.dtype, device=h.device)
    _check(_fn("routed", "plm_moe_gemm")(
        _p(h), d, pairs.top, _p(w_gate_up), _p(out), F, _dt(h, "h"), 0, _p(pairs.tile_expert), _p(pairs.sorted),
        pairs.max_tiles, pairs.bm, F, d, 1 if interleaved else 0, _stream()),
        f"moe_gate_up tiles<={pairs.max_tiles}x{pairs.bm} F={F} d={d}",
        flops=2 * pairs.n_tokens * pairs.top * F2 * d, nbytes=w_gate_up.numel() * w_gate_up.element_size())
    return out


def moe_down(act: torch.Tensor, w_down: torch.Tensor, pairs: SortedPairs) -> torch.Tensor:
    """W_down[e] act for every sorted pair: `act` [rows, F] in sorted order, `w_down` [E, d, F]; float32 [rows, d]."""
    _dev(act, "act"), _dev(w_down, "w_down")
    E, d, F = w_down.shape
    if act.dtype != w_down.dtype or act.shape != (pairs.rows, F):
        raise KernelError("moe_down: act [rows, F] and w_down [E, d, F] of one type are expected")
    out = torch.empty((pairs.rows, d), dtype=torch.float32, device=act.device)
    _check(_fn("routed", "plm_moe_gemm")(
        _p(act), F, pairs.top, _p(w_down), _p(out), d, _dt(act, "act"), 1, _p(pairs.tile_expert), _p(pairs.sorted),
        pairs.max_tiles, pairs.bm, d, F, 0, _stream()), f"moe_down tiles<={pairs.max_tiles}x{pairs.bm} d={d} F={F}",
        flops=2 * pairs.n_tokens * pairs.top * F * d, nbytes=w_down.numel() * w_down.element_size())
    return out


def moe_gather(h: torch.Tensor, pairs: SortedPairs) -> torch.Tensor:
    """The tokens' rows in sorted order, [rows, d] (zero rows where a tile is not full): the left operand of a
    product that takes whole tiles."""
    _dev(h, "h")
    T, d = h.shape
    out = torch.empty((pairs.rows, d), dtype=h.dtype, device=h.device)
    _check(_fn("routed", "plm_moe_gather")(_p(h), _p(out), _p(pairs.sorted), pairs.rows, pairs.top, d * h.element_size(),
                                           _stream()), f"moe_gather rows={pairs.rows}", nbytes=2 * out.numel() * out.element_size())
    return out


def moe_combine(y: torch.Tensor, pairs: SortedPairs, weights: torch.Tensor, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None, ident: Optional[torch.Tensor] = None,
                add: Optional[torch.Tensor] = None, out_scale: float = 1.0,
                into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sum[t] = sum_k weights[t, k] * y[row of pair (t, k)] (+ gate[t] * shared[t]): float32 [T, d], k ascending.  A pair
    that the sort left out (an expert whose output is its input) enters as weights[t, k] * ident[t] (`ident` [T, d],
    float32 or the run's type).  Returns `out_scale * (sum + add)` (`add`: float32 [T, d] or None), or with `into`
    (float32 [T, d], the residual stream) adds that to it in place and returns it."""
    _dev(y, "y"), _dev(weights, "weights")
    d = y.shape[1]
    T, top = weights.shape
    if y.dtype != torch.float32 or weights.dtype != torch.float32 or y.shape[0] != pairs.rows or (T, top) != (pairs.n_tokens, pairs.top):
        raise KernelError("moe_combine: y float32 [rows, d] and weights float32 [T, top] are expected")
    for t, n, shape in ((shared, "shared", (T, d)), (gate, "gate", (T,))):
        if t is not None:
            _dev(t, n)
            if t.dtype != torch.float32 or tuple(t.shape) != shape:
                raise KernelError(f"moe_combine: {n} must be float32 {shape}")
    for t, n in ((add, "add"), (into, "into")):
        if t is not None:
            _dev(t, n)
            if t.dtype != torch.float32 or tuple(t.shape) != (T, d):
                raise KernelError(f"moe_combine: {n} must be float32 {(T, d)}")
    if ident is not None:
        _dev(ident, "ident")
        if tuple(ident.shape) != (T, d):
            raise KernelError(f"moe_combine: ident must be {(T, d)}")
    out = into if into is not None else torch.empty((T, d), dtype=torch.float32, device=y.device)
    _check(_fn("routed", "plm_moe_combine")(_p(y), d, _p(pairs.where), _p(weights), top, _p(shared), _p(gate), _p(out), T, d,
                                            _p(ident), _dt(ident, "ident") if ident is not None else 0, _p(add),
                                            float(out_scale), 1 if into is not None else 0,
                                            _stream()), f"moe_combine T={T} d={d}",
           nbytes=(top + 1 + (shared is not None) + (add is not None) + (into is not None)) * T * d * 4)
    return out


def moe_tc_supported(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> bool:
    """Whether the experts' products can run on tcgen05 (`moe_gate_up_tc`, `moe_down_tc`): bfloat16, an inner width
    that is a multiple of 64, rows that TMA can address."""
    E, F2, d = w_gate_up.shape
    F = F2 // 2
    return (h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
            and F % 64 == 0 and d % 8 == 0 and d >= 64 and w_gate_up.data_ptr() % 16 == 0 and w_down.data_ptr() % 16 == 0)


def _grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, pairs: SortedPairs, what: str) -> torch.Tensor:
    E, N, K = w.shape
    if pairs.bm != 128 or x.shape != (pairs.rows, K) or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError(f"{what}: tiles of 128 sorted rows [rows, {K}] in bfloat16 are expected")
    _check(_fn("gemm_tc_wide", "plm_gemm_tc_wide_grouped")(
        _p(x), _p(w), _p(out), _dt(out, "out"), epilogue, pairs.rows, N, K, K, K, out.shape[1], E, _p(pairs.tile_expert),
        _p(status_word(x.device)), _stream()), f"{what} tiles<={pairs.max_tiles}x128 N={N} K={K}",
        flops=2 * pairs.n_tokens * pairs.top * N * K, nbytes=w.numel() * 2)
    return out


def moe_gate_up_tc(x_sorted: torch.Tensor, w_gate_up: torch.Tensor, pairs: SortedPairs) -> torch.Tensor:
    """`moe_gate_up` on tcgen05 for tiles of 128 rows: `x_sorted` [rows, d] from `moe_gather`, `w_gate_up` [E, 2F, d]
    interleaved in turns of 64 rows; the activation in the product's epilogue; [rows, F] bfloat16."""
    _dev(x_sorted, "x_sorted"), _dev(w_gate_up, "w_gate_up")
    out = torch.empty((pairs.rows, w_gate_up.shape[1] // 2), dtype=torch.bfloat16, device=x_sorted.device)
    return _grouped(x_sorted, w_gate_up, out, 1, pairs, "moe_gate_up_tc")


def moe_down_tc(act: torch.Tensor, w_down: torch.Tensor, pairs: SortedPairs) -> torch.Tensor:
    """`moe_down` on tcgen05 for tiles of 128 rows; float32 [rows, d]."""
    _dev(act, "act"), _dev(w_down, "w_down")
    out = torch.empty((pairs.rows, w_down.shape[1]), dtype=torch.float32, device=act.device)
    return _grouped(act, w_down, out, 0, pairs, "moe_down_tc")
