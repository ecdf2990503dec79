"""Attention through a latent: keys and values of all heads are linear maps of one short row per position
(`c = RMSNorm(W_dkv h)`), and that row (with, in some designs, one rotated key part that the heads share) is all the
cache keeps.

The products with the per-head maps are moved to the query's side, so that no key or value is ever made:
`q_h . (U_k,h c_j) = (U_k,h^T q_h) . c_j` and `sum_j p_j (U_v,h c_j) = U_v,h (sum_j p_j c_j)`.  What runs over the
cache is therefore attention of `heads` query heads of size kv_rank over ONE key head whose values are its keys,
which the library's attention kernels do as they stand (paged cache, sliding window, ragged steps).  A rotated
part rides along: the cache's row is [rotated key part | c], a head's query [rotated query part | U_k^T q], their
product the sum of both scores, and of the attention's result only the columns behind the rotated part are used.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.sequence_cache import KVLayerCache
from ..cache.spec import CacheSpec
from .base import Part, WeightSpec, build_part, register_part
from .mixer import _stack_rows


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: hidden_size, heads, dim (query/key size of a head), vdim, kv_rank, q_rank, scale, window (None: all
    keys), eps.  Queries go through a latent too (`q = W_uq RMSNorm(W_dq h)`); the concatenated heads are multiplied
    by `sigmoid(W_g h)` before the output projection.

    Optional, for designs that have them (absent: no position encoding, the plain softmax, a gate per element):
      rot_dim       every head's query has `rot_dim` more components behind its `dim`, and `W_dkv` has `rot_dim` more
                    rows behind its kv_rank (not normed): one key part that all heads share.  Both are rotated by the
                    position (`position`: a PartSpec of the position family over rot_dim components) and their product
                    is added to the head's score.  The cache keeps the rotated key part in front of the latent.
      chunk         a mask of chunks of that many positions instead of a window (see `ops.key_mask`)
      sink_name     a tensor [heads]: head h's denominator also holds exp(sink[h])
      gate_per_head True: `W_g` is [heads, hidden] and head h's output is multiplied by sigmoid(W_g h)_h

    Tensors: dq [q_rank, hidden], dq.norm [q_rank], uq [heads (dim + rot_dim), q_rank], dkv [kv_rank + rot_dim, hidden],
    dkv.norm [kv_rank], uk [heads dim, kv_rank], uv [heads vdim, kv_rank], g [heads vdim or heads, hidden], o [hidden,
    heads vdim]."""

    graph_safe = True
    graph_safe_prompts = True       # padding tokens of a captured prompt step write the null page and are attended by nobody

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.H, self.dk, self.dv = p["hidden_size"], p["heads"], p["dim"], p["vdim"]
        self.R, self.Rq, self.scale, self.window = p["kv_rank"], p["q_rank"], float(p["scale"]), p.get("window")
        self.eps = float(p["eps"])
        self.rot = int(p.get("rot_dim") or 0)
        self.chunk = p.get("chunk")
        if self.chunk is not None and (self.window is not None or int(self.chunk) <= 0):
            raise ValueError("a mask of chunks needs a positive size and excludes a sliding window")
        self.sink_name = p.get("sink_name")
        self.gate_per_head = bool(p.get("gate_per_head", False))
        self.position = None
        if self.rot:
            if p.get("position") is None:
                raise ValueError("latent_attention: a rotated part needs a position encoding")
            self.position = build_part("position", p["position"], runtime)
            if not hasattr(self.position, "rotation"):
                raise ValueError("latent_attention: the position encoding must be a rotation")
        # what a position keeps: [rotated key part | latent], padded to a width the attention kernels take
        self.row = self.rot + self.R
        self.hd_c = -(-self.row // 16) * 16 if self.rot else self.R

    def weight_specs(self):
        H, dk, dv, R, Rq, d, rot = self.H, self.dk, self.dv, self.R, self.Rq, self.d, self.rot
        specs = {
            "dq": WeightSpec((Rq, d)), "dq.norm": WeightSpec((Rq,), init="ones_normal"), "uq": WeightSpec((H * (dk + rot), Rq)),
            "dkv": WeightSpec((R + rot, d)), "dkv.norm": WeightSpec((R,), init="ones_normal"),
            "uk": WeightSpec((H * dk, R)), "uv": WeightSpec((H * dv, R)),
            "g": WeightSpec((H if self.gate_per_head else H * dv, d)), "o": WeightSpec((d, H * dv)),
        }
        if self.sink_name is not None:
            specs[self.sink_name] = WeightSpec((H,), init="normal_scaled", scale=1.0)
        return specs

    def load(self, tensors):
        H, dk, dv, R, rot, hd_c = self.H, self.dk, self.dv, self.R, self.rot, self.hd_c
        dkv = tensors["dkv"]
        # one projection for everything that reads h: rows [dq | rotated key part | latent | g]
        self.w_h = _stack_rows([tensors["dq"], dkv[R:], dkv[:R], tensors["g"]])
        self.w_uq, self.w_o = tensors["uq"], tensors["o"]
        self.q_norm_w = tensors["dq.norm"].to(torch.float32).contiguous()
        self.c_norm_w = tensors["dkv.norm"].to(torch.float32).contiguous()
        self.sink = None if self.sink_name is None else tensors[self.sink_name].to(torch.float32).contiguous()
        # per head: [I | U_k^T] takes a query [dim | rot] to [rot | kv_rank] (the rotated part passes, in front; the
        # rest into the latent's space), U_v [vdim, kv_rank] brings the result back from behind the rotated part
        uk, uv = tensors["uk"].view(H, dk, R), tensors["uv"].view(H, dv, R)
        absorb = torch.zeros((H, hd_c, dk + rot), dtype=uk.dtype, device=uk.device)
        absorb[:, rot:rot + R, :dk] = uk.transpose(1, 2)
        if rot:
            absorb[:, :rot, dk:] = torch.eye(rot, dtype=uk.dtype, device=uk.device)
        expand = torch.zeros((H, dv, hd_c), dtype=uv.dtype, device=uv.device)
        expand[:, :, rot:rot + R] = uv
        self.w_absorb, self.w_expand = absorb.contiguous(), expand.contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_h, self.w_uq, self.w_absorb, self.w_expand, self.w_o))

    def cache_spec(self):
        return CacheSpec.kv(1, self.hd_c, self.window, values=False)

    def prepare(self, max_seq_tokens: int) -> None:
        if self.position is not None:
            self.position.prepare(max_seq_tokens)

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        Rq, row = self.Rq, self.row
        rotation = self.position.rotation() if self.position is not None else None
        # norms and the rotation work on the float32 sums where there is a rotated part
        proj = ops.linear(h, self.w_h, torch.float32 if self.rot else dt)
        # the queries' latent is normed by the kernel that makes the cache's row
        c_q = ops.latent_store(proj[:, Rq:Rq + row], self.c_norm_w, self.eps, rotation, self.rot, cache.k, step, cache.block_table,
                               store=cache.writable, q_rows=proj[:, :Rq], q_weight=self.q_norm_w)
        q = ops.linear(c_q, self.w_uq, dt)
        q_lat = ops.head_linear(q, self.w_absorb)
        if self.rot:
            ops.rope_rows(q_lat, rotation, step.tok_pos, self.H, self.hd_c)
        latent = KVLayerCache(cache.k, cache.k, cache.block_table, cache.window, cache.writable)
        o_lat = ops.attention(q_lat.view(h.shape[0], self.H, self.hd_c), latent, step, 1, self.scale, chunk=self.chunk,
                              sink=self.sink)
        ctx = ops.head_linear(o_lat, self.w_expand, gate=proj[:, Rq + row:], gate_per_head=self.gate_per_head)
        return ops.linear(ctx, self.w_o, torch.float32, defer=True)
