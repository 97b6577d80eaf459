"""Attention through a latent: keys and values of all heads are linear maps of one short row per position
(`c = RMSNorm(W_dkv h)`), and that row is all the cache keeps.

The products with the per-head maps are moved to the query's side, so that no key or value is ever made:
`q_h . (U_k,h c_j) = (U_k,h^T q_h) . c_j` and `sum_j p_j (U_v,h c_j) = U_v,h (sum_j p_j c_j)`.  What runs over the
cache is therefore attention of `heads` query heads of size kv_rank over ONE key head whose values are its keys,
which the library's attention kernels do as they stand (paged cache, sliding window, ragged steps).
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.sequence_cache import KVLayerCache
from ..cache.spec import CacheSpec
from .base import Part, WeightSpec, register_part
from .mixer import _stack_rows


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    """params: hidden_size, heads, dim (query/key size of a head), vdim, kv_rank, q_rank, scale, window (None: all
    keys), eps.  No position encoding.  Queries go through a latent too (`q = W_uq RMSNorm(W_dq h)`); the
    concatenated heads are multiplied by `sigmoid(W_g h)` before the output projection.

    Tensors: dq [q_rank, hidden], dq.norm [q_rank], uq [heads dim, q_rank], dkv [kv_rank, hidden], dkv.norm [kv_rank],
    uk [heads dim, kv_rank], uv [heads vdim, kv_rank], g [heads vdim, hidden], o [hidden, heads vdim]."""

    graph_safe = True
    graph_safe_prompts = True       # padding tokens of a captured prompt step write the null page and are attended by nobody

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.d, self.H, self.dk, self.dv = p["hidden_size"], p["heads"], p["dim"], p["vdim"]
        self.R, self.Rq, self.scale, self.window = p["kv_rank"], p["q_rank"], float(p["scale"]), p.get("window")
        self.eps = float(p["eps"])

    def weight_specs(self):
        H, dk, dv, R, Rq, d = self.H, self.dk, self.dv, self.R, self.Rq, self.d
        return {
            "dq": WeightSpec((Rq, d)), "dq.norm": WeightSpec((Rq,), init="ones_normal"), "uq": WeightSpec((H * dk, Rq)),
            "dkv": WeightSpec((R, d)), "dkv.norm": WeightSpec((R,), init="ones_normal"),
            "uk": WeightSpec((H * dk, R)), "uv": WeightSpec((H * dv, R)),
            "g": WeightSpec((H * dv, d)), "o": WeightSpec((d, H * dv)),
        }

    def load(self, tensors):
        H, dk, dv, R = self.H, self.dk, self.dv, self.R
        # one projection for everything that reads h: rows [dq | dkv | g]
        self.w_h = _stack_rows([tensors["dq"], tensors["dkv"], tensors["g"]])
        self.w_uq, self.w_o = tensors["uq"], tensors["o"]
        self.q_norm_w = tensors["dq.norm"].to(torch.float32).contiguous()
        self.c_norm_w = tensors["dkv.norm"].to(torch.float32).contiguous()
        # per head: U_k^T [kv_rank, dim] takes a query into the latent's space, U_v [vdim, kv_rank] brings the result back
        self.w_absorb = tensors["uk"].view(H, dk, R).transpose(1, 2).contiguous()
        self.w_expand = tensors["uv"].view(H, dv, R).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_h, self.w_uq, self.w_absorb, self.w_expand, self.w_o))

    def cache_spec(self):
        return CacheSpec.kv(1, self.R, self.window, values=False)

    def forward(self, h, step, cache):
        dt = self.runtime.dtype
        Rq, R = self.Rq, self.R
        proj = ops.linear(h, self.w_h, dt)
        c_q = ops.gated_norm(proj[:, :Rq], dt, weight=self.q_norm_w, eps=self.eps)
        c = ops.gated_norm(proj[:, Rq:Rq + R], dt, weight=self.c_norm_w, eps=self.eps)
        if cache.writable:
            ops.store_rows_paged(c, cache.k, step, cache.block_table)
        q = ops.linear(c_q, self.w_uq, dt)
        q_lat = ops.head_linear(q, self.w_absorb).view(h.shape[0], self.H, R)
        latent = KVLayerCache(cache.k, cache.k, cache.block_table, cache.window, cache.writable)
        o_lat = ops.attention(q_lat, latent, step, 1, self.scale)
        ctx = ops.head_linear(o_lat, self.w_expand, gate=proj[:, Rq + R:])
        return ops.linear(ctx, self.w_o, torch.float32, defer=True)
