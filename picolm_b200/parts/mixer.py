"""Mixers: the part of a layer that lets tokens see other tokens.

Interface of the family: `cache_spec()` says what the layer needs of the cache
(`CacheSpec.kv`, `CacheSpec.state` or None); `prepare(max_seq_tokens)` runs once
before the first step; `forward(h, step, cache)` takes the normed activations
[T, d] of the step's tokens and returns the residual delta [T, d] in fp32.

Attention as the reference computes it: q/k/v projections without bias, RoPE on
q and k, keys and values appended to the cache, causal softmax(q.K * scale) . V
with consecutive query heads sharing a KV head (`g = h / (H/G)`), then the output
projection (picolm/model_core.c:1849-2151, picolm/model_attention.c:43-140).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..cache.spec import CacheSpec
from ..config.spec import PartSpec
from .base import Part, WeightSpec, build_part, register_part
from .stream import BiasedDelta


def _stack_rows(tensors):
    """Concatenate weight matrices along the output features.  If their stored
    types differ, all are widened to float32 (exact)."""
    if len({t.dtype for t in tensors}) > 1:
        tensors = [t.to(torch.float32) for t in tensors]
    return torch.cat(list(tensors), dim=0).contiguous()


@register_part("mixer", "attention")
class Attention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, scale (None:
    1/sqrt(head_dim)), window (None: all keys), position (a PartSpec of the
    position family), q_name/k_name/v_name/o_name (relative tensor names).

    Optional, for designs that have them (absent: the reference's attention):
      value_dim     width of a value head where it differs from head_dim (the keys' and queries')
      chunk         a mask of chunks: a query sees the earlier keys of its own chunk of that many positions, chunks
                    counted from position 0 of the sequence
      bias          True: q, k, v and o have biases, tensors `<name><bias_suffix>` (default ".b")
      qk_norm       {"eps", "q_name", "k_name"}: queries and keys are divided by their root mean square over ALL heads
                    at once and multiplied by those weights ([H * head_dim], [G * head_dim]), after the bias and
                    before the rotation
      own_kv        False: the layer has no key and value tensors (projections, biases, key norm); it attends over
                    what the layer it borrows its cache from wrote
    With any of value_dim, bias, qk_norm or own_kv=False, what stands between the QKV product and attention is one
    kernel (`ops.qk_norm_rope_store`: bias, norm and rotation in float32 on the product's float32 result) and the
    cache keeps heads of one width, max(head_dim, value_dim) rounded up to 16, the narrower of keys and values padded
    with zeros (the output projection's columns are padded likewise, once, when the weights are loaded)."""

    @property
    def graph_safe(self) -> bool:
        """forward() launches kernels whose dependence on the step goes through device buffers only (apart
        from sizes fixed per batch size); the position encoding has to say the same of itself."""
        return bool(getattr(self.position, "graph_safe", False))

    @property
    def graph_safe_prompts(self) -> bool:
        return bool(getattr(self.position, "graph_safe_prompts", False))

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = self.params
        self.H, self.G, self.hd, self.d = p["num_heads"], p["num_kv_heads"], p["head_dim"], p["hidden_size"]
        if self.H % self.G:
            raise ValueError(f"num_heads={self.H} is not a multiple of num_kv_heads={self.G}")
        self.scale = float(p["scale"]) if p.get("scale") is not None else 1.0 / math.sqrt(self.hd)
        self.window = p.get("window")
        self.chunk = p.get("chunk")
        if self.chunk is not None and (self.window is not None or int(self.chunk) <= 0):
            raise ValueError("a mask of chunks needs a positive size and excludes a sliding window")
        self.vd = int(p.get("value_dim") or self.hd)
        self.bias = bool(p.get("bias", False))
        self.qk_norm = p.get("qk_norm")
        self.own_kv = bool(p.get("own_kv", True))
        # the general form: its own kernel between the product and attention, a cache of padded heads
        self.general = self.vd != self.hd or self.bias or self.qk_norm is not None or not self.own_kv
        self.hd_c = -(-max(self.hd, self.vd) // 16) * 16 if self.general else self.hd
        pos = p.get("position") or PartSpec("none")
        self.position = build_part("position", pos, runtime)
        if self.general and not hasattr(self.position, "rotation") and pos.kind != "none":
            raise ValueError(f"attention with a bias, a norm of q and k or values of another width needs a position "
                             f"encoding that is a rotation (or none), not {pos.kind!r}")

    def _names(self):
        """(tensor names of the projections that feed attention, in the order of their rows in the one product)."""
        p = self.params
        return [p["q_name"]] + ([p["k_name"], p["v_name"]] if self.own_kv else [])

    def weight_specs(self):
        p, H, G, hd, vd, d = self.params, self.H, self.G, self.hd, self.vd, self.d
        specs = {p["q_name"]: WeightSpec((H * hd, d)), p["o_name"]: WeightSpec((d, H * vd))}
        if self.own_kv:
            specs[p["k_name"]] = WeightSpec((G * hd, d))
            specs[p["v_name"]] = WeightSpec((G * vd, d))
        if self.bias:
            sfx = p.get("bias_suffix", ".b")
            for name in self._names() + [p["o_name"]]:
                specs[name + sfx] = WeightSpec((specs[name].shape[0],), init="normal")
        if self.qk_norm is not None:
            specs[self.qk_norm["q_name"]] = WeightSpec((H * hd,), init="ones_normal")
            if self.own_kv:
                specs[self.qk_norm["k_name"]] = WeightSpec((G * hd,), init="ones_normal")
        return specs

    def load(self, tensors):
        p = self.params
        # one projection for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = _stack_rows([tensors[n] for n in self._names()])
        self.w_o = tensors[p["o_name"]]
        self.b_qkv = self.b_o = self.w_qn = self.w_kn = None
        if self.bias:
            sfx = p.get("bias_suffix", ".b")
            self.b_qkv = torch.cat([tensors[n + sfx].to(torch.float32) for n in self._names()]).contiguous()
            self.b_o = tensors[p["o_name"] + sfx].to(torch.float32).contiguous()
        if self.qk_norm is not None:
            self.w_qn = tensors[self.qk_norm["q_name"]].to(self.runtime.dtype).contiguous()
            if self.own_kv:
                self.w_kn = tensors[self.qk_norm["k_name"]].to(self.runtime.dtype).contiguous()
        if self.general and self.hd_c != self.vd:
            # attention hands back heads of the cache's width: the columns beyond a value head's own meet zeros
            w = torch.zeros((self.d, self.H, self.hd_c), dtype=self.w_o.dtype, device=self.w_o.device)
            w[:, :, :self.vd] = self.w_o.view(self.d, self.H, self.vd)
            self.w_o = w.view(self.d, self.H * self.hd_c).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def cache_spec(self):
        # (chunks: pages are kept; a layer that borrows this cache may cut its chunks elsewhere)
        return CacheSpec.kv(self.G, self.hd_c, self.window)

    def prepare(self, max_seq_tokens: int) -> None:
        self.position.prepare(max_seq_tokens)

    takes_scaled_rows = True          # h goes into a product and nowhere else

    def _forward_general(self, h, step, cache):
        dt = self.runtime.dtype
        if self.own_kv and not cache.writable:
            raise RuntimeError("a layer that reads another layer's cache must be built with own_kv=False")
        qkv = ops.linear(h, self.w_qkv, torch.float32)       # bias, norm and rotation work on the float32 sums
        q = torch.empty((h.shape[0], self.H, self.hd_c), dtype=dt, device=h.device)
        rotation = self.position.rotation() if hasattr(self.position, "rotation") else None
        ops.qk_norm_rope_store(qkv, self.b_qkv, self.w_qn, self.w_kn, self.qk_norm["eps"] if self.qk_norm else 0.0, q,
                               cache, rotation, step, self.H, self.G, self.hd, self.vd, own_kv=self.own_kv)
        ctx = ops.attention(q, cache, step, self.G, self.scale, chunk=self.chunk)
        delta = ops.linear(ctx, self.w_o, torch.float32, defer=True)
        return BiasedDelta(delta, self.b_o) if self.b_o is not None else delta

    def forward(self, h, step, cache):
        if self.general:
            return self._forward_general(h, step, cache)
        dt = self.runtime.dtype
        qkv = ops.linear(h, self.w_qkv, dt)
        # a position encoding that can describe itself as a rotation (`rotation()`) may be applied, and the
        # cache written, by the decode attention kernel itself
        rotation = (self.position.rotation() if step.is_decode and not self.chunk and hasattr(self.position, "rotation")
                    else None)
        if rotation is not None and ops.attention_decode_rope_supported(qkv, cache, rotation, self.hd):
            ctx = ops.attention_decode_rope(qkv, cache, step, self.H, self.G, self.hd, self.scale, rotation)
        else:
            q = torch.empty((h.shape[0], self.H, self.hd), dtype=dt, device=h.device)
            self.position.apply(qkv, q, cache, step, self.H, self.G, self.hd)
            ctx = ops.attention(q, cache, step, self.G, self.scale, chunk=self.chunk)
        return ops.linear(ctx, self.w_o, torch.float32, defer=True)
