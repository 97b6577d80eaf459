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
