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
                       num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, own_kv: bool = True) -> None:
    """What stands between a QKV product and attention where queries and keys are normalised over all their heads at
    once: per token, in fp32, `q + bias` and `k + bias` are divided by their root mean square over ALL their columns
    and multiplied by `q_norm` / `k_norm` (None: no norm), the leading `rotation.rotary_dim` components of every head
    are rotated by the token's position, `v + bias` passes.  `qkv` [T, H*D (+ G*D + G*Dv)] float32 or the run's type;
    queries go to `q_out` [T, H, hd_c], keys and values (`own_kv`) into the pages of `kv` (a `KVLayerCache` whose
    head size hd_c >= D, Dv: what lies beyond a head's own width is written as zero).  `rotation`: `ops.Rotation` or
    None."""
    _dev(qkv, "qkv"), _dev(q_out, "q_out")
    _i32(step.tok_pos, "tok_pos"), _i32(step.tok_seq, "tok_seq"), _i32(kv.block_table, "block_table")
    T = qkv.shape[0]
    H, G, D, Dv = num_heads, num_kv_heads, key_dim, value_dim
    hd_c = q_out.shape[2]
    cols = H * D + ((G * D + G * Dv) if own_kv else 0)
    if qkv.shape != (T, cols) or q_out.shape != (T, H, hd_c):
        raise KernelError("qk_norm_rope_store: qkv / q_out shapes do not match the head counts")
    if own_kv:
        for c, n in ((kv.k, "k_cache"), (kv.v, "v_cache")):
            _dev(c, n)
            if c.dtype != q_out.dtype or c.shape[1:] != (G, PAGE_TOKENS, hd_c):
                raise KernelError(f"qk_norm_rope_store: {n} must be [pages, {G}, {PAGE_TOKENS}, {hd_c}] of {q_out.dtype}")
    if bias is not None and (bias.dtype != torch.float32 or bias.shape != (cols,) or not bias.is_cuda):
        raise KernelError("qk_norm_rope_store: bias must be float32, one per column of qkv")
    for wn, n, size in ((q_norm, "q_norm", H * D), (k_norm if own_kv else None, "k_norm", G * D)):
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
        0 if pairing == "half" else 1, 1 if own_kv else 0, _stream()), f"qk_norm_rope_store T={T}",
        nbytes=qkv.numel() * qkv.element_size() + T * (H + (2 * G if own_kv else 0)) * hd_c * q_out.element_size())
