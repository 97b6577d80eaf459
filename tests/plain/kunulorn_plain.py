"""A plain, slow implementation of the Kunulorn design: one function per
mechanism, written from the design's equations.  It shares no code with
picolm_b200 (it has its own safetensors reader) and runs on the CPU in float64
or float32.

The design in this file's notation.  Token embedding times a constant; layers
listed one by one in config.json, each `x += mixer(LN1(x))` and then, if the
layer has a feed-forward, `x += ff(LN2(x))`, LN a layer norm with a weight and no
bias; attention with biased projections, an RMS norm over the whole of q and of
k, a rotation of the leading components of every head in neighbouring pairs, a
mask of chunks, grouped key/value heads whose keys and values may have different
widths, and layers that read another layer's keys and values; a dense
feed-forward with clamped branches, or a routed one (sigmoid scores, a
correction for the choice only, groups of experts, a shared expert behind a
sigmoid gate); final layer norm; logits against the embedding table.

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
def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis, var the mean squared deviation."""
    mu = x.mean(dim=-1, keepdim=True)
    var = ((x - mu) ** 2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def rotate_pairs(x, positions, dims, base):
    """x [T, heads, size]: components (2i, 2i+1), i < dims/2, of every head turned by the angle
    position * base^(-2i/dims); the components from `dims` on stay."""
    T = x.shape[0]
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = torch.as_tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    ang = torch.as_tensor(positions, dtype=x.dtype)[:, None] * freq[None, :]            # [T, dims/2]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def chunk_mask(T, size):
    """[T, T] True where query i sees key j: j <= i and both in the same chunk of `size` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


# --------------------------------------------------------------------- attention
def attention_keys_values(h, W, m, eps):
    """What a layer keeps: keys after norm and rotation [T, G, dim], values [T, G, vdim]."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = h @ W["k"].T + W["k.b"]
    v = h @ W["v"].T + W["v.b"]
    k = rms_norm(k, W["k.norm"], eps).reshape(T, G, D)
    if m.get("rot") is not None:                            # (a mixer whose configuration names no rotation has none)
        k = rotate_pairs(k, list(range(T)), m["rot"]["dims"], m["rot"]["base"])
    return k, v.reshape(T, G, Dv)


def attention(h, W, m, eps, keys_values=None):
    """The mixer.  `keys_values`: another layer's (keys, values) for a layer that has none of its own."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ W["q"].T + W["q.b"]
    q = rms_norm(q, W["q.norm"], eps).reshape(T, H, D)
    if m.get("rot") is not None:
        q = rotate_pairs(q, list(range(T)), m["rot"]["dims"], m["rot"]["base"])
    k, v = keys_values if keys_values is not None else attention_keys_values(h, W, m, eps)
    # (a mixer whose configuration names no mask sees every earlier key: one chunk as long as the sequence)
    mask = chunk_mask(T, m["mask"]["size"] if m.get("mask") is not None else max(T, 1))
    out = torch.zeros(T, H, Dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head, :] = torch.softmax(s, dim=-1) @ v[:, g, :]
    return out.reshape(T, H * Dv) @ W["o"].T + W["o.b"], (k, v)


# ------------------------------------------------------------------ feed-forward
def dense_feed_forward(h, W, limit):
    g = torch.clamp(h @ W["gate"].T, max=limit)
    u = torch.clamp(h @ W["up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W["down"].T


def expert(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def route(h, w_router, correction, r):
    """Per token: the chosen experts [T, top] and their weights [T, top]."""
    E, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w_router.T)                       # [T, E]
    choice = s + correction
    groups = r.get("groups")
    if groups is not None:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        by_group = choice.reshape(-1, n, per)
        gscore = by_group.topk(min(2, per), dim=-1).values.sum(dim=-1)      # [T, n]
        best = gscore.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20) * r["scale"]
    return idx, w


def routed_feed_forward(h, W, mlp):
    r = mlp["router"]
    idx, w = route(h, W["router"], W["correction"], r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), w[t]):
            out[t] += a * expert(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if mlp.get("shared") is not None:
        gate = torch.sigmoid(h @ W["shared.sg"].T)          # [T, 1]
        out = out + gate * expert(h, W["shared.gate"], W["shared.up"], W["shared.down"])
    return out


def feed_forward(h, W, mlp):
    if mlp["kind"] == "dense":
        return dense_feed_forward(h, W, mlp["limit"])
    if mlp["kind"] == "moe":
        return routed_feed_forward(h, W, mlp)
    raise ValueError(mlp["kind"])


# ------------------------------------------------------------------------- model
def _sub(tensors, prefix, dtype):
    n = len(prefix)
    return {k[n:]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def forward(tensors, cfg, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence from its first token; `layers_out` (a list) receives the stream after
    every layer."""
    eps = cfg["norm"]["eps"]
    embed = tensors["embed"].to(dtype)
    x = embed[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, tensors[p + "norm1"].to(dtype), eps)
        src = m.get("kv_from")
        delta, kv = attention(h, _sub(tensors, p + "mix.", dtype), m, eps, kept[src] if src is not None else None)
        kept[i] = kv
        x = x + delta
        if layer.get("mlp") is not None:
            h = layer_norm(x, tensors[p + "norm2"].to(dtype), eps)
            x = x + feed_forward(h, _sub(tensors, p + "mlp.", dtype), layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    h = layer_norm(x, tensors["final.norm"].to(dtype), eps)
    return h @ embed.T
