"""A plain, slow implementation of the Potuzen design: one function per
mechanism, written from the design's equations, token by token where the design
is recurrent.  It shares no code with picolm_b200 (it has its own safetensors
reader) and runs on the CPU in float64 or float32.

Notation.  `h` is a mixer's input [T, width] for ONE sequence whose first row is
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
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def dense_feed_forward(h, w_gate, w_up, w_down):
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


# -------------------------------------------------------------- latent attention
def latent_attention(h, W, m, eps):
    """`W`: the mixer's tensors by their short names; `m`: its sizes and constants."""
    T = h.shape[0]
    H, dk, dv, window, scale = m["heads"], m["dim"], m["vdim"], m["mask"]["size"], m["scale"]
    c_q = rms_norm(h @ W["dq"].T, W["dq.norm"], eps)
    q = (c_q @ W["uq"].T).view(T, H, dk)
    c = rms_norm(h @ W["dkv"].T, W["dkv.norm"], eps)              # [T, kv_rank]: all that a cache must hold
    k = (c @ W["uk"].T).view(T, H, dk)
    v = (c @ W["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - window + 1)                               # 0 <= i - j < window
        s = torch.einsum("hd,jhd->hj", q[i], k[lo:i + 1]) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("hj,jhd->hd", p, v[lo:i + 1])
    gate = torch.sigmoid(h @ W["g"].T)
    return (out.reshape(T, H * dv) * gate) @ W["o"].T


# ----------------------------------------------------------------------- mamba2
def causal_conv(u, w, b):
    """u [T, C]; w [C, taps], the last column being the current token's; zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for t in range(T):
        out[t] = (padded[t:t + taps].T * w).sum(dim=1) + b
    return out


def mamba2(h, W, m, eps):
    T = h.shape[0]
    H, P, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    zxbcdt = h @ W["in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W["dt_bias"])                              # [T, H], no clamp
    rate = torch.exp(W["A_log"])                                  # [H]
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = torch.exp(-rate[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)                             # the gate comes before the norm
    y = rms_norm(y.view(T, ng, inner // ng), None, eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


# -------------------------------------------------------------------------- gla
def gla(h, W, m, eps):
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ W["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ W["k"].T).view(T, H, dk)
    v = (h @ W["v"].T).view(T, H, dv)
    zz = (h @ W["a1"].T) @ W["a2"].T + W["a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(zz) / tau).view(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, W["norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ W["g"].T)) @ W["o"].T


MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2, "gla": gla}


# -------------------------------------------------------------------- the model
def layer_tensors(tensors, config, i, dtype):
    """The tensors of layer i (those of layer `weights_of` where it has none), split into norms, mixer, mlp."""
    j = config["layers"][i].get("weights_of", i)
    pre = f"l{j}."
    own = {n[len(pre):]: t.to(dtype) for n, t in tensors.items() if n.startswith(pre)}
    mix = {n[4:]: t for n, t in own.items() if n.startswith("mix.")}
    mlp = {n[4:]: t for n, t in own.items() if n.startswith("mlp.")}
    return own, mix, mlp


def forward(tensors, config, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence run from its first token.  `layers_out`, if a list, receives
    the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = tensors["embed"].to(dtype)[torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        own, mix, mlp = layer_tensors(tensors, config, i, dtype)
        delta = MIXERS[layer["type"]](rms_norm(x, own["norm1"], eps), mix, layer["mixer"], eps)
        x = x + rms_norm(delta, own["norm1b"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            delta = dense_feed_forward(rms_norm(x, own["norm2"], eps), mlp["gate"], mlp["up"], mlp["down"])
            x = x + rms_norm(delta, own["norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, tensors["final.norm"].to(dtype), eps) @ tensors["head"].to(dtype).T
