"""The Kunulorn design through the library, against the plain implementation in
`tests/plain/kunulorn_plain.py`: each mechanism alone (kernels against plain functions), whole models in
every cut (prompts against token-by-token decoding, portions down to two tokens, batches of unequal
requests, slots and pages used again), chunk edges and page borders, far keys inside a long chunk, sizes
that make special cases (one kv head, one group, groups of one expert, one choice, no shared expert, no
feed-forward, values wider and narrower than keys, a rotation of part of a head, a width no tensor map
takes), and greedy generation through the library's entry point.

Weights are random; where random weights would hide a fault they are reshaped: the attention's scale is
raised so that the softmax is peaked (one key at a chunk's edge then decides a row of logits).
"""
import json
import math
import os

import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import kunulorn_plain as P
from util import random_tokens

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-4          # of the logits' spread; two float32 computations in different orders of summation
DEV = "cuda:0"


def _attn(heads=4, kv_heads=2, dim=16, vdim=24, chunk=7, scale=0.9, rot=8, base=300.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk},
         "rot": {"base": base, "dims": rot}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _dense(ff=56, limit=0.7):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(experts=6, top=2, ff=20, scale=1.25, groups=(3, 2), shared=28):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        out["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def _config(layers, width=40, vocab=97, eps=1e-5, embed_scale=3.5):
    out = []
    for layer in layers:
        layer = dict(layer)
        layer.setdefault("mlp", _dense())
        out.append(layer)
    return {"architecture": "Kunulorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "layers": out}


def _make(tmp_path, name, config, seed, std=0.12):
    """A model folder with random weights for `config`; returns (folder, plain tensors, config)."""
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors, save_safetensors
    cfg = config_from_dict(config)
    tensors = random_tensors(cfg, seed, std=std, norm_std=0.2)
    d = str(tmp_path / name)
    os.makedirs(d, exist_ok=True)
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    return d, P.read_safetensors(os.path.join(d, "model.safetensors")), cfg.to_dict()


def _plain(tensors, config, tokens, dtype=torch.float64):
    return P.forward(tensors, config, tokens, dtype).to(torch.float32)


def _close(got, want, tol=FP32_TOL, what=""):
    err = (got.double() - want.double()).abs().max().item()
    spread = want.double().std().item()
    assert err <= tol * spread, f"{what}: max |diff| {err:.3e} is {err / spread:.2e} of the logits' spread (limit {tol})"


def _engine(d, dtype="float32", max_tokens=64 * 40, **kw):
    from picolm_b200.engine import Engine
    return Engine.from_folder(d, dtype=dtype, max_tokens=max_tokens, **kw)


# ------------------------------------------------------------------------------------------- kernels alone
class _Step:
    """What the kernels read of a step, for sequences that bring `lens` tokens each from position `starts`."""

    def __init__(self, lens, starts=None, dev=DEV):
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + n)
        i32 = dict(dtype=torch.int32, device=dev)
        starts = starts or [0] * len(lens)
        self.n_seqs, self.n_tokens, self.max_new = len(lens), offs[-1], max(lens)
        self.is_decode = all(n == 1 for n in lens)
        self.max_position = max(s + n for s, n in zip(starts, lens)) - 1
        self.seq_start = torch.tensor(offs, **i32)
        self.seq_kv_len = torch.tensor([s + n for s, n in zip(starts, lens)], **i32)
        self.tok_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], **i32)
        self.tok_pos = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], **i32)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [37, 200, 2304])
def test_layer_norm_kernel(out_dtype, d):
    """Mean, variance and weight; a delta and a projection's bias folded in and written back; gathered rows."""
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(d)
    x = torch.randn(9, d, generator=g) * 3 + 1.5
    delta, bias = torch.randn(9, d, generator=g), torch.randn(d, generator=g)
    w = (1 + 0.3 * torch.randn(d, generator=g)).to(out_dtype)
    tol = 1e-5 if out_dtype == torch.float32 else 1.2e-2
    xd = x.to(DEV)
    got = ops.layernorm(xd, w.to(DEV), 1e-5, out_dtype)
    want = P.layer_norm(x.double(), w.double(), 1e-5)
    assert (got.cpu().double() - want).abs().max() <= tol * want.abs().max() and torch.equal(xd.cpu(), x)
    got = ops.layernorm(xd, w.to(DEV), 1e-5, out_dtype, delta=delta.to(DEV), bias=bias.to(DEV))
    s = x + delta + bias
    want = P.layer_norm(s.double(), w.double(), 1e-5)
    assert (got.cpu().double() - want).abs().max() <= tol * want.abs().max()
    assert (xd.cpu() - s).abs().max() < 1e-5, "the sum is the new stream"
    rows = torch.tensor([4, 0, 4], dtype=torch.int32, device=DEV)
    got = ops.layernorm(xd, w.to(DEV), 1e-5, out_dtype, bias=bias.to(DEV), rows=rows)
    want = P.layer_norm((s + bias)[[4, 0, 4]].double(), w.double(), 1e-5)
    assert (got.cpu().double() - want).abs().max() <= tol * want.abs().max()
    assert (xd.cpu() - s).abs().max() < 1e-5, "gathered rows leave the stream"
    b = ops.add_bias(xd, bias.to(DEV))
    assert (b.cpu() - (s + bias)).abs().max() < 1e-5


def _paged(n_pages, G, hd, dtype):
    return torch.full((n_pages, G, 64, hd), 7.0, dtype=dtype, device=DEV)


@pytest.mark.parametrize("H,G,D,Dv,rot,pairing", [(3, 1, 10, 20, 4, "adjacent"), (4, 2, 16, 16, 16, "adjacent"),
                                                  (2, 2, 24, 8, 0, "adjacent"), (4, 4, 32, 48, 32, "half")])
@pytest.mark.parametrize("own", [True, False])
def test_bias_norm_over_all_heads_rotation_and_cache_write(H, G, D, Dv, rot, pairing, own):
    """The kernel between the QKV product and attention, against plain functions: two sequences at different
    positions on pages out of order; heads padded with zeros to the cache's width; a layer without keys and values
    writes nothing."""
    from picolm_b200 import ops
    from picolm_b200.cache.sequence_cache import KVLayerCache
    g = torch.Generator().manual_seed(H * 100 + D)
    lens, starts = [5, 3], [62, 0]
    step = _Step(lens, starts)
    T = sum(lens)
    hd_c = -(-max(D, Dv) // 16) * 16
    cols = H * D + ((G * D + G * Dv) if own else 0)
    qkv = torch.randn(T, cols, generator=g)
    bias = torch.randn(cols, generator=g)
    wq, wk = 1 + 0.2 * torch.randn(H * D, generator=g), 1 + 0.2 * torch.randn(G * D, generator=g)
    table = torch.tensor([[3, 1], [2, 0]], dtype=torch.int32, device=DEV)
    kv = KVLayerCache(_paged(4, G, hd_c, torch.float32), _paged(4, G, hd_c, torch.float32), table, None, own)
    rotation = None
    if rot:
        ang = torch.arange(80, dtype=torch.float64)[:, None] * (300.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot))[None]
        rotation = ops.Rotation(ang.cos().float().to(DEV), ang.sin().float().to(DEV), rot, pairing)
    q_out = torch.empty(T, H, hd_c, device=DEV)
    ops.qk_norm_rope_store(qkv.to(DEV), bias.to(DEV), wq.to(DEV), wk.to(DEV), 1e-5, q_out, kv, rotation, step, H, G, D, Dv,
                           own_kv=own)
    pos = step.tok_pos.cpu().tolist()

    def turn(x, heads, w):
        x = P.rms_norm(x.double(), w.double(), 1e-5).reshape(T, heads, D)
        if not rot:
            return x
        if pairing == "adjacent":
            return P.rotate_pairs(x, pos, rot, 300.0)
        y = x.clone()                                        # half-split pairs: (i, i + rot/2)
        perm = [2 * i for i in range(rot // 2)] + [2 * i + 1 for i in range(rot // 2)]
        inter = torch.empty_like(x[..., :rot])
        inter[..., perm] = x[..., :rot]
        y[..., :rot] = P.rotate_pairs(inter, pos, rot, 300.0)[..., perm]
        return y

    want_q = turn(qkv[:, :H * D] + bias[:H * D], H, wq)
    assert (q_out[..., :D].cpu().double() - want_q).abs().max() < 2e-5
    assert (q_out[..., D:] == 0).all()
    if not own:
        assert (kv.k == 7).all() and (kv.v == 7).all()
        return
    want_k = turn(qkv[:, H * D:H * D + G * D] + bias[H * D:H * D + G * D], G, wk)
    want_v = (qkv[:, H * D + G * D:] + bias[H * D + G * D:]).reshape(T, G, Dv)
    for t in range(T):
        b, p = int(step.tok_seq[t]), pos[t]
        page = int(table[b, p // 64])
        assert (kv.k[page, :, p % 64, :D].cpu().double() - want_k[t]).abs().max() < 2e-5
        assert (kv.v[page, :, p % 64, :Dv].cpu() - want_v[t]).abs().max() < 1e-6
        assert (kv.k[page, :, p % 64, D:] == 0).all() and (kv.v[page, :, p % 64, Dv:] == 0).all()
    assert (kv.k[0, :, 8:] == 7).all(), "rows of other positions are left alone"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_kernel(dtype):
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(5)
    gu = (torch.randn(7, 2 * 52, generator=g) * 2).to(dtype)
    gate, up = gu[:, :52].double(), gu[:, 52:].double()
    gc, uc = gate.clamp(max=0.8), up.clamp(-0.8, 0.8)
    want = gc * torch.sigmoid(1.702 * gc) * (uc + 1)
    got = ops.swiglu(gu.to(DEV), activation="swish_clamped", limit=0.8, slope=1.702).cpu().double()
    assert (got - want).abs().max() <= (1e-6 if dtype == torch.float32 else 8e-3)


@pytest.mark.parametrize("T", [8, 200, 1024])
def test_clamped_gate_in_the_products_epilogue(T):
    """The tensor-core products with the clamped gate in their epilogue (decode-shaped, prompt-shaped, pairs of CTAs),
    two limits one after the other (the constants travel with each launch), and the router's logits kernel."""
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(T)
    F, K = 512, 256
    x = torch.randn(T, K, generator=g).to(torch.bfloat16)
    wg, wu = (torch.randn(F, K, generator=g) * 0.1).to(torch.bfloat16), (torch.randn(F, K, generator=g) * 0.1).to(torch.bfloat16)
    w = ops.interleave_gate_up(wg.to(DEV), wu.to(DEV))
    for limit in (0.6, 2.5):
        gate = (x.double() @ wg.double().T).to(torch.bfloat16).double().clamp(max=limit)
        up = (x.double() @ wu.double().T).to(torch.bfloat16).double().clamp(-limit, limit)
        want = gate * torch.sigmoid(1.702 * gate) * (up + 1)
        got = ops.linear_swiglu(x.to(DEV), w, activation="swish_clamped", limit=limit, slope=1.702).cpu().double()
        assert (got - want).abs().max() <= 2e-2 * want.abs().max(), f"limit {limit}"
    logits = ops.router_logits(x.to(DEV), wg[:37].contiguous().to(DEV)).cpu().double()
    assert (logits - x.double() @ wg[:37].double().T).abs().max() < 1e-4
    ops.check_status()


@pytest.mark.parametrize("E,top,groups,scale", [(16, 3, (4, 2), 1.75), (6, 2, (3, 2), 1.0), (8, 1, None, 2.5), (6, 2, (6, 3), 1.0),
                                                (12, 4, (1, 1), 0.5), (64, 6, (8, 3), 2.0)])
def test_router_choice_kernel(E, top, groups, scale):
    """Sigmoid scores, the correction for the choice only, groups by the sum of their two best, experts outside the
    kept groups never chosen although choice scores are negative, weights from the scores without the correction."""
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(E + top)
    T = 50
    logits = torch.randn(T, E + 1, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.5 - 2.0                        # every choice score is negative
    r = {"experts": E, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    w_id = torch.eye(E, dtype=torch.float64)
    idx, w = P.route(logits[:, :E].double(), w_id, corr.double(), r)
    ids, weights, gate = ops.route_topk(logits.to(DEV), E, top, corr.to(DEV), groups[0] if groups else 1,
                                        groups[1] if groups else 1, scale, gate_col=E)
    assert torch.equal(ids.cpu().long(), idx), "the chosen experts, in the order of their choice scores"
    assert (weights.cpu().double() - w).abs().max() < 1e-6
    assert (gate.cpu().double() - torch.sigmoid(logits[:, E].double())).abs().max() < 1e-6
    ids2, w2, none = ops.route_topk(logits[:, :E].contiguous().to(DEV), E, top, None, 1, 1, scale)
    idx2, wp2 = P.route(logits[:, :E].double(), w_id, torch.zeros(E, dtype=torch.float64), {"experts": E, "top": top, "scale": scale})
    assert none is None and torch.equal(ids2.cpu().long(), idx2) and (w2.cpu().double() - wp2).abs().max() < 1e-6


@pytest.mark.parametrize("T,E,top,F,d", [(5, 8, 2, 20, 40), (150, 4, 3, 36, 72), (33, 16, 1, 64, 24)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_products_over_sorted_pairs(T, E, top, F, d, dtype):
    """Sort by expert, the two products over the sorted tiles (small and large tiles), the weighted sum with a
    shared expert behind a gate: against a loop over tokens and their experts."""
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, d, generator=g).to(dtype)
    wg, wu = (torch.randn(E, F, d, generator=g) * 0.3).to(dtype), (torch.randn(E, F, d, generator=g) * 0.3).to(dtype)
    wd = (torch.randn(E, d, F, generator=g) * 0.3).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 100:
        ids[:90, 0] = 1                                               # one expert with more rows than a tile
        ids[:90, 1:] = torch.tensor([0, 2])[None, :top - 1]
    weights = torch.rand(T, top, generator=g)
    shared, gate = torch.randn(T, d, generator=g), torch.rand(T, generator=g)
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            want[t] += weights[t, k].double() * P.expert(h[t:t + 1].double(), wg[e].double(), wu[e].double(), wd[e].double())[0]
    want += gate.double()[:, None] * shared.double()
    for bm in (16, 64):
        pairs = ops.moe_align(ids.to(DEV), E, bm)
        srt, te = pairs.sorted.cpu(), pairs.tile_expert.cpu()
        live = srt[srt >= 0]
        assert sorted(live.tolist()) == list(range(T * top)), "every pair exactly once"
        for tile in range(pairs.max_tiles):
            rows = srt[tile * bm:(tile + 1) * bm]
            rows = rows[rows >= 0]
            assert (te[tile] < 0 and rows.numel() == 0) or all(int(ids.view(-1)[r]) == int(te[tile]) for r in rows)
        assert all(int(srt[p]) == i for i, p in enumerate(pairs.where.cpu().tolist()))
        act = ops.moe_gate_up(h.to(DEV), torch.cat([wg, wu], dim=1).contiguous().to(DEV), pairs)
        y = ops.moe_down(act, wd.to(DEV), pairs)
        got = ops.moe_combine(y, pairs, weights.to(DEV), shared.to(DEV), gate.to(DEV)).cpu().double()
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert (got - want).abs().max() <= tol * want.abs().max(), f"tiles of {bm}"
        gathered = ops.moe_gather(h.to(DEV), pairs).cpu()
        assert torch.equal(gathered[pairs.where.cpu().long()], h[torch.arange(T * top) // top])


@pytest.mark.parametrize("T,E,top,F,d", [(300, 4, 2, 128, 128), (40, 8, 3, 64, 96), (700, 3, 1, 192, 320)])
def test_experts_products_on_the_tensor_cores(T, E, top, F, d):
    """bfloat16 with an inner width that is a multiple of 64: gate and up rows in turns of 64, tiles of 16 rows on
    mma.sync and tiles of 128 rows on tcgen05 (the rows laid out in sorted order first), against a loop over tokens."""
    from picolm_b200 import ops
    g = torch.Generator().manual_seed(T + F)
    bf = torch.bfloat16
    h = torch.randn(T, d, generator=g).to(bf)
    wg, wu = (torch.randn(E, F, d, generator=g) * 0.2).to(bf), (torch.randn(E, F, d, generator=g) * 0.2).to(bf)
    wd = (torch.randn(E, d, F, generator=g) * 0.2).to(bf)
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    ids[: T // 2, 0] = E - 1                                             # one expert far busier than the others,
    if top > 1:
        ids[: T // 2, 1:] = torch.arange(top - 1)[None]
    if E > 3:
        ids[ids == 1] = 2 if top == 1 else ids[ids == 1]                    # (and, where it can be, one without any row)
    weights = torch.rand(T, top, generator=g)
    want = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(ids[t, k])
            want[t] += weights[t, k].double() * P.expert(h[t:t + 1].double(), wg[e].double(), wu[e].double(), wd[e].double())[0]
    w_gu = torch.stack([ops.interleave_gate_up(a.to(DEV), b.to(DEV)) for a, b in zip(wg, wu)]).contiguous()
    hd, wdd = h.to(DEV), wd.to(DEV)
    assert ops.moe_tc_supported(hd, w_gu, wdd)
    small = ops.moe_align(ids.to(DEV), E, 16)
    y = ops.moe_down(ops.moe_gate_up(hd, w_gu, small, interleaved=True), wdd, small)
    got = ops.moe_combine(y, small, weights.to(DEV)).cpu().double()
    assert (got - want).abs().max() <= 2e-2 * want.abs().max(), "tiles of 16 rows (mma.sync)"
    big = ops.moe_align(ids.to(DEV), E, 128)
    y = ops.moe_down_tc(ops.moe_gate_up_tc(ops.moe_gather(hd, big), w_gu, big), wdd, big)
    got2 = ops.moe_combine(y, big, weights.to(DEV)).cpu().double()
    assert (got2 - want).abs().max() <= 2e-2 * want.abs().max(), "tiles of 128 rows (tcgen05)"
    ops.check_status()


def _attention_plain(q, k, v, pos_q, scale, chunk):
    """q [n, H, D], k/v [L, G, D]: every query at its position over keys 0..pos of its chunk."""
    n, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for i, p in enumerate(pos_q):
        lo = p - p % chunk
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:p + 1, g].double() @ q[i, h].double()) * scale
            out[i, h] = torch.softmax(s, dim=0) @ v[lo:p + 1, g].double()
    return out


@pytest.mark.parametrize("hd,H,G,chunk,how", [
    (48, 4, 2, 64, "mma"), (32, 6, 2, 65, "mma"), (16, 2, 1, 5, "mma"), (80, 3, 3, 130, "mma"), (256, 2, 1, 63, "mma"),
    (64, 4, 2, 64, "tc"), (64, 2, 2, 100, "tc"), (128, 4, 1, 65, "tc"), (128, 2, 2, 7, "tc"),
    (24, 3, 1, 33, "rows"), (48, 2, 2, 128, "rows32"), (20, 2, 1, 1, "rows32")])
def test_attention_kernels_under_a_mask_of_chunks(hd, H, G, chunk, how):
    """Every attention kernel with chunks of sizes at, beside and across page borders: a prompt of 300 tokens, a portion
    that starts inside a chunk after a cached prefix, and single tokens just before, at and after chunk starts.  Every
    query is aimed at the first key of its chunk or the key before it (a large score), so a chunk cut one position
    off moves the row far beyond the tolerance."""
    from picolm_b200 import ops
    dtype = torch.float32 if how == "rows32" else torch.bfloat16
    g = torch.Generator().manual_seed(hd + chunk)
    L = 300
    k = torch.randn(L, G, hd, generator=g)
    v = torch.randn(L, G, hd, generator=g)
    q = torch.randn(L, H, hd, generator=g) * 0.3
    for p in range(L):
        lo = p - p % chunk
        aim = lo if p % 2 == 0 else max(lo - 1, 0)                      # even rows at the chunk's first key, odd rows just outside
        for h in range(H):
            q[p, h] += 4.0 * k[aim, h // (H // G)] / k[aim, h // (H // G)].norm()
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    scale = 1.3
    want = _attention_plain(q.float(), k.float(), v.float(), list(range(L)), scale, chunk)
    off = _attention_plain(q.float(), k.float(), v.float(), list(range(L)), scale, chunk + 1)
    assert ((off - want).abs().amax(dim=(1, 2)) > 0.3).sum() > L // (4 * max(chunk, 2)), "the inputs do not make the edge show"
    n_pages = (L + 63) // 64
    order = [3, 5, 1, 4, 2][:n_pages]
    kc, vc = torch.zeros(6, G, 64, hd, dtype=dtype), torch.zeros(6, G, 64, hd, dtype=dtype)
    for p in range(L):
        kc[order[p // 64], :, p % 64] = k[p]
        vc[order[p // 64], :, p % 64] = v[p]
    kc, vc = kc.to(DEV), vc.to(DEV)
    table = torch.tensor([order + [0]], dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2

    def check(got, rows, what):
        err = (got.view(len(rows), H, hd).cpu().double() - want[rows]).abs().max()
        assert err <= tol * max(1.0, want.abs().max().item()), f"{what}: {err:.3e}"

    def prompt(first, last):
        rows = list(range(first, last))
        step = _Step([last - first], [first])
        qd = q[first:last].contiguous().to(DEV)
        if how == "tc":
            got = ops.attention_prefill_tc(qd, kc, vc, step.seq_start, step.seq_kv_len, table, step.max_new, G, scale, window=-chunk)
        elif how == "mma":
            got = ops.attention_prefill(qd, kc, vc, step.seq_start, step.seq_kv_len, table, step.max_new, G, scale, window=-chunk)
        else:
            got = ops.attention_rows(qd, kc, vc, step.tok_pos, step.tok_seq, table, G, scale, window=-chunk)
        check(got, rows, f"prompt rows {first}..{last}")

    prompt(0, L)
    prompt(chunk + chunk // 2, min(L, 3 * chunk + 2))                  # a portion that starts inside a chunk
    prompt(L - 2, L)                                                  # two tokens
    singles = sorted({p for c in range(chunk, L, chunk) for p in (c - 1, c, c + 1) if 0 < p < L} | {0, 1, 63, 64, 65, L - 1})
    singles = singles[:40] + singles[-10:]
    for p in singles:
        step = _Step([1], [p])
        qd = q[p:p + 1].contiguous().to(DEV)
        if how in ("tc", "mma"):
            for splits in (1, 2, 5):
                got = ops.attention_decode(qd, kc, vc, step.tok_pos, step.tok_seq, table, G, scale, splits, window=-chunk)
                check(got, [p], f"single token at {p}, {splits} ranges")
        else:
            got = ops.attention_rows(qd, kc, vc, step.tok_pos, step.tok_seq, table, G, scale, window=-chunk)
            check(got, [p], f"single token at {p}")


# ------------------------------------------------------------------------------------------- whole models
MODELS = {
    # one layer of each feed-forward
    "dense": ([_attn()], {}),
    "routed": ([dict(_attn(chunk=9), mlp=_moe())], {}),
    # borrowed keys and values under another chunk size, a layer that only mixes, one kv head, values narrower than keys
    "borrowed": ([_attn(heads=4, kv_heads=1, dim=16, vdim=8, chunk=11), dict(_attn(heads=2, kv_heads=2, dim=8, vdim=8, rot=2), mlp=_moe(experts=4, top=1, groups=None, shared=None)),
                  dict(_attn(heads=2, kv_heads=1, dim=16, vdim=8, chunk=4, kv_from=0), mlp=None),
                  dict(_attn(heads=4, kv_heads=2, dim=8, vdim=8, rot=2, chunk=64, kv_from=1), mlp=_moe(experts=6, top=3, groups=(6, 4), shared=12))], {}),
    # a width that no tensor map takes, an odd head size, no rotation in one layer, a rotation of the whole head in another
    "odd": ([_attn(heads=3, kv_heads=3, dim=10, vdim=6, rot=0, chunk=3), dict(_attn(heads=2, kv_heads=1, dim=12, vdim=20, rot=12, chunk=70), mlp=_moe(experts=5, top=2, groups=(1, 1), ff=9))],
            {"width": 42, "vocab": 101}),
    # a mixer whose configuration names neither a mask nor a rotation: every earlier key, nothing turned
    "plain_causal": ([{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.8}}, dict(_attn(chunk=40), mlp=_moe(groups=None))], {}),
    # head sizes that take the tensor-core kernels in bfloat16 runs (their float32 twins run here)
    "wide_heads": ([_attn(heads=2, kv_heads=1, dim=64, vdim=64, rot=32, chunk=50, scale=0.3), _attn(heads=2, kv_heads=2, dim=32, vdim=128, rot=32, chunk=130, scale=0.4)],
                   {"width": 64}),
}


@pytest.mark.parametrize("name", sorted(MODELS))
def test_float32_model_matches_plain_in_every_cut(tmp_path, name):
    layers, kw = MODELS[name]
    d, tensors, config = _make(tmp_path, name, _config(layers, **kw), seed=len(name))
    vocab = config["vocab"]
    eng = _engine(d)
    a, b, c = random_tokens(150, vocab, 1), random_tokens(67, vocab, 2), random_tokens(1, vocab, 3)
    want = {id(t): _plain(tensors, config, t) for t in (a, b, c)}
    for t in (a, b, c):
        _close(run_whole(eng, t), want[id(t)], what="whole")
    _close(run_tail(eng, a, tail=90), want[id(a)], what="prompt, then 90 single tokens")       # over a page border
    _close(run_tail(eng, b, tail=len(b)), want[id(b)], what="token by token from the first")
    for sizes in ([64, 64, 22], [3, 2, 61, 2, 2, 80], [149, 1], [2] * 33 + [1]):
        t = a if sum(sizes) == 150 else b
        _close(run_chunks(eng, t, sizes), want[id(t)], what=f"portions {sizes[:6]}")
    outs = run_batch(eng, [b, c, a], [40, 1, 129])
    for got, t in zip(outs, (b, c, a)):
        _close(got, want[id(t)], what="batch of unequal requests")
    # slots and pages that were used are used again, and give the same
    _close(run_whole(eng, a), want[id(a)], what="whole, again")
    eng.cache.check()
    assert eng.cache.slots.used == 0 and all(g.pool.used == 0 for g in eng.cache.kv_groups)


def test_layer_without_keys_and_values_reads_its_owner(tmp_path):
    """The folder holds no key or value tensors for the borrowing layers, the cache no pages for them."""
    layers, kw = MODELS["borrowed"]
    d, tensors, config = _make(tmp_path, "b", _config(layers, **kw), seed=3)
    for i in (2, 3):
        assert not any(n.startswith(f"l{i}.mix.k") or n.startswith(f"l{i}.mix.v") for n in tensors)
        assert f"l{i}.mix.q.norm" in tensors and f"l{i}.mix.o.b" in tensors
    assert "l2.norm2" not in tensors
    eng = _engine(d)
    assert sum(len(g.layers) for g in eng.cache.kv_groups) == 2


# -------------------------------------------------------------------------------------------- chunk edges
@pytest.mark.parametrize("chunk", [5, 64, 65, 130])
def test_chunk_edges_decide_logits_and_are_right(tmp_path, chunk):
    """With a peaked softmax one key often holds most of a row's weight: a chunk that is cut one token off changes rows'
    logits by far more than the tolerance (the test first makes sure of that with the plain implementation), in
    prompts, in portions that start inside a chunk and in single tokens, with chunks that end on a page's border and
    just beside it; the first tokens of a sequence and of every chunk see only what their chunk holds."""
    layers = [_attn(heads=2, kv_heads=1, dim=16, vdim=8, chunk=chunk, scale=2.0, rot=8),
              dict(_attn(heads=2, kv_heads=2, dim=16, vdim=16, chunk=chunk + 3, scale=2.0, kv_from=None), mlp=_moe())]
    d, tensors, config = _make(tmp_path, f"c{chunk}", _config(layers), seed=chunk)
    t = random_tokens(290, 97, chunk)
    want = _plain(tensors, config, t)
    for off in (-1, 1):
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = chunk + off
        diff = (_plain(tensors, other, t) - want).abs().amax(dim=1) / want.std()
        assert (diff > 50 * FP32_TOL).sum() >= 3, "the weights do not make the chunk's edge show"
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=150), want, what="single tokens over chunk starts")
    _close(run_chunks(eng, t, [chunk - 1, 2, chunk, 3, 290 - 2 * chunk - 4]), want, what="portions around the edges")
    outs = run_batch(eng, [t, t[:chunk + 1], t[:3]], [chunk, chunk - 1, 1])
    _close(outs[0], want, what="batch")
    _close(outs[1], want[:chunk + 1], what="batch, a request that just fills a chunk")
    eng.cache.check()


def test_far_keys_inside_a_long_chunk(tmp_path):
    """A chunk longer than the prompt: the first tokens of a 600-token prompt still move the last logits, through
    prompts, portions and 200 single tokens alike (nine pages, keys far from the query)."""
    layers = [_attn(heads=2, kv_heads=1, dim=16, vdim=16, chunk=1000, scale=1.5, rot=16, base=50000.0), dict(_attn(chunk=640, scale=1.2), mlp=_moe())]
    d, tensors, config = _make(tmp_path, "far", _config(layers), seed=21)
    t = random_tokens(600, 97, 8)
    want = _plain(tensors, config, t)
    changed = list(t)
    changed[3] = (changed[3] + 1) % 97
    assert (_plain(tensors, config, changed)[-1] - want[-1]).abs().max() > 20 * FP32_TOL * want.std()
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=200), want, what="200 single tokens")
    _close(run_chunks(eng, t, [333, 67, 200]), want, what="portions")


# ------------------------------------------------------------------------------------------------ bfloat16
@pytest.mark.parametrize("name", ["wide_heads", "serving"])
def test_bfloat16_follows_the_plain_implementation(tmp_path, name):
    """The serving precision stays within rounding of the exact logits, and its own cuts agree with each other far
    more closely than that.  `wide_heads`: head sizes 64 and 128 (the tcgen05 prompt attention); `serving`: 48 and 16
    (the mma.sync kernels), a routed layer whose sizes take the tensor-core products."""
    if name == "wide_heads":
        layers, kw = MODELS[name]
    else:
        layers = [_attn(heads=4, kv_heads=2, dim=48, vdim=32, rot=16, chunk=70, scale=0.5),
                  dict(_attn(heads=8, kv_heads=2, dim=16, vdim=16, chunk=33, scale=0.6), mlp=_moe(experts=8, top=2, ff=64, groups=(4, 2), shared=64)),
                  dict(_attn(heads=4, kv_heads=2, dim=48, vdim=32, rot=16, chunk=100, scale=0.5, kv_from=0), mlp=_dense(ff=128))]
        kw = {"width": 128}
    d, tensors, config = _make(tmp_path, "bf16" + name, _config(layers, **kw), seed=3, std=0.08)
    t, u = random_tokens(200, 97, 5), random_tokens(31, 97, 6)
    want = _plain(tensors, config, t)
    eng = _engine(d, dtype="bfloat16")
    whole = run_whole(eng, t)
    rel = ((whole - want).double().pow(2).mean().sqrt() / want.double().std()).item()
    assert rel < 0.05, f"bfloat16 logits are {rel:.3f} of the spread away from the exact ones"
    for got in (run_tail(eng, t, tail=70), run_chunks(eng, t, [64, 2, 134]), run_batch(eng, [u, t], [11, 130])[1]):
        rel = ((got - whole).double().pow(2).mean().sqrt() / want.double().std()).item()
        assert rel < 0.03, f"two cuts of the same request differ by {rel:.3f} of the spread"
    eng.cache.check()


# ---------------------------------------------------------------------------------------------- generation
GEN = [_attn(chunk=6), dict(_attn(heads=2, kv_heads=1, dim=8, vdim=16, chunk=20), mlp=_moe()), dict(_attn(chunk=9, kv_from=0), mlp=None)]


def _greedy(tensors, config, p, n):
    seq, out = list(p), []
    for _ in range(n):
        out.append(int(_plain(tensors, config, seq)[-1].argmax()))
        seq.append(out[-1])
    return out


def test_greedy_generation_through_the_entry_point(tmp_path):
    """`generate` (batch planning, captured decode steps, sampled ids fed back on the device) gives the plain
    implementation's greedy tokens; more requests than fit one batch, so slots and pages are used again."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "gen", _config(GEN), seed=13)
    prompts = [random_tokens(n, 97, 30 + i) for i, n in enumerate([5, 70, 1, 19, 33])]
    want = [_greedy(tensors, config, p, 8) for p in prompts]
    eng = model_load(d, dtype="float32", max_batch=2)
    got, stats = generate(eng, prompts, max_tokens=8, temperature=0.0, stop_ids=[], return_stats=True)
    assert got == want
    assert stats.batches == 3 and eng.cache.slots.used == 0
    assert eng.use_graphs, "decode steps of this design are meant to replay captured graphs"
    eng.cache.check()


def test_bfloat16_generation_with_captured_prompt_steps(tmp_path):
    """In bfloat16 `generate` replays captured graphs for the prompts' step too (tokens padded to a size class, the
    padding in a sequence of its own, whose rows the router sorts like any others): every generated token is, by the
    logits of the same prompts launched kernel by kernel, the best or within rounding of it, and by the exact logits
    close to the best."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "pgraph", _config(GEN, width=64), seed=23, std=0.08)
    prompts = [random_tokens(n, 97, 60 + i) for i, n in enumerate([70, 9, 200])]
    eng = model_load(d, dtype="bfloat16", max_batch=4)
    assert eng.prompt_graphs, "every part of the design declares itself safe for captured prompt steps"
    got = generate(eng, prompts, max_tokens=6, temperature=0.0, stop_ids=[])
    assert eng._prompt_graphs, "the prompts' step was not replayed from a graph"
    plain_eng = _engine(d, dtype="bfloat16", use_graphs=False)
    slots = [plain_eng.new_sequence() for _ in prompts]
    logits = plain_eng.step(list(zip(slots, prompts))).float().cpu()
    seqs = [list(p) for p in prompts]
    for step in range(6):
        for i, row in enumerate(logits):
            tok = got[i][step]
            assert row[tok] >= row.max() - 0.02 * row.std(), f"request {i}, step {step}: graph and single launches disagree"
            exact = _plain(tensors, config, seqs[i])[-1]
            assert exact[tok] >= exact.max() - 0.25 * exact.std(), f"request {i}, step {step}: far from the exact best token"
            seqs[i].append(tok)
        logits = plain_eng.step([(s, [got[i][step]]) for i, s in enumerate(slots)]).float().cpu()
    for s in slots:
        plain_eng.end_sequence(s)
    eng.cache.check()


def test_trace_replay_as_a_user_runs_it(tmp_path):
    """bin/trace_run on a Kunulorn folder: a batch of unequal prompts, single tokens until the shorter requests end,
    a request alone afterwards in the slot that was given back."""
    from test_gpu_trace_run import Replay
    d, tensors, config = _make(tmp_path, "replay", _config(GEN), seed=17)
    reqs = {f"q{i}": random_tokens(n, 97, 300 + i) for i, n in enumerate([70, 9, 1, 30, 3, 2])}
    ref = {k: _plain(tensors, config, t) for k, t in reqs.items()}
    rp = Replay(d, "float32", str(tmp_path / "out"), max_tokens=128)
    try:
        batch = ["q0", "q1", "q2", "q4", "q5"]
        pos = {"q0": 50, "q1": 4, "q2": 1, "q4": 2, "q5": 1}
        got = rp.send([{"id": k, "tokens": reqs[k][:pos[k]], "want": [pos[k] - 1]} for k in batch],
                      end=[k for k in batch if pos[k] == len(reqs[k])])
        for row, k in enumerate(batch):
            _close(got[row:row + 1], ref[k][pos[k] - 1:pos[k]], what=f"prompt of {k}")
        live = [k for k in batch if pos[k] < len(reqs[k])]
        while live:
            ending = [k for k in live if pos[k] + 1 == len(reqs[k])]
            got = rp.send([{"id": k, "tokens": [reqs[k][pos[k]]], "want": [0]} for k in live], end=ending)
            for row, k in enumerate(live):
                _close(got[row:row + 1], ref[k][pos[k]:pos[k] + 1], what=f"{k} at {pos[k]}")
                pos[k] += 1
            live = [k for k in live if pos[k] < len(reqs[k])]
        got = rp.send([{"id": "again", "tokens": reqs["q3"], "want": [0, 29]}], end=["again"])
        _close(got, ref["q3"][[0, 29]], what="alone, afterwards")
    finally:
        rp.close()


def test_command_line(tmp_path):
    """The library's command line on a Kunulorn folder: random weights from a config.json, greedy tokens equal to the
    plain implementation's, sampling, the per-layer benchmark with a row for every layer."""
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = [sys.executable, os.path.join(root, "bin", "picolm_b200")]
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(_config(GEN), f)
    d = str(tmp_path / "model")
    r = subprocess.run(exe + ["--random-weights", cfg_path, "--out", d, "-s", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    tensors = P.read_safetensors(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json")) as f:
        config = json.load(f)
    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0", "--dtype", "float32", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [[int(t) for t in ln.split()] for ln in r.stdout.strip().splitlines()] == [_greedy(tensors, config, [5, 6, 7], 6),
                                                                                    _greedy(tensors, config, [9], 6)]
    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0.8", "-k", "40", "--top-p", "0.9", "-s", "5", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [len(ln.split()) for ln in r.stdout.strip().splitlines()] == [6, 6]
    r = subprocess.run(exe + [d, "-p", "5,6,7,8", "-n", "5", "--benchmark"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [ln.split(",") for ln in r.stderr.splitlines() if re.fullmatch(r"\d+,[0-9.]+,[0-9.]+,[0-9.]+,\d+", ln)]
    assert [int(x[0]) for x in rows] == [0, 1, 2] * 3
    r = subprocess.run(exe + [d, "--list-tensors"], capture_output=True, text=True, timeout=60)
    assert "l1.mlp.correction\t[6]\tBF16" in r.stdout and "l2.mix.k" not in r.stdout
