"""The Potuzen design through the library, against the plain implementation in
`tests/plain/potuzen_plain.py`: each mechanism alone (kernels against plain functions, then one-mixer
models), prompts against token-by-token decoding, portions, batches, pages and slots used again, window
edges and page borders, long decoding, sizes that make special cases (1 head, 1 group, one norm group, a
window of 1, no feed-forward, shared weights), and greedy generation through the library's entry point.

Weights are random; where random weights would hide a fault they are reshaped: the queries' and keys' maps
are scaled up so that the softmax is peaked (one key at the window's edge then decides a row of logits),
decays are drawn close to 1 so that far tokens stay in a state.
"""
import json
import os

import pytest
import torch

from harness import run_batch, run_chunks, run_tail, run_whole
from plain import potuzen_plain as P
from util import random_tokens

pytestmark = pytest.mark.gpu

FP32_TOL = 2e-4          # of the logits' spread; two float32 computations in different orders of summation


def _latent(heads=3, dim=8, vdim=12, kv_rank=20, q_rank=24, window=7, scale=0.4):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                      "mask": {"size": window}}}


def _mamba(heads=6, vdim=12, state=8, groups=3, conv=3, norm_groups=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def _gla(heads=2, dim=12, vdim=20, tau=4.0, decay_rank=5):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}}


def _config(layers, width=40, vocab=97, ff=56, eps=1e-5):
    out = []
    for layer in layers:
        layer = dict(layer)
        layer.setdefault("mlp", {"kind": "dense", "ff": ff})
        out.append(layer)
    return {"architecture": "Potuzen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": out}


def _make(tmp_path, name, config, seed, sharpen=6.0):
    """A model folder with random weights for `config`; returns (folder, plain tensors, config)."""
    from picolm_b200.config import config_from_dict
    from picolm_b200.weights import random_tensors, save_safetensors
    cfg = config_from_dict(config)
    tensors = random_tensors(cfg, seed, std=0.12, norm_std=0.2)
    for n in tensors:
        if n.endswith(".mix.uq") or n.endswith(".mix.uk"):
            tensors[n] = (tensors[n].float() * sharpen).to(tensors[n].dtype)
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


MIXED = [_latent(), _mamba(), _gla(), dict(_latent(), weights_of=0), _gla(heads=1, dim=16, vdim=8, tau=16.0, decay_rank=3)]


# ------------------------------------------------------------------------------------------- kernels alone
class _Step:
    """What the kernels read of a step, for sequences that bring `lens` tokens each."""

    def __init__(self, lens, slots, dev, starts=None):
        offs = [0]
        for n in lens:
            offs.append(offs[-1] + n)
        i32 = dict(dtype=torch.int32, device=dev)
        self.n_seqs, self.n_tokens, self.max_new = len(lens), offs[-1], max(lens)
        self.is_decode = all(n == 1 for n in lens)
        self.seq_start = torch.tensor(offs, **i32)
        self.seq_slot = torch.tensor(slots, **i32)
        self.tok_seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], **i32)
        starts = starts or [0] * len(lens)
        self.tok_pos = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], **i32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4])
@pytest.mark.parametrize("C", [37, 48])            # 48: bfloat16 channels in eights, the vectorised kernel
def test_causal_conv_kernel(dtype, taps, C):
    """Ragged prompts, then portions that are shorter than the taps, then single tokens: the state carries over."""
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(taps)
    lens = [9, 1, 2]
    total = [n + 2 + 1 + 3 for n in lens]
    pad = 5 if C % 8 else 16                                                      # column slices of a wider matrix
    u = [torch.randn(n, C + pad, generator=g).to(dtype) for n in total]
    w = torch.randn(C, taps, generator=g)
    b = torch.randn(C, generator=g)
    lo = 2 if C % 8 else 8
    want = [P.silu(P.causal_conv(x[:, lo:lo + C].double(), w.double(), b.double())) for x in u]
    state = torch.zeros(5, (taps - 1) * C + 3, device=dev)                        # rows wider than the state
    slots = [3, 0, 2]
    got, at = [[] for _ in lens], [0, 0, 0]
    for cut in ([9, 1, 2], [2, 2, 2], [1, 1, 1], [3, 3, 3]):
        step = _Step(cut, slots, dev)
        rows = torch.cat([u[i][at[i]:at[i] + n] for i, n in enumerate(cut)]).to(dev)
        out = ops.causal_conv(rows[:, lo:lo + C], w.t().contiguous().to(dev), b.to(dev), state[:, :(taps - 1) * C], step)
        o = 0
        for i, n in enumerate(cut):
            got[i].append(out[o:o + n].float().cpu())
            o, at[i] = o + n, at[i] + n
    for i in range(3):
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=tol, rtol=tol), f"sequence {i}"
    assert state[:, (taps - 1) * C:].abs().max() == 0 and state[1].abs().max() == 0 and state[4].abs().max() == 0


@pytest.mark.parametrize("mode", ["step", "sigmoid"])
@pytest.mark.parametrize("N,P_,H,hpg,lens,cuts", [
    (8, 12, 6, 2, [23, 4], ([7, 1], [1, 1], [15, 2])), (5, 33, 2, 1, [23, 4], ([7, 1], [1, 1], [15, 2])),
    (48, 64, 4, 4, [23, 4], ([7, 1], [1, 1], [15, 2])), (130, 8, 1, 1, [23, 4], ([7, 1], [1, 1], [15, 2])),
    (20, 36, 2, 2, [521, 270], ([200, 3], [1, 1], [320, 266])),
    (16, 64, 2, 1, [521, 270], ([200, 3], [1, 1], [320, 266]))])        # sizes in eights: bfloat16 rows are read 16 bytes at a time
def test_linear_scan_kernel(mode, N, P_, H, hpg, lens, cuts):
    """The recurrence alone against a loop over tokens, cut into steps of several sizes (one token included), with
    key sizes that are no multiple of four and value sizes that are no multiple of the tile; the long case runs in
    segments side by side (a sequence of one segment beside one of several, a last segment that is short)."""
    from picolm_b200 import ops
    if mode == "sigmoid":
        hpg = 1
    dev = "cuda:0"
    g = torch.Generator().manual_seed(N * 7 + P_)
    G = H // hpg
    dt = torch.bfloat16 if (N, P_) == (16, 64) else torch.float32
    q = [torch.randn(n, G * N, generator=g).to(dt) for n in lens]
    k = [torch.randn(n, G * N, generator=g).to(dt) for n in lens]
    v = [torch.randn(n, H * P_, generator=g).to(dt) for n in lens]
    if mode == "step":
        raw = [torch.randn(n, H, generator=g).to(dt) for n in lens]
        p0, p1, skip = torch.randn(H, generator=g), torch.randn(H, generator=g) - 1.0, torch.randn(H, generator=g)
        power, q_scale = 1.0, 1.0
    else:
        raw = [(torch.randn(n, H * N, generator=g) * 2).to(dt) for n in lens]
        p0, p1, skip = torch.randn(H * N, generator=g) + 2.0, None, None
        power, q_scale = 1.0 / 3.0, N ** -0.5

    def plain(i):
        S = torch.zeros(H, N, P_, dtype=torch.float64)
        ys = []
        for t in range(lens[i]):
            y = torch.zeros(H, P_, dtype=torch.float64)
            for h in range(H):
                gq = h // hpg
                qq = q[i][t, gq * N:(gq + 1) * N].double() * q_scale
                kk = k[i][t, gq * N:(gq + 1) * N].double()
                vv = v[i][t, h * P_:(h + 1) * P_].double()
                if mode == "step":
                    dt = P.softplus(raw[i][t, h].double() + p0[h].double())
                    S[h] = torch.exp(-torch.exp(p1[h].double()) * dt) * S[h] + dt * torch.outer(kk, vv)
                    y[h] = S[h].T @ qq + skip[h].double() * vv
                else:
                    d = torch.sigmoid(raw[i][t, h * N:(h + 1) * N].double() + p0[h * N:(h + 1) * N].double()) ** power
                    S[h] = d[:, None] * S[h] + torch.outer(kk, vv)
                    y[h] = S[h].T @ qq
            ys.append(y.reshape(-1))
        return torch.stack(ys), S

    state = torch.zeros(4, H * N * P_, device=dev)
    slots = [2, 0]
    got, at = [[], []], [0, 0]
    for cut in cuts:
        step = _Step(cut, slots, dev)
        cat = lambda xs: torch.cat([xs[i][at[i]:at[i] + n] for i, n in enumerate(cut)]).to(dev)   # noqa: E731
        y = ops.linear_scan(cat(q), cat(k), cat(v), cat(raw), ops.DECAY_STEP if mode == "step" else ops.DECAY_SIGMOID,
                            p0.to(dev), None if p1 is None else p1.to(dev), None if skip is None else skip.to(dev),
                            q_scale, power, state, step, H, N, P_, hpg)
        o = 0
        for i, n in enumerate(cut):
            got[i].append(y[o:o + n].cpu())
            o, at[i] = o + n, at[i] + n
    for i in range(2):
        want, S = plain(i)
        have = torch.cat(got[i]).double()
        assert (have - want).abs().max() <= 2e-5 * max(1.0, want.abs().max()), f"sequence {i}"
        assert (state[slots[i]].cpu().double().view(H, N, P_) - S).abs().max() <= 2e-5 * max(1.0, S.abs().max())
    assert state[1].abs().max() == 0 and state[3].abs().max() == 0


def test_gated_norm_and_head_linear_kernels():
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(5)
    T, C, group = 7, 60, 20
    wide = torch.randn(T, C + 9, generator=g).to(dev)
    x, gate = wide[:, 4:4 + C], torch.randn(T, C, generator=g).to(dev)
    w_all, w_grp = torch.randn(C, generator=g).to(dev), torch.randn(group, generator=g).to(dev)
    xd, gd = x.double().cpu(), gate.double().cpu()
    before = P.rms_norm((xd * P.silu(gd)).view(T, C // group, group), None, 1e-3).reshape(T, C) * w_all.double().cpu()
    after = P.rms_norm(xd.view(T, C // group, group), w_grp.double().cpu(), 1e-3).reshape(T, C) * P.silu(gd)
    plain = P.rms_norm(xd, w_all.double().cpu(), 1e-3)
    got = ops.gated_norm(x, torch.float32, weight=w_all, eps=1e-3, group=group, gate=gate, gate_mode=ops.GATE_BEFORE_NORM)
    assert torch.allclose(got.double().cpu(), before, atol=1e-5, rtol=1e-5)
    got = ops.gated_norm(x, torch.float32, weight=w_grp, eps=1e-3, group=group, weight_per_group=True, gate=gate,
                         gate_mode=ops.GATE_AFTER_NORM)
    assert torch.allclose(got.double().cpu(), after, atol=1e-5, rtol=1e-5)
    assert torch.allclose(ops.gated_norm(x, torch.float32, weight=w_all, eps=1e-3).double().cpu(), plain, atol=1e-5, rtol=1e-5)
    got = ops.gated_norm(x.to(torch.bfloat16), torch.bfloat16, weight=w_all, eps=1e-3)
    assert torch.allclose(got.double().cpu(), P.rms_norm(x.to(torch.bfloat16).double().cpu(), w_all.double().cpu(), 1e-3),
                          atol=3e-2, rtol=1e-2)
    # groups wider than a warp keeps in registers: the kernel that reads them twice
    wide2 = torch.randn(3, 1200, generator=g).to(dev)
    w600 = torch.randn(600, generator=g).to(dev)
    got = ops.gated_norm(wide2, torch.float32, weight=w600, eps=1e-3, group=600, weight_per_group=True)
    want = P.rms_norm(wide2.double().cpu().view(3, 2, 600), w600.double().cpu(), 1e-3).reshape(3, 1200)
    assert torch.allclose(got.double().cpu(), want, atol=1e-5, rtol=1e-5)
    # one small matrix per head, sizes that fill no tile, with and without the sigmoid gate; a prompt's many tokens
    # and a decode step's few go through different kernels
    for T in (21, 5):
        H, O, I = 3, 70, 37
        xs, W = torch.randn(T, H * I + 2, generator=g).to(dev), torch.randn(H, O, I, generator=g).to(dev)
        gt = torch.randn(T, H * O, generator=g).to(dev)
        want = torch.einsum("hoi,thi->tho", W.double().cpu(), xs[:, 2:].double().cpu().view(T, H, I)).reshape(T, H * O)
        assert torch.allclose(ops.head_linear(xs[:, 2:], W).double().cpu(), want, atol=1e-4, rtol=1e-5)
        assert torch.allclose(ops.head_linear(xs[:, 2:], W, gate=gt).double().cpu(), want * torch.sigmoid(gt.double().cpu()),
                              atol=1e-4, rtol=1e-5)


def test_closing_norm_add_and_opening_norm_in_one_kernel():
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(11)
    for T, d, wt in ((5, 40, torch.float32), (3, 2048, torch.bfloat16), (2, 5000, torch.float32)):
        x, delta = torch.randn(T, d, generator=g).to(dev), (3 * torch.randn(T, d, generator=g)).to(dev)
        w1, w2 = torch.randn(d, generator=g).to(wt).to(dev), torch.randn(d, generator=g).to(wt).to(dev)
        new_x = x.double().cpu() + P.rms_norm(delta.double().cpu(), w1.double().cpu(), 1e-5)
        want = P.rms_norm(new_x, w2.double().cpu(), 1e-6)
        got = ops.post_pre_norm(x, delta, w1, 1e-5, w2, 1e-6, torch.float32)
        assert torch.allclose(x.double().cpu(), new_x, atol=1e-5, rtol=1e-5)
        assert torch.allclose(got.double().cpu(), want, atol=1e-5, rtol=1e-5)
    # the same bits as the two kernels it stands for
    x, delta = torch.randn(4, 64, generator=g).to(dev), torch.randn(4, 64, generator=g).to(dev)
    w1, w2 = torch.randn(64, generator=g).to(dev), torch.randn(64, generator=g).to(dev)
    xa, xb = x.clone(), x.clone()
    one = ops.post_pre_norm(xa, delta, w1, 1e-5, w2, 1e-5, torch.float32)
    two = ops.rmsnorm(xb, w2, 1e-5, torch.float32, delta=ops.rmsnorm(delta.clone(), w1, 1e-5, torch.float32))
    assert torch.equal(xa, xb) and torch.equal(one, two)


def test_gated_product_with_the_tanh_form_of_gelu():
    """The feed-forward's first product with GELU in its epilogue (a build variant of the tensor-core kernels), for
    a decode-shaped and a prompt-shaped step, against the activation worked out from the rounded products."""
    from picolm_b200 import ops
    dev = "cuda:0"
    g = torch.Generator().manual_seed(12)
    K, F = 256, 384
    gate = (torch.randn(F, K, generator=g) / 8).to(torch.bfloat16).to(dev)
    up = (torch.randn(F, K, generator=g) / 8).to(torch.bfloat16).to(dev)
    w = ops.interleave_gate_up(gate, up)
    for T in (7, 300):
        h = torch.randn(T, K, generator=g).to(torch.bfloat16).to(dev)
        gg = (h.double().cpu() @ gate.double().cpu().T).to(torch.bfloat16).double()
        uu = (h.double().cpu() @ up.double().cpu().T).to(torch.bfloat16).double()
        want = P.gelu_tanh(gg) * uu
        got = ops.linear_swiglu(h, w, activation="gelu_tanh").double().cpu()
        assert (got - want).abs().max() <= 0.02 * want.abs().max(), T
        silu = ops.linear_swiglu(h, w).double().cpu()
        assert (silu - P.silu(gg) * uu).abs().max() <= 0.02 * want.abs().max(), "the plain build still applies SiLU"


# ------------------------------------------------------------------------------------ each mixer as a model
ALONE = {
    "latent": [_latent(), _latent(heads=1, dim=16, vdim=4, kv_rank=16, q_rank=8, window=70, scale=0.25)],
    "latent_window_1": [_latent(window=1)],
    "latent_wide_window": [_latent(window=1000, kv_rank=32)],
    # a latent wider than any head the library had (a small scale keeps the scores, sums over 300 products of
    # scaled-up maps, where float32 resolves them to the tolerance)
    "latent_wide_rank": [_latent(kv_rank=300, q_rank=40, heads=2, scale=0.03)],
    "mamba2": [_mamba(), _mamba(heads=4, vdim=8, state=16, groups=1, conv=4, norm_groups=1)],
    "mamba2_groups_are_heads": [_mamba(heads=2, vdim=40, state=6, groups=2, conv=2, norm_groups=4)],
    "mamba2_one_tap": [_mamba(conv=1), _mamba(heads=3, vdim=8, state=40, groups=1, conv=7, norm_groups=3)],
    "gla": [_gla(), _gla(heads=3, dim=8, vdim=8, tau=1.0, decay_rank=2)],
    "no_feed_forward": [dict(_gla(), mlp=None), dict(_latent(), mlp=None), dict(_mamba(), mlp=None)],
    "mixed": MIXED,
    # a width that is no multiple of 4 (the fused norm kernel refuses it, the two norm kernels run) nor of 8 (no tensor map)
    "odd_width": [_latent(), _mamba(), _gla()],
}
WIDTHS = {"odd_width": 42}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_float32_model_matches_plain_in_every_cut(tmp_path, name):
    d, tensors, config = _make(tmp_path, name, _config(ALONE[name], width=WIDTHS.get(name, 40)), seed=len(name))
    eng = _engine(d)
    a, b, c = random_tokens(150, 97, 1), random_tokens(67, 97, 2), random_tokens(1, 97, 3)
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


def test_layer_that_shares_weights_has_a_state_of_its_own(tmp_path):
    """The schedule names the owner twice; every run keeps its own cache or state, and the folder holds the owner's
    tensors only."""
    layers = [_mamba(), _latent(), dict(_mamba(), weights_of=0), dict(_latent(), weights_of=1)]
    d, tensors, config = _make(tmp_path, "shared", _config(layers), seed=9)
    assert not any(n.startswith("l2.") or n.startswith("l3.") for n in tensors)
    eng = _engine(d)
    assert eng.model.spec.schedule == (0, 1, 0, 1) and len(eng.cache.state) == 2 and len(eng.cache.kv_groups[0].layers) == 2
    t = random_tokens(80, 97, 4)
    _close(run_tail(eng, t, tail=20), _plain(tensors, config, t), what="shared weights")


# -------------------------------------------------------------------------------------------- window edges
@pytest.mark.parametrize("window", [5, 64, 65, 130])
def test_window_edges_decide_logits_and_are_right(tmp_path, window):
    """With a peaked softmax the key at distance window - 1 often holds most of a row's weight: a window that is one
    token off changes those rows' logits by far more than the tolerance (the test first makes sure of that with the
    plain implementation), in prompts, in portions that start inside the window and in single tokens, with windows
    that end on a page's border and just beside it."""
    layers = [_latent(window=window, heads=2, dim=16, vdim=8, kv_rank=24, q_rank=16, scale=0.35), _gla()]
    d, tensors, config = _make(tmp_path, f"w{window}", _config(layers), seed=window, sharpen=10.0)
    t = random_tokens(290, 97, window)
    want = _plain(tensors, config, t)
    for off in (-1, 1):
        other = json.loads(json.dumps(config))
        other["layers"][0]["mixer"]["mask"]["size"] = window + off
        diff = (_plain(tensors, other, t) - want).abs().amax(dim=1) / want.std()
        assert (diff > 50 * FP32_TOL).sum() >= 3, "the weights do not make the window's edge show"
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=150), want, what="single tokens past the window")
    _close(run_chunks(eng, t, [window - 1, 2, window, 3, 290 - 2 * window - 4]), want, what="portions around the window")
    outs = run_batch(eng, [t, t[:window + 1], t[:3]], [window, window - 1, 1])
    _close(outs[0], want, what="batch")
    _close(outs[1], want[:window + 1], what="batch, a request that just fills the window")
    # pages that left the window were given back while the sequence lived
    s = eng.new_sequence()
    eng.step([(s, t)], [[0]])
    held = sum(1 for p in eng.cache.kv_groups[0].pages[s] if p)
    assert held <= (window + 63) // 64 + 1
    eng.end_sequence(s)
    eng.cache.check()


def test_far_tokens_stay_in_the_states(tmp_path):
    """Decays close to 1 keep a token in the state for hundreds of steps: the first tokens of a 600-token prompt
    still move the last logits, through prompts, portions and 200 single tokens alike."""
    layers = [_gla(tau=64.0), _mamba(), _latent(window=500, kv_rank=16)]
    d, tensors, config = _make(tmp_path, "far", _config(layers), seed=21)
    t = random_tokens(600, 97, 8)
    want = _plain(tensors, config, t)
    changed = list(t)
    changed[3] = (changed[3] + 1) % 97
    assert (_plain(tensors, config, changed)[-1] - want[-1]).abs().max() > 100 * FP32_TOL * want.std()
    eng = _engine(d)
    _close(run_whole(eng, t), want, what="whole")
    _close(run_tail(eng, t, tail=200), want, what="200 single tokens")
    _close(run_chunks(eng, t, [333, 67, 200]), want, what="portions")


# ------------------------------------------------------------------------------------------------ bfloat16
def test_bfloat16_follows_the_plain_implementation(tmp_path):
    """The serving precision stays within rounding of the exact logits, and its own cuts agree with each other far
    more closely than that."""
    d, tensors, config = _make(tmp_path, "bf16", _config(MIXED, width=64, ff=128), seed=3, sharpen=2.0)
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


@pytest.mark.parametrize("R,H,window", [(64, 3, 33), (128, 2, 64), (32, 5, 65), (80, 1, 9), (256, 2, 130), (48, 4, 1), (24, 3, 70)])
def test_attention_over_a_latent_cache_at_the_window_edge(R, H, window):
    """What the latent attention asks of the library's bfloat16 attention kernels (the tcgen05 prompt kernel at 64
    and 128, the mma.sync prompt and decode kernels at other multiples of 16, the CUDA cores otherwise): H query heads
    over ONE kv head whose values are its keys, behind a window, in pages that are out of order.  Every query is
    aimed at one key with a score that dwarfs the others: even rows at the last key inside the window, odd rows at
    the first key outside it, which must not be seen.  A portion of a prompt after a cached prefix, then single tokens."""
    from picolm_b200 import ops
    from picolm_b200.cache.sequence_cache import KVLayerCache
    dev = "cuda:0"
    g = torch.Generator().manual_seed(R + window)
    L, start = 230, 100
    c = torch.randn(L, R, generator=g).to(torch.bfloat16)
    n_pages = (L + 63) // 64
    order = [3, 1, 4, 2][:n_pages]
    pages = torch.zeros(6, 1, 64, R, dtype=torch.bfloat16)
    pages[0] = 7.0                                                   # the null page holds what nobody may read
    for b_, pg in enumerate(order):
        chunk = c[b_ * 64:(b_ + 1) * 64]
        pages[pg, 0, :chunk.shape[0]] = chunk
    pages = pages.to(dev)
    scale = 0.5

    def queries(positions):
        q = torch.zeros(len(positions), H, R)
        for r, i in enumerate(positions):
            target = i - window + 1 if r % 2 == 0 else i - window
            target = min(max(target, 0), i)
            for h in range(H):
                # along the target's latent, long enough that its score stands 30 above an ordinary key's
                q[r, h] = c[target].float() * (30.0 + 4 * h) / (scale * c[target].float().pow(2).sum())
        return q.to(torch.bfloat16)

    def plain(q, positions):
        out = torch.zeros(len(positions), H, R, dtype=torch.float64)
        cd = c.double()
        for r, i in enumerate(positions):
            lo = max(0, i - window + 1)
            sc = (q[r].double() @ cd[lo:i + 1].T) * scale
            out[r] = torch.softmax(sc, dim=-1) @ cd[lo:i + 1]
        return out.reshape(len(positions), H * R)

    def check(got, want, what):
        err = (got.double().cpu() - want).abs().max().item()
        assert err <= 0.03 * want.abs().max().item(), f"{what}: max |diff| {err:.3f} of values up to {want.abs().max():.2f}"

    table = torch.tensor([order + [0] * (5 - len(order))], dtype=torch.int32, device=dev)
    # a portion of a prompt: positions start .. L - 1 of one sequence whose first `start` positions are cached
    pos = list(range(start, L))
    step = _Step([len(pos)], [0], dev, starts=[start])
    step.seq_kv_len = torch.tensor([L], dtype=torch.int32, device=dev)
    step.max_position = L - 1
    q = queries(pos)
    kv = KVLayerCache(pages, pages, table, window, True)
    check(ops.attention(q.to(dev), kv, step, 1, scale), plain(q, pos), "portion of a prompt")
    # single tokens: four sequences on the same pages at different lengths (one ends on a page's first position)
    pos = [L - 1, 128, 191, 70]
    step = _Step([1] * 4, [0, 1, 2, 3], dev, starts=pos)
    step.seq_kv_len = torch.tensor([p_ + 1 for p_ in pos], dtype=torch.int32, device=dev)
    step.max_position = max(pos)
    q = queries(pos)
    kv = KVLayerCache(pages, pages, table.repeat(4, 1).contiguous(), window, True)
    check(ops.attention(q.to(dev), kv, step, 1, scale), plain(q, pos), "single tokens")


# ---------------------------------------------------------------------------------------------- generation
def test_greedy_generation_through_the_entry_point(tmp_path):
    """`generate` (batch planning, captured decode steps, sampled ids fed back on the device) gives the plain
    implementation's greedy tokens; more requests than fit one batch, so slots and states are used again."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "gen", _config(MIXED), seed=13, sharpen=3.0)
    prompts = [random_tokens(n, 97, 30 + i) for i, n in enumerate([5, 70, 1, 19, 33])]

    def greedy(p, n):
        seq, out = list(p), []
        for _ in range(n):
            tok = int(_plain(tensors, config, seq)[-1].argmax())
            out.append(tok)
            seq.append(tok)
        return out

    want = [greedy(p, 8) for p in prompts]
    eng = model_load(d, dtype="float32", max_batch=2)
    got, stats = generate(eng, prompts, max_tokens=8, temperature=0.0, stop_ids=[], return_stats=True)
    assert got == want
    assert stats.batches == 3 and eng.cache.slots.used == 0
    assert eng.use_graphs, "decode steps of this design are meant to replay captured graphs"
    eng.cache.check()


def test_bfloat16_generation_with_captured_prompt_steps(tmp_path):
    """In bfloat16 `generate` replays captured graphs for the prompts' step too (tokens padded to a size class, the
    padding in a sequence of its own): the logits of such a step equal those of the same prompts launched kernel by
    kernel, states and caches are left the same (the tokens generated afterwards agree), and every generated token
    is, by the exact logits, the best or within rounding of it."""
    from picolm_b200.api import generate, model_load
    d, tensors, config = _make(tmp_path, "pgraph", _config(MIXED, width=64, ff=128), seed=23, sharpen=1.0)
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
    """bin/trace_run on a Potuzen folder: a batch of unequal prompts, single tokens until the shorter requests end,
    a request alone afterwards in the slot that was given back; more requests of a few tokens than the token count
    alone would give pages for."""
    from test_gpu_trace_run import Replay
    d, tensors, config = _make(tmp_path, "replay", _config(MIXED), seed=17)
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
    """The library's command line on a Potuzen folder: random weights from a config.json, greedy tokens equal to the plain
    implementation's, sampling, the per-layer benchmark with a row for every run of the schedule (a layer that shares
    weights is its owner's second run)."""
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = [sys.executable, os.path.join(root, "bin", "picolm_b200")]
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(_config([_latent(window=6), _mamba(), dict(_gla(), mlp=None), dict(_latent(window=6), weights_of=0)]), f)
    d = str(tmp_path / "model")
    r = subprocess.run(exe + ["--random-weights", cfg_path, "--out", d, "-s", "3"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    tensors = P.read_safetensors(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "config.json")) as f:
        config = json.load(f)

    def greedy(p, n):
        seq, out = list(p), []
        for _ in range(n):
            out.append(int(_plain(tensors, config, seq)[-1].argmax()))
            seq.append(out[-1])
        return out

    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0", "--dtype", "float32", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [[int(t) for t in ln.split()] for ln in r.stdout.strip().splitlines()] == [greedy([5, 6, 7], 6), greedy([9], 6)]
    r = subprocess.run(exe + [d, "-p", "5,6,7; 9", "-n", "6", "-t", "0.8", "-k", "40", "--top-p", "0.9", "-s", "5", "--stop-id", "-1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    assert [len(ln.split()) for ln in r.stdout.strip().splitlines()] == [6, 6]
    r = subprocess.run(exe + [d, "-p", "5,6,7,8", "-n", "5", "--benchmark"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    rows = [ln.split(",") for ln in r.stderr.splitlines() if re.fullmatch(r"\d+,[0-9.]+,[0-9.]+,[0-9.]+,\d+", ln)]
    assert [int(x[0]) for x in rows] == [0, 1, 2, 0] * 3
    r = subprocess.run(exe + [d, "--list-tensors"], capture_output=True, text=True, timeout=60)
    assert "l1.mix.A_log\t[6]\tBF16" in r.stdout and "l3." not in r.stdout
