"""Nigenex (layer-list model with an fp32 residual stream) through the framework's own entry points — Context,
TextModelBase, Sessions, Master — against the plain fp32 restatement in oracle/nigenex_plain.py, on small configurations
made here with random weights.

What a schedule must not change: the logits at a position are the same whether the prompt went in whole, token by token
or in portions, whatever ran before in the same cache, and whatever other request is interleaved.  fp32 (D = float) is the
sharp comparison: the GPU and the plain code differ by summation order only, so the bar is 2e-4 of the logits' spread;
bf16 rounds every matrix operand and is held to 4e-2.  Where random weights would hide a fault — one key among many at
a window's edge — the weights are rigged so that one key dominates its row (``_spike``).
"""
import numpy as np
import pytest
import torch

from cake_b200.config import Config, LayerSpec
from cake_b200.synth import make_listed_checkpoint
from oracle import nigenex_plain as P

TOL = {"f32": 2e-4, "bf16": 4e-2}


def small_config(layers=None, width=48, vocab=61, logit_softcap=12.0, eps=1e-5, max_seq=512) -> Config:
    layers = layers or [
        LayerSpec(heads=4, kv_heads=2, head_dim=24, window=7, scale=0.3, softcap=9.0, ff=40),
        LayerSpec(heads=3, kv_heads=3, head_dim=8, window=0, scale=0.5, softcap=0.0, ff=0),        # full context, no cap, no ff
        LayerSpec(heads=6, kv_heads=1, head_dim=40, window=33, scale=0.11, softcap=50.0, ff=72),
        LayerSpec(heads=2, kv_heads=2, head_dim=16, window=1, scale=0.25, softcap=4.0, ff=16),      # sees itself only
    ]
    return Config(hidden_size=width, intermediate_size=max(s.ff for s in layers), vocab_size=vocab, num_hidden_layers=len(layers),
                  num_attention_heads=layers[0].heads, num_key_value_heads=layers[0].kv_heads, rms_norm_eps=eps,
                  head_dim=layers[0].head_dim, max_seq_len=max_seq, block_kind="nigenex", layers=layers,
                  logit_softcap=logit_softcap, model_prefix="")


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def rel_err(got, want):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all()
    return float(np.abs(got - want).max() / max(float(want.std()), 1e-3))


def plain(cfg, sd, toks, dtype):
    sdf = {k: v.float() for k, v in sd.items()}
    return P.model_logits(cfg, sdf, toks, "bf16" if dtype == "bf16" else "f32").numpy()


class Runner:
    """The framework side: a model on the GPU and its Sessions."""

    def __init__(self, cfg, sd, dtype, max_seq=None):
        from cake_b200.model import Context, Sessions, TextModelBase
        self.ctx = Context(cfg, sd, dtype, device=0, max_seq=max_seq or cfg.max_seq_len)
        self.model = TextModelBase.load(self.ctx)
        self.ses = Sessions(self.model, max_seq or cfg.max_seq_len)

    def run(self, rid, toks, cuts=None, end=True):
        """Feed ``toks`` as request ``rid`` in portions of the sizes ``cuts`` (cycled; None = whole) -> logits of every position."""
        out, p, i = [], 0, 0
        while p < len(toks):
            n = len(toks) - p if not cuts else min(cuts[i % len(cuts)], len(toks) - p)
            lg = self.ses.step(rid, toks[p:p + n], want=list(range(n)))
            self.ctx.sync()
            out.append(lg.cpu().numpy())
            p, i = p + n, i + 1
        if end:
            self.ses.end(rid)
        return np.concatenate(out, 0)

    def close(self):
        self.ctx.close()


# ---------------------------------------------------------------------------------------------- no GPU needed
def test_config_round_trip_and_refusals():
    cfg = small_config()
    d = cfg.to_hf()
    assert d["architecture"] == "Nigenex" and d["layers"][1]["mlp"] is None and d["layers"][0]["mixer"]["mask"]["size"] == 7
    back = Config.from_hf(d)
    assert back.layers == cfg.layers and back.logit_softcap == cfg.logit_softcap and back.layer_list
    assert back.layer_name(3) == "l3" and back.head_tensor_names() == ("embed", "final.norm", "head")
    bad = cfg.to_hf()
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError):
        Config.from_hf(bad)
    bad = cfg.to_hf()
    bad["layers"][0]["mixer"]["vdim"] = 12
    with pytest.raises(ValueError):
        Config.from_hf(bad)


def test_loader_checks_listed_shapes(tmp_path):
    from cake_b200.loader import listed_block_tensors, open_model, save_checkpoint
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, "bf16", seed=3)
    save_checkpoint(str(tmp_path), cfg, sd)
    cfg2, vb = open_model(str(tmp_path))
    assert cfg2.layers == cfg.layers
    t = listed_block_tensors(vb, cfg2, 1)
    assert t["ff_gate"] is None and t["v"] is None and tuple(t["q"].shape) == (24, 48) and tuple(t["norm"].shape) == ()
    sd["l0.mix.k"] = sd["l0.mix.k"][:-1]
    with pytest.raises(ValueError):
        listed_block_tensors(sd, cfg, 0)


def test_plain_mechanisms_alone():
    """The plain restatement's pieces against hand-computed values."""
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(P.rms_norm_scalar(x, 2.0, 0.0), x / (12.5 ** 0.5) * 2.0)
    h = torch.tensor([[1.0, 1.0], [3.0, 5.0]])
    assert torch.equal(P.token_shift(h, torch.tensor([0.5, 0.0])), torch.tensor([[0.5, 1.0], [2.0, 5.0]]))
    assert P.window_mask(4, 2).tolist() == [[True, False, False, False], [True, True, False, False], [False, True, True, False], [False, False, True, True]]
    assert P.window_mask(3, 0).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    b = P.distance_bias(3, torch.tensor([2.0]), torch.tensor([1.0]))
    assert torch.allclose(b[0, 2], torch.tensor([2 * np.log(3.0), 2 * np.log(2.0), 0.0]).float())
    assert abs(float(P.soft_cap(torch.tensor(100.0), 5.0)) - 5.0) < 1e-4 and float(P.soft_cap(torch.tensor(100.0), 0.0)) == 100.0


# ---------------------------------------------------------------------------------------------- on the GPU
gpu = pytest.mark.gpu


@gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_whole_prompt_matches_plain(dtype):
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, dtype, seed=11)
    toks = tokens(90, cfg.vocab_size, 1)
    r = Runner(cfg, sd, dtype)
    try:
        assert rel_err(r.run("a", toks), plain(cfg, sd, toks, dtype)) < TOL[dtype]
    finally:
        r.close()


@gpu
def test_residual_after_every_layer():
    from cake_b200.capi import check, lib, ptr
    import ctypes
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, "f32", seed=12)
    toks = tokens(40, cfg.vocab_size, 2)
    res = []
    P.model_logits(cfg, {k: v.float() for k, v in sd.items()}, toks, residuals=res)
    r = Runner(cfg, sd, "f32")
    try:
        ctx = r.ctx
        ids = np.ascontiguousarray([toks], dtype=np.uint32)
        x = ctx.empty(1, len(toks), cfg.hidden_size, dtype=torch.float32)
        check(lib().cake_b200_embed(ctx.h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), 1, len(toks), ptr(x)))
        for i, blk in enumerate(r.model.blocks):
            x = blk.forward_batch(x, [(blk.layer_name(), 0, i)], ctx, blocks=[blk])
            ctx.sync()
            assert rel_err(x[0].cpu().numpy(), res[i].numpy()) < 1e-4, i
    finally:
        r.close()


def _neutral(cfg, sd):
    """Weights that switch every mechanism of the mixer off except plain windowed attention: no shift, no bias, gate 1/2."""
    for i in range(cfg.num_hidden_layers):
        sd[f"l{i}.shift"].zero_()
        sd[f"l{i}.mix.r1"].zero_()
        sd[f"l{i}.mix.g"].zero_()
    return sd


@gpu
@pytest.mark.parametrize("which", ["norm_and_logit_cap", "shift", "bias", "gate", "softcap", "ff"])
def test_each_mechanism_alone(which):
    """One layer; everything but the mechanism under test is neutralised in the WEIGHTS (not in the code under test), and
    the expectation is assembled from the plain functions of that mechanism only."""
    sp = LayerSpec(heads=2, kv_heads=1, head_dim=16, window=0, scale=0.4, softcap=0.0, ff=24 if which == "ff" else 0)
    if which == "softcap":
        sp.softcap, sp.scale = 1.5, 3.0      # scores far into the flat part of the tanh
    cfg = small_config([sp], width=32, vocab=37, logit_softcap=3.0 if which == "norm_and_logit_cap" else 0.0)
    sd = _neutral(cfg, make_listed_checkpoint(cfg, "f32", seed=20, std=0.3))
    toks = tokens(12, cfg.vocab_size, 3)
    f = {k: v.float() for k, v in sd.items()}
    eps = cfg.rms_norm_eps
    x0 = f["embed"][toks]
    if which == "norm_and_logit_cap":   # the block adds nothing: logits = cap(head . norm(embed))
        sd["l0.mix.o"].zero_()
        want = P.soft_cap(P.rms_norm_scalar(x0, f["final.norm"], eps) @ f["head"].t(), 3.0)
    else:
        if which == "shift":
            sd["l0.shift"].copy_(torch.linspace(0.0, 1.0, 32))
        if which == "bias":
            sd["l0.mix.r1"].copy_(torch.tensor([0.7, 2.0]))
        if which == "gate":
            sd["l0.mix.g"].copy_(torch.randn(2, 32, generator=torch.Generator().manual_seed(1)))
        f = {k: v.float() for k, v in sd.items()}
        h = P.rms_norm_scalar(x0, f["l0.norm1"], eps)
        hs = P.token_shift(h, f["l0.shift"])
        S = len(toks)
        q = (hs @ f["l0.mix.q"].t()).view(S, 2, 16)
        k = (hs @ f["l0.mix.k"].t()).view(S, 1, 16).repeat_interleave(2, 1)
        s = P.soft_cap(torch.einsum("ihd,jhd->hij", q, k) * sp.scale, sp.softcap) - P.distance_bias(S, f["l0.mix.r1"], f["l0.mix.r2"])
        p = torch.softmax(s.masked_fill(~P.window_mask(S, 0)[None], float("-inf")), -1)
        o = torch.einsum("hij,jhd->ihd", p, k) * torch.sigmoid(hs @ f["l0.mix.g"].t())[:, :, None]
        x1 = x0 + o.reshape(S, 32) @ f["l0.mix.o"].t()
        if which == "ff":
            x1 = x1 + (P.gelu_tanh(h @ f["l0.mlp.gate"].t()) * (h @ f["l0.mlp.up"].t())) @ f["l0.mlp.down"].t()
        want = P.rms_norm_scalar(x1, f["final.norm"], eps) @ f["head"].t()
    r = Runner(cfg, sd, "f32")
    try:
        assert rel_err(r.run("a", toks), want.numpy()) < TOL["f32"]
    finally:
        r.close()


@gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_prefill_decode_and_portions_agree(dtype):
    """whole == token by token == portions of 2, 3, 5 / 17 / 64, 1 — and all equal the plain code; the first tokens of a
    sequence (shift state zero, windows not yet full) are part of every comparison."""
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, dtype, seed=13)
    toks = tokens(150, cfg.vocab_size, 4)
    want = plain(cfg, sd, toks, dtype)
    r = Runner(cfg, sd, dtype)
    try:
        whole = r.run("w", toks)
        assert rel_err(whole, want) < TOL[dtype]
        for cuts in ([1], [2], [2, 3, 5], [17], [64, 1], [7, 1, 1, 1, 30]):
            got = r.run("c", toks, cuts)
            assert rel_err(got, want) < TOL[dtype], cuts
            assert rel_err(got, whole) < (1e-4 if dtype == "f32" else TOL[dtype]), cuts
    finally:
        r.close()


def _spike(cfg, sd, layer, tok, gain=6.0):
    """Make token id ``tok`` a key that dominates every row that can see it in ``layer``: its embedding is scaled up, and the
    layer's q and k projections are made equal (G == H there) so that q . k is a large positive square for that key.
    The distance bias is switched off so that a far key keeps its lead."""
    sd["embed"][tok] *= gain
    sd[f"l{layer}.mix.q"].copy_(sd[f"l{layer}.mix.k"])
    sd[f"l{layer}.mix.r1"].zero_()
    return sd


@gpu
@pytest.mark.parametrize("mode", ["prompt", "decode", "portions"])
def test_window_edges_with_a_dominant_key(mode):
    """A dominant key at position j: the rows j + w - 1 (last that sees it) and j + w (first that does not) differ by a
    lot, so a window that is one off cannot hide.  Also a far key under a full-context layer, hundreds of positions back."""
    w = 19
    layers = [LayerSpec(heads=2, kv_heads=2, head_dim=16, window=w, scale=0.6, softcap=20.0, ff=0),
              LayerSpec(heads=2, kv_heads=2, head_dim=16, window=0, scale=0.6, softcap=20.0, ff=24)]
    cfg = small_config(layers, width=32, vocab=50, logit_softcap=0.0)
    sd = make_listed_checkpoint(cfg, "f32", seed=14, std=0.25)
    _spike(cfg, sd, 0, 7)
    _spike(cfg, sd, 1, 7, gain=1.0)
    rng = np.random.default_rng(5)
    toks = [int(t) for t in rng.integers(8, 50, 330)]     # the special token occurs only where it is put
    j = 40
    toks[j] = 7
    want = plain(cfg, sd, toks, "f32")
    sdf = {k: v.float() for k, v in sd.items()}
    # the rig works: taking the key out of the window changes the row a lot (so an off-by-one would show)
    assert np.abs(want[j + w - 1] - want[j + w]).max() > 50 * TOL["f32"] * want.std()
    r = Runner(cfg, sd, "f32")
    try:
        if mode == "prompt":
            got = r.run("a", toks)
        elif mode == "decode":
            got = np.concatenate([r.run("a", toks[:j + 3], end=False), r.run("a", toks[j + 3:], [1])], 0)
        else:
            got = r.run("a", toks, [w - 1, 2, w, w + 1, 5])
        for p in (0, 1, j - 1, j, j + 1, j + w - 2, j + w - 1, j + w, j + w + 1, 329):
            assert rel_err(got[p], want[p]) < TOL["f32"], (mode, p)
        assert rel_err(got, want) < TOL["f32"]
    finally:
        r.close()
    del sdf


@gpu
@pytest.mark.parametrize("hd", [128, 64, 96, 160, 256, 24])
def test_window_edges_on_tensor_core_shapes(hd):
    """The same rig in bf16 at sizes the tensor-core kernels take (tcgen05 attention for head size 128, mma.sync for 64 and
    96; tcgen05 GEMMs for width 128) and at head sizes they do not take: prompt in one step, in portions around the
    window's size, and decoded (the eight-lanes-per-key kernel with one to four 16-byte pieces per lane; 24 = three pieces
    per key, five lanes of a group idle)."""
    w = 70
    layers = [LayerSpec(heads=2, kv_heads=2, head_dim=hd, window=w, scale=0.3, softcap=20.0, ff=0),
              LayerSpec(heads=2, kv_heads=2, head_dim=hd, window=0, scale=0.3, softcap=20.0, ff=128)]
    cfg = small_config(layers, width=128, vocab=128, logit_softcap=0.0)
    sd = make_listed_checkpoint(cfg, "bf16", seed=18, std=0.12)
    _spike(cfg, sd, 0, 7, gain=4.0)
    _spike(cfg, sd, 1, 7, gain=1.0)
    rng = np.random.default_rng(6)
    toks = [int(t) for t in rng.integers(8, 128, 420)]
    j = 150
    toks[j] = 7
    want = plain(cfg, sd, toks, "bf16")
    assert np.abs(want[j + w - 1] - want[j + w]).max() > 20 * TOL["bf16"] * want.std()
    r = Runner(cfg, sd, "bf16")
    try:
        runs = {"prompt": r.run("a", toks), "portions": r.run("b", toks, [w - 1, 2, w, w + 1, 129, 16]),
                "decode": np.concatenate([r.run("c", toks[:j + 3], end=False), r.run("c", toks[j + 3:j + w + 40], [1])], 0)}
        for mode, got in runs.items():
            n = got.shape[0]
            for p in (0, 1, j, j + 1, j + w - 2, j + w - 1, j + w, j + w + 1, n - 1):
                assert rel_err(got[p], want[p]) < TOL["bf16"], (mode, p)
            assert rel_err(got, want[:n]) < TOL["bf16"], mode
    finally:
        r.close()


@gpu
def test_interleaved_requests_and_reused_caches():
    """Two unequal requests stepped in turn equal each one alone; a cache given back by a finished request and taken by the
    next (longer and shorter than its predecessor) leaves no trace of the old rows or of the old shift state."""
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, "f32", seed=15)
    a, b, c = tokens(70, cfg.vocab_size, 6), tokens(31, cfg.vocab_size, 7), tokens(95, cfg.vocab_size, 8)
    wa, wb, wc = (plain(cfg, sd, t, "f32") for t in (a, b, c))
    r = Runner(cfg, sd, "f32")
    try:
        ga, gb = [], []
        pa = pb = 0
        while pa < len(a) or pb < len(b):
            if pa < len(a):
                n = min(9, len(a) - pa)
                ga.append(r.ses.step("A", a[pa:pa + n], want=list(range(n)))); r.ctx.sync(); ga[-1] = ga[-1].cpu().numpy(); pa += n
            if pb < len(b):
                n = min(4, len(b) - pb)
                gb.append(r.ses.step("B", b[pb:pb + n], want=list(range(n)))); r.ctx.sync(); gb[-1] = gb[-1].cpu().numpy(); pb += n
        assert rel_err(np.concatenate(ga, 0), wa) < TOL["f32"] and rel_err(np.concatenate(gb, 0), wb) < TOL["f32"]
        r.ses.end("A"); r.ses.end("B")
        assert len(r.ses.free) == 2
        for rid, t, w in (("C", c, wc), ("D", b, wb), ("E", a, wa)):   # every one of them runs in a used cache
            assert rel_err(r.run(rid, t, [13, 2]), w) < TOL["f32"], rid
            assert len(r.ses.free) == 2
    finally:
        r.close()


@gpu
def test_long_decode_past_every_window():
    cfg = small_config()
    sd = make_listed_checkpoint(cfg, "bf16", seed=16)
    toks = tokens(5 + 4 * 33, cfg.vocab_size, 9)
    want = plain(cfg, sd, toks, "bf16")
    r = Runner(cfg, sd, "bf16")
    try:
        got = np.concatenate([r.run("a", toks[:5], end=False), r.run("a", toks[5:], [1])], 0)
        assert rel_err(got, want) < TOL["bf16"]
    finally:
        r.close()


@gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_other_sizes(dtype):
    """Sizes that exercise the tensor-core shapes (width and ff multiples of 64, head sizes 64 and 128) and ones that do not
    (width 42, head size 20, ff 101), heads == kv_heads and one kv head, ff != width, a window longer than the sequence."""
    for seed, (width, layers) in enumerate([
        (128, [LayerSpec(heads=4, kv_heads=1, head_dim=64, window=50, scale=0.125, softcap=30.0, ff=256),
               LayerSpec(heads=2, kv_heads=2, head_dim=128, window=4000, scale=0.09, softcap=15.0, ff=128)]),
        (42, [LayerSpec(heads=5, kv_heads=5, head_dim=20, window=3, scale=0.2, softcap=8.0, ff=101)]),   # rows that are no multiple of 16 bytes
        (192, [LayerSpec(heads=6, kv_heads=3, head_dim=96, window=64, scale=0.1, softcap=25.0, ff=320)] * 2),
    ]):
        cfg = small_config(layers, width=width, vocab=130)
        sd = make_listed_checkpoint(cfg, dtype, seed=30 + seed)
        toks = tokens(200, cfg.vocab_size, seed)
        want = plain(cfg, sd, toks, dtype)
        r = Runner(cfg, sd, dtype)
        try:
            assert rel_err(r.run("a", toks), want) < TOL[dtype], width
            assert rel_err(r.run("b", toks, [128, 3, 1]), want) < TOL[dtype], width
        finally:
            r.close()


@gpu
def test_greedy_generation_through_master():
    """Master.generate_text (prefill, then one token per step through next_token and the device-side argmax) == plain greedy."""
    from cake_b200.model import Context, Master, TextModelBase
    cfg = small_config(logit_softcap=0.0)
    sd = make_listed_checkpoint(cfg, "f32", seed=17, std=0.2)
    sd["head"] = (sd["embed"].float() * 0.5).to(sd["head"].dtype)       # peaked logits: wide top-1 / top-2 margins
    prompt = tokens(9, cfg.vocab_size, 10)
    want = P.greedy(cfg, {k: v.float() for k, v in sd.items()}, prompt, 12)
    ctx = Context(cfg, sd, "f32", device=0, max_seq=64)
    try:
        out = Master(TextModelBase.load(ctx)).generate_text(prompt, 12)
        assert out["tokens"] == want
        assert ctx.launch_count() > 0
    finally:
        ctx.close()
