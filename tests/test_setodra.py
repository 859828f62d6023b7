"""Setodra (mixer-list model: latent attention, retention, state-space layers, routed feed-forward, looped layer ranges)
through the framework's own entry points (Context, TextModelBase, Sessions, Master) against the plain restatement in
oracle/setodra_plain.py, on small configurations made here with random weights.

What a schedule must not change: the logits at a position are the same whether the prompt went in whole, token by token
or in portions, whatever ran before in the same cache slot, and whatever other request is interleaved.  fp32 (D = float)
is the sharp comparison: the GPU and the plain code differ by summation order only.  bf16 rounds every projection, so a
router's close call may flip there: the bf16 bar is asked of 95 % of the positions.  The error of a position is the root
mean square over the vocabulary of the difference (mean removed) over the spread of the expected logits.
"""
import json

import numpy as np
import pytest
import torch

from cake_b200.config import Config, MixerSpec, MoeSpec, RotarySpec
from cake_b200.synth import make_mixer_checkpoint
from oracle import setodra_plain as P

TOL = {"f32": 2e-4, "bf16": 5e-2, "f16": 2e-2}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, scale=0.2, base=5000.0, scaling=True, moe=None):
    rot = RotarySpec(dims=rot_dim, base=base, factor=4.0, fast=16.0, slow=1.0, original=64) if scaling else RotarySpec(dims=rot_dim, base=base)
    return MixerSpec(type="latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale, rot=rot, moe=moe)


def retention(heads=3, dim=16, vdim=24, rot_dims=8, decay=None, moe=None):
    decay = decay or [0.9, 0.97, 0.995, 0.8, 0.99][:heads]
    return MixerSpec(type="retention", heads=heads, dim=dim, vdim=vdim, decay=decay, rot=RotarySpec(dims=rot_dims, base=777.0), moe=moe)


def mamba(heads=4, vdim=12, state=20, groups=2, conv=4, norm_groups=3, moe=None):
    return MixerSpec(type="mamba2", heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups, moe=moe)


def moe(experts=5, identity=1, top=2, scale=1.7, ff=24, shared_ff=40):
    return MoeSpec(experts=experts, identity=identity, top=top, scale=scale, ff=ff, shared_ff=shared_ff)


def make_config(layers, loop=None, width=40, vocab=53, eps=1e-5, embed_scale=2.5, max_seq=512) -> Config:
    return Config(hidden_size=width, intermediate_size=0, vocab_size=vocab, num_hidden_layers=len(layers), num_attention_heads=layers[0].heads,
                  num_key_value_heads=layers[0].heads, rms_norm_eps=eps, head_dim=layers[0].vdim, max_seq_len=max_seq, block_kind="setodra",
                  layers=layers, model_prefix="", embed_scale=embed_scale, loop=loop)


def full_config(**kw) -> Config:
    """Every mechanism, unequal sizes, a loop over the middle layers, one layer without a feed-forward."""
    layers = [retention(moe=moe()), mamba(moe=moe(experts=4, identity=2, top=3, shared_ff=0)), latent(moe=None),
              mamba(heads=2, vdim=16, state=8, groups=1, conv=2, norm_groups=1, moe=moe(experts=3, identity=0, top=1, ff=16, shared_ff=8)),
              latent(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16, scaling=False, moe=moe())]
    return make_config(layers, loop={"start": 1, "stop": 4, "times": 2}, **kw)


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def errors(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.isfinite(got).all()
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / max(float(want.std()), 1e-3)


def close(got, want, dtype, what=""):
    e = errors(got, want)
    if dtype == "f32":
        assert e.max() < TOL[dtype], f"{what}: worst {e.max():.3g} at position {int(e.argmax())}"
    else:
        assert np.quantile(e, 0.95) < TOL[dtype], f"{what}: 95 % of positions within {np.quantile(e, 0.95):.3g}"


def plain(cfg, sd, toks, trace=None):
    wt = {k: v.float() for k, v in sd.items()}
    return P.forward(cfg.to_hf(), wt, toks, dt=torch.float32, trace=trace).numpy()


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
def test_config_round_trip_and_run_plan():
    cfg = full_config()
    d = cfg.to_hf()
    assert d["architecture"] == "Setodra" and len(d["layers"]) == 5 and d["layers"][2]["mlp"] is None
    back = Config.from_hf(json.loads(json.dumps(d)))
    assert back.layers == cfg.layers and back.loop == cfg.loop and back.embed_scale == cfg.embed_scale
    assert back.layer_list and not back.scalar_final_norm
    assert cfg.run_plan() == [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None), (4, None)]
    assert P.layer_runs(d) == cfg.run_plan()
    assert make_config([retention()], loop=None).run_plan() == [(0, None)]
    assert make_config([retention(), mamba()], loop={"start": 0, "stop": 2, "times": 3}).run_plan() == \
        [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None)]
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "attention"
    with pytest.raises(ValueError):
        Config.from_hf(bad)
    bad = json.loads(json.dumps(d))
    bad["loop"]["stop"] = 9
    with pytest.raises(ValueError):
        Config.from_hf(bad)


def test_checkpoint_names_and_shapes():
    from cake_b200.loader import mixer_block_tensors
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, "bf16", seed=1)
    assert sd["loop.step"].shape == (2, cfg.hidden_size) and sd["final.norm"].shape == (cfg.hidden_size,)
    for i, sp in enumerate(cfg.layers):
        t = mixer_block_tensors(sd, cfg, i)
        assert t["o"].shape == (cfg.hidden_size, sp.inner)
        if sp.moe is not None:
            assert len(t["e_gate"]) == sp.moe.experts and t["router"].shape[0] == sp.moe.experts + sp.moe.identity
            assert ("s_sg" in t) == bool(sp.moe.shared_ff)
        else:
            assert "router" not in t
    broken = dict(sd)
    broken["l2.mix.uk"] = sd["l2.mix.uk"][:-1]
    with pytest.raises(ValueError):
        mixer_block_tensors(broken, cfg, 2)


def test_plain_retention_equals_its_parallel_form():
    """The token-by-token recurrence of the oracle against the same layer written as a decayed causal product."""
    torch.manual_seed(0)
    m = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.9, 0.97], "rot": {"dims": 4, "base": 100.0}}
    S, W = 9, 12
    wt = {"l0.mix." + k: torch.randn(n, W) * 0.3 for k, n in (("q", 12), ("k", 12), ("v", 10), ("g", 10))}
    wt["l0.mix.o"] = torch.randn(W, 10) * 0.3
    h = torch.randn(S, W)
    got = P.retention(h, wt, "l0.", m, 1e-6)
    q = P.rotate(P.lin(wt["l0.mix.q"], h).view(S, 2, 6), m["rot"])
    k = P.rotate(P.lin(wt["l0.mix.k"], h).view(S, 2, 6), m["rot"]) * 6 ** -0.5
    v = P.lin(wt["l0.mix.v"], h).view(S, 2, 5)
    i, j = torch.arange(S)[:, None], torch.arange(S)[None, :]
    o = torch.zeros(S, 2, 5)
    for hd, g in enumerate(m["decay"]):
        a = (q[:, hd] @ k[:, hd].t()) * torch.where(i >= j, torch.tensor(g) ** (i - j).clamp(min=0).float(), torch.tensor(0.0))
        o[:, hd] = a @ v[:, hd]
    want = P.lin(wt["l0.mix.o"], P.rms_unit(o, 1e-6).reshape(S, 10) * P.silu(P.lin(wt["l0.mix.g"], h)))
    assert torch.allclose(got, want, atol=1e-5)


def test_plain_rotation_keeps_position_zero_and_ramp_ends():
    rot = {"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "fast": 16.0, "slow": 1.0, "original": 64}}
    f, amp = P.rope_frequencies(rot)
    f0, _ = P.rope_frequencies({"dims": 8, "base": 10000.0})
    assert abs(amp - (0.1 * np.log(4.0) + 1)) < 1e-12
    assert torch.all(f <= f0 + 1e-15) and torch.all(f >= f0 / 4 - 1e-15)
    v = torch.randn(1, 2, 10)
    out = P.rotate(v, rot)
    assert torch.allclose(out[..., :8], v[..., :8] * amp) and torch.equal(out[..., 8:], v[..., 8:])


# ---------------------------------------------------------------------------------------------- on the GPU
MECHANISMS = {
    "retention": lambda: make_config([retention()]),
    "retention_full_rotation_one_head": lambda: make_config([retention(heads=1, dim=8, vdim=8, rot_dims=8, decay=[0.93])]),
    "retention_no_rotation": lambda: make_config([retention(rot_dims=0)]),
    "state_space": lambda: make_config([mamba()]),
    "state_space_one_group_two_taps": lambda: make_config([mamba(heads=3, vdim=8, state=16, groups=1, conv=2, norm_groups=1)]),
    "state_space_groups_equal_heads": lambda: make_config([mamba(heads=4, vdim=16, state=8, groups=4, conv=5, norm_groups=4)]),
    "latent": lambda: make_config([latent()]),
    "latent_plain_rotation_wide": lambda: make_config([latent(heads=2, dim=16, rot_dim=32, vdim=8, kv_rank=200, scaling=False)]),
    "latent_sharp": lambda: make_config([latent(scale=3.0)]),
    "moe": lambda: make_config([retention(moe=moe())]),
    "moe_identity_only_choice": lambda: make_config([retention(moe=moe(experts=2, identity=3, top=4, shared_ff=0))]),
    "moe_top1_no_identity": lambda: make_config([mamba(moe=moe(experts=6, identity=0, top=1, ff=8, shared_ff=16))]),
    "moe_many_experts": lambda: make_config([retention(moe=moe(experts=40, identity=3, top=5, ff=8, shared_ff=16))]),
    "state_space_key_size_48": lambda: make_config([mamba(heads=2, vdim=32, state=48, groups=1, conv=3, norm_groups=2)]),
    "state_space_key_size_256": lambda: make_config([mamba(heads=1, vdim=64, state=256, groups=1, conv=2, norm_groups=1)]),
    "retention_key_size_96": lambda: make_config([retention(heads=2, dim=96, vdim=32, rot_dims=64, decay=[0.9, 0.99])]),
    "retention_key_size_128": lambda: make_config([retention(heads=1, dim=128, vdim=64, rot_dims=128, decay=[0.98])]),
    "retention_key_size_192": lambda: make_config([retention(heads=1, dim=192, vdim=32, rot_dims=32, decay=[0.95])]),
    "latent_rank_400": lambda: make_config([latent(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=400, scale=0.3)]),
    "loop_from_layer0": lambda: make_config([retention(), latent()], loop={"start": 0, "stop": 2, "times": 3}),
    "loop_once_tail_only": lambda: make_config([mamba(), retention()], loop={"start": 1, "stop": 2, "times": 1}),
    "no_embedding_scale": lambda: make_config([latent(moe=moe())], embed_scale=1.0),
}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    cfg = MECHANISMS[name]()
    sd = make_mixer_checkpoint(cfg, "f32", seed=11)
    toks = tokens(45, cfg.vocab_size, seed=3)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("a", toks), want, "f32", name)
        close(r.run("b", toks, cuts=[1]), want, "f32", name + " token by token")
        close(r.run("c", toks, cuts=[7, 2, 3]), want, "f32", name + " portions")
    finally:
        r.close()


@pytest.mark.gpu
def test_residual_after_every_layer_run():
    """Block by block with the framework's own calls: the stream after every run of the plan, injections included."""
    import ctypes
    from cake_b200.capi import c_uint32, check, lib, ptr
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, "f32", seed=5)
    toks = tokens(19, cfg.vocab_size, seed=8)
    trace = []
    plain(cfg, sd, toks, trace)
    r = Runner(cfg, sd, "f32")
    try:
        ctx, model = r.ctx, r.model
        ids = np.ascontiguousarray([toks], dtype=np.uint32)
        x0 = ctx.empty(1, len(toks), cfg.hidden_size, dtype=torch.float32)
        check(lib().cake_b200_embed(ctx.h, ids.ctypes.data_as(ctypes.POINTER(c_uint32)), 1, len(toks), ptr(x0)))
        with torch.cuda.stream(ctx.torch_stream):
            x = x0.clone()
        assert sorted(model.injections) == [1, 4]
        for j, blk in enumerate(model.blocks):
            if j in model.injections:
                t = model.injections[j]
                check(lib().cake_b200_stream_inject(ctx.h, ptr(x), ptr(x0) if t > 0 else None, ptr(model.loop_steps[t]), t, len(toks)))
            x = blk.forward_batch(x, [(blk.layer_name(), 0, j)], ctx, blocks=[blk])
            ctx.sync()
            want = trace[j].numpy()
            assert np.abs(x[0].cpu().numpy() - want).max() < 2e-4 * max(1.0, np.abs(want).max()), f"run {j} ({blk.layer_name()})"
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_schedules_agree_with_the_plain_model(dtype):
    """Whole, token by token and portions down to two tokens, first tokens included, on the model with everything."""
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, dtype, seed=21)
    toks = tokens(83, cfg.vocab_size, seed=4)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, dtype)
    try:
        whole = r.run("w", toks)
        close(whole, want, dtype, "whole")
        for cuts in ([1], [2], [2, 3, 5], [17], [64, 1], [1, 40, 2]):
            got = r.run("c", toks, cuts=cuts)
            close(got, want, dtype, f"portions {cuts}")
            if dtype == "f32":
                close(got, whole, dtype, f"portions {cuts} against whole")
        close(r.run("f", toks[:3], cuts=[1]), want[:3], dtype, "the first tokens")
    finally:
        r.close()


@pytest.mark.gpu
def test_interleaved_requests_and_reused_slots():
    """Two unequal requests whose steps alternate give what each gives alone; a slot that a longer request left behind is
    reused by a shorter one and by a longer one (state and cache rows of the previous owner must not leak)."""
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, "f32", seed=31)
    a, b, c = tokens(37, cfg.vocab_size, 1), tokens(12, cfg.vocab_size, 2), tokens(50, cfg.vocab_size, 3)
    wa, wb, wc = plain(cfg, sd, a), plain(cfg, sd, b), plain(cfg, sd, c)
    r = Runner(cfg, sd, "f32")
    try:
        ga, gb, pa, pb = [], [], 0, 0
        while pa < len(a) or pb < len(b):
            if pa < len(a):
                n = min(5, len(a) - pa)
                ga.append(r.ses.step("a", a[pa:pa + n], want=list(range(n))).cpu().numpy())
                pa += n
            if pb < len(b):
                n = min(2, len(b) - pb)
                gb.append(r.ses.step("b", b[pb:pb + n], want=list(range(n))).cpu().numpy())
                pb += n
        close(np.concatenate(ga), wa, "f32", "interleaved a")
        close(np.concatenate(gb), wb, "f32", "interleaved b")
        r.ses.end("a")
        r.ses.end("b")
        n_caches = len(r.ses.free)
        close(r.run("b2", b, cuts=[3]), wb, "f32", "shorter request in a used slot")
        close(r.run("c", c, cuts=[9, 1]), wc, "f32", "longer request in a used slot")
        close(r.run("a2", a), wa, "f32", "whole prompt in a used slot")
        assert len(r.ses.free) == n_caches   # slots were reused, none added
    finally:
        r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
def test_batch_rows_against_each_alone(dtype):
    """Three equal-length rows in one call (a prompt portion, a second portion, then single tokens) give what each row gives
    alone: cache rows, recurrent state, convolution history and expert plans are per batch row."""
    from cake_b200.model import Cache
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, dtype, seed=91)
    rows = [tokens(40, cfg.vocab_size, seed=20 + i) for i in range(3)]
    want = np.stack([plain(cfg, sd, r) for r in rows])          # [3, 40, vocab]
    r = Runner(cfg, sd, dtype)
    try:
        ctx, model = r.ctx, r.model
        ctx.cache = Cache(ctx, 3, cfg.max_seq_len)
        got, pos = [[] for _ in rows], 0
        for n in (23, 9, 1, 1, 6):
            ids = np.array([row[pos:pos + n] for row in rows], dtype=np.uint32)
            lg = model.forward(ids, pos, want=list(range(3 * n))).cpu().numpy().reshape(3, n, -1)
            for b in range(3):
                got[b].append(lg[b])
            pos += n
        for b in range(3):
            close(np.concatenate(got[b]), want[b], dtype, f"batch row {b}")
    finally:
        r.close()


@pytest.mark.gpu
def test_far_key_in_prompt_portions_and_decoding():
    """A sharp latent attention (one key dominates each row, most of them far back) over a few hundred positions: whole,
    in portions, and with the tail decoded token by token.  That the far keys matter is checked on the plain model itself:
    without the first half of the sequence its last rows come out differently (the rotation is relative, so nothing else
    changes for them)."""
    cfg = make_config([latent(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, scale=2.5), latent(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=72, scale=1.5)])
    sd = make_mixer_checkpoint(cfg, "f32", seed=41)
    toks = tokens(330, cfg.vocab_size, seed=6)
    want = plain(cfg, sd, toks)
    tail = plain(cfg, sd, toks[165:])
    assert errors(tail[-20:], want[-20:]).max() > 50 * TOL["f32"]
    for dtype in ("f32", "bf16"):
        r = Runner(cfg, make_mixer_checkpoint(cfg, dtype, seed=41), dtype)
        try:
            close(r.run("w", toks), want, dtype, "whole")
            close(r.run("d", toks, cuts=[128] * 2 + [1] * 74), want, dtype, "prompt portions then decoding")
            close(r.run("p", toks, cuts=[63, 2, 31]), want, dtype, "odd portions")
        finally:
            r.close()


@pytest.mark.gpu
def test_long_decoding_through_recurrent_state():
    """Recurrent layers decoded token by token far past anything a portion covered, with a slowly decaying head."""
    cfg = make_config([retention(heads=2, decay=[0.999, 0.9]), mamba(heads=2, groups=1), retention(heads=1, dim=8, vdim=8, decay=[0.99])])
    sd = make_mixer_checkpoint(cfg, "f32", seed=43)
    toks = tokens(260, cfg.vocab_size, seed=7)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "f32")
    try:
        close(r.run("d", toks, cuts=[40] + [1] * 220), want, "f32", "a short prompt then long decoding")
    finally:
        r.close()


@pytest.mark.gpu
def test_other_sizes_bf16_and_tensor_core_shapes():
    """Sizes whose projections take the tensor-core GEMM (multiples of 128 / 64) next to ones that do not."""
    layers = [retention(heads=2, dim=64, vdim=64, rot_dims=32, decay=[0.95, 0.99], moe=moe(experts=4, identity=1, top=2, ff=64, shared_ff=64)),
              latent(heads=2, dim=32, rot_dim=32, vdim=64, kv_rank=64, scale=0.1, moe=None),
              mamba(heads=4, vdim=32, state=32, groups=2, conv=3, norm_groups=2, moe=moe(experts=3, identity=0, top=2, ff=128, shared_ff=0))]
    cfg = make_config(layers, width=128, vocab=256)
    for dtype in ("bf16", "f32"):
        sd = make_mixer_checkpoint(cfg, dtype, seed=51)
        toks = tokens(70, cfg.vocab_size, seed=9)
        want = plain(cfg, sd, toks)
        r = Runner(cfg, sd, dtype)
        try:
            close(r.run("w", toks), want, dtype, "whole")
            close(r.run("c", toks, cuts=[33, 2, 1]), want, dtype, "portions")
        finally:
            r.close()


@pytest.mark.gpu
def test_long_portions_on_the_tensor_cores():
    """Sizes at which long portions in bf16 take the matrix-product form of the latent attention (several blocks of rows, with
    and without keys from earlier portions) and the grouped expert products, against the plain model and against the same
    positions decoded through the per-row kernels."""
    layers = [latent(heads=8, dim=32, rot_dim=64, vdim=32, kv_rank=128, scale=0.6, moe=moe(experts=6, identity=1, top=2, ff=64, shared_ff=128)),
              retention(heads=2, dim=32, vdim=64, rot_dims=32, decay=[0.97, 0.995], moe=None)]
    cfg = make_config(layers, width=128, vocab=96, max_seq=1024)
    sd = make_mixer_checkpoint(cfg, "bf16", seed=71)
    toks = tokens(700, cfg.vocab_size, seed=13)
    want = plain(cfg, sd, toks)
    r = Runner(cfg, sd, "bf16")
    try:
        whole = r.run("w", toks)
        close(whole, want, "bf16", "whole")
        cut = r.run("c", toks, cuts=[300, 390, 2, 1])
        close(cut, want, "bf16", "portions")
        small = r.run("s", toks, cuts=[100])       # every portion below the matrix-product threshold
        close(small, want, "bf16", "short portions")
        assert np.quantile(errors(whole, small), 0.95) < TOL["bf16"]
        # two batch rows through the same long-portion kernels, then a second portion on top
        from cake_b200.model import Cache
        a, b = toks[:340], toks[340:680]
        wa, wb = plain(cfg, sd, a), plain(cfg, sd, b)
        r.ctx.cache = Cache(r.ctx, 2, cfg.max_seq_len)
        g1 = r.model.forward(np.array([a[:200], b[:200]], dtype=np.uint32), 0, want=list(range(400))).cpu().numpy().reshape(2, 200, -1)
        g2 = r.model.forward(np.array([a[200:], b[200:]], dtype=np.uint32), 200, want=list(range(280))).cpu().numpy().reshape(2, 140, -1)
        close(np.concatenate([g1[0], g2[0]]), wa, "bf16", "batch row 0")
        close(np.concatenate([g1[1], g2[1]]), wb, "bf16", "batch row 1")
    finally:
        r.close()


@pytest.mark.gpu
def test_greedy_generation_through_master():
    from cake_b200.model import Context, Master, TextModelBase
    cfg = full_config()
    sd = make_mixer_checkpoint(cfg, "f32", seed=61)
    prompt = tokens(9, cfg.vocab_size, seed=12)
    ctx = Context(cfg, sd, "f32", device=0, max_seq=64)
    try:
        out = Master(TextModelBase.load(ctx)).generate_text(prompt, 12)["tokens"]
    finally:
        ctx.close()
    seq = list(prompt)
    for tok in out:   # every generated token is the plain model's greedy choice, or within a hair of it
        lg = plain(cfg, sd, seq)[-1]
        assert lg[tok] >= lg.max() - 1e-2 * np.abs(lg).max(), (len(seq), tok, int(lg.argmax()))   # the sampler reads 16-bit logits
        seq.append(tok)
    assert len(out) == 12


@pytest.mark.gpu
def test_checkpoint_on_disk_through_the_trace_replayer_and_the_generate_command(tmp_path):
    """config.json + model.safetensors on disk -> `bin/trace_run` (steps on standard input, logits as files) and
    `python -m cake_b200.run` (token ids out): the model class follows the config in both."""
    import os
    import subprocess
    import sys
    from cake_b200.loader import open_model, save_checkpoint
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = full_config(max_seq=64)
    sd = make_mixer_checkpoint(cfg, "bf16", seed=81)
    model_dir, out_dir = str(tmp_path / "model"), str(tmp_path / "out")
    save_checkpoint(model_dir, cfg, sd)
    back, vb = open_model(model_dir)
    assert back.layers == cfg.layers and back.loop == cfg.loop and set(vb.keys()) == set(sd.keys())
    toks = tokens(21, cfg.vocab_size, seed=14)
    want = plain(cfg, sd, toks)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:9], "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[9:11], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[11:], "want": [9]}], "end": ["r"]},
             {"step": 3, "entries": [{"id": "s", "tokens": toks[:4], "want": [3]}], "end": ["s"]}]
    for dtype in ("float32", "bfloat16"):
        res = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens", "40"],
                             input="".join(json.dumps(x) + "\n" for x in steps), capture_output=True, text=True, timeout=900)
        assert res.returncode == 0, res.stderr[-2000:]
        assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        assert not os.path.exists(os.path.join(out_dir, "1.f32"))
        got = {i: np.fromfile(os.path.join(out_dir, f"{i}.f32"), dtype="<f4").reshape(-1, cfg.vocab_size) for i in (0, 2, 3)}
        short = "f32" if dtype == "float32" else "bf16"
        close(np.concatenate([got[0], got[2], got[3]]), want[[0, 8, 20, 3]], short, f"trace replay in {dtype}")
    res = subprocess.run([sys.executable, "-m", "cake_b200.run", model_dir, "--prompt-ids", ",".join(map(str, toks[:6])), "-n", "5", "--dtype", "f32"],
                         capture_output=True, text=True, timeout=900, cwd=root)
    assert res.returncode == 0, res.stderr[-2000:]
    out = [int(t) for t in res.stdout.split("tokens:")[1].splitlines()[0].split()]
    assert len(out) == 5 and all(0 <= t < cfg.vocab_size for t in out)
