"""Plain, slow restatement of the Nigenex design in fp32 torch on the CPU: one function per mechanism, whole sequences
only (no cache, no state, no chunks — which is the point: the framework's scheduled runs are compared with it).
Test infrastructure: nothing under cake_b200/ imports it and it imports nothing from there.

Notation: x [S, W] residual stream, h its normed copy, H query heads, G key/value heads, D head size, w window.
``mm`` chooses how matrix products round: "f32" (none) or "bf16" (operands and result rounded to bfloat16, fp32 sum)."""
import math

import torch


def linear(W, x, mm="f32"):
    if mm == "bf16":
        return (x.to(torch.bfloat16).float() @ W.float().t()).to(torch.bfloat16).float()
    return x @ W.float().t()


def rms_norm_scalar(x, g, eps):
    """x / sqrt(mean(x^2) + eps) * g with g a single number."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * float(g)


def token_shift(h, mu):
    """row t becomes h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu.float()


def soft_cap(s, cap):
    return cap * torch.tanh(s / cap) if cap > 0 else s


def distance_bias(S, r1, r2):
    """[H, S, S]: r1_h * ln(1 + r2_h * (i - j)) for j <= i (0 elsewhere; those entries are masked anyway)."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    d = (i - j).clamp(min=0).float()
    return r1.float()[:, None, None] * torch.log(1 + r2.float()[:, None, None] * d[None])


def window_mask(S, w):
    """[S, S] bool: entry (i, j) is set iff i - w < j <= i (w == 0: every j <= i)."""
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    vis = i - j >= 0
    if w > 0:
        vis = vis & (i - j < w)
    return vis


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def attention_mixer(hs, wt, sp, mm="f32"):
    """hs [S, W] (already shifted) -> [S, W].  The keys double as values; one sigmoid gate per head, computed from hs as well."""
    S = hs.shape[0]
    H, G, D = sp.heads, sp.kv_heads, sp.head_dim
    q = linear(wt["q"], hs, mm).view(S, H, D)
    k = linear(wt["k"], hs, mm).view(S, G, D).repeat_interleave(H // G, dim=1)
    s = soft_cap(torch.einsum("ihd,jhd->hij", q, k) * sp.scale, sp.softcap)
    s = s - distance_bias(S, wt["r1"], wt["r2"])
    s = s.masked_fill(~window_mask(S, sp.window)[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", p, k)
    gate = torch.sigmoid(linear(wt["g"], hs, mm))           # [S, H]
    return linear(wt["o"], (o * gate[:, :, None]).reshape(S, H * D), mm)


def feed_forward(h, wt, mm="f32"):
    return linear(wt["down"], gelu_tanh(linear(wt["gate"], h, mm)) * linear(wt["up"], h, mm), mm)


def layer(x, wt, sp, eps, mm="f32"):
    """Parallel block: one norm, mixer on the shifted copy, feed-forward on the plain one, both added to x."""
    h = rms_norm_scalar(x, wt["norm1"], eps)
    y = attention_mixer(token_shift(h, wt["shift"]), wt, sp, mm)
    if sp.ff:
        y = y + feed_forward(h, wt, mm)
    return x + y


def layer_weights(sd, name, sp):
    wt = {"norm1": sd[f"{name}.norm1"], "shift": sd[f"{name}.shift"]}
    for k in ("q", "k", "o", "g", "r1", "r2"):
        wt[k] = sd[f"{name}.mix.{k}"]
    if sp.ff:
        for k in ("gate", "up", "down"):
            wt[k] = sd[f"{name}.mlp.{k}"]
    return wt


def model_logits(cfg, sd, tokens, mm="f32", residuals=None):
    """tokens [S] -> logits [S, vocab] (fp32).  ``residuals``: a list that receives x after every layer."""
    x = sd["embed"].float()[torch.as_tensor(tokens, dtype=torch.long)]
    for i, sp in enumerate(cfg.layers):
        x = layer(x, layer_weights(sd, f"l{i}", sp), sp, cfg.rms_norm_eps, mm)
        if residuals is not None:
            residuals.append(x.clone())
    lg = linear(sd["head"], rms_norm_scalar(x, sd["final.norm"], cfg.rms_norm_eps), mm)
    return soft_cap(lg, cfg.logit_softcap)


def greedy(cfg, sd, prompt, n, mm="f32"):
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = int(model_logits(cfg, sd, toks, mm)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
