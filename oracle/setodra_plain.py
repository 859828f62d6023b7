"""Plain, slow restatement of the Setodra design in torch on the CPU: one function per mechanism, whole sequences only
(no cache, no carried state, no portions, which is the point: the framework's scheduled runs are compared with it).
Test infrastructure: nothing under cake_b200/ imports it and it imports nothing from there.

Notation: x [S, W] residual stream, h a normed copy, H heads.  The model is a plain dict ``cfg`` (the parsed config.json)
and a dict ``wt`` name -> tensor.  ``dt`` is the torch dtype the arithmetic runs in (float32, or float64 for a sharper bar)."""
import math

import torch


def lin(W, x):
    return x @ W.to(x.dtype).t()


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w.to(x.dtype)


def silu(z):
    return z * torch.sigmoid(z)


def rope_frequencies(rot, dt=torch.float64):
    """(f [dims/2], amplitude): f_i = base^(-2i/dims), optionally blended towards f_i / factor by a linear ramp over the
    pair index whose ends come from two wavelength bounds; the amplitude multiplies cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dt)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def pair_of(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, rot, pos0=0):
    """v [S, H, D]: the first rot.dims entries of every head are rotated pairwise (i with i + dims/2) by pos * f_i."""
    if not rot or not int(rot["dims"]):
        return v
    dims = int(rot["dims"])
    f, amp = rope_frequencies(rot, torch.float64)
    p = torch.arange(pos0, pos0 + v.shape[0], dtype=torch.float64)
    ang = p[:, None] * f[None, :]
    c, s = (torch.cos(ang) * amp).to(v.dtype)[:, None, :], (torch.sin(ang) * amp).to(v.dtype)[:, None, :]
    a, b = v[..., : dims // 2], v[..., dims // 2: dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], -1)


def latent_attention(h, wt, p, m, eps):
    """Keys and values are expanded from a shared low-rank latent; one rotated key part is shared by all heads."""
    S = h.shape[0]
    H, D, R, V, C = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = lin(wt[p + "mix.q"], h).view(S, H, D + R)
    dkv = lin(wt[p + "mix.dkv"], h)
    c = rms_norm(dkv[:, :C], wt[p + "mix.dkv.norm"], eps)
    kr = rotate(dkv[:, None, C:], m["rot"])                      # [S, 1, R]
    qr = rotate(q[..., D:].contiguous(), m["rot"])               # [S, H, R]
    kn = lin(wt[p + "mix.uk"], c).view(S, H, D)
    v = lin(wt[p + "mix.uv"], c).view(S, H, V)
    s = (torch.einsum("ihd,jhd->hij", q[..., :D], kn) + torch.einsum("ihr,jr->hij", qr, kr[:, 0])) * float(m["scale"])
    vis = torch.arange(S)[:, None] >= torch.arange(S)[None, :]
    s = s.masked_fill(~vis[None], float("-inf"))
    pr = torch.softmax(s, -1)
    o = torch.einsum("hij,jhv->ihv", pr, v).reshape(S, H * V)
    return lin(wt[p + "mix.o"], o)


def retention(h, wt, p, m, eps):
    """Linear attention with one fixed decay per head: S_t = g S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    S = h.shape[0]
    H, D, V = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate(lin(wt[p + "mix.q"], h).view(S, H, D), m["rot"])
    k = rotate(lin(wt[p + "mix.k"], h).view(S, H, D), m["rot"]) * D ** -0.5
    v = lin(wt[p + "mix.v"], h).view(S, H, V)
    g = torch.tensor([float(x) for x in m["decay"]], dtype=h.dtype)
    st = torch.zeros(H, D, V, dtype=h.dtype)
    o = torch.zeros(S, H, V, dtype=h.dtype)
    for t in range(S):
        st = g[:, None, None] * st + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", st, q[t])
    o = rms_unit(o, eps).reshape(S, H * V) * silu(lin(wt[p + "mix.g"], h))
    return lin(wt[p + "mix.o"], o)


def causal_conv(u, w, b):
    """u [S, C], w [C, taps] (last column multiplies the current token), zeros before the start."""
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    out = b.to(u.dtype)[None, :].expand(u.shape[0], -1).clone()
    for j in range(taps):
        out = out + pad[j: j + u.shape[0]] * w.to(u.dtype)[:, j][None, :]
    return out


def mamba2(h, wt, p, m, eps):
    """State-space layer: S_t = exp(-exp(A) dt_t) S_{t-1} + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; gate, grouped norm."""
    S = h.shape[0]
    H, V, N, G, NG = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["norm_groups"])
    inner = H * V
    u = lin(wt[p + "mix.in"], h)
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, wt[p + "mix.conv"], wt[p + "mix.conv.b"]))
    x = xbc[:, :inner].view(S, H, V)
    Bm = xbc[:, inner: inner + G * N].view(S, G, N)
    Cm = xbc[:, inner + G * N:].view(S, G, N)
    dt = torch.nn.functional.softplus(dt + wt[p + "mix.dt_bias"].to(h.dtype), threshold=1e9)
    a = torch.exp(-torch.exp(wt[p + "mix.A_log"].to(h.dtype))[None, :] * dt)      # [S, H]
    grp = torch.arange(H) // (H // G)
    st = torch.zeros(H, N, V, dtype=h.dtype)
    y = torch.zeros(S, H, V, dtype=h.dtype)
    for t in range(S):
        st = a[t][:, None, None] * st + dt[t][:, None, None] * Bm[t][grp][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", st, Cm[t][grp]) + wt[p + "mix.D"].to(h.dtype)[:, None] * x[t]
    y = y.reshape(S, inner) * silu(z)
    y = rms_unit(y.view(S, NG, inner // NG), eps).reshape(S, inner) * wt[p + "mix.norm"].to(h.dtype)
    return lin(wt[p + "mix.o"], y)


def gated_expert(h, wt, p):
    return lin(wt[p + "down"], silu(lin(wt[p + "gate"], h)) * lin(wt[p + "up"], h))


def route(h, wt, p, r):
    """-> (chosen [S, top], weights [S, top]).  The choice uses softmax scores plus a per-expert offset, the weights the
    scores themselves, renormalised over the chosen ones and scaled."""
    s = torch.softmax(lin(wt[p + "router"], h), -1)
    chosen = torch.topk(s + wt[p + "correction"].to(h.dtype), int(r["top"]), dim=-1).indices
    w = torch.gather(s, 1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])


def moe(h, wt, p, mlp):
    r = mlp["router"]
    E = int(r["experts"])
    chosen, w = route(h, wt, p + "mlp.", r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t].tolist(), w[t]):
            out[t] += we * (h[t] if e >= E else gated_expert(h[t: t + 1], wt, f"{p}mlp.e{e}.")[0])   # e >= E: identity expert
    if mlp.get("shared"):
        out = out + torch.sigmoid(lin(wt[p + "mlp.shared.sg"], h)) * gated_expert(h, wt, p + "mlp.shared.")
    return out


MIXERS = {"latent_attention": latent_attention, "retention": retention, "mamba2": mamba2}


def layer_runs(cfg):
    """[(layer index, pass number t or None)]: t is set on the first layer of every pass of the looped range."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None) for i in range(a)]
    for t in range(n):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, L)]


def forward(cfg, wt, tokens, dt=torch.float32, trace=None):
    """tokens [S] -> logits [S, vocab]; ``trace`` (a list) receives the residual stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = wt["embed"].to(dt)[torch.as_tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x = x0.clone()
    for i, t in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if t is not None:
            if t > 0:
                x = x + x0
            x = x + wt["loop.step"].to(dt)[t]
        x = x + MIXERS[L["type"]](rms_norm(x, wt[p + "norm1"], eps), wt, p, L["mixer"], eps)
        if L.get("mlp"):
            x = x + moe(rms_norm(x, wt[p + "norm2"], eps), wt, p, L["mlp"])
        if trace is not None:
            trace.append(x.clone())
    return lin(wt["head"], rms_norm(x, wt["final.norm"], eps))
