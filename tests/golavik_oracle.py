"""Plain, slow restatement of the Golavik decoder for the tests: one function per mechanism, whole sequences only (no
cache, no batching, no kernels), PyTorch on the CPU in whatever float dtype the weights come in (the tests use float64).
Nothing here is imported by the package and nothing of the package is imported here.

Notation: T tokens, C = width, H heads, D = per-head key size, E = per-head value size, R = latent size, P = rotated
size. Weights are a dict name -> tensor with linear weights stored [out, in]; `m` is a layer's `mixer` dictionary.
"""
import math

import torch


# ------------------------------------------------------------------------------------------------ elementwise pieces
def silu(z):
    return z * torch.sigmoid(z)


def unit(x, eps=1e-6):
    """x / sqrt(sum(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + eps)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def group_rms_norm(x, w, groups, eps):
    """The last axis is cut into `groups` equal consecutive parts; each is divided by its own root mean square."""
    T, C = x.shape
    return (rms(x.reshape(T, groups, C // groups), eps)).reshape(T, C) * w


def causal_conv(h, w):
    """h [T, C], w [C, taps] -> c with c_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before t = 0 (the last
    column multiplies the current token)."""
    T, C = h.shape
    taps = w.shape[1]
    c = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                c[t] += w[:, j] * h[s]
    return c


# ------------------------------------------------------------------------------------------------ rotation
def yarn_frequencies(dims, base, scaling, dtype=torch.float64):
    """Frequencies f_i (i < dims/2) after the YaRN blend, and the factor both cos and sin are multiplied with."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, freqs, mult):
    """x [T, ..., P]: pair (2i, 2i+1) of the first 2 * len(freqs) entries turned by positions * freqs[i]; cos and sin
    scaled by mult; further entries pass."""
    n = freqs.shape[0]
    ang = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = (torch.cos(ang) * mult).reshape(shape), (torch.sin(ang) * mult).reshape(shape)
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * c - v * s
    out[..., 1:2 * n:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def latent_attention(h, W, pfx, m, eps):
    """Attention whose keys and values are expanded from a shared low-rank latent; a rotated key part shared by the
    heads; sliding window; ordinary softmax; sigmoid output gate."""
    T = h.shape[0]
    H, D, P, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window = m["mask"]["size"]
    pos = torch.arange(T)
    freqs, mult = yarn_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = (h @ W[pfx + "q"].T).view(T, H, D + P)
    q_plain, q_rot = q[..., :D], rotate_interleaved(q[..., D:], pos, freqs, mult)
    dkv = h @ W[pfx + "dkv"].T
    c = rms(dkv[:, :R], eps) * W[pfx + "dkv.norm"]
    k_rot = rotate_interleaved(dkv[:, R:], pos, freqs, mult)
    k_plain = (c @ W[pfx + "uk"].T).view(T, H, D)
    v = (c @ W[pfx + "uv"].T).view(T, H, E)
    o = torch.zeros(T, H, E, dtype=h.dtype)
    for hd in range(H):
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k_plain[lo:i + 1, hd] @ q_plain[i, hd] + k_rot[lo:i + 1] @ q_rot[i, hd]) * m["scale"]
            o[i, hd] = torch.softmax(s, dim=0) @ v[lo:i + 1, hd]
    gate = torch.sigmoid(h @ W[pfx + "g"].T)
    return (o.reshape(T, H * E) * gate) @ W[pfx + "o"].T


def gated_delta_recurrence(q, k, v, beta, g):
    """q, k, g [T, H, D], v [T, H, E], beta [T, H]. Per head: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q."""
    T, H, D = q.shape
    E = v.shape[2]
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for hd in range(H):
        S = torch.zeros(D, E, dtype=q.dtype)
        for t in range(T):
            S = g[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, hd])
            S = S + torch.outer(k[t, hd], u)
            o[t, hd] = S.T @ q[t, hd]
    return o


def channel_delta(h, W, pfx, m, eps):
    T = h.shape[0]
    H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rep = H // G

    def branch(name):
        return silu(causal_conv(h @ W[pfx + name].T, W[pfx + name + ".conv"]))

    q = unit(branch("q").view(T, G, D)) * D ** -0.5
    k = unit(branch("k").view(T, G, D))
    v = branch("v").view(T, H, E)
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[pfx + "b"].T)
    a = (h @ W[pfx + "a1"].T) @ W[pfx + "a2"].T + W[pfx + "dt_bias"]
    rate = torch.exp(W[pfx + "A_log"])[None, :, None]
    g = torch.exp(-rate * torch.nn.functional.softplus(a).view(T, H, D))
    o = gated_delta_recurrence(q, k, v, beta, g)
    o = rms(o, eps) * W[pfx + "norm"]
    gate = torch.sigmoid((h @ W[pfx + "g1"].T) @ W[pfx + "g2"].T)
    return (o.reshape(T, H * E) * gate) @ W[pfx + "o"].T


def general_delta_recurrence(r, k, v, w, a):
    """All [T, H, D]. S_t = diag(w) S - (a * u)(u^T S) + k v^T with u the unit key, both terms on the old S; o = S^T r."""
    T, H, D = r.shape
    u = unit(k)
    o = torch.zeros(T, H, D, dtype=r.dtype)
    for hd in range(H):
        S = torch.zeros(D, D, dtype=r.dtype)
        for t in range(T):
            S = w[t, hd][:, None] * S - torch.outer(a[t, hd] * u[t, hd], S.T @ u[t, hd]) + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ r[t, hd]
    return o


def general_delta(h, W, pfx, m, eps):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ W[pfx + "r"].T).view(T, H, D)
    k = (h @ W[pfx + "k"].T).view(T, H, D)
    v = (h @ W[pfx + "v"].T).view(T, H, D)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[pfx + "w1"].T) @ W[pfx + "w2"].T + W[pfx + "w0"]))
    a = torch.sigmoid(h @ W[pfx + "a"].T + W[pfx + "a.b"])
    o = general_delta_recurrence(r, k, v, w.view(T, H, D), a.view(T, H, D))
    o = rms(o, eps).reshape(T, H * D) * W[pfx + "norm"]
    return (o * torch.sigmoid(h @ W[pfx + "g"].T)) @ W[pfx + "o"].T


MIXERS = {"latent_attention": latent_attention, "channel_delta": channel_delta, "general_delta": general_delta}


# ------------------------------------------------------------------------------------------------ feed-forward
def route(z, top, n_groups, keep, scale):
    """z [T, n] router logits -> (chosen [T, top] expert numbers, weights [T, top])."""
    s = torch.sigmoid(z)
    T, n = s.shape
    per = n // n_groups
    gs = s.view(T, n_groups, per).topk(min(2, per), dim=-1).values.sum(-1)
    best = gs.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed.repeat_interleave(per, dim=1), s, torch.full_like(s, -1.0))
    chosen = masked.topk(top, dim=-1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(-1, keepdim=True) + 1e-20) * scale


def moe(h, W, pfx, mlp):
    r = mlp["router"]
    chosen, w = route(h @ W[pfx + "router"].T, r["top"], r["groups"]["count"], r["groups"]["keep"], r["scale"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t].tolist(), w[t]):
            p = f"{pfx}e{e}."
            out[t] += we * ((silu(h[t] @ W[p + "gate"].T) * (h[t] @ W[p + "up"].T)) @ W[p + "down"].T)
    return out


# ------------------------------------------------------------------------------------------------ whole model
def layer_runs(cfg):
    """The order in which layers run: (layer, pass) with pass = None outside the loop; the first layer of each pass is
    marked."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


def forward(cfg, W, tokens, return_residuals=False):
    """tokens: list of ids of ONE sequence -> logits [T, vocab] (and the residual stream after every layer run)."""
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = W["embed"][torch.tensor(tokens)]
    res = []
    for i, t, first in layer_runs(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = x + W["loop.step"][t]
        h = group_rms_norm(x, W[p + "norm1"], groups, eps)
        y = MIXERS[L["type"]](h + causal_conv(h, W[p + "canon1"]), W, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            y = y + moe(h + causal_conv(h, W[p + "canon2"]), W, p + "mlp.", L["mlp"])
        x = x + y
        res.append(x)
    logits = group_rms_norm(x, W["final.norm"], groups, eps) @ W["embed"].T
    return (logits, res) if return_residuals else logits


# ------------------------------------------------------------------------------------------------ random checkpoints
def random_weights(cfg, seed=0, ranks=(5, 7, 6), dtype=torch.float64):
    """Random weights of a configuration, rounded to bfloat16 (what a checkpoint stores) and returned in `dtype`.
    ranks: bottleneck sizes of the decay and gate projections of channel_delta and of the decay of general_delta."""
    g = torch.Generator().manual_seed(seed)
    C, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(name, out, inp, scale=1.0):
        W[name] = torch.randn(out, inp, generator=g) * scale / math.sqrt(inp)

    def vec(name, n, mean=0.0, std=1.0):
        W[name] = mean + std * torch.randn(n, generator=g)

    W["embed"] = torch.randn(V, C, generator=g)
    vec("final.norm", C, 1.0, 0.1)
    if cfg.get("loop"):
        W["loop.step"] = torch.randn(cfg["loop"]["times"], C, generator=g) * 0.5
    taps = cfg["canon"]["taps"]
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", C, 1.0, 0.1)
        W[p + "canon1"] = torch.randn(C, taps, generator=g) * 0.3
        x = p + "mix."
        if L["type"] == "latent_attention":
            H, D, P, E, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(x + "q", H * (D + P), C, 2.0)
            mat(x + "dkv", R + P, C, 2.0)
            vec(x + "dkv.norm", R, 1.0, 0.1)
            mat(x + "uk", H * D, R, 2.0)
            mat(x + "uv", H * E, R)
            mat(x + "g", H * E, C)
            mat(x + "o", C, H * E)
        elif L["type"] == "channel_delta":
            H, G, D, E = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * E)):
                mat(x + n, rows, C, 2.0)
                W[x + n + ".conv"] = torch.randn(rows, m["conv"], generator=g) * 0.5
            mat(x + "b", H, C)
            W[x + "A_log"] = torch.rand(H, generator=g) * 2.0 - 2.0
            vec(x + "norm", E, 1.0, 0.1)
            mat(x + "a1", ranks[0], C)
            mat(x + "a2", H * D, ranks[0], 2.0)
            vec(x + "dt_bias", H * D, -1.0, 1.0)
            mat(x + "g1", ranks[1], C)
            mat(x + "g2", H * E, ranks[1], 2.0)
            mat(x + "o", C, H * E)
        else:
            H, D = m["heads"], m["dim"]
            for n in ("r", "k", "v", "a", "g"):
                mat(x + n, H * D, C, 1.5)
            vec(x + "a.b", H * D, 0.0, 0.5)
            mat(x + "w1", ranks[2], C)
            mat(x + "w2", H * D, ranks[2], 2.0)
            vec(x + "w0", H * D, -0.5, 1.0)
            vec(x + "norm", H * D, 1.0, 0.1)
            mat(x + "o", C, H * D)
        if L.get("mlp"):
            W[p + "canon2"] = torch.randn(C, taps, generator=g) * 0.3
            f, n = L["mlp"]["expert"]["ff"], L["mlp"]["router"]["experts"]
            mat(p + "mlp.router", n, C, 2.0)
            for e in range(n):
                mat(f"{p}mlp.e{e}.gate", f, C)
                mat(f"{p}mlp.e{e}.up", f, C)
                mat(f"{p}mlp.e{e}.down", C, f)
    return {k: v.to(torch.bfloat16).to(dtype) for k, v in W.items()}
