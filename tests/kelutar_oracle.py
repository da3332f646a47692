"""Plain, slow restatement of the Kelutar decoder for the tests: one function per mechanism, whole sequences only (no
cache, no batching, no kernels), PyTorch on the CPU in whatever float dtype the weights come in (the tests use float64).
Nothing here is imported by the package and nothing of the package is imported here.

Notation: T tokens, C = width, H query heads, G key heads, D = per-head query/key size, E = per-head value size.
Weights are a dict name -> tensor with linear weights stored [out, in].
"""
import math

import torch


def rms_norm(x, w, eps):
    """y = x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def short_conv_residual(h, w):
    """h [T, C], w [C, taps]  ->  h + c with c_t = sum_j w[:, j] * h_(t - taps + 1 + j), zeros before t = 0."""
    T, C = h.shape
    taps = w.shape[1]
    c = torch.zeros_like(h)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                c[t] += w[:, j] * h[s]
    return h + c


def sliding_softmax_attention(q, k, v, window, scale_per_head):
    """q [T, H, D], k [T, G, D], v [T, G, E]; query i sees keys j with 0 <= i - j < window; head h reads key head
    h // (H / G); score = q . k * scale_per_head[h]. Returns [T, H, E]."""
    T, H, D = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // rep
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale_per_head[h]
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h, W, pfx, m, eps):
    """The gated sliding-window attention mixer: per-head RMS norm of q and k, the values are the un-normed keys,
    per-head temperature, sigmoid output gate read from the mixer's input."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[pfx + "q"].T + W[pfx + "q.b"]).view(T, H, D)
    k = (h @ W[pfx + "k"].T + W[pfx + "k.b"]).view(T, G, D)
    v = k
    qn = rms_norm(q, W[pfx + "q.norm"], eps)
    kn = rms_norm(k, W[pfx + "k.norm"], eps)
    o = sliding_softmax_attention(qn, kn, v, m["mask"]["size"], m["scale"] * W[pfx + "temp"])
    gate = torch.sigmoid(h @ W[pfx + "g"].T)
    return (o.reshape(T, H * D) * gate) @ W[pfx + "o"].T


def gated_linear_recurrence(q, f, v, state=None):
    """q, f [T, H, D], v [T, H, E]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T (S is [D, E] per head), o_t = S_t^T q_t.
    Returns (o [T, H, E], final S [H, D, E])."""
    T, H, D = q.shape
    E = v.shape[2]
    S = torch.zeros(H, D, E, dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, E, dtype=q.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, q[t])
    return o, S


def hgrn2_mixer(h, W, pfx, m, eps):
    T = h.shape[0]
    H, D, E = m["heads"], m["dim"], m["vdim"]
    q = torch.nn.functional.silu(h @ W[pfx + "q"].T).view(T, H, D)
    v = (h @ W[pfx + "v"].T).view(T, H, E)
    low = W[pfx + "lower"]
    f = (low + (1 - low) * torch.sigmoid(h @ W[pfx + "f"].T + W[pfx + "f.b"])).view(T, H, D)
    o, _ = gated_linear_recurrence(q, f, v)
    o = rms_norm(o, W[pfx + "norm"], eps)
    return o.reshape(T, H * E) @ W[pfx + "o"].T


def relu2_ff(h, W, pfx):
    return (torch.relu(h @ W[pfx + "up"].T) ** 2) @ W[pfx + "down"].T


def forward(tokens, W, cfg, return_layers=False):
    """tokens: list of ints (one sequence from position 0) -> logits [T, vocab] (and the residual after every layer)."""
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    ids = torch.tensor(tokens, dtype=torch.long)
    x = W["embed"][ids] * cfg["embedding"]["scale"] + W["pos"][:T]
    per_layer = []
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = "l%d." % src
        h = short_conv_residual(x, W[p + "canon1"])
        if layer["type"] == "attention":
            y = attention_mixer(h, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "hgrn2":
            y = hgrn2_mixer(h, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            x = x + rms_norm(relu2_ff(x, W, p + "mlp."), W[p + "norm2"], eps)
        per_layer.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    if return_layers:
        return logits, torch.stack(per_layer)
    return logits


def random_weights(cfg, seed=0, dtype=torch.float64, std=None):
    """Random weights for a config dict (rounded through bfloat16 so that a bf16 run reads the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    C = cfg["width"]

    def mat(o, i, s=None):
        s = (1.0 / math.sqrt(i)) if s is None else s
        return (torch.randn(o, i, generator=g) * s).to(torch.bfloat16).to(dtype)

    def vec(n, mean=1.0, s=0.1):
        return (mean + torch.randn(n, generator=g) * s).to(torch.bfloat16).to(dtype)

    W = {"embed": mat(cfg["vocab"], C, 1.0 / math.sqrt(C)), "pos": mat(cfg["max_positions"], C, 0.5),
         "final.norm": vec(C), "head": mat(cfg["vocab"], C)}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p, m = "l%d." % i, layer["mixer"]
        W[p + "norm1"] = vec(C)
        W[p + "canon1"] = mat(C, cfg["canon"]["taps"], 0.3)
        H, D = m["heads"], m["dim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            W[p + "mix.q"], W[p + "mix.q.b"] = mat(H * D, C), vec(H * D, 0.0, 0.2)
            W[p + "mix.k"], W[p + "mix.k.b"] = mat(G * D, C), vec(G * D, 0.0, 0.2)
            W[p + "mix.q.norm"], W[p + "mix.k.norm"] = vec(D), vec(D)
            W[p + "mix.temp"] = vec(H, 1.0, 0.3)
            W[p + "mix.g"] = mat(H * D, C)
            W[p + "mix.o"] = mat(C, H * D)
        else:
            E = m["vdim"]
            W[p + "mix.q"], W[p + "mix.f"], W[p + "mix.v"] = mat(H * D, C), mat(H * D, C), mat(H * E, C)
            W[p + "mix.f.b"] = vec(H * D, 1.0, 1.0)
            W[p + "mix.lower"] = torch.rand(H * D, generator=g).mul(0.9).to(torch.bfloat16).to(dtype)
            W[p + "mix.norm"] = vec(E)
            W[p + "mix.o"] = mat(C, H * E)
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            W[p + "norm2"] = vec(C)
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(F, C), mat(C, F)
    return W
