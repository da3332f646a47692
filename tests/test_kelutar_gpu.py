"""Kelutar on the GPU against the plain restatement in tests/kelutar_oracle.py (float64 on the CPU): every mechanism
alone through its op, then the whole model through the engine's step function, the slot cache, the scheduler and
generate(). Configurations are small and deliberately unlike each other: grouped key heads, head sizes that are not
multiples of 16 or 32, a vocabulary that is not a multiple of 8, windows of 1 to 9, 1 to 4 convolution taps, attention
first or last, feed-forwards on either kind of layer, layers that reuse weights."""
import math

import pytest
import torch

import kelutar_oracle as ko

pytestmark = pytest.mark.gpu
F32, F64, BF16 = torch.float32, torch.float64, torch.bfloat16


def _dev():
    return torch.device("cuda:0")


def _layout(lens, pos0, slots):
    from llark_b200.state_cache import StepLayout

    return StepLayout(lens, pos0, slots, _dev())


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def _logit_err(got, want):
    """Difference of logits as a serving check reads it: mean over the vocabulary taken off, rms, relative to the rms of
    the expected logits."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double().cpu()
    w = w - w.mean(dim=-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()).max().item()


# ------------------------------------------------------------------------------------------------ configurations
def _hg(heads, dim, vdim, mlp=None, weights_of=None):
    e = {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _at(heads, kv, dim, window, scale=None, mlp=None, weights_of=None):
    e = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim,
                                        "mask": {"size": window}, "scale": scale or 1.0 / math.sqrt(dim)}, "mlp": mlp}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


def _cfg(layers, vocab=97, width=72, taps=4, max_positions=256, scale=3.0, eps=1e-5):
    return {"architecture": "Kelutar", "vocab": vocab, "width": width, "max_positions": max_positions,
            "embedding": {"scale": scale}, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": layers}


FF = {"kind": "dense", "ff": 100}
CONFIGS = {
    # recurrence first, grouped key heads, odd vocabulary, 4 taps, reuse of both kinds of layer
    "mixed": _cfg([_hg(3, 20, 24), _at(4, 2, 24, 7, mlp=FF), _hg(3, 20, 24, weights_of=0),
                   _at(4, 2, 24, 7, mlp=FF, weights_of=1)]),
    # attention first, window 1 (sees itself only) and a wide one, no convolution (1 tap), ff on the recurrence
    "attn_first": _cfg([_at(2, 1, 40, 1), _hg(1, 36, 8, mlp={"kind": "dense", "ff": 64}), _at(6, 6, 16, 9)],
                       vocab=64, width=48, taps=1, scale=1.0, eps=1e-3),
    # head sizes the tensor-core attention takes (multiples of 16), a window wider than one key tile, three taps
    "tc_heads": _cfg([_at(4, 2, 32, 70, mlp=FF), _hg(2, 32, 48), _at(4, 2, 32, 70, mlp=FF, weights_of=0),
                      _at(2, 2, 64, 3)], vocab=120, width=64, taps=3),
    # nothing is a multiple of 4: every op takes its scalar route, the linears the tiled SIMT kernel
    "odd_sizes": _cfg([_hg(3, 10, 7), _at(3, 1, 10, 4, mlp={"kind": "dense", "ff": 21}), _hg(1, 5, 33)],
                      vocab=33, width=50, taps=3, max_positions=130),
    # two taps, one head, head sizes above 32 and 128
    "wide_heads": _cfg([_hg(2, 144, 40), _at(1, 1, 72, 5, scale=0.2, mlp=FF)], vocab=50, width=80, taps=2),
}


def _model(cfg, W, dtype):
    from llark_b200.models.kelutar import KelutarConfig, KelutarForCausalLM

    return KelutarForCausalLM(KelutarConfig.from_dict(cfg), W, device="cuda:0", dtype=dtype)


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("M,N,K", [(1, 50, 72), (3, 97, 100), (8, 64, 33), (23, 96, 72), (40, 97, 72), (130, 200, 64),
                                   (17, 24, 7), (20, 64, 16), (9, 8, 8), (300, 64, 64), (65, 72, 320),
                                   (3, 4800, 72), (1, 4737, 64), (8, 4739, 33)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_linear_every_route(M, N, K, dtype):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(M * 1000 + N)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(dtype)
    b = torch.randn(N, generator=g)
    want = a.double() @ w.double().T + b.double()
    for out_dtype in ((F32,) if dtype == F32 else (F32, BF16)):
        got = ops.linear(a.to(_dev()), w.to(_dev()), bias=b.to(_dev()), out_dtype=out_dtype)
        tol = 2e-6 if out_dtype == F32 and dtype == F32 else (1e-5 if out_dtype == F32 else 6e-3)
        assert _rel(got, want) < tol, (M, N, K, dtype, out_dtype)
    got = ops.linear(a.to(_dev()), w.to(_dev()), out_dtype=F32)
    assert _rel(got, a.double() @ w.double().T) < 1e-5


@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_short_conv_carries_its_inputs_across_steps(taps):
    from llark_b200 import ops

    C = 40
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(19 + 150, C, generator=g), torch.randn(11 + 70, C, generator=g)]
    want = [ko.short_conv_residual(s.double(), w.double()) for s in seqs]
    tail = torch.full((6, max(taps - 1, 1), C), 7.0, device=_dev())  # other slots hold other requests' inputs
    tail[[4, 1]] = 0.0  # what alloc() does for the two slots in use
    slots = [4, 1]
    # request 0 in portions 5, 1, 1, 2, 10; request 1 in portions 2, 1, 8 (it ends earlier)
    # ... then long portions (the row-blocked kernel: a request that starts in the middle of a block of rows)
    plan = [([5, 2], [0, 1]), ([1, 1], [0, 1]), ([1, 8], [0, 1]), ([2], [0]), ([10], [0]), ([97, 3], [0, 1]),
            ([53, 67], [0, 1])]
    at = [0, 0]
    got = [[], []]
    for lens, who in plan:
        st = _layout(lens, [at[b] for b in who], [slots[b] for b in who])
        h = torch.cat([seqs[b][at[b]:at[b] + n] for n, b in zip(lens, who)]).to(_dev())
        y = ops.seq_short_conv(h, w.to(_dev()), tail, st, F32)
        r = 0
        for n, b in zip(lens, who):
            got[b].append(y[r:r + n].cpu())
            r += n
            at[b] += n
    for b in range(2):
        assert _rel(torch.cat(got[b]), want[b]) < 1e-6


def _run_window_attention(q, k, v, window, scale_h, portions, act, cap=None):
    """q [T, H, D], k / v [T, G, D] through seq_swa_attn + the ring, cut into `portions`; slot 2 of a 4-slot ring."""
    from llark_b200 import ops

    T, H, D = q.shape
    G = k.shape[1]
    cap = cap or window
    kring = torch.full((4, cap, G * D), float("nan"), device=_dev(), dtype=act)
    vring = torch.full((4, cap, G * D), float("nan"), device=_dev(), dtype=act)
    sc = scale_h.to(_dev(), F32)
    outs, at = [], 0
    for n in portions:
        st = _layout([n], [at], [2])
        qq = q[at:at + n].reshape(n, H * D).to(_dev(), act).contiguous()
        kk = k[at:at + n].reshape(n, G * D).to(_dev(), act).contiguous()
        vv = v[at:at + n].reshape(n, G * D).to(_dev(), act).contiguous()
        if n == 1:  # the decode order: ring first, then attention over the ring alone
            ops.seq_kv_ring_write(kk, vv, kring, vring, st, cap)
            o = ops.seq_swa_attn(qq, None, None, kring, vring, None, 0, sc, st, H, G, D, D, window, cap, True)
        else:
            o = ops.seq_swa_attn(qq, kk, vv, kring, vring, None, 0, sc, st, H, G, D, D, window, cap, False)
            ops.seq_kv_ring_write(kk, vv, kring, vring, st, cap)
        outs.append(o.view(n, H, D).cpu())
        at += n
    assert at == T
    return torch.cat(outs)


@pytest.mark.parametrize("window", [1, 2, 5, 33, 70])
def test_window_attention_sees_exactly_its_window(window):
    """One key per query is made to dominate the softmax: the one at distance window - 1 (just inside) for even
    positions, the one at distance window (just outside) for odd ones. An edge that is one token off flips which
    value comes out."""
    T, H, G, D = 150, 4, 2, 24
    g = torch.Generator().manual_seed(window)
    q = torch.randn(T, H, D, generator=g) * 0.1
    k = torch.randn(T, G, D, generator=g) * 0.1
    v = torch.randn(T, G, D, generator=g)
    for i in range(T):
        j = i - (window - 1) if i % 2 == 0 else i - window
        if j >= 0:
            u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)  # this query's own direction
            q[i] += 6.0 * u
            k[j] += 6.0 * u
    scale_h = torch.tensor([1.0, 0.7, 1.3, 0.5])
    want = ko.sliding_softmax_attention(q.double(), k.double(), v.double(), window, scale_h.double())
    whole = _run_window_attention(q, k, v, window, scale_h, [T], F32)
    assert _rel(whole, want) < 2e-5
    # a prompt, then portions down to two tokens, then decoding across several turns of the ring
    cut = _run_window_attention(q, k, v, window, scale_h, [37, 2, 3, 2, 16] + [1] * 90, F32)
    assert _rel(cut, want) < 2e-5
    assert (cut - whole).abs().max() < 1e-4
    bf = _run_window_attention(q, k, v, window, scale_h, [60] + [1] * 90, BF16)
    q16, k16, v16 = (t.to(BF16).double() for t in (q, k, v))
    assert _rel(bf, ko.sliding_softmax_attention(q16, k16, v16, window, scale_h.double())) < 1e-2


@pytest.mark.parametrize("D,window", [(16, 1), (48, 5), (32, 64), (64, 65), (128, 100), (80, 31), (192, 70)])
def test_window_attention_on_the_tensor_core_path(D, window):
    """Prompts and portions of 16 tokens or more take the 64-query tensor-core kernel: same needles at the window's edge,
    tiles that start before position 0, queries whose window misses a whole key tile, keys from the ring and from the
    step, grouped key heads."""
    T, H, G = 230, 4, 2
    g = torch.Generator().manual_seed(D + window)
    q = torch.randn(T, H, D, generator=g) * 0.1
    k = torch.randn(T, G, D, generator=g) * 0.1
    v = torch.randn(T, G, D, generator=g)
    for i in range(T):
        j = i - (window - 1) if i % 2 == 0 else i - window
        if j >= 0:
            u = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
            q[i] += 5.0 * u
            k[j] += 5.0 * u
    scale_h = torch.tensor([1.0, 0.7, 1.3, 0.5])
    q16, k16, v16 = (t.to(BF16).double() for t in (q, k, v))
    want = ko.sliding_softmax_attention(q16, k16, v16, window, scale_h.double())
    for portions in ([T], [130, 40, 17, 1, 1, 41], [16, 16, 64, 70, 64]):
        got = _run_window_attention(q, k, v, window, scale_h, portions, BF16)
        assert _rel(got, want) < 1e-2, portions


def test_qk_headnorm_and_gate_through_the_mixer():
    from llark_b200.mixers import GatedWindowAttention
    from llark_b200.state_cache import StateCache

    spec = {"heads": 6, "kv_heads": 3, "dim": 20, "vdim": 20, "mask": {"size": 6}, "scale": 0.3}
    cfg = _cfg([{"type": "attention", "mixer": spec, "mlp": None}], width=56)
    W = ko.random_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(31, 56, generator=g).to(BF16).double()
    want = ko.attention_mixer(h, W, "l0.mix.", spec, 1e-5)
    for act, tol in ((F32, 2e-5), (BF16, 2e-2)):
        cache = StateCache(_dev())
        mx = GatedWindowAttention(GatedWindowAttention.Weights(W, "l0.mix.", spec, 56, _dev(), act), cache, 1e-5, act, 256)
        slot = cache.alloc()
        outs = []
        for lo, n in ((0, 13), (13, 2), (15, 1), (16, 1), (17, 14)):
            st = cache.layout([slot], [n])
            outs.append(mx.forward(h[lo:lo + n].to(_dev(), act), st, cache).cpu())
            cache.advance([slot], [n])
        assert _rel(torch.cat(outs), want) < tol


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("H,D,E", [(3, 20, 24), (1, 144, 40), (2, 16, 130), (5, 48, 64)])
def test_gated_recurrence_remembers_far_tokens(H, D, E, chunked, monkeypatch):
    """Every seventh channel forgets almost nothing (gate ~ 1) except at step 3, where its gate opens and a large value
    is written; 300 steps later that value still carries the output, so a lost or re-zeroed state shows. The steps are
    cut into a prompt, portions and single tokens; a second request shares the batch and ends early."""
    from llark_b200 import ops

    if chunked:  # the three-pass form: chunks of 16 rows (the last one partial) for every portion of 32 rows or more
        monkeypatch.setattr(ops, "GLR_CHUNK", 16)
        monkeypatch.setattr(ops, "GLR_CHUNK_MIN_LEN", 32)
    T = 330
    g = torch.Generator().manual_seed(H * D + E)
    ld = 2 * H * D + H * E + 3  # a padded row, as a fused projection may have
    src = torch.randn(2, T, ld, generator=g)
    lower = torch.rand(H * D, generator=g) * 0.5
    lower[::7] = 0.0
    src[:, :, H * D:2 * H * D][:, :, ::7] = 12.0   # f_pre: the gate stays ~ 1 (keep, write nothing) ...
    src[:, 3, H * D:2 * H * D][:, ::7] = -12.0     # ... but opens at step 3
    src[:, 3, 2 * H * D:2 * H * D + H * E] *= 50.0
    want = []
    for b in range(2):
        s = src[b].double()
        q = torch.nn.functional.silu(s[:, :H * D]).view(T, H, D)
        low = lower.double()
        f = (low + (1 - low) * torch.sigmoid(s[:, H * D:2 * H * D])).view(T, H, D)
        v = s[:, 2 * H * D:2 * H * D + H * E].view(T, H, E)
        want.append(ko.gated_linear_recurrence(q, f, v)[0].reshape(T, H * E))
        if b == 0:  # what a state lost at step 200 would give at step 320: far from the truth
            lost = ko.gated_linear_recurrence(q[200:], f[200:], v[200:])[0].reshape(T - 200, H * E)
            assert (lost[120] - want[0][320]).abs().max() > 0.5
    state = torch.full((5, H, D, E), 3.0, device=_dev())
    state[[3, 0]] = 0.0  # what alloc() does for the two slots in use; the others hold another request's leftovers
    slots = [3, 0]
    plan = [([200, 17], [0, 1]), ([2, 1], [0, 1]), ([1, 1], [0, 1]), ([1, 40], [0, 1]), ([50], [0]), ([1], [0])] + \
           [([1], [0])] * 20 + [([55], [0])]
    at = [0, 0]
    got = [[], []]
    for lens, who in plan:
        st = _layout(lens, [at[b] for b in who], [slots[b] for b in who])
        rows = torch.cat([src[b, at[b]:at[b] + n] for n, b in zip(lens, who)]).to(_dev())
        o = ops.seq_glr_scan(rows, 0, H * D, 2 * H * D, lower.to(_dev()), state, st, H, D, E)
        r = 0
        for n, b in zip(lens, who):
            got[b].append(o[r:r + n].cpu())
            r += n
            at[b] += n
    assert at[0] == T
    assert _rel(torch.cat(got[0]), want[0]) < 2e-5
    assert _rel(torch.cat(got[1]), want[1][:at[1]]) < 2e-5
    assert (state[[1, 2, 4]] == 3.0).all()


def test_norms_and_relu2():
    from llark_b200 import ops

    g = torch.Generator().manual_seed(0)
    x, y, w = torch.randn(9, 70, generator=g), torch.randn(9, 70, generator=g) * 3, torch.randn(70, generator=g)
    want = x.double() + ko.rms_norm(y.double(), w.double(), 1e-3)
    out, xa = ops.seq_add_rmsnorm(x.to(_dev()), y.to(_dev()), w.to(_dev()), 1e-3, act=BF16)
    assert _rel(out, want) < 1e-6 and _rel(xa, want) < 4e-3
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    got = ops.seq_rmsnorm_rows(x.to(_dev()), rows.to(_dev()), w.to(_dev()), 1e-3, F32)
    assert _rel(got, ko.rms_norm(x.double()[rows.long()], w.double(), 1e-3)) < 1e-6
    o = torch.randn(5, 3 * 24, generator=g)
    wn = torch.randn(24, generator=g)
    got = ops.seq_head_rmsnorm(o.to(_dev()), wn.to(_dev()), 24, 1e-5, F32)
    assert _rel(got, ko.rms_norm(o.double().view(5, 3, 24), wn.double(), 1e-5).reshape(5, 72)) < 1e-6
    u = torch.randn(1000, generator=g)
    assert _rel(ops.seq_relu2(u.to(_dev())), torch.relu(u.double()) ** 2) < 1e-6


# ------------------------------------------------------------------------------------------------ the whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_matches_the_restatement(name):
    cfg = CONFIGS[name]
    W = ko.random_weights(cfg, seed=11)
    toks = _tokens(61, cfg["vocab"], 1)
    want, want_layers = ko.forward(toks, W, cfg, return_layers=True)
    m = _model(cfg, W, F32)
    cache = m.new_cache()
    s = cache.alloc()
    logits, res = m.engine.step(cache, [s], [toks], want=[list(range(61))], return_residuals=True)
    for i, r in enumerate(res):
        assert _rel(r, want_layers[i]) < 2e-5, f"residual after layer {i}"
    assert _logit_err(logits, want) < 5e-5
    m16 = _model(cfg, W, BF16)
    c16 = m16.new_cache()
    got16 = m16.engine.step(c16, [c16.alloc()], [toks], want=[list(range(61))])
    assert _logit_err(got16, want) < 6e-2


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_portions_and_decoding_agree(name, dtype):
    """The same 90 tokens: in one step; as a prompt and then token by token (long decoding, several turns of every
    ring); in portions of 7, 2, 2, 30, 1, 1, 2, ... Every position's logits must agree beyond rounding."""
    cfg = CONFIGS[name]
    W = ko.random_weights(cfg, seed=3)
    toks = _tokens(90, cfg["vocab"], 2)
    m = _model(cfg, W, dtype)
    want = ko.forward(toks, W, cfg)

    def run(portions):
        cache = m.new_cache()
        s = cache.alloc()
        out, at = [], 0
        for n in portions:
            out.append(m.engine.step(cache, [s], [toks[at:at + n]], want=[list(range(n))]))
            at += n
        assert at == 90 and cache.length[s] == 90
        return torch.cat(out)

    tol = 5e-5 if dtype == F32 else 6e-2
    whole = run([90])
    assert _logit_err(whole, want) < tol
    for portions in ([30] + [1] * 60, [1] * 90, [7, 2, 2, 30, 1, 1, 2, 3, 2, 40]):
        got = run(portions)
        assert _logit_err(got, want) < tol
        assert _logit_err(got, whole) < (2e-5 if dtype == F32 else 4e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_unequal_batch_equals_each_request_alone_and_slots_are_reused(dtype):
    cfg = CONFIGS["mixed"]
    W = ko.random_weights(cfg, seed=4)
    m = _model(cfg, W, dtype)
    prompts = [_tokens(n, cfg["vocab"], 10 + n) for n in (1, 33, 5, 70, 12)]
    tails = [_tokens(6, cfg["vocab"], 50 + i) for i in range(5)]
    stop_after = [2, 6, 1, 4, 6]  # decode steps each request takes part in

    def alone(cache, i):
        s = cache.alloc()
        out = [m.engine.step(cache, [s], [prompts[i]], want=[list(range(len(prompts[i])))])]
        for k in range(stop_after[i]):
            out.append(m.engine.step(cache, [s], [[tails[i][k]]]))
        cache.release(s)
        return torch.cat(out)

    cache = m.new_cache(n_slots=2)  # five requests: the stores have to grow while two are live
    ref = [alone(cache, i) for i in range(5)]  # one after the other: the same slot again and again
    assert cache.allocs == 5 and cache.n_slots == 2 and not cache.in_use()
    # now together, in slots that hold the leftovers of the runs above
    slots = [cache.alloc() for _ in range(5)]
    assert cache.n_slots >= 5
    got = [[] for _ in range(5)]
    lg = m.engine.step(cache, slots, prompts, want=[list(range(len(p))) for p in prompts])
    r = 0
    for i, p in enumerate(prompts):
        got[i].append(lg[r:r + len(p)])
        r += len(p)
    live = list(range(5))
    for k in range(6):
        live = [i for i in live if stop_after[i] > k]
        lg = m.engine.step(cache, [slots[i] for i in live], [[tails[i][k]] for i in live])
        for j, i in enumerate(live):
            got[i].append(lg[j:j + 1])
        for i in list(live):
            if stop_after[i] == k + 1:
                cache.release(slots[i])
    for i in range(5):
        assert _logit_err(torch.cat(got[i]), ref[i]) < (2e-5 if dtype == F32 else 4e-2), i
    want0 = ko.forward(prompts[3] + tails[3][:4], W, cfg)
    assert _logit_err(ref[3], want0) < (5e-5 if dtype == F32 else 6e-2)
    assert not cache.in_use()


def test_first_tokens_of_a_sequence():
    """Position 0 alone, and every prompt length up to a little beyond the widest window and the taps."""
    cfg = CONFIGS["mixed"]
    W = ko.random_weights(cfg, seed=6)
    m = _model(cfg, W, F32)
    toks = _tokens(12, cfg["vocab"], 6)
    want = ko.forward(toks, W, cfg)
    cache = m.new_cache()
    for n in range(1, 13):
        s = cache.alloc()
        got = m.engine.step(cache, [s], [toks[:n]], want=[list(range(n))])
        assert _logit_err(got, want[:n]) < 5e-5, n
        cache.release(s)


def test_checkpoint_folder_registry_and_greedy_generation(tmp_path):
    """config.json + model.safetensors -> the registry picks the class; generate() and the scheduler reproduce the
    restatement's greedy continuation (fp32, so that the argmax is the restatement's)."""
    import json

    from llark_b200.models.registry import load_model
    from llark_b200.safetensors_io import save_file
    from llark_b200.scheduler import BatchScheduler, Request

    cfg = CONFIGS["mixed"]
    W = ko.random_weights(cfg, seed=8)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    m = load_model(str(tmp_path), dtype=F32)

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(ko.forward(seq, W, cfg)[-1].argmax()))
        return seq

    prompts = [_tokens(9, cfg["vocab"], 1), _tokens(9, cfg["vocab"], 2)]
    want = [oracle_greedy(p, 12) for p in prompts]
    out = m.generate(input_ids=torch.tensor(prompts, device="cuda:0"), max_new_tokens=12)
    assert out.tolist() == want
    # unequal prompts and budgets through the scheduler; an eos id ends one request early
    reqs = [Request(prompt=prompts[0], max_new_tokens=12), Request(prompt=prompts[1][:4], max_new_tokens=5),
            Request(prompt=prompts[1], max_new_tokens=12, eos_token_id=[want[1][9 + 3]])]
    sched = BatchScheduler(m.engine, max_batch=2)
    for r in reqs:
        sched.submit(r)
    sched.run()
    assert reqs[0].output == want[0][9:]
    assert reqs[1].output == oracle_greedy(prompts[1][:4], 5)[4:]
    first_eos = want[1][9:].index(want[1][9 + 3])
    assert reqs[2].output == want[1][9:9 + first_eos + 1]
    assert all(r.finished for r in reqs) and not sched.cache.in_use()


def test_command_line_and_trace_runner(tmp_path, monkeypatch, capsys):
    """The two command-line entries on a checkpoint folder: generate_cli (scheduler, greedy) and the trace runner (given
    tokens step by step: two requests start together with unequal prompts, decode together, one ends earlier, a third
    starts later in the slot that was given back)."""
    import io
    import json

    import numpy as np

    from llark_b200 import generate_cli, trace_runner
    from llark_b200.safetensors_io import save_file

    cfg = CONFIGS["tc_heads"]
    W = ko.random_weights(cfg, seed=9)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    V = cfg["vocab"]
    a, b, c = _tokens(40, V, 1), _tokens(9, V, 2), _tokens(21, V, 3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]},
                                     {"id": "b", "tokens": b[:5], "want": []}], "end": []}]
    for k in range(4):
        steps.append({"step": 1 + k, "entries": [{"id": "a", "tokens": [a[30 + k]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + k]], "want": [0]}],
                      "end": ["b"] if k == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [20]},
                                         ], "end": ["c"]})
    steps.append({"step": 6, "entries": [{"id": "a", "tokens": a[34:], "want": [5]}], "end": ["a"]})
    out = tmp_path / "out"
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "80"]) == 0
    printed = capsys.readouterr().out.split("\n")
    assert [l for l in printed if l.startswith("done")] == ["done %d" % i for i in range(7)]
    la, lb, lc = ko.forward(a, W, cfg), ko.forward(b, W, cfg), ko.forward(c, W, cfg)

    def rows(i):
        return torch.from_numpy(np.fromfile(out / ("%d.f32" % i), dtype="<f4").reshape(-1, V).copy())

    assert _logit_err(rows(0), la[[0, 29]]) < 5e-5
    for k in range(4):
        assert _logit_err(rows(1 + k), torch.stack([la[30 + k], lb[5 + k]])) < 5e-5
    assert _logit_err(rows(5), lc[[20]]) < 5e-5
    assert _logit_err(rows(6), la[[39]]) < 5e-5

    prompts = tmp_path / "p.jsonl"
    prompts.write_text(json.dumps({"id": "x", "tokens": a[:7], "max_new_tokens": 6}) + "\n" +
                       json.dumps({"tokens": b[:3]}) + "\n")
    assert generate_cli.main(["--model", str(tmp_path), "--prompts", str(prompts), "--dtype", "float32",
                              "--max-new-tokens", "4"]) == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.strip().split("\n")]

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(ko.forward(seq, W, cfg)[-1].argmax()))
        return seq[len(prompt):]

    assert lines == [{"id": "x", "tokens": oracle_greedy(a[:7], 6)}, {"id": "1", "tokens": oracle_greedy(b[:3], 4)}]
