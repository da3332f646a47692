"""Golavik on the GPU against the plain restatement in tests/golavik_oracle.py (float64 on the CPU): every mechanism
alone through its ops or its mixer class, then the whole model through the engine's step function, the slot cache, the
scheduler and generate(). Configurations are small and deliberately unlike each other: key heads shared by several heads,
key / value / latent / rotated sizes that all differ, partial rotation with and without the frequency blend, 1 to 4
convolution taps, 1 to 4 norm groups, routers with one group or several, a loop over a part of the layers, layers without
a feed-forward, every mixer first or last."""
import math

import pytest
import torch

import golavik_oracle as go

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


def _logit_err(got, want, worst=1.0):
    """Difference of logits with the mean over the vocabulary taken off, rms, relative to the rms of the expected ones:
    the largest over the positions, or (worst < 1) the value that this share of the positions stays under. The bfloat16
    comparisons allow a tenth of the positions to be off: a router whose two best scores nearly tie may pick the other
    expert once its input is rounded, which the 32-bit comparisons (every position) do not suffer from."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(dim=-1, keepdim=True)
    w = want.double().cpu()
    w = w - w.mean(dim=-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()
    return e.max().item() if worst >= 1.0 else torch.quantile(e, worst).item()


def _share(dtype):
    return 1.0 if dtype == F32 else 0.9


# ------------------------------------------------------------------------------------------------ configurations
def _moe(experts, top, groups, keep, ff, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}


def _la(heads, dim, rot_dim, vdim, rank, window, rot_dims=None, scaling=None, base=10000.0, scale=None, mlp=None):
    rot = {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": scale or 1.0 / math.sqrt(dim + rot_dim), "mask": {"size": window}, "rot": rot}}


def _cd(heads, kv, dim, vdim, conv, mlp=None):
    return {"type": "channel_delta", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}


def _gd(heads, dim, mlp=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def _cfg(layers, vocab=97, width=72, taps=3, groups=2, eps=1e-5, loop=None):
    return {"architecture": "Golavik", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "canon": {"taps": taps}, "loop": loop, "layers": layers}


YARN = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}
CONFIGS = {
    # every size differs from every other; key heads shared by two heads; a loop over the middle two layers run three
    # times; router with three groups of which two are kept; the last layer has no feed-forward
    "mixed": _cfg([_gd(2, 12, mlp=_moe(6, 3, 3, 2, 20, 2.0)), _la(3, 10, 6, 14, 20, 5, rot_dims=4, mlp=_moe(4, 1, 1, 1, 9)),
                   _cd(4, 2, 8, 12, 3, mlp=_moe(6, 2, 2, 1, 16, 0.5)), _cd(2, 2, 20, 6, 2)],
                  loop={"start": 1, "stop": 3, "times": 3}),
    # attention first and last, window 1 (a token sees itself only) and a window wider than a key tile, frequency blend,
    # one tap (no convolution), one norm group, no loop, head sizes the tensor-core attention takes (latent + rotated
    # part a multiple of 16)
    "attn_ends": _cfg([_la(2, 16, 8, 16, 24, 1, scaling=YARN, mlp=_moe(8, 4, 4, 2, 12)), _gd(1, 36),
                       _la(4, 8, 16, 24, 48, 70, scaling=YARN, base=500.0, mlp=_moe(3, 3, 1, 1, 30, 1.5))],
                      vocab=64, width=48, taps=1, groups=1, eps=1e-3),
    # nothing is a multiple of 4: scalar routes everywhere; four taps; three norm groups; the whole model is one loop
    "odd_sizes": _cfg([_cd(3, 1, 10, 7, 4, mlp=_moe(5, 2, 5, 3, 11)), _la(3, 6, 2, 5, 9, 4, mlp=None), _gd(3, 10)],
                      vocab=33, width=51, taps=4, groups=3, loop={"start": 0, "stop": 3, "times": 2}),
    # wide heads (state rows split over several lanes), two taps, a loop of one pass
    "wide_heads": _cfg([_cd(2, 1, 144, 40, 2), _gd(1, 72, mlp=_moe(4, 2, 2, 2, 24)),
                        _la(1, 40, 24, 72, 40, 9, rot_dims=24, scaling=YARN)],
                       vocab=50, width=80, taps=2, groups=4, loop={"start": 2, "stop": 3, "times": 1}),
}


def _model(cfg, W, dtype):
    from llark_b200.models.golavik import GolavikConfig, GolavikForCausalLM

    return GolavikForCausalLM(GolavikConfig.from_dict(cfg), W, device="cuda:0", dtype=dtype)


def _tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


class _Stores:
    """Stand-in cache for a mixer used alone: slot stores filled with garbage except where alloc() would zero them."""

    def __init__(self, n_slots=4):
        self.t, self.n = [], n_slots

    def add_store(self, shape, dtype, zero_on_alloc):
        fill = 0.0 if zero_on_alloc else float("nan")
        self.t.append(torch.full((self.n,) + tuple(shape), fill, device=_dev(), dtype=dtype))
        return len(self.t) - 1

    def view(self, h):
        return self.t[h]


def _run_mixer(cls, W, spec, width, h, portions, act, eps=1e-5, slot=2):
    """h [T, width] through mixer `cls` cut into `portions` (one request in `slot`)."""
    weights = cls.Weights({k: v.to(F32) for k, v in W.items()}, "m.", spec, width, _dev(), act)
    stores = _Stores()
    mixer = cls(weights, stores, eps, act, None)
    outs, at = [], 0
    for n in portions:
        st = _layout([n], [at], [slot])
        outs.append(mixer.forward(h[at:at + n].to(_dev(), act).contiguous(), st, stores).cpu())
        at += n
    assert at == h.shape[0]
    return torch.cat(outs)


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("groups,C", [(1, 40), (2, 72), (3, 51), (4, 1024), (1, 4100), (2, 4096)])
def test_group_norm(groups, C):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(C)
    x, w, add = torch.randn(9, C, generator=g) * 3, torch.randn(C, generator=g), torch.randn(C, generator=g)
    x[:, : C // groups] *= 50.0  # a part that would swamp a norm taken over the whole row
    got = ops.seq_group_rmsnorm(x.to(_dev()), w.to(_dev()), groups, 1e-5)
    assert _rel(got, go.group_rms_norm(x.double(), w.double(), groups, 1e-5)) < 1e-6
    x2, got2 = ops.seq_group_rmsnorm(x.to(_dev()), w.to(_dev()), groups, 1e-5, add_vec=add.to(_dev()))
    assert _rel(x2, x.double() + add.double()) < 1e-7
    assert _rel(got2, go.group_rms_norm(x.double() + add.double(), w.double(), groups, 1e-5)) < 1e-6
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    got3 = ops.seq_group_rmsnorm(x.to(_dev()), w.to(_dev()), groups, 1e-5, out_dtype=BF16, rows=rows.to(_dev()))
    assert _rel(got3, go.group_rms_norm(x.double(), w.double(), groups, 1e-5)[rows.long()]) < 5e-3


@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_conv_act_carries_its_inputs_across_steps(taps):
    from llark_b200 import ops

    C, extra = 37, 5  # the channels are a column slice of a wider matrix
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(60 + 130, C + extra, generator=g), torch.randn(31 + 75, C + extra, generator=g)]
    want = [go.silu(go.causal_conv(s[:, 2:2 + C].double(), w.double())) for s in seqs]
    carry = torch.full((6, max(taps - 1, 1), C), 7.0, device=_dev())
    carry[[4, 1]] = 0.0
    slots = [4, 1]
    # short portions and single tokens (row-per-block kernel), then long ones (the kernel that walks runs of rows: a
    # request that starts in the middle of a run)
    plan = [([5, 2], [0, 1]), ([1, 1], [0, 1]), ([1, 8], [0, 1]), ([2], [0]), ([10, 20], [0, 1]), ([1], [0]), ([40], [0]),
            ([97, 3], [0, 1]), ([33, 72], [0, 1])]
    at, got = [0, 0], [[], []]
    for lens, who in plan:
        st = _layout(lens, [at[b] for b in who], [slots[b] for b in who])
        src = torch.cat([seqs[b][at[b]:at[b] + n] for n, b in zip(lens, who)]).to(_dev())
        y = ops.seq_conv_act(src[:, 2:2 + C], w.to(_dev()), carry, st, silu=True)
        r = 0
        for n, b in zip(lens, who):
            got[b].append(y[r:r + n].cpu())
            r += n
            at[b] += n
    for b in range(2):
        assert _rel(torch.cat(got[b]), want[b]) < 1e-6
    assert (carry[0] == 7.0).all()


def _scan(rule, q, k, v, dec, mix, H, G, D, E, portions, dec_bias=None, rate_log=None, slot=1):
    from llark_b200 import ops

    state = torch.full((3, H, D, E), float("nan"), device=_dev())
    state[slot] = 0.0
    outs, at = [], 0
    for n in portions:
        st = _layout([n], [at], [slot])
        sl = slice(at, at + n)
        vec = ops.seq_delta_prep(rule, q[sl].to(_dev()).contiguous(), k[sl].to(_dev()).contiguous(),
                                 dec[sl].to(_dev()).contiguous(), mix[sl].to(_dev()).contiguous(), H, G, D,
                                 dec_bias=dec_bias.to(_dev()) if dec_bias is not None else None,
                                 rate_log=rate_log.to(_dev()) if rate_log is not None else None)
        outs.append(ops.seq_delta_scan(vec, v[sl].to(_dev()).contiguous(), state, st, H, D, E).cpu())
        at += n
    return torch.cat(outs), state[slot].cpu()


@pytest.mark.parametrize("H,G,D,E", [(4, 2, 8, 12), (3, 1, 10, 7), (2, 2, 64, 64), (1, 1, 144, 40), (2, 1, 256, 16),
                                     (1, 1, 400, 3), (1, 1, 640, 9)])
def test_gated_delta_scan(H, G, D, E):
    from llark_b200 import ops

    T = 75
    g = torch.Generator().manual_seed(D)
    q, k = torch.randn(T, G * D, generator=g), torch.randn(T, G * D, generator=g)
    v = torch.randn(T, H * E, generator=g)
    dec, mix = torch.randn(T, H * D, generator=g), torch.randn(T, H, generator=g)
    dt, a_log = torch.randn(H * D, generator=g) - 1.0, torch.rand(H, generator=g) * 2 - 2
    rep = H // G
    qd = (go.unit(q.double().view(T, G, D)) * D ** -0.5).repeat_interleave(rep, 1)
    kd = go.unit(k.double().view(T, G, D)).repeat_interleave(rep, 1)
    gd = torch.exp(-torch.exp(a_log.double())[None, :, None] *
                   torch.nn.functional.softplus(dec.double() + dt.double()).view(T, H, D))
    want = go.gated_delta_recurrence(qd, kd, v.double().view(T, H, E), torch.sigmoid(mix.double()), gd).reshape(T, H * E)
    for portions in ([T], [40, 2, 3] + [1] * 30, [1] * T, [9, 8, 7, 51]):
        got, _ = _scan(ops.DELTA_GATED, q, k, v, dec, mix, H, G, D, E, portions, dec_bias=dt, rate_log=a_log)
        assert _rel(got, want) < 2e-5, portions


@pytest.mark.parametrize("H,D", [(2, 12), (3, 10), (1, 72), (2, 128)])
def test_generalized_delta_scan(H, D):
    from llark_b200 import ops

    T = 75
    g = torch.Generator().manual_seed(D + 1)
    r, k, v = (torch.randn(T, H * D, generator=g) for _ in range(3))
    dec, mix = torch.randn(T, H * D, generator=g), torch.randn(T, H * D, generator=g)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(dec.double())).view(T, H, D)
    a = torch.sigmoid(mix.double()).view(T, H, D)
    want = go.general_delta_recurrence(r.double().view(T, H, D), k.double().view(T, H, D), v.double().view(T, H, D), w,
                                       a).reshape(T, H * D)
    for portions in ([T], [40, 2, 3] + [1] * 30, [1] * T):
        got, _ = _scan(ops.DELTA_GENERALIZED, r, k, v, dec, mix, H, H, D, D, portions)
        assert _rel(got, want) < 2e-5, portions


@pytest.mark.parametrize("portions", [[400], [250] + [1] * 150, [100, 2, 298]])
def test_delta_state_keeps_a_value_for_hundreds_of_steps(portions):
    """A value is written once with a key no later token uses, under a decay close to one; 390 steps later a query along
    that key must read it back among the hundreds of other writes. A state that is lost, reset or decayed per head
    instead of per channel shows as a wrong read-out."""
    from llark_b200 import ops

    T, H, D, E = 400, 2, 16, 8
    g = torch.Generator().manual_seed(5)
    k = torch.randn(T, H * D, generator=g)
    k.view(T, H, D)[:, :, 0] = 0.0           # channel 0 belongs to the needle
    k.view(T, H, D)[5, :, :] = 0.0
    k.view(T, H, D)[5, :, 0] = 3.0
    q = torch.randn(T, H * D, generator=g) * 0.01
    q.view(T, H, D)[395, :, :] = 0.0
    q.view(T, H, D)[395, :, 0] = 2.0
    v = torch.randn(T, H * E, generator=g)
    mix = torch.full((T, H), 20.0)           # beta = 1: the write is complete
    dec = torch.randn(T, H * D, generator=g)
    dec.view(T, H, D)[:, :, 0] = -30.0       # softplus ~ 0: channel 0 does not decay, the others do
    dt, a_log = torch.zeros(H * D), torch.zeros(H)
    got, state = _scan(ops.DELTA_GATED, q, k, v, dec, mix, H, H, D, E, portions, dec_bias=dt, rate_log=a_log)
    gd = torch.exp(-torch.nn.functional.softplus(dec.double()).view(T, H, D))
    want = go.gated_delta_recurrence(go.unit(q.double().view(T, H, D)) * D ** -0.5, go.unit(k.double().view(T, H, D)),
                                     v.double().view(T, H, E), torch.sigmoid(mix.double()), gd).reshape(T, H * E)
    assert _rel(got, want) < 2e-5
    # the read-out at 395 is the value written at 5 (unit q and k along channel 0, q scaled by D^-1/2)
    assert _rel(got[395] * math.sqrt(D), v[5]) < 1e-3
    assert _rel(state[:, 0, :].reshape(-1), v[5]) < 1e-3


def _needle_attention_inputs(window, T, H, Dn, P, E, R, seed):
    """Weights and inputs of a latent attention mixer in which every query has one key that dominates its softmax: at
    distance window - 1 (just inside) for even positions, at distance window (just outside) for odd ones. The input
    projections copy columns of h, the key expansion is the identity, so the test sets queries and latents directly."""
    g = torch.Generator().manual_seed(seed)
    assert Dn == R
    width = H * (Dn + P) + R + P
    eye = torch.eye(width)
    W = {"m.q": eye[:H * (Dn + P)], "m.dkv": eye[H * (Dn + P):], "m.dkv.norm": torch.ones(R),
         "m.uk": torch.eye(R).repeat(H, 1), "m.uv": torch.randn(H * E, R, generator=g) / math.sqrt(R),
         "m.g": torch.randn(H * E, width, generator=g) * 0.05, "m.o": torch.randn(width, H * E, generator=g) / math.sqrt(H * E)}
    W = {k: v.to(BF16).to(F64) for k, v in W.items()}
    q = torch.randn(T, H, Dn + P, generator=g) * 0.1
    lat = torch.randn(T, R, generator=g) * 0.02
    rot_k = torch.randn(T, P, generator=g) * 0.1
    dirs = torch.nn.functional.normalize(torch.randn(T, R, generator=g), dim=1)
    for i in range(T):
        j = i - (window - 1) if i % 2 == 0 else i - window
        if j >= 0:
            q[i, :, :Dn] += 3.0 * dirs[i]     # query i looks along its own direction ...
            lat[j] += dirs[i]                 # ... which key j carries (a key serves at most two queries)
    h = torch.cat([q.reshape(T, H * (Dn + P)), lat, rot_k], dim=1)
    return W, h.to(BF16).to(F64), width


@pytest.mark.parametrize("window", [1, 2, 5, 33, 70])
def test_latent_attention_sees_exactly_its_window(window):
    from llark_b200.mixers import LatentWindowAttention

    T, H, Dn, P, E, R = 150, 3, 24, 8, 10, 24
    spec = {"heads": H, "dim": Dn, "rot_dim": P, "vdim": E, "kv_rank": R, "scale": 1.0, "mask": {"size": window},
            "rot": {"base": 100.0, "dims": P}}
    W, h, width = _needle_attention_inputs(window, T, H, Dn, P, E, R, window)
    want = go.latent_attention(h, W, "m.", spec, 1e-5)
    whole = _run_mixer(LatentWindowAttention, W, spec, width, h, [T], F32)
    assert _rel(whole, want) < 2e-5
    # a prompt, portions down to two tokens, then decoding over several turns of the ring
    cut = _run_mixer(LatentWindowAttention, W, spec, width, h, [37, 2, 3, 2, 16] + [1] * 90, F32)
    assert _rel(cut, want) < 2e-5
    # bf16: prompts on the tensor-core kernel (latent + rotated part = 32 channels), single tokens on the SIMT kernel
    bf = _run_mixer(LatentWindowAttention, W, spec, width, h, [60, 20] + [1] * 70, BF16)
    assert _rel(bf, want) < 3e-2


def test_rotation_is_relative_and_blended():
    """The frequency table against the restatement's (plain, partial and blended), and the rotated score's dependence on
    the distance only: the same tokens later in a sequence (behind a prefix that the window has dropped) give the same
    output."""
    from llark_b200.mixers import LatentWindowAttention, rotary_frequencies

    for dims, base, sc in ((8, 100.0, None), (32, 5e5, {"factor": 6.0, "original": 2048, "fast": 16.0, "slow": 2.0}),
                           (24, 500.0, YARN), (64, 10000.0, {"factor": 40.0, "original": 4096, "fast": 32, "slow": 1})):
        f, m = rotary_frequencies(dims, base, sc)
        f2, m2 = go.yarn_frequencies(dims, base, sc)
        assert torch.allclose(f, f2, rtol=1e-12) and abs(m - m2) < 1e-12
    T, H, Dn, P, E, R, window = 40, 2, 8, 16, 8, 8, 6
    spec = {"heads": H, "dim": Dn, "rot_dim": P, "vdim": E, "kv_rank": R, "scale": 0.5, "mask": {"size": window},
            "rot": {"base": 50.0, "dims": 12, "scaling": YARN}}
    cfg = _cfg([{"type": "latent_attention", "mixer": spec, "mlp": None}], width=40)
    W = {k.replace("l0.mix.", "m."): v for k, v in go.random_weights(cfg, 3).items() if k.startswith("l0.mix.")}
    g = torch.Generator().manual_seed(0)
    h = torch.randn(T, 40, generator=g).to(BF16).to(F64)
    want = go.latent_attention(h, W, "m.", spec, 1e-5)
    got = _run_mixer(LatentWindowAttention, W, spec, 40, h, [T], F32)
    assert _rel(got, want) < 2e-5
    shifted = _run_mixer(LatentWindowAttention, W, spec, 40, torch.cat([h[:17], h]), [17 + T], F32)
    assert _rel(shifted[17 + window:], want[window:]) < 2e-5


@pytest.mark.parametrize("n,top,groups,keep", [(16, 3, 4, 2), (6, 3, 3, 2), (8, 8, 1, 1), (5, 2, 5, 3), (64, 6, 8, 4), (12, 1, 4, 4)])
def test_router(n, top, groups, keep):
    from llark_b200 import ops

    g = torch.Generator().manual_seed(n)
    z = torch.randn(300, n, generator=g) * 2
    ids, wts = ops.seq_moe_route(z.to(_dev()), groups, keep, top, 1.7)
    want_ids, want_w = go.route(z.double(), top, groups, keep, 1.7)
    order = ids.cpu().long().argsort(dim=1)
    worder = want_ids.argsort(dim=1)
    assert (ids.cpu().long().gather(1, order) == want_ids.gather(1, worder)).all()
    assert _rel(wts.cpu().gather(1, order), want_w.gather(1, worder)) < 1e-6


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("n_tok", [1, 7, 200])
def test_routed_experts(dtype, n_tok):
    """Experts in groups, more tokens than a row tile, an expert nobody picks: the residual sum against the restatement."""
    from llark_b200.mixers import RoutedExperts

    C = 40
    mlp = _moe(7, 3, 7, 4, 18, 1.3)
    cfg = _cfg([_gd(1, 8, mlp=mlp)], width=C)
    W = {k.replace("l0.mlp.", "f."): v for k, v in go.random_weights(cfg, 2).items() if k.startswith("l0.mlp.")}
    W["f.router"][3] = 0.0
    W["f.router"][3, 0] = -16.0  # with h[:, 0] = 2 expert 3 never wins
    g = torch.Generator().manual_seed(n_tok)
    h = torch.randn(n_tok, C, generator=g)
    h[:, 0] = 2.0
    h = h.to(BF16).to(F64)
    x, y = torch.randn(n_tok, C, generator=g), torch.randn(n_tok, C, generator=g)
    ff = RoutedExperts(RoutedExperts.Weights({k: v.to(F32) for k, v in W.items()}, "f.", mlp, C, _dev(), dtype), dtype)
    got = ff.residual(x.to(_dev()), y.to(_dev()), h.to(_dev(), dtype))
    want = x.double() + (y.double() + go.moe(h, W, "f.", mlp))
    assert _rel(got, want) < (2e-6 if dtype == F32 else 5e-3)


def test_routed_experts_large_step_takes_the_gemm_core():
    """A bf16 step with thousands of (token, choice) entries sorts its rows by expert and runs every run of rows through
    the tensor-core GEMM in one launch: runs of unequal length, one shorter than a tile, one empty, tiles that straddle
    nothing. Against the restatement and against the small-step kernels on the same rows."""
    from llark_b200 import ops
    from llark_b200.mixers import RoutedExperts

    C, n_tok = 64, 1500
    mlp = _moe(6, 2, 3, 2, 72, 1.0)
    cfg = _cfg([_gd(1, 8, mlp=mlp)], width=C)
    W = {k.replace("l0.mlp.", "f."): v for k, v in go.random_weights(cfg, 5).items() if k.startswith("l0.mlp.")}
    W["f.router"][3] = 0.0
    W["f.router"][3, 0] = -16.0          # expert 3 gets no rows
    W["f.router"][4] *= 0.05
    W["f.router"][4, 0] = -1.5           # expert 4 gets few
    g = torch.Generator().manual_seed(1)
    h = torch.randn(n_tok, C, generator=g)
    h[:, 0] = 2.0
    h = h.to(BF16).to(F64)
    x, y = torch.randn(n_tok, C, generator=g), torch.randn(n_tok, C, generator=g)
    ff = RoutedExperts(RoutedExperts.Weights({k: v.to(F32) for k, v in W.items()}, "f.", mlp, C, _dev(), BF16), BF16)
    assert n_tok * 2 >= ops.MOE_DENSE_MIN_ENTRIES
    got = ff.residual(x.to(_dev()), y.to(_dev()), h.to(_dev(), BF16))
    want = x.double() + (y.double() + go.moe(h, W, "f.", mlp))
    assert _rel(got, want) < 5e-3
    ids, _ = ff.route(h.to(_dev(), BF16))
    counts = torch.bincount(ids.flatten().cpu().long(), minlength=6)
    assert counts[3] == 0 and 0 < counts[4] < 256 and counts.max() > 256
    old, ops.MOE_DENSE_MIN_ENTRIES = ops.MOE_DENSE_MIN_ENTRIES, 10 ** 9
    try:
        small = ff.residual(x.to(_dev()), y.to(_dev()), h.to(_dev(), BF16))
    finally:
        ops.MOE_DENSE_MIN_ENTRIES = old
    assert _rel(got, small) < 5e-3


# ------------------------------------------------------------------------------------------------ whole model
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer(name):
    cfg = CONFIGS[name]
    W = go.random_weights(cfg, seed=1)
    toks = _tokens(61, cfg["vocab"], 1)
    want, want_layers = go.forward(cfg, W, toks, return_residuals=True)
    m = _model(cfg, W, F32)
    cache = m.new_cache()
    logits, res = m.engine.step(cache, [cache.alloc()], [toks], want=[list(range(61))], return_residuals=True)
    assert len(res) == len(want_layers)
    for i, r in enumerate(res):
        assert _rel(r, want_layers[i]) < 2e-5, f"residual after layer run {i}"
    assert _logit_err(logits, want) < 5e-5
    m16 = _model(cfg, W, BF16)
    c16 = m16.new_cache()
    got16 = m16.engine.step(c16, [c16.alloc()], [toks], want=[list(range(61))])
    assert _logit_err(got16, want, 0.9) < 8e-2


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_prefill_portions_and_decoding_agree(name, dtype):
    """The same 90 tokens: in one step; as a prompt and then token by token (long decoding, several turns of every ring);
    token by token from the start; in portions of 7, 2, 2, 30, 1, 1, 2, ..."""
    cfg = CONFIGS[name]
    W = go.random_weights(cfg, seed=3)
    toks = _tokens(90, cfg["vocab"], 2)
    m = _model(cfg, W, dtype)
    want = go.forward(cfg, W, toks)

    def run(portions):
        cache = m.new_cache()
        s = cache.alloc()
        out, at = [], 0
        for n in portions:
            out.append(m.engine.step(cache, [s], [toks[at:at + n]], want=[list(range(n))]))
            at += n
        assert at == 90 and cache.length[s] == 90
        return torch.cat(out)

    tol = 5e-5 if dtype == F32 else 8e-2
    whole = run([90])
    assert _logit_err(whole, want, _share(dtype)) < tol
    for portions in ([30] + [1] * 60, [1] * 90, [7, 2, 2, 30, 1, 1, 2, 3, 2, 40]):
        got = run(portions)
        assert _logit_err(got, want, _share(dtype)) < tol
        assert _logit_err(got, whole, _share(dtype)) < (2e-5 if dtype == F32 else 8e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_unequal_batch_equals_each_request_alone_and_slots_are_reused(dtype):
    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=4)
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
    slots = [cache.alloc() for _ in range(5)]  # together, in slots that hold the leftovers of the runs above
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
        assert _logit_err(torch.cat(got[i]), ref[i], _share(dtype)) < (2e-5 if dtype == F32 else 8e-2), i
    want0 = go.forward(cfg, W, prompts[3] + tails[3][:4])
    assert _logit_err(ref[3], want0, _share(dtype)) < (5e-5 if dtype == F32 else 8e-2)
    assert not cache.in_use()


def test_first_tokens_of_a_sequence():
    """Position 0 alone, and every prompt length up to a little beyond the windows and the taps."""
    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=6)
    m = _model(cfg, W, F32)
    toks = _tokens(12, cfg["vocab"], 6)
    want = go.forward(cfg, W, toks)
    cache = m.new_cache()
    for n in range(1, 13):
        s = cache.alloc()
        got = m.engine.step(cache, [s], [toks[:n]], want=[list(range(n))])
        assert _logit_err(got, want[:n]) < 5e-5, n
        cache.release(s)


def test_long_prompt_and_long_decoding():
    """700 tokens, the last 150 decoded one by one: windows pass over decoded tokens many times, the recurrent states
    run for hundreds of steps, the tiled kernels see prompts longer than their tiles."""
    cfg = CONFIGS["attn_ends"]
    W = go.random_weights(cfg, seed=7)
    toks = _tokens(700, cfg["vocab"], 7)
    want = go.forward(cfg, W, toks)
    for dtype, tol in ((F32, 1e-4), (BF16, 8e-2)):
        m = _model(cfg, W, dtype)
        cache = m.new_cache()
        s = cache.alloc()
        out = [m.engine.step(cache, [s], [toks[:550]], want=[[0, 1, 68, 69, 70, 71, 300, 549]])]
        for t in range(550, 700):
            out.append(m.engine.step(cache, [s], [[toks[t]]]))
        idx = [0, 1, 68, 69, 70, 71, 300, 549] + list(range(550, 700))
        assert _logit_err(torch.cat(out), want[idx], _share(dtype)) < tol


def test_checkpoint_folder_registry_and_greedy_generation(tmp_path):
    """config.json + model.safetensors -> the registry picks the class; generate() and the scheduler reproduce the
    restatement's greedy continuation (fp32, so that the argmax is the restatement's)."""
    import json

    from llark_b200.models.registry import load_model
    from llark_b200.safetensors_io import save_file
    from llark_b200.scheduler import BatchScheduler, Request

    cfg = CONFIGS["mixed"]
    W = go.random_weights(cfg, seed=8)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(BF16) for k, v in W.items()}, str(tmp_path / "model.safetensors"))
    m = load_model(str(tmp_path), dtype=F32)
    assert type(m).__name__ == "GolavikForCausalLM"

    def oracle_greedy(prompt, n):
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(go.forward(cfg, W, seq)[-1].argmax()))
        return seq

    prompts = [_tokens(9, cfg["vocab"], 1), _tokens(9, cfg["vocab"], 2)]
    want = [oracle_greedy(p, 12) for p in prompts]
    out = m.generate(input_ids=torch.tensor(prompts, device="cuda:0"), max_new_tokens=12)
    assert out.tolist() == want
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
    """generate_cli (scheduler, greedy) and the trace runner (given tokens step by step: two requests start together with
    unequal prompts, decode together, one ends earlier, a third starts later in the slot that was given back)."""
    import io
    import json

    import numpy as np

    from llark_b200 import generate_cli, trace_runner
    from llark_b200.safetensors_io import save_file

    cfg = CONFIGS["attn_ends"]
    W = go.random_weights(cfg, seed=9)
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
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": c, "want": [20]}], "end": ["c"]})
    steps.append({"step": 6, "entries": [{"id": "a", "tokens": a[34:], "want": [5]}], "end": ["a"]})
    out = tmp_path / "out"
    monkeypatch.setattr("sys.stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "80"]) == 0
    printed = capsys.readouterr().out.split("\n")
    assert [l for l in printed if l.startswith("done")] == ["done %d" % i for i in range(7)]
    la, lb, lc = go.forward(cfg, W, a), go.forward(cfg, W, b), go.forward(cfg, W, c)

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
            seq.append(int(go.forward(cfg, W, seq)[-1].argmax()))
        return seq[len(prompt):]

    assert lines == [{"id": "x", "tokens": oracle_greedy(a[:7], 6)}, {"id": "1", "tokens": oracle_greedy(b[:3], 4)}]
