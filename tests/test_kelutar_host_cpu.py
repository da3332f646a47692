"""Host side of the generation path of native checkpoints, on the CPU: the safetensors container, configuration and
registry, the slot cache and packed-step descriptor, and the scheduler's batching over a stand-in engine."""
import json

import pytest
import torch

from llark_b200.models.kelutar import KelutarConfig
from llark_b200.models.registry import model_class_for
from llark_b200.safetensors_io import load_file, save_file
from llark_b200.scheduler import BatchScheduler, Request
from llark_b200.state_cache import StateCache, StepLayout


def test_safetensors_round_trip(tmp_path):
    g = torch.Generator().manual_seed(0)
    t = {"a.b": torch.randn(3, 5, generator=g).to(torch.bfloat16), "c": torch.arange(7, dtype=torch.int32),
         "d.e.f": torch.randn(2, 2, 2, generator=g), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "m.safetensors")
    save_file(t, p, metadata={"k": 1})
    back = load_file(p)
    assert set(back) == set(t)
    for k in t:
        assert back[k].dtype == t[k].dtype and back[k].shape == t[k].shape and torch.equal(back[k], t[k])
    raw = open(p, "rb").read()
    n = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + n])
    assert header["a.b"]["dtype"] == "BF16" and header["__metadata__"] == {"k": "1"}
    with open(p, "r+b") as f:
        f.truncate(len(raw) - 3)
    with pytest.raises(ValueError):
        load_file(p)


def _cfg():
    hg = {"type": "hgrn2", "mixer": {"heads": 2, "dim": 8, "vdim": 12}, "mlp": None}
    at = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "mask": {"size": 5},
                                         "scale": 0.5}, "mlp": {"kind": "dense", "ff": 40}}
    return {"architecture": "Kelutar", "vocab": 31, "width": 24, "max_positions": 64, "embedding": {"scale": 2.0},
            "norm": {"eps": 1e-4}, "canon": {"taps": 2}, "layers": [hg, at, dict(hg, weights_of=0)]}


def test_config_and_registry():
    c = KelutarConfig.from_dict(_cfg())
    assert (c.vocab, c.width, c.taps, c.eps, c.embedding_scale) == (31, 24, 2, 1e-4, 2.0)
    assert [l.type for l in c.layers] == ["hgrn2", "attention", "hgrn2"] and c.layers[2].weights_of == 0
    assert KelutarConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    assert model_class_for(_cfg()).__name__ == "KelutarForCausalLM"
    assert model_class_for({"model_type": "wrapped_llamav2"}).__name__ == "WrappedLlamav2ForCausalLM"
    with pytest.raises(ValueError):
        model_class_for({"architecture": "nothing"})
    bad = _cfg()
    bad["layers"][2]["weights_of"] = 1  # another type
    with pytest.raises(ValueError):
        KelutarConfig.from_dict(bad)
    bad = _cfg()
    bad["layers"][0]["type"] = "conv"
    with pytest.raises(ValueError):
        KelutarConfig.from_dict(bad)


def test_step_layout():
    st = StepLayout([3, 1, 2], [0, 17, 5], [4, 0, 2], "cpu")
    assert st.tok_seq.tolist() == [0, 0, 0, 1, 2, 2] and st.cu.tolist() == [0, 3, 4, 6]
    assert st.pos0.tolist() == [0, 17, 5] and st.slot.tolist() == [4, 0, 2]
    assert (st.n_tok, st.n_seq, st.max_len) == (6, 3, 3)
    with pytest.raises(ValueError):
        StepLayout([2, 0], [0, 0], [0, 1], "cpu")


def test_state_cache_slots_zeroing_and_growth():
    c = StateCache("cpu", n_slots=2)
    h_state = c.add_store((2, 3), torch.float32, zero_on_alloc=True)
    h_state2 = c.add_store((2, 3), torch.float32, zero_on_alloc=True)
    h_ring = c.add_store((4, 5), torch.bfloat16, zero_on_alloc=False)
    a, b = c.alloc(), c.alloc()
    assert {a, b} == {0, 1} and c.view(h_state).shape == (2, 2, 3) and c.view(h_ring).shape == (2, 4, 5)
    assert c.view(h_state).is_contiguous() and c.view(h_state2).is_contiguous()
    c.view(h_state)[a] = 5.0
    c.view(h_state2)[b] = 6.0
    c.view(h_ring)[a] = 7.0
    c.advance([a, b], [3, 9])
    assert c.tokens_held() == 12
    st = c.layout([b, a], [1, 2])
    assert st.pos0.tolist() == [9, 3] and st.slot.tolist() == [b, a]
    with pytest.raises(ValueError):
        c.layout([a, a], [1, 1])
    third = c.alloc()  # no free slot: the stores double and keep what they held
    assert third == 2 and c.n_slots == 4
    assert (c.view(h_state)[a] == 5.0).all() and (c.view(h_state2)[b] == 6.0).all() and (c.view(h_ring)[a] == 7.0).all()
    c.release(a)
    with pytest.raises(KeyError):
        c.layout([a], [1])
    again = c.alloc()  # the freed slot comes back with its recurrent state zeroed; a ring needs no clearing
    assert again == a and (c.view(h_state)[a] == 0).all() and c.length[a] == 0
    assert (c.view(h_state2)[b] == 6.0).all()
    assert c.allocs == 4 and c.in_use() == sorted([a, b, third])
    assert c.bytes_per_slot() == 2 * 6 * 4 + 20 * 2


class _EchoEngine:
    """Stand-in for the step function: the 'logits' of a row put all mass on (sum of the request's tokens so far) % 13,
    so that a request's continuation depends on its own history only. Records the batches it was given."""

    def __init__(self):
        self.batches = []

    def new_cache(self):
        c = StateCache("cpu", n_slots=1)
        self.h = c.add_store((1,), torch.int64, zero_on_alloc=True)
        return c

    def step(self, cache, slots, tokens, want=None):
        self.batches.append([len(t) for t in tokens])
        acc = cache.view(self.h)
        out = torch.zeros(len(slots), 13)
        for i, (s, ts) in enumerate(zip(slots, tokens)):
            acc[s, 0] += sum(ts)
            out[i, int(acc[s, 0]) % 13] = 1.0
        cache.advance(slots, [len(t) for t in tokens])
        return out


def _expected(prompt, n, eos=()):
    acc, out = sum(prompt), []
    for _ in range(n):
        t = acc % 13
        out.append(t)
        acc += t
        if t in eos:
            break
    return out


def test_scheduler_static_batches():
    eng = _EchoEngine()
    sched = BatchScheduler(eng, max_batch=3, max_tokens=40)
    reqs = [Request([1, 2, 3], 5), Request([4], 2), Request([5, 5], 9, eos_token_id=[3]), Request([7] * 20, 15),
            Request([2, 2], 0)]
    for r in reqs:
        sched.submit(r)
    served = sched.run()
    assert served == reqs and all(r.finished and r.slot is None for r in reqs)
    for r in reqs:
        assert r.output == _expected(list(r.prompt), r.max_new_tokens, tuple(r.eos_token_id or ()))
    # first batch: three requests (3 + 5, 1 + 2, 2 + 9 tokens fit the budget of 40); the fourth (35) waits, and the
    # fifth cannot join the fourth's batch (35 + 2 fits, so it does)
    assert eng.batches[0] == [3, 1, 2]
    assert [20, 2] in eng.batches
    # a finished request leaves the batch: decode batches never grow
    first_decodes = eng.batches[1:eng.batches.index([20, 2])]
    assert all(b == [1] * len(b) for b in first_decodes)
    assert [len(b) for b in first_decodes] == sorted([len(b) for b in first_decodes], reverse=True)
    assert not sched.cache.in_use()
