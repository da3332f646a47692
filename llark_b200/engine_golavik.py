"""Execution schedule of the Golavik decoder on the generation path: a list of layers with side-by-side sublayers,

    h  = group_rmsnorm(x) * w                   RMS norm in `norm.groups` equal parts of the width
    x  = x + (mixer(h + conv1(h)) + ff(h + conv2(h)))

each sublayer behind its own short causal convolution over time (carry of the last taps-1 inputs per request), the mixer
chosen per layer from llark_b200.mixers.MIXERS ("latent_attention", "channel_delta", "general_delta"), the feed-forward a
routed mixture of experts (or none). A block of layers can run several times in a row with the same weights (`loop`): each
pass has state of its own and starts by adding a learned vector `loop.step[pass]` to the stream. A final grouped norm and
the embedding table as the output matrix give the logits.

The step function is llark_b200.engine_seq.LayerListEngine.step; state lives in a llark_b200.state_cache.StateCache.
Precision: the residual stream, norms, convolution carries, rotation angles, attention scores and softmax, router, decays,
gates of the recurrences and their states are fp32 in both modes; matrix products and the activations between them are
bf16 with fp32 accumulation (dtype=torch.bfloat16) or true fp32 (dtype=torch.float32).
"""
import torch

from . import ops
from .engine_seq import LayerListEngine
from .mixers import FEED_FORWARDS, MIXERS
from .state_cache import StateCache

F32 = torch.float32


class GolavikEngine(LayerListEngine):
    def __init__(self, config, weights, device, dtype=torch.bfloat16):
        """config: llark_b200.models.golavik.GolavikConfig; weights: name -> tensor (any device / float dtype)."""
        dev = self._init_device(device, dtype)
        self.cfg = config
        C = config.width
        self.embed = weights["embed"].to(device=dev, dtype=dtype).contiguous()
        self.final_norm = weights["final.norm"].to(device=dev, dtype=F32).contiguous()
        if tuple(self.embed.shape) != (config.vocab, C):
            raise ValueError("embed does not fit vocab x width")
        self.loop_step = None
        if config.loop is not None:
            self.loop_step = weights["loop.step"].to(device=dev, dtype=F32).contiguous()
            if tuple(self.loop_step.shape) != (config.loop["times"], C):
                raise ValueError("loop.step does not fit times x width")
        self._packed = []
        for i, layer in enumerate(config.layers):
            p = f"l{i}."
            pk = {"mixer": MIXERS[layer.type].Weights(weights, p + "mix.", layer.mixer, C, dev, dtype),
                  "norm1": weights[p + "norm1"].to(device=dev, dtype=F32).contiguous(),
                  "canon1": weights[p + "canon1"].to(device=dev, dtype=F32).contiguous()}
            if layer.mlp is not None:
                pk["ff"] = FEED_FORWARDS[layer.mlp["kind"]].Weights(weights, p + "mlp.", layer.mlp, C, dev, dtype)
                pk["canon2"] = weights[p + "canon2"].to(device=dev, dtype=F32).contiguous()
            for name in ("canon1", "canon2"):
                if name in pk and tuple(pk[name].shape) != (C, config.taps):
                    raise ValueError(f"{p}{name} does not fit width x taps")
            self._packed.append(pk)

    # ------------------------------------------------------------------------------------------ state
    def new_cache(self, n_slots=4):
        """A StateCache with the stores of every layer RUN declared (a layer inside the loop runs once per pass, each time
        on state of its own): two convolution carries, and what the run's mixer keeps."""
        cfg = self.cfg
        cache = StateCache(self.device, n_slots=n_slots)
        runs = []
        carry = (max(cfg.taps - 1, 1), cfg.width)
        for i, t, first in cfg.layer_runs():
            pk, layer = self._packed[i], cfg.layers[i]
            runs.append({"pk": pk, "pass_vec": self.loop_step[t] if first else None,
                         "tail1": cache.add_store(carry, F32, zero_on_alloc=True),
                         "tail2": cache.add_store(carry, F32, zero_on_alloc=True) if layer.mlp is not None else None,
                         "mixer": MIXERS[layer.type](pk["mixer"], cache, cfg.eps, self.act, self.max_positions),
                         "ff": FEED_FORWARDS[layer.mlp["kind"]](pk["ff"], self.act) if layer.mlp is not None else None})
        cache.layers = runs
        return cache

    # ------------------------------------------------------------------------------------------ one step (hooks)
    def _embed(self, ids, st):
        return ops.seq_embed(ids, st, self.embed, None, 1.0)

    def _run_layers(self, cache, x, st, residuals):
        cfg = self.cfg
        for run in cache.layers:
            pk = run["pk"]
            if run["pass_vec"] is not None:
                x, h = ops.seq_group_rmsnorm(x, pk["norm1"], cfg.groups, cfg.eps, add_vec=run["pass_vec"])
            else:
                h = ops.seq_group_rmsnorm(x, pk["norm1"], cfg.groups, cfg.eps)
            y = run["mixer"].forward(ops.seq_short_conv(h, pk["canon1"], cache.view(run["tail1"]), st, self.act), st, cache)
            if run["ff"] is None:
                x = ops.seq_residual_combine(x, y)
            else:
                h2 = ops.seq_short_conv(h, pk["canon2"], cache.view(run["tail2"]), st, self.act)
                x = run["ff"].residual(x, y, h2)
            if residuals is not None:
                residuals.append(x)
        return x

    def _logits(self, x, rows):
        hn = ops.seq_group_rmsnorm(x, self.final_norm, self.cfg.groups, self.cfg.eps, out_dtype=self.act, rows=rows)
        return ops.linear(hn, self.embed, out_dtype=F32)
