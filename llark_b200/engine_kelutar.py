"""Execution schedule of the Kelutar decoder on the generation path: a list of layers, each

    h  = x + short_conv(x)                 causal depthwise convolution over time on the mixer's input
    x  = x + rmsnorm(mixer(h)) * w1        the norm sits on the sublayer's OUTPUT; the sublayers read x itself
    x  = x + rmsnorm(ff(x)) * w2           only in layers that have a feed-forward

with the mixer chosen per layer from llark_b200.mixers.MIXERS ("attention", "hgrn2"), a learned absolute position table
added to the scaled token embedding, a final RMS norm and an untied head. A layer may name another layer whose weights
it reuses; its state is its own.

The step function is llark_b200.engine_seq.LayerListEngine.step (one function for prefill and decode of a packed batch);
this class states what Kelutar's layers do. Precision: the residual stream,
norms, attention scores and softmax, gates and the recurrent state are fp32 in both modes; matrix products and the
activations between them are bf16 with fp32 accumulation (dtype=torch.bfloat16, the serving mode: tcgen05 GEMM core for
prefill, weight-streaming linears for decode) or true fp32 (dtype=torch.float32: SIMT linears, no TF32).
"""
import torch

from . import ops
from .engine_seq import LayerListEngine
from .mixers import FEED_FORWARDS, MIXERS
from .state_cache import StateCache

F32 = torch.float32


class KelutarEngine(LayerListEngine):
    def __init__(self, config, weights, device, dtype=torch.bfloat16):
        """config: llark_b200.models.kelutar.KelutarConfig; weights: name -> tensor (any device / float dtype)."""
        dev = self._init_device(device, dtype)
        self.cfg = config
        self.max_positions = config.max_positions
        C = config.width
        self.embed = weights["embed"].to(device=dev, dtype=dtype).contiguous()
        self.pos = weights["pos"].to(device=dev, dtype=dtype).contiguous()
        self.head = weights["head"].to(device=dev, dtype=dtype).contiguous()
        self.final_norm = weights["final.norm"].to(device=dev, dtype=F32).contiguous()
        if self.embed.shape != (config.vocab, C) or self.head.shape != (config.vocab, C):
            raise ValueError("embed / head do not fit vocab x width")
        if self.pos.shape != (config.max_positions, C):
            raise ValueError("pos does not fit max_positions x width")
        # packed weights per SOURCE layer (a layer with weights_of = j reads layer j's)
        self._packed = {}
        for i, layer in enumerate(config.layers):
            j = layer.weights_of if layer.weights_of is not None else i
            if j in self._packed:
                continue
            src = config.layers[j]
            p = f"l{j}."
            pk = {"mixer": MIXERS[src.type].Weights(weights, p + "mix.", src.mixer, C, dev, dtype),
                  "norm1": weights[p + "norm1"].to(device=dev, dtype=F32).contiguous(),
                  "canon": weights[p + "canon1"].to(device=dev, dtype=F32).contiguous()}
            if tuple(pk["canon"].shape) != (C, config.taps):
                raise ValueError(f"{p}canon1 does not fit width x taps")
            if src.mlp is not None:
                pk["ff"] = FEED_FORWARDS[src.mlp["kind"]].Weights(weights, p + "mlp.", src.mlp, C, dev, dtype)
                pk["norm2"] = weights[p + "norm2"].to(device=dev, dtype=F32).contiguous()
            self._packed[j] = pk
        self.launches = 0

    # ------------------------------------------------------------------------------------------ state
    def new_cache(self, n_slots=4):
        """A StateCache with every layer's stores declared: the convolution carry of every layer, a key / value ring per
        attention layer, a recurrent state per hgrn2 layer."""
        cfg = self.cfg
        cache = StateCache(self.device, n_slots=n_slots)
        layers = []
        for i, layer in enumerate(cfg.layers):
            pk = self._packed[layer.weights_of if layer.weights_of is not None else i]
            entry = {"pk": pk,
                     "tail": cache.add_store((max(cfg.taps - 1, 1), cfg.width), F32, zero_on_alloc=True),
                     "mixer": MIXERS[layer.type](pk["mixer"], cache, cfg.eps, self.act, cfg.max_positions),
                     "ff": FEED_FORWARDS[layer.mlp["kind"]](pk["ff"], self.act) if layer.mlp is not None else None}
            layers.append(entry)
        cache.layers = layers
        return cache

    # ------------------------------------------------------------------------------------------ one step (hooks)
    def _embed(self, ids, st):
        return ops.seq_embed(ids, st, self.embed, self.pos, self.cfg.embedding_scale)

    def _run_layers(self, cache, x, st, residuals):
        cfg = self.cfg
        for entry in cache.layers:
            pk = entry["pk"]
            hc = ops.seq_short_conv(x, pk["canon"], cache.view(entry["tail"]), st, self.act)
            y = entry["mixer"].forward(hc, st, cache)
            if entry["ff"] is None:
                x = ops.seq_add_rmsnorm(x, y, pk["norm1"], cfg.eps)
            else:
                x, xa = ops.seq_add_rmsnorm(x, y, pk["norm1"], cfg.eps, act=self.act)
                x = ops.seq_add_rmsnorm(x, entry["ff"].forward(xa), pk["norm2"], cfg.eps)
            if residuals is not None:
                residuals.append(x)
        return x

    def _logits(self, x, rows):
        hn = ops.seq_rmsnorm_rows(x, rows, self.final_norm, self.cfg.eps, self.act)
        return ops.linear(hn, self.head, out_dtype=F32)
