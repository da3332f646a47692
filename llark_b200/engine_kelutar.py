"""Execution schedule of the Kelutar decoder on the generation path: a list of layers, each

    h  = x + short_conv(x)                 causal depthwise convolution over time on the mixer's input
    x  = x + rmsnorm(mixer(h)) * w1        the norm sits on the sublayer's OUTPUT; the sublayers read x itself
    x  = x + rmsnorm(ff(x)) * w2           only in layers that have a feed-forward

with the mixer chosen per layer from llark_b200.mixers.MIXERS ("attention", "hgrn2"), a learned absolute position table
added to the scaled token embedding, a final RMS norm and an untied head. A layer may name another layer whose weights
it reuses; its state is its own.

The engine is host-side orchestration only, like LlamaEngine: every FLOP is a C-ABI call. One `step()` runs a PACKED
batch (llark_b200.state_cache): requests that start, go on by a portion of their prompt or decode one token are the
same kernels with other numbers, so there is one step function for prefill and decode. Precision: the residual stream,
norms, attention scores and softmax, gates and the recurrent state are fp32 in both modes; matrix products and the
activations between them are bf16 with fp32 accumulation (dtype=torch.bfloat16, the serving mode: tcgen05 GEMM core for
prefill, weight-streaming linears for decode) or true fp32 (dtype=torch.float32: SIMT linears, no TF32).
"""
import torch

from . import ops
from .mixers import FEED_FORWARDS, MIXERS
from .state_cache import StateCache

F32 = torch.float32


class KelutarEngine:
    def __init__(self, config, weights, device, dtype=torch.bfloat16):
        """config: llark_b200.models.kelutar.KelutarConfig; weights: name -> tensor (any device / float dtype)."""
        dev = torch.device(device)
        if dev.type != "cuda":
            raise RuntimeError("llark_b200 has no CPU path: the engine needs a CUDA device (B200)")
        if dtype not in (torch.bfloat16, torch.float32):
            raise TypeError("dtype must be torch.bfloat16 or torch.float32")
        self.cfg, self.device, self.act = config, dev, dtype
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

    # ------------------------------------------------------------------------------------------ one step
    @torch.no_grad()
    def step(self, cache, slots, tokens, want=None, return_residuals=False):
        """slots: the requests of this step; tokens[b]: the next token ids of request slots[b] (they continue at the
        position where the request stopped); want[b]: indices into tokens[b] whose logits are asked for (None: the last
        one of each). Returns fp32 logits [n_wanted, vocab] in the order of the requests and of `want` (None when nothing
        is wanted). The caches advance by the step's tokens."""
        cfg = self.cfg
        lens = [len(t) for t in tokens]
        st = cache.layout(slots, lens)
        for s, n in zip(slots, lens):
            if cache.length[s] + n > cfg.max_positions:
                raise ValueError("a request grows past max_positions")
        flat = [int(t) for ts in tokens for t in ts]
        if flat and (min(flat) < 0 or max(flat) >= cfg.vocab):
            raise ValueError("token id outside the vocabulary")
        ids = torch.tensor(flat, dtype=torch.int32).to(self.device, non_blocking=True)
        if want is None:
            want = [[n - 1] for n in lens]
        rows = [st.cu_host[b] + int(k) for b, w in enumerate(want) for k in w]
        for b, w in enumerate(want):
            if any(k < 0 or k >= lens[b] for k in w):
                raise ValueError("a wanted place lies outside the request's tokens")
        x = ops.seq_embed(ids, st, self.embed, self.pos, cfg.embedding_scale)
        residuals = []
        for entry in cache.layers:
            pk = entry["pk"]
            hc = ops.seq_short_conv(x, pk["canon"], cache.view(entry["tail"]), st, self.act)
            y = entry["mixer"].forward(hc, st, cache)
            if entry["ff"] is None:
                x = ops.seq_add_rmsnorm(x, y, pk["norm1"], cfg.eps)
            else:
                x, xa = ops.seq_add_rmsnorm(x, y, pk["norm1"], cfg.eps, act=self.act)
                x = ops.seq_add_rmsnorm(x, entry["ff"].forward(xa), pk["norm2"], cfg.eps)
            if return_residuals:
                residuals.append(x)
        cache.advance(slots, lens)
        logits = None
        if rows:
            idx = torch.tensor(rows, dtype=torch.int32).to(self.device, non_blocking=True)
            hn = ops.seq_rmsnorm_rows(x, idx, self.final_norm, cfg.eps, self.act)
            logits = ops.linear(hn, self.head, out_dtype=F32)
        if return_residuals:
            return logits, residuals
        return logits
