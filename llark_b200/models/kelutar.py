"""Kelutar: a small decoder-only language model assembled from a per-layer list of mixers -- HGRN2 gated linear
recurrences and gated sliding-window attention -- behind a short causal convolution, with RMS norms on the sublayer
OUTPUTS, a learned position table, squared-ReLU feed-forwards in some layers and layers that reuse another layer's
weights. The reference has no such model; it is served here the way the Llama path is: configuration and weights from
a checkpoint folder (config.json + model.safetensors), the CUDA engine (llark_b200.engine_kelutar), the slot cache
(llark_b200.state_cache), `generate()` through llark_b200.generate and batches through llark_b200.scheduler.

config.json keys: architecture ("Kelutar"), vocab, width, max_positions, embedding.scale, norm.eps, canon.taps, layers[]
with type ("hgrn2" | "attention"), mixer {heads, dim, vdim, kv_heads, mask.size, scale}, mlp (null | {kind: "dense", ff}),
weights_of (optional). Tensor names: embed, pos, final.norm, head, l<i>.norm1, l<i>.norm2, l<i>.canon1, l<i>.mix.*
(hgrn2: q, f, f.b, lower, v, norm, o; attention: q, q.b, k, k.b, q.norm, k.norm, temp, g, o), l<i>.mlp.up / down.
"""
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

ARCHITECTURE = "Kelutar"


@dataclass
class KelutarLayer:
    type: str
    mixer: dict
    mlp: Optional[dict] = None
    weights_of: Optional[int] = None


@dataclass
class KelutarConfig:
    vocab: int
    width: int
    max_positions: int
    embedding_scale: float
    eps: float
    taps: int
    layers: List[KelutarLayer] = field(default_factory=list)
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d):
        from llark_b200.mixers import FEED_FORWARDS, MIXERS

        if d.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration: architecture = {d.get('architecture')!r}")
        layers = []
        for i, e in enumerate(d["layers"]):
            if e["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {e['type']!r} (known: {sorted(MIXERS)})")
            mlp = e.get("mlp")
            if mlp is not None and mlp.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            wo = e.get("weights_of")
            if wo is not None:
                wo = int(wo)
                if not 0 <= wo < len(d["layers"]) or d["layers"][wo].get("weights_of") is not None:
                    raise ValueError(f"layer {i}: weights_of must name a layer that has tensors of its own")
                if d["layers"][wo]["type"] != e["type"]:
                    raise ValueError(f"layer {i}: weights_of names a layer of another type")
            layers.append(KelutarLayer(type=e["type"], mixer=dict(e["mixer"]), mlp=dict(mlp) if mlp else None,
                                       weights_of=wo))
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), max_positions=int(d["max_positions"]),
                   embedding_scale=float(d["embedding"]["scale"]), eps=float(d["norm"]["eps"]),
                   taps=int(d["canon"]["taps"]), layers=layers, eos_token_id=d.get("eos_token_id"),
                   pad_token_id=d.get("pad_token_id"))

    def to_dict(self):
        layers = []
        for l in self.layers:
            e = {"type": l.type, "mixer": l.mixer, "mlp": l.mlp}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            layers.append(e)
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "max_positions": self.max_positions, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.eps}, "canon": {"taps": self.taps}, "layers": layers}


class KelutarForCausalLM(torch.nn.Module):
    """Inference-only model object: configuration + engine. `generate` has the call shape of the Llama wrapper's."""

    def __init__(self, config: KelutarConfig, weights, device="cuda:0", dtype=torch.bfloat16):
        super().__init__()
        from llark_b200.engine_kelutar import KelutarEngine

        self.config = config
        self.generation_config = None
        self.engine = KelutarEngine(config, weights, device, dtype)
        self.device_, self.dtype_ = torch.device(device), dtype

    @classmethod
    def from_pretrained(cls, folder, dtype=torch.bfloat16, device="cuda:0"):
        from llark_b200.safetensors_io import load_file

        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
            config = KelutarConfig.from_dict(json.load(f))
        weights = load_file(os.path.join(folder, "model.safetensors"))
        return cls(config, weights, device=device, dtype=dtype)

    def new_cache(self, n_slots=4):
        return self.engine.new_cache(n_slots=n_slots)

    @torch.no_grad()
    def forward(self, input_ids):
        """Logits fp32 [B, T, vocab] of whole prompts (fresh slots, released afterwards)."""
        ids = input_ids.tolist()
        cache = self.new_cache(n_slots=max(len(ids), 1))
        slots = [cache.alloc() for _ in ids]
        logits = self.engine.step(cache, slots, ids, want=[list(range(len(r))) for r in ids])
        return logits.view(len(ids), len(ids[0]), -1)

    @torch.no_grad()
    def generate(self, inputs=None, input_ids=None, stopping_criteria=None, max_new_tokens=None, max_length=None,
                 do_sample=None, num_beams=None, eos_token_id=None, pad_token_id=None, **kwargs):
        """Greedy decoding of a batch of equal-length prompts [B, T] -> [B, T + new] through the framework's
        generate_with_model: the prompts are prefilled into fresh slots of a StateCache in one packed step, every
        further token of every row is one decode step."""
        from llark_b200.generate import generate_with_model

        state = {"cache": None, "slots": None}

        def step_logits(ids):
            if state["cache"] is None:
                state["cache"] = self.new_cache(n_slots=max(ids.shape[0], 1))
                state["slots"] = [state["cache"].alloc() for _ in range(ids.shape[0])]
                toks = ids.tolist()
            else:
                toks = ids[:, -1:].tolist()
            return self.engine.step(state["cache"], state["slots"], toks)

        return generate_with_model(self, step_logits, inputs=inputs, input_ids=input_ids,
                                   stopping_criteria=stopping_criteria, max_new_tokens=max_new_tokens,
                                   max_length=max_length, do_sample=do_sample, num_beams=num_beams,
                                   eos_token_id=eos_token_id, pad_token_id=pad_token_id)
