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
from dataclasses import dataclass, field
from typing import List, Optional

from llark_b200.models.native import NativeCausalLM

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


class KelutarForCausalLM(NativeCausalLM):
    """Inference-only model object: configuration + engine (llark_b200.models.native.NativeCausalLM)."""
    config_class = KelutarConfig

    @staticmethod
    def engine_class():
        from llark_b200.engine_kelutar import KelutarEngine

        return KelutarEngine
