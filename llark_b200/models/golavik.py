"""Golavik: a small decoder-only language model assembled from a per-layer list of mixers -- latent attention with a
sliding window, a gated delta rule with per-channel decay, a generalized delta rule -- with side-by-side sublayers behind
one grouped RMS norm, a short causal convolution in front of every sublayer, routed mixtures of experts as feed-forwards,
a block of layers that runs several times with the same weights, and the embedding table as the output matrix. The
reference has no such model; it is served the way the other native decoder is: configuration and weights from a
checkpoint folder (config.json + model.safetensors), the CUDA engine (llark_b200.engine_golavik), the slot cache
(llark_b200.state_cache), `generate()` through llark_b200.generate and batches through llark_b200.scheduler.

config.json keys: architecture ("Golavik"), vocab, width, norm.eps, norm.groups, canon.taps, loop (null | {start, stop,
times}), layers[] with type ("latent_attention" | "channel_delta" | "general_delta"), mixer {...}, mlp (null | {kind: "moe",
expert.ff, router {experts, top, scale, groups {count, keep}}}).
  latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, scale, mask.size, rot {base, dims, scaling {factor, original,
                          fast, slow}};  tensors q, dkv, dkv.norm, uk, uv, g, o
  channel_delta mixer:    heads, kv_heads, dim, vdim, conv;  tensors q, k, v (+ .conv each), b, A_log, a1, a2, dt_bias, g1,
                          g2, norm, o
  general_delta mixer:    heads, dim;  tensors r, k, v, w1, w2, w0, a, a.b, g, norm, o
Other tensors: embed, loop.step, final.norm, l<i>.norm1, l<i>.canon1, l<i>.canon2, l<i>.mlp.router, l<i>.mlp.e<j>.gate / up /
down.
"""
from dataclasses import dataclass, field
from typing import List, Optional

from llark_b200.models.native import NativeCausalLM

ARCHITECTURE = "Golavik"
LAYER_TYPES = ("latent_attention", "channel_delta", "general_delta")


@dataclass
class GolavikLayer:
    type: str
    mixer: dict
    mlp: Optional[dict] = None


@dataclass
class GolavikConfig:
    vocab: int
    width: int
    eps: float
    groups: int
    taps: int
    layers: List[GolavikLayer] = field(default_factory=list)
    loop: Optional[dict] = None
    eos_token_id: Optional[int] = None
    pad_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d):
        from llark_b200.mixers import FEED_FORWARDS, MIXERS

        if d.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration: architecture = {d.get('architecture')!r}")
        layers = []
        for i, e in enumerate(d["layers"]):
            if e["type"] not in LAYER_TYPES or e["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {e['type']!r} (known: {list(LAYER_TYPES)})")
            mlp = e.get("mlp")
            if mlp is not None and not hasattr(FEED_FORWARDS.get(mlp.get("kind")), "residual"):
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} cannot run beside a mixer")
            layers.append(GolavikLayer(type=e["type"], mixer=dict(e["mixer"]), mlp=dict(mlp) if mlp else None))
        width, groups = int(d["width"]), int(d["norm"].get("groups", 1))
        if groups < 1 or width % groups:
            raise ValueError("norm.groups must divide width")
        loop = d.get("loop")
        if loop is not None:
            loop = {k: int(loop[k]) for k in ("start", "stop", "times")}
            if not (0 <= loop["start"] <= loop["stop"] <= len(layers)) or loop["times"] < 1:
                raise ValueError("loop must name a range of layers and a positive number of passes")
            if loop["start"] == loop["stop"]:
                loop = None
        return cls(vocab=int(d["vocab"]), width=width, eps=float(d["norm"]["eps"]), groups=groups,
                   taps=int(d["canon"]["taps"]), layers=layers, loop=loop, eos_token_id=d.get("eos_token_id"),
                   pad_token_id=d.get("pad_token_id"))

    def layer_runs(self):
        """(layer, pass, first layer of a pass?) in the order the layers run; pass is None outside the loop."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        runs = [(i, None, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t, i == a) for i in range(a, b)]
        return runs + [(i, None, False) for i in range(b, n)]

    def to_dict(self):
        return {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps, "groups": self.groups}, "canon": {"taps": self.taps}, "loop": self.loop,
                "layers": [{"type": l.type, "mixer": l.mixer, "mlp": l.mlp} for l in self.layers]}


class GolavikForCausalLM(NativeCausalLM):
    """Inference-only model object: configuration + engine (llark_b200.models.native.NativeCausalLM)."""
    config_class = GolavikConfig

    @staticmethod
    def engine_class():
        from llark_b200.engine_golavik import GolavikEngine

        return GolavikEngine
