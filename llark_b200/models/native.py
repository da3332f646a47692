"""What the native decoders (checkpoint folder = config.json + model.safetensors) share as model objects: loading, a
slot cache, whole-prompt logits and `generate()` with the call shape of the Llama wrapper's. A model names its
configuration class and its engine class."""
import json
import os

import torch


class NativeCausalLM(torch.nn.Module):
    """Inference-only model object: configuration + engine."""
    config_class = None

    @staticmethod
    def engine_class():
        raise NotImplementedError

    def __init__(self, config, weights, device="cuda:0", dtype=torch.bfloat16):
        super().__init__()
        self.config = config
        self.generation_config = None
        self.engine = self.engine_class()(config, weights, device, dtype)
        self.device_, self.dtype_ = torch.device(device), dtype

    @classmethod
    def from_pretrained(cls, folder, dtype=torch.bfloat16, device="cuda:0"):
        from llark_b200.safetensors_io import load_file

        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as f:
            config = cls.config_class.from_dict(json.load(f))
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
