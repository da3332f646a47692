"""Request scheduler of the generation path for models that run on a StateCache (llark_b200.state_cache).

The reference decodes one prompt at a time through transformers' generate (m2t/infer.py:146-152). Here requests of
different lengths are served in STATIC batches: the scheduler takes waiting requests (up to max_batch, and as long as
the tokens they may hold fit max_tokens), prefills all of them in ONE packed step, then decodes them together, one
token per request and step. A request that finishes (eos, its token budget, a stopping callback) gives its slot back at
once and the batch goes on without it; no request joins a running batch. Sampling is the framework's: greedy argmax over
the fp32 logits unless a `sample` callable (logits [n, vocab] -> token ids [n]) is given.
"""
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int
    eos_token_id: Optional[Sequence[int]] = None
    request_id: Optional[str] = None
    output: List[int] = field(default_factory=list)
    finished: bool = False
    slot: Optional[int] = None


def greedy(logits: torch.Tensor) -> torch.Tensor:
    return logits.float().argmax(dim=-1)


class BatchScheduler:
    def __init__(self, engine, cache=None, max_batch=32, max_tokens=None, sample: Callable = greedy):
        self.engine = engine
        self.cache = cache if cache is not None else engine.new_cache()
        self.max_batch, self.max_tokens, self.sample = int(max_batch), max_tokens, sample
        self.waiting: List[Request] = []
        self.steps = 0

    def submit(self, request: Request):
        if len(request.prompt) == 0:
            raise ValueError("a request needs a prompt of at least one token")
        self.waiting.append(request)
        return request

    def _next_batch(self):
        batch, budget = [], 0
        while self.waiting and len(batch) < self.max_batch:
            r = self.waiting[0]
            need = len(r.prompt) + max(int(r.max_new_tokens), 0)
            if batch and self.max_tokens is not None and budget + need > self.max_tokens:
                break
            batch.append(self.waiting.pop(0))
            budget += need
        return batch

    def _finish(self, r):
        r.finished = True
        self.cache.release(r.slot)
        r.slot = None

    def _take(self, live, logits):
        """Append one sampled token to every live request; returns the requests that go on."""
        nxt = self.sample(logits).tolist()
        still = []
        for r, t in zip(live, nxt):
            r.output.append(int(t))
            eos = r.eos_token_id or ()
            if int(t) in eos or len(r.output) >= r.max_new_tokens:
                self._finish(r)
            else:
                still.append(r)
        return still

    def run_batch(self, batch):
        for r in batch:
            r.slot = self.cache.alloc()
        live = []
        for r in batch:  # nothing to generate: the prompt is still run (its state would be needed by a caller)
            live.append(r)
        logits = self.engine.step(self.cache, [r.slot for r in live], [list(r.prompt) for r in live])
        self.steps += 1
        done_now = [r for r in live if r.max_new_tokens <= 0]
        for r in done_now:
            self._finish(r)
        keep = [i for i, r in enumerate(live) if not r.finished]
        live = [live[i] for i in keep]
        if live:
            live = self._take(live, logits[keep])
        while live:
            logits = self.engine.step(self.cache, [r.slot for r in live], [[r.output[-1]] for r in live])
            self.steps += 1
            live = self._take(live, logits)

    def run(self):
        """Serve every waiting request; returns them in the order they were served."""
        served = []
        while self.waiting:
            batch = self._next_batch()
            self.run_batch(batch)
            served.extend(batch)
        return served
