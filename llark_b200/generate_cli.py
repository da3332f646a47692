"""Text-free generation from the command line for native checkpoints (config.json + model.safetensors):

    python -m llark_b200.generate_cli --model DIR --prompts prompts.jsonl --max-new-tokens 64 [--dtype bfloat16]
    echo '{"id": "a", "tokens": [5, 17, 3]}' | python -m llark_b200.generate_cli --model DIR --max-new-tokens 8

Every input line is a JSON object with `tokens` (the prompt's token ids) and optionally `id`, `max_new_tokens`,
`eos_token_id`. The model class comes from config.json (llark_b200.models.registry); requests are served by the
BatchScheduler in static batches (greedy decoding) and one JSON line per request is printed: {"id", "tokens": [...new ids]}.
The audio-conditioned Llama / MPT checkpoints keep their own entry point, llark_b200.infer_cli."""
import argparse
import json
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--prompts", default="-", help="JSON-lines file of requests ('-': standard input)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--max-new-tokens", type=int, default=32, help="token budget of requests that name none")
    ap.add_argument("--eos-token-id", type=int, action="append", default=None)
    ap.add_argument("--max-batch", type=int, default=32, help="most requests in one static batch")
    ap.add_argument("--max-tokens", type=int, default=None, help="most tokens (prompt + budget) one batch may hold")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    from llark_b200.build import ensure_built

    ensure_built()
    from llark_b200.models.registry import load_model
    from llark_b200.scheduler import BatchScheduler, Request

    model = load_model(a.model, dtype=torch.bfloat16 if a.dtype == "bfloat16" else torch.float32, device=a.device)
    sched = BatchScheduler(model.engine, max_batch=a.max_batch, max_tokens=a.max_tokens)
    src = sys.stdin if a.prompts == "-" else open(a.prompts, "r", encoding="utf-8")
    n = 0
    with src:
        for line in src:
            line = line.strip()
            if not line:
                continue
            d = json.loads(line)
            eos = d.get("eos_token_id", a.eos_token_id)
            if isinstance(eos, int):
                eos = [eos]
            sched.submit(Request(prompt=[int(t) for t in d["tokens"]],
                                 max_new_tokens=int(d.get("max_new_tokens", a.max_new_tokens)), eos_token_id=eos,
                                 request_id=str(d.get("id", n))))
            n += 1
    for r in sched.run():
        sys.stdout.write(json.dumps({"id": r.request_id, "tokens": r.output}) + "\n")
    sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
