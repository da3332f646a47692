"""Trace runner: feeds given token ids through a model, step by step, and writes logits. It samples nothing; it drives
the same model object, step function, StateCache and kernels as `generate()` and the BatchScheduler.

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

`entries`: for each request its next tokens (a request seen for the first time starts at position 0 in a fresh slot)
and `want`, the places among these tokens whose logits are asked for. All entries of a step are one packed batch. `end`:
requests that are finished after the step; their slots are released. For a step in which something is wanted the fp32
logits [wanted, vocab] are written to <out>/<step>.f32 (little-endian, in the order of the entries and of `want`); after
every step `done <step>` is printed and flushed.
"""
import argparse
import json
import os
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="bfloat16: the serving kernels; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder the <step>.f32 files are written to")
    ap.add_argument("--max-tokens", type=int, default=None,
                    help="most tokens live requests hold at any time (bounds a request's length where the model names no bound)")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    from llark_b200.models.registry import load_model

    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    torch.cuda.set_device(torch.device(a.device))
    model = load_model(a.model, dtype=dtype, device=a.device)
    engine = model.engine
    if a.max_tokens and engine.max_positions is None:
        engine.max_positions = int(a.max_tokens)  # no request outgrows what all live requests may hold: bounds the rings
    cache = model.new_cache()
    os.makedirs(a.out, exist_ok=True)
    slots = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = [e for e in step.get("entries", []) if e.get("tokens")]  # an entry without tokens asks for nothing
        if entries:
            for e in entries:
                if e["id"] not in slots:
                    slots[e["id"]] = cache.alloc()
            logits = engine.step(cache, [slots[e["id"]] for e in entries], [e["tokens"] for e in entries],
                                 want=[e.get("want", []) for e in entries])
            if logits is not None:
                data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(a.out, ".%s.part" % step["step"])
                with open(tmp, "wb") as f:
                    f.write(data.tobytes())
                os.replace(tmp, os.path.join(a.out, "%s.f32" % step["step"]))
            else:
                torch.cuda.synchronize()
        for rid in step.get("end", []):
            if rid in slots:
                cache.release(slots.pop(rid))
        sys.stdout.write("done %s\n" % step["step"])
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
