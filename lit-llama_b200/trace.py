"""Trace replay: feed given token ids through a model step by step and write the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step with wanted places, OUT/<step>.f32 receives the logits [wanted, vocab] as little-endian f32, in the order
of the entries and of `want`; after every step the line `done <step>` is printed.  Requests listed under `end` give
their state slot back.  Nothing is sampled.  The model class comes from config.json (registry), the steps run through
`Engine.step`, i.e. the state pool, kernels and step function that generation uses."""
import argparse
import json
import os
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, default=0)
    ap.add_argument("--slots", type=int, default=4)
    a = ap.parse_args(argv)

    from .engine import Engine
    from .registry import load_model

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device (there is no CPU fallback)", file=sys.stderr)
        return 2
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    device = torch.device("cuda", 0)
    model = load_model(a.model, dtype=dtype, device=device, max_positions=a.max_tokens)
    engine = Engine(model, n_slots=a.slots, max_tokens=a.max_tokens, device=device)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        outs = engine.step(msg.get("entries", []), msg.get("end", []))
        rows = [o for o in outs if o.numel()]
        if rows:
            data = torch.cat(rows, dim=0).to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
            tmp = os.path.join(a.out, ".%d.part" % msg["step"])
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, "%d.f32" % msg["step"]))
        else:
            torch.cuda.synchronize(device)
        sys.stdout.write("done %d\n" % msg["step"])
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
