"""Replays a trace of steps through the engine's step function and writes the logits that were asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line, ``{"step": n, "entries": [{"id", "tokens", "want"}, ...], "end": [ids]}``: each
entry brings the next tokens of a request (a request is admitted at its first entry) and the places among them whose logits are
wanted; all entries of a line run as one batch through ``ModelRunner.execute``; the requests named in ``end`` give their blocks and
state slot back afterwards.  For a step with wanted places the f32 logits [wanted, vocab] go to ``<out>/<step>.f32`` (little endian,
entry order); after every step the line ``done <step>`` is printed.  Nothing is sampled.  The cache pool holds ``--max-tokens`` tokens
(rounded up to whole blocks) and ``--slots`` state slots, so blocks and slots are handed from finished requests to new ones.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--block-size", type=int, default=64)
    a = ap.parse_args(argv)

    from ._lib import ensure_built
    from .registry import build_group_of
    ensure_built(build_group_of(a.model))
    from .engine import ModelRunner
    from .registry import load_model
    torch.cuda.set_device(0)
    dtype = torch.bfloat16 if a.dtype == "bfloat16" else torch.float32
    bs = a.block_size
    num_blocks = max(1, -(-a.max_tokens // bs))
    model = load_model(a.model, dtype=dtype, block_size=bs, max_pos=max(a.max_tokens, bs))
    runner = ModelRunner(model, num_blocks, a.slots, bs)
    os.makedirs(a.out, exist_ok=True)
    ids, next_id = {}, 0
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries = []
        for e in msg.get("entries", []):
            if e["id"] not in ids:
                ids[e["id"]] = next_id
                next_id += 1
                runner.admit(ids[e["id"]])
            if e["tokens"]:
                entries.append(dict(seq_id=ids[e["id"]], tokens=e["tokens"], want=e.get("want", [])))
        logits = runner.execute(entries)
        if logits is not None:
            host = logits.float().cpu().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{msg['step']}.part")
            host.tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{msg['step']}.f32"))
        else:
            torch.cuda.synchronize()
        for name in msg.get("end", []):
            if name in ids:
                runner.release(ids.pop(name))
        sys.stdout.write(f"done {msg['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
