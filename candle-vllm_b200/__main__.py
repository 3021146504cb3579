"""Command line: ``python -m candle_vllm_b200 <command>``.

  generate   token ids in, token ids out, through LLMEngine (the framework carries no tokenizer)
  trace      replay a step trace and write logits (what bin/trace_run starts)
  models     list the registered architectures
"""
from __future__ import annotations

import argparse
import json
import sys


def _generate(argv) -> int:
    import torch
    from ._lib import ensure_built
    from .engine import LLMEngine
    from .sampling import SamplingParams
    ap = argparse.ArgumentParser(prog="generate")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for a batch")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--num-blocks", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=4)
    ap.add_argument("--prefill-chunk", type=int, default=512)
    ap.add_argument("--decode-graphs", action="store_true", help="replay captured CUDA graphs for steps of single tokens")
    a = ap.parse_args(argv)
    from .registry import build_group_of
    ensure_built(build_group_of(a.model))
    prompts = [[int(t) for t in p.split(",") if t.strip()] for p in a.prompt_ids]
    eng = LLMEngine.from_pretrained(a.model, dtype=torch.bfloat16 if a.dtype == "bfloat16" else torch.float32, num_blocks=a.num_blocks,
                                    max_num_seqs=a.max_num_seqs, prefill_chunk=a.prefill_chunk, decode_graphs=a.decode_graphs,
                                    max_model_len=max(len(p) for p in prompts) + a.max_new_tokens + 1)
    sp = SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, max_tokens=a.max_new_tokens, seed=a.seed)
    for p, out in zip(prompts, eng.generate(prompts, sp)):
        print(json.dumps({"prompt": p, "output": out}))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "generate":
        return _generate(rest)
    if cmd == "trace":
        from .trace_runner import main as trace_main
        return trace_main(rest)
    if cmd == "models":
        from .registry import registered
        print("\n".join(registered()))
        return 0
    print(f"unknown command {cmd!r}\n{__doc__}", file=sys.stderr)
    return 2


if __name__ == "__main__":
    sys.exit(main())
