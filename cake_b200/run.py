"""`python -m cake_b200.run` — generate from a checkpoint on a B200 through the Python host (Context, TextModelBase, Master),
the twin of cake_b200/host/cake_run (reference: `cake run`, sharding/master.rs:109-168) that also serves the layer-list
models (Nigenex), which the compiled host does not load.  Token ids in, token ids out (tokenizer and chat template stay with
the caller):

    python -m cake_b200.run <model_dir> --prompt-ids 1,2,3 [-n 32] [--dtype bf16|f16|f32] [--max-seq S]
                            [--temperature T] [--top-k K] [--top-p P] [--seed N] [--repeat-penalty R]
    python -m cake_b200.run <model_dir> --show-config          # resolve config.json only (needs no GPU)

<model_dir> holds config.json + model.safetensors (or an index + shards).  The model class follows config.json.
"""
from __future__ import annotations

import argparse
import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m cake_b200.run")
    ap.add_argument("model_dir")
    ap.add_argument("--prompt-ids", default="")
    ap.add_argument("-n", type=int, default=32)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16", "f32"])
    ap.add_argument("--max-seq", type=int, default=0)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int)
    ap.add_argument("--top-p", type=float)
    ap.add_argument("--seed", type=int, default=299792458)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--show-config", action="store_true")
    a = ap.parse_args(argv)
    from .loader import open_model
    cfg, vb = open_model(a.model_dir)
    if a.show_config:
        print(cfg)
        return 0
    if a.dtype == "f32" and not cfg.layer_list:
        print("error: f32 is served for layer-list models only", file=sys.stderr)
        return 2
    prompt = [int(t) for t in a.prompt_ids.split(",") if t.strip()]
    if not prompt:
        print("error: --prompt-ids is empty", file=sys.stderr)
        return 2
    from .build import build
    build(host=False, quiet=True)
    from .model import Context, Master, TextModelBase
    max_seq = a.max_seq or min(cfg.max_seq_len, len(prompt) + a.n + 1)
    ctx = Context(cfg, vb, a.dtype, device=a.device, max_seq=max_seq)
    try:
        model = TextModelBase.load(ctx, repeat_penalty=a.repeat_penalty, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p, seed=a.seed)
        out = Master(model).generate_text(prompt, a.n)
        print("tokens: " + " ".join(str(t) for t in out["tokens"]))
        print(f"tok/s: {out['tok_s']:.2f}")
    finally:
        ctx.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
