"""Command line of the serving stack.

  python -m wf_bitnet.cli generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] --max-new-tokens 16 [--temperature T --top-k K --top-p P]
  python -m wf_bitnet.cli trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (bin/trace_run)

`generate` queues the prompts on the scheduler and prints one JSON line per finished request.  `trace` replays a schedule given on
standard input, one JSON object per line — {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]} — through the same model,
cache manager and batch execution, writes the logits of the wanted positions to OUT/<step>.f32 (little-endian float32 [wanted, vocab])
and answers `done <step>` after every step.  Both pick the model class from config.json through the registry.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from . import checkpoint, registry


def load_model(model_dir, dtype: str, max_tokens: int, slots: int, page_size: int, max_step_tokens: int):
    """config.json -> model class (registry) -> a loaded model that implements the step interface."""
    cfg = checkpoint.read_config(model_dir)
    cls = registry.resolve(cfg)
    if not hasattr(cls, "step") or not hasattr(cls, "from_pretrained"):
        raise SystemExit(f"{cls.__name__} does not implement the step interface this command drives")
    return cls.from_pretrained(model_dir, cfg, dtype=dtype, max_tokens=max_tokens, slots=slots, page_size=max(page_size, getattr(cls, "min_page_size", 1)),
                               max_step_tokens=max_step_tokens, build=True)


def cmd_generate(a) -> int:
    from .scheduler import Request, SamplingParams, Scheduler
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids]
    need = sum(len(p) + a.max_new_tokens + a.page_size for p in prompts)
    model = load_model(a.model, a.dtype, a.max_tokens or need, a.slots, a.page_size, a.max_step_tokens)
    sched = Scheduler(model, max_prefill_chunk=a.prefill_chunk or None)
    for i, p in enumerate(prompts):
        sched.add(Request(f"r{i}", p, a.max_new_tokens, SamplingParams(a.temperature, a.top_k, a.top_p, a.seed + i)))
    for r in sorted(sched.run(), key=lambda r: r.rid):
        print(json.dumps({"id": r.rid, "prompt_tokens": len(r.prompt), "output_ids": r.output}), flush=True)
    model.close()
    return 0


def cmd_trace(a) -> int:
    from .scheduler import execute
    model = load_model(a.model, a.dtype, a.max_tokens, a.slots, a.page_size, a.max_step_tokens)
    out = Path(a.out)
    slot_of = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries, want = [], []
        for ent in st.get("entries", []):
            rid = ent["id"]
            if rid not in slot_of:
                slot = model.admit()
                if slot < 0:
                    raise RuntimeError(f"no free state slot for request {rid!r}")
                slot_of[rid] = slot
            if not ent.get("tokens"):
                continue                                   # admitted, brings nothing in this step
            want.extend((len(entries), int(w)) for w in ent.get("want", []))
            entries.append((slot_of[rid], ent["tokens"]))
        if entries:
            rows = execute(model, entries, want, fetch=True)
            if want:
                rows.astype("<f4").tofile(out / f"{st['step']}.f32")
        for rid in st.get("end", []):
            if rid in slot_of:
                model.release(slot_of.pop(rid))
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    model.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="wf_bitnet.cli")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("generate", "trace"):
        p = sub.add_parser(name)
        p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
        p.add_argument("--max-tokens", type=int, default=0 if name == "generate" else 4096, help="cache pool size in tokens")
        p.add_argument("--slots", type=int, default=4, help="sequences alive at once")
        p.add_argument("--page-size", type=int, default=16)
        p.add_argument("--max-step-tokens", type=int, default=1024 if name == "generate" else 4096, help="most tokens in one engine step (larger batches are cut)")
        if name == "generate":
            p.add_argument("--prompt-ids", action="append", required=True, help="comma-separated token ids; repeat for several requests")
            p.add_argument("--max-new-tokens", type=int, default=16)
            p.add_argument("--temperature", type=float, default=0.0)
            p.add_argument("--top-k", type=int, default=0)
            p.add_argument("--top-p", type=float, default=1.0)
            p.add_argument("--seed", type=int, default=0)
            p.add_argument("--prefill-chunk", type=int, default=0)
        else:
            p.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    return cmd_generate(a) if a.cmd == "generate" else cmd_trace(a)


if __name__ == "__main__":
    sys.exit(main())
