"""Trace replay: feeds given token ids through a model step by step and writes logits; samples nothing.

The model is chosen from config.json by model/registry.py; the steps run through serving.StepScheduler.run_step - the same
packed step, page pool and slots that generation uses. Standard input carries one JSON object per line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

entries: per request its next tokens and the offsets among them whose logits are wanted; all entries of a step are one batch; a
request is admitted at its first entry and may skip steps. end: requests finished after this step (their pages and slot are
freed). For a step with wanted rows the file OUT/<step>.f32 receives [wanted, vocab] little-endian fp32 logits in the order of
the entries; after every step "done <step>" is printed and flushed. Exit code 0 at the end of input; 3 if the model has no
implementation in the requested dtype.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16", help="compute dtype")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to whole pages): size of the cache pool")
    ap.add_argument("--slots", type=int, default=4, help="requests live at the same time")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    import torch
    from .model import registry
    from .serving import StepScheduler
    dtype = getattr(torch, a.dtype)
    cfg = registry.read_config(a.model)
    cls = registry.model_class_for(cfg)
    if not hasattr(cls, "step"):
        print(f"{cls.__name__} has no packed step(): it cannot replay a trace", file=sys.stderr)
        return 3
    try:
        model = registry.load_model(a.model, device=a.device, dtype=dtype)
    except ValueError as e:   # a model without this compute dtype
        print(str(e), file=sys.stderr)
        return 3
    sched = StepScheduler(model, max_tokens=a.max_tokens, slots=a.slots)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want", [])) for e in st["entries"]]
        logits = sched.run_step(entries, st.get("end", []))
        if logits is not None:
            data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
            tmp = os.path.join(a.out, f".{st['step']}.f32.part")
            with open(tmp, "wb") as fh:
                fh.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{st['step']}.f32"))
        else:
            torch.cuda.synchronize()
        print(f"done {st['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
