"""Trace replay: feeds given token ids through a model step by step and writes the logits of the requested positions.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl

Each input line is one step: {"step": n, "entries": [{"id": ..., "tokens": [...], "want": [...]}], "end": [ids]}.
An entry continues its request from the state the earlier steps left (the framework's inference-state holders, one set per
live request); "want" lists the positions among the entry's tokens whose logits go to DIR/<n>.f32 (little-endian fp32,
[wanted, vocab], entries in order); "end" releases the requests' states.  After every step the line "done <n>" is printed.
Nothing is sampled.  The model class is chosen by the folder's config.json; the model call is the one the generation loop
makes: model(ids, inference_params_dict=state) with state["mha"].seqlen_offset set to the request's length so far.
Exit code 3: the model class cannot run in the requested dtype."""
from __future__ import annotations

import argparse
import json
import os
import sys

_DTYPES = {"bfloat16": "bfloat16", "float32": "float32"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="replay a trace of token steps through a model and write the requested logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=sorted(_DTYPES))
    ap.add_argument("--out", required=True, help="folder for <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=8192, help="most tokens live requests hold at any time (sizes the caches)")
    ap.add_argument("--device", default="cuda:0")
    a = ap.parse_args(argv)

    import torch
    from . import build as _build
    from .models import ARCHITECTURES, load_model_dir, read_architecture

    dtype = getattr(torch, _DTYPES[a.dtype])
    arch, _ = read_architecture(a.model)
    if dtype not in ARCHITECTURES[arch][1]:
        sys.stderr.write(f"{arch} does not run in {a.dtype}\n")
        return 3
    _build.build()                                  # compiles the CUDA library on the first call of a fresh checkout
    model = load_model_dir(a.model, device=a.device, dtype=dtype)
    os.makedirs(a.out, exist_ok=True)
    live = {}                                       # request id -> [state, tokens so far]
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        chunks = []
        for e in step.get("entries", []):
            rid, tokens, want = e["id"], e["tokens"], e.get("want", [])
            if rid not in live:
                live[rid] = [model.initialize_inference_params(max_seqlen=max(a.max_tokens, len(tokens)), max_batch_size=1), 0]
            state, done = live[rid]
            if not tokens:
                continue
            state["mha"].seqlen_offset = state["hyena"].seqlen_offset = done
            ids = torch.tensor([tokens], dtype=torch.long, device=a.device)
            logits, _ = model(ids, inference_params_dict=state, logits_rows=list(want))
            live[rid][1] = done + len(tokens)
            if want:
                chunks.append(logits.float().cpu())
        if chunks:
            data = torch.cat(chunks, 0).contiguous().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{step['step']}.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in step.get("end", []):
            live.pop(rid, None)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
