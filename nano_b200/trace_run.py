"""Trace replay: feeds given token ids through a model folder, step by step, and writes logits.  Nothing is sampled.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}

Every entry gives a request's NEXT tokens (a request is opened the first time its id appears) and the places among them whose logits
are wanted.  They run through the engine's own step function (nano_b200.engine.Engine.step -> nb200_step): a portion of several
tokens takes the prefill kernels, a single token the decode kernels, from the cache pages and the state slot the request holds.
Requests named in "end" give their pages and slot back after the step.  For a step with wanted places the file OUT/<step>.f32
receives the logits, little-endian fp32 [wanted, vocab], in the order of the entries and of "want"; after every step the line
"done <step>" is printed.  The runner ends with 0 when its input ends.

--dtype bfloat16 keeps the stored bfloat16 weights (tensor-core products with fp32 accumulation; residual stream, norms, router,
attention weights and recurrences in fp32); --dtype float32 widens the weights and computes everything with fp32 FMAs.

In a checkout without built libraries the first call compiles the units a model folder needs (nano_b200.build.build_layered).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, default=4096, help="tokens all live requests may hold together (sizes the cache)")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args(argv)

    from . import build as nb_build
    if not os.path.exists(os.environ.get("NB200_ENGINE_SO", nb_build.ENGINE_SO)):
        nb_build.build_layered()
    from . import engine as E

    eng = E.Engine(a.model, max(1, a.max_tokens), device=a.device, flags=E.FLAG_F32 if a.dtype == "float32" else 0)
    os.makedirs(a.out, exist_ok=True)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        rows = []
        for ent in step.get("entries", []):
            rid = ent["id"]
            if rid not in live:
                live[rid] = eng.seq_open()
            toks = ent.get("tokens", [])
            want = list(ent.get("want", []))
            if not toks:
                continue
            order = np.argsort(np.asarray(want, np.int64), kind="stable") if want else np.zeros(0, np.int64)
            got = eng.step(live[rid], toks, sorted(want))
            if want:
                back = np.empty_like(order)
                back[order] = np.arange(order.size)
                rows.append(got[back])            # in the order "want" lists them
        for rid in step.get("end", []):
            if rid in live:
                eng.seq_close(live.pop(rid))
        if rows:
            tmp = os.path.join(a.out, ".%s.part" % step["step"])
            np.concatenate(rows, axis=0).astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(a.out, "%s.f32" % step["step"]))
        sys.stdout.write("done %s\n" % step["step"])
        sys.stdout.flush()
    eng.close()
    return 0
