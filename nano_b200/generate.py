"""Token-level generation from the command line, for models without a tokenizer section (model folders) and for model files alike:

    python -m nano_b200.generate --model DIR_OR_FILE --prompt-ids 5,17,3 --max-new 32 [--temperature 0.8 --top-p 0.9 --seed 1]
                                 [--repetition-penalty 1.1] [--dtype float32] [--max-tokens 4096]

Greedy (temperature 0) runs the engine's device-resident loop (nb200_decode_greedy) unless a repetition penalty asks for the
per-token path; sampling draws its coins on the host (xorshift, as the session loop of the reference host does) and samples on the
device (nb200_next_sampled).  Prints the ids, one line.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", required=True, help="comma-separated token ids")
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="model folders: compute type")
    ap.add_argument("--max-tokens", type=int, default=0, help="cache capacity (default: prompt + max-new)")
    a = ap.parse_args(argv)
    from . import build as nb_build, engine as E
    if os.path.isdir(a.model) and not os.path.exists(nb_build.ENGINE_SO):
        nb_build.build_layered()
    prompt = [int(x) for x in a.prompt_ids.split(",") if x.strip()]
    total = len(prompt) + a.max_new
    eng = E.Engine(a.model, max(a.max_tokens, total + 1), flags=E.FLAG_F32 if (a.dtype == "float32" and os.path.isdir(a.model)) else 0)
    ids = np.zeros(total + 1, np.uint32); ids[:len(prompt)] = prompt
    if a.temperature <= 0.0 and a.repetition_penalty == 1.0:
        eng.decode_greedy(ids, len(prompt), total)
    else:
        state = np.uint64(a.seed or 1)

        def coin():                                   # xorshift64* -> [0, 1)
            nonlocal state
            x = int(state); x ^= x >> 12; x ^= (x << 25) & 0xFFFFFFFFFFFFFFFF; x ^= x >> 27
            state = np.uint64(x)
            return ((x * 0x2545F4914F6CDD1D & 0xFFFFFFFFFFFFFFFF) >> 40) / 16777216.0
        for pos in range(total - 1):
            if pos < len(prompt) - 1:
                eng.next_greedy(ids, pos, 1)
            elif a.temperature <= 0.0:
                ids[pos + 1] = eng.next_greedy(ids, pos, 0, a.repetition_penalty)
            else:
                ids[pos + 1] = eng.next_sampled(ids, pos, a.repetition_penalty, a.temperature, a.top_p, coin())[0]
    print(" ".join(str(int(x)) for x in ids[:total]))
    eng.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
