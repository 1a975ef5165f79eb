"""Rakarax on the layered runtime against the plain restatement in tests/rakarax_oracle.py: every mechanism alone, prefill against
token-by-token decoding, portions of several sizes, interleaved requests, pages and slots used again, window edges and page
borders, far tokens carried by the recurrent states, the first tokens of a sequence, long decoding, sizes that defeat every vector
width, and greedy generation through the engine's own entry points.  Small random models, each written to a temporary folder and
loaded by the engine like any model folder."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md

from rakarax_oracle import forward as oracle_forward

pytestmark = pytest.mark.gpu

RET = {"heads": 3, "dim": 24, "vdim": 40, "decay": [0.9, 0.97, 0.995], "rot": {"dims": 16, "base": 10000.0}}
LEFT = {"heads": 6, "kv_heads": 2, "dim": 20, "vdim": 20, "conv": 3, "scale": 0.3, "softcap": 15.0, "mask": {"size": 13}}
RIGHT = {"inner": 48, "state": 10, "dt_rank": 5, "conv": 4}
PAR = {"left": LEFT, "right": RIGHT, "left_scale": 0.7, "right_scale": 1.2}


def par(left=None, right=None, ls=0.7, rs=1.2):
    a, b = dict(LEFT), dict(RIGHT)
    a.update(left or {}); b.update(right or {})
    for k in [k for k, v in a.items() if v is None]:
        del a[k]
    return {"left": a, "right": b, "left_scale": ls, "right_scale": rs}


def build(tmp_path, cfg, seed=0, f32=True, max_tokens=512, keep=False, chunk=None, name="m", tweak=None):
    w = md.rakarax_random(cfg, seed)
    if tweak:
        tweak(w)
    path = md.write_model_dir(str(tmp_path / name), cfg, w)
    os.environ.pop("NB200_KEEP_RESIDUALS", None); os.environ.pop("NB200_CHUNK", None)
    if keep: os.environ["NB200_KEEP_RESIDUALS"] = "1"
    if chunk: os.environ["NB200_CHUNK"] = str(chunk)
    try:
        eng = E.Engine(path, max_tokens, flags=E.FLAG_F32 if f32 else 0)
    finally:
        os.environ.pop("NB200_KEEP_RESIDUALS", None); os.environ.pop("NB200_CHUNK", None)
    return eng, w


def toks(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).astype(np.uint32)


def rows(got, want):
    """rms of the difference over the rms of the reference, per row (mean taken off: logits are shift-invariant)"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1) + 1e-30)


def rel(got, want):
    return float(rows(got, want).max())


F32_TOL, BF16_TOL = 3e-5, 4e-2


def whole(eng, t, want=None):
    s = eng.seq_open()
    out = eng.step(s, t, range(len(t)) if want is None else want)
    eng.seq_close(s)
    return out


def in_cuts(eng, t, cuts):
    s = eng.seq_open()
    out, at = [], 0
    for c in cuts:
        part = t[at:at + c]
        if len(part):
            out.append(eng.step(s, part, range(len(part))))
        at += c
    eng.seq_close(s)
    assert at >= len(t)
    return np.concatenate(out)


MIXERS = [
    ("retention", RET),
    ("retention", {"heads": 1, "dim": 8, "vdim": 8, "decay": [1.0], "rot": {"dims": 8, "base": 100.0}}),            # every coordinate turns, no decay
    ("retention", {"heads": 2, "dim": 70, "vdim": 33, "decay": [0.5, 0.99], "rot": {"dims": 2, "base": 7.0}}),       # one pair turns; odd sizes
    ("retention", {"heads": 5, "dim": 36, "vdim": 12, "decay": [0.9, 0.8, 0.99, 0.999, 0.7], "rot": None}),          # no rotation at all
    ("retention", {"heads": 2, "dim": 130, "vdim": 16, "decay": [0.95, 0.99], "rot": {"dims": 64, "base": 1e6}}),
    ("parallel", PAR),
    ("parallel", par({"heads": 4, "kv_heads": 4, "dim": 16, "vdim": 16, "conv": 1, "mask": {"size": 1}}, {"conv": 1, "state": 1, "dt_rank": 1})),
    ("parallel", par({"heads": 3, "kv_heads": 1, "dim": 37, "vdim": 37, "conv": 2, "mask": {"size": 40}, "softcap": None}, {"inner": 50, "state": 24, "dt_rank": 7, "conv": 2})),
    ("parallel", par({"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "mask": None}, {"inner": 20, "state": 33, "dt_rank": 3})),      # no window
    ("parallel", par({"heads": 20, "kv_heads": 5, "dim": 12, "vdim": 12, "mask": {"size": 33}}, {"state": 70})),                     # two heads per warp
    ("parallel", par({"heads": 2, "kv_heads": 2, "dim": 132, "vdim": 132, "mask": {"size": 32}}, {"state": 130 - 2}, ls=0.0, rs=2.0)),
    ("parallel", par({"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "mask": {"size": 64}, "scale": 0.125}, {"state": 16}, ls=1.0, rs=0.0)),
]


# ---- each mechanism alone: one layer, no feed-forward, residual after the layer and logits; whole, token by token, short portions ----
@pytest.mark.parametrize("kind,mixer", MIXERS)
def test_mixer_alone(tmp_path, kind, mixer):
    cfg = md.rakarax_config(61, 72, [(kind, mixer, None)], max_positions=96)
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 75)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    res = eng.read_residual(0, len(t))
    assert np.abs(res - trace[0]).max() <= 3e-5 * np.abs(trace[0]).max()
    assert rel(got, ref) < F32_TOL
    for cuts in ([1] * 75, [2, 3, 4] * 9, [5, 1, 30, 2, 37]):
        assert rel(in_cuts(eng, t, cuts), ref) < F32_TOL, cuts[:3]
    eng.close()


@pytest.mark.parametrize("ff", [40, 7, 129])
def test_feed_forward(tmp_path, ff):
    cfg = md.rakarax_config(50, 64, [("retention", RET, ff)], max_positions=64)
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 50)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert np.abs(eng.read_residual(0, len(t)) - trace[0]).max() <= 3e-5 * np.abs(trace[0]).max()
    assert rel(in_cuts(eng, t[:20], [1] * 20), ref[:20]) < F32_TOL
    eng.close()


def mixed_cfg(vocab=97, width=72, max_positions=700, window=13):
    p2 = par({"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 4, "mask": {"size": window}}, {"inner": 40, "state": 8, "dt_rank": 4, "conv": 3})
    return md.rakarax_config(vocab, width, [("parallel", PAR, 40), ("retention", RET, 56), ("parallel", PAR, 40, 0), ("parallel", p2, None),
                                            ("retention", RET, 56, 1), ("retention", {"heads": 2, "dim": 32, "vdim": 32, "decay": [0.99, 0.999], "rot": {"dims": 32, "base": 1e4}}, 24)],
                             max_positions=max_positions)


def test_layer_order_and_shared_weights(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 60)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    for r, x in enumerate(trace):
        assert np.abs(eng.read_residual(r, len(t)) - x).max() <= 4e-5 * np.abs(x).max(), f"layer run {r}"
    assert rel(got, ref) < F32_TOL
    eng.close()


# ---- prefill against token-by-token decoding, portions down to two tokens, the engine's own chunking ----
@pytest.mark.parametrize("f32", [True, False])
def test_portions_and_decoding(tmp_path, f32):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=f32)
    t = toks(cfg, 150)
    ref = oracle_forward(cfg, w, t, np.float64)
    tol = F32_TOL if f32 else BF16_TOL
    full = whole(eng, t)
    assert rel(full, ref) < tol
    for cuts in ([1] * 150, [2] * 75, [3, 2, 64, 5, 1, 1, 33, 2, 39], [100] + [1] * 50, [31, 1, 32, 33, 53], [7] * 22):
        got = in_cuts(eng, t, cuts)
        assert rel(got, ref) < tol, cuts[:4]
        assert rel(got, full) < (F32_TOL if f32 else BF16_TOL)
    eng.close()
    eng, _ = build(tmp_path, cfg, f32=f32, chunk=16, name="c")       # chunks of 16 inside one step
    assert rel(whole(eng, t), ref) < tol
    eng.close()


def test_batches_of_unequal_requests_and_reuse(tmp_path):
    """Requests interleaved step by step equal each alone; pages and slots that were freed hold other requests' numbers."""
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, max_tokens=400)
    ts = [toks(cfg, n, seed=10 + n) for n in (90, 33, 140, 5)]
    refs = [oracle_forward(cfg, w, t, np.float64) for t in ts]
    free0 = eng.free_pages
    for rounds in range(2):                      # the second round runs in pages and slots of the first
        seqs = [eng.seq_open() for _ in ts]
        outs, at = [[] for _ in ts], [0] * len(ts)
        sizes = [[40, 1, 1, 48], [2, 31], [64, 64, 3, 1, 1, 1, 6], [5]]
        step = 0
        while any(a < len(t) for a, t in zip(at, ts)):
            for i, t in enumerate(ts):
                if at[i] >= len(t) or step >= len(sizes[i]):
                    continue
                n = sizes[i][step]
                outs[i].append(eng.step(seqs[i], t[at[i]:at[i] + n], range(n)))
                at[i] += n
                if at[i] == len(t):
                    eng.seq_close(seqs[i])
            step += 1
        for o, r in zip(outs, refs):
            assert rel(np.concatenate(o), r) < F32_TOL
        assert eng.free_pages == free0
    eng.close()


# ---- the window's edge, where random weights would hide it: sharp scores, one key that stands out ----
@pytest.mark.parametrize("window", [5, 32, 33, 45])
def test_window_edge_shows(tmp_path, window):
    """One token's key is made huge for one head, so a query that still sees it differs visibly from one that just lost it."""
    mixer = par({"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "conv": 1, "scale": 1.0, "softcap": 30.0, "mask": {"size": window}}, ls=1.0, rs=0.05)
    cfg = md.rakarax_config(40, 48, [("parallel", mixer, None)], max_positions=200)
    eng, w = build(tmp_path, cfg)
    t = toks(cfg, 150, seed=3)
    ref = oracle_forward(cfg, w, t, np.float64)
    wider = copy.deepcopy(cfg); wider["layers"][0]["mixer"]["left"]["mask"]["size"] = window + 1
    narrower = copy.deepcopy(cfg); narrower["layers"][0]["mixer"]["left"]["mask"]["size"] = max(1, window - 1)
    off_by_one = min(rel(oracle_forward(wider, w, t, np.float64), ref), rel(oracle_forward(narrower, w, t, np.float64), ref) if window > 1 else 1.0)
    assert off_by_one > 100 * F32_TOL                # the oracle itself tells the sizes apart
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [100] + [1] * 50), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [29, 2, 2, 31, 1, 1, 64, 20]), ref) < F32_TOL
    eng.close()


@pytest.mark.parametrize("window", [150, None])
def test_wide_window_decoding_splits_keys(tmp_path, window):
    """Short portions deal a wide window's key pages out to several blocks and merge: same logits as the whole prompt."""
    mixer = par({"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 24, "conv": 2, "scale": 0.8, "mask": {"size": window} if window else None}, ls=1.0, rs=0.3)
    cfg = md.rakarax_config(40, 48, [("parallel", mixer, 24), ("parallel", mixer, 24, 0)], max_positions=400)
    eng, w = build(tmp_path, cfg, max_tokens=400)
    t = toks(cfg, 330, seed=6)
    ref = oracle_forward(cfg, w, t, np.float64)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [140] + [1] * 60 + [2, 3, 4, 1] * 13), ref) < F32_TOL
    eng.close()


def test_far_tokens_through_the_states(tmp_path):
    """A slow decay and a slow scan carry the first tokens over hundreds of positions: changing token 0 changes the last logits."""
    ret = {"heads": 2, "dim": 16, "vdim": 16, "decay": [0.9999, 1.0], "rot": {"dims": 16, "base": 1e4}}
    mixer = par({"mask": {"size": 8}}, {"inner": 32, "state": 4, "dt_rank": 2})

    def slow(w):
        w["l1.mix.right.dt.b"] = np.full_like(w["l1.mix.right.dt.b"], -6.0)
        w["l1.mix.right.A_log"] = np.full_like(w["l1.mix.right.A_log"], -3.0)
    cfg = md.rakarax_config(40, 48, [("retention", ret, None), ("parallel", mixer, 32)], max_positions=640)
    eng, w = build(tmp_path, cfg, max_tokens=640, tweak=slow)
    t = toks(cfg, 600, seed=5)
    ref = oracle_forward(cfg, w, t, np.float64)
    t2 = t.copy(); t2[0] = (t2[0] + 1) % cfg["vocab"]
    assert rel(oracle_forward(cfg, w, t2, np.float64)[-20:], ref[-20:]) > 100 * F32_TOL
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(in_cuts(eng, t, [560] + [1] * 40)[-60:], ref[-60:]) < F32_TOL
    eng.close()


def test_long_decoding(tmp_path):
    cfg = mixed_cfg(max_positions=700, window=45)
    eng, w = build(tmp_path, cfg, max_tokens=700)
    t = toks(cfg, 650, seed=8)
    ref = oracle_forward(cfg, w, t, np.float64)
    got = in_cuts(eng, t, [3] + [1] * 647)
    assert rel(got, ref) < 2 * F32_TOL
    eng.close()


def test_first_tokens_and_single_token_requests(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg)
    for n in (1, 2, 3, 5):
        t = toks(cfg, n, seed=20 + n)
        ref = oracle_forward(cfg, w, t, np.float64)
        assert rel(whole(eng, t), ref) < F32_TOL
        assert rel(in_cuts(eng, t, [1] * n), ref) < F32_TOL
    eng.close()


def test_bf16_close_to_oracle(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=False)
    t = toks(cfg, 120)
    ref = oracle_forward(cfg, w, t, np.float64)
    r = rows(whole(eng, t), ref)
    assert r.max() < BF16_TOL and np.median(r) < BF16_TOL / 3
    eng.close()


# ---- generation through the engine's own entry points ----
def test_greedy_generation(tmp_path):
    cfg = mixed_cfg(vocab=53)
    eng, w = build(tmp_path, cfg)
    prompt = toks(cfg, 17, seed=4)
    total = 60
    ids = np.zeros(total + 1, np.uint32); ids[:17] = prompt
    eng.decode_greedy(ids, 17, total)
    # the oracle follows the engine's ids and must agree on every choice whose margin is not a rounding matter
    ref = oracle_forward(cfg, w, ids[:total - 1], np.float64)
    for pos in range(16, total - 1):
        top = np.sort(ref[pos])[-2:]
        if top[1] - top[0] > 1e-3:
            assert int(np.argmax(ref[pos])) == int(ids[pos + 1]), pos
    ids2 = np.zeros(total + 1, np.uint32); ids2[:17] = prompt
    for pos in range(total - 1):
        nxt = eng.next_greedy(ids2, pos, 1 if pos < 16 else 0)
        if pos >= 16:
            ids2[pos + 1] = nxt
    assert np.array_equal(ids[:total], ids2[:total])
    eng.close()
    # the generation command on the same folder
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, "-m", "nano_b200.generate", "--model", str(tmp_path / "m"), "--prompt-ids", ",".join(str(int(x)) for x in prompt),
                        "--max-new", str(total - 17), "--dtype", "float32"], cwd=root, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(x) for x in p.stdout.split()] == [int(x) for x in ids[:total]]


def test_position_limit_is_refused(tmp_path):
    cfg = md.rakarax_config(30, 32, [("retention", {"heads": 1, "dim": 8, "vdim": 8, "decay": [0.9], "rot": {"dims": 8, "base": 100.0}}, None)], max_positions=16)
    eng, _ = build(tmp_path, cfg, max_tokens=64)
    s = eng.seq_open()
    eng.step(s, toks(cfg, 16), [15])
    with pytest.raises(E.NB200Error):
        eng.step(s, toks(cfg, 1), [0])
    eng.seq_close(s)
    eng.close()


def test_replay_command(tmp_path):
    """bin/trace_run on a Rakarax folder: portions, single tokens, a step that wants nothing, two requests one after the other."""
    cfg = mixed_cfg()
    w = md.rakarax_random(cfg, 2)
    path = md.write_model_dir(str(tmp_path / "m"), cfg, w)
    a, b = toks(cfg, 70, seed=1), toks(cfg, 9, seed=2)
    ra, rb = oracle_forward(cfg, w, a, np.float64), oracle_forward(cfg, w, b, np.float64)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40].tolist(), "want": [39, 3]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[40:42].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[42:43].tolist(), "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[43:70].tolist(), "want": [26]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": b.tolist(), "want": [8]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == ["done %d" % i for i in range(5)]
        V = cfg["vocab"]
        g0 = np.fromfile(out / "0.f32", "<f4").reshape(-1, V)
        assert rel(g0, ra[[39, 3]]) < tol
        assert not (out / "1.f32").exists()
        assert rel(np.fromfile(out / "2.f32", "<f4").reshape(-1, V), ra[[42]]) < tol
        assert rel(np.fromfile(out / "3.f32", "<f4").reshape(-1, V), ra[[69]]) < tol
        assert rel(np.fromfile(out / "4.f32", "<f4").reshape(-1, V), rb[[8]]) < tol
