"""Famudra on the layered runtime against the plain restatement in tests/famudra_oracle.py: every mechanism alone, prefill against
token-by-token decoding, portions of several sizes, interleaved requests, pages and slots used again, sharp attention over far keys and
page borders, ragged sizes, long decoding, and greedy generation through the engine's own entry points.  Small random models, each
written to a temporary folder and loaded by the engine like any model folder."""
import os

import numpy as np
import pytest

from nano_b200 import engine as E, modeldir as md

from famudra_oracle import forward as oracle_forward

pytestmark = pytest.mark.gpu

ATT = {"heads": 3, "dim": 24, "vdim": 40, "kv_rank": 48, "q_rank": 56, "scale": 0.25}
REC = {"width": 96, "blocks": 3, "conv": 4}
MOE = {"experts": 5, "top": 2, "ff": 40, "shared_ff": 24}


def build(tmp_path, cfg, seed=0, f32=True, max_tokens=512, keep=False, chunk=None, name="m"):
    w = md.famudra_random(cfg, seed)
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


def rel(got, want):
    """rms of the difference over the rms of the reference, per row (mean taken off: logits are shift-invariant)"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1) + 1e-30)).max())


F32_TOL, BF16_TOL = 2e-5, 4e-2


def rows(got, want):
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1) + 1e-30)


def close(got, want, f32):
    """fp32: every row within rounding.  bf16: operand rounding may flip a router's close call at a token or two (another expert is a
    legitimately different answer there), so up to 3 % of the rows may be off while the rest stay within bf16 rounding."""
    r = rows(got, want)
    return bool(r.max() < F32_TOL) if f32 else bool((r < BF16_TOL).mean() >= 0.97 and np.median(r) < BF16_TOL / 4)


def whole(eng, t, want=None):
    s = eng.seq_open()
    out = eng.step(s, t, range(len(t)) if want is None else want)
    eng.seq_close(s)
    return out


# ---- each mechanism alone: one layer, no feed-forward, residual after the layer and logits ----
@pytest.mark.parametrize("kind,mixer", [("rglru", REC), ("rglru", {"width": 64, "blocks": 1, "conv": 1}), ("rglru", {"width": 80, "blocks": 5, "conv": 2}),
                                        ("latent_attention", ATT), ("latent_attention", {"heads": 1, "dim": 16, "vdim": 8, "kv_rank": 20, "q_rank": 12, "scale": 0.5}),
                                        ("latent_attention", {"heads": 10, "dim": 8, "vdim": 8, "kv_rank": 96, "q_rank": 32, "scale": 0.3}),
                                        # latent ranks of 64 / 128 / 256 take the attention kernel's compile-time-rank instances
                                        ("latent_attention", {"heads": 4, "dim": 8, "vdim": 12, "kv_rank": 64, "q_rank": 24, "scale": 0.4}),
                                        ("latent_attention", {"heads": 9, "dim": 12, "vdim": 8, "kv_rank": 128, "q_rank": 20, "scale": 0.3}),
                                        ("latent_attention", {"heads": 2, "dim": 8, "vdim": 8, "kv_rank": 256, "q_rank": 16, "scale": 0.2}),
                                        # the widest register tile: a general rank above 256 and the constant 512
                                        ("latent_attention", {"heads": 3, "dim": 8, "vdim": 8, "kv_rank": 330, "q_rank": 16, "scale": 0.2}),
                                        ("latent_attention", {"heads": 2, "dim": 8, "vdim": 8, "kv_rank": 512, "q_rank": 16, "scale": 0.15})])
def test_mixer_alone(tmp_path, kind, mixer):
    cfg = md.famudra_config(61, 72, [(kind, mixer, None)])
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 45)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    res = eng.read_residual(0, len(t))
    assert np.abs(res - trace[0]).max() <= 2e-5 * np.abs(trace[0]).max()
    assert rel(got, ref) < F32_TOL
    for cuts in ([1] * 45, [2, 3, 4] * 5):                  # the short-portion kernels of the same mechanism
        s = eng.seq_open()
        out, at = [], 0
        for c in cuts:
            out.append(eng.step(s, t[at:at + c], range(c)))
            at += c
        eng.seq_close(s)
        assert rel(np.concatenate(out), ref) < F32_TOL, cuts[:3]
    eng.close()


@pytest.mark.parametrize("mlp", [MOE, {"experts": 4, "top": 1, "ff": 24, "shared_ff": None}, {"experts": 3, "top": 3, "ff": 16, "shared_ff": 50},
                                 {"experts": 16, "top": 4, "ff": 8, "shared_ff": 8}])
def test_feed_forward_with_router(tmp_path, mlp):
    cfg = md.famudra_config(50, 64, [("rglru", {"width": 32, "blocks": 2, "conv": 3}, mlp)])
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 70)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    assert np.abs(eng.read_residual(0, len(t)) - trace[0]).max() <= 2e-5 * np.abs(trace[0]).max()
    assert rel(got, ref) < F32_TOL
    # the decode kernels take the same routes
    s = eng.seq_open()
    one = np.concatenate([eng.step(s, t[i:i + 1], [0]) for i in range(20)])
    eng.seq_close(s)
    assert rel(one, ref[:20]) < F32_TOL
    eng.close()


def mixed_cfg(loop=(1, 3, 2), vocab=97, width=72):
    return md.famudra_config(vocab, width, [("rglru", REC, MOE), ("latent_attention", ATT, MOE), ("rglru", {"width": 48, "blocks": 2, "conv": 3}, None),
                                            ("latent_attention", {"heads": 2, "dim": 16, "vdim": 24, "kv_rank": 40, "q_rank": 24, "scale": 0.4}, {"experts": 3, "top": 1, "ff": 32, "shared_ff": None})],
                             loop=loop)


@pytest.mark.parametrize("loop", [None, (0, 4, 1), (1, 3, 2), (0, 4, 3), (2, 4, 2), (3, 3, 5)])
def test_layer_order_and_passes(tmp_path, loop):
    cfg = mixed_cfg(loop)
    eng, w = build(tmp_path, cfg, keep=True)
    t = toks(cfg, 40)
    trace = []
    ref = oracle_forward(cfg, w, t, np.float64, trace)
    got = whole(eng, t)
    for r, x in enumerate(trace):
        assert np.abs(eng.read_residual(r, len(t)) - x).max() <= 3e-5 * np.abs(x).max(), f"layer run {r}"
    assert rel(got, ref) < F32_TOL
    eng.close()


# ---- prefill against token-by-token decoding, portions down to two tokens, the first tokens of a sequence ----
@pytest.mark.parametrize("f32", [True, False])
def test_portions_and_decode_agree(tmp_path, f32):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, f32=f32)
    n = 150
    t = toks(cfg, n, 3)
    ref = oracle_forward(cfg, w, t, np.float64)
    assert close(whole(eng, t), ref, f32)
    for cuts in ([1] * n, [2] * (n // 2), [3, 2, 5, 4, 7, 1, 1, 31, 32, 33, 2, 29], [64, 64, 22], [33, 1, 1, 1, 62, 2, 2, 48]):
        s = eng.seq_open()
        out, at = [], 0
        for c in cuts:
            out.append(eng.step(s, t[at:at + c], range(c)))
            at += c
        eng.seq_close(s)
        got = np.concatenate(out)
        assert close(got, ref[:at], f32), cuts[:4]
        assert rel(got[:4], ref[:4]) < (F32_TOL if f32 else BF16_TOL)       # the first tokens: empty cache, zero state, zero convolution tail
    eng.close()


def test_engine_chunks_long_portions(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, chunk=16)
    t = toks(cfg, 100, 5)
    ref = oracle_forward(cfg, w, t, np.float64)
    assert rel(whole(eng, t), ref) < F32_TOL
    assert rel(whole(eng, t, [0, 15, 16, 17, 63, 64, 99]), ref[[0, 15, 16, 17, 63, 64, 99]]) < F32_TOL
    eng.close()


# ---- requests side by side, pages and slots used again ----
def test_interleaved_requests_and_reuse(tmp_path):
    cfg = mixed_cfg()
    eng, w = build(tmp_path, cfg, max_tokens=400)
    free0 = eng.free_pages
    ta, tb, tc = toks(cfg, 90, 7), toks(cfg, 41, 8), toks(cfg, 130, 9)
    ra, rb, rc = (oracle_forward(cfg, w, x, np.float64) for x in (ta, tb, tc))
    a, b = eng.seq_open(), eng.seq_open()
    ga = [eng.step(a, ta[:30], range(30))]
    gb = [eng.step(b, tb[:5], range(5))]
    ga.append(eng.step(a, ta[30:31], [0]))
    gb.append(eng.step(b, tb[5:41], range(36)))
    eng.seq_close(b)                                   # b's pages and slot go back while a lives on
    c = eng.seq_open()                                 # ... and c gets them, with b's old contents in them
    gc = [eng.step(c, tc[:70], range(70))]
    ga.append(eng.step(a, ta[31:90], range(59)))
    gc.append(eng.step(c, tc[70:130], range(60)))
    eng.seq_close(a); eng.seq_close(c)
    assert rel(np.concatenate(ga), ra) < F32_TOL
    assert rel(np.concatenate(gb), rb) < F32_TOL
    assert rel(np.concatenate(gc), rc) < F32_TOL
    assert eng.free_pages == free0
    for _ in range(3):                                 # the same slot and pages again and again
        assert rel(whole(eng, tb), rb) < F32_TOL
    assert eng.free_pages == free0
    with pytest.raises(E.NB200Error, match="cache is full"):
        s = eng.seq_open()
        try:
            eng.step(s, toks(cfg, 400, 1), []); eng.step(s, toks(cfg, 400, 2), [])
        finally:
            eng.seq_close(s)
    assert eng.free_pages == free0
    eng.close()


# ---- sharp attention: a single far key carries the output, in prompts and in decoding, across page borders ----
def test_far_keys_and_page_borders(tmp_path):
    att = {"heads": 2, "dim": 16, "vdim": 16, "kv_rank": 24, "q_rank": 16, "scale": 6.0}     # scores spread over tens of units
    cfg = md.famudra_config(40, 48, [("latent_attention", att, None), ("latent_attention", dict(att, heads=4, scale=9.0), None)])
    eng, w = build(tmp_path, cfg, max_tokens=700)
    n = 420
    t = toks(cfg, n, 11)
    t[0], t[31], t[32], t[63], t[64] = 39, 38, 37, 36, 35     # rare ids at the edges of the first pages
    t[1:31][t[1:31] >= 35] = 3; t[65:][t[65:] >= 35] = 5
    t[300:310] = [39, 38, 37, 36, 35, 39, 38, 37, 36, 35]     # far queries that match those keys
    ref = oracle_forward(cfg, w, t, np.float64)
    assert rel(whole(eng, t), ref) < 5e-5
    s = eng.seq_open()
    out = [eng.step(s, t[:290], range(290))]
    for i in range(290, n):
        out.append(eng.step(s, t[i:i + 1], [0]))
    eng.seq_close(s)
    assert rel(np.concatenate(out), ref) < 5e-5
    # the far keys do matter: without the first page's tokens the logits at the matching queries change
    alt = t.copy(); alt[0], alt[31] = 1, 2
    assert rel(oracle_forward(cfg, w, alt, np.float64)[300:310], ref[300:310]) > 1e-2
    eng.close()


# ---- sizes that are no multiples of the kernels' vector widths ----
def test_ragged_sizes(tmp_path):
    cfg = md.famudra_config(33, 70, [("rglru", {"width": 54, "blocks": 6, "conv": 5}, {"experts": 7, "top": 3, "ff": 30, "shared_ff": 18}),
                                     ("latent_attention", {"heads": 5, "dim": 6, "vdim": 10, "kv_rank": 34, "q_rank": 22, "scale": 0.7}, {"experts": 2, "top": 2, "ff": 14, "shared_ff": None})],
                            loop=(0, 2, 2), eps=1e-3)
    for f32 in (True, False):
        eng, w = build(tmp_path, cfg, f32=f32, name=f"r{int(f32)}")
        t = toks(cfg, 75, 13)
        ref = oracle_forward(cfg, w, t, np.float64)
        assert close(whole(eng, t), ref, f32)
        s = eng.seq_open()
        got = np.concatenate([eng.step(s, t[:37], range(37)), eng.step(s, t[37:40], range(3))] + [eng.step(s, t[i:i + 1], [0]) for i in range(40, 75)])
        eng.seq_close(s)
        assert close(got, ref, f32)
        eng.close()


# ---- long decoding: the recurrent state and the cache carry over hundreds of single-token steps ----
def test_long_decoding(tmp_path):
    cfg = mixed_cfg(vocab=64)
    eng, w = build(tmp_path, cfg, max_tokens=700)
    t = toks(cfg, 600, 17)
    ref = oracle_forward(cfg, w, t, np.float64)
    s = eng.seq_open()
    eng.step(s, t[:3], [])
    got = np.concatenate([eng.step(s, t[i:i + 1], [0]) for i in range(3, 600)])
    eng.seq_close(s)
    assert rel(got, ref[3:]) < 5e-5
    eng.close()


# ---- generation through the engine's own entry points ----
def oracle_greedy(cfg, w, prompt, n_total):
    ids = list(prompt)
    while len(ids) < n_total:
        ids.append(int(np.argmax(oracle_forward(cfg, w, ids, np.float64)[-1])))
    return ids


def test_greedy_generation(tmp_path):
    cfg = mixed_cfg(vocab=80)
    eng, w = build(tmp_path, cfg)
    prompt, n_total = [5, 17, 3, 44, 9, 61, 2], 40
    want = oracle_greedy(cfg, w, prompt, n_total)
    ids = np.zeros(64, np.uint32); ids[:len(prompt)] = prompt
    eng.decode_greedy(ids, len(prompt), n_total)                  # device-resident loop
    assert ids[:n_total].tolist() == want
    ids2 = np.zeros(64, np.uint32); ids2[:len(prompt)] = prompt    # the per-token host API (what the session loop calls)
    for pos in range(n_total - 1):
        ids2[pos + 1] = eng.next_greedy(ids2, pos, 1 if pos < len(prompt) - 1 else 0)
    assert ids2[:n_total].tolist() == want
    ref = oracle_forward(cfg, w, want[:n_total - 1], np.float64)[-1]
    assert rel(eng.logits()[None], ref[None]) < F32_TOL
    ids3 = np.zeros(64, np.uint32); ids3[:len(prompt)] = prompt    # a host that jumps to the end of the prompt: the engine prefills the gap
    nxt = eng.next_greedy(ids3, 0, 1)
    nxt = eng.next_greedy(ids3, len(prompt) - 1, 0)
    assert nxt == want[len(prompt)]
    eng.close()


def test_sampled_generation_and_penalty(tmp_path):
    cfg = mixed_cfg(vocab=80)
    eng, w = build(tmp_path, cfg)
    prompt = [5, 17, 3, 44]
    ids = np.zeros(32, np.uint32); ids[:4] = prompt
    for pos in range(3):
        eng.next_greedy(ids, pos, 1)
    tok, top6 = eng.next_sampled(ids, 3, 1.0, 0.8, 0.95, 0.01)
    ref = oracle_forward(cfg, w, prompt, np.float64)[-1]
    assert top6[0] == int(np.argmax(ref)) and tok == top6[0]          # a coin near 0 takes the most probable token
    # repetition penalty: the greedy choice is the argmax of the penalised logits
    eng.forward(5, 0); eng.forward(17, 1)
    pen = oracle_forward(cfg, w, [5, 17, 3], np.float64)[-1].copy()
    for i in (5, 17):
        pen[i] = pen[i] / 50.0 if pen[i] > 0 else pen[i] * 50.0
    ids[:3] = [5, 17, 3]
    assert eng.next_greedy(ids, 2, 0, 50.0) == int(np.argmax(pen))
    with pytest.raises(E.NB200Error, match="positions arrive in order"):
        eng.forward(1, 1)
    eng.close()


def test_single_number_gains_stored_as_vectors_of_one(tmp_path):
    cfg = md.famudra_config(40, 32, [("rglru", {"width": 16, "blocks": 1, "conv": 2}, {"experts": 2, "top": 1, "ff": 8, "shared_ff": None})])
    w = md.famudra_random(cfg, 3)
    w1 = {k: (np.reshape(v, (1,)) if np.ndim(v) == 0 else v) for k, v in w.items()}
    path = md.write_model_dir(str(tmp_path / "v1"), cfg, w1)
    eng = E.Engine(path, 64, flags=E.FLAG_F32)
    t = toks(cfg, 12)
    assert rel(whole(eng, t), oracle_forward(cfg, w, t, np.float64)) < F32_TOL
    eng.close()


def test_other_families_refuse_cleanly(tmp_path):
    cfg = md.famudra_config(40, 32, [("rglru", {"width": 16, "blocks": 1, "conv": 2}, None)])
    eng, _ = build(tmp_path, cfg)
    with pytest.raises(E.NB200Error, match="Nano family"):
        eng.run_layer(0, 0)
    eng.close()


# ---- the replay command: token steps on standard input, logits files out, through the same engine calls ----
def test_trace_replay_command(tmp_path):
    import json, subprocess, sys
    cfg = mixed_cfg(vocab=70)
    w = md.famudra_random(cfg, 4)
    path = md.write_model_dir(str(tmp_path / "m"), cfg, w)
    ta, tb = toks(cfg, 50, 21), toks(cfg, 9, 22)
    ra, rb = oracle_forward(cfg, w, ta, np.float64), oracle_forward(cfg, w, tb, np.float64)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ta[:33].tolist(), "want": [32, 0, 5]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ta[33:35].tolist(), "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": ta[35:36].tolist(), "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": ta[36:50].tolist(), "want": [13]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": tb.tolist(), "want": [8, 7]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == ["done %d" % i for i in range(5)]
        got = {i: np.fromfile(out / ("%d.f32" % i), "<f4").reshape(-1, cfg["vocab"]) for i in (0, 2, 3, 4)}
        assert not (out / "1.f32").exists()
        assert rel(got[0], ra[[32, 0, 5]]) < tol                      # in the order "want" lists them
        assert rel(got[2], ra[[35]]) < tol and rel(got[3], ra[[49]]) < tol
        assert rel(got[4], rb[[8, 7]]) < tol
