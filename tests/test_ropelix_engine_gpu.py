"""The Ropelix decoder through the library's engine against the plain implementation: whole prompts, prompts
against token-by-token decoding, portions down to two tokens, unequal batches against each request alone,
slots and pages used again, decoding far past windows and pages, the first tokens one by one, greedy
generation through ``Engine.generate`` and the replay program; in float32 and bfloat16, on four
configurations that differ in every size and option."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_ropelix as P
import ropelix_configs as RC
from ropelix_configs import CONFIGS, prompts, read_folder, rel_rms, write_ropelix

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
_plain = {}
_noise = {}


def plain(folder, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain:
        cfg, weights = read_folder(folder)
        _plain[key] = P.forward(cfg, weights, list(tokens))
    return _plain[key]


def noise_of(folder, tokens, dtype=torch.bfloat16):
    key = (folder, tuple(tokens), dtype)
    if key not in _noise:
        cfg, weights = read_folder(folder)
        _noise[key] = RC.noise(cfg, weights, tokens, plain(folder, tokens), dtype)
    return _noise[key]


def assert_rows(got, want, dtype, what, folder, tokens):
    """``tokens``: the sequence whose rows are compared, all of them in order, or a list of (sequence, places)
    for rows of several sequences; the rounding noise is theirs, row by row."""
    pairs = tokens if tokens and isinstance(tokens[0], tuple) else [(tokens, list(range(len(tokens))))]
    n = torch.cat([noise_of(folder, t, dtype)[places] for t, places in pairs])
    RC.assert_rows(got, want, dtype, what, n)


def engine_for(folder, dtype, **kw):
    from mivi_v4_b200 import Engine, load_model
    kw.setdefault("max_tokens", 4096)
    return Engine(load_model(folder, dtype, "cuda:0"), **kw)


def folder_for(tmp_path, name):
    cfg, seed = CONFIGS[name]
    return cfg, seed, write_ropelix(tmp_path, cfg, seed)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_and_every_cut(name, dtype, tmp_path):
    cfg, seed, folder = folder_for(tmp_path, name)
    eng = engine_for(folder, dtype)
    for toks in prompts(cfg["vocab"], [1, 2, 23, 150], seed):
        want = plain(folder, toks)
        s = eng.open()
        assert_rows(eng.step([(s, toks)], "all"), want, dtype, f"{name} whole {len(toks)}", folder, toks)
        eng.close(s)
        for piece in (1, 2, 7, 64, 65):
            if piece > len(toks) and piece != 1:
                continue
            s = eng.open()
            got = torch.cat([eng.step([(s, toks[i:i + piece])], "all") for i in range(0, len(toks), piece)])
            eng.close(s)
            assert_rows(got, want, dtype, f"{name} {len(toks)} tokens in portions of {piece}", folder, toks)
    eng.cache.check()
    assert eng.cache.slots.free_count == eng.cache.n_slots


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prompt_then_long_decoding_past_windows_and_pages(name, dtype, tmp_path):
    cfg, seed, folder = folder_for(tmp_path, name)
    toks = prompts(cfg["vocab"], [230], seed + 1)[0]
    want = plain(folder, toks)
    eng = engine_for(folder, dtype)
    s = eng.open()
    rows = [eng.step([(s, toks[:40])], "all")]
    for t in toks[40:]:
        rows.append(eng.step([(s, [t])], "last"))
    assert_rows(torch.cat(rows), want, dtype, f"{name} decoding", folder, toks)
    assert eng.graph_replays > 100                       # decode steps ran from recordings
    eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_unequal_batches_slots_and_pages_used_again(name, dtype, tmp_path):
    cfg, seed, folder = folder_for(tmp_path, name)
    eng = engine_for(folder, dtype, max_tokens=64 * 12, max_batch=4)
    for round_ in range(3):                              # the same slots and pages serve one batch after another
        reqs = prompts(cfg["vocab"], [3 + 40 * round_, 97, 1, 66], seed + 10 * round_)
        n_prompt = [max(1, len(r) - 20) for r in reqs]
        slots = [eng.open() for _ in reqs]
        got = [[] for _ in reqs]
        out = eng.step([(s, r[:n]) for s, r, n in zip(slots, reqs, n_prompt)], "all")
        at = 0
        for i, n in enumerate(n_prompt):
            got[i].append(out[at:at + n])
            at += n
        live = list(range(len(reqs)))
        step = 0
        while live:
            live = [i for i in live if n_prompt[i] + step < len(reqs[i])]
            if not live:
                break
            out = eng.step([(slots[i], [reqs[i][n_prompt[i] + step]]) for i in live], "last")
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            step += 1
        for i, r in enumerate(reqs):
            assert_rows(torch.cat(got[i]), plain(folder, r), dtype, f"{name} round {round_} request {i}", folder, r)
            eng.close(slots[i])
        eng.cache.check()
    assert all(p.free_count == p.n for p in eng.cache.pages.values())


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_generate_and_more_requests_than_slots(dtype, tmp_path):
    from mivi_v4_b200 import SamplingParams
    cfg, seed, folder = folder_for(tmp_path, "A")
    reqs = prompts(cfg["vocab"], [5, 31, 12, 70, 2], 9)
    eng = engine_for(folder, dtype, max_tokens=64 * 8, max_batch=2)
    outs = eng.generate(reqs, max_new_tokens=12, sampling=SamplingParams.greedy(), stop_token_ids=[])
    c, weights = read_folder(folder)
    for r, o in zip(reqs, outs):
        assert len(o) == 12
        # a run may break a near tie otherwise; every token must be near the top of the plain logits of its own prefix
        logits = P.forward(c, weights, r + o)
        for i, t in enumerate(o):
            row = logits[len(r) + i - 1]
            slack = 1e-4 if dtype == torch.float32 else 0.05
            assert row[t] >= row.max() - slack * (row.max() - row.mean()), (i, t)
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program_whole_decoded_and_batched(dtype, tmp_path):
    cfg, seed, folder = folder_for(tmp_path, "C")
    V = cfg["vocab"]
    reqs = {f"r{i}": p for i, p in enumerate(prompts(V, [40, 75, 140], seed=7))}
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    steps, expect, n = [], [], 0
    for k, v in reqs.items():                                # whole
        steps.append({"step": n, "entries": [{"id": k, "tokens": v, "want": [0, len(v) // 2, len(v) - 1]}], "end": [k]})
        expect.append([(k, [0, len(v) // 2, len(v) - 1])])
        n += 1
    cut = {k: len(v) - 33 for k, v in reqs.items()}           # together: prompts in one batch, then decoded together
    steps.append({"step": n, "entries": [{"id": k + "b", "tokens": v[:cut[k]], "want": [cut[k] - 1]} for k, v in reqs.items()],
                  "end": []})
    expect.append([(k, [cut[k] - 1]) for k in reqs])
    n += 1
    for i in range(33):
        steps.append({"step": n, "entries": [{"id": k + "b", "tokens": [v[cut[k] + i]], "want": [0] if i % 2 else []}
                                            for k, v in reqs.items()], "end": [k + "b" for k in reqs] if i == 32 else []})
        expect.append([(k, [cut[k] + i]) for k in reqs] if i % 2 else [])
        n += 1
    out = tmp_path / f"out_{dtype}"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "600"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    for s, exp in zip(steps, expect):
        path = os.path.join(str(out), f"{s['step']}.f32")
        if not exp:
            assert not os.path.exists(path)
            continue
        got = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(-1, V).copy())
        want = torch.cat([plain(folder, reqs[k])[places] for k, places in exp])
        assert_rows(got, want, tdt, f"step {s['step']}", folder, [(reqs[k], places) for k, places in exp])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_steps_and_batches_of_long_prompts(name, dtype, tmp_path):
    """Steps of hundreds of tokens (the kernels for long steps), whole and in large portions, alone and as a batch."""
    cfg, seed, folder = folder_for(tmp_path, name)
    toks = prompts(cfg["vocab"], [290], seed + 3)[0]
    want = plain(folder, toks)
    eng = engine_for(folder, dtype)
    for piece in (290, 129, 65):
        s = eng.open()
        got = torch.cat([eng.step([(s, toks[i:i + piece])], "all") for i in range(0, len(toks), piece)])
        eng.close(s)
        assert_rows(got, want, dtype, f"{name} portions of {piece}", folder, toks)
    reqs = prompts(cfg["vocab"], [140, 9, 275], seed + 4)
    slots = [eng.open() for _ in reqs]
    out = eng.step(list(zip(slots, reqs)), "all")
    at = 0
    for sl, r in zip(slots, reqs):
        assert_rows(out[at:at + len(r)], plain(folder, r), dtype, f"{name} a batch", folder, r)
        at += len(r)
        eng.close(sl)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_far_keys_and_decoding_after_them(dtype, tmp_path):
    """Prompts of several hundred tokens on a fifth configuration: whole, in two unequal portions, and as a batch of
    three that is then decoded together for 40 tokens, the shortest request ending first."""
    cfg, seed = RC.ROP_E, 45
    folder = write_ropelix(tmp_path, cfg, seed)
    eng = engine_for(folder, dtype, max_tokens=4096, max_batch=4)
    toks = prompts(cfg["vocab"], [700], seed)[0]
    want = plain(folder, toks)
    s = eng.open()
    assert_rows(eng.step([(s, toks)], "all"), want, dtype, "whole", folder, toks)
    eng.close(s)
    s = eng.open()
    got = torch.cat([eng.step([(s, toks[:437])], "all"), eng.step([(s, toks[437:])], "all")])
    eng.close(s)
    assert_rows(got, want, dtype, "two portions", folder, toks)
    reqs = prompts(cfg["vocab"], [340, 75, 521], seed + 1)
    n_prompt = [len(r) - 40 for r in reqs[:2]] + [len(reqs[2]) - 25]
    slots = [eng.open() for _ in reqs]
    out = eng.step([(sl, r[:n]) for sl, r, n in zip(slots, reqs, n_prompt)], "all")
    got, at = [[] for _ in reqs], 0
    for i, n in enumerate(n_prompt):
        got[i].append(out[at:at + n])
        at += n
    for step in range(40):
        live = [i for i in range(3) if n_prompt[i] + step < len(reqs[i])]
        out = eng.step([(slots[i], [reqs[i][n_prompt[i] + step]]) for i in live], "last")
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
    for i, r in enumerate(reqs):
        assert_rows(torch.cat(got[i]), plain(folder, r), dtype, f"request {i}", folder, r)
        eng.close(slots[i])
    eng.cache.check()
