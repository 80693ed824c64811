"""bin/trace_run as a user runs it: a trace on standard input, logits in files, compared with the
plain implementation under every way of cutting and batching, in 32-bit and in bfloat16."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import F32_TOL, assert_bf16_close, bf16_tol, clear_tokens, mixed_schedule, model_folder, tokens_for
from plain.m3_plain import PlainM3
from tiny_configs import ALL

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def run_trace(folder, dtype, out_dir, max_tokens, steps, extra=()):
    lines = "".join(json.dumps(s) + "\n" for s in steps)
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                        "--max-tokens", str(max_tokens), *extra], input=lines, capture_output=True, text=True,
                       timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    return p


def read_logits(out_dir, step, vocab):
    a = np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4")
    return torch.from_numpy(a.reshape(-1, vocab).copy())


def check(got, ref, dtype, margins, what, prefix_only=False, name=""):
    if dtype == "float32":
        torch.testing.assert_close(got, ref[: got.shape[0]], **F32_TOL, msg=lambda m: f"{what}: {m}")
    else:
        assert_bf16_close(got, ref, margins, what, prefix_only=prefix_only, name=name)


# B (tied head, softmax router, no QK norm) runs with its own pages of 8 tokens; D has block-sparse layers,
# where bfloat16 is compared before the first near-tie of a sequence only.
@pytest.mark.parametrize("name,dtype", [(n, d) for n in "ABCD" for d in ("float32", "bfloat16")])
def test_trace_replay(name, dtype, tmp_path_factory, tmp_path):
    folder = model_folder(tmp_path_factory.getbasetemp(), name, ALL[name])
    plain = PlainM3(folder)
    V = plain.cfg.vocab
    sparse = name == "D"
    lengths = {"a": 70, "b": 100, "c": 45, "d": 64, "e": 90, "f": 33}
    seqs = {r: (clear_tokens(plain, n, 50 + 40 * i, 30) if sparse else tokens_for(V, n, 50 + i))
            for i, (r, n) in enumerate(lengths.items())}
    steps, where = [], {}  # where[(request, mode)] = list of (step, rows, first position)
    n = 0

    def add(entries, end=()):
        nonlocal n
        steps.append({"step": n, "entries": entries, "end": list(end)})
        n += 1
        return n - 1

    # 1. whole, every position wanted
    s = add([{"id": "w", "tokens": seqs["a"], "want": list(range(70))}], end=["w"])
    where["whole"] = [(s, 70, 0)]
    # 2. most of it in one step (nothing wanted), then the last 32 one by one
    add([{"id": "t", "tokens": seqs["a"][:38], "want": []}])
    where["tail"] = []
    for i in range(38, 70):
        s = add([{"id": "t", "tokens": [seqs["a"][i]], "want": [0]}], end=["t"] if i == 69 else [])
        where["tail"].append((s, 1, i))
    # 3. portions of changing size, down to two tokens; only some places wanted
    i, where["cuts"] = 0, []
    for c in [7, 2, 13, 2, 5, 3, 2, 17, 2, 9, 2, 6]:
        s = add([{"id": "c", "tokens": seqs["a"][i:i + c], "want": [0, c - 1]}], end=["c"] if i + c == 70 else [])
        where["cuts"].append((s, c, i))
        i += c
    assert i == 70
    # 4. mixed, up to four live, in a pool of 4 x 128 tokens so that pages are used again
    fed = {r: 0 for r in seqs}
    mixed = {r: [] for r in seqs}
    for stepdef in mixed_schedule(lengths, seed=8):
        entries, ends = [], []
        for r, k in stepdef.items():
            entries.append({"id": "m" + r, "tokens": seqs[r][fed[r]:fed[r] + k], "want": list(range(k))})
        s = add(entries)
        for r, k in stepdef.items():
            mixed[r].append((s, k, fed[r]))
            fed[r] += k
            if fed[r] == lengths[r]:
                steps[-1]["end"].append("m" + r)
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, out_dir, 4 * 128, steps, extra=("--page-size", "8") if name == "B" else ())

    ref = {r: plain.logits(t) for r, t in seqs.items()}
    marg = {r: plain.router_margins(t) for r, t in seqs.items()}
    if sparse:  # a flip spreads to later tokens: everything after the first near-tie counts as unsure
        for r, m in marg.items():
            unsure = m <= 0
            if unsure.any():
                m[int(unsure.float().argmax()):] = 0
    check(read_logits(out_dir, where["whole"][0][0], V), ref["a"], dtype, marg["a"], "whole", sparse, name)
    tail = torch.cat([read_logits(out_dir, s, V) for s, _, _ in where["tail"]])
    if not (sparse and dtype == "bfloat16"):  # (a tail of a sparse sequence lies behind its first near-tie)
        check(tail, ref["a"][38:], dtype, marg["a"][38:], "tail", name=name)
    else:
        assert torch.isfinite(tail).all() and (tail - ref["a"][38:]).abs().max() < 0.5
    assert not os.path.exists(os.path.join(out_dir, "1.f32"))  # nothing was wanted in that step
    rows, places = [], []
    for s, c, i in where["cuts"]:
        got = read_logits(out_dir, s, V)
        assert got.shape[0] == 2  # the first and the last place of the portion were wanted
        rows.append(got)
        places += [i, i + c - 1]
    idx = torch.tensor(places)
    if sparse and dtype == "bfloat16":
        keep = marg["a"][idx] > 0
        torch.testing.assert_close(torch.cat(rows)[keep], ref["a"][idx][keep], **bf16_tol(name))
    else:
        check(torch.cat(rows), ref["a"][idx], dtype, marg["a"][idx], "portions of changing size", name=name)
    files = {}
    for r in seqs:
        rows = []
        for s, k, pos in mixed[r]:
            if s not in files:
                files[s] = read_logits(out_dir, s, V)
            entry_ids = [e["id"] for e in steps[s]["entries"]]
            off = sum(len(e["want"]) for e in steps[s]["entries"][: entry_ids.index("m" + r)])
            rows.append(files[s][off:off + k])
        check(torch.cat(rows), ref[r], dtype, marg[r], f"mixed {r}", sparse, name)


def test_trace_run_reports_errors(tmp_path_factory, tmp_path):
    folder = model_folder(tmp_path_factory.getbasetemp(), "A", ALL["A"])
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", str(tmp_path / "nothing"), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True, text=True)
    assert p.returncode != 0 and "config.json" in p.stderr
    too_many = json.dumps({"step": 0, "entries": [{"id": "a", "tokens": list(range(100)), "want": []}], "end": []})
    p = subprocess.run([sys.executable, TRACE_RUN, "--model", folder, "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input=too_many + "\n",
                       capture_output=True, text=True)
    assert p.returncode != 0 and "done 0" not in p.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_long_steps(dtype, tmp_path_factory, tmp_path):
    """Steps of more than 128 tokens with heads of 128: in bfloat16 these run the tensor-core
    attention kernel.  A request whole, the same in two long portions and ten single tokens, and a
    long portion beside single tokens of another request."""
    folder = model_folder(tmp_path_factory.getbasetemp(), "E", ALL["E"])
    plain = PlainM3(folder)
    V = plain.cfg.vocab
    a, b = tokens_for(V, 300, 61), tokens_for(V, 180, 62)
    steps = [
        {"step": 0, "entries": [{"id": "w", "tokens": a, "want": list(range(300))}], "end": ["w"]},
        {"step": 1, "entries": [{"id": "p", "tokens": a[:160], "want": [0, 159]}], "end": []},
        {"step": 2, "entries": [{"id": "p", "tokens": a[160:290], "want": list(range(130))},
                                {"id": "q", "tokens": b[:20], "want": [19]}], "end": []},
    ]
    for i in range(10):
        steps.append({"step": 3 + i, "entries": [{"id": "p", "tokens": [a[290 + i]], "want": [0]},
                                                 {"id": "q", "tokens": [b[20 + i]], "want": [0]}],
                      "end": ["p"] if i == 9 else []})
    steps.append({"step": 13, "entries": [{"id": "q", "tokens": b[30:], "want": list(range(150))}], "end": ["q"]})
    out_dir = str(tmp_path / "out")
    run_trace(folder, dtype, out_dir, 1024, steps)
    ra, rb = plain.logits(a), plain.logits(b)
    ma, mb = plain.router_margins(a), plain.router_margins(b)
    check(read_logits(out_dir, 0, V), ra, dtype, ma, "300 tokens whole")
    idx = torch.tensor([0, 159])
    check(read_logits(out_dir, 1, V), ra[idx], dtype, ma[idx], "first portion")
    got = read_logits(out_dir, 2, V)
    check(got[:130], ra[160:290], dtype, ma[160:290], "second portion beside another request")
    check(got[130:], rb[19:20], dtype, mb[19:20], "short portion beside a long one")
    pa = torch.cat([read_logits(out_dir, 3 + i, V)[:1] for i in range(10)])
    qb = torch.cat([read_logits(out_dir, 3 + i, V)[1:] for i in range(10)])
    check(pa, ra[290:], dtype, ma[290:], "decoded after long portions")
    check(qb, rb[20:30], dtype, mb[20:30], "decoded beside")
    check(read_logits(out_dir, 13, V), rb[30:], dtype, mb[30:], "a long portion over earlier keys")
