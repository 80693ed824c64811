"""The command line as a user calls it (``freetoken <command> ...`` = ``cli.main([...])``): a model
folder made by ``make-model``, tokens from ``generate`` compared with the plain model's greedy choice,
logits from ``replay`` compared with the plain model's.  On the CPU the kernels are replaced by their
plain statements, so the commands' own code (options, files, printing) is what runs; the ``gpu`` test
runs the same commands on the device with the real kernels.

The reference's dispatcher is a name -> function table as well (python/freetoken/cli.py:93-126)."""

from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

import kernel_refs
from freetoken_b200 import cli
from plain.m3_plain import PlainM3
from tiny_configs import TINY_A, TINY_B


def make_model(tmp_path, raw, capsys, seed=3):
    cfg = tmp_path / "config_in.json"
    cfg.write_text(json.dumps(raw))
    out = str(tmp_path / "model")
    assert cli.main(["make-model", "--config", str(cfg), "--out", out, "--seed", str(seed)]) == 0
    assert capsys.readouterr().out.strip() == out
    assert os.path.isfile(os.path.join(out, "config.json")) and os.path.isfile(os.path.join(out, "model.safetensors"))
    return out


def generate_and_replay(folder, device, dtype, capsys, tmp_path, plain):
    V = plain.cfg.vocab
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, V, (n,), generator=g).tolist() for n in (6, 11)]
    pf = tmp_path / "prompts.json"
    pf.write_text(json.dumps(prompts[1:]))
    rc = cli.main(["generate", "--model-path", folder, "--device", device, "--dtype", dtype, "--page-size", "4",
                   "--num-pages", "40", "--max-prefill-length", "8", "--max-running-requests", "2",
                   "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-file", str(pf), "--max-tokens", "5",
                   "--ignore-eos"])
    assert rc == 0
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert len(lines) == 2
    for p, r in zip(prompts, lines):
        assert r["finish_reason"] == "length" and len(r["token_ids"]) == 5
        toks = list(p)
        for got in r["token_ids"]:
            logits = plain.logits(toks)[-1]
            top2 = torch.topk(logits, 2).values
            if dtype == "float32" or float(top2[0] - top2[1]) > 0.05:
                assert got == int(torch.argmax(logits))
            toks.append(got)
    # replay: the same tokens in two portions and one at a time, logits wanted at the ends
    toks = prompts[1]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[7:9], "want": [0, 1]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[9:10], "want": [0]},
                                     {"id": "b", "tokens": toks[:3], "want": [2]}], "end": ["a", "b"]}]
    out_dir = str(tmp_path / "logits")
    import io
    import sys

    stdin = sys.stdin
    sys.stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    try:
        rc = cli.main(["replay", "--model", folder, "--dtype", dtype, "--out", out_dir, "--max-tokens", "128",
                       "--device", device])
    finally:
        sys.stdin = stdin
    assert rc == 0
    assert [l for l in capsys.readouterr().out.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = plain.logits(toks)
    tol = dict(rtol=1e-4, atol=2e-5) if dtype == "float32" else dict(rtol=2e-2, atol=8e-3)
    read = lambda s: torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{s}.f32"), dtype="<f4").reshape(-1, V).copy())
    torch.testing.assert_close(read(0), ref[6:7], **tol)
    torch.testing.assert_close(read(1), ref[7:9], **tol)
    torch.testing.assert_close(read(2), torch.cat([ref[9:10], ref[2:3]]), **tol)


def test_make_model_generate_and_replay_on_the_cpu(tmp_path, capsys, monkeypatch):
    kernel_refs.install(monkeypatch)
    folder = make_model(tmp_path, TINY_A, capsys)
    generate_and_replay(folder, "cpu", "float32", capsys, tmp_path, PlainM3(folder))


def test_unknown_commands_and_missing_folders_are_reported(tmp_path, capsys):
    assert cli.main([]) == 2
    assert cli.main(["--help"]) == 0 and "make-model" in capsys.readouterr().out
    assert cli.main(["serve"]) == 2 and "unknown command" in capsys.readouterr().err
    rc = cli.main(["generate", "--model-path", str(tmp_path / "none"), "--device", "cpu", "--prompt-ids", "1,2"])
    assert rc == 1 and "config.json" in capsys.readouterr().err
    with pytest.raises(SystemExit):  # argparse: no prompt given
        cli.main(["generate", "--model-path", str(tmp_path)])


def test_console_scripts_are_declared():
    """``freetoken`` and ``ft`` (the reference's name, its pyproject.toml:69-70) both point at ``cli.main``."""
    import tomllib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "pyproject.toml"), "rb") as f:
        scripts = tomllib.load(f)["project"]["scripts"]
    assert scripts["freetoken"] == scripts["ft"] == "freetoken_b200.cli:main"


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_make_model_generate_and_replay_on_the_device(name, dtype, tmp_path, capsys):
    folder = make_model(tmp_path, {"A": TINY_A, "B": TINY_B}[name], capsys)
    generate_and_replay(folder, "cuda:0", dtype, capsys, tmp_path, PlainM3(folder))
