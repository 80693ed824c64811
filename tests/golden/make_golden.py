"""Compares the plain implementation with the pieces of the reference that run on a CPU, once,
and writes their small outputs to ``tests/golden/golden.json``.

The reference's model forward cannot run without a GPU (its norm, rope, attention and expert
kernels are Triton or library CUDA code), and importing its layers needs the ``flashlib``
package, which is not installed; a three-line stand-in for ``flashlib.kernels.slot_cache`` is
written to a temporary folder so that two pure-PyTorch pieces import:

* ``RotaryEmbedding._cos_sin_cache`` (python/freetoken/layers/rotary.py:49-59): the cos/sin table;
* ``MiniMaxM3SparseMoeBlock._route`` (python/freetoken/models/minimax_m3/moe.py:71-81): the router.

Run from the repository root with the reference mounted:

    python tests/golden/make_golden.py /path/to/reference

It asserts that the plain implementation agrees and stores inputs' seeds and the reference's
outputs, which ``tests/test_plain.py`` compares against without needing the reference.
"""

from __future__ import annotations

import json
import os
import sys
import tempfile
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from plain import m3_plain  # noqa: E402


def main(reference_root: str) -> None:
    stub = tempfile.mkdtemp()
    os.makedirs(os.path.join(stub, "flashlib", "kernels"))
    open(os.path.join(stub, "flashlib", "__init__.py"), "w").close()
    open(os.path.join(stub, "flashlib", "kernels", "__init__.py"), "w").close()
    with open(os.path.join(stub, "flashlib", "kernels", "slot_cache.py"), "w") as f:
        f.write("N_STATS = 8\nclass Stat: ...\ndef lru_ensure(*a, **k): raise NotImplementedError\n")
    sys.path.insert(0, stub)
    sys.path.insert(0, os.path.join(reference_root, "python"))
    from freetoken.layers.rotary import RotaryEmbedding
    from freetoken.models.minimax_m3.moe import MiniMaxM3SparseMoeBlock

    golden = {"rope": [], "router": []}
    for head, rd, theta, n in [(64, 64, 10000.0, 40), (128, 64, 5e6, 33), (64, 16, 1e6, 50)]:
        table = RotaryEmbedding(head, rd, n, theta)._cos_sin_cache
        cos, sin = m3_plain.rope_table(rd, theta, n, torch.float32)
        assert torch.equal(torch.cat((cos, sin), -1), table), "rope table differs"
        golden["rope"].append({"rotary_dim": rd, "theta": theta, "positions": n,
                               "rows": {str(p): table[p].tolist() for p in (0, 1, n - 1)}})
    for seed, (T, H, E, k, scale) in enumerate([(9, 48, 8, 2, 1.0), (5, 32, 16, 4, 2.0), (7, 64, 6, 3, 2.0)]):
        g = torch.Generator().manual_seed(seed)
        h = torch.randn(T, H, generator=g)
        w = torch.randn(E, H, generator=g) * 0.1
        b = torch.randn(E, generator=g) * 0.01
        me = types.SimpleNamespace(gate=types.SimpleNamespace(weight=w), e_score_correction_bias=b,
                                   top_k=k, norm_topk_prob=True, routed_scaling_factor=scale)
        wts, ids = MiniMaxM3SparseMoeBlock._route(me, h)
        cfg = types.SimpleNamespace(scoring="sigmoid", top_k=k, scale=scale)
        pw, pi = m3_plain.router(h, w, b, cfg)
        assert torch.equal(pi.to(torch.int32), ids), "router choice differs"
        torch.testing.assert_close(pw, wts, rtol=1e-6, atol=1e-7)
        golden["router"].append({"seed": seed, "T": T, "H": H, "E": E, "k": k, "scale": scale,
                                 "ids": ids.tolist(), "weights": wts.tolist()})
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(golden, f)
    print("plain implementation agrees with the reference's rope table and router; golden.json written")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
