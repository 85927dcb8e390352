"""Generates tests/golden/moe_cases.npz: outputs of the CPU oracle on small seeded layers.

The reference itself is Rust and cannot be compiled in this environment, so these vectors come
from the oracle after it has been pinned to the reference's known-answer material
(tests/test_oracle_pins.py).  Inputs are not stored: every case is rebuilt from its seeds by
`cases()`; the file holds ids, routing weights and layer outputs.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from moe4all_b200 import synth  # noqa: E402
from oracle import oracle as orc  # noqa: E402

OUT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_cases.npz")


def cases():
    """name -> (layer kwargs, rows, x seed, routing kwargs)"""
    return {
        "tiny_softmax": (dict(seed=21, ne=256, n_expert=8, n_ff=256, sh_ff=256, router_std=0.05), 3, 31,
                         dict(n_used=2)),
        "mid_softmax_noshared": (dict(seed=22, ne=512, n_expert=32, n_ff=256, router_std=0.05), 4, 32,
                                 dict(n_used=4, scale=1.3)),
        "grouped_sigmoid_bias": (dict(seed=23, ne=512, n_expert=32, n_ff=256, sh_ff=256, gated_shared=False,
                                      bias_std=0.05, router_std=0.05), 5, 33,
                                 dict(n_used=4, scale=2.5, gating=1, groups=4, groups_used=2)),
        "odd_blocks": (dict(seed=24, ne=768, n_expert=8, n_ff=768, sh_ff=256, router_std=0.05), 2, 34,
                       dict(n_used=3)),
    }


def run_case(layer_kw, rows, xseed, route_kw):
    kw = dict(layer_kw)
    seed = kw.pop("seed")
    L = synth.make_layer(seed, kw.pop("ne"), kw.pop("n_expert"), kw.pop("n_ff"), **kw)
    x = synth.activations(xseed, rows, L.ne)
    r = dict(route_kw)
    n_used = r.pop("n_used")
    okw = dict(n_expert=L.n_expert, n_used=n_used, n_ff_exp=L.n_ff, bias=L.bias, threads=2, **r)
    if L.sh_gate is not None:
        res = orc.moe_layer(x, L.router, L.gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down, L.sh_gate_inp, L.sh_ff, **okw)
    else:
        res = orc.moe_ffn(x, L.router, L.gate, L.up, L.down, **okw)
    return L, x, res


if __name__ == "__main__":
    out = {}
    for name, c in cases().items():
        _, _, res = run_case(*c)
        out[name + ".dst"], out[name + ".ids"], out[name + ".wts"] = res.dst, res.ids, res.wts
    np.savez_compressed(OUT, **out)
    print("wrote", OUT, os.path.getsize(OUT), "bytes")
