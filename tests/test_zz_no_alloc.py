"""GPU: the allocation-free routing entry point against the ordinary one, through the C ABI.

Collected last on purpose (file name): a run that stops at the first failure has then already run
every other test.  The check is self-contained, so it also passes alone in a fresh process.

Who needs this entry point: hosts that cannot let a library allocate device memory at call time -
a serving process whose own pool already owns the whole GPU, or a loop that cannot tolerate the
device-wide synchronisation a cudaMalloc implies.  `infr_cuda_moe_route_noalloc` computes the same
routing with its scratch in a fixed array inside the library (8 rows x 1024 experts at most).
"""
import ctypes as C

import numpy as np
import pytest

from moe4all_b200 import MoeFfn, MoeGating, synth
from oracle import oracle as orc

from helpers import near_tie_rows

pytestmark = pytest.mark.gpu


def route_both(be, L, x, n_used, gating=MoeGating.Softmax, groups=0, groups_used=0, scale=1.0):
    import torch

    # one stream for both entry points and for the copies, so that everything is ordered
    stream = torch.cuda.Stream(device=be.device)
    be.set_stream(stream.cuda_stream)
    try:
        return _route_both(be, stream.cuda_stream, L, x, n_used, gating, groups, groups_used, scale)
    finally:
        be.sync()
        be.set_stream(None)


def _route_both(be, cuda_stream, L, x, n_used, gating, groups, groups_used, scale):
    rows = x.shape[0]
    xb, router = be.from_host(x), be.from_host(L.router)
    bias = be.from_host(L.bias) if L.bias is not None else None
    # ordinary entry point (per-context scratch, grown with cudaMalloc on demand)
    ids_a, wts_a = be.alloc(rows * n_used * 4), be.alloc(rows * n_used * 4)
    be.moe_route(MoeFfn(x=xb, router=router, gate_exps=router, up_exps=router, down_exps=router, dst=xb, rows=rows,
                        ne=L.ne, n_expert=L.n_expert, n_used=n_used, n_ff_exp=L.n_ff, scale=scale, gating=gating,
                        exp_probs_b=bias, n_expert_groups=groups, n_expert_groups_used=groups_used,
                        ids_out=ids_a, wts_out=wts_a))
    be.sync()
    # allocation-free entry point: plain device pointers, same stream
    ids_b, wts_b = be.alloc(rows * n_used * 4), be.alloc(rows * n_used * 4)
    err = C.create_string_buffer(256)
    rc = be._lib.infr_cuda_moe_route_noalloc(be.device, cuda_stream, xb.device_ptr, router.device_ptr,
                                             bias.device_ptr if bias is not None else None, ids_b.device_ptr,
                                             wts_b.device_ptr, rows, L.ne, L.n_expert, n_used, scale, int(gating), 1,
                                             groups, groups_used, err, 256)
    assert rc == 0, err.value.decode()
    a = (be.download(ids_a, np.int32), be.download(wts_a, np.float32))
    b = (be.download(ids_b, np.int32), be.download(wts_b, np.float32))  # same stream: ordered after the kernels
    return a, b


def test_noalloc_route_matches_and_repeats(backend):
    be = backend
    L = synth.make_layer(61, 1024, 64, 256, bias_std=0.05, router_std=0.05)
    for call, (rows, seed) in enumerate([(4, 1), (7, 2)]):  # two calls in a row share the built-in scratch
        x = synth.activations(seed, rows, 1024)
        (ids_a, wts_a), (ids_b, wts_b) = route_both(be, L, x, 6, gating=MoeGating.Sigmoid, groups=8, groups_used=4,
                                                    scale=2.5)
        assert np.array_equal(ids_a, ids_b), f"call {call}: expert ids differ"
        np.testing.assert_allclose(wts_b, wts_a, rtol=2e-6, atol=1e-9)
        assert len(set(ids_b.tolist())) > 6  # not a degenerate selection
        # and against the CPU oracle's routing of the same rows (a one-expert band: routing only)
        res = orc.moe_ffn(x, L.router, L.gate, L.up, L.down, n_expert=L.n_expert, n_used=6, n_ff_exp=L.n_ff, scale=2.5, gating=1,
                          bias=L.bias, groups=8, groups_used=4, ep_band=(L.n_expert - 1, 1))
        keep = [r for r in range(rows) if r not in set(near_tie_rows(res, 6).tolist())]
        assert keep and np.array_equal(ids_b.reshape(rows, 6)[keep], res.ids[keep]), f"call {call}: ids differ from the oracle's"
        np.testing.assert_allclose(wts_b.reshape(rows, 6)[keep], res.wts[keep], rtol=1e-5, atol=1e-8)


def test_noalloc_route_softmax_shape_of_the_benchmark(backend):
    L = synth.make_layer(62, 2048, 256, 256)
    x = synth.activations(3, 1, 2048)
    (ids_a, wts_a), (ids_b, wts_b) = route_both(backend, L, x, 8)
    assert np.array_equal(ids_a, ids_b)
    np.testing.assert_allclose(wts_b, wts_a, rtol=2e-6, atol=1e-9)
    res = orc.moe_ffn(x, L.router, L.gate, L.up, L.down, n_expert=256, n_used=8, n_ff_exp=L.n_ff, ep_band=(255, 1))
    if len(near_tie_rows(res, 8)) == 0:
        assert np.array_equal(ids_b.reshape(1, 8), res.ids)
        np.testing.assert_allclose(wts_b.reshape(1, 8), res.wts, rtol=1e-5, atol=1e-8)


def test_noalloc_route_sqrt_softplus_and_untouched_ids_marker(backend):
    # the third gating function goes through the same entry point; and the ids buffer is pre-filled with -1
    # by the call itself, so a caller can tell "nothing was produced" from a result (no id is ever -1 here)
    L = synth.make_layer(63, 1024, 64, 256, router_std=0.05)
    x = synth.activations(4, 3, 1024)
    (ids_a, wts_a), (ids_b, wts_b) = route_both(backend, L, x, 4, gating=MoeGating.SqrtSoftplus, scale=1.5)
    assert np.array_equal(ids_a, ids_b) and (ids_b >= 0).all()
    np.testing.assert_allclose(wts_b, wts_a, rtol=2e-6, atol=1e-9)


def test_noalloc_route_rejects_sizes_beyond_the_scratch(backend):
    be = backend
    buf = be.alloc(4096)
    err = C.create_string_buffer(256)
    p = buf.device_ptr
    args = lambda rows, n_expert: (be.device, None, p, p, None, p, p, rows, 256, n_expert, 2, 1.0, 0, 1, 0, 0, err, 256)
    assert be._lib.infr_cuda_moe_route_noalloc(*args(9, 64)) == -1      # more than 8 rows
    assert b"8 rows" in err.value
    assert be._lib.infr_cuda_moe_route_noalloc(*args(1, 2048)) == -1    # more than 1024 experts
    assert be._lib.infr_cuda_moe_route_noalloc(be.device, None, None, p, None, p, p, 1, 256, 8, 2, 1.0, 0, 1, 0, 0, err, 256) == -1
