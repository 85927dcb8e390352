"""Host-paced plans: decode steps recorded once and launched once, each step released by the host through
the bell word and reported back through the done word (infr_cuda_upload_gated / host_signal / host_ring /
host_await / host_reset), instead of one launch and one stream wait per step - the decode replay of
Backend::compile / Backend::execute (crates/infr-core/src/backend.rs:907-908) without the per-token
launch.  Results must equal the CPU oracle's, step by step; a ticket that never comes must end as an
error status with the context still usable (the wait is bounded; nothing here faults or hangs a GPU)."""
import ctypes
import dataclasses

import numpy as np
import pytest

from moe4all_b200 import BackendError, MoeFfn, Unsupported, synth

from helpers import GpuLayer, assert_close, oracle_layer

pytestmark = pytest.mark.gpu


def pinned(n_floats):
    import torch

    t = torch.empty(n_floats, dtype=torch.float32).pin_memory()
    return t, t.data_ptr()


def layer_op(be, g, L, x_in, dst, rows, n_used):
    return MoeFfn(x=x_in, router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=rows, ne=L.ne,
                  n_expert=L.n_expert, n_used=n_used, n_ff_exp=L.n_ff, sh_gate=g.sh_gate, sh_up=g.sh_up, sh_down=g.sh_down,
                  sh_gate_inp=g.sh_gate_inp, sh_ff=L.sh_ff)


@pytest.mark.parametrize("rows,host_dst", [(1, True), (3, True), (12, False)])
def test_paced_steps_match_oracle(backend, rows, host_dst):
    be = backend
    L = synth.make_layer(61, 512, 16, 256, sh_ff=256, router_std=0.05)
    g = GpuLayer(be, L)
    steps, n = 5, rows * L.ne
    stage_t, stage_ptr = pinned(n)
    out_t, out_ptr = pinned(n)
    x_in = be.alloc(n * 4)
    dst_dev = be.alloc(n * 4)
    dst = be.wrap(out_ptr, n * 4) if host_dst else dst_dev  # small results: the last kernel writes pinned memory itself
    be.moe_ffn(layer_op(be, g, L, x_in, dst, rows, 4))  # once un-recorded: scratch cannot grow inside a recording
    be.sync()
    be.graph_begin()
    for s in range(steps):
        be.upload_ptr_gated(x_in, stage_ptr, n * 4, s + 1)
        be.moe_ffn(layer_op(be, g, L, x_in, dst, rows, 4))
        if not host_dst:
            be.download_ptr_async(dst_dev, out_ptr, n * 4)
        be.host_signal(s + 1)
    plan = be.graph_end()
    xs = [synth.activations(300 + s, rows, L.ne) for s in range(steps)]
    want = [oracle_layer(L, x, 4).dst for x in xs]
    # a run of steps in one call, every step's result copied out
    outs = [np.empty(n, np.float32) for _ in range(steps)]
    be.host_reset()
    be.execute(plan)
    be.host_steps(1, stage_ptr, [x.ctypes.data for x in xs], n * 4, out_ptr, [o.ctypes.data for o in outs], n * 4)
    be.sync()
    for s in range(steps):
        assert_close(outs[s].reshape(rows, L.ne), want[s])
    for rep in range(2):  # the second replay checks that the words were set back
        be.host_reset()
        be.execute(plan)
        for s in range(steps):
            if rep == 0:
                ctypes.memmove(stage_ptr, xs[s].ctypes.data, n * 4)
                be.host_ring(s + 1)
                be.host_await(s + 1)
            else:  # the same three things in one call
                be.host_step(s + 1, stage_ptr, xs[s].ctypes.data, n * 4)
            got = out_t.numpy().reshape(rows, L.ne).copy()
            assert_close(got, want[s])
        be.sync()
    plan.free()


def test_ticket_that_never_comes_is_an_error_and_the_plan_drains(backend):
    be = backend
    L = synth.make_layer(62, 512, 16, 256, sh_ff=256, router_std=0.05)
    g = GpuLayer(be, L)
    n = L.ne
    stage_t, stage_ptr = pinned(n)
    x_in, dst = be.alloc(n * 4), be.alloc(n * 4)
    old = be.get_config().gate_timeout_ms
    be.set_config(gate_timeout_ms=40)
    try:
        be.host_reset()
        # three gated steps queued, nothing rung: the first gate runs out, the others no longer wait
        for t in (1, 2, 3):
            be.upload_ptr_gated(x_in, stage_ptr, n * 4, t)
            be.moe_ffn(layer_op(be, g, L, x_in, dst, 1, 4))
            be.host_signal(t)
        with pytest.raises(BackendError) as e:
            be.host_await(1)
        assert "bounded device-side wait" in str(e.value) or "not signalled" in str(e.value)
    finally:
        be.set_config(gate_timeout_ms=old)
    # the context is usable afterwards
    be.host_reset()
    x = synth.activations(7, 2, L.ne)
    out, _, _ = g.run(x, 4)
    assert_close(out, oracle_layer(L, x, 4).dst)


def test_gated_upload_wants_pinned_memory(backend):
    be = backend
    buf = be.alloc(4096)
    pageable = np.zeros(1024, np.float32)
    with pytest.raises(Unsupported):
        be.upload_ptr_gated(buf, pageable.ctypes.data, 4096, 1)
    with pytest.raises(BackendError):
        be.upload_ptr_gated(buf, pageable.ctypes.data, 4096, 0)  # ticket 0 is "nothing rung yet"
