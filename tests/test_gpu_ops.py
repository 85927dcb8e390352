"""GPU: the ops around Op::MoeFfn, descriptor validation, golden vectors and record/replay."""
import importlib.util
import os

import numpy as np
import pytest

from moe4all_b200 import BackendError, DType, MoeFfn, Unsupported, synth
from oracle import oracle as orc

from helpers import GpuLayer, assert_close, oracle_layer

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_golden_cases(backend):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    gold = np.load(os.path.join(ROOT, "tests", "golden", "moe_cases.npz"))
    for name, (layer_kw, rows, xseed, route_kw) in mg.cases().items():
        kw = dict(layer_kw)
        L = synth.make_layer(kw.pop("seed"), kw.pop("ne"), kw.pop("n_expert"), kw.pop("n_ff"), **kw)
        x = synth.activations(xseed, rows, L.ne)
        r = dict(route_kw)
        out, ids, wts = GpuLayer(backend, L).run(x, r.pop("n_used"), **r)
        assert np.array_equal(ids, gold[name + ".ids"]), name
        np.testing.assert_allclose(wts, gold[name + ".wts"], rtol=2e-6, atol=1e-9)
        assert_close(out, gold[name + ".dst"], what=name)


@pytest.mark.parametrize("dt,name,in_f,out_f", [(DType.F32, None, 320, 7), (DType.Q4K, "Q4K", 512, 33),
                                                (DType.Q6K, "Q6K", 768, 19), (DType.Q6K, "Q6K", 256, 64)])
def test_linear(backend, dt, name, in_f, out_f):
    rng = np.random.default_rng(in_f + out_f)
    m = 3
    x = rng.normal(size=(m, in_f)).astype(np.float32)
    if name is None:
        w = rng.normal(size=(out_f, in_f)).astype(np.float32)
    else:
        w = synth.testkit_weight(name, out_f * in_f, seed=77)  # the reference's synthetic blocks
    be = backend
    wb, xb, yb = be.from_host(w), be.from_host(x), be.alloc(m * out_f * 4)
    be.linear(dt, wb, xb, yb, m, in_f, out_f)
    got = be.download(yb, np.float32).reshape(m, out_f)
    assert_close(got, orc.linear(int(dt), w, x, out_f), tol=1e-4, what=f"linear {dt.name}")


def test_elementwise_ops(backend):
    be = backend
    rng = np.random.default_rng(3)
    g, u = rng.normal(size=(4, 96)).astype(np.float32), rng.normal(size=(4, 96)).astype(np.float32)
    gb, ub, db = be.from_host(g), be.from_host(u), be.alloc(g.nbytes)
    be.gated_act(gb, ub, db, g.size)
    assert_close(be.download(db), orc.gated_act_silu(g, u), tol=1e-6)
    gate = rng.normal(size=4).astype(np.float32)
    be.moe_shared_expert_add(gb, ub, be.from_host(gate), db, 4, 96)
    assert_close(be.download(db), orc.moe_shared_add(g, u, gate), tol=1e-6)
    w = rng.normal(size=96).astype(np.float32)
    be.rms_norm(gb, be.from_host(w), db, 4, 96, 1e-6)
    assert_close(be.download(db), orc.rmsnorm(g, w, 1e-6), tol=1e-6)
    be.add(gb, ub, db, g.size)
    assert np.array_equal(be.download(db).reshape(4, 96), g + u)


def test_unfused_shared_expert_matches_fused(backend):
    # the graph builder's op sequence (runner.rs:8088-8175) against the fused call
    be = backend
    L = synth.make_layer(17, 512, 16, 256, sh_ff=256)
    x = synth.activations(5, 3, 512)
    g = GpuLayer(be, L)
    fused, _, _ = g.run(x, 4)
    moe, _, _ = g.run(x, 4, shared=False)
    xb = be.from_host(x)
    gl, sg, su = be.alloc(3 * 4), be.alloc(3 * 256 * 4), be.alloc(3 * 256 * 4)
    act, sd, dst = be.alloc(3 * 256 * 4), be.alloc(3 * 512 * 4), be.alloc(3 * 512 * 4)
    be.linear(DType.F32, g.sh_gate_inp, xb, gl, 3, 512, 1)
    be.linear(DType.Q4K, g.sh_gate, xb, sg, 3, 512, 256)
    be.linear(DType.Q4K, g.sh_up, xb, su, 3, 512, 256)
    be.gated_act(sg, su, act, 3 * 256)
    be.linear(DType.Q6K, g.sh_down, act, sd, 3, 256, 512)
    be.moe_shared_expert_add(be.from_host(moe), sd, gl, dst, 3, 512)
    unfused = be.download(dst).reshape(3, 512)
    assert_close(unfused, fused, tol=1e-4)  # the fused kernels take x in 16-bit fixed point
    assert_close(unfused, oracle_layer(L, x, 4).dst)


def test_descriptor_validation(backend):
    be = backend
    L = synth.make_layer(2, 256, 8, 256)
    g = GpuLayer(be, L)
    x = be.from_host(synth.activations(1, 1, 256))
    dst = be.alloc(1024)

    def op(**kw):
        base = dict(x=x, router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=1, ne=256,
                    n_expert=8, n_used=2, n_ff_exp=256)
        base.update(kw)
        return MoeFfn(**base)

    be.moe_ffn(op())
    be.sync()
    with pytest.raises(Unsupported):
        be.moe_ffn(op(gate_dtype=DType.F32))      # gate bank dtype without a kernel
    with pytest.raises(BackendError):
        be.moe_ffn(op(gate_dtype=DType.Q6K))      # a covered format, but the bank holds Q4_K's bytes: too small
    with pytest.raises(Unsupported):
        be.moe_ffn(op(router_dtype=DType.Q4K))
    with pytest.raises(BackendError):
        be.moe_ffn(op(n_used=9))                  # more than n_expert
    with pytest.raises(BackendError):
        be.moe_ffn(op(rows=0))
    with pytest.raises(BackendError):
        be.moe_ffn(op(rows=2))                    # x and dst hold one row only
    with pytest.raises(BackendError):
        be.moe_ffn(op(n_expert=16))               # banks hold 8 experts
    with pytest.raises(BackendError):
        be.moe_ffn(op(ep_band=(4, 8)))            # band past n_expert
    with pytest.raises(BackendError):
        be.upload(dst, np.zeros(2048, np.uint8))  # copy bounds are an error, not a panic
    # the context stays usable after rejected calls
    be.moe_ffn(op())
    be.sync()


def test_record_replay_matches_eager(backend):
    be = backend
    L = synth.make_layer(31, 512, 16, 256, sh_ff=256)
    g = GpuLayer(be, L)
    x = synth.activations(8, 2, 512)
    eager, _, _ = g.run(x, 4)
    xb, dst = be.from_host(x), be.alloc(2 * 512 * 4)
    op = MoeFfn(x=xb, router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=2, ne=512,
                n_expert=16, n_used=4, n_ff_exp=256, sh_gate=g.sh_gate, sh_up=g.sh_up, sh_down=g.sh_down,
                sh_gate_inp=g.sh_gate_inp, sh_ff=256)
    n0 = be.launch_count()
    be.graph_begin()
    be.moe_ffn(op)
    be.moe_ffn(op)
    plan = be.graph_end()
    assert be.launch_count() == n0  # recorded launches have not run
    be.execute(plan)
    be.sync()
    assert be.launch_count() == n0 + 6
    assert np.array_equal(be.download(dst).reshape(2, 512), eager)
    # new input in the same buffer, replayed
    x2 = synth.activations(9, 2, 512)
    be.upload(xb, x2)
    be.execute(plan)
    be.sync()
    assert_close(be.download(dst).reshape(2, 512), oracle_layer(L, x2, 4).dst)
    plan.free()
