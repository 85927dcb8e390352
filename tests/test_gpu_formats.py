"""Expert banks in other GGUF formats than the Q4_K / Q6_K pair: Q5_K, Q8_0 and mixes, through the
C ABI against the CPU oracle, on the small-m kernels, the grouped GEMM tiles, the un-fused Linear op and
the expert-parallel band form (the reference takes gate, up and down formats independently:
crates/infr-core/src/tensor.rs:172-196; op parity per dtype in the style of
crates/infr-llama/tests/seam_op_parity.rs)."""
import numpy as np
import pytest

from moe4all_b200 import BackendError, DType, synth
from oracle import oracle as orc

from helpers import GpuLayer, assert_close, near_tie_rows, oracle_layer

pytestmark = pytest.mark.gpu

Q8_0, Q4K, Q5K, Q6K, IQ4NL, IQ4XS = 8, 12, 13, 14, 20, 23
Q4_0, Q4_1, Q5_0, Q5_1, Q2K, Q3K, MXFP4, NVFP4, Q2_0 = 2, 3, 6, 7, 10, 11, 39, 40, 42
IQ2XS, IQ3XXS, IQ3S, IQ2S = 17, 18, 21, 22
MIXES = [(Q5K, Q5K, Q6K), (Q8_0, Q8_0, Q8_0), (Q5K, Q5K, Q5K), (Q4K, Q5K, Q8_0), (Q6K, Q6K, Q4K), (Q8_0, Q4K, Q6K),
         (IQ4XS, IQ4XS, Q6K), (IQ4NL, IQ4NL, IQ4NL), (IQ4XS, IQ4NL, IQ4XS),
         (Q4_0, Q4_0, Q4_0), (Q4_1, Q4_1, Q5_1), (Q5_0, Q5_1, Q5_0), (Q2K, Q2K, Q3K), (Q3K, Q3K, Q6K), (Q3K, Q2K, Q2K),
         (MXFP4, MXFP4, MXFP4), (MXFP4, MXFP4, Q6K),
         (NVFP4, NVFP4, NVFP4), (Q2_0, Q2_0, Q2_0), (Q2_0, NVFP4, Q4K),
         (IQ2XS, IQ2XS, IQ3S), (IQ3XXS, IQ3XXS, IQ2S), (IQ3S, IQ2S, Q6K), (IQ2S, IQ3XXS, IQ2XS)]


@pytest.fixture(autouse=True)
def grid_tables(backend):
    # the grid codebook formats need their tables: stand-ins with the real ones' shape, alphabet and first entry,
    # the same on both sides
    for dt in synth.CODEBOOKS:
        backend.set_codebook(DType(dt), synth.codebook(dt))
        orc.set_codebook(dt, synth.codebook(dt))


def check(out, ids, ref, n_used):
    ties = set(near_tie_rows(ref, n_used).tolist())
    for r in range(ids.shape[0]):
        if r not in ties:
            assert ids[r].tolist() == ref.ids[r].tolist()
    return assert_close(out, ref.dst)


@pytest.mark.parametrize("mix", MIXES)
@pytest.mark.parametrize("rows,path", [(1, 0), (5, 1), (40, 1), (40, 2), (300, 0)])
def test_format_mix_matches_oracle(backend, mix, rows, path):
    L = synth.make_layer(31 + mix[0], 512, 16, 256, sh_ff=256, router_std=0.05, dtypes=mix)
    x = synth.activations(200 + rows, rows, 512)
    g = GpuLayer(backend, L)
    n0 = backend.launch_count()
    out, ids, _ = g.run(x, 4, path=path)
    assert backend.launch_count() > n0
    check(out, ids, oracle_layer(L, x, 4), 4)


@pytest.mark.parametrize("mix", [(Q5K, Q5K, Q6K), (Q8_0, Q8_0, Q8_0), (IQ4XS, IQ4XS, Q6K)])
def test_config1_shape(backend, mix):
    # hidden 2048, 256 experts top-8, intermediate 512, gated shared expert: decode rows and a batched call
    L = synth.make_layer(5, 2048, 256, 512, sh_ff=512, dtypes=mix)
    g = GpuLayer(backend, L)
    for rows in (1, 4, 400):
        x = synth.activations(50 + rows, rows, 2048)
        out, ids, _ = g.run(x, 8)
        sel = np.arange(rows) if rows <= 4 else np.random.default_rng(1).choice(rows, 6, replace=False)
        ref = oracle_layer(L, x[sel], 8)
        check(out[sel], ids[sel], ref, 8)


@pytest.mark.parametrize("mix", [(Q5K, Q5K, Q6K), (Q8_0, Q8_0, Q8_0), (IQ4XS, IQ4XS, IQ4NL)])
def test_variants_and_bands(backend, mix):
    L = synth.make_layer(77, 512, 16, 256, sh_ff=256, router_std=0.05, dtypes=mix)
    g = GpuLayer(backend, L)
    x = synth.activations(9, 6, 512)
    ds = np.linspace(0.5, 1.5, 16).astype(np.float32)
    for path in (1, 2):
        # weight on the expert's input, GELU, clamp, a per-expert output scale, a fused gate/up bank
        for kw in (dict(weight_before=True), dict(act=1), dict(swiglu_clamp=0.02), dict(down_scale=ds), dict(fused_gate_up=True)):
            out, ids, _ = g.run(x, 4, path=path, **kw)
            check(out, ids, oracle_layer(L, x, 4, **kw), 4)
        # two expert-parallel bands sum to the whole layer's routed part
        full = oracle_layer(L, x, 4, shared=False).dst
        parts = [g.run(x, 4, path=path, shared=False, ep_band=(lo, 8))[0] for lo in (0, 8)]
        assert_close(parts[0] + parts[1], full)


@pytest.mark.parametrize("dt,name,in_f,out_f", [(Q5K, "Q5K", 512, 64), (Q8_0, "Q8_0", 512, 64), (Q8_0, "Q8_0", 96, 40),
                                                (IQ4XS, "IQ4XS", 512, 64), (IQ4NL, "IQ4NL", 160, 24), (Q4_0, "Q4_0", 96, 16),
                                                (Q4_1, "Q4_1", 512, 16), (Q5_0, "Q5_0", 512, 16), (Q5_1, "Q5_1", 64, 16),
                                                (Q2K, "Q2K", 512, 32), (Q3K, "Q3K", 768, 32), (MXFP4, "MXFP4", 96, 24),
                                                (NVFP4, "NVFP4", 192, 24), (Q2_0, "Q2_0", 320, 16),
                                                (IQ2XS, "IQ2XS", 512, 24), (IQ2S, "IQ2S", 256, 16), (IQ3XXS, "IQ3XXS", 768, 16),
                                                (IQ3S, "IQ3S", 512, 24)])
def test_linear_op(backend, dt, name, in_f, out_f):
    # Op::Linear on the reference's synthesised weights (crates/infr-testkit/src/lib.rs:74-123); Q8_0 rows
    # need whole 32-weight blocks only
    w = synth.testkit_weight(name, out_f * in_f, seed=0x77).reshape(-1)
    x = synth.gen_f32(3 * in_f, 5).reshape(3, in_f)
    be = backend
    wb, xb, yb = be.from_host(w), be.from_host(x), be.alloc(3 * out_f * 4)
    be.linear(DType(dt), wb, xb, yb, 3, in_f, out_f)
    be.sync()
    got = be.download(yb, np.float32).reshape(3, out_f)
    assert_close(got, orc.linear(dt, w, x, out_f), tol=1e-4)
    if dt == Q5K:
        with pytest.raises(BackendError):
            be.linear(DType(dt), wb, xb, yb, 3, 96, 8)  # not a whole number of 256-weight blocks


def test_codebook_format_needs_its_table():
    # a context that was never given the table refuses the format (and says how to fix it); wrong tables are refused too
    from moe4all_b200 import CudaBackend, Unsupported

    be = CudaBackend(0)
    try:
        w = be.from_host(synth.testkit_weight("IQ3S", 512 * 8, seed=1).reshape(-1))
        x, y = be.from_host(synth.gen_f32(512, 2)), be.alloc(8 * 4)
        with pytest.raises(Unsupported) as e:
            be.linear(DType(IQ3S), w, x, y, 1, 512, 8)
        assert "infr_cuda_set_codebook" in str(e.value)
        with pytest.raises(BackendError):
            be.set_codebook(DType(IQ3S), synth.codebook(IQ3S)[:-1])  # wrong size
        with pytest.raises(BackendError):
            be.set_codebook(DType(IQ3S), synth.codebook(IQ3S) | 0x80)  # grid bytes must stay below 128
        with pytest.raises(BackendError):
            be.set_codebook(DType(Q4K), synth.codebook(IQ3S))  # not a codebook format
        be.set_codebook(DType(IQ3S), synth.codebook(IQ3S))
        be.linear(DType(IQ3S), w, x, y, 1, 512, 8)
        be.sync()
        want = orc.linear(IQ3S, be.download(w, np.uint8), synth.gen_f32(512, 2).reshape(1, 512), 8)
        assert_close(be.download(y, np.float32).reshape(1, 8), want, tol=1e-4)
    finally:
        be.close()
    # the table outlives the context that set it: another context of the device that was given it keeps working
    be2 = CudaBackend(0)
    try:
        be2.set_codebook(DType(IQ3S), synth.codebook(IQ3S))
        be3 = CudaBackend(0)
        be3.set_codebook(DType(IQ3S), synth.codebook(IQ3S))
        be3.close()
        w2, x2, y2 = be2.from_host(synth.testkit_weight("IQ3S", 512 * 8, seed=1).reshape(-1)), be2.from_host(synth.gen_f32(512, 2)), be2.alloc(32)
        be2.linear(DType(IQ3S), w2, x2, y2, 1, 512, 8)
        be2.sync()
        assert_close(be2.download(y2, np.float32).reshape(1, 8), want, tol=1e-4)
    finally:
        be2.close()


def test_unknown_format_refused(backend):
    L = synth.make_layer(3, 256, 8, 256)
    g = GpuLayer(backend, L)
    L.gate_dtype = 0  # F32 banks: not covered
    with pytest.raises(BackendError) as e:
        g.run(synth.activations(1, 1, 256), 2)
    assert "expert banks must be one of" in str(e.value)
    L.gate_dtype = 12
