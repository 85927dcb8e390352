"""GPU parity of the expert-major small-m kernels (one CTA per expert and all its tokens, integer
tensor-core tiles) against the CPU oracle, through the C ABI.  The same calls through the per-pair
kernels are covered in test_gpu_decode.py; here the context's `expert_major` switch forces the other
form at every row count, including the ones where it would not be chosen on its own."""
import numpy as np
import pytest

from moe4all_b200 import MoeFfn, MoeGating, synth

from helpers import GpuLayer, assert_close, near_tie_rows, oracle_layer, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture()
def em(backend):
    backend.set_config(expert_major=2)
    try:
        yield backend
    finally:
        backend.sync()
        backend.set_config(expert_major=0)


def check_ids(ids, ref, n_used):
    ties = set(near_tie_rows(ref, n_used).tolist())
    keep = [r for r in range(ids.shape[0]) if r not in ties]
    assert np.array_equal(ids[keep], ref.ids[keep])
    return keep


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16, 17, 33, 64])
def test_small_layer_all_group_counts(em, rows):
    # segments hold up to 8 token rows: the shared expert (every row) and busy experts span several
    L = synth.make_layer(21, 512, 16, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(200 + rows, rows, 512)
    out, ids, wts = GpuLayer(em, L).run(x, 4, path=1)
    ref = oracle_layer(L, x, 4)
    keep = check_ids(ids, ref, 4)
    assert_close(out[keep], ref.dst[keep])


@pytest.mark.parametrize("rows", [4, 32])
def test_config1_shape(em, rows):
    # hidden 2048, 256 experts, top-8, intermediate 512, gated shared expert: the benchmark's 4- and 32-stream steps
    L = synth.make_layer(1, 2048, 256, 512, sh_ff=512)
    x = synth.activations(7, rows, 2048)
    g = GpuLayer(em, L)
    out, ids, wts = g.run(x, 8, path=1)
    ref = oracle_layer(L, x, 8)
    keep = check_ids(ids, ref, 8)
    assert_close(out[keep], ref.dst[keep])
    out2, _, _ = g.run(x, 8, shared=False, path=1)
    assert_close(out2[keep], oracle_layer(L, x, 8, shared=False).dst[keep])


@pytest.mark.parametrize("rows", [1, 5, 24, 64])
@pytest.mark.parametrize("dims", [(512, 16, 256, 256, 4), (2048, 32, 512, 512, 8), (1024, 16, 768, 256, 4)])
def test_q4k_down_banks(em, rows, dims):
    # the other half of a Q4_K_M file's layers: down banks in Q4_K (144-byte blocks, scale and min per 32 weights);
    # one, two and three blocks per row, shared expert narrower than the routed ones in the last case
    ne, n_expert, nff, sh_ff, n_used = dims
    L = synth.make_layer(71, ne, n_expert, nff, sh_ff=sh_ff, down_q4k=True, router_std=0.05)
    x = synth.activations(400 + rows, rows, ne)
    n0 = em.launch_count()
    out, ids, wts = GpuLayer(em, L).run(x, n_used, path=1)
    assert em.launch_count() - n0 == 5  # router, bucket, gate/up, down, combine: the expert-major kernels ran
    ref = oracle_layer(L, x, n_used)
    keep = check_ids(ids, ref, n_used)
    assert_close(out[keep], ref.dst[keep])


def test_matches_per_pair_kernels_closely(backend):
    # both forms use the same fixed-point activations for gate/up; they differ in the granularity of the
    # down kernel's activation scales (one per row against one per 128 elements), so they agree far inside the oracle bound
    L = synth.make_layer(22, 1024, 32, 512, sh_ff=512, router_std=0.05)
    x = synth.activations(5, 12, 1024)
    g = GpuLayer(backend, L)
    backend.set_config(expert_major=1)
    a, ids_a, _ = g.run(x, 4, path=1)
    backend.set_config(expert_major=2)
    b, ids_b, _ = g.run(x, 4, path=1)
    backend.set_config(expert_major=0)
    assert np.array_equal(ids_a, ids_b)
    assert rel_err(b, a)[0] < 2e-4
    # and run twice it is bit-identical (no atomics on the data path)
    backend.set_config(expert_major=2)
    c, _, _ = g.run(x, 4, path=1)
    backend.set_config(expert_major=0)
    assert np.array_equal(b, c)


def test_wider_shared_expert_and_no_shared_expert(em):
    L = synth.make_layer(23, 512, 16, 256, sh_ff=768, router_std=0.05)
    x = synth.activations(8, 10, 512)
    g = GpuLayer(em, L)
    out, ids, _ = g.run(x, 4, path=1)
    ref = oracle_layer(L, x, 4)
    keep = check_ids(ids, ref, 4)
    assert_close(out[keep], ref.dst[keep])
    out, _, _ = g.run(x, 4, path=1, shared=False)
    assert_close(out[keep], oracle_layer(L, x, 4, shared=False).dst[keep])


def test_config0_and_deepseek_dims(em):
    # intermediate 768 (down rows of 630 bytes: only 2-byte aligned) and hidden 7168 / intermediate 2048
    # (K streamed through the stage ring, 28 blocks per row)
    L = synth.make_layer(0, 2048, 128, 768)
    x = synth.activations(0, 6, 2048)
    out, ids, _ = GpuLayer(em, L).run(x, 8, path=1)
    ref = oracle_layer(L, x, 8)
    keep = check_ids(ids, ref, 8)
    assert_close(out[keep], ref.dst[keep])
    L = synth.make_layer(24, 7168, 16, 2048, sh_ff=2048, gated_shared=False, router_std=0.05)
    x = synth.activations(1, 20, 7168)
    out, ids, _ = GpuLayer(em, L).run(x, 4, path=1, gating=MoeGating.Sigmoid, scale=2.5)
    ref = oracle_layer(L, x, 4, gating=1, scale=2.5)
    keep = check_ids(ids, ref, 4)
    assert_close(out[keep], ref.dst[keep])


VARIANTS = {
    "gelu": dict(act=1),
    "clamp": dict(swiglu_clamp=0.05),
    "weight_before": dict(weight_before=True, gating=MoeGating.Sigmoid, norm_w=False),
    "down_scale": dict(down_scale=np.linspace(0.5, 1.5, 32).astype(np.float32)),
    "fused_gate_up": dict(fused_gate_up=True, act=1),
    "sigmoid_act": dict(act=2),
    "band": dict(ep_band=(8, 16)),
}


@pytest.mark.parametrize("rows", [2, 24])
@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_op_variants(em, rows, variant):
    L = synth.make_layer(61, 512, 32, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(63, rows, 512)
    kw = VARIANTS[variant]
    out, ids, wts = GpuLayer(em, L).run(x, 4, path=1, **kw)
    ref = oracle_layer(L, x, 4, **kw)
    keep = check_ids(ids, ref, 4)
    assert_close(out[keep], ref.dst[keep])


@pytest.mark.parametrize("rows", [4, 20])
def test_routing_from_outside_with_foreign_pairs(backend, rows):
    # what an expert-parallel rank runs: ids and weights are inputs (stages 2 + 4 + 8), pairs of other ranks
    # carry a negative id; run on a context of its own so that nothing an earlier call left in scratch helps
    from moe4all_b200 import CudaBackend
    L = synth.make_layer(47, 512, 32, 256, router_std=0.05)
    x = synth.activations(6, rows, 512)
    ref = oracle_layer(L, x, 4, ep_band=(8, 16))
    local = np.where((ref.ids >= 8) & (ref.ids < 24), ref.ids, -1).astype(np.int32)
    for form in (1, 2):
        be = CudaBackend(0)
        try:
            be.set_config(expert_major=form)
            g = GpuLayer(be, L)
            dst = be.alloc(rows * 512 * 4)
            op = MoeFfn(x=be.from_host(x), router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=rows, ne=512,
                        n_expert=32, n_used=4, n_ff_exp=256, ids_out=be.from_host(local), wts_out=be.from_host(ref.wts), stages=14, path=1)
            be.moe_ffn(op)
            be.sync()
            got = be.download(dst, np.float32).reshape(rows, 512)
            assert_close(got, ref.dst, what=f"form {form}")
        finally:
            be.close()


def test_bad_expert_id_is_reported(backend):
    from moe4all_b200 import BackendError
    L = synth.make_layer(47, 512, 32, 256, router_std=0.05)
    rows = 6
    x = synth.activations(6, rows, 512)
    ids = np.zeros((rows, 4), np.int32)
    ids[:, :] = np.arange(4)
    ids[3, 2] = 99  # outside [0, 32)
    wts = np.full((rows, 4), 0.25, np.float32)
    be = backend
    g = GpuLayer(be, L)
    be.set_config(expert_major=2)
    try:
        dst = be.alloc(rows * 512 * 4)
        be.moe_ffn(MoeFfn(x=be.from_host(x), router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=rows, ne=512,
                          n_expert=32, n_used=4, n_ff_exp=256, ids_out=be.from_host(ids), wts_out=be.from_host(wts), stages=14, path=1))
        with pytest.raises(BackendError, match="expert id"):
            be.sync()
    finally:
        be.set_config(expert_major=0)
    # the batched path reports it as well (ids received from peers, router not run)
    rows = 40
    x = synth.activations(7, rows, 512)
    ids = np.tile(np.arange(4, dtype=np.int32), (rows, 1))
    ids[5, 1] = 32
    wts = np.full((rows, 4), 0.25, np.float32)
    dst = be.alloc(rows * 512 * 4)
    be.moe_ffn(MoeFfn(x=be.from_host(x), router=g.router, gate_exps=g.gate, up_exps=g.up, down_exps=g.down, dst=dst, rows=rows, ne=512,
                      n_expert=32, n_used=4, n_ff_exp=256, ids_out=be.from_host(ids), wts_out=be.from_host(wts), stages=14, path=2))
    with pytest.raises(BackendError, match="expert id"):
        be.sync()
