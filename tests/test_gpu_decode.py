"""GPU parity of the small-m (decode) kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from moe4all_b200 import MoeGating, synth

from helpers import GpuLayer, assert_close, near_tie_rows, oracle_layer, rel_err

pytestmark = pytest.mark.gpu


def check_ids(ids, wts, ref, n_used):
    ties = set(near_tie_rows(ref, n_used).tolist())
    for r in range(ids.shape[0]):
        if r in ties:
            continue
        assert ids[r].tolist() == ref.ids[r].tolist(), f"row {r}: ids {ids[r]} != oracle {ref.ids[r]}"
        np.testing.assert_allclose(wts[r], ref.wts[r], rtol=2e-6, atol=1e-9)
    assert len(ties) < max(2, ids.shape[0] // 50), "too many near-tie rows: the case does not test routing"


@pytest.mark.parametrize("rows", [1, 2, 4, 8])
def test_tiny_layer(backend, rows):
    # smallest block-aligned layer: ne = nff = 256, E = 8, k = 2
    L = synth.make_layer(11, 256, 8, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(100 + rows, rows, 256)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 2)
    ref = oracle_layer(L, x, 2)
    check_ids(ids, wts, ref, 2)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows", [1, 4])
def test_config0_layer(backend, rows):
    # hidden 2048, 128 experts, top-8, intermediate 768, no shared expert, seed 0
    L = synth.make_layer(0, 2048, 128, 768)
    x = synth.activations(0, rows, 2048)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 8)
    ref = oracle_layer(L, x, 8)
    check_ids(ids, wts, ref, 8)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows", [1, 4])
def test_config1_layer(backend, rows):
    # Qwen3.6-35B-A3B shape: hidden 2048, 256 experts, top-8, intermediate 512, gated shared expert
    L = synth.make_layer(1, 2048, 256, 512, sh_ff=512)
    x = synth.activations(7, rows, 2048)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 8)
    ref = oracle_layer(L, x, 8)
    check_ids(ids, wts, ref, 8)
    assert_close(out, ref.dst)
    # routed part alone (no shared expert) must match too
    out2, _, _ = g.run(x, 8, shared=False)
    assert_close(out2, oracle_layer(L, x, 8, shared=False).dst)


@pytest.mark.parametrize("rows", [12, 40])
def test_config1_layer_more_rows(backend, rows):
    # above eight rows the small-m expert kernels run behind the batched router
    L = synth.make_layer(1, 2048, 256, 512, sh_ff=512)
    x = synth.activations(17, rows, 2048)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 8, path=1)
    ref = oracle_layer(L, x, 8)
    check_ids(ids, wts, ref, 8)
    assert_close(out, ref.dst)
    out_auto, ids_auto, _ = g.run(x, 8)
    assert np.array_equal(out_auto, out) and np.array_equal(ids_auto, ids)


@pytest.mark.parametrize("rows", [1, 4, 20])
def test_q4k_down_banks(backend, rows):
    # a Q4_K_M model file stores most layers' down banks in Q4_K (the rest in Q6_K)
    L = synth.make_layer(61, 2048, 32, 512, sh_ff=512, down_q4k=True)
    x = synth.activations(19, rows, 2048)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 8, path=1)
    ref = oracle_layer(L, x, 8)
    check_ids(ids, wts, ref, 8)
    assert_close(out, ref.dst)


def test_determinism(backend):
    L = synth.make_layer(3, 2048, 64, 512, sh_ff=512)
    x = synth.activations(9, 4, 2048)
    g = GpuLayer(backend, L)
    a = g.run(x, 8)
    b = g.run(x, 8)
    for u, v in zip(a, b):
        assert np.array_equal(u, v)


def test_grouped_sigmoid_bias_routing(backend):
    # DeepSeek-style: sigmoid gating, 8 groups / 4 used, selection bias, scale 2.5, ungated shared expert
    L = synth.make_layer(5, 1024, 64, 256, sh_ff=256, gated_shared=False, bias_std=0.05, router_std=0.05)
    x = synth.activations(21, 8, 1024)
    g = GpuLayer(backend, L)
    kw = dict(scale=2.5, gating=MoeGating.Sigmoid, groups=8, groups_used=4)
    out, ids, wts = g.run(x, 6, **kw)
    ref = oracle_layer(L, x, 6, **kw)
    check_ids(ids, wts, ref, 6)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows", [1, 8])
def test_wide_logit_range(backend, rows):
    # logits spread over hundreds of units: most softmax terms are denormal or zero, which takes the
    # selection off its fast division and onto the full-range one
    L = synth.make_layer(31, 256, 64, 256, router_std=2.0)
    x = synth.activations(33, rows, 256)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 4)
    ref = oracle_layer(L, x, 4)
    lg = x @ L.router.reshape(64, 256).T
    assert (lg.max(1) - lg.min(1)).min() > 110, "the case does not reach the denormal range"
    for r in range(rows):
        assert ids[r].tolist() == ref.ids[r].tolist()
        np.testing.assert_allclose(wts[r], ref.wts[r], rtol=2e-6, atol=1e-12)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows", [1, 8, 40])
def test_sqrt_softplus_gating(backend, rows):
    # DeepSeek-V4 gating: sqrt(ln(1 + exp(v))), the logit itself above 20; router scaled so that both
    # branches occur
    L = synth.make_layer(41, 512, 32, 256, router_std=0.6)
    x = synth.activations(43, rows, 512)
    lg = x @ L.router.reshape(32, 512).T
    assert (lg > 20).any() and (lg < 20).any()
    g = GpuLayer(backend, L)
    kw = dict(gating=MoeGating.SqrtSoftplus, scale=1.5)
    out, ids, wts = g.run(x, 4, **kw)
    ref = oracle_layer(L, x, 4, **kw)
    check_ids(ids, wts, ref, 4)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows,gating", [(1, MoeGating.Softmax), (6, MoeGating.SqrtSoftplus), (40, MoeGating.Softmax)])
def test_caller_selected_experts(backend, rows, gating):
    # hash-routed layers: the experts come from a table; the weights are still the router's own
    # probabilities at those experts
    L = synth.make_layer(45, 512, 32, 256, router_std=0.05)
    x = synth.activations(47, rows, 512)
    rng = np.random.default_rng(5)
    given = np.stack([rng.permutation(32)[:4] for _ in range(rows)]).astype(np.int32)
    g = GpuLayer(backend, L)
    kw = dict(gating=gating, expert_ids=given)
    out, ids, wts = g.run(x, 4, **kw)
    ref = oracle_layer(L, x, 4, **kw)
    assert (ids == given).all() and (ref.ids == given).all()
    np.testing.assert_allclose(wts, ref.wts, rtol=2e-6, atol=1e-9)
    assert_close(out, ref.dst)


def test_caller_selected_experts_refusals(backend):
    L = synth.make_layer(45, 512, 32, 256, bias_std=0.05)
    g = GpuLayer(backend, L)
    x = synth.activations(47, 2, 512)
    given = np.zeros((2, 4), np.int32)
    with pytest.raises(Exception, match="expert_ids excludes"):
        g.run(x, 4, expert_ids=given)
    # an id past n_expert: the CPU panics (crates/infr-cpu/src/lib.rs:3782-3788); here the wait that
    # follows the call fails, and the context stays usable
    L2 = synth.make_layer(45, 512, 32, 256)
    g2 = GpuLayer(backend, L2)
    with pytest.raises(Exception, match="outside"):
        g2.run(x, 4, expert_ids=np.full((2, 4), 40, np.int32))
    out, ids, _ = g2.run(x, 4)
    assert_close(out, oracle_layer(L2, x, 4).dst)


def test_ep_band_partials_sum_to_full(backend):
    # Op::MoeFfn::ep_band: the per-band partial outputs add up to the unbanded output
    L = synth.make_layer(8, 1024, 32, 256)
    x = synth.activations(4, 4, 1024)
    g = GpuLayer(backend, L)
    full, ids, _ = g.run(x, 4)
    parts = [g.run(x, 4, ep_band=(lo, 16))[0] for lo in (0, 16)]
    ref0 = oracle_layer(L, x, 4, ep_band=(0, 16))
    assert_close(parts[0], ref0.dst)
    assert_close(parts[0] + parts[1], full, tol=1e-5)


def test_wide_hidden(backend):
    # ne = 7168 exercises lanes that own several 64-element groups; nff = 2048 several units
    L = synth.make_layer(13, 7168, 16, 2048, sh_ff=2048, gated_shared=False)
    x = synth.activations(2, 2, 7168)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 4, gating=MoeGating.Sigmoid, scale=2.5)
    ref = oracle_layer(L, x, 4, gating=1, scale=2.5)
    check_ids(ids, wts, ref, 4)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows,ne", [(6, 7168), (16, 2048), (33, 1024), (64, 512)])
def test_router_row_groups(backend, rows, ne):
    # calls of more rows than one router CTA holds run as groups of tokens (one selecting CTA and
    # one counter each); at hidden 7168 a group is four rows.  Small-m kernels forced.
    L = synth.make_layer(51, ne, 64, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(53, rows, ne)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 4, path=1)
    ref = oracle_layer(L, x, 4)
    check_ids(ids, wts, ref, 4)
    assert_close(out, ref.dst)


VARIANTS = {
    "gelu": dict(act=1),
    "clamp": dict(swiglu_clamp=0.05),
    "weight_before": dict(weight_before=True, gating=MoeGating.Sigmoid, norm_w=False),
    "down_scale": dict(down_scale=np.linspace(0.5, 1.5, 32).astype(np.float32)),
    "gelu_clamp_scale": dict(act=1, swiglu_clamp=0.08, down_scale=np.linspace(1.5, 0.25, 32).astype(np.float32)),
    "fused_gate_up": dict(fused_gate_up=True, act=1),
    "sigmoid_act": dict(act=2),
}


@pytest.mark.parametrize("rows,path", [(1, 1), (5, 1), (24, 1), (70, 2), (70, 3)])
@pytest.mark.parametrize("variant", sorted(VARIANTS))
def test_op_variants(backend, rows, path, variant):
    # the remaining Op::MoeFfn forms (GELU, SwiGLU clamp, llama4's weight_before, per-expert down
    # scale, gate and up in one bank) through the small-m kernels, the tcgen05 tiles and the mma.sync tiles
    L = synth.make_layer(61, 512, 32, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(63, rows, 512)
    kw = VARIANTS[variant]
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 4, path=path, **kw)
    ref = oracle_layer(L, x, 4, **kw)
    base = oracle_layer(L, x, 4, **{k: v for k, v in kw.items() if k in ("gating", "norm_w")})
    assert rel_err(ref.dst, base.dst)[0] > 1e-2, "the variant does not change the result: the case tests nothing"
    check_ids(ids, wts, ref, 4)
    assert_close(out, ref.dst)


def test_op_variant_refusals(backend):
    L = synth.make_layer(61, 512, 32, 256)
    g = GpuLayer(backend, L)
    x = synth.activations(63, 2, 512)
    with pytest.raises(Exception, match="swiglu_clamp excludes weight_before"):
        g.run(x, 4, swiglu_clamp=1.0, weight_before=True)
    with pytest.raises(Exception, match="act must be"):
        g.run(x, 4, act=3)


@pytest.mark.parametrize("rows,n_expert", [(3, 1024), (12, 600)])
def test_many_experts(backend, rows, n_expert):
    # more router CTAs than SMs (the selecting CTA waits while the rest take turns), 32 experts per
    # lane in the top-k, and with 12 rows two token groups
    L = synth.make_layer(71, 256, n_expert, 256, router_std=0.05)
    x = synth.activations(73, rows, 256)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 8, path=1)
    ref = oracle_layer(L, x, 8)
    check_ids(ids, wts, ref, 8)
    assert_close(out, ref.dst)


@pytest.mark.parametrize("rows,n_expert,ne", [(20, 20, 512), (9, 44, 768), (40, 100, 256)])
def test_streamed_router_ragged_experts(backend, rows, n_expert, ne):
    # 9 .. 64 rows take the streamed router; an expert count that is no multiple of a CTA's eight router
    # rows leaves the last CTA a partial share, a row count that is no multiple of eight a partial group
    L = synth.make_layer(91, ne, n_expert, 256, sh_ff=256, router_std=0.05)
    x = synth.activations(93, rows, ne)
    g = GpuLayer(backend, L)
    out, ids, wts = g.run(x, 3, path=1)
    ref = oracle_layer(L, x, 3)
    check_ids(ids, wts, ref, 3)
    assert_close(out, ref.dst)
    # the caller's selection through the same kernel: weights of the given experts
    given = ref.ids[:, ::-1].copy()
    out2, ids2, wts2 = g.run(x, 3, path=1, expert_ids=given)
    ref2 = oracle_layer(L, x, 3, expert_ids=given)
    assert np.array_equal(ids2, given)
    np.testing.assert_allclose(wts2, ref2.wts, rtol=2e-6, atol=1e-9)
    assert_close(out2, ref2.dst)
