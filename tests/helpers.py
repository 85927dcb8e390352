"""Shared pieces of the parity tests: run one MoE layer through the CUDA library (via the C ABI)
and through the CPU oracle on the same bytes, and score with the reference's own metric
(crates/infr-testkit/src/lib.rs:372-386: rel = max|got - want| / max(max|want|, 1e-3); an
all-zero oracle is a failure, :250-253)."""
from __future__ import annotations

import numpy as np

from moe4all_b200 import DType, MoeFfn, MoeGating
from oracle import oracle as orc

TOL_REL = 2e-3  # stated bound on layer outputs against the CPU reference


def rel_err(got: np.ndarray, want: np.ndarray):
    got = np.asarray(got, np.float32).reshape(-1)
    want = np.asarray(want, np.float32).reshape(-1)
    assert got.shape == want.shape
    ref_mag = float(np.max(np.abs(want)))
    abs_err = float(np.max(np.abs(got - want)))
    return abs_err / max(ref_mag, 1e-3), ref_mag


def assert_close(got, want, tol=TOL_REL, what="output"):
    assert np.all(np.isfinite(got)), f"{what}: non-finite values from the GPU"
    rel, mag = rel_err(got, want)
    assert mag > 0.0, f"{what}: oracle output is all zero, the case is vacuous"
    assert rel <= tol, f"{what}: rel err {rel:.3e} > {tol:.1e} (ref magnitude {mag:.3e})"
    return rel


def fused_bank(L):
    """gate and up banks as one [n_expert, 2*n_ff, row bytes] bank: an expert's gate rows, then its up rows."""
    g = np.asarray(L.gate, np.uint8).reshape(L.n_expert, -1)
    u = np.asarray(L.up, np.uint8).reshape(L.n_expert, -1)
    return np.ascontiguousarray(np.concatenate([g, u], axis=1)).reshape(-1)


class GpuLayer:
    """Device copies of a synth.LayerWeights."""

    def __init__(self, be, L):
        self.be, self.L = be, L
        self.router = be.from_host(L.router)
        self.gate, self.up, self.down = be.from_host(L.gate), be.from_host(L.up), be.from_host(L.down)
        self.sh_gate = be.from_host(L.sh_gate) if L.sh_gate is not None else None
        self.sh_up = be.from_host(L.sh_up) if L.sh_up is not None else None
        self.sh_down = be.from_host(L.sh_down) if L.sh_down is not None else None
        self.sh_gate_inp = be.from_host(L.sh_gate_inp) if L.sh_gate_inp is not None else None
        self.bias = be.from_host(L.bias) if L.bias is not None else None

    def run(self, x, n_used, *, router_x=None, scale=1.0, gating=MoeGating.Softmax, norm_w=True,
            groups=0, groups_used=0, ep_band=None, shared=True, path=0, expert_ids=None, down_scale=None,
            act=0, weight_before=False, swiglu_clamp=0.0, fused_gate_up=False):
        be, L = self.be, self.L
        x = np.ascontiguousarray(x, np.float32)
        rows = x.shape[0]
        xb = be.from_host(x)
        rxb = be.from_host(np.ascontiguousarray(router_x, np.float32)) if router_x is not None else None
        dst = be.alloc(rows * L.ne * 4)
        ids = be.alloc(rows * n_used * 4)
        wts = be.alloc(rows * n_used * 4)
        use_sh = shared and self.sh_gate is not None
        given = be.from_host(np.ascontiguousarray(expert_ids, np.int32)) if expert_ids is not None else None
        dsc = be.from_host(np.ascontiguousarray(down_scale, np.float32)) if down_scale is not None else None
        gate_b, up_b = self.gate, self.up
        if fused_gate_up:  # one bank, an expert's gate rows then its up rows; up_exps gets the same handle and is not read
            gate_b = up_b = be.from_host(fused_bank(L))
        op = MoeFfn(x=xb, router_x=rxb, router=self.router, gate_exps=gate_b, up_exps=up_b,
                    down_exps=self.down, dst=dst, rows=rows, ne=L.ne, n_expert=L.n_expert,
                    n_used=n_used, n_ff_exp=L.n_ff, scale=scale, gating=gating, norm_w=norm_w,
                    exp_probs_b=self.bias, n_expert_groups=groups, n_expert_groups_used=groups_used,
                    ep_band=ep_band, ids_out=ids, wts_out=wts,
                    sh_gate=self.sh_gate if use_sh else None, sh_up=self.sh_up if use_sh else None,
                    sh_down=self.sh_down if use_sh else None,
                    sh_gate_inp=self.sh_gate_inp if use_sh else None,
                    sh_ff=L.sh_ff if use_sh else 0, path=path, down_dtype=DType(getattr(L, "down_dtype", 14)),
                    gate_dtype=DType(getattr(L, "gate_dtype", 12)), up_dtype=DType(getattr(L, "up_dtype", 12)),
                    expert_ids=given, down_scale=dsc, act=act, weight_before=weight_before, swiglu_clamp=swiglu_clamp,
                    fused_gate_up=fused_gate_up)
        be.moe_ffn(op)
        be.sync()
        out = be.download(dst, np.float32).reshape(rows, L.ne)
        return out, be.download(ids, np.int32).reshape(rows, n_used), be.download(wts, np.float32).reshape(rows, n_used)


def oracle_layer(L, x, n_used, *, router_x=None, scale=1.0, gating=0, norm_w=True, groups=0,
                 groups_used=0, ep_band=None, shared=True, threads=0, expert_ids=None, down_scale=None, act=0,
                 weight_before=False, swiglu_clamp=0.0, fused_gate_up=False):
    kw = dict(n_expert=L.n_expert, n_used=n_used, n_ff_exp=L.n_ff, scale=scale, gating=int(gating),
              norm_w=norm_w, bias=L.bias, groups=groups, groups_used=groups_used, ep_band=ep_band,
              threads=threads, router_x=router_x, down_dtype=getattr(L, "down_dtype", 14), gate_dtype=getattr(L, "gate_dtype", 12),
              up_dtype=getattr(L, "up_dtype", 12), expert_ids=expert_ids,
              down_scale=down_scale, act=int(act), weight_before=weight_before, swiglu_clamp=swiglu_clamp,
              fused_gate_up=fused_gate_up)
    gate = fused_bank(L) if fused_gate_up else L.gate
    if shared and L.sh_gate is not None:
        return orc.moe_layer(x, L.router, gate, L.up, L.down, L.sh_gate, L.sh_up, L.sh_down,
                             L.sh_gate_inp, L.sh_ff, **kw)
    return orc.moe_ffn(x, L.router, gate, L.up, L.down, **kw)


def near_tie_rows(res, n_used, ulps=8):
    """Rows whose selection is within a few ulps of flipping in the oracle: the k-th and (k+1)-th
    selection scores (or two neighbours inside the top-k) nearly coincide.  The GPU's exp is
    correctly rounded while libm's may differ in the last bit, so only these rows may legitimately
    differ in ids."""
    sel = np.sort(res.sel, axis=1)[:, ::-1][:, : n_used + 1].astype(np.float64)
    gap = sel[:, :-1] - sel[:, 1:]
    scale = np.maximum(np.abs(sel[:, :-1]), 1e-30)
    eps = np.finfo(np.float32).eps
    return np.where((gap <= ulps * eps * scale).any(axis=1))[0]
