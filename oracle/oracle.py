"""ctypes front-end of the CPU oracle (oracle/moe_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's
CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libmoe_oracle.so")

DT_F32, DT_Q4K, DT_Q6K = 0, 12, 14
DT_Q8_0, DT_Q5K = 8, 13
DT_IQ4NL, DT_IQ4XS, DT_MXFP4, DT_NVFP4, DT_Q2_0 = 20, 23, 39, 40, 42
DT_IQ2XS, DT_IQ3XXS, DT_IQ3S, DT_IQ2S = 17, 18, 21, 22
DT_Q4_0, DT_Q4_1, DT_Q5_0, DT_Q5_1, DT_Q2K, DT_Q3K = 2, 3, 6, 7, 10, 11
GATING_SOFTMAX, GATING_SIGMOID, GATING_SQRT_SOFTPLUS = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (g++, -ffp-contract=off)."""
    src = os.path.join(_HERE, "moe_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


class _Desc(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("router_x", C.c_void_p), ("router", C.c_void_p),
        ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
        ("exp_probs_b", C.c_void_p), ("dst", C.c_void_p), ("ids_out", C.c_void_p),
        ("wts_out", C.c_void_p), ("logits_out", C.c_void_p), ("sel_out", C.c_void_p),
        ("rows", C.c_uint32), ("ne", C.c_uint32), ("n_expert", C.c_uint32),
        ("n_used", C.c_uint32), ("n_ff_exp", C.c_uint32), ("scale", C.c_float),
        ("router_dtype", C.c_int32), ("gate_dtype", C.c_int32), ("up_dtype", C.c_int32),
        ("down_dtype", C.c_int32), ("gating", C.c_uint32), ("norm_w", C.c_uint32),
        ("n_expert_groups", C.c_uint32), ("n_expert_groups_used", C.c_uint32),
        ("ep_lo", C.c_uint32), ("ep_n_local", C.c_uint32), ("threads", C.c_int32),
        ("expert_ids", C.c_void_p), ("down_scale", C.c_void_p), ("act", C.c_uint32),
        ("weight_before", C.c_uint32), ("swiglu_clamp", C.c_float), ("fused_gate_up", C.c_uint32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_int, C.c_size_t]
        L.orc_dequant.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
        L.orc_set_codebook.argtypes = [C.c_int, C.c_void_p, C.c_size_t]
        L.orc_dot.restype = C.c_float
        L.orc_dot.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_dot_scalar.restype = C.c_float
        L.orc_dot_scalar.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_moe_ffn.argtypes = [C.POINTER(_Desc)]
        L.orc_linear.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                 C.c_uint32, C.c_void_p, C.c_int32]
        L.orc_gated_act_silu.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_moe_shared_add.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_uint32, C.c_uint32]
        L.orc_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                  C.c_float]
        L.orc_add.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]
        L.orc_moe_layer.argtypes = [C.POINTER(_Desc), C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_void_p, C.c_uint32, C.c_void_p]
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint8).reshape(-1)


def hw_threads() -> int:
    return int(lib().orc_hw_threads())


def set_codebook(dtype: int, table: np.ndarray) -> None:
    """Hand in the grid table of a codebook format (IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S) as its little-endian bytes."""
    t = np.ascontiguousarray(table).view(np.uint8).reshape(-1)
    if lib().orc_set_codebook(dtype, _p(t), t.nbytes) != 0:
        raise ValueError(f"dtype {dtype}: not a grid codebook format, or a table of the wrong size")


def row_bytes(dtype: int, n_elem: int) -> int:
    return int(lib().orc_row_bytes(dtype, n_elem))


def dequant(dtype: int, raw, n_elem: int) -> np.ndarray:
    raw = _u8(raw)
    out = np.empty(n_elem, dtype=np.float32)
    if lib().orc_dequant(dtype, _p(raw), n_elem, _p(out)) != 0:
        raise ValueError("oracle: unsupported dtype or ragged block count")
    return out


def dot(a, b, scalar: bool = False) -> np.float32:
    a, b = _f32(a), _f32(b)
    n = min(a.size, b.size)
    f = lib().orc_dot_scalar if scalar else lib().orc_dot
    return np.float32(f(_p(a), _p(b), n))


@dataclass
class MoeResult:
    dst: np.ndarray
    ids: np.ndarray
    wts: np.ndarray
    logits: np.ndarray
    sel: np.ndarray


def _desc(x, router_x, router, gate, up, down, *, n_expert, n_used, n_ff_exp, scale=1.0,
          router_dtype=DT_F32, gate_dtype=DT_Q4K, up_dtype=DT_Q4K, down_dtype=DT_Q6K,
          gating=GATING_SOFTMAX, norm_w=True, bias=None, groups=0, groups_used=0,
          ep_band=None, threads=0, expert_ids=None, down_scale=None, act=0, weight_before=False,
          swiglu_clamp=0.0, fused_gate_up=False):
    x = _f32(x)
    rows, ne = x.shape
    router_x = x if router_x is None else _f32(router_x)
    keep = dict(x=x, router_x=router_x, router=_u8(router), gate=_u8(gate), up=_u8(up),
                down=_u8(down), bias=None if bias is None else _f32(bias),
                dscale=None if down_scale is None else _f32(down_scale),
                given=None if expert_ids is None else np.ascontiguousarray(expert_ids, np.int32).reshape(rows, n_used),
                dst=np.zeros((rows, ne), np.float32), ids=np.zeros((rows, n_used), np.int32),
                wts=np.zeros((rows, n_used), np.float32),
                logits=np.zeros((rows, n_expert), np.float32),
                sel=np.zeros((rows, n_expert), np.float32))
    d = _Desc()
    d.x, d.router_x, d.router = _p(keep["x"]), _p(keep["router_x"]), _p(keep["router"])
    d.gate_exps, d.up_exps, d.down_exps = _p(keep["gate"]), _p(keep["up"]), _p(keep["down"])
    d.exp_probs_b = _p(keep["bias"])
    d.dst, d.ids_out, d.wts_out = _p(keep["dst"]), _p(keep["ids"]), _p(keep["wts"])
    d.logits_out, d.sel_out = _p(keep["logits"]), _p(keep["sel"])
    d.rows, d.ne, d.n_expert, d.n_used, d.n_ff_exp = rows, ne, n_expert, n_used, n_ff_exp
    d.scale = scale
    d.router_dtype, d.gate_dtype, d.up_dtype, d.down_dtype = router_dtype, gate_dtype, up_dtype, down_dtype
    d.gating, d.norm_w = gating, int(bool(norm_w))
    d.n_expert_groups, d.n_expert_groups_used = groups, groups_used
    d.ep_lo, d.ep_n_local = (ep_band if ep_band else (0, 0))
    d.threads = threads
    d.expert_ids = _p(keep["given"])
    d.fused_gate_up = int(bool(fused_gate_up))
    d.down_scale, d.act, d.weight_before, d.swiglu_clamp = _p(keep["dscale"]), int(act), int(bool(weight_before)), float(swiglu_clamp)
    return d, keep


def moe_ffn(x, router, gate, up, down, *, router_x=None, **kw) -> MoeResult:
    """Op::MoeFfn in the reference's f32 reference mode.  x: [rows, ne] f32."""
    d, keep = _desc(x, router_x, router, gate, up, down, **kw)
    rc = lib().orc_moe_ffn(C.byref(d))
    if rc != 0:
        raise ValueError(f"oracle moe_ffn rejected the descriptor (rc={rc})")
    return MoeResult(keep["dst"], keep["ids"], keep["wts"], keep["logits"], keep["sel"])


def moe_layer(x, router, gate, up, down, sh_gate, sh_up, sh_down, sh_gate_inp, sh_ff, *,
              router_x=None, **kw) -> MoeResult:
    """MoeFfn + shared expert (sigmoid-gated when sh_gate_inp is given, plain sum otherwise)."""
    d, keep = _desc(x, router_x, router, gate, up, down, **kw)
    out = np.zeros_like(keep["dst"])
    sg = None if sh_gate is None else _u8(sh_gate)
    su = None if sh_up is None else _u8(sh_up)
    sd = None if sh_down is None else _u8(sh_down)
    gi = None if sh_gate_inp is None else _f32(sh_gate_inp)
    rc = lib().orc_moe_layer(C.byref(d), _p(sg), _p(su), _p(sd), _p(gi), sh_ff, _p(out))
    if rc != 0:
        raise ValueError(f"oracle moe_layer rejected the descriptor (rc={rc})")
    return MoeResult(out, keep["ids"], keep["wts"], keep["logits"], keep["sel"])


def linear(dtype: int, w, x, out_f: int, threads: int = 0) -> np.ndarray:
    x = _f32(x)
    m, in_f = x.shape
    w = _u8(w)
    y = np.zeros((m, out_f), np.float32)
    if lib().orc_linear(dtype, _p(w), _p(x), m, in_f, out_f, _p(y), threads) != 0:
        raise ValueError("oracle linear: unsupported dtype")
    return y


def gated_act_silu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().orc_gated_act_silu(_p(gate), _p(up), _p(out), gate.size)
    return out


def moe_shared_add(moe, shexp, gate) -> np.ndarray:
    moe, shexp, gate = _f32(moe), _f32(shexp), _f32(gate)
    rows, n = moe.shape
    out = np.empty_like(moe)
    lib().orc_moe_shared_add(_p(moe), _p(shexp), _p(gate), _p(out), rows, n)
    return out


def rmsnorm(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    rows, dim = x.shape
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(w), _p(out), rows, dim, eps)
    return out


def add(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().orc_add(_p(a), _p(b), _p(out), a.size)
    return out
