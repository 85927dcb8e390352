"""Host-side mirror of the reference's backend seam over the C ABI (include/infr_cuda.h).

Names and argument meaning follow the reference so that tests read like its own:
`CudaBackend.alloc/upload/download/sync` are `Backend::alloc/upload/download/sync`
(crates/infr-core/src/backend.rs:652-760, 1006), `MoeFfn` carries the fields of `Op::MoeFfn`
(crates/infr-core/src/graph.rs:1259-1352) and `CudaBackend.execute` runs one op the way
`Backend::execute` runs a one-op graph (backend.rs:908).  Errors surface as `BackendError`
(`Error::Backend`) or `Unsupported` (`Error::Unsupported`), crates/infr-core/src/error.rs:11-50.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_lib", "libinfr_cuda.so")

# Every symbol include/infr_cuda.h declares; the loader refuses a library that lacks one.
EXPORTS = [
    "infr_cuda_create", "infr_cuda_destroy", "infr_cuda_last_error", "infr_cuda_name",
    "infr_cuda_set_stream", "infr_cuda_alloc", "infr_cuda_wrap", "infr_cuda_free",
    "infr_cuda_buf_len", "infr_cuda_buf_ptr", "infr_cuda_upload", "infr_cuda_download",
    "infr_cuda_upload_async", "infr_cuda_download_async",
    "infr_cuda_upload_gated", "infr_cuda_host_signal", "infr_cuda_host_ring", "infr_cuda_host_await", "infr_cuda_host_reset", "infr_cuda_host_step", "infr_cuda_host_steps", "infr_cuda_set_codebook",
    "infr_cuda_gguf_open", "infr_cuda_gguf_close", "infr_cuda_gguf_tensor_count", "infr_cuda_gguf_tensor_name", "infr_cuda_gguf_find",
    "infr_cuda_gguf_meta_u64", "infr_cuda_gguf_meta_f64", "infr_cuda_gguf_meta_str", "infr_cuda_gguf_upload",
    "infr_cuda_sync", "infr_cuda_moe_ffn", "infr_cuda_moe_route", "infr_cuda_linear",
    "infr_cuda_gated_act", "infr_cuda_moe_shared_add", "infr_cuda_rmsnorm", "infr_cuda_add",
    "infr_cuda_moe_expert_rows", "infr_cuda_launch_count",
    "infr_cuda_graph_begin", "infr_cuda_graph_end", "infr_cuda_graph_launch", "infr_cuda_graph_free", "infr_cuda_set_trace", "infr_cuda_moe_route_noalloc", "infr_cuda_moe_combine", "infr_cuda_umma_selftest",
    "infr_cuda_get_config", "infr_cuda_set_config",
    "infr_cuda_ep_unique_id", "infr_cuda_ep_init", "infr_cuda_ep_finalize", "infr_cuda_ep_last_phases",
]

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6


class BackendError(RuntimeError):
    """`infr_core::error::Error::Backend`."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"backend: {msg} (status {code})")
        self.code = code


class Unsupported(BackendError):
    """`infr_core::error::Error::Unsupported`: the op, dtype or shape has no CUDA kernel."""


class DType(enum.IntEnum):
    """crates/infr-core/src/tensor.rs:7-57, numbered as in the GGUF file format."""
    F32 = 0
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q2K = 10
    Q3K = 11
    Q4K = 12
    Q5K = 13
    Q6K = 14
    IQ4NL = 20
    IQ4XS = 23
    MXFP4 = 39
    NVFP4 = 40
    Q2_0 = 42
    IQ2XS = 17
    IQ3XXS = 18
    IQ3S = 21
    IQ2S = 22

    def row_bytes(self, n_elem: int) -> int:
        """crates/infr-core/src/decode_spec.rs:315-335: elements and bytes per block."""
        if self is DType.F32:
            return n_elem * 4
        elems, nbytes = {DType.Q8_0: (32, 34), DType.Q4K: (256, 144), DType.Q5K: (256, 176), DType.Q6K: (256, 210),
                         DType.IQ4NL: (32, 18), DType.IQ4XS: (256, 136), DType.Q4_0: (32, 18), DType.Q4_1: (32, 20),
                         DType.Q5_0: (32, 22), DType.Q5_1: (32, 24), DType.Q2K: (256, 84), DType.Q3K: (256, 110), DType.MXFP4: (32, 17),
                         DType.NVFP4: (64, 36), DType.Q2_0: (64, 18), DType.IQ2XS: (256, 74), DType.IQ2S: (256, 82),
                         DType.IQ3XXS: (256, 98), DType.IQ3S: (256, 110)}[self]
        if n_elem % elems:
            raise ValueError(f"{self.name}: {n_elem} elements is not a whole number of {elems}-element blocks")
        return n_elem // elems * nbytes


class MoeGating(enum.IntEnum):
    """crates/infr-core/src/graph.rs:73-85."""
    Softmax = 0
    Sigmoid = 1
    SqrtSoftplus = 2


class Activation(enum.IntEnum):
    """crates/infr-core/src/graph.rs Activation; the gated forms of crates/infr-cpu/src/kernels.rs:6662-6683."""
    Silu = 0
    Gelu = 1
    Sigmoid = 2


class _Desc(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("router_x", C.c_void_p), ("router", C.c_void_p),
        ("gate_exps", C.c_void_p), ("up_exps", C.c_void_p), ("down_exps", C.c_void_p),
        ("exp_probs_b", C.c_void_p), ("dst", C.c_void_p), ("ids_out", C.c_void_p),
        ("wts_out", C.c_void_p),
        ("rows", C.c_uint32), ("ne", C.c_uint32), ("n_expert", C.c_uint32),
        ("n_used", C.c_uint32), ("n_ff_exp", C.c_uint32), ("scale", C.c_float),
        ("router_dtype", C.c_int32), ("gate_dtype", C.c_int32), ("up_dtype", C.c_int32),
        ("down_dtype", C.c_int32), ("gating", C.c_uint32), ("norm_w", C.c_uint32),
        ("n_expert_groups", C.c_uint32), ("n_expert_groups_used", C.c_uint32),
        ("ep_lo", C.c_uint32), ("ep_n_local", C.c_uint32),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
        ("sh_gate_inp", C.c_void_p), ("sh_ff", C.c_uint32), ("path", C.c_uint32),
        ("norm_weight", C.c_void_p), ("residual", C.c_void_p), ("norm_eps", C.c_float),
        ("stages", C.c_uint32), ("expert_ids", C.c_void_p), ("down_scale", C.c_void_p),
        ("act", C.c_uint32), ("weight_before", C.c_uint32), ("swiglu_clamp", C.c_float),
        ("fused_gate_up", C.c_uint32),
    ]


class Config(C.Structure):
    """`infr_cuda_config`: the context's tuning switches (the reference's typed kernel config,
    crates/infr-core/src/config/mod.rs:1-29)."""
    _fields_ = [
        ("gu_warps", C.c_uint32), ("gu_chunks", C.c_uint32), ("dn_warps", C.c_uint32), ("upload_by_copy", C.c_uint32),
        ("trace_tile", C.c_uint32), ("expert_major", C.c_uint32),
        ("sync_timeout_ms", C.c_uint32), ("raw_rows_f32", C.c_uint32), ("gate_timeout_ms", C.c_uint32),
        ("reserved", C.c_uint32 * 7),
    ]


EP_ID_BYTES = 128

_lib = None


def load_library(path: Optional[str] = None):
    """dlopen the CUDA library and bind every exported symbol.  Raises when it is missing:
    there is no other implementation to fall back to."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or _LIB_PATH
    if not os.path.exists(p):
        raise BackendError(ERR_UNSUPPORTED, f"CUDA library not built: {p} (run `python -m moe4all_b200.build`)")
    L = C.CDLL(p)
    missing = [s for s in EXPORTS if not hasattr(L, s)]
    if missing:
        raise BackendError(ERR_UNSUPPORTED, f"{p} lacks symbols: {missing}")
    vp, u32, i32, sz = C.c_void_p, C.c_uint32, C.c_int32, C.c_size_t
    L.infr_cuda_create.argtypes = [i32, C.POINTER(vp)]
    L.infr_cuda_destroy.argtypes = [vp]
    L.infr_cuda_destroy.restype = None
    L.infr_cuda_last_error.argtypes = [vp]
    L.infr_cuda_last_error.restype = C.c_char_p
    L.infr_cuda_name.restype = C.c_char_p
    L.infr_cuda_set_stream.argtypes = [vp, vp]
    L.infr_cuda_alloc.argtypes = [vp, sz, i32, C.POINTER(vp)]
    L.infr_cuda_wrap.argtypes = [vp, vp, sz, C.POINTER(vp)]
    L.infr_cuda_free.argtypes = [vp, vp]
    L.infr_cuda_free.restype = None
    L.infr_cuda_buf_len.argtypes = [vp]
    L.infr_cuda_buf_len.restype = sz
    L.infr_cuda_buf_ptr.argtypes = [vp]
    L.infr_cuda_buf_ptr.restype = vp
    L.infr_cuda_upload.argtypes = [vp, vp, sz, vp, sz]
    L.infr_cuda_download.argtypes = [vp, vp, sz, vp, sz]
    L.infr_cuda_upload_async.argtypes = [vp, vp, sz, vp, sz]
    L.infr_cuda_download_async.argtypes = [vp, vp, sz, vp, sz]
    L.infr_cuda_upload_gated.argtypes = [vp, vp, sz, vp, sz, C.c_uint64]
    L.infr_cuda_host_signal.argtypes = [vp, C.c_uint64]
    L.infr_cuda_host_ring.argtypes = [vp, C.c_uint64]
    L.infr_cuda_host_await.argtypes = [vp, C.c_uint64]
    L.infr_cuda_host_reset.argtypes = [vp]
    L.infr_cuda_set_codebook.argtypes = [vp, C.c_int32, vp, sz]
    L.infr_cuda_host_step.argtypes = [vp, C.c_uint64, vp, vp, sz]
    L.infr_cuda_host_steps.argtypes = [vp, C.c_uint64, C.c_uint32, vp, C.POINTER(C.c_void_p), sz, vp, C.POINTER(C.c_void_p), sz]
    L.infr_cuda_sync.argtypes = [vp]
    L.infr_cuda_moe_ffn.argtypes = [vp, C.POINTER(_Desc)]
    L.infr_cuda_moe_route.argtypes = [vp, C.POINTER(_Desc)]
    L.infr_cuda_linear.argtypes = [vp, i32, vp, vp, vp, u32, u32, u32]
    L.infr_cuda_gated_act.argtypes = [vp, vp, vp, vp, sz]
    L.infr_cuda_moe_shared_add.argtypes = [vp, vp, vp, vp, vp, u32, u32]
    L.infr_cuda_rmsnorm.argtypes = [vp, vp, vp, vp, u32, u32, C.c_float]
    L.infr_cuda_add.argtypes = [vp, vp, vp, vp, sz]
    L.infr_cuda_moe_expert_rows.argtypes = [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, i32, i32, i32]
    L.infr_cuda_graph_begin.argtypes = [vp]
    L.infr_cuda_graph_end.argtypes = [vp, C.POINTER(vp)]
    L.infr_cuda_graph_launch.argtypes = [vp, vp]
    L.infr_cuda_graph_free.argtypes = [vp, vp]
    L.infr_cuda_graph_free.restype = None
    L.infr_cuda_set_trace.argtypes = [vp, vp]
    L.infr_cuda_umma_selftest.argtypes = [vp, vp, vp, vp, u32]
    L.infr_cuda_moe_combine.argtypes = [vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32]
    L.infr_cuda_moe_route_noalloc.argtypes = [i32, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, C.c_float, u32, u32, u32, u32,
                                              C.c_char_p, sz]
    L.infr_cuda_get_config.argtypes = [vp, C.POINTER(Config)]
    L.infr_cuda_set_config.argtypes = [vp, C.POINTER(Config)]
    L.infr_cuda_ep_unique_id.argtypes = [C.c_char_p]
    L.infr_cuda_ep_init.argtypes = [vp, C.c_char_p, i32, i32]
    L.infr_cuda_ep_finalize.argtypes = [vp]
    L.infr_cuda_ep_last_phases.argtypes = [vp, C.POINTER(C.c_float)]
    L.infr_cuda_launch_count.argtypes = [vp]
    L.infr_cuda_launch_count.restype = C.c_uint64
    for name in EXPORTS:
        f = getattr(L, name)
        if f.restype is C.c_int:  # default: every remaining entry point returns an int32 status
            f.restype = i32
    if path is None:
        _lib = L
    return L


class Buffer:
    """`trait Buffer` (backend.rs:423-452): an opaque device allocation owned by the model."""

    def __init__(self, backend: "CudaBackend", handle: int, nbytes: int):
        self._be, self._h, self._n = backend, handle, nbytes

    def len_bytes(self) -> int:
        return self._n

    @property
    def handle(self) -> int:
        return self._h

    @property
    def device_ptr(self) -> int:
        return int(self._be._lib.infr_cuda_buf_ptr(self._h))

    def free(self) -> None:
        if self._h:
            self._be._lib.infr_cuda_free(self._be._ctx, self._h)
            self._h = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Plan:
    """`trait Plan` (backend.rs:468-482): a recorded sequence of ops, replayed by `execute`."""

    def __init__(self, backend: "CudaBackend", handle: int):
        self._be, self._h = backend, handle

    def free(self) -> None:
        if self._h:
            self._be._lib.infr_cuda_graph_free(self._be._ctx, self._h)
            self._h = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _h(buf: Optional[Buffer]):
    return None if buf is None else buf.handle


@dataclass
class MoeFfn:
    """`Op::MoeFfn` (graph.rs:1259-1352) for the forms this backend executes; the optional
    shared-expert fields fold the Linear/GatedAct/Linear/MoeSharedExpertAdd tail of a
    qwen35moe / DeepSeek layer (runner.rs:8088-8175) into the same call."""
    x: Buffer
    router: Buffer
    gate_exps: Buffer
    up_exps: Buffer
    down_exps: Buffer
    dst: Buffer
    rows: int
    ne: int
    n_expert: int
    n_used: int
    n_ff_exp: int
    router_x: Optional[Buffer] = None  # defaults to x
    scale: float = 1.0
    gating: MoeGating = MoeGating.Softmax
    norm_w: bool = True
    exp_probs_b: Optional[Buffer] = None
    n_expert_groups: int = 0
    n_expert_groups_used: int = 0
    ep_band: Optional[tuple] = None  # (lo, n_local)
    router_dtype: DType = DType.F32
    gate_dtype: DType = DType.Q4K
    up_dtype: DType = DType.Q4K
    down_dtype: DType = DType.Q6K
    ids_out: Optional[Buffer] = None
    wts_out: Optional[Buffer] = None
    sh_gate: Optional[Buffer] = None
    sh_up: Optional[Buffer] = None
    sh_down: Optional[Buffer] = None
    sh_gate_inp: Optional[Buffer] = None
    sh_ff: int = 0
    path: int = 0  # 0 auto, 1 small-m kernels, 2 grouped-GEMM kernels
    stages: int = 0  # 0 whole op; mask 1 router+top-k, 2 gate/up, 4 down (timing one kernel alone)
    norm_weight: Optional[Buffer] = None  # RmsNorm -> MoeFfn fusion (fusion.rs:17-25): x is the un-normed row
    norm_eps: float = 1e-6
    residual: Optional[Buffer] = None     # MoeFfn -> Add fusion: added to the result, may be dst itself
    expert_ids: Optional[Buffer] = None   # [rows, n_used] i32 selection made by the caller (graph.rs:1320-1351)
    down_scale: Optional[Buffer] = None   # [n_expert] f32 on the expert's down output (graph.rs:1273-1276)
    act: int = 0                          # Activation
    weight_before: bool = False           # routing weight before the activation (graph.rs:1298-1303)
    swiglu_clamp: float = 0.0             # > 0: clamp gate from above and up on both sides (graph.rs:1283-1290)
    fused_gate_up: bool = False           # gate_exps is [n_expert, 2*n_ff_exp, ne]; up_exps unused (graph.rs:1277-1282)
    _keep: list = field(default_factory=list, repr=False)

    def to_desc(self) -> _Desc:
        d = _Desc()
        d.x = _h(self.x)
        d.router_x = _h(self.router_x if self.router_x is not None else self.x)
        d.router, d.gate_exps, d.up_exps, d.down_exps = _h(self.router), _h(self.gate_exps), _h(self.up_exps), _h(self.down_exps)
        d.exp_probs_b, d.dst, d.ids_out, d.wts_out = _h(self.exp_probs_b), _h(self.dst), _h(self.ids_out), _h(self.wts_out)
        d.rows, d.ne, d.n_expert, d.n_used, d.n_ff_exp = self.rows, self.ne, self.n_expert, self.n_used, self.n_ff_exp
        d.scale = self.scale
        d.router_dtype, d.gate_dtype, d.up_dtype, d.down_dtype = int(self.router_dtype), int(self.gate_dtype), int(self.up_dtype), int(self.down_dtype)
        d.gating, d.norm_w = int(self.gating), int(bool(self.norm_w))
        d.n_expert_groups, d.n_expert_groups_used = self.n_expert_groups, self.n_expert_groups_used
        d.ep_lo, d.ep_n_local = self.ep_band if self.ep_band else (0, 0)
        d.sh_gate, d.sh_up, d.sh_down, d.sh_gate_inp = _h(self.sh_gate), _h(self.sh_up), _h(self.sh_down), _h(self.sh_gate_inp)
        d.sh_ff, d.path, d.stages = self.sh_ff, self.path, self.stages
        d.norm_weight, d.residual, d.norm_eps = _h(self.norm_weight), _h(self.residual), self.norm_eps
        d.expert_ids = _h(self.expert_ids)
        d.down_scale, d.act = _h(self.down_scale), int(self.act)
        d.weight_before, d.swiglu_clamp = int(bool(self.weight_before)), float(self.swiglu_clamp)
        d.fused_gate_up = int(bool(self.fused_gate_up))
        d._op = self  # the descriptor holds raw handle pointers: the op (and its Buffer objects) must outlive it
        return d


class CudaBackend:
    """`impl Backend for …` over the C ABI: one device, one stream, calls serialised by the
    caller (backend.rs:891-899)."""

    def __init__(self, device: int = 0, lib_path: Optional[str] = None):
        self._lib = load_library(lib_path)
        ctx = C.c_void_p()
        rc = self._lib.infr_cuda_create(device, C.byref(ctx))
        if rc != OK:
            cls = Unsupported if rc == ERR_UNSUPPORTED else BackendError
            raise cls(rc, f"infr_cuda_create(device={device}) failed")
        self._ctx = ctx
        self.device = device

    # -- plumbing --------------------------------------------------------------------------------
    def _check(self, rc: int) -> None:
        if rc == OK:
            return
        msg = self._lib.infr_cuda_last_error(self._ctx).decode("utf-8", "replace")
        raise (Unsupported if rc == ERR_UNSUPPORTED else BackendError)(rc, msg)

    def close(self) -> None:
        if getattr(self, "_ctx", None):
            self._lib.infr_cuda_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- Backend ---------------------------------------------------------------------------------
    def name(self) -> str:
        return self._lib.infr_cuda_name().decode()

    def alloc(self, nbytes: int) -> Buffer:
        """Zero-initialised (the calloc contract of backend.rs:647-651)."""
        h = C.c_void_p()
        self._check(self._lib.infr_cuda_alloc(self._ctx, nbytes, 1, C.byref(h)))
        return Buffer(self, h.value, nbytes)

    def alloc_uninit(self, nbytes: int) -> Buffer:
        h = C.c_void_p()
        self._check(self._lib.infr_cuda_alloc(self._ctx, nbytes, 0, C.byref(h)))
        return Buffer(self, h.value, nbytes)

    def wrap(self, device_ptr: int, nbytes: int) -> Buffer:
        """A handle on device memory someone else owns (a torch tensor's storage)."""
        h = C.c_void_p()
        self._check(self._lib.infr_cuda_wrap(self._ctx, device_ptr, nbytes, C.byref(h)))
        return Buffer(self, h.value, nbytes)

    def wrap_tensor(self, t) -> Buffer:
        if not t.is_cuda or not t.is_contiguous():
            raise ValueError("wrap_tensor wants a contiguous CUDA tensor")
        b = self.wrap(t.data_ptr(), t.numel() * t.element_size())
        b._owner = t  # keep the storage alive as long as the handle
        return b

    def set_stream(self, cuda_stream: int) -> None:
        self._check(self._lib.infr_cuda_set_stream(self._ctx, cuda_stream))

    def upload(self, dst: Buffer, src, offset: int = 0) -> None:
        a = np.ascontiguousarray(src)
        self._check(self._lib.infr_cuda_upload(self._ctx, dst.handle, offset, a.ctypes.data_as(C.c_void_p), a.nbytes))

    def upload_ptr(self, dst: Buffer, host_ptr: int, nbytes: int, offset: int = 0) -> None:
        self._check(self._lib.infr_cuda_upload(self._ctx, dst.handle, offset, host_ptr, nbytes))

    def upload_ptr_async(self, dst: Buffer, host_ptr: int, nbytes: int, offset: int = 0) -> None:
        """Queued copy: the host range must stay untouched until `sync()`."""
        self._check(self._lib.infr_cuda_upload_async(self._ctx, dst.handle, offset, host_ptr, nbytes))

    # -- host-paced plans: steps recorded once, launched once, paced through two words in pinned memory --
    def upload_ptr_gated(self, dst: Buffer, host_ptr: int, nbytes: int, ticket: int, offset: int = 0) -> None:
        """Queued fetch of pinned host rows that first waits (bounded) until the host has rung `ticket`."""
        self._check(self._lib.infr_cuda_upload_gated(self._ctx, dst.handle, offset, host_ptr, nbytes, ticket))

    def host_signal(self, ticket: int) -> None:
        """Queued: publish `ticket` to the host once everything queued before it has finished."""
        self._check(self._lib.infr_cuda_host_signal(self._ctx, ticket))

    def host_ring(self, ticket: int) -> None:
        """Host side: the rows of step `ticket` are in pinned memory, let its gated fetch go."""
        self._check(self._lib.infr_cuda_host_ring(self._ctx, ticket))

    def host_await(self, ticket: int) -> None:
        """Host side: spin until `ticket` has been signalled (bounded; raises on a recorded device status)."""
        self._check(self._lib.infr_cuda_host_await(self._ctx, ticket))

    def host_step(self, ticket: int, stage_ptr: int, rows_ptr: int, nbytes: int) -> None:
        """One step in one call: rows -> pinned staging range, ring, await."""
        self._check(self._lib.infr_cuda_host_step(self._ctx, ticket, stage_ptr, rows_ptr, nbytes))

    def host_steps(self, first_ticket: int, stage_ptr: int, row_ptrs, nbytes_in: int, result_ptr: int = 0, result_out_ptrs=None,
                   nbytes_out: int = 0) -> None:
        """`len(row_ptrs)` consecutive steps in one call (inputs known in advance); each step's result is copied
        from the pinned range `result_ptr` to `result_out_ptrs[i]` when given."""
        n = len(row_ptrs)
        rows = (C.c_void_p * n)(*row_ptrs)
        outs = (C.c_void_p * n)(*result_out_ptrs) if result_out_ptrs is not None else None
        self._check(self._lib.infr_cuda_host_steps(self._ctx, first_ticket, n, stage_ptr, rows, nbytes_in, result_ptr or None, outs, nbytes_out))

    def host_reset(self) -> None:
        """Drain the stream and set both pacing words back to zero (before a plan whose tickets restart at 1)."""
        self._check(self._lib.infr_cuda_host_reset(self._ctx))

    def download_ptr_async(self, src: Buffer, host_ptr: int, nbytes: int, offset: int = 0) -> None:
        """Queued copy: the host range holds the data after `sync()`."""
        self._check(self._lib.infr_cuda_download_async(self._ctx, src.handle, offset, host_ptr, nbytes))

    def download(self, src: Buffer, dtype=np.float32, count: Optional[int] = None, offset: int = 0) -> np.ndarray:
        itemsize = np.dtype(dtype).itemsize
        n = (src.len_bytes() - offset) // itemsize if count is None else count
        out = np.empty(n, dtype=dtype)
        self._check(self._lib.infr_cuda_download(self._ctx, src.handle, offset, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def download_ptr(self, src: Buffer, host_ptr: int, nbytes: int, offset: int = 0) -> None:
        self._check(self._lib.infr_cuda_download(self._ctx, src.handle, offset, host_ptr, nbytes))

    def sync(self) -> None:
        self._check(self._lib.infr_cuda_sync(self._ctx))

    def from_host(self, array) -> Buffer:
        a = np.ascontiguousarray(array)
        b = self.alloc_uninit(max(a.nbytes, 16))
        b._n = a.nbytes
        self.upload(b, a)
        return b

    # -- tuning switches ------------------------------------------------------------------------
    def set_codebook(self, dtype: "DType", table: np.ndarray) -> None:
        """Hand over the grid table of a codebook format (IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S) as its little-endian bytes."""
        t = np.ascontiguousarray(table).view(np.uint8).reshape(-1)
        self._check(self._lib.infr_cuda_set_codebook(self._ctx, int(dtype), t.ctypes.data_as(C.c_void_p), t.nbytes))

    def get_config(self) -> Config:
        c = Config()
        self._check(self._lib.infr_cuda_get_config(self._ctx, C.byref(c)))
        return c

    def set_config(self, **fields) -> Config:
        """Change the named fields of the context's config; returns the config now in force."""
        c = self.get_config()
        for k, v in fields.items():
            if not hasattr(c, k) or k == "reserved":
                raise ValueError(f"no such config field: {k}")
            setattr(c, k, int(v))
        self._check(self._lib.infr_cuda_set_config(self._ctx, C.byref(c)))
        return c

    # -- expert parallelism (crates/infr-vulkan/src/ep.rs) ------------------------------------------
    def ep_unique_id(self) -> bytes:
        """Rank 0 makes the communicator id; the host hands it to the other ranks."""
        buf = C.create_string_buffer(EP_ID_BYTES)
        rc = self._lib.infr_cuda_ep_unique_id(buf)
        if rc != OK:
            raise (Unsupported if rc == ERR_UNSUPPORTED else BackendError)(rc, "ep_unique_id failed (is libnccl.so.2 loadable?)")
        return buf.raw

    def ep_init(self, unique_id: bytes, rank: int, world: int) -> None:
        """Joins the communicator (collective).  After it, a `MoeFfn` whose `ep_band` is this rank's
        band runs expert-parallel inside the library."""
        if len(unique_id) != EP_ID_BYTES:
            raise ValueError("unique_id must be 128 bytes")
        self._check(self._lib.infr_cuda_ep_init(self._ctx, unique_id, rank, world))
        self.ep_rank, self.ep_world = rank, world

    def ep_finalize(self) -> None:
        self._check(self._lib.infr_cuda_ep_finalize(self._ctx))

    def ep_last_phases(self):
        """ms from the call's start: routed, dispatched, band done, partials back, result written."""
        out = (C.c_float * 5)()
        self._check(self._lib.infr_cuda_ep_last_phases(self._ctx, out))
        return [float(v) for v in out]

    def set_trace(self, buf: Optional[Buffer]) -> None:
        self._check(self._lib.infr_cuda_set_trace(self._ctx, _h(buf)))

    def launch_count(self) -> int:
        return int(self._lib.infr_cuda_launch_count(self._ctx))

    # -- record once, replay (Backend::compile + decode replay) ----------------------------------
    def graph_begin(self) -> None:
        self._check(self._lib.infr_cuda_graph_begin(self._ctx))

    def graph_end(self) -> "Plan":
        h = C.c_void_p()
        self._check(self._lib.infr_cuda_graph_end(self._ctx, C.byref(h)))
        return Plan(self, h.value)

    def execute(self, plan: "Plan") -> None:
        """`Backend::execute(plan, bindings)` for a recorded plan (backend.rs:908)."""
        self._check(self._lib.infr_cuda_graph_launch(self._ctx, plan._h))

    # -- ops (Backend::execute of a one-op graph) ----------------------------------------------------
    def moe_ffn(self, op: MoeFfn) -> None:
        d = op.to_desc()
        self._check(self._lib.infr_cuda_moe_ffn(self._ctx, C.byref(d)))

    def moe_route(self, op: MoeFfn) -> None:
        d = op.to_desc()
        self._check(self._lib.infr_cuda_moe_route(self._ctx, C.byref(d)))

    def moe_expert_rows(self, x_rows: Buffer, seg_off: Buffer, gate_exps: Buffer, up_exps: Buffer, down_exps: Buffer,
                        y_rows: Buffer, n_rows: int, n_local: int, ne: int, n_ff_exp: int,
                        gate_dtype: DType = DType.Q4K, up_dtype: DType = DType.Q4K, down_dtype: DType = DType.Q6K) -> None:
        """Expert FFN over rows already grouped by local expert (what an expert-parallel rank runs
        between the dispatch and the combine exchange, crates/infr-vulkan/src/ep.rs:454-493)."""
        self._check(self._lib.infr_cuda_moe_expert_rows(self._ctx, x_rows.handle, seg_off.handle, gate_exps.handle,
                                                        up_exps.handle, down_exps.handle, y_rows.handle, n_rows, n_local,
                                                        ne, n_ff_exp, int(gate_dtype), int(up_dtype), int(down_dtype)))

    def moe_combine(self, y_rows: Buffer, pos_of_pair: Buffer, wts: Buffer, dst: Buffer, rows: int, n_used: int, ne: int,
                    n_y_rows: int, sh_rows: Optional[Buffer] = None, sh_logit: Optional[Buffer] = None) -> None:
        """Rank-ordered weighted sum of per-pair expert outputs plus the shared expert."""
        self._check(self._lib.infr_cuda_moe_combine(self._ctx, y_rows.handle, pos_of_pair.handle, wts.handle, _h(sh_rows),
                                                    _h(sh_logit), dst.handle, rows, n_used, ne, n_y_rows))

    def linear(self, dtype: DType, w: Buffer, x: Buffer, y: Buffer, m: int, in_f: int, out_f: int) -> None:
        self._check(self._lib.infr_cuda_linear(self._ctx, int(dtype), w.handle, x.handle, y.handle, m, in_f, out_f))

    def gated_act(self, gate: Buffer, up: Buffer, dst: Buffer, n: int) -> None:
        self._check(self._lib.infr_cuda_gated_act(self._ctx, gate.handle, up.handle, dst.handle, n))

    def moe_shared_expert_add(self, moe: Buffer, shexp: Buffer, gate: Buffer, dst: Buffer, rows: int, n: int) -> None:
        self._check(self._lib.infr_cuda_moe_shared_add(self._ctx, moe.handle, shexp.handle, gate.handle, dst.handle, rows, n))

    def rms_norm(self, x: Buffer, weight: Buffer, dst: Buffer, rows: int, dim: int, eps: float) -> None:
        self._check(self._lib.infr_cuda_rmsnorm(self._ctx, x.handle, weight.handle, dst.handle, rows, dim, eps))

    def add(self, a: Buffer, b: Buffer, dst: Buffer, n: int) -> None:
        self._check(self._lib.infr_cuda_add(self._ctx, a.handle, b.handle, dst.handle, n))
