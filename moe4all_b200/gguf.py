"""MoE FFN tensors straight from a GGUF model file (ctypes mirror of the `infr_cuda_gguf_*` entry
points).  The reference's loader is crates/infr-gguf/src/lib.rs:443-1000; tensor names and which
of them a layer has follow crates/infr-llama/src/seam/runner.rs:2560-2595.  Bytes go to the device
exactly as the file stores them."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
import os
import re
from typing import Dict, List, Optional, Tuple

from .backend import BackendError, Buffer, CudaBackend, DType, ERR_INVALID_ARG, MoeFfn, load_library


class _Tensor(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("offset", C.c_uint64),
                ("nbytes", C.c_uint64)]


@dataclass
class TensorInfo:
    dtype: int
    dims: Tuple[int, ...]   # GGUF order: fastest axis first
    offset: int
    nbytes: int


def _bind(L):
    vp = C.c_void_p
    L.infr_cuda_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp), C.c_char_p, C.c_size_t]
    L.infr_cuda_gguf_close.argtypes = [vp]
    L.infr_cuda_gguf_close.restype = None
    L.infr_cuda_gguf_tensor_count.argtypes = [vp]
    L.infr_cuda_gguf_tensor_count.restype = C.c_uint64
    L.infr_cuda_gguf_tensor_name.argtypes = [vp, C.c_uint64, C.c_char_p, C.c_size_t]
    L.infr_cuda_gguf_find.argtypes = [vp, C.c_char_p, C.POINTER(_Tensor)]
    L.infr_cuda_gguf_meta_u64.argtypes = [vp, C.c_char_p, C.POINTER(C.c_uint64)]
    L.infr_cuda_gguf_meta_f64.argtypes = [vp, C.c_char_p, C.POINTER(C.c_double)]
    L.infr_cuda_gguf_meta_str.argtypes = [vp, C.c_char_p, C.c_char_p, C.c_size_t]
    L.infr_cuda_gguf_upload.argtypes = [vp, vp, C.c_char_p, C.POINTER(vp)]
    return L


class GgufFile:
    """A parsed model file.  Opening needs no GPU; `upload` needs a backend."""

    def __init__(self, path: str):
        self._lib = _bind(load_library())
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        rc = self._lib.infr_cuda_gguf_open(path.encode(), C.byref(h), err, len(err))
        if rc:
            raise BackendError(rc, err.value.decode(errors="replace") or "GGUF: open failed")
        self._h = h

    def close(self) -> None:
        if self._h:
            self._lib.infr_cuda_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensor_count(self) -> int:
        return int(self._lib.infr_cuda_gguf_tensor_count(self._h))

    def tensor_names(self) -> List[str]:
        out, b = [], C.create_string_buffer(512)
        for i in range(self.tensor_count()):
            if self._lib.infr_cuda_gguf_tensor_name(self._h, i, b, len(b)):
                raise BackendError(ERR_INVALID_ARG, f"GGUF: tensor {i} has no readable name")
            out.append(b.value.decode())
        return out

    def find(self, name: str) -> Optional[TensorInfo]:
        t = _Tensor()
        if self._lib.infr_cuda_gguf_find(self._h, name.encode(), C.byref(t)):
            return None
        return TensorInfo(int(t.dtype), tuple(int(t.dims[i]) for i in range(t.n_dims)), int(t.offset), int(t.nbytes))

    def meta_u64(self, key: str) -> Optional[int]:
        v = C.c_uint64()
        return None if self._lib.infr_cuda_gguf_meta_u64(self._h, key.encode(), C.byref(v)) else int(v.value)

    def meta_f64(self, key: str) -> Optional[float]:
        v = C.c_double()
        return None if self._lib.infr_cuda_gguf_meta_f64(self._h, key.encode(), C.byref(v)) else float(v.value)

    def meta_str(self, key: str) -> Optional[str]:
        b = C.create_string_buffer(256)
        return None if self._lib.infr_cuda_gguf_meta_str(self._h, key.encode(), b, len(b)) else b.value.decode()

    def upload(self, be: CudaBackend, name: str) -> Buffer:
        h = C.c_void_p()
        be._check(self._lib.infr_cuda_gguf_upload(be._ctx, self._h, name.encode(), C.byref(h)))
        info = self.find(name)
        return Buffer(be, h.value, info.nbytes + 16)


# ---- split models (llama.cpp gguf-split): <base>-NNNNN-of-MMMMM.gguf ---------------------------------------

_SHARD = re.compile(r"^(?P<base>.*)-(?P<idx>\d{1,5})-of-(?P<total>\d{1,5})\.gguf$", re.IGNORECASE)


def parse_shard(fname: str) -> Optional[Tuple[str, int, int, int]]:
    """(base, one-based index, total, field width) of a shard file name, or None (crates/infr-core/src/gguf_split.rs:
    42-67: both number fields all digits, equally wide, at most five digits)."""
    m = _SHARD.match(fname)
    if not m or len(m["idx"]) != len(m["total"]):
        return None
    return m["base"], int(m["idx"]), int(m["total"]), len(m["total"])


def shard_set(chosen: str) -> List[str]:
    """All file names of the set `chosen` belongs to, in order; a file that is no shard is its own set (gguf_split.rs:69-86)."""
    d, f = os.path.split(chosen)
    s = parse_shard(f)
    if s is None or s[2] < 1:
        return [chosen]
    base, _, total, w = s
    return [os.path.join(d, f"{base}-{i:0{w}d}-of-{total:0{w}d}.gguf") for i in range(1, total + 1)]


class GgufModel:
    """One model: a single file, or every shard of a split set opened through any one of them
    (crates/infr-gguf/src/lib.rs:470-520).  Checked as the reference checks: the file names' total equals
    `split.count` in every shard, a shard's zero-based `split.no` is the position its name claims, the assembled
    index has exactly `split.tensors.count` tensors and no name twice.  Metadata come from the first shard (the
    others carry only the three split keys); a tensor is uploaded from the shard that holds it."""

    def __init__(self, path: str):
        first = GgufFile(path)
        count = first.meta_u64("split.count")
        if not count or count <= 1:
            self.shards = [first]
            self._where = {n: 0 for n in first.tensor_names()}
            return
        first.close()
        names = shard_set(path)
        if len(names) != count:
            raise BackendError(ERR_INVALID_ARG, f"GGUF: {os.path.basename(path)} says split.count = {count} but its name belongs to a set of {len(names)}")
        self.shards = []
        try:
            for n in names:
                if not os.path.exists(n):
                    raise BackendError(ERR_INVALID_ARG, f"GGUF: shard {os.path.basename(n)} of the set is missing")
                self.shards.append(GgufFile(n))
            self._where = {}
            for pos, sh in enumerate(self.shards):
                if sh.meta_u64("split.count") != count:
                    raise BackendError(ERR_INVALID_ARG, f"GGUF: shard {pos + 1} disagrees on split.count")
                if sh.meta_u64("split.no") != pos:
                    raise BackendError(ERR_INVALID_ARG, f"GGUF: shard {pos + 1} carries split.no = {sh.meta_u64('split.no')}, its name says {pos}")
                for t in sh.tensor_names():
                    if t in self._where:
                        raise BackendError(ERR_INVALID_ARG, f"GGUF: tensor {t} appears in shards {self._where[t] + 1} and {pos + 1}")
                    self._where[t] = pos
            want = self.shards[0].meta_u64("split.tensors.count")
            if want is not None and want != len(self._where):
                raise BackendError(ERR_INVALID_ARG, f"GGUF: the set holds {len(self._where)} tensors, split.tensors.count says {want}")
        except Exception:
            self.close()
            raise

    def close(self) -> None:
        for s in self.shards:
            s.close()

    def tensor_count(self) -> int:
        return len(self._where)

    def find(self, name: str) -> Optional[TensorInfo]:
        pos = self._where.get(name)
        return None if pos is None else self.shards[pos].find(name)

    def meta_u64(self, key: str) -> Optional[int]:
        return self.shards[0].meta_u64(key)

    def meta_f64(self, key: str) -> Optional[float]:
        return self.shards[0].meta_f64(key)

    def meta_str(self, key: str) -> Optional[str]:
        return self.shards[0].meta_str(key)

    def upload(self, be: CudaBackend, name: str) -> Buffer:
        pos = self._where.get(name)
        if pos is None:
            raise BackendError(ERR_INVALID_ARG, f"GGUF: no tensor {name}")
        return self.shards[pos].upload(be, name)


def moe_layer_op(be: CudaBackend, gg, layer: int, arch: Optional[str] = None) -> Tuple[MoeFfn, Dict[str, Buffer]]:
    """Uploads layer `layer`'s MoE FFN tensors and returns an `Op::MoeFfn` template (x, dst, rows
    left for the caller) together with the buffers it refers to."""
    arch = arch or gg.meta_str("general.architecture")
    p = f"blk.{layer}."
    need = {"router": p + "ffn_gate_inp.weight", "gate": p + "ffn_gate_exps.weight", "up": p + "ffn_up_exps.weight",
            "down": p + "ffn_down_exps.weight"}
    info = {k: gg.find(n) for k, n in need.items()}
    for k, n in need.items():
        if info[k] is None:
            raise BackendError(ERR_INVALID_ARG, f"GGUF: layer {layer} has no tensor {n}")
    ne, n_expert = info["router"].dims[0], info["router"].dims[1]
    g_ne, n_ff, g_e = info["gate"].dims
    d_ff, d_ne, d_e = info["down"].dims
    if not (g_ne == ne == d_ne and g_e == n_expert == d_e and d_ff == n_ff and info["up"].dims == info["gate"].dims):
        raise BackendError(ERR_INVALID_ARG, f"GGUF: layer {layer}: expert bank shapes disagree")
    n_used = gg.meta_u64(f"{arch}.expert_used_count") if arch else None
    if not n_used:
        raise BackendError(ERR_INVALID_ARG, "GGUF: no expert_used_count in the metadata")
    b = {k: gg.upload(be, n) for k, n in need.items()}
    op = MoeFfn(x=None, router=b["router"], gate_exps=b["gate"], up_exps=b["up"], down_exps=b["down"], dst=None, rows=0, ne=ne,
                n_expert=n_expert, n_used=int(n_used), n_ff_exp=n_ff, router_dtype=DType(info["router"].dtype),
                gate_dtype=DType(info["gate"].dtype), up_dtype=DType(info["up"].dtype), down_dtype=DType(info["down"].dtype))
    if gg.find(p + "exp_probs_b.bias") is not None:
        b["bias"] = gg.upload(be, p + "exp_probs_b.bias")
        op.exp_probs_b = b["bias"]
    sh = gg.find(p + "ffn_gate_shexp.weight")
    if sh is not None:
        b["sh_gate"] = gg.upload(be, p + "ffn_gate_shexp.weight")
        b["sh_up"] = gg.upload(be, p + "ffn_up_shexp.weight")
        b["sh_down"] = gg.upload(be, p + "ffn_down_shexp.weight")
        op.sh_gate, op.sh_up, op.sh_down, op.sh_ff = b["sh_gate"], b["sh_up"], b["sh_down"], sh.dims[1]
        if gg.find(p + "ffn_gate_inp_shexp.weight") is not None:
            b["sh_gate_inp"] = gg.upload(be, p + "ffn_gate_inp_shexp.weight")
            op.sh_gate_inp = b["sh_gate_inp"]
    scale = gg.meta_f64(f"{arch}.expert_weights_scale") if arch else None
    if scale:
        op.scale = float(scale)
    return op, b
