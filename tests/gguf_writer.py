"""A minimal GGUF (version 3) writer for the tests: metadata scalars / strings / arrays and raw
tensor payloads, laid out as the file format prescribes (little-endian, tensor data aligned to
`general.alignment`, offsets relative to the aligned data region)."""
import struct

import numpy as np

T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 = range(13)


def _s(b: str) -> bytes:
    e = b.encode()
    return struct.pack("<Q", len(e)) + e


def _val(vtype, v) -> bytes:
    fmt = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f", T_BOOL: "<B", T_U64: "<Q",
           T_I64: "<q", T_F64: "<d"}
    if vtype == T_STR:
        return _s(v)
    if vtype == T_ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_val(et, i) for i in items)
    return struct.pack(fmt[vtype], v)


def write_gguf(path, meta, tensors, alignment=32, version=3, write_alignment_key=True):
    """meta: list of (key, type, value); tensors: list of (name, dims_fastest_first, ggml_type, bytes)."""
    kv = list(meta)
    if write_alignment_key:
        kv.append(("general.alignment", T_U32, alignment))
    out = bytearray(struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(kv)))
    for k, t, v in kv:
        out += _s(k) + struct.pack("<I", t) + _val(t, v)
    off = 0
    offsets = []
    for name, dims, gtype, payload in tensors:
        offsets.append(off)
        out += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", gtype, off)
        off += (len(payload) + alignment - 1) // alignment * alignment
    pad = (-len(out)) % alignment
    out += b"\0" * pad
    for (name, dims, gtype, payload), o in zip(tensors, offsets):
        assert len(out) % alignment == 0
        out += bytes(payload)
        out += b"\0" * ((-len(payload)) % alignment)
    with open(path, "wb") as f:
        f.write(out)


def layer_to_gguf(path, L, layer=0, arch="qwen35moe", n_used=8, alignment=32, extra_meta=()):
    """Writes one synthetic MoE layer (moe4all_b200.synth.LayerWeights) under the reference's tensor names."""
    p = f"blk.{layer}."
    meta = [("general.architecture", T_STR, arch), (f"{arch}.expert_count", T_U32, L.n_expert), (f"{arch}.expert_used_count", T_U32, n_used),
            (f"{arch}.expert_feed_forward_length", T_U32, L.n_ff), ("tokenizer.ggml.tokens", T_ARR, (T_STR, ["a", "b", "c"])),
            ("some.nested", T_ARR, (T_ARR, [(T_I32, [1, 2]), (T_I32, [3])]))] + list(extra_meta)
    gd, ud, dd = getattr(L, "gate_dtype", 12), getattr(L, "up_dtype", 12), getattr(L, "down_dtype", 14)
    t = [("token_embd.weight", (L.ne, 4), 0, np.zeros((4, L.ne), np.float32).tobytes()),
         (p + "ffn_gate_inp.weight", (L.ne, L.n_expert), 0, np.ascontiguousarray(L.router, np.float32).tobytes()),
         (p + "ffn_gate_exps.weight", (L.ne, L.n_ff, L.n_expert), gd, L.gate.tobytes()),
         (p + "ffn_up_exps.weight", (L.ne, L.n_ff, L.n_expert), ud, L.up.tobytes()),
         (p + "ffn_down_exps.weight", (L.n_ff, L.ne, L.n_expert), dd, L.down.tobytes())]
    if L.sh_gate is not None:
        t += [(p + "ffn_gate_shexp.weight", (L.ne, L.sh_ff), gd, L.sh_gate.tobytes()),
              (p + "ffn_up_shexp.weight", (L.ne, L.sh_ff), ud, L.sh_up.tobytes()),
              (p + "ffn_down_shexp.weight", (L.sh_ff, L.ne), dd, L.sh_down.tobytes())]
        if L.sh_gate_inp is not None:
            t.append((p + "ffn_gate_inp_shexp.weight", (L.ne,), 0, np.ascontiguousarray(L.sh_gate_inp, np.float32).tobytes()))
    if L.bias is not None:
        t.append((p + "exp_probs_b.bias", (L.n_expert,), 0, np.ascontiguousarray(L.bias, np.float32).tobytes()))
    write_gguf(path, meta, t, alignment=alignment)
    return t
