"""GGUF ingest: the reader finds the MoE FFN tensors of a model file and hands their bytes over
unchanged (reference loader: crates/infr-gguf/src/lib.rs:745-870), refuses malformed files with a
message, and a layer loaded from a file computes what the oracle computes."""
import struct

import numpy as np
import pytest

from moe4all_b200 import BackendError, synth
from moe4all_b200.gguf import GgufFile, moe_layer_op

import gguf_writer as gw


def small_layer():
    return synth.make_layer(23, 256, 8, 256, sh_ff=256, router_std=0.05, bias_std=0.05)


def test_reader_finds_tensors_and_metadata(tmp_path):
    L = small_layer()
    path = str(tmp_path / "m.gguf")
    tensors = gw.layer_to_gguf(path, L, layer=3, n_used=2, alignment=64,
                               extra_meta=[("qwen35moe.expert_weights_scale", gw.T_F32, 2.5), ("x.neg", gw.T_I64, -7)])
    g = GgufFile(path)
    assert g.tensor_count() == len(tensors)
    assert g.meta_str("general.architecture") == "qwen35moe"
    assert g.meta_u64("qwen35moe.expert_count") == 8 and g.meta_u64("qwen35moe.expert_used_count") == 2
    assert g.meta_f64("qwen35moe.expert_weights_scale") == 2.5
    assert g.meta_u64("x.neg") is None and g.meta_f64("x.neg") == -7.0
    assert g.meta_u64("tokenizer.ggml.tokens") is None  # arrays are skipped, not mis-read
    raw = open(path, "rb").read()
    for name, dims, gtype, payload in tensors:
        t = g.find(name)
        assert t is not None and t.dtype == gtype and t.dims == tuple(dims) and t.nbytes == len(payload)
        assert t.offset % 64 == 0 and raw[t.offset:t.offset + t.nbytes] == bytes(payload)
    assert g.find("blk.3.nope") is None
    gate = g.find("blk.3.ffn_gate_exps.weight")
    assert gate.dims == (256, 256, 8) and gate.nbytes == 8 * 256 * 144
    g.close()


def test_default_alignment_and_version_2(tmp_path):
    path = str(tmp_path / "v2.gguf")
    gw.write_gguf(path, [("general.architecture", gw.T_STR, "llama")], [("a", (32,), 8, bytes(range(34))), ("b", (3,), 0, b"\1" * 12)],
                  alignment=32, version=2, write_alignment_key=False)
    g = GgufFile(path)
    a, b = g.find("a"), g.find("b")
    assert a.nbytes == 34 and b.nbytes == 12 and a.offset % 32 == 0 and b.offset == a.offset + 64


@pytest.mark.parametrize("case", ["magic", "version", "truncated", "alignment", "blocks", "beyond", "duplicate", "dims"])
def test_malformed_files_are_refused(tmp_path, case):
    path = str(tmp_path / "bad.gguf")
    q4 = bytes(144)
    if case == "alignment":
        gw.write_gguf(path, [("general.alignment", gw.T_U32, 24)], [("a", (256,), 12, q4)], write_alignment_key=False)
    elif case == "blocks":
        gw.write_gguf(path, [], [("a", (100,), 12, q4)])
    elif case == "duplicate":
        gw.write_gguf(path, [], [("a", (256,), 12, q4), ("a", (256,), 12, q4)])
    elif case == "dims":
        gw.write_gguf(path, [], [("a", (256, 1, 1, 1, 1), 12, q4)])
    else:
        gw.write_gguf(path, [("k", gw.T_U32, 1)], [("a", (256,), 12, q4)])
        raw = bytearray(open(path, "rb").read())
        if case == "magic":
            raw[0] = 0x00
        elif case == "version":
            raw[4:8] = struct.pack("<I", 7)
        elif case == "truncated":
            raw = raw[:40]
        elif case == "beyond":
            raw = raw[:-100]
        open(path, "wb").write(bytes(raw))
    with pytest.raises(BackendError) as e:
        GgufFile(path)
    assert str(e.value)


@pytest.mark.gpu
@pytest.mark.parametrize("dtypes", [None, (13, 13, 14), (8, 8, 8)])
def test_layer_from_file_matches_oracle(backend, tmp_path, dtypes):
    from helpers import assert_close, near_tie_rows, oracle_layer
    # the file's tensor types (Q4_K / Q6_K, a Q5_K_M-like mix, Q8_0 throughout) travel into the op
    L = small_layer() if dtypes is None else synth.make_layer(4, 256, 8, 256, sh_ff=256, router_std=0.05, dtypes=dtypes)
    path = str(tmp_path / "layer.gguf")
    gw.layer_to_gguf(path, L, layer=0, n_used=2)
    g = GgufFile(path)
    op, bufs = moe_layer_op(backend, g, 0)
    assert (op.ne, op.n_expert, op.n_used, op.n_ff_exp, op.sh_ff) == (256, 8, 2, 256, 256)
    if dtypes is not None:
        assert (int(op.gate_dtype), int(op.up_dtype), int(op.down_dtype)) == dtypes
    # bytes on the device are the file's bytes
    got = backend.download(bufs["down"], np.uint8, count=L.down.size)
    assert np.array_equal(got, L.down.reshape(-1))
    x = synth.activations(77, 4, 256)
    op.x = backend.from_host(x)
    op.dst = backend.alloc(4 * 256 * 4)
    op.ids_out = backend.alloc(4 * 2 * 4)
    op.rows = 4
    backend.moe_ffn(op)
    backend.sync()
    out = backend.download(op.dst, np.float32).reshape(4, 256)
    ids = backend.download(op.ids_out, np.int32).reshape(4, 2)
    ref = oracle_layer(L, x, 2)
    ties = set(near_tie_rows(ref, 2).tolist())
    for r in range(4):
        if r not in ties:
            assert ids[r].tolist() == ref.ids[r].tolist()
    assert_close(out, ref.dst)
