"""GGUF ingest: the reader finds the MoE FFN tensors of a model file and hands their bytes over
unchanged (reference loader: crates/infr-gguf/src/lib.rs:745-870), refuses malformed files with a
message, and a layer loaded from a file computes what the oracle computes."""
import struct

import numpy as np
import pytest

from moe4all_b200 import BackendError, synth
from moe4all_b200.gguf import GgufFile, GgufModel, moe_layer_op, parse_shard, shard_set

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


def test_shard_names():
    # the reference's own vectors (crates/infr-core/src/gguf_split.rs `parse_shard_pattern`,
    # `an_over_wide_shard_total_is_not_a_shard`, and the set a shard name stands for)
    assert parse_shard("model-Q4_K_M-00001-of-00003.gguf") == ("model-Q4_K_M", 1, 3, 5)
    assert parse_shard("m-00003-of-00005.gguf")[1] == 3
    assert parse_shard("model-Q4_K_M.gguf") is None
    assert parse_shard("m-1-of-003.gguf") is None and parse_shard("m-000ab-of-00003.gguf") is None
    assert parse_shard("m-Q4_K_M-0000000001-of-4294967295.gguf") is None and parse_shard("m-000001-of-999999.gguf") is None
    assert shard_set("/d/m-00002-of-00003.gguf") == [f"/d/m-0000{i}-of-00003.gguf" for i in (1, 2, 3)]
    assert shard_set("/d/plain.gguf") == ["/d/plain.gguf"]


def write_split(tmp_path, L, parts=3, count=None, numbers=None, tensors_count=None, dup=False, base="m"):
    """One layer's tensors dealt over `parts` shard files the way gguf-split writes them: the model's metadata in
    the first shard, only the three split keys in the others (crates/infr-gguf/src/lib.rs:69-90)."""
    ref_path = str(tmp_path / "whole.gguf")
    tensors = gw.layer_to_gguf(ref_path, L, layer=0, n_used=2)
    groups = [tensors[i::parts] for i in range(parts)]
    if dup:
        groups[1] = groups[1] + [groups[0][0]]
    total = sum(len(g_) for g_ in groups) if tensors_count is None else tensors_count
    paths = []
    for i, grp in enumerate(groups):
        split = [("split.no", gw.T_U16, i if numbers is None else numbers[i]), ("split.count", gw.T_U16, parts if count is None else count),
                 ("split.tensors.count", gw.T_I32, total)]
        meta = split if i else [("general.architecture", gw.T_STR, "qwen35moe"), ("qwen35moe.expert_used_count", gw.T_U32, 2)] + split
        path = str(tmp_path / f"{base}-{i + 1:05d}-of-{parts:05d}.gguf")
        gw.write_gguf(path, meta, grp)
        paths.append(path)
    return paths, tensors


def test_split_model_opens_through_any_shard(tmp_path):
    L = small_layer()
    paths, tensors = write_split(tmp_path, L)
    for chosen in (paths[0], paths[2]):
        m = GgufModel(chosen)
        assert len(m.shards) == 3 and m.tensor_count() == len(tensors)
        assert m.meta_str("general.architecture") == "qwen35moe" and m.meta_u64("qwen35moe.expert_used_count") == 2
        for name, dims, gtype, payload in tensors:
            t = m.find(name)
            assert t is not None and t.dtype == gtype and t.dims == tuple(dims) and t.nbytes == len(payload)
        assert m.find("blk.0.nope") is None
        m.close()
    whole = GgufModel(str(tmp_path / "whole.gguf"))  # a single file is a model of one shard
    assert len(whole.shards) == 1 and whole.tensor_count() == len(tensors)
    whole.close()


@pytest.mark.parametrize("case", ["missing", "count", "number", "tensors", "duplicate"])
def test_broken_split_sets_are_refused(tmp_path, case):
    import os
    L = small_layer()
    kw = {"count": dict(count=4), "number": dict(numbers=[0, 2, 1]), "tensors": dict(tensors_count=99), "duplicate": dict(dup=True)}.get(case, {})
    paths, _ = write_split(tmp_path, L, **kw)
    if case == "missing":
        os.remove(paths[1])
    with pytest.raises(BackendError) as e:
        GgufModel(paths[0])
    assert {"missing": "is missing", "count": "split.count", "number": "split.no", "tensors": "split.tensors.count", "duplicate": "appears in shards"}[case] in str(e.value)


@pytest.mark.gpu
def test_layer_from_split_model_matches_oracle(backend, tmp_path):
    from helpers import assert_close, oracle_layer
    L = small_layer()
    paths, _ = write_split(tmp_path, L)
    m = GgufModel(paths[1])
    op, bufs = moe_layer_op(backend, m, 0)
    assert np.array_equal(backend.download(bufs["gate"], np.uint8, count=L.gate.size), L.gate.reshape(-1))
    x = synth.activations(78, 3, 256)
    op.x, op.dst, op.rows = backend.from_host(x), backend.alloc(3 * 256 * 4), 3
    backend.moe_ffn(op)
    backend.sync()
    assert_close(backend.download(op.dst, np.float32).reshape(3, 256), oracle_layer(L, x, 2).dst)
    m.close()


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
