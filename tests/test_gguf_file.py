"""The GGUF container reader against files written by ggml's own Python writer (no GPU).

Mirrors Tests/IshizukiKitTests/GGUFTests.swift: block geometry, a written file read back
(metadata of every kind, tensor table, data offsets, bytes), and the refusals."""
import struct

import numpy as np
import pytest

from ishizuki_b200 import _lib, synth
from ishizuki_b200.gguf_file import GGUFError, GGUFFile

gguf = pytest.importorskip("gguf")


def test_block_geometry_of_every_type():
    lib = _lib.load()
    # Tests/IshizukiKitTests/GGUFTests.swift:17-35 and Sources/IshizukiKit/Config/GGUFFile.swift:44-80
    want = {0: (1, 4), 1: (1, 2), 30: (1, 2), 2: (32, 18), 8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144),
            13: (256, 176), 14: (256, 210), 16: (256, 66), 17: (256, 74), 18: (256, 98), 19: (256, 50), 20: (32, 18),
            21: (256, 110), 22: (256, 82), 23: (256, 136), 29: (256, 56)}
    for t, (block, size) in want.items():
        assert (lib.ishi_gguf_type_block_size(t), lib.ishi_gguf_type_size(t)) == (block, size), t
        # the ggml project's own table agrees
        assert gguf.GGML_QUANT_SIZES[gguf.GGMLQuantizationType(t)] == (block, size)
    assert lib.ishi_gguf_type_name(17) == b"IQ2_XS" and lib.ishi_gguf_type_name(99) is None
    assert lib.ishi_gguf_type_size(5) == 0  # removed type ids stay unknown


def write_sample(path, alignment=None):
    rng = np.random.default_rng(5)
    w = gguf.GGUFWriter(str(path), "qwen35")
    if alignment:
        w.add_custom_alignment(alignment)
    w.add_uint32("qwen35.block_count", 64)
    w.add_float32("qwen35.rope.freq_base", 10000.5)
    w.add_bool("general.flag", True)
    w.add_string("general.name", "sample pack")
    w.add_array("tokenizer.ggml.tokens", ["a", "bc", "def"])
    w.add_array("qwen35.rope.sections", [11, 11, 10])
    w.add_int32("general.negative", -7)
    tensors = {
        "token_embd.weight": (synth.ggml_blocks(rng, 29, 16, 256), 29, (16, 256)),
        "blk.0.ffn_up.weight": (synth.ggml_blocks(rng, 22, 256, 512), 22, (256, 512)),
        "blk.0.attn_q.weight": (synth.ggml_blocks(rng, 12, 8, 1024), 12, (8, 1024)),
        "blk.0.attn_norm.weight": (rng.standard_normal(256).astype(np.float32), 0, (256,)),
    }
    for name, (data, type_id, shape) in tensors.items():
        if type_id == 0:
            w.add_tensor(name, data)
        else:
            ts = synth.TYPE_SIZE[type_id]
            raw = data.reshape(shape[0], shape[1] // 256 * ts)
            w.add_tensor(name, raw, raw_dtype=gguf.GGMLQuantizationType(type_id))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return tensors


def test_a_written_file_reads_back(tmp_path):
    path = tmp_path / "sample.gguf"
    tensors = write_sample(path)
    f = GGUFFile(path)
    assert f.version == 3 and f.alignment == 32 and f.dataOffset % 32 == 0
    assert f.architecture == "qwen35"
    assert f.architectureValue("block_count") == 64
    assert abs(f["qwen35.rope.freq_base"] - 10000.5) < 1e-3
    assert f["general.flag"] is True and f["general.negative"] == -7
    assert f["general.name"] == "sample pack"
    assert f["tokenizer.ggml.tokens"] == ["a", "bc", "def"]
    assert f["qwen35.rope.sections"] == [11, 11, 10]
    assert f["no.such.key"] is None
    assert [t.name for t in f.tensors] == list(tensors)
    for name, (data, type_id, shape) in tensors.items():
        t = f.tensor(name)
        assert t.shape == shape and t.type == type_id  # row-major: rows of `shape[-1]` inputs
        assert t.offset % 32 == 0
        assert t.byteCount == data.view(np.uint8).size
        assert np.array_equal(f.data(t), data.view(np.uint8).reshape(-1))
    assert dict(f.typeHistogram) == {29: 1, 22: 1, 12: 1, 0: 1}
    # ggml's own reader sees the same table
    theirs = gguf.GGUFReader(str(path))
    assert [t.name for t in theirs.tensors] == [t.name for t in f.tensors]
    assert [int(t.data_offset) for t in theirs.tensors] == [f.dataOffset + t.offset for t in f.tensors]
    f.close()


def test_a_custom_alignment_moves_the_data_section(tmp_path):
    path = tmp_path / "aligned.gguf"
    write_sample(path, alignment=256)
    f = GGUFFile(path)
    assert f.alignment == 256 and f.dataOffset % 256 == 0
    assert all(t.offset % 256 == 0 for t in f.tensors)


def header(version=3, tensors=0, kvs=0, magic=0x46554747) -> bytes:
    return struct.pack("<IIQQ", magic, version, tensors, kvs)


def gstr(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def tensor_entry(name, dims, type_id, offset=0) -> bytes:
    return gstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", type_id, offset)


@pytest.mark.parametrize("blob,reason", [
    (header(magic=0x12345678), "not a GGUF"),
    (header(version=1), "version 1"),
    (header(tensors=2_000_000), "implausible"),
    (header(kvs=1) + gstr("k") + struct.pack("<I", 99), "type 99"),
    (header(kvs=1) + struct.pack("<Q", 1 << 30), "implausible"),
    (header(kvs=1) + gstr("k") + struct.pack("<IIQ", 9, 4, 1 << 27), "implausible"),
    (header(kvs=1) + gstr("k"), "mid-field"),
    (header(kvs=1) + gstr("general.alignment") + struct.pack("<II", 4, 24) , "power of two"),
    (header(tensors=1) + tensor_entry("w", [1, 1, 1, 1, 1], 0), "rank 5"),
    (header(tensors=1) + tensor_entry("w", [256], 5), "unknown GGML type 5"),
    (header(tensors=1) + tensor_entry("w", [100], 12), "not a multiple"),
])
def test_refusals(tmp_path, blob, reason):
    path = tmp_path / "bad.gguf"
    path.write_bytes(blob)
    with pytest.raises(GGUFError) as err:
        GGUFFile(path)
    assert reason in str(err.value)


def test_a_tensor_past_the_end_of_the_file_is_refused_when_read(tmp_path):
    path = tmp_path / "short.gguf"
    blob = header(tensors=1) + tensor_entry("w", [256, 4], 12, offset=0)
    blob += b"\\0" * ((-len(blob)) % 32) + b"\\1" * 100  # 576 bytes promised, 100 present
    path.write_bytes(blob)
    f = GGUFFile(path)
    assert f.tensor("w").shape == (4, 256) and f.tensor("w").byteCount == 576
    with pytest.raises(GGUFError) as err:
        f.data("w")
    assert "past the end" in str(err.value)
