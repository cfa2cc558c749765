"""The GGUF reader (infr_gguf_*): what Gguf::open accepts and rejects (crates/infr-gguf/src/lib.rs:476, :735-870 and
its tests :1219-1700 — bad magic, unsupported version, truncation, absurd counts, alignment, block-misaligned
tensors, data outside the file).  No GPU needed."""
import struct

import numpy as np
import pytest

import infr_b200
from infr_b200 import synth
from infr_b200.gguf_file import GGML_F16, GGML_F32, GGML_Q4_K, GGML_Q6_K, GgufFile
from fixtures import Q4K, Q6K
import gguf_writer as gw


def _model_file(tmp_path, alignment=32):
    w4 = synth.weight(Q4K, 8, 512, seed=1)
    w6 = synth.weight(Q6K, 4, 256, seed=2)
    nrm = np.linspace(0.5, 1.5, 512, dtype=np.float32)
    half = np.arange(64, dtype=np.float16)
    meta = [("general.architecture", gw.STR, "llama"), ("general.alignment", gw.U32, alignment), ("llama.block_count", gw.U32, 2),
            ("llama.rope.freq_base", gw.F32, 500000.0), ("llama.attention.layer_norm_rms_epsilon", gw.F64, 1e-5), ("some.flag", gw.BOOL, 1),
            ("some.negative", gw.I32, -7), ("tokenizer.ggml.tokens", gw.ARR, (gw.STR, ["a", "bc", "def"])),
            ("tokenizer.ggml.scores", gw.ARR, (gw.F32, [0.5, -1.0, 2.0])), ("nested", gw.ARR, (gw.ARR, [(gw.U8, [1, 2]), (gw.U8, [3])]))]
    tensors = [("blk.0.attn_q.weight", (512, 8), GGML_Q4_K, w4), ("blk.0.attn_v.weight", (256, 4), GGML_Q6_K, w6),
               ("blk.0.attn_norm.weight", (512,), GGML_F32, nrm), ("half", (64,), GGML_F16, half)]
    p = tmp_path / "m.gguf"
    gw.write_gguf(p, meta, tensors, alignment=alignment)
    return p, dict(w4=w4, w6=w6, nrm=nrm, half=half)


@pytest.mark.parametrize("alignment", [32, 64, 4096])
def test_reads_tensors_and_metadata(tmp_path, alignment):
    p, want = _model_file(tmp_path, alignment)
    with GgufFile(p) as g:
        assert g.version == 3 and g.alignment == alignment
        assert list(g.tensors) == ["blk.0.attn_q.weight", "blk.0.attn_v.weight", "blk.0.attn_norm.weight", "half"]
        t = g.tensors["blk.0.attn_q.weight"]
        assert (t.ggml_type, t.dtype, t.dims, t.numel, t.nbytes) == (GGML_Q4_K, Q4K, (512, 8), 4096, 16 * 144)
        assert t.file_offset % alignment == 0
        t6 = g.tensors["blk.0.attn_v.weight"]
        assert (t6.dtype, t6.nbytes) == (Q6K, 4 * 210)
        np.testing.assert_array_equal(g.data("blk.0.attn_q.weight"), want["w4"])
        np.testing.assert_array_equal(g.data("blk.0.attn_v.weight"), want["w6"])
        np.testing.assert_array_equal(g.data("blk.0.attn_norm.weight").view(np.float32), want["nrm"])
        np.testing.assert_array_equal(g.data("half").view(np.float16), want["half"])
        assert g.meta("general.architecture") == "llama"
        assert g.meta("llama.block_count") == 2 and g.meta("some.negative") == -7 and g.meta("some.flag") is True
        assert g.meta("llama.rope.freq_base") == 500000.0 and abs(g.meta("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        assert g.meta("tokenizer.ggml.tokens") == 3  # strings: the count
        np.testing.assert_array_equal(g.meta("tokenizer.ggml.scores"), np.array([0.5, -1.0, 2.0], np.float32))
        assert g.meta("nested") == 2 and g.meta("absent") is None and g.meta("absent", 5) == 5
        assert "llama.block_count" in g.keys() and len(g.keys()) == 10


def test_a_file_written_by_the_gguf_package_reads_the_same(tmp_path):
    """An independent producer: the `gguf` Python package's writer."""
    gguf = pytest.importorskip("gguf")
    w4 = synth.weight(Q4K, 4, 256, seed=5)
    f32 = np.arange(12, dtype=np.float32).reshape(3, 4)
    p = tmp_path / "pkg.gguf"
    wr = gguf.GGUFWriter(str(p), "llama")
    wr.add_uint32("llama.block_count", 1)
    wr.add_float32("llama.rope.freq_base", 10000.0)
    wr.add_tensor("f32", f32)
    wr.add_tensor("q4", w4.reshape(4, 144), raw_dtype=gguf.GGMLQuantizationType.Q4_K)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    with GgufFile(p) as g:
        assert g.meta("general.architecture") == "llama" and g.meta("llama.block_count") == 1
        assert g.tensors["f32"].dims == (4, 3) and g.tensors["f32"].ggml_type == GGML_F32
        np.testing.assert_array_equal(g.data("f32").view(np.float32).reshape(3, 4), f32)
        t = g.tensors["q4"]
        assert t.dtype == Q4K and t.numel == 4 * 256 and t.dims[0] == 256
        np.testing.assert_array_equal(g.data("q4"), w4)


def _expect(path, code, needle):
    with pytest.raises(infr_b200.BackendError) as e:
        GgufFile(path)
    assert e.value.code == code and needle in str(e.value), str(e.value)


def test_malformed_files_are_errors_not_faults(tmp_path):
    w4 = synth.weight(Q4K, 2, 256, seed=3)
    ok_meta = [("general.architecture", gw.STR, "llama")]
    ok_t = [("w", (256, 2), GGML_Q4_K, w4)]
    p = tmp_path / "x.gguf"
    good = gw.write_gguf(p, ok_meta, ok_t)
    GgufFile(p).close()

    def put(b):
        p.write_bytes(b)
        return p
    _expect(put(b"GGML" + good[4:]), infr_b200.E_INVALID, "not a GGUF file")
    _expect(put(good[:4] + struct.pack("<I", 1) + good[8:]), infr_b200.E_UNSUPPORTED, "version 1")
    _expect(put(good[:10]), infr_b200.E_INVALID, "shorter than a header")
    for cut in (30, 60, len(good) - 300, len(good) - 1):  # inside the metadata, the tensor table, the data
        _expect(put(good[:cut]), infr_b200.E_INVALID, "GGUF")
    # counts that no file of this size can hold
    _expect(put(good[:8] + struct.pack("<QQ", 1 << 60, 1) + good[24:]), infr_b200.E_INVALID, "counts exceed")
    _expect(put(good[:8] + struct.pack("<QQ", 1, 1 << 60) + good[24:]), infr_b200.E_INVALID, "counts exceed")
    # alignment: zero, not a power of two, absurd
    for a in (0, 48, 1 << 30):
        gw.write_gguf(p, ok_meta + [("general.alignment", gw.U32, a)], ok_t, alignment=32)
        _expect(p, infr_b200.E_INVALID, "general.alignment")
    # a quantised tensor that is not a whole number of blocks; a shape that overflows; too many dimensions
    gw.write_gguf(p, ok_meta, [("w", (100, 1), GGML_Q4_K, w4[:144])])
    _expect(p, infr_b200.E_INVALID, "whole number of 256-element blocks")
    gw.write_gguf(p, ok_meta, [("w", (1 << 40, 1 << 40), GGML_F32, w4)])
    _expect(p, infr_b200.E_INVALID, "overflows")
    gw.write_gguf(p, ok_meta, [("w", (2,) * 9, GGML_F32, w4)])
    _expect(p, infr_b200.E_INVALID, "more than 8 dimensions")
    # data outside the file; an unknown tensor type; the same name twice
    gw.write_gguf(p, ok_meta, [("w", (256, 64), GGML_Q4_K, w4)])
    _expect(p, infr_b200.E_INVALID, "outside the file")
    gw.write_gguf(p, ok_meta, [("w", (256, 2), 99, w4)])
    _expect(p, infr_b200.E_UNSUPPORTED, "ggml type 99")
    gw.write_gguf(p, ok_meta, ok_t + ok_t)
    _expect(p, infr_b200.E_INVALID, "appears twice")
    # metadata: an unknown value type, a string longer than the file, nesting beyond the limit
    _expect(put(good[:24] + gw._s(b"k") + struct.pack("<I", 77) + good[24:]), infr_b200.E_INVALID, "GGUF")
    gw.write_gguf(p, [("k", gw.STR, "x")], ok_t)
    raw = bytearray(p.read_bytes())
    at = raw.index(b"\x01\x00\x00\x00\x00\x00\x00\x00x")
    raw[at:at + 8] = struct.pack("<Q", 1 << 50)
    _expect(put(bytes(raw)), infr_b200.E_INVALID, "GGUF")
    deep = (gw.U8, [1])
    for _ in range(70):
        deep = (gw.ARR, [deep])
    gw.write_gguf(p, [("deep", gw.ARR, deep)], ok_t)
    _expect(p, infr_b200.E_INVALID, "nested deeper")
    with pytest.raises(infr_b200.BackendError):
        GgufFile(tmp_path / "does-not-exist.gguf")


@pytest.mark.parametrize("ggml_type,dt,cols", [(GGML_Q4_K, Q4K, 512), (GGML_Q6_K, Q6K, 768), (42, 27, 320)])
def test_quantised_embedding_rows_decode_like_the_cpu(tmp_path, ggml_type, dt, cols):
    """A Q4_K_M file ships token_embd in a block format: the host-side lookup decodes one row per token
    (gguf_file.dequant_blocks), bit for bit what the CPU restatement of dequant.rs gives - seeded weights and raw
    random blocks (every scale / min bit pattern)."""
    from infr_b200 import gguf_file
    from oracle.cpu_oracle import Oracle

    orc = Oracle()
    for raw in (synth.weight(dt, 6, cols, seed=9), synth.random_blocks(dt, 6 * cols, 10)):
        want = orc.dequant(dt, raw).reshape(6, cols)
        np.testing.assert_array_equal(gguf_file.dequant_blocks(ggml_type, raw).view(np.uint32), want.reshape(-1).view(np.uint32))
        p = tmp_path / f"e{ggml_type}.gguf"
        gw.write_gguf(p, [("general.architecture", gw.STR, "llama")], [("token_embd.weight", (cols, 6), ggml_type, raw)])
        with GgufFile(p) as g:
            for row in (0, 3, 5):
                np.testing.assert_array_equal(gguf_file._f32_row(g, "token_embd.weight", row).view(np.uint32), want[row].view(np.uint32))
