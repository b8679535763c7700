"""Checkpoint format layer: the cases of the reference's core/tests/test_format.py (same inputs, same error
messages), plus manifest building from real safetensors files written on the fly, fused layouts, and the
tensor-parallel slicing rules checked for exactness against the oracle."""
from __future__ import annotations

import json
import struct

import numpy as np
import pytest

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.format import (BitsK, Codebook, FormatError, FusionKind, SplitError, TensorInfo, admissible_tp_degrees,
                                       build_manifest, build_matrix_spec, column_slice, even_shard, kv_shard_index,
                                       load_manifest, make_layout, row_slice)
from trellis_serve_b200.format.safetensors_header import parse_header, read_header


def _linear(k, n, words, marker="mul1"):
    t = {"trellis": TensorInfo("m.trellis", "I16", (k // 16, n // 16, words)),
         "suh": TensorInfo("m.suh", "F16", (k,)), "svh": TensorInfo("m.svh", "F16", (n,))}
    if marker:
        t[marker] = TensorInfo(f"m.{marker}", "I32", ())
    return t


def test_spec_reads_bits_and_codebook_from_shapes():
    spec = build_matrix_spec("m", _linear(256, 512, 48))
    assert (spec.k, spec.n, spec.bits.value, spec.codebook) == (256, 512, 3.0, Codebook.MUL1)
    assert build_matrix_spec("m", _linear(256, 512, 64, "mcg")).codebook is Codebook.MCG
    assert build_matrix_spec("m", _linear(256, 512, 64, None)).codebook is Codebook.INST3
    assert [c.kernel_id for c in (Codebook.INST3, Codebook.MCG, Codebook.MUL1)] == [0, 1, 2]


def test_half_bitrates_need_mul1():
    assert build_matrix_spec("m", _linear(128, 128, 40)).bits == BitsK(5)
    with pytest.raises(FormatError, match="requires the mul1 codebook"):
        build_matrix_spec("m", _linear(128, 128, 40, "mcg"))
    with pytest.raises(FormatError, match="not a valid EXL3 bitrate"):
        build_matrix_spec("m", _linear(128, 128, 12))


def test_rejects_broken_linears():
    t = _linear(128, 128, 32)
    del t["suh"]
    with pytest.raises(FormatError, match="expected exactly one of"):
        build_matrix_spec("m", t)
    with pytest.raises(FormatError, match="not multiples of 128"):
        build_matrix_spec("m", _linear(144, 128, 32))
    t = _linear(128, 128, 32)
    t["extra"] = TensorInfo("m.extra", "F16", (1,))
    with pytest.raises(FormatError, match="unknown tensors"):
        build_matrix_spec("m", t)
    t = _linear(128, 128, 32)
    t["mcg"] = TensorInfo("m.mcg", "I32", ())
    with pytest.raises(FormatError, match="both .mcg and .mul1"):
        build_matrix_spec("m", t)
    t = _linear(128, 128, 32)
    t["su"] = TensorInfo("m.su", "I16", (8,))
    del t["suh"]
    with pytest.raises(FormatError, match="mixed legacy/modern"):
        build_matrix_spec("m", t)


def test_legacy_sign_tensors_and_bias():
    t = {"trellis": TensorInfo("m.trellis", "I16", (8, 16, 48)), "su": TensorInfo("m.su", "I16", (8,)),
         "sv": TensorInfo("m.sv", "I16", (16,)), "bias": TensorInfo("m.bias", "F32", (256,))}
    spec = build_matrix_spec("m", t)
    assert spec.legacy_signs and spec.has_bias and spec.codebook is Codebook.INST3


def test_header_parser_reads_names_shapes_and_sizes():
    doc = {"__metadata__": {"format": "pt"},
           "m.trellis": {"dtype": "I16", "shape": [8, 8, 48], "data_offsets": [0, 6144]},
           "m.suh": {"dtype": "F16", "shape": [128], "data_offsets": [6144, 6400]}}
    h = parse_header(json.dumps(doc).encode(), "shard.safetensors")
    assert h.metadata == {"format": "pt"}
    assert h.tensors["m.trellis"].shape == (8, 8, 48) and h.tensors["m.trellis"].nbytes == 6144


def test_header_parser_rejects_a_reversed_byte_range():
    empty = {"w": {"dtype": "F16", "shape": [0], "data_offsets": [4, 4]}}
    assert parse_header(json.dumps(empty).encode(), "s").tensors["w"].nbytes == 0
    raw = json.dumps({"w": {"dtype": "F16", "shape": [2], "data_offsets": [10, 4]}}).encode()
    with pytest.raises(FormatError, match="reversed"):
        parse_header(raw, "shard.safetensors")
    with pytest.raises(FormatError, match="not valid JSON"):
        parse_header(b"{not json", "s")


def _write_safetensors(path, tensors: dict, metadata=None):
    header, blobs, at = {}, [], 0
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def test_manifest_from_a_checkpoint_directory(tmp_path):
    K = 3
    tr = seeded_trellis(1, 8, 8, K).view(np.int16)
    lin = {"model.layers.0.q_proj.trellis": ("I16", tr), "model.layers.0.q_proj.suh": ("F16", seeded_signs(2, 128)),
           "model.layers.0.q_proj.svh": ("F16", seeded_signs(3, 128)), "model.layers.0.q_proj.mcg": ("I32", np.zeros((), np.int32)),
           "model.norm.weight": ("F16", np.ones(128, np.float16))}
    _write_safetensors(tmp_path / "model-00001.safetensors", lin)
    (tmp_path / "config.json").write_text(json.dumps({"quantization_config": {"quant_method": "exl3", "codebook": "mul1", "bits": 3.0}}))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {n: "model-00001.safetensors" for n in lin}}))
    man = load_manifest(tmp_path)
    assert list(man.matrices) == ["model.layers.0.q_proj"]
    spec = man.matrices["model.layers.0.q_proj"]
    assert (spec.k, spec.n, str(spec.bits), spec.codebook) == (128, 128, "3", Codebook.MCG)
    assert "model.norm.weight" in man.unquantized and man.is_quantized("model.layers.0.q_proj")
    assert any("quantization_config.codebook" in w for w in man.warnings)          # declared mul1, stored mcg
    s = man.summary()
    assert s["quantized_linears"] == 1 and s["by_bits_codebook"] == {"K=3 mcg": 1}
    assert read_header(tmp_path / "model-00001.safetensors").tensors["model.norm.weight"].nbytes == 256
    with pytest.raises(FormatError, match="no .safetensors files"):
        load_manifest(tmp_path / "nowhere")


def test_manifest_rejects_nested_and_ambiguous_tensors():
    a = parse_header(json.dumps({"m.trellis": {"dtype": "I16", "shape": [8, 8, 48], "data_offsets": [0, 6144]},
                                 "m.suh": {"dtype": "F16", "shape": [128], "data_offsets": [0, 256]},
                                 "m.svh": {"dtype": "F16", "shape": [128], "data_offsets": [0, 256]},
                                 "m.rank0.trellis": {"dtype": "I16", "shape": [8, 8, 48], "data_offsets": [0, 6144]}}).encode(), "a")
    with pytest.raises(FormatError, match="nested under EXL3 linear"):
        build_manifest([a])
    b = parse_header(json.dumps({"w": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode(), "b")
    c = parse_header(json.dumps({"w": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode(), "c")
    with pytest.raises(FormatError, match="does not say which one is live"):
        build_manifest([b, c])
    assert "w" in build_manifest([b, c], weight_map={"w": "c"}).unquantized


def test_fused_layout_spans_and_fusion_kind():
    q = build_matrix_spec("q", _linear(256, 512, 48, None))
    k = build_matrix_spec("k", _linear(256, 128, 48, None))
    lay = make_layout(["q", "k"], [q, k], [512, 128])
    assert lay.in_width == 256 and lay.out_width == 640 and lay.spans() == [(0, 512), (512, 128)]
    assert lay.best_fusion is FusionKind.SHARD_MAP
    assert make_layout(["g", "u"], [q, q], [512, 512]).best_fusion is FusionKind.UNIFORM
    assert make_layout([None], [q], [500]).best_fusion is FusionKind.SINGLE
    with pytest.raises(ValueError, match="share their input width"):
        make_layout([0, 1], [q, build_matrix_spec("z", _linear(128, 128, 48, None))], [512, 128])


def test_tp_arithmetic():
    assert even_shard(5120, 8, 3) == (1920, 640)
    assert kv_shard_index(8, 5, 8) == (5, 8) and kv_shard_index(16, 5, 8) == (2, 8)
    assert admissible_tp_degrees(17408) == [1, 2, 4, 8]            # 17408 / 8 = 2176 = 17 * 128
    assert admissible_tp_degrees(512) == [1, 2, 4]                 # MoE intermediate: no 8-way split
    with pytest.raises(SplitError):
        even_shard(5120, 3, 0)


def test_slices_reproduce_the_full_matrix_exactly():
    """A 128-aligned column slice decodes to exactly those columns; row slices sum to the full product."""
    K, cb, k, n = 3, 0, 512, 384
    tr = seeded_trellis(21, k // 16, n // 16, K)
    suh, svh = seeded_signs(22, k), seeded_signs(23, n)
    spec = build_matrix_spec("m", _linear(k, n, 16 * K, None))
    x = np.random.default_rng(24).standard_normal((2, k)).astype(np.float16)
    full = orc.c_linear_forward(x, tr, suh, svh, K, cb)
    sl = column_slice(spec, 128, 256)
    assert sl.sliced_dims(spec) == (k, 256) and sl.suh is None and sl.trellis == type(sl.trellis)(1, 8, 16)
    part = orc.c_linear_forward(x, tr[:, 8:24], suh, svh[128:384], K, cb)
    assert np.array_equal(part, full[:, 128:384])                  # same arithmetic, same bits
    total = np.zeros_like(full, dtype=np.float64)
    for start in (0, 128, 256, 384):
        rs = row_slice(spec, start, 128)
        assert rs.keep_bias == (start == 0) and rs.svh is None
        t0 = rs.trellis.start
        total += orc.c_linear_forward(x[:, start:start + 128], tr[t0:t0 + 8], suh[start:start + 128], svh, K, cb)
    assert orc.max_over_rms(total, full) < 1e-5
    with pytest.raises(SplitError, match="not aligned"):
        column_slice(spec, 64, 128)
    with pytest.raises(SplitError, match="outside the stored width"):
        row_slice(spec, 512, 128)
