"""Load path: a small checkpoint directory written with the safetensors library (modern suh/svh, legacy packed su/sv, an
mcg marker, a bias, a 128-padded output width) is scanned by the manifest, read back, and -- on a GPU -- prepared and run
against the oracle's forward of the same stored tensors."""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.format import FormatError, load_manifest
from trellis_serve_b200.runtime import loader

K = 3
HID, Q, KV = 256, 256, 128


def _pack_signs(v: np.ndarray) -> np.ndarray:
    bits = ((1 - v.astype(np.int32)) // 2).reshape(-1, 16)                # 1 = negative
    return (bits << np.arange(16)).sum(1).astype(np.uint16).view(np.int16)


def _write_checkpoint(tmp_path):
    from safetensors.numpy import save_file
    mats = {}
    t = {}
    for i, (key, k, n) in enumerate([("m.q_proj", HID, Q), ("m.k_proj", HID, KV), ("m.o_proj", Q, HID)]):
        tr = seeded_trellis(40 + i, k // 16, n // 16, K)
        suh, svh = seeded_signs(50 + i, k), seeded_signs(60 + i, n)
        mats[key] = (tr, suh, svh)
        t[f"{key}.trellis"] = tr.view(np.int16)
        if key == "m.k_proj":                                             # legacy packed signs
            t[f"{key}.su"], t[f"{key}.sv"] = _pack_signs(suh), _pack_signs(svh)
        else:
            t[f"{key}.suh"], t[f"{key}.svh"] = suh, svh
    t["m.o_proj.mcg"] = np.array([1], dtype=np.int32)
    bias = np.linspace(-1, 1, HID).astype(np.float16)
    t["m.o_proj.bias"] = bias
    t["m.norm.weight"] = np.ones(HID, dtype=np.float16)
    half = {k: v for i, (k, v) in enumerate(sorted(t.items())) if i % 2 == 0}
    rest = {k: v for k, v in t.items() if k not in half}
    save_file(half, os.path.join(tmp_path, "model-00001-of-00002.safetensors"))
    save_file(rest, os.path.join(tmp_path, "model-00002-of-00002.safetensors"))
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"quantization_config": {"quant_method": "exl3", "bits": 3.0}}, f)
    return mats, bias


def test_unpack_signs_is_the_inverse_of_the_legacy_packing():
    v = seeded_signs(7, 256)
    got = loader.unpack_signs(torch.from_numpy(_pack_signs(v)))
    assert got.dtype == torch.float16 and np.array_equal(got.numpy(), v)
    with pytest.raises(FormatError):
        loader.unpack_signs(torch.zeros(4, dtype=torch.int32))


def test_manifest_and_tensor_reads_of_a_two_shard_checkpoint(tmp_path):
    mats, bias = _write_checkpoint(tmp_path)
    man = load_manifest(tmp_path)
    assert sorted(man.matrices) == ["m.k_proj", "m.o_proj", "m.q_proj"] and list(man.unquantized) == ["m.norm.weight"]
    assert man.matrices["m.k_proj"].legacy_signs and man.matrices["m.o_proj"].has_bias
    assert man.matrices["m.o_proj"].codebook.value == "mcg" and man.matrices["m.q_proj"].codebook.value == "3inst"
    got = loader.read_tensors(tmp_path, man.matrices["m.k_proj"])
    assert sorted(got) == ["su", "sv", "trellis"]
    assert np.array_equal(got["trellis"].numpy().view(np.uint16), mats["m.k_proj"][0])
    assert np.array_equal(loader.unpack_signs(got["su"]).numpy(), mats["m.k_proj"][1])
    with pytest.raises(FormatError):
        loader.load_group(tmp_path, ["m.norm"], device="cpu", manifest=man)
    q, o = man.matrices["m.q_proj"], man.matrices["m.o_proj"]
    with pytest.raises(FormatError):                                      # different codebooks do not fuse
        loader.group_from_tensors([q, o], [loader.read_tensors(tmp_path, q), loader.read_tensors(tmp_path, o)], "cpu")


@pytest.mark.gpu
def test_loaded_groups_match_the_oracle(tmp_path):
    mats, bias = _write_checkpoint(tmp_path)
    x = np.random.default_rng(1).standard_normal((3, HID)).astype(np.float16)
    qk = loader.load_group(tmp_path, ["m.q_proj", "m.k_proj"], out_widths=[Q, 100])       # k_proj's true width is 100 of 128
    assert qk.ends == [Q] and qk.out_widths == [Q, 100] and qk.codebook == 0
    y = qk.forward(torch.from_numpy(x).cuda()).float().cpu().numpy()
    assert y.shape == (3, Q + 100)
    ref_q = orc.c_linear_forward(x, *mats["m.q_proj"], K, 0)
    ref_k = orc.c_linear_forward(x, *mats["m.k_proj"], K, 0)[:, :100]
    assert orc.rel_norm(y, np.concatenate([ref_q, ref_k], 1)) <= 2e-3
    o = loader.load_group(tmp_path, ["m.o_proj"])
    a = np.random.default_rng(2).standard_normal((2, Q)).astype(np.float16)
    yo = o.forward(torch.from_numpy(a).cuda()).float().cpu().numpy()
    ref_o = orc.c_linear_forward(a, *mats["m.o_proj"], K, 1) + bias.astype(np.float32)
    assert orc.rel_norm(yo, ref_o) <= 2e-3
