"""The backend contract (kernels/base.py): the B200 backend object satisfies the protocol, refuses what it cannot serve
with a reason at load time, and -- on a GPU -- prepares, warms and runs a fused module to the oracle's answer."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.format import TensorInfo, build_matrix_spec, make_layout
from trellis_serve_b200.kernels.base import B200Backend, Backend, KernelKey, Op, ParityClass


def _key(layout_class, cap=(10, 0), dtype="float16", op=Op.LINEAR):
    return KernelKey(op, tuple(layout_class), 16, dtype, dtype, cap)


def test_protocol_and_load_time_refusals():
    be = B200Backend()
    assert isinstance(be, Backend) and be.name == "b200"
    ok = be.supports(_key([(512, 256, 6, "3inst"), (512, 128, 6, "3inst")]))
    assert ok.ok and ok.reason == ""
    assert be.parity(_key([(512, 256, 6, "mcg")])) is ParityClass.NUMERICAL and be.graph_safe(_key([(512, 256, 6, "mcg")]))
    for key, word in [(_key([(512, 256, 5, "mul1")]), "integer bitrates"), (_key([(512, 256, 6, "3inst")], cap=(9, 0)), "sm_100"),
                      (_key([(512, 256, 6, "3inst"), (512, 128, 8, "3inst")]), "share"), (_key([(500, 256, 6, "3inst")]), "128"),
                      (_key([(512, 256, 6, "3inst")], dtype="float32"), "fp16"), (_key([(512, 256, 6, "3inst")], op=Op.MOE), "experts")]:
        got = be.supports(key)
        assert not got.ok and word in got.reason, (key, got)


@pytest.mark.gpu
def test_prepare_warm_run_matches_the_oracle():
    K, cb, k, ns, rows = 3, 0, 512, [256, 128], 2
    dev = torch.device("cuda", 0)
    parts = [(seeded_trellis(70 + i, k // 16, n // 16, K), seeded_signs(71 + i, k), seeded_signs(74 + i, n)) for i, n in enumerate(ns)]
    specs = [build_matrix_spec(f"m{i}", {"trellis": TensorInfo(f"m{i}.trellis", "I16", (k // 16, n // 16, 16 * K)),
                                         "suh": TensorInfo(f"m{i}.suh", "F16", (k,)), "svh": TensorInfo(f"m{i}.svh", "F16", (n,))})
             for i, n in enumerate(ns)]
    layout = make_layout(["a", "b"], specs, ns)
    be = B200Backend()
    assert be.probe().available
    key = KernelKey(Op.LINEAR, tuple((k, n, 2 * K, "3inst") for n in ns), 16, "float16", "float16", torch.cuda.get_device_capability(dev))
    assert be.supports(key).ok
    tensors = [{"trellis": torch.from_numpy(t.view(np.int16)).to(dev), "suh": torch.from_numpy(su).to(dev), "svh": torch.from_numpy(sv).to(dev)}
               for t, su, sv in parts]
    handle = be.prepare_linear(layout, tensors)
    assert be.workspace(key, 16).nbytes > 0
    be.warm(handle, key, None)
    x = np.random.default_rng(4).standard_normal((rows, k)).astype(np.float16)
    out = torch.empty((rows, sum(ns)), dtype=torch.float16, device=dev)
    be.run_linear(handle, torch.from_numpy(x).to(dev), out, None)
    ref = np.concatenate([orc.c_linear_forward(x, t, su, sv, K, cb) for t, su, sv in parts], axis=1)
    assert orc.rel_norm(out.float().cpu().numpy(), ref) <= 2e-3
