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
                      (_key([(512, 256, 6, "3inst")], dtype="float32"), "fp16"), (_key([(512, 256, 6, "3inst")], op=Op.MOE), "gate, up and down"),
                      (_key([(512, 256, 6, "mcg"), (512, 256, 6, "mcg"), (512, 256, 6, "mcg")], op=Op.MOE), "mirrors")]:
        got = be.supports(key)
        assert not got.ok and word in got.reason, (key, got)
    moe_key = _key([(512, 256, 6, "mcg"), (512, 256, 6, "mcg"), (256, 512, 6, "mcg")], op=Op.MOE)
    assert be.supports(moe_key).ok
    for method in ("prepare_moe", "run_moe", "prepare_linear", "run_linear", "warm", "workspace"):
        assert callable(getattr(be, method))


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


@pytest.mark.gpu
def test_after_warm_the_run_path_allocates_nothing_and_captures():
    """The contract's central promise (cuda/src/sglang_exl3/kernels/base.py:74-77): after warm(), run_linear on the
    caller's workspace leaves the allocator untouched and can be captured right away, for row counts on both sides of
    the switch between the decode and the tensor-core kernel."""
    K, k, ns = 4, 1024, [512, 256]
    dev = torch.device("cuda", 0)
    parts = [(seeded_trellis(170 + i, k // 16, n // 16, K), seeded_signs(171 + i, k),
              (seeded_signs(174 + i, n).astype(np.float32) / 32).astype(np.float16)) for i, n in enumerate(ns)]
    specs = [build_matrix_spec(f"m{i}", {"trellis": TensorInfo(f"m{i}.trellis", "I16", (k // 16, n // 16, 16 * K)),
                                         "suh": TensorInfo(f"m{i}.suh", "F16", (k,)), "svh": TensorInfo(f"m{i}.svh", "F16", (n,)),
                                         "mcg": TensorInfo(f"m{i}.mcg", "I32", ())})
             for i, n in enumerate(ns)]
    layout = make_layout(["a", "b"], specs, ns)
    be = B200Backend()
    key = KernelKey(Op.LINEAR, tuple((k, n, 2 * K, "mcg") for n in ns), 300, "float16", "float16", torch.cuda.get_device_capability(dev))
    assert be.supports(key).ok
    tensors = [{"trellis": torch.from_numpy(t.view(np.int16)).to(dev), "suh": torch.from_numpy(su).to(dev), "svh": torch.from_numpy(sv).to(dev)}
               for t, su, sv in parts]
    handle = be.prepare_linear(layout, tensors)
    ws = torch.zeros(be.workspace(key, 300).nbytes, dtype=torch.uint8, device=dev)
    be.warm(handle, key, ws)
    rng = np.random.default_rng(8)
    for rows in (1, 16, 17, 300):
        x = torch.from_numpy(rng.standard_normal((rows, k)).astype(np.float16)).to(dev)
        out = torch.empty((rows, sum(ns)), dtype=torch.float16, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        be.run_linear(handle, x, out, ws)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before, rows
        eager = out.clone()
        g = torch.cuda.CUDAGraph()
        out.zero_()
        with torch.cuda.graph(g):
            be.run_linear(handle, x, out, ws)
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, eager), rows
        ref = np.concatenate([orc.c_linear_forward(x.cpu().numpy(), t, su, sv, K, 1) for t, su, sv in parts], axis=1)
        assert orc.rel_norm(out.float().cpu().numpy(), ref) <= 2e-3, rows


@pytest.mark.gpu
def test_routed_experts_through_the_contract():
    """prepare_moe / warm / run_moe on a caller-owned workspace: the float64 layer's answer, no allocation on the run path,
    and an engine-style expert map (experts 1 and 3 held elsewhere) drops exactly those experts' contributions."""
    E, hidden, inter, top_k, K, cb, tokens = 6, 256, 128, 2, 3, 0, 5
    dev = torch.device("cuda", 0)

    def proj(k, n, base):
        return [(seeded_trellis(base + e, k // 16, n // 16, K), seeded_signs(base + 100 + e, k),
                 (seeded_signs(base + 200 + e, n).astype(np.float32) / 8).astype(np.float16)) for e in range(E)]
    gate, up, down = proj(hidden, inter, 300), proj(hidden, inter, 1300), proj(inter, hidden, 2300)

    def spec(name, k, n):
        return build_matrix_spec(name, {"trellis": TensorInfo(name + ".trellis", "I16", (k // 16, n // 16, 16 * K)),
                                        "suh": TensorInfo(name + ".suh", "F16", (k,)), "svh": TensorInfo(name + ".svh", "F16", (n,))})
    to_dev = lambda lst: [{"trellis": torch.from_numpy(t.view(np.int16)).to(dev), "suh": torch.from_numpy(su).to(dev),
                           "svh": torch.from_numpy(sv).to(dev)} for t, su, sv in lst]
    be = B200Backend(max_top_k=top_k, max_experts=E)
    key = KernelKey(Op.MOE, ((hidden, inter, 2 * K, "3inst"), (hidden, inter, 2 * K, "3inst"), (inter, hidden, 2 * K, "3inst")), 8,
                    "float16", "float16", torch.cuda.get_device_capability(dev))
    assert be.supports(key).ok
    emap = torch.tensor([0, -1, 1, -1, 2, 3], dtype=torch.int32, device=dev)         # engine view: this rank holds 0, 2, 4, 5
    held = [0, 2, 4, 5]
    handle = be.prepare_moe([spec(f"g{e}", hidden, inter) for e in range(E)], [spec(f"u{e}", hidden, inter) for e in range(E)],
                            [spec(f"d{e}", inter, hidden) for e in range(E)],
                            {"gate": to_dev(gate), "up": to_dev(up), "down": to_dev(down)})
    local = be.prepare_moe([spec(f"g{e}", hidden, inter) for e in held], [spec(f"u{e}", hidden, inter) for e in held],
                           [spec(f"d{e}", inter, hidden) for e in held],
                           {"gate": to_dev([gate[e] for e in held]), "up": to_dev([up[e] for e in held]),
                            "down": to_dev([down[e] for e in held]), "expert_map": emap})
    ws = torch.zeros(be.workspace(key, 8).nbytes, dtype=torch.uint8, device=dev)
    be.warm(handle, key, ws)
    be.warm(local, key, ws)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((tokens, hidden)).astype(np.float16)
    ids = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, top_k)).astype(np.float32)
    cols = lambda lst: tuple([p[i] for p in lst] for i in range(3))
    xs, idt, wt = torch.from_numpy(x).to(dev), torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev)
    out, out2 = torch.empty_like(xs), torch.empty_like(xs)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    be.run_moe(handle, xs, idt, wt, out, ws, None)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    ref = orc.np_moe_layer(x, ids, w, cols(gate), cols(up), cols(down), K, cb)
    assert orc.rel_norm(out.float().cpu().numpy(), ref) <= 3e-3
    be.run_moe(local, xs, idt, wt, out2, ws, emap)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    ids_held = np.where(np.isin(ids, held), ids, -1)
    ref2 = orc.np_moe_layer(x, ids_held, w, cols(gate), cols(up), cols(down), K, cb)
    assert orc.rel_norm(out2.float().cpu().numpy(), ref2) <= 3e-3
