"""Engine glue (trellis_serve_b200/sglang_glue): driven without an engine through doubles of its three layer classes, from a
small checkpoint directory written with the safetensors library.  CPU: config scan and lookups, placeholder registration,
loader bookkeeping and every refusal.  GPU: create_weights -> weight loaders -> process_weights_after_loading -> apply against
the oracle, tensor-parallel shares of one layer against the whole, and the routed experts (whole layer and an
expert-parallel share)."""
from __future__ import annotations

import json
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from conftest import seeded_signs, seeded_trellis
from oracle import exl3_oracle as orc
from trellis_serve_b200.sglang_glue import Exl3Config, Exl3LinearMethod, Exl3MoEMethod

K, HID, Q, KV, INTER, E = 3, 256, 256, 128, 128, 4


class LinearBase(torch.nn.Module):
    """Double of the engine's linear layer: only the class name and the tp attributes matter to the glue."""

    def __init__(self, tp_rank=0, tp_size=1):
        super().__init__()
        self.tp_rank, self.tp_size = tp_rank, tp_size


class ParallelLMHead(torch.nn.Module):
    pass


class FusedMoE(torch.nn.Module):
    moe_tp_size = 1


def _pack_signs(v: np.ndarray) -> np.ndarray:
    bits = ((1 - v.astype(np.int32)) // 2).reshape(-1, 16)
    return (bits << np.arange(16)).sum(1).astype(np.uint16).view(np.int16)


def _checkpoint(tmp_path):
    from safetensors.numpy import save_file
    t, mats = {}, {}
    layout = [("model.layers.0.self_attn.q_proj", HID, Q), ("model.layers.0.self_attn.k_proj", HID, KV),
              ("model.layers.0.self_attn.v_proj", HID, KV), ("model.layers.0.self_attn.o_proj", Q, HID), ("lm_head", HID, 384)]
    for e in range(E):
        layout += [(f"model.layers.0.mlp.experts.{e}.gate_proj", HID, INTER), (f"model.layers.0.mlp.experts.{e}.up_proj", HID, INTER),
                   (f"model.layers.0.mlp.experts.{e}.down_proj", INTER, HID)]
    for i, (key, k, n) in enumerate(layout):
        tr = seeded_trellis(400 + i, k // 16, n // 16, K)
        suh = seeded_signs(500 + i, k)
        svh = (seeded_signs(600 + i, n).astype(np.float32) / 8).astype(np.float16)
        mats[key] = (tr, suh, svh)
        t[f"{key}.trellis"] = tr.view(np.int16)
        if key.endswith("k_proj"):                                        # legacy packed signs (svh then is +-1)
            svh = seeded_signs(600 + i, n)
            mats[key] = (tr, suh, svh)
            t[f"{key}.su"], t[f"{key}.sv"] = _pack_signs(suh), _pack_signs(svh)
        else:
            t[f"{key}.suh"], t[f"{key}.svh"] = suh, svh
    t["model.norm.weight"] = np.ones(HID, dtype=np.float16)
    t["model.layers.0.mlp.gate.weight"] = np.zeros((E, HID), dtype=np.float16)
    save_file(t, os.path.join(tmp_path, "model.safetensors"))
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump({"quantization_config": {"quant_method": "exl3", "bits": 3.0}}, f)
    return mats, t


def _deliver(layer, tensors: dict, key: str, shard_id=None, **kw):
    """What a model's load_weights does: every stored tensor of `key` goes to the parameter named like its suffix."""
    for name, value in tensors.items():
        if name.startswith(key + "."):
            suffix = name[len(key) + 1:]
            param = getattr(layer, kw.get("param_prefix", "") + suffix)
            v = torch.from_numpy(np.ascontiguousarray(value))
            if "expert_id" in kw:
                param.weight_loader(param, v, name, shard_id=shard_id, expert_id=kw["expert_id"])
            else:
                param.weight_loader(param, v, shard_id) if shard_id is not None else param.weight_loader(param, v)


# ------------------------------------------------------------------------------------------------ CPU

def test_config_scans_headers_and_hands_out_methods(tmp_path):
    _checkpoint(tmp_path)
    cfg = Exl3Config.from_config({"hf_config": SimpleNamespace(_name_or_path=str(tmp_path))})
    assert cfg.get_name() == "exl3" and cfg.get_min_capability() == 100 and not cfg.can_fuse_shared_expert()
    assert Exl3Config.override_quantization_method({"quant_method": "exl3"}, None) == "exl3"
    assert Exl3Config.override_quantization_method({"quant_method": "awq"}, None) is None
    assert cfg.modules["lm_head"] == (HID, 384, 2 * K, "3inst", False, False)
    assert cfg.modules["model.layers.0.self_attn.k_proj"][5] is True                     # legacy signs
    # prefix spellings an engine uses
    assert cfg.lookup("model.language_model.layers.0.self_attn.q_proj") == cfg.modules["model.layers.0.self_attn.q_proj"]
    assert cfg.lookup("model.layers.0.self_attn.nope") is None
    assert cfg.sources("model.layers.0.self_attn.qkv_proj") == [f"model.layers.0.self_attn.{p}_proj" for p in "qkv"]
    m = cfg.get_quant_method(LinearBase(), "model.layers.0.self_attn.qkv_proj")
    assert isinstance(m, Exl3LinearMethod) and len(m.infos) == 3
    assert isinstance(cfg.get_quant_method(ParallelLMHead(), "lm_head"), Exl3LinearMethod)
    moe = cfg.get_quant_method(FusedMoE(), "model.layers.0.mlp.experts")
    assert isinstance(moe, Exl3MoEMethod) and len(moe.infos) == 3 * E and ("down", E - 1) in moe.infos
    assert cfg.get_quant_method(LinearBase(), "model.layers.0.mlp.gate") is None         # left unquantized, no engine here
    assert cfg.get_quant_method(torch.nn.LayerNorm(4), "model.norm") is None
    cfg.modules.pop("model.layers.0.self_attn.v_proj")
    with pytest.raises(ValueError, match="mixes EXL3 and unquantized"):
        cfg.get_quant_method(LinearBase(), "model.layers.0.self_attn.qkv_proj")
    with pytest.raises(ValueError, match="no local checkpoint"):
        Exl3Config.from_config({"hf_config": SimpleNamespace(_name_or_path="/nonexistent/dir")})


def test_linear_method_bookkeeping_and_refusals(tmp_path):
    mats, tensors = _checkpoint(tmp_path)
    cfg = Exl3Config(model_path=str(tmp_path))
    method = cfg.get_quant_method(LinearBase(), "model.layers.0.self_attn.qkv_proj")
    layer = LinearBase()
    method.create_weights(layer, HID, [Q, KV, KV], HID, Q + 2 * KV, torch.float16)
    for suffix in ("trellis", "suh", "svh", "su", "sv", "mcg", "mul1"):
        p = getattr(layer, suffix)
        assert p.numel() == 0 and p.exl3_placeholder and callable(p.weight_loader)
    _deliver(layer, tensors, "model.layers.0.self_attn.q_proj", "q")
    with pytest.raises(ValueError, match="loaded twice"):
        _deliver(layer, tensors, "model.layers.0.self_attn.q_proj", "q")
    with pytest.raises(ValueError, match="expected 3 EXL3 matrices"):
        method.process_weights_after_loading(layer)
    # an LM head gets a zero-width `.weight` with one row per output
    head, hm = ParallelLMHead(), cfg.get_quant_method(ParallelLMHead(), "lm_head")
    hm.create_weights(head, HID, [384], HID, 384, torch.bfloat16)
    assert tuple(head.weight.shape) == (384, 0)
    hm.process_weights_after_loading(head)                                   # nothing delivered: left empty, not an error
    with pytest.raises(RuntimeError, match="never loaded"):
        hm.apply(head, torch.zeros(1, HID))
    # a shard whose tensors contradict the header scan
    wrong = LinearBase()
    om = Exl3LinearMethod("model.layers.0.self_attn.o_proj", [(Q, HID, 8, "3inst", False, False)])
    om.create_weights(wrong, Q, [HID], Q, HID, torch.float16)
    _deliver(wrong, tensors, "model.layers.0.self_attn.o_proj")
    with pytest.raises(ValueError, match="does not match the header scan"):
        om.process_weights_after_loading(wrong)
    # partition sizes that need tensor-parallel coordinates the layer does not have
    with pytest.raises(NotImplementedError, match="tp_rank"):
        om.create_weights(LinearBase(), Q // 2, [HID], Q, HID, torch.float16)


def test_moe_method_bookkeeping_and_refusals(tmp_path):
    mats, tensors = _checkpoint(tmp_path)
    cfg = Exl3Config(model_path=str(tmp_path))
    method = cfg.get_quant_method(FusedMoE(), "model.layers.0.mlp.experts")
    layer = FusedMoE()
    method.create_weights(layer, E, HID, INTER, torch.float16)
    assert all(hasattr(layer, f"{w}_{s}") for w in ("w13", "w2") for s in ("trellis", "suh", "svh", "su", "sv", "mcg", "mul1"))
    _deliver(layer, tensors, "model.layers.0.mlp.experts.0.gate_proj", "w1", expert_id=0, param_prefix="w13_")
    with pytest.raises(ValueError, match="loaded twice"):
        _deliver(layer, tensors, "model.layers.0.mlp.experts.0.gate_proj", "w1", expert_id=0, param_prefix="w13_")
    with pytest.raises(ValueError, match="unexpected expert shard"):
        layer.w13_trellis.weight_loader(layer.w13_trellis, torch.zeros(1), "x", shard_id="w9", expert_id=0)
    with pytest.raises(ValueError, match="delivered for 1 experts"):
        method.process_weights_after_loading(layer)
    for bad, word in [(SimpleNamespace(activation="gelu", is_gated=True), "SiLU"),
                      (SimpleNamespace(activation="silu", apply_router_weight_on_input=True), "apply_router_weight_on_input"),
                      (SimpleNamespace(activation="silu", routed_scaling_factor=2.5), "routed_scaling_factor")]:
        with pytest.raises(NotImplementedError, match=word):
            method.create_moe_runner(layer, bad)
    method.create_moe_runner(layer, SimpleNamespace(activation="silu", top_k=2))
    shared = FusedMoE()
    shared.num_fused_shared_experts = 1
    with pytest.raises(NotImplementedError, match="shared experts"):
        method.create_weights(shared, E, HID, INTER, torch.float16)
    with pytest.raises(ValueError, match="unexpected EXL3 matrix"):
        Exl3MoEMethod(cfg, "p", {"model.layers.0.mlp.experts.0.router": (1, 1, 6, "3inst", False, False)})


# ------------------------------------------------------------------------------------------------ GPU

def _loaded_linear(cfg, tensors, prefix, shard_keys, in_size, out_sizes, tp=(0, 1), mode="none"):
    layer = LinearBase(*tp)
    method = cfg.get_quant_method(layer, prefix)
    full_in, full_out = in_size, sum(out_sizes)
    part_in = in_size // tp[1] if mode == "row" else in_size
    part_out = [w // tp[1] for w in out_sizes] if mode == "column" else list(out_sizes)
    method.create_weights(layer, part_in, part_out, full_in, full_out, torch.float16)
    for key, sid in shard_keys:
        _deliver(layer, tensors, key, sid)
    method.process_weights_after_loading(layer)
    return layer, method


@pytest.mark.gpu
def test_linear_layers_end_to_end_and_tensor_parallel_shares(tmp_path):
    mats, tensors = _checkpoint(tmp_path)
    cfg = Exl3Config(model_path=str(tmp_path))
    qkv_keys = [(f"model.layers.0.self_attn.{p}_proj", p) for p in "qkv"]
    layer, method = _loaded_linear(cfg, tensors, "model.layers.0.self_attn.qkv_proj", qkv_keys, HID, [Q, KV, KV])
    assert not hasattr(layer, "trellis") and layer.exl3_count == 3 and layer.exl3_widths == [Q, KV, KV]
    x = np.random.default_rng(1).standard_normal((2, 3, HID)).astype(np.float16)
    y = method.apply(layer, torch.from_numpy(x).cuda())
    assert y.shape == (2, 3, Q + 2 * KV)
    ref = np.concatenate([orc.c_linear_forward(x.reshape(6, HID), *mats[k], K, 0) for k, _ in qkv_keys], axis=1)
    assert orc.rel_norm(y.float().cpu().numpy().reshape(6, -1), ref) <= 2e-3
    bias = torch.linspace(-1, 1, Q + 2 * KV, device="cuda", dtype=torch.float16)
    assert torch.equal(method.apply(layer, torch.from_numpy(x).cuda(), bias), y + bias)
    o_keys = [("model.layers.0.self_attn.o_proj", None)]
    whole, wm = _loaded_linear(cfg, tensors, "model.layers.0.self_attn.o_proj", o_keys, Q, [HID])
    a = torch.from_numpy(np.random.default_rng(2).standard_normal((4, Q)).astype(np.float16)).cuda()
    full = wm.apply(whole, a).float()
    parts = []
    for r in range(2):                                                        # row-parallel: each rank sees its half of the input
        shard, sm = _loaded_linear(cfg, tensors, "model.layers.0.self_attn.o_proj", o_keys, Q, [HID], tp=(r, 2), mode="row")
        parts.append(sm.apply(shard, a[:, r * Q // 2:(r + 1) * Q // 2].contiguous()).float())
    assert orc.rel_norm((parts[0] + parts[1]).cpu().numpy(), full.cpu().numpy()) <= 2e-3
    cols = []
    for r in range(2):                                                        # column-parallel: each rank owns half of the outputs
        shard, sm = _loaded_linear(cfg, tensors, "model.layers.0.self_attn.o_proj", o_keys, Q, [HID], tp=(r, 2), mode="column")
        cols.append(sm.apply(shard, a))
    assert torch.equal(torch.cat(cols, dim=1), wm.apply(whole, a))


@pytest.mark.gpu
def test_routed_experts_end_to_end_and_an_expert_parallel_share(tmp_path):
    mats, tensors = _checkpoint(tmp_path)
    cfg = Exl3Config(model_path=str(tmp_path))
    top_k, tokens = 2, 5

    def build(experts, expert_map=None):
        layer = FusedMoE()
        if expert_map is not None:
            layer.expert_map = expert_map
        method = cfg.get_quant_method(layer, "model.layers.0.mlp.experts")
        method.create_weights(layer, len(experts), HID, INTER, torch.float16)
        method.create_moe_runner(layer, SimpleNamespace(activation="silu", top_k=top_k))
        for local, e in enumerate(experts):
            for proj, sid, w in (("gate_proj", "w1", "w13_"), ("up_proj", "w3", "w13_"), ("down_proj", "w2", "w2_")):
                _deliver(layer, tensors, f"model.layers.0.mlp.experts.{e}.{proj}", sid, expert_id=local, param_prefix=w)
        method.process_weights_after_loading(layer)
        return layer, method
    rng = np.random.default_rng(5)
    x = rng.standard_normal((tokens, HID)).astype(np.float16)
    ids = np.stack([rng.choice(E, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, top_k)).astype(np.float32)
    cols = lambda proj, es: tuple([mats[f"model.layers.0.mlp.experts.{e}.{proj}"][i] for e in es] for i in range(3))
    dispatch = SimpleNamespace(hidden_states=torch.from_numpy(x).cuda(),
                               topk_output=SimpleNamespace(topk_weights=torch.from_numpy(w).cuda(), topk_ids=torch.from_numpy(ids).cuda()))
    layer, method = build(range(E))
    assert not hasattr(layer, "w13_trellis")
    y = method.apply(layer, dispatch).hidden_states
    ref = orc.np_moe_layer(x, ids, w, cols("gate_proj", range(E)), cols("up_proj", range(E)), cols("down_proj", range(E)), K, 0)
    assert orc.rel_norm(y.float().cpu().numpy(), ref) <= 3e-3
    held = [1, 3]                                                             # an expert-parallel share: experts 1 and 3 only
    emap = torch.tensor([-1, 0, -1, 1], dtype=torch.int32, device="cuda")
    part, pm = build(held, emap)
    yp = pm.apply(part, dispatch).hidden_states
    ids_held = np.where(np.isin(ids, held), ids, -1)
    refp = orc.np_moe_layer(x, ids_held, w, cols("gate_proj", range(E)), cols("up_proj", range(E)), cols("down_proj", range(E)), K, 0)
    assert orc.rel_norm(yp.float().cpu().numpy(), refp) <= 3e-3
