"""`Exl3MoEMethod`: EXL3 routed experts for an engine's fused MoE layer.

Interface and loader semantics of the reference's cuda/src/sglang_exl3/sglang_glue/moe.py (create_weights :69,
create_moe_runner :109, process_weights_after_loading :121, apply :231): the model's `load_weights` maps
`experts.E.{gate,up,down}_proj.<suffix>` to parameters named `w13_<suffix>` (shard ids w1 = gate, w3 = up) and
`w2_<suffix>` (w2 = down) and calls `param.weight_loader(param, tensor, name, shard_id=, expert_id=)`; placeholders with
those names are registered for every suffix an EXL3 checkpoint can carry, the loader files the tensors under (projection,
suffix, expert) on the CPU until the layer is complete, and `process_weights_after_loading` checks them against the
header scan and builds the resident expert stacks.

Beyond the reference (which serves one bitrate per layer, tensor and expert parallel degree 1): experts of mixed bit rate
are grouped into one pack per bitrate class, and a layer that holds only some experts (expert parallelism: the engine
hands the layer an `expert_map` of global -> local ids) routes through that map; the sum over ranks is the engine's.
"""
from __future__ import annotations

import logging
import re

import torch

from ..kernels import moe as moe_kernels
from ..runtime import loader
from ._engine import FusedMoEMethodBase, StandardCombineInput, set_weight_attrs

logger = logging.getLogger(__name__)
SUFFIXES = ("trellis", "suh", "svh", "su", "sv", "mcg", "mul1")
_CODEBOOK_ID = {"3inst": 0, "mcg": 1, "mul1": 2}
_ROLE = {"w1": "gate", "w3": "up", "w2": "down"}
_KEY_RE = re.compile(r"\.experts\.(\d+)\.(gate_proj|up_proj|down_proj)$")
WARM_TOKENS = 8


class Exl3MoEMethod(FusedMoEMethodBase):
    """`experts`: checkpoint key -> (k, n, twice the bitrate, codebook name, has_bias, legacy signs) for every matrix under
    this layer's `.experts.` (from `Exl3Config.modules`)."""

    def __init__(self, config, prefix: str, experts: dict[str, tuple]):
        self.config = config
        self.prefix = prefix
        self.runner = None                      # the engine reads quant_method.runner; its MoE runner stack is bypassed
        self.moe_runner_config = None
        self.infos: dict[tuple[str, int], tuple] = {}
        for key, info in experts.items():
            m = _KEY_RE.search(key)
            if m is None:
                raise ValueError(f"{prefix}: unexpected EXL3 matrix under the experts: {key}")
            self.infos[(m.group(2)[:-5], int(m.group(1)))] = info

    # ---------------------------------------------------------------------------------------------- weights
    def create_weights(self, layer, num_experts, hidden_size, intermediate_size_per_partition, params_dtype, **extra_weight_attrs):
        if getattr(layer, "moe_tp_size", 1) != 1:
            raise NotImplementedError(f"{self.prefix}: experts are not split along their intermediate dimension; use expert parallelism")
        if getattr(layer, "num_fused_shared_experts", 0):
            raise NotImplementedError(f"{self.prefix}: fused shared experts are not supported by the EXL3 MoE method; "
                                      f"run with --disable-shared-experts-fusion")
        if extra_weight_attrs.get("with_bias"):
            raise NotImplementedError(f"{self.prefix}: EXL3 experts with bias are not implemented")
        layer.exl3_store = {}                   # (role, suffix) -> {expert id as the loader names it: tensor (CPU copy)}
        layer.exl3_num_experts = num_experts    # experts this layer holds (all of them, or this rank's share)
        layer.exl3_hidden = hidden_size
        layer.exl3_inter = intermediate_size_per_partition
        for w in ("w13", "w2"):
            for suffix in SUFFIXES:
                p = torch.nn.Parameter(torch.empty(0, dtype=torch.uint8), requires_grad=False)
                set_weight_attrs(p, {"weight_loader": self._make_loader(layer, suffix), "exl3_placeholder": True})
                layer.register_parameter(f"{w}_{suffix}", p)

    def _make_loader(self, layer, suffix: str):
        def load(param, loaded_weight, weight_name=None, shard_id=None, expert_id=None, *args, **kwargs):
            role = _ROLE.get(shard_id)
            if role is None or expert_id is None:
                raise ValueError(f"{self.prefix}.{suffix}: unexpected expert shard {shard_id!r} / expert {expert_id!r}")
            store = layer.exl3_store.setdefault((role, suffix), {})
            e = int(expert_id)
            if e in store:
                raise ValueError(f"{self.prefix}: {role} {suffix} of expert {e} loaded twice")
            store[e] = loaded_weight.detach().to("cpu", copy=True)
        return load

    def create_moe_runner(self, layer, moe_runner_config):
        self.moe_runner_config = cfg = moe_runner_config
        if getattr(cfg, "activation", "silu") != "silu" or not getattr(cfg, "is_gated", True):
            raise NotImplementedError(f"{self.prefix}: only SiLU-gated experts are implemented (got {getattr(cfg, 'activation', None)})")
        if getattr(cfg, "apply_router_weight_on_input", False):
            raise NotImplementedError(f"{self.prefix}: apply_router_weight_on_input is not supported")
        if getattr(cfg, "routed_scaling_factor", None) not in (None, 1.0):
            raise NotImplementedError(f"{self.prefix}: routed_scaling_factor {cfg.routed_scaling_factor} is not supported")
        if getattr(cfg, "num_fused_shared_experts", 0):
            raise NotImplementedError(f"{self.prefix}: fused shared experts are not supported (--disable-shared-experts-fusion)")

    def process_weights_after_loading(self, layer) -> None:
        store, n = layer.exl3_store, layer.exl3_num_experts
        held = sorted(store.get(("gate", "trellis"), {}))
        if len(held) != n:
            raise ValueError(f"{self.prefix}: gate_proj trellis delivered for {len(held)} experts, the layer holds {n}")
        books = set()
        per: dict[str, tuple[list, list, list]] = {}
        for role in ("gate", "up", "down"):
            tensors = {s: store.get((role, s), {}) for s in SUFFIXES}
            missing = [e for e in held if e not in tensors["trellis"]]
            if missing:
                raise ValueError(f"{self.prefix}: {role}_proj trellis missing for {len(missing)} experts, e.g. {missing[0]}")
            trellis, suh, svh = [], [], []
            for e in held:
                t = tensors["trellis"][e]
                su, sv = tensors["suh"].get(e), tensors["svh"].get(e)
                if su is None and e in tensors["su"]:
                    su, sv = loader.unpack_signs(tensors["su"][e]), loader.unpack_signs(tensors["sv"][e])
                if su is None or sv is None:
                    raise ValueError(f"{self.prefix}: {role}_proj of expert {e} has a trellis but no scale vectors")
                codebook = "mcg" if e in tensors["mcg"] else "mul1" if e in tensors["mul1"] else "3inst"
                info = self.infos.get((role, e))
                if info is not None and (t.shape[0] * 16, t.shape[1] * 16, t.shape[2] // 8, codebook) != tuple(info[:4]):
                    raise ValueError(f"{self.prefix}: {role}_proj expert {e} {tuple(t.shape)}/{codebook} does not match "
                                     f"the header scan {tuple(info[:4])}")
                books.add(codebook)
                trellis.append(t.contiguous())
                suh.append(su.to(torch.float16).contiguous())
                svh.append(sv.to(torch.float16).contiguous())
            per[role] = (trellis, suh, svh)
        if len(books) != 1:
            raise NotImplementedError(f"{self.prefix}: mixed codebooks {sorted(books)}")
        if any(g.shape[2] != u.shape[2] for g, u in zip(per["gate"][0], per["up"][0])):
            raise NotImplementedError(f"{self.prefix}: gate and up bitrates of an expert differ")
        kt, nt = per["gate"][0][0].shape[:2]
        if kt * 16 != layer.exl3_hidden or nt * 16 != layer.exl3_inter or per["down"][0][0].shape[:2] != (nt, kt):
            raise ValueError(f"{self.prefix}: expert shapes {tuple(per['gate'][0][0].shape)} / {tuple(per['down'][0][0].shape)} "
                             f"do not fit hidden {layer.exl3_hidden}, intermediate {layer.exl3_inter}")
        layer.exl3_codebook = _CODEBOOK_ID[books.pop()]
        store.clear()
        del layer.exl3_store
        for w in ("w13", "w2"):
            for suffix in SUFFIXES:
                delattr(layer, f"{w}_{suffix}")
        dev = torch.device("cuda", torch.cuda.current_device())
        to_dev = lambda group: tuple([t.to(dev) for t in lst] for lst in group)
        pack = moe_kernels.prepare_mixed(to_dev(per["gate"]), to_dev(per["up"]), to_dev(per["down"]), layer.exl3_codebook)
        for c, pk in enumerate(pack.packs):
            for name, t in zip(("w13", "w2", "suh13", "svh13", "suh2", "svh2"), pk.tensors()):
                layer.register_buffer(f"exl3_pack{c}_{name}", t, persistent=False)
        layer.exl3_pack = pack
        layer.exl3_bits = pack.bits
        # an engine that spreads the experts over ranks gives the layer a map from global expert ids to the local ones
        emap = getattr(layer, "expert_map", None)
        layer.exl3_maps = None
        if emap is not None:
            em = emap.to(dev).to(torch.int64)
            heldmask = em >= 0
            layer.exl3_maps = []
            for cmap in pack.expert_maps:
                m = torch.full_like(em, -1, dtype=torch.int32)
                m[heldmask] = cmap[em[heldmask]]
                layer.exl3_maps.append(m.contiguous())
        del per
        torch.cuda.empty_cache()
        logger.info("%s: %d experts, bit rates %s, codebook %d", self.prefix, n, sorted(set(pack.bits)), layer.exl3_codebook)
        self._warm(layer, dev)

    @torch.no_grad()
    def _warm(self, layer, dev) -> None:
        """Runs the serving path once per token count an engine warms with, so that the scratch this module owns has its
        final size before any CUDA-graph capture (reference moe.py:202-213)."""
        top_k = getattr(self.moe_runner_config, "top_k", None) or min(8, layer.exl3_num_experts)
        n_global = layer.exl3_maps[0].numel() if layer.exl3_maps else layer.exl3_num_experts
        tokens = max(1, WARM_TOKENS)
        x = torch.zeros((tokens, layer.exl3_hidden), dtype=torch.bfloat16, device=dev)
        ids = ((torch.arange(tokens * top_k, device=dev).view(tokens, top_k) * 37) % n_global).to(torch.int32)
        w = torch.full((tokens, top_k), 1.0 / top_k, dtype=torch.float32, device=dev)
        for t in (tokens, 1):
            self._experts(layer, x[:t], ids[:t].contiguous(), w[:t])
        torch.cuda.synchronize(dev)

    # ---------------------------------------------------------------------------------------------- forward
    def _experts(self, layer, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
        pack = layer.exl3_pack
        tokens = x.shape[0]
        out = torch.empty_like(x)
        if tokens == 0:
            return out
        need = moe_kernels.layer_workspace_bytes([p.num_experts for p in pack.packs], pack.hidden, pack.inter, pack.codebook, tokens,
                                                 topk_ids.shape[1])
        ws = moe_kernels._reserve(x.device, need)
        return moe_kernels.run_layer(x.contiguous(), topk_weights, topk_ids, pack, out, ws, layer.exl3_maps)

    def apply(self, layer, dispatch_output):
        x = dispatch_output.hidden_states
        topk_output = dispatch_output.topk_output
        topk_weights, topk_ids = topk_output.topk_weights, topk_output.topk_ids
        flat = x.reshape(-1, x.shape[-1])
        y = self._experts(layer, flat, topk_ids.reshape(flat.shape[0], -1), topk_weights.reshape(flat.shape[0], -1))
        return StandardCombineInput(hidden_states=y.view_as(x))

    def get_triton_quant_info(self, layer):
        raise NotImplementedError("EXL3 experts do not run on the Triton MoE runner")
