"""`Exl3Config`: which modules of a checkpoint are EXL3, read from the safetensors headers (never from JSON hints).

Interface of the reference's cuda/src/sglang_exl3/sglang_glue/config.py: `get_name`, `from_config`,
`override_quantization_method`, `lookup` with the engine's prefix spellings (:98-117), and `get_quant_method` (:121-144),
which hands an engine layer the method that serves it -- `Exl3LinearMethod` for linears and the LM head,
`Exl3MoEMethod` for the fused experts, the engine's own unquantized method for linears the checkpoint left in 16 bits.
Layers are recognised by the names of their classes, so the same code serves SGLang's layers and test doubles.
"""
from __future__ import annotations

import logging
import os
from typing import Any

import torch

from ..format import load_manifest
from ._engine import QuantizationConfig, class_names

logger = logging.getLogger(__name__)
MODEL_PATH_ENV = "SGLANG_EXL3_MODEL_PATH"

DEFAULT_PACKED = {
    "qkv_proj": ["q_proj", "k_proj", "v_proj"],
    "gate_up_proj": ["gate_proj", "up_proj"],
    "in_proj_qkvz": ["in_proj_qkv", "in_proj_z"],
    "in_proj_ba": ["in_proj_b", "in_proj_a"],
}
_ALIASES = (("model.language_model.", "model."), (".self_attn.", "."))


class Exl3Config(QuantizationConfig):
    """One instance per model load.  `modules` maps a checkpoint module key (e.g. `model.layers.3.self_attn.q_proj`,
    `lm_head`) to (k, n, twice the bitrate, codebook name, has_bias, legacy signs)."""

    def __init__(self, declared: dict[str, Any] | None = None, model_path: str | None = None):
        super().__init__()
        self.declared = {k: v for k, v in (declared or {}).items() if k not in ("hf_config", "packed_modules_mapping")}
        self.model_path = model_path
        self.modules: dict[str, tuple] = {}
        self.warnings: list[str] = []
        if not getattr(self, "packed_modules_mapping", None):
            self.packed_modules_mapping = {}
        if model_path:
            self._scan(model_path)

    # ---- what an engine asks of a quantization config
    def get_name(self) -> str:
        return "exl3"

    def get_supported_act_dtypes(self) -> list[torch.dtype]:
        return [torch.float16, torch.bfloat16]

    @classmethod
    def get_min_capability(cls) -> int:
        return 100                               # these kernels are sm_100a only

    @staticmethod
    def get_config_filenames() -> list[str]:
        return []

    @classmethod
    def from_config(cls, config: dict[str, Any]) -> "Exl3Config":
        hf_config = config.get("hf_config")
        hf_path = getattr(hf_config, "_name_or_path", None)
        path = hf_path if hf_path and os.path.isdir(hf_path) else (os.environ.get(MODEL_PATH_ENV) or hf_path)
        if not path or not os.path.isdir(path):
            raise ValueError(f"EXL3: no local checkpoint directory known for {path!r} (set {MODEL_PATH_ENV})")
        cfg = cls(config, path)
        cfg.packed_modules_mapping = dict(config.get("packed_modules_mapping") or {})
        return cfg

    @classmethod
    def override_quantization_method(cls, hf_quant_cfg, user_quant) -> str | None:
        if isinstance(hf_quant_cfg, dict) and hf_quant_cfg.get("quant_method") == "exl3" and user_quant in (None, "exl3"):
            return "exl3"
        return None

    def get_scaled_act_names(self) -> list[str]:
        return []

    def can_fuse_shared_expert(self) -> bool:    # shared experts stay ordinary EXL3 linears
        return False

    # ---- checkpoint scan
    def _scan(self, model_path: str) -> None:
        man = load_manifest(model_path)
        self.modules = {k: (m.k, m.n, m.bits.twice, m.codebook.value, m.has_bias, m.legacy_signs) for k, m in man.matrices.items()}
        self.warnings = list(man.warnings)
        for w in man.warnings:
            logger.warning("EXL3 checkpoint: %s", w)

    def lookup(self, key: str):
        """The header-scan entry of a module, tolerant of an engine's prefix spellings (`model.` for
        `model.language_model.`, `.self_attn.` dropped or kept, `mtp.` for a draft model's layers)."""
        if key in self.modules:
            return self.modules[key]
        cands = {key}
        for a, b in _ALIASES:
            for c in list(cands):
                cands.add(c.replace(a, b))
                cands.add(c.replace(b, a))
        for c in list(cands):
            if c.startswith("model.layers."):
                cands.add("mtp." + c[len("model."):])
        for c in cands:
            if c in self.modules:
                return self.modules[c]
        return None

    def sources(self, prefix: str) -> list[str]:
        """Checkpoint keys behind an engine module: a fused module (`qkv_proj`, `gate_up_proj`) has several."""
        parent, _, leaf = prefix.rpartition(".")
        packed = (self.packed_modules_mapping or DEFAULT_PACKED).get(leaf) or DEFAULT_PACKED.get(leaf)
        return [f"{parent}.{s}" if parent else s for s in packed] if packed else [prefix]

    def experts_under(self, prefix: str) -> dict[str, tuple]:
        def norm(s: str) -> str:
            for a, b in _ALIASES:
                s = s.replace(a, b)
            return s
        stem = norm(prefix) + "."
        return {k: v for k, v in self.modules.items() if norm(k).startswith(stem) and ".experts." in k}

    def get_quant_method(self, layer: torch.nn.Module, prefix: str):
        from .linear import Exl3LinearMethod
        from .moe import Exl3MoEMethod
        kinds = class_names(layer)
        if "FusedMoE" in kinds:
            experts = self.experts_under(prefix)
            return Exl3MoEMethod(self, prefix, experts) if experts else None
        if "ParallelLMHead" in kinds:
            info = self.lookup(prefix)
            return Exl3LinearMethod(prefix, [info]) if info else None
        if "LinearBase" not in kinds:
            return None
        infos = [self.lookup(p) for p in self.sources(prefix)]
        if not any(infos):
            return self._unquantized()
        if not all(infos):
            raise ValueError(f"{prefix}: fused module mixes EXL3 and unquantized sources {self.sources(prefix)}")
        return Exl3LinearMethod(prefix, infos)

    @staticmethod
    def _unquantized():
        """The engine's own method for linears the checkpoint left unquantized; None without an engine."""
        try:
            from sglang.srt.layers.quantization.unquant import UnquantizedLinearMethod
        except ImportError:
            return None
        return UnquantizedLinearMethod()
