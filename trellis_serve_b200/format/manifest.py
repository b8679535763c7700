"""Checkpoint manifest built from safetensors headers only: which module keys are EXL3 linears, at which K and
codebook, and what is left unquantized.  Tensor headers are the truth; quantization_config is cross-checked and
reported as warnings.  API of core/src/trellis_core/format/manifest.py of 0xSero/trellis-serve.
"""
from __future__ import annotations

import glob
import json
import os
from collections import Counter
from dataclasses import dataclass, field

from .safetensors_header import ShardHeader, read_header
from .spec import INPUT_SCALE, OUTPUT_SCALE, REQUIRED_TRELLIS, FormatError, MatrixSpec, TensorInfo, build_matrix_spec

NGRAM_FORMAT = "exl3_ngram_trellis"


@dataclass(frozen=True)
class NgramTable:
    file: str
    metadata: dict
    tensors: dict

    @property
    def nbytes(self) -> int:
        return sum(t.nbytes for t in self.tensors.values())


@dataclass
class Manifest:
    matrices: dict = field(default_factory=dict)
    unquantized: dict = field(default_factory=dict)
    ngram_tables: list = field(default_factory=list)
    quant_config: dict = field(default_factory=dict)
    warnings: list = field(default_factory=list)

    def is_quantized(self, key: str) -> bool:
        return key in self.matrices

    def children(self, prefix: str) -> dict:
        stem = prefix.rstrip(".") + "."
        return {k: m for k, m in self.matrices.items() if k.startswith(stem)}

    def summary(self) -> dict:
        classes = Counter((str(m.bits), m.codebook.value) for m in self.matrices.values())
        declared_keys = ("version", "bits", "head_bits", "mtp_bits", "vision_bits", "codebook", "out_scales")
        return {
            "quantized_linears": len(self.matrices),
            "quantized_bytes": sum(m.nbytes for m in self.matrices.values()),
            "unquantized_tensors": len(self.unquantized),
            "unquantized_bytes": sum(t.nbytes for t in self.unquantized.values()),
            "ngram_tables": len(self.ngram_tables),
            "ngram_bytes": sum(t.nbytes for t in self.ngram_tables),
            "by_bits_codebook": {f"K={k} {cb}": c for (k, cb), c in sorted(classes.items())},
            "legacy_sign_linears": sum(m.legacy_signs for m in self.matrices.values()),
            "biased_linears": sum(m.has_bias for m in self.matrices.values()),
            "declared": {k: self.quant_config[k] for k in declared_keys if k in self.quant_config},
            "warnings": list(self.warnings),
        }


def _parents(key: str):
    while "." in key:
        key = key.rsplit(".", 1)[0]
        yield key


def build_manifest(headers: list, quant_config: dict | None = None, weight_map: dict | None = None) -> Manifest:
    """`weight_map` (model.safetensors.index.json) decides which copy is live when a tensor is stored in two shards."""
    man = Manifest(quant_config=dict(quant_config or {}))
    weight_map = weight_map or {}
    live: dict[str, TensorInfo] = {}
    twice = []
    for h in headers:
        if h.metadata.get("format") == NGRAM_FORMAT:
            man.ngram_tables.append(NgramTable(h.file, h.metadata, h.tensors))
            continue
        for name, info in h.tensors.items():
            if name in live:
                owner = weight_map.get(name)
                if owner not in (live[name].file, h.file):
                    raise FormatError(f"tensor {name} appears in both {live[name].file} and {h.file} "
                                      f"and the index does not say which one is live")
                twice.append(name)
                if owner != h.file:
                    continue
            live[name] = info
    if twice:
        man.warnings.append(f"{len(twice)} tensors are stored in more than one shard (index decides), e.g. {twice[0]}")

    suffix = "." + REQUIRED_TRELLIS
    keys = {name[: -len(suffix)] for name in live if name.endswith(suffix)}
    for key in keys:
        outer = next((k for k in _parents(key) if k in keys), None)
        if outer is not None:
            raise FormatError(f"{key}.trellis: unexpected tensor nested under EXL3 linear {outer}")
    groups: dict[str, dict[str, TensorInfo]] = {}
    for name, info in live.items():
        key, _, tail = name.rpartition(".")
        if key in keys:
            groups.setdefault(key, {})[tail] = info
            continue
        outer = next((k for k in _parents(key) if k in keys), None)
        if outer is not None:
            raise FormatError(f"{name}: unexpected tensor nested under EXL3 linear {outer}")
        man.unquantized[name] = info
    for key in sorted(groups):
        man.matrices[key] = build_matrix_spec(key, groups[key])

    declared = man.quant_config.get("codebook")
    if declared and man.matrices:
        used = {m.codebook.value for m in man.matrices.values()}
        if used != {declared}:
            man.warnings.append(f"quantization_config.codebook={declared!r} but tensors use {sorted(used)}")
    scale_names = INPUT_SCALE + OUTPUT_SCALE
    stray = [n for n in man.unquantized if n.rpartition(".")[2] in scale_names and n.rpartition(".")[0] not in man.matrices]
    if stray:
        man.warnings.append(f"{len(stray)} scale tensors without a trellis, e.g. {stray[0]}")
    return man


def _quant_config(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        cfg = json.load(f)
    qc = cfg.get("quantization_config") or (cfg.get("text_config") or {}).get("quantization_config") or {}
    if qc and qc.get("quant_method") != "exl3":
        raise FormatError(f"{model_dir}: quant_method is {qc.get('quant_method')!r}, not 'exl3'")
    return qc


def load_manifest(model_dir) -> Manifest:
    """Manifest of a local checkpoint directory; reads headers only."""
    model_dir = os.fspath(model_dir)
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FormatError(f"{model_dir}: no .safetensors files")
    headers = [read_header(f) for f in files]
    weight_map = {}
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            weight_map = json.load(f).get("weight_map", {})
    man = build_manifest(headers, _quant_config(model_dir), weight_map)
    if weight_map:
        have = {n for h in headers if h.metadata.get("format") != NGRAM_FORMAT for n in h.tensors}
        missing = sorted(set(weight_map) - have)
        if missing:
            raise FormatError(f"{len(missing)} tensors listed in the index are in no shard, e.g. {missing[0]}")
        extra = sorted(have - set(weight_map))
        if extra:
            man.warnings.append(f"{len(extra)} tensors are not in model.safetensors.index.json, e.g. {extra[0]}")
    return man
