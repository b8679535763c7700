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


def _ancestors(key: str):
    """'a.b.c' -> 'a.b', 'a'."""
    parts = key.split(".")
    for end in range(len(parts) - 1, 0, -1):
        yield ".".join(parts[:end])


def _live_tensors(headers: list, weight_map: dict, man: Manifest) -> dict:
    """name -> TensorInfo over all model shards.  A name stored in two shards is an error unless the index names the shard
    that counts; n-gram side tables are set aside into `man.ngram_tables`."""
    live: dict[str, TensorInfo] = {}
    duplicated = []
    for header in headers:
        if header.metadata.get("format") == NGRAM_FORMAT:
            man.ngram_tables.append(NgramTable(header.file, header.metadata, header.tensors))
            continue
        for name, info in header.tensors.items():
            seen = live.get(name)
            if seen is None:
                live[name] = info
                continue
            owner = weight_map.get(name)
            if owner != seen.file and owner != header.file:
                raise FormatError(f"tensor {name} appears in both {seen.file} and {header.file} "
                                  f"and the index does not say which one is live")
            duplicated.append(name)
            if owner == header.file:
                live[name] = info
    if duplicated:
        man.warnings.append(f"{len(duplicated)} tensors are stored in more than one shard (index decides), e.g. {duplicated[0]}")
    return live


def build_manifest(headers: list, quant_config: dict | None = None, weight_map: dict | None = None) -> Manifest:
    """Sorts the tensors of all shards into EXL3 linears (every key that has a `.trellis`) and the rest.  `weight_map`
    (the `weight_map` of model.safetensors.index.json) decides between copies of a tensor stored twice."""
    man = Manifest(quant_config=dict(quant_config or {}))
    live = _live_tensors(headers, weight_map or {}, man)

    tail = "." + REQUIRED_TRELLIS
    linear_keys = {name[:-len(tail)] for name in live if name.endswith(tail)}

    def enclosing_linear(key: str):
        return next((a for a in _ancestors(key) if a in linear_keys), None)

    by_key: dict[str, dict[str, TensorInfo]] = {key: {} for key in linear_keys}
    for name, info in live.items():
        owner, _, suffix = name.rpartition(".")
        outer = enclosing_linear(owner)
        if outer is not None:                     # something below a linear that is not one of its own tensors
            what = f"{name}: unexpected tensor" if owner not in linear_keys else f"{owner}.trellis: unexpected tensor"
            raise FormatError(f"{what} nested under EXL3 linear {outer}")
        if owner in linear_keys:
            by_key[owner][suffix] = info
        else:
            man.unquantized[name] = info
    for key in sorted(by_key):
        man.matrices[key] = build_matrix_spec(key, by_key[key])

    declared = man.quant_config.get("codebook")
    stored = {spec.codebook.value for spec in man.matrices.values()}
    if declared and stored and stored != {declared}:
        man.warnings.append(f"quantization_config.codebook={declared!r} but tensors use {sorted(stored)}")
    orphans = [name for name in man.unquantized if name.rpartition(".")[2] in INPUT_SCALE + OUTPUT_SCALE]
    if orphans:
        man.warnings.append(f"{len(orphans)} scale tensors without a trellis, e.g. {orphans[0]}")
    return man


def _quant_config(model_dir: str) -> dict:
    """quantization_config of config.json (also looked for under text_config); {} when there is none."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        config = json.load(f)
    found = config.get("quantization_config") or (config.get("text_config") or {}).get("quantization_config") or {}
    method = found.get("quant_method") if found else None
    if found and method != "exl3":
        raise FormatError(f"{model_dir}: quant_method is {method!r}, not 'exl3'")
    return found


def load_manifest(model_dir) -> Manifest:
    """Manifest of a local checkpoint directory, from the headers of its *.safetensors files only."""
    model_dir = os.fspath(model_dir)
    shard_paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not shard_paths:
        raise FormatError(f"{model_dir}: no .safetensors files")
    headers = [read_header(path) for path in shard_paths]
    index_path = os.path.join(model_dir, "model.safetensors.index.json")
    weight_map = {}
    if os.path.exists(index_path):
        with open(index_path) as f:
            weight_map = json.load(f).get("weight_map", {})
    man = build_manifest(headers, _quant_config(model_dir), weight_map)
    if weight_map:
        stored = set()
        for header in headers:
            if header.metadata.get("format") != NGRAM_FORMAT:
                stored.update(header.tensors)
        absent = sorted(set(weight_map) - stored)
        if absent:
            raise FormatError(f"{len(absent)} tensors listed in the index are in no shard, e.g. {absent[0]}")
        unlisted = sorted(stored - set(weight_map))
        if unlisted:
            man.warnings.append(f"{len(unlisted)} tensors are not in model.safetensors.index.json, e.g. {unlisted[0]}")
    return man
