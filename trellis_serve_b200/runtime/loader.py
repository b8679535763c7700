"""Checkpoint -> resident groups: the load path on the caller's side of `kernels.linear.prepare`.

What an engine's weight loader does for the reference plugin (cuda/src/sglang_exl3/sglang_glue/linear.py:61-63 legacy sign
unpacking, :107-183 `process_weights_after_loading`: checks against the header scan, codebook from the marker tensors,
fused groups in checkpoint order, true output widths), without the engine: the manifest (headers only) says which
keys are EXL3 linears, the tensors of the requested keys are read from their safetensors shards, legacy packed signs are
expanded, the group is checked and handed to `prepare`, and the result runs through the `linear` operator.

    group = load_group(model_dir, ["model.layers.0.self_attn.q_proj", "...k_proj", "...v_proj"])
    y = group.forward(x)                     # [..., sum(out_widths)]
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import torch

from ..format import FormatError, Manifest, MatrixSpec, load_manifest
from ..kernels import linear as lin

CODEBOOK_ID = {"3inst": 0, "mcg": 1, "mul1": 2}          # numbering of core/src/trellis_core/reference.py:27


def unpack_signs(packed: torch.Tensor) -> torch.Tensor:
    """Legacy `su` / `sv`: int16 [w / 16], bit b of word i is the sign of element 16 * i + b (1 = negative) -> fp16 [w]
    of +-1 (sglang_glue/linear.py:61-63)."""
    if packed.dtype != torch.int16 or packed.dim() != 1:
        raise FormatError(f"packed signs must be 1-D int16, got {packed.dtype} {tuple(packed.shape)}")
    bits = (packed.to(torch.int32).unsqueeze(1) >> torch.arange(16, device=packed.device)) & 1
    return (1.0 - 2.0 * bits.flatten().to(torch.float32)).to(torch.float16)


def read_tensors(model_dir, spec: MatrixSpec) -> dict:
    """The stored tensors of one EXL3 linear, by suffix, on the CPU, from the shard files its header entries name."""
    from safetensors import safe_open
    by_file: dict[str, list[str]] = {}
    for suffix, info in spec.tensors.items():
        by_file.setdefault(info.file, []).append(suffix)
    out = {}
    for file, suffixes in by_file.items():
        with safe_open(os.path.join(os.fspath(model_dir), file), framework="pt", device="cpu") as f:
            for suffix in suffixes:
                out[suffix] = f.get_tensor(f"{spec.key}.{suffix}")
    return out


@dataclass
class LinearGroup:
    """One fused group in the resident layout, ready for the `linear` operator."""
    keys: list[str]
    packed: torch.Tensor
    suh_cat: torch.Tensor
    svh_cat: torch.Tensor
    ends: list[int]
    codebook: int
    out_widths: list[int]
    k: int
    bias: torch.Tensor | None = None
    specs: list[MatrixSpec] = field(default_factory=list)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from . import ops
        y = ops.linear(x, [], [], [], [], [], 0, [self.packed, self.suh_cat, self.svh_cat], self.ends, [self.codebook], self.out_widths)
        return y if self.bias is None else y + self.bias.to(y.dtype)


def group_from_tensors(specs: list[MatrixSpec], tensors: list[dict], device, out_widths: list[int] | None = None) -> LinearGroup:
    """`tensors[i]` = stored tensors of `specs[i]` by suffix (CPU or device).  Matrices of a group share the input
    width, the bitrate and the codebook; `out_widths` are the true output widths (stored widths are 128-padded)."""
    if not specs:
        raise FormatError("an empty group")
    dev = torch.device(device)
    first = specs[0]
    for s in specs[1:]:
        if (s.k, s.bits, s.codebook) != (first.k, first.bits, first.codebook):
            raise FormatError(f"{s.key} cannot be fused with {first.key}: input width, bitrate and codebook must agree "
                              f"({s.k}, K={s.bits}, {s.codebook.value} against {first.k}, K={first.bits}, {first.codebook.value})")
    if first.bits.is_half:
        raise FormatError(f"{first.key}: half-integer K={first.bits} is not served by these kernels")
    trellis, suh, svh, bias = [], [], [], []
    for spec, got in zip(specs, tensors):
        tr = got["trellis"].to(dev).contiguous()
        if (tr.shape[0] * 16, tr.shape[1] * 16, tr.shape[2]) != (spec.k, spec.n, spec.bits.trellis_words):
            raise FormatError(f"{spec.key}: trellis {tuple(tr.shape)} does not match the header scan")
        if spec.legacy_signs:
            su, sv = unpack_signs(got["su"].to(dev)), unpack_signs(got["sv"].to(dev))
        else:
            su, sv = got["suh"].to(dev), got["svh"].to(dev)
        if su.shape != (spec.k,) or sv.shape != (spec.n,):
            raise FormatError(f"{spec.key}: scale vectors {tuple(su.shape)}, {tuple(sv.shape)} do not match ({spec.k},), ({spec.n},)")
        trellis.append(tr)
        suh.append(su.to(torch.float16).contiguous())
        svh.append(sv.to(torch.float16).contiguous())
        bias.append(got["bias"].to(dev) if spec.has_bias else None)
    widths = list(out_widths) if out_widths is not None else [s.n for s in specs]
    if len(widths) != len(specs) or any(w < 1 or w > s.n for w, s in zip(widths, specs)):
        raise FormatError(f"out_widths {widths} do not fit the stored widths {[s.n for s in specs]}")
    codebook = CODEBOOK_ID[first.codebook.value]
    ok, why = lin.supports(trellis, [s.n for s in specs], [codebook] * len(specs))      # true widths are trimmed by the operator
    if not ok:
        raise FormatError(f"{first.key}: {why}")
    packed, suh_cat, svh_cat, ends = lin.prepare(trellis, suh, svh)
    b = None
    if any(x is not None for x in bias):
        b = torch.cat([(bi[:w] if bi is not None else torch.zeros(w, device=dev)).to(torch.float32) for bi, w in zip(bias, widths)])
    return LinearGroup([s.key for s in specs], packed, suh_cat, svh_cat, ends, codebook, widths, first.k, b, list(specs))


def load_group(model_dir, keys: list[str], device="cuda", manifest: Manifest | None = None,
               out_widths: list[int] | None = None) -> LinearGroup:
    """Reads the EXL3 linears `keys` (fused in that order) of a local checkpoint directory and prepares them."""
    man = manifest if manifest is not None else load_manifest(model_dir)
    missing = [k for k in keys if k not in man.matrices]
    if missing:
        raise FormatError(f"{os.fspath(model_dir)}: not EXL3 linears: {missing}")
    specs = [man.matrices[k] for k in keys]
    return group_from_tensors(specs, [read_tensors(model_dir, s) for s in specs], device, out_widths)
