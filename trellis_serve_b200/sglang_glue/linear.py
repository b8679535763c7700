"""`Exl3LinearMethod`: EXL3 storage and forward for an engine's linear layers and LM head.

Interface and loader semantics of the reference's cuda/src/sglang_exl3/sglang_glue/linear.py (create_weights :72,
process_weights_after_loading :107, apply :185): every source matrix of a fused module (q, k, v / gate, up) keeps its own
trellis, suh and svh; placeholders named like the checkpoint suffixes are registered so that the model's own
`load_weights` hands `<layer>.<suffix>` (+ shard id) to this loader, which keeps whole tensors per shard id; after
loading the group is checked against the header scan, brought into the resident layout and the stored copies dropped.

Beyond the reference: a layer that is a tensor-parallel shard (the layer says so through `tp_rank` / `tp_size`, or the
partition sizes passed to create_weights are smaller than the full sizes) takes its 128-aligned slice of every source
matrix by the format layer's rules (column slices: trellis dim 1 and svh; row slices: trellis dim 0 and suh).  The sum
over the ranks of a row-parallel layer is the engine's business (its RowParallelLinear reduces), as with any quantization.
"""
from __future__ import annotations

import logging

import torch

from ..format import FormatError, TensorInfo, build_matrix_spec, column_slice, row_slice
from ..runtime import loader
from ._engine import LinearMethodBase, set_weight_attrs

logger = logging.getLogger(__name__)
SUFFIXES = ("trellis", "suh", "svh", "su", "sv", "mcg", "mul1")
_QKV = {"q": 0, "k": 1, "v": 2}


def _partitions(shard_id) -> tuple[int, ...]:
    """Output partitions of the fused layer a checkpoint shard covers: none (whole layer), one, or a tuple of them."""
    if shard_id is None:
        return ()
    if isinstance(shard_id, (tuple, list)):
        return tuple(_QKV.get(s, s) for s in shard_id)
    return (_QKV.get(shard_id, shard_id),)


class Exl3LinearMethod(LinearMethodBase):
    """`infos`: per source matrix in checkpoint order, (k, n, twice the bitrate, codebook name, has_bias, legacy signs) from
    the header scan (`Exl3Config.modules`)."""

    def __init__(self, prefix: str, infos: list[tuple]):
        self.prefix = prefix
        self.infos = list(infos)

    # ---------------------------------------------------------------------------------------------- weights
    def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size, params_dtype,
                       **extra_weight_attrs):
        tp_size = int(getattr(layer, "tp_size", 1) or 1)
        tp_rank = int(getattr(layer, "tp_rank", 0) or 0)
        row_parallel = input_size_per_partition != input_size
        col_parallel = sum(output_partition_sizes) != output_size
        if (row_parallel or col_parallel) and tp_size == 1:
            raise NotImplementedError(f"{self.prefix}: partition sizes {input_size_per_partition}/{sum(output_partition_sizes)} of "
                                      f"{input_size}/{output_size} need the layer's tp_rank and tp_size")
        if row_parallel and col_parallel:
            raise NotImplementedError(f"{self.prefix}: a layer split along both dimensions is not supported")
        layer.exl3_out_sizes = list(output_partition_sizes)
        layer.exl3_in_size = input_size_per_partition
        layer.exl3_tp = (tp_rank, tp_size, "row" if row_parallel else "column" if col_parallel else "none")
        layer.exl3_shards = {s: {} for s in SUFFIXES}
        for suffix in SUFFIXES:
            p = torch.nn.Parameter(torch.empty(0, dtype=torch.uint8), requires_grad=False)
            set_weight_attrs(p, {"weight_loader": self._make_loader(layer, suffix), "exl3_placeholder": True})
            layer.register_parameter(suffix, p)
        if not hasattr(layer, "weight"):
            # An LM head is asked for `.weight` by the engine (embedding tying, hot-token slicing): a zero-width stand-in
            # with one row per output keeps those code paths alive (reference linear.py:86-93).
            w = torch.nn.Parameter(torch.empty((sum(output_partition_sizes), 0), dtype=params_dtype), requires_grad=False)
            set_weight_attrs(w, {"weight_loader": self._ignore_dense, "exl3_placeholder": True})
            layer.register_parameter("weight", w)

    @staticmethod
    def _ignore_dense(param, loaded_weight, *args, **kwargs):
        logger.warning("EXL3: ignoring a dense .weight delivered to a quantized layer (shape %s)", tuple(loaded_weight.shape))

    def _make_loader(self, layer, suffix: str):
        def load(param, loaded_weight, loaded_shard_id=None, *args, **kwargs):
            store = layer.exl3_shards[suffix]
            key = tuple(loaded_shard_id) if isinstance(loaded_shard_id, list) else loaded_shard_id
            if key in store:
                raise ValueError(f"{self.prefix}.{suffix}: shard {key!r} loaded twice")
            store[key] = loaded_weight.detach().clone()              # whole tensor; sliced and moved once the group is complete
        return load

    def process_weights_after_loading(self, layer) -> None:
        got = layer.exl3_shards
        ids = sorted(got["trellis"], key=lambda sid: _partitions(sid) or (0,))
        if not ids:
            # e.g. a draft model's own LM head that the target's replaces: nothing was ever delivered (reference :110-114)
            logger.warning("%s: no EXL3 tensors were delivered; layer left empty", self.prefix)
            layer.exl3_group = None
            return
        if len(ids) != len(self.infos):
            raise ValueError(f"{self.prefix}: expected {len(self.infos)} EXL3 matrices, checkpoint delivered {len(ids)} ({ids})")
        tp_rank, tp_size, mode = layer.exl3_tp
        specs, tensors, widths = [], [], []
        for i, sid in enumerate(ids):
            mat = {s: got[s][sid] for s in SUFFIXES if sid in got[s]}
            if "suh" not in mat and "su" not in mat:
                raise ValueError(f"{self.prefix}: shard {sid!r} has a trellis but no scale vectors")
            info = {s: TensorInfo(f"{self.prefix}[{i}].{s}", _dtype_tag(t), tuple(t.shape)) for s, t in mat.items()}
            spec = build_matrix_spec(f"{self.prefix}[{i}]", info)
            k, n, twice, declared = self.infos[i][:4]
            if (spec.k, spec.n, spec.bits.twice, spec.codebook.value) != (k, n, twice, declared):
                raise ValueError(f"{self.prefix}: shard {sid!r} {tuple(mat['trellis'].shape)}/{spec.codebook.value} does not match "
                                 f"the header scan {(k, n, twice, declared)}")
            parts = _partitions(sid)
            width = sum(layer.exl3_out_sizes[p] for p in parts) if parts else sum(layer.exl3_out_sizes)
            if mode != "none":
                spec, mat = _tp_slice(spec, mat, mode, tp_rank, tp_size)
            specs.append(spec)
            tensors.append(mat)
            widths.append(width)
        if sum(widths) != sum(layer.exl3_out_sizes):
            raise ValueError(f"{self.prefix}: shards cover {sum(widths)} of {sum(layer.exl3_out_sizes)} output columns")
        dev = torch.device("cuda", torch.cuda.current_device())
        try:
            group = loader.group_from_tensors(specs, tensors, dev, out_widths=widths)
        except FormatError as e:
            raise ValueError(f"{self.prefix}: {e}") from e
        for suffix in SUFFIXES:
            delattr(layer, suffix)
        del layer.exl3_shards
        for name, t in (("packed", group.packed), ("suh", group.suh_cat), ("svh", group.svh_cat)):
            layer.register_buffer(f"exl3_{name}", t, persistent=False)
        group.packed, group.suh_cat, group.svh_cat = layer.exl3_packed, layer.exl3_suh, layer.exl3_svh
        layer.exl3_group = group
        layer.exl3_count, layer.exl3_codebooks, layer.exl3_widths = len(ids), [group.codebook] * len(ids), widths

    # ---------------------------------------------------------------------------------------------- forward
    def apply(self, layer, x: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        group = getattr(layer, "exl3_group", None)
        if group is None:
            raise RuntimeError(f"{self.prefix}: EXL3 layer has no weights (never loaded)")
        from ..runtime import ops
        y = ops.linear(x, [], [], [], [], [], 0, [layer.exl3_packed, layer.exl3_suh, layer.exl3_svh], group.ends,
                       layer.exl3_codebooks, layer.exl3_widths)
        return y if bias is None else y + bias


_DTYPE_TAGS = {torch.int16: "I16", torch.float16: "F16", torch.int32: "I32", torch.float32: "F32", torch.bfloat16: "BF16"}


def _dtype_tag(t: torch.Tensor) -> str:
    return _DTYPE_TAGS.get(t.dtype, str(t.dtype))


def _tp_slice(spec, mat: dict, mode: str, rank: int, size: int):
    """This rank's 128-aligned share of one source matrix and the spec that describes it."""
    if mode == "column":
        if spec.n % size or (spec.n // size) % 128:
            raise ValueError(f"{spec.key}: {spec.n} output columns cannot be split over {size} ranks at 128-aligned boundaries")
        sl = column_slice(spec, rank * (spec.n // size), spec.n // size)
    else:
        if spec.k % size or (spec.k // size) % 128:
            raise ValueError(f"{spec.key}: {spec.k} input rows cannot be split over {size} ranks at 128-aligned boundaries")
        sl = row_slice(spec, rank * (spec.k // size), spec.k // size)

    def cut(t, nr):
        if t is None or nr is None:
            return t
        index = [slice(None)] * nr.dim + [slice(nr.start, nr.start + nr.length)]
        return t[tuple(index)].contiguous()
    out = dict(mat)
    out["trellis"] = cut(mat["trellis"], sl.trellis)
    if "suh" in mat:
        out["suh"], out["svh"] = cut(mat["suh"], sl.suh), cut(mat["svh"], sl.svh)
    else:                                                        # legacy packed signs: expand, then slice
        out.pop("su"), out.pop("sv")
        out["suh"], out["svh"] = cut(loader.unpack_signs(mat["su"]), sl.suh), cut(loader.unpack_signs(mat["sv"]), sl.svh)
    info = {s: TensorInfo(f"{spec.key}.{s}", _dtype_tag(t), tuple(t.shape)) for s, t in out.items()}
    return build_matrix_spec(spec.key, info), out
