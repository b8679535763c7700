"""EXL3 on-disk format, checkpoint manifest and shard geometry.  Pure Python: no torch.
Same public names as the reference's core/src/trellis_core/format package."""
from .geometry import MatrixSlice, Narrow, SplitError, admissible_tp_degrees, ceil_block, column_slice, even_shard, kv_shard_index, row_slice
from .layout import FusedLayout, FusionKind, LogicalMatrix, make_layout
from .manifest import Manifest, build_manifest, load_manifest
from .spec import BitsK, Codebook, FormatError, MatrixSpec, TensorInfo, build_matrix_spec

__all__ = ["BitsK", "Codebook", "FormatError", "FusedLayout", "FusionKind", "LogicalMatrix", "Manifest", "MatrixSlice",
           "MatrixSpec", "Narrow", "SplitError", "TensorInfo", "admissible_tp_degrees", "build_manifest", "build_matrix_spec",
           "ceil_block", "column_slice", "even_shard", "kv_shard_index", "load_manifest", "make_layout", "row_slice"]
