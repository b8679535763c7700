"""Engine glue: the quantization method SGLang asks for when it meets an EXL3 checkpoint.

Mirrors the interface of the reference plugin's `sglang_glue` package (cuda/src/sglang_exl3/sglang_glue/ of
0xSero/trellis-serve): `Exl3Config` (config.py there), `Exl3LinearMethod` (linear.py), `Exl3MoEMethod` (moe.py), with the
same method names, loader semantics and refusals, over this library's kernels.  SGLang itself is optional: when it cannot be
imported the classes derive from small stand-ins with the same constructor-free base-class surface, so everything here
loads, and is tested, without an engine.  What this glue adds to the reference's: tensor-parallel layers (the reference
refuses them, linear.py:74-75) are sliced by the exact rules of the format layer, and experts of mixed bit rate in one
layer are served.
"""
from ._engine import ENGINE_AVAILABLE
from .config import Exl3Config
from .linear import Exl3LinearMethod
from .moe import Exl3MoEMethod

__all__ = ["ENGINE_AVAILABLE", "Exl3Config", "Exl3LinearMethod", "Exl3MoEMethod"]
