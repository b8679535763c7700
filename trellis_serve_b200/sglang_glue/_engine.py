"""The few names the glue needs from SGLang, or stand-ins with the same surface when SGLang is not installed."""
from __future__ import annotations

from dataclasses import dataclass

try:                                                            # SGLang 0.5.x module paths
    from sglang.srt.layers.quantization.base_config import FusedMoEMethodBase, LinearMethodBase, QuantizationConfig
    from sglang.srt.utils.common import set_weight_attrs
    try:
        from sglang.srt.layers.moe.token_dispatcher.standard import StandardCombineInput
    except ImportError:                                         # pragma: no cover
        StandardCombineInput = None
    ENGINE_AVAILABLE = True
except ImportError:
    ENGINE_AVAILABLE = False

    class QuantizationConfig:                                   # noqa: D401
        """Stand-in: what an engine's quantization config base class provides to subclasses here."""

        def __init__(self):
            self.packed_modules_mapping = {}

    class LinearMethodBase:
        """Stand-in: create_weights / process_weights_after_loading / apply are defined by the subclass."""

    class FusedMoEMethodBase:
        """Stand-in: create_weights / create_moe_runner / process_weights_after_loading / apply by the subclass."""

    def set_weight_attrs(param, attrs: dict) -> None:
        for name, value in attrs.items():
            setattr(param, name, value)

    StandardCombineInput = None

if StandardCombineInput is None:
    @dataclass
    class StandardCombineInput:                                 # type: ignore[no-redef]
        hidden_states: object


def class_names(obj) -> set[str]:
    """Names of every class in the object's ancestry: layer kinds are recognised by name, so that the glue can be driven by
    an engine's real layers and by test doubles alike."""
    return {c.__name__ for c in type(obj).__mro__}
