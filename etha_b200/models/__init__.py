"""Weight-shape catalogs of the model families used by the benchmarks and examples."""

from .catalog import (
    LayoutRule,
    ModelSpec,
    TensorSpec,
    fsdp_layout,
    llama3_8b,
    mixtral_8x7b,
    qwen2_7b,
    qwen3_0p6b,
    tiny_llama,
    vllm_tp_layout,
)

__all__ = [
    "ModelSpec", "TensorSpec", "LayoutRule", "llama3_8b", "qwen2_7b", "mixtral_8x7b", "qwen3_0p6b", "tiny_llama",
    "fsdp_layout", "vllm_tp_layout",
]


def __getattr__(name):
    # helpers that load the CUDA library or spawn agents are imported on first use
    if name == "WeightSync":
        from .sync import WeightSync

        return WeightSync
    if name in ("bus_roundtrip", "BusItem"):
        from . import bus_sync

        return getattr(bus_sync, name)
    raise AttributeError(name)
