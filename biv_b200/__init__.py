"""bivmoe for B200: the qwen35moe MoE feed-forward layer of the biv inference
engine as sm_100a CUDA behind a C ABI (``include/bivmoe.h``), with this thin
Python host layer over it."""
from . import workloads  # noqa: F401

__all__ = ["workloads", "Moe", "MoeStack"]


def __getattr__(name):
    if name in ("Moe", "MoeStack", "launch_count"):
        from . import moe
        return getattr(moe, name)
    raise AttributeError(name)
