"""B200-native paged decode attention and fused RoPE + paged-KV write.

A from-scratch sm_100a implementation of one path of the Loom Kernels project,
behind that project's own C ABIs. ``attnarc_b200.ops`` is the PyTorch-facing
API; ``attnarc_b200.multi_gpu`` shards the work over the GPUs of one node;
``python -m attnarc_b200.build`` compiles the native library.
"""

from ._native import LIBRARY_PATH, BridgeError, NativeLibraryMissing

__all__ = ["LIBRARY_PATH", "BridgeError", "NativeLibraryMissing", "ops"]


def __getattr__(name):
    # torch is imported only when the operators are asked for.
    if name in ("ops", "multi_gpu"):
        import importlib

        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
