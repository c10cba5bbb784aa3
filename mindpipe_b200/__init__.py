"""mindpipe_b200: B200 (sm_100a) kernels for MindPipe's quantized-linear forward.

The package keeps the reference's module/operator interface for that path
(real-quant twins of its Linear modules) and runs it on hand-written CUDA
kernels behind a C ABI (``include/mindpipe_b200.h``).  There is no CPU or
eager fallback: importing is cheap, the first kernel call loads the shared
library and raises if it is missing.
"""
from . import synth  # noqa: F401

__all__ = ["synth", "ops", "modules", "install", "build"]
__version__ = "0.1.0"


def __getattr__(name):
    if name in ("ops", "modules", "install", "build", "_lib"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
