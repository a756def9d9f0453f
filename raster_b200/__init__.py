"""raster_b200 -- Blackwell (sm_100a) quantized matmul behind Raster's operator API.

The compute lives in ``lib/librstq.so`` (CUDA, built from ``csrc/`` by
``python -m raster_b200.build``) behind the C ABI of ``include/rstq.h``; the
``quant`` subpackage mirrors the reference's Clojure namespaces one to one.
"""
from . import _lib  # noqa: F401
from .runtime import Context, DeviceBuffer, QWeight, default_context  # noqa: F401

__all__ = ["Context", "DeviceBuffer", "QWeight", "default_context"]
