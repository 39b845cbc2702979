"""adaptq_b200 -- the AdapTQ quantized KV-cache append / decode-attention path on
NVIDIA B200 (sm_100a), behind upstream's own interfaces:

* the C ABI of include/adaptq.h (+ batched additions in include/adaptq_b200.h),
  implemented by ``libadaptq_b200.so``;
* ``MHAContext`` (upstream's pybind class ``adaptq_py.MHAContext``);
* ``Engine`` (upstream ``adaptq.Engine``), ``AdaptQAttention`` and its
  many-sequence form ``BatchedAdaptQAttention``; ``LayerStack`` (all layers of a
  model behind one handle);
* ``adaptq_b200.runtime`` (upstream's second stack: ``RuntimeContext``, AQSS v2
  snapshots, ``IKernelBackend``) and ``adaptq_b200.hf_cache`` (Hugging Face
  ``DynamicCache`` + fused attention function).
"""
from ._lib import LIB_PATH, last_error, load  # noqa: F401
from .core import Engine  # noqa: F401
from .mha import MHAContext  # noqa: F401
from .stack import LayerStack  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("AdaptQAttention", "BatchedAdaptQAttention"):  # lazy: importing torch is slow
        from . import torch_adapter
        return getattr(torch_adapter, name)
    raise AttributeError(name)
