"""fxpr_vllm for B200: the reference plugin's operator surface (``torch.ops.fxpr.*``,
the ``fixedpoint`` quantization config, the ``CUSTOM`` attention backend,
``DeterministicRMSNorm``) on hand-written sm_100a CUDA kernels behind a C ABI.

Importing the package defines the ``fxpr`` op library and its fake impls, as
``fxpr_vllm/__init__.py:1-2`` of the reference does.
"""
from . import _lib  # noqa: F401
from . import library_ops  # noqa: F401
