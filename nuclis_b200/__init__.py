"""nuclis_b200: a B200 (sm_100a) backend for nuclis's quantized-weight matmul path.

The product is ``libnuclis_cuda.so`` (CUDA kernels behind the C ABI of
``include/nuclis_cuda.h``). This package is the Python host side: a ctypes
mirror of the engine's ``metal.Backend`` operator interface (``Backend``,
``Buffer``, ``Matrix``), seeded generators of synthetic GGUF blocks, the
GGUF reader, the host-side mirror of the load-time re-layout (``planar``), the
tensor-parallel shard tables and the synthetic decode layer stack.

There is no CPU fallback: importing works anywhere, but creating a
``Backend`` without the built library or without a B200 raises.
"""
from .errors import NuclisError  # noqa: F401
from .backend import Backend, Buffer, Matrix, ExpertMatrix, Segment, SegmentMode, CombineShape  # noqa: F401
from . import encoding  # noqa: F401
