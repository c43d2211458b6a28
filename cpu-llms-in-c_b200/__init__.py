"""Host-side mirror of libq4b200's C ABI (include/q4b200.h) over ctypes.

The product is the shared library; this package only loads it, mirrors the
reference's operator interface for the affine-Q4 path (open / load image
segments / project / wait, with the same status codes and error strings) and
adds the column-parallel multi-GPU layer.  There is no CPU fallback: importing
works anywhere, but every compute entry point needs the CUDA library and a B200.
"""
from __future__ import annotations

from .host import (  # noqa: F401
    BF16, F16, F32, NONE, Q4Context, Q4Error, Q4Graph, Q4Barrier, Q4Comm, Q4Sequence, Q4Weight, DeviceBuffer,
    declared_symbols, library, library_path,
)
from .shapes import (  # noqa: F401
    LAYER_27B, LAYER_SMALL, Projection, algorithmic_bytes, algorithmic_flops,
    layer_bytes, layer_flops,
)
