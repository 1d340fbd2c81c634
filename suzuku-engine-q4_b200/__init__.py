"""B200 device layer for the IQ3_S x 8-bit-activation MoE feed-forward path.

The product is the C-ABI shared library libq4cuda.so (include/q4cuda.h).  This
package loads it (capi), mirrors the engine's host-side MoE call sequence on top
of it (host) and generates seeded synthetic inputs (synth).  The directory name
is not an importable identifier; load it with `__graft_entry__.load_package()`
or importlib under the module name `suzuku_engine_q4_b200`.
"""
from . import capi, synth  # noqa: F401
from .host import Device, MoeLayer  # noqa: F401
