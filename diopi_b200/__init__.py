"""diopi_b200: a B200-native DIOPI backend for the LLM-inference hot path.

The product is ``lib/libdiopi_impl.so`` (C ABI declared in ``include/diopi_b200.h``). This
package adds what is needed to drive it from Python: the build recipe, a small consumer-side
run time, and call forms named after the reference's own Python wrappers.
"""
from . import functions, runtime  # noqa: F401
from ._lib import load  # noqa: F401

__all__ = ["functions", "runtime", "load"]
