"""cavs_b200: B200-native level-batched vertex-function execution (forward and backward)
behind the reference's graph-op / OpImpl / GraphSupport interface.

The Python layer only binds the C ABI (include/cavs_b200.h) for tests and the benchmark;
the product is the shared library built from cavs_b200/csrc."""
from ._abi import CavsError, check, declared_symbols, lib  # noqa: F401
from . import schedule  # noqa: F401
