"""dali_b200: B200-native back end for Dali's lazy expression-fusion path.

The product is the C-ABI shared library (include/dali_b200.h) and the C++
Array / op:: layer above it; this Python package is only the harness that
loads the library for tests and benchmarks (device memory and process groups
come from torch).
"""
from .capi import Library, DaliB200Error, load_library  # noqa: F401
