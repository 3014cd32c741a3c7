"""B200-native int8 affine engine behind Marian's operator surface.

The directory name carries a hyphen, so it is imported through the ``marian_dev_b200`` module at the
repository root, which points its package path here.

Modules: ``ops`` (affine / dot / affineWithReluDropout on intgemm8 weights), ``packed8`` (the packed8avx512
scheme), ``binary_io`` (model container and conversion), ``decoder`` / ``model`` (decode driver),
``parallel`` (sharding), ``binding`` (ctypes view of libmarian_i8.so; there is no CPU fallback).
"""
from .binding import LIB_PATH, Mi8Error, build_library, lib, multiply_plan  # noqa: F401
