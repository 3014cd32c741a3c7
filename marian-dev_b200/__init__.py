"""B200-native int8 affine engine behind Marian's operator surface.

The directory name carries a hyphen, so it is imported through the ``marian_dev_b200`` module at the
repository root, which points its package path here.
"""
from .binding import LIB_PATH, Mi8Error, build_library, lib, multiply_plan  # noqa: F401
