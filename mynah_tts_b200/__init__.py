"""B200-native decode path for mynah-tts's Magpie decoder step.

The product is the C-ABI shared library built from csrc/ (see
include/mynah_b200.h).  `capi` binds it with ctypes, `backend` mirrors the
reference's backend/decoder interface on top of it, `synth` makes the seeded
synthetic weights the tests and the benchmark run on.
"""
from . import synth  # noqa: F401

__all__ = ["synth", "capi", "backend"]
