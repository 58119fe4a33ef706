"""CPU oracle for the block-scaled GEMM path (test infrastructure only).

Only the tests, the smoke check and the benchmark's cpu_baseline / reference arm import
this package.  The shipped library never does.
"""
from .oracle import *  # noqa: F401,F403
from . import sampled  # noqa: F401,E402
