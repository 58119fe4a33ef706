"""deepgemm (B200): host-side mirror of the reference crate's operator API over the C ABI of
libdeepgemm_b200.so.  See include/deepgemm_b200.h for the boundary."""
from .api import *  # noqa: F401,F403
from .types import *  # noqa: F401,F403
from . import _lib  # noqa: F401
