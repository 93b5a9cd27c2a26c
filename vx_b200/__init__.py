"""vx_b200: the B200 dispatch library for Vx's tensor operators and its host
side.  Everything computes through libvx_cuda_dispatch.so (lib.py); there is no
other path."""
from . import abi, collective, llama, ops  # noqa: F401
from .lib import LIB_PATH, lib  # noqa: F401
