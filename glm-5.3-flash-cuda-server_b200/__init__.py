"""B200-native NVFP4 weight path: ctypes door into libb200nvfp4.so (no CPU fallback)."""
from .binding import *  # noqa: F401,F403
from . import ep, ep_gpu  # noqa: F401
