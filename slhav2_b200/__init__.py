"""slhav2_b200 -- B200 (sm_100a) implementation of the SLHA v2 KV-cache tile hot
path (encode, eq. 2.3 scoring, top-k, CCOS elastic pool) behind the reference's
C ABI.  The compute lives in libslha_b200.so (CUDA); this package is the thin
host-side mirror of the reference's operator surface."""
from .api import *  # noqa: F401,F403
from .api import load_library, LIB_PATH, SIGNATURES  # noqa: F401
from . import shard  # noqa: F401
