"""B200-native KV4 attention path (codec, flash-decode, verify, prefill, sharded decode) behind the
reference's operator interface.  Importing this package does not touch the GPU; the CUDA library is
loaded on first use and there is no non-CUDA path."""
from . import _lib  # noqa: F401
from ._lib import F16, BF16, F32, ALGO_AUTO, ALGO_SCALAR, ALGO_MMA, Kv4Error  # noqa: F401
