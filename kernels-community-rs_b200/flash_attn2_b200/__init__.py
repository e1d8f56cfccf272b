"""B200 (sm_100a) FlashAttention-2 behind the flash-attn2-rs operator surface."""
from . import cabi_ops  # noqa: F401
