"""Model families: Wan2.2-style DiT, LTX-style DiT, MiniMax-H3-style packed-document DiT, VAEs."""
from .wan import WanConfig, WanDiT, wan_preset  # noqa: F401
