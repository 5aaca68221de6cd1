"""socket_b200 — B200-native sparse-attention decode path of SOCKET (soft-LSH key scoring,
top-k select, GQA sparse flash-decode) behind the reference's operator surface."""
from .config import PRESETS, SocketConfig  # noqa: F401

__all__ = ["SocketConfig", "PRESETS"]
