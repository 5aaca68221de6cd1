"""Drop-in counterparts of the reference's `GPT-FAST/kernels` package."""
from .sparse import build_sparse_list_decode, build_sparse_list_native, sparse_attention_fwd  # noqa: F401
