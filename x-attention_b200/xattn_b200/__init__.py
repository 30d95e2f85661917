"""xattn_b200 -- the XAttention prefill hot path (estimate -> select -> block-sparse attention) on
NVIDIA B200 (sm_100a).  Same operator interface as mit-han-lab/x-attention's xattn.src.Xattention."""
from .api import Xattention_prefill, block_sparse_attn_func, find_blocks_chunked, xattn_estimate  # noqa: F401
from .host_pipeline import Xattention_prefill_host  # noqa: F401
from .ops import check_device_status, get_estimate_semantics, set_estimate_semantics  # noqa: F401
