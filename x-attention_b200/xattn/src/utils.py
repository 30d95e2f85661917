"""Drop-in for the reference module of the same import path (xattn/src/utils.py)."""
from xattn_b200.api import find_blocks_chunked  # noqa: F401
