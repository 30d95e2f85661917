"""Drop-in for the reference module of the same import path (xattn/src/Xattention.py)."""
from xattn_b200.api import Xattention_prefill, xattn_estimate  # noqa: F401
