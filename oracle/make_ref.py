"""Stage the reference's own Python sources of the prefill hot path next to the oracle.  TEST/BENCH INFRASTRUCTURE.

    python oracle/make_ref.py [--reference /path/to/x-attention]

Copies, unmodified, the three files that hold the path in mit-han-lab/x-attention

    xattn/src/Xattention.py   (xattn_estimate, Xattention_prefill)
    xattn/src/kernels.py      (the Triton estimate kernels and their launchers)
    xattn/src/utils.py        (find_blocks_chunked)

from a checkout of the reference into ``oracle/_ref/xattn/src/`` (plus empty package markers).  That folder is
a build product: it is listed in .gitignore, never committed, and exists only so that the benchmark's
reference arm can time the reference's own code -- on the host cores, and on the GPU for the secondary
``reference_gpu`` figures -- on a machine that has no checkout.  When no checkout is given or found the script
does nothing and the benchmark falls back to the CPU restatement in ``oracle/xattn_oracle.py``.

``load()`` imports the staged copy as ``xattn.src.Xattention`` with the two shims the reference needs outside
its own environment (none of its files is changed):
  * a stub module ``block_sparse_attn`` (imported unconditionally at xattn/src/Xattention.py:10; the package
    is a third-party CUDA extension that is not part of the reference tree),
  * for the CPU arm (and always on a machine without a GPU), ``Tensor.to("cuda")`` of a CPU tensor made a
    no-op (hard-coded at xattn/src/Xattention.py:43,47,185,251); see ``keep_on_cpu``.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = ("xattn/src/Xattention.py", "xattn/src/kernels.py", "xattn/src/utils.py")
DEFAULT_CHECKOUT = os.environ.get("XATTN_REFERENCE", "/root/reference")


def stage(reference: str = DEFAULT_CHECKOUT, quiet: bool = False) -> bool:
    """Copy the files; returns False (and leaves an existing copy alone) when the checkout is absent."""
    if not all(os.path.exists(os.path.join(reference, f)) for f in FILES):
        if not quiet:
            print(f"make_ref: no reference checkout at {reference}; nothing staged")
        return False
    for f in FILES:
        dst = os.path.join(REF_DIR, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, f), dst)
    for pkg in ("xattn", "xattn/src"):
        open(os.path.join(REF_DIR, pkg, "__init__.py"), "w").close()
    if not quiet:
        print(f"make_ref: staged {len(FILES)} files under {REF_DIR}")
    return True


def available() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in FILES)


_keep_on_cpu = False


def keep_on_cpu(flag: bool) -> None:
    """While set, the reference's hard-coded ``.to("cuda")`` calls are no-ops, so CPU tensors stay on the CPU
    (always the case on a machine without a GPU).  The CPU arm sets it; the GPU figures clear it."""
    global _keep_on_cpu
    _keep_on_cpu = bool(flag)


def load():
    """Import the staged reference; returns the module ``xattn.src.Xattention`` of the staged copy."""
    if not available():
        raise ImportError("oracle/_ref is empty: run oracle/make_ref.py where the reference is checked out")
    import torch
    if "block_sparse_attn" not in sys.modules:
        stub = types.ModuleType("block_sparse_attn")
        stub.block_sparse_attn_func = None
        sys.modules["block_sparse_attn"] = stub
    if not getattr(torch.Tensor.to, "_xattn_ref_shim", False):
        orig = torch.Tensor.to

        def _to(self, *a, **k):
            if (_keep_on_cpu or not torch.cuda.is_available()) and a and isinstance(a[0], str) \
                    and a[0].startswith("cuda") and not self.is_cuda:
                return self
            return orig(self, *a, **k)

        _to._xattn_ref_shim = True
        torch.Tensor.to = _to
    if "xattn.src.Xattention" in sys.modules and \
            os.path.abspath(getattr(sys.modules["xattn.src.Xattention"], "__file__", "")).startswith(REF_DIR):
        return sys.modules["xattn.src.Xattention"]
    # the staged copy must win over the package's own `xattn` import-path shim
    for name in [n for n in sys.modules if n == "xattn" or n.startswith("xattn.")]:
        del sys.modules[name]
    sys.path.insert(0, REF_DIR)
    try:
        import xattn.src.Xattention as mod
    finally:
        sys.path.remove(REF_DIR)
    assert os.path.abspath(mod.__file__).startswith(REF_DIR)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_CHECKOUT)
    stage(ap.parse_args().reference)
