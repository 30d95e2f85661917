"""The bounded-wait abort path of the kernels, exercised without faulting or hanging anything: a test-only kernel
(tests/cuda/wait_timeout_probe.cu, built here with a wait limit of about a millisecond) waits on a barrier nobody
arrives on; the wait must run out, every waiting role must give up, the status word must read 101
(XATTN_B200_ERR_DEVICE_WAIT), the host API must turn that into an exception, and the context must stay usable."""
import ctypes
import os
import shutil
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available to build the probe")
    out = str(tmp_path / "libwait_probe.so")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
           "-DXB_WAIT_CYCLE_LIMIT=2000000LL", "-I", os.path.join(ROOT, "x-attention_b200", "xattn_b200", "csrc"),
           "-o", out, os.path.join(ROOT, "tests", "cuda", "wait_timeout_probe.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return ctypes.CDLL(out)


def test_a_wait_that_runs_out_reports_101_and_leaves_the_context_usable(tmp_path):
    import xattn_b200
    from xattn_b200 import ops
    from xattn_b200._lib import XattnB200Error
    lib = _build(tmp_path)
    lib.wait_timeout_probe.restype = ctypes.c_int
    lib.wait_timeout_probe.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    dev = torch.device("cuda", torch.cuda.current_device())
    status = ops._status(dev)                     # the pinned word the library's own kernels report to
    assert int(status[0]) == 0
    seen = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.wait_timeout_probe(status.data_ptr(), seen.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()                      # returns: the kernel ended by itself after ~1 ms
    assert int(seen[0]) == 2                      # both waiting roles gave up
    assert int(status[0]) == 101
    with pytest.raises(XattnB200Error, match="bounded wait"):
        xattn_b200.check_device_status(dev)
    assert int(status[0]) == 0                    # reading the status clears it
    # the context is intact: a regular call still works
    q = torch.randn(1, 2, 512, 128, device=dev).bfloat16()
    out = xattn_b200.Xattention_prefill(q, q, q, 16, threshold=0.9, chunk_size=2048)
    xattn_b200.check_device_status(dev)
    assert torch.isfinite(out.float()).all()
