"""Regenerate llama_thresholds.npz from a checkout of the reference.

    python make_threshold_tables.py --reference /path/to/x-attention

The reference ships per-(layer, head) selection thresholds for Llama-3.1-8B-Instruct, one 32x32 table per stride
(xattn/threshold/llama_threshold.py: llama_fuse_4, llama_fuse_8, llama_fuse_16), which its FastPrefillConfig uses
when no threshold is given (xattn/src/load_llama.py:253-261).  They are model data (the output of the reference's
threshold profiler), stored here as float32 arrays so that FastPrefillConfig(threshold=None) behaves the same.
"""
import argparse
import os
import sys

import numpy as np

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from xattn.threshold import llama_threshold as t
    out = {f"fuse_{s}": np.asarray(getattr(t, f"llama_fuse_{s}"), dtype=np.float32) for s in (4, 8, 16)}
    for k, v in out.items():
        assert v.shape == (32, 32), (k, v.shape)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "llama_thresholds.npz"), **out)
    print({k: (v.shape, float(v.mean())) for k, v in out.items()})
