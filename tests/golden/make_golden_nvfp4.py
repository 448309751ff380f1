"""Generates tests/golden/nvfp4_weight.json by running the REFERENCE's own NVFP4 weight rounding (quantize_nvfp4, compiled
from the reference project's model.cu into oracle/_ref/libling_refquant.so by `make -C oracle ref_quant`) on seeded inputs.

    python tests/golden/make_golden_nvfp4.py

The fixture travels with the repository; the reference project does not.  Inputs are numpy PCG64 draws from the seeds below
(stored too, as BF16 bit patterns, so the test needs no generator agreement); some blocks are built to land values exactly
on the midpoints between two E2M1 codes and on the 2^-9 floor of the block scale.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import lo as lom  # noqa: E402


def bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def cases():
    rng = np.random.default_rng(20260101)
    out = []
    for N, K, std, spikes in [(8, 64, 0.02, 0.02), (5, 32, 1.0, 0.0), (3, 16, 7.0, 0.3), (16, 128, 0.02, 0.01)]:
        w = (rng.standard_normal((N, K)) * std).astype(np.float32)
        w[rng.random((N, K)) < spikes] *= 30
        out.append(("normal N=%d K=%d std=%g" % (N, K, std), w))
    # midpoints: the matrix maximum 2688 makes the tensor scale exactly 1; a block whose largest value is 6 * 2^e gets the
    # scale 2^e, and the multiples of 2^e below sit on codes and midpoints
    mid = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 0.0], np.float32)
    w = np.stack([mid * 2.0 ** e for e in (-3, 0, 2, 5)])
    w = np.concatenate([w, np.full((4, 16), 0, np.float32)], axis=1)
    w[0, 16] = 2688.0
    out.append(("midpoints", w.astype(np.float32)))
    # tiny blocks beside a large maximum: the block scale's floor of 2^-9
    w = np.zeros((2, 32), np.float32)
    w[0, 0] = 1000.0
    w[0, 16:32] = np.linspace(-1e-4, 1e-4, 16)
    w[1, :16] = np.linspace(-2e-3, 2e-3, 16)
    out.append(("scale floor", w))
    out.append(("all zero", np.zeros((2, 16), np.float32)))
    return out


def main():
    ref = lom.refquant()
    if ref is None:
        raise SystemExit("oracle/_ref/libling_refquant.so is missing: make -C oracle ref_quant REF=<reference checkout>")
    golden = []
    for name, w in cases():
        bits = bf16_bits(w)
        q, sf, s2 = lom.nvfp4_quantize_weight(bits, use_reference=True)
        golden.append({"name": name, "N": int(w.shape[0]), "K": int(w.shape[1]), "w_bf16": bits.ravel().tolist(),
                       "values": q.ravel().tolist(), "scales": sf.ravel().tolist(),
                       "scale2_bits": int(np.float32(s2).view(np.uint32))})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nvfp4_weight.json")
    with open(path, "w") as f:
        json.dump(golden, f, separators=(",", ":"))
    print(path, os.path.getsize(path), "bytes,", len(golden), "cases")


if __name__ == "__main__":
    main()
