"""Generates tests/golden/quant_linear_v1.npz from the NumPy oracle.

The reference project has no numeric implementation of this path, so these
vectors pin THIS repository's format specification (see oracle/oracle.py), not
reference output.  Run from the repository root:  python tests/golden/make_golden.py
The C restatement must reproduce every array bit-for-bit (checked here and in
tests/test_oracle.py); the CUDA library is checked against the same file on the GPU.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle as o  # noqa: E402
import oracle_c as oc  # noqa: E402

SEED = o.DEFAULT_SEED
CASES = [  # (name, tensor ids (w, x), M, N, K)
    ("a", (11, 12), 1, 17, 256),
    ("b", (13, 14), 3, 37, 384),
    ("c", (15, 16), 8, 73, 1024),
]


def main():
    out = {}
    for name, (tw, tx), m, n, k in CASES:
        w = o.planted_case_weights(SEED, tw, n, k)  # regenerated from the seed by the tests, not stored
        x = o.synth_activations(SEED, tx, m, k)
        p, s = o.aq4_quantize(w)
        c, cs = o.fp8_quantize(w)
        p2, s2 = oc.aq4_quantize(w)
        c2, cs2 = oc.fp8_quantize(w)
        assert np.array_equal(p, p2) and np.array_equal(s.view(np.uint16), s2.view(np.uint16))
        assert np.array_equal(c, c2) and np.array_equal(cs, cs2)
        out[f"{name}_x_bits"] = o.f32_to_bf16_bits(x).reshape(m, k)
        out[f"{name}_aq4_packed"] = p
        out[f"{name}_aq4_scales_bits"] = s.view(np.uint16)
        out[f"{name}_fp8_codes"] = c
        out[f"{name}_fp8_scale"] = cs
        out[f"{name}_y_aq4_bits"] = o.f32_to_bf16_bits(o.linear(x, o.aq4_dequantize(p, s))).reshape(m, n)
        out[f"{name}_y_fp8_bits"] = o.f32_to_bf16_bits(o.linear(x, o.fp8_dequantize(c, cs))).reshape(m, n)
    out["synth_normal_t7_first64"] = o.synth_normal(SEED, 7, 0, 64)
    out["e4m3_table"] = o.E4M3_TABLE
    path = os.path.join(ROOT, "tests", "golden", "quant_linear_v1.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
