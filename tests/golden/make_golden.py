"""Writes tests/golden/oracle_vectors.json: small outputs of the CPU oracle on fixed seeds, committed so that a change
to the oracle (or to the seeded generators the GPU fills mirror) cannot go unnoticed.  The reference implementation is
Rust and cannot be run in this environment, so these vectors pin this repository's restatement; the reference's own
known-answer values are asserted directly in tests/test_oracle_golden.py.

Run from the repository root: python tests/golden/make_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import oracle  # noqa: E402
from util import values  # noqa: E402

x = values(64, 11)
w = oracle.fill_codes(5, 0, 4 * 64).reshape(4, 64)
s = oracle.fill_scales(5, 1, 4 * 2, 0.02 / 127).reshape(4, 2)
y, exact, _ = oracle.gemv_q8(w, s, x)
packed, scales = oracle.q4(values(128, 5))
token, gap = oracle.sample_greedy(values(4000, 9) * 40.0, softcap=30.0)
out = {
    "fill_codes_7_3": [int(v) for v in oracle.fill_codes(7, 3, 16)],
    "fill_scales_7_4": [int(v) for v in oracle.fill_scales(7, 4, 8, 0.02 / 127)],
    "values_11": [float(v) for v in x[:8]],
    "gemv_exact": [float(v) for v in exact],
    "gemv_f32": [float(v) for v in y],
    "q4_packed": [int(v) for v in packed[:8]],
    "q4_scales": [int(v) for v in scales],
    "greedy_token": token,
}
with open(os.path.join(HERE, "oracle_vectors.json"), "w") as f:
    json.dump(out, f, indent=1)
print("wrote", os.path.join(HERE, "oracle_vectors.json"))
