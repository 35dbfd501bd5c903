#!/usr/bin/env python
"""Regenerates tests/golden/*.npz and kat.json.   python tests/golden/make_golden.py

For every case of cases.py the plan is run through the C++ oracle and through its independent numpy float64
restatement; the two must agree to one FP16 unit in the last place on every element (bit-exactly for the
activations without transcendental functions) before the C++ result is written. Inputs are stored by hash only:
they are regenerated from the seeds in cases.py.
"""
import hashlib
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

from oracle import oracle as O  # noqa: E402
import cases  # noqa: E402

HERE = Path(__file__).resolve().parent


def ulp_distance(a_bits, b_bits):
    def key(u):                       # monotone integer key of an FP16 bit pattern
        u = u.astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - (u & 0x7fff), 0x8000 + u)
    return np.abs(key(a_bits) - key(b_bits))


def main():
    index = {}
    for name in cases.CASES:
        plan, x = cases.build(name)
        got_c = cases.output_rows(plan, O.run_plan(plan, x))
        got_np = cases.output_rows(plan, O.run_plan(plan, x, use_numpy=True))
        d = ulp_distance(got_c, got_np)
        exact = all(w.act in (0, 1, 4) for w in plan.waves)
        assert d.max() <= (0 if exact else 1), f"{name}: oracle and numpy restatement differ by {d.max()} ulp"
        np.savez_compressed(HERE / f"{name}.npz", out=got_c)
        index[name] = {"input_sha256": hashlib.sha256(np.ascontiguousarray(x).tobytes()).hexdigest(),
                       "weights_sha256": hashlib.sha256(b"".join(np.ascontiguousarray(w.weights).tobytes() for w in plan.waves)).hexdigest(),
                       "out_sha256": hashlib.sha256(got_c.tobytes()).hexdigest(), "elements": int(got_c.size),
                       "max_ulp_vs_numpy": int(d.max())}
        print(name, index[name]["elements"], "elements, max ulp vs numpy", int(d.max()))
    # known answers that do not come from this code base: FNV-1a-64 test vectors of the published algorithm,
    # IEEE-754 binary16 encodings, and the 16x16-tile vector index formula evaluated by hand
    kat = {
        "fnv1a64": {"": "cbf29ce484222325", "a": "af63dc4c8601ec8c", "foobar": "85944171f73967e8"},
        "f32_to_f16": {"1.0": "3c00", "-2.0": "c000", "65504.0": "7bff", "65520.0": "7c00", "1e-8": "0000", "5.960464477539063e-08": "0001",
                       "2.9802322387695312e-08": "0000", "8.940696716308594e-08": "0002", "0.333251953125": "3555", "inf": "7c00"},
        "wmma_vec_index": [{"j": 0, "k8": 0, "B": 64, "index": 0}, {"j": 1, "k8": 0, "B": 64, "index": 1}, {"j": 0, "k8": 1, "B": 64, "index": 16},
                           {"j": 17, "k8": 3, "B": 64, "index": 177}, {"j": 35, "k8": 6, "B": 128, "index": 611}],
        "cases": index,
    }
    (HERE / "kat.json").write_text(json.dumps(kat, indent=1) + "\n")


if __name__ == "__main__":
    main()
