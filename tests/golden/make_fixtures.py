"""Regenerate tests/golden/oracle_fixtures.json from the CPU oracle.

    python tests/golden/make_fixtures.py

The fixture pins (a) the synthetic-data stream every test and the bench draw
their inputs from and (b) oracle products on small seeded inputs, so a change
to the oracle or the generator cannot go unnoticed.  The reference (Rust,
todo!() bodies) cannot be executed; its own hand-computed constants live in
a4_hand_cases.json and were transcribed from its spec files.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.oracle_lib import ACC_F64, ACC_NATIVE, BF16, F16, F32, Oracle  # noqa: E402


def main():
    o = Oracle()
    fx = {"fill": [], "matmul": []}
    for tag, name in ((F32, "f32"), (BF16, "bf16"), (F16, "f16")):
        for dist, scale in (("uniform", 1.0), ("normal", 0.02)):
            x = o.fill((16,), tag, seed=7, stream=3, dist=dist, scale=scale)
            fx["fill"].append({"dtype": name, "dist": dist, "scale": scale, "seed": 7, "stream": 3,
                               "bits": [int(v) for v in x.view(np.uint32 if tag == F32 else np.uint16)]})
    for tag, name in ((F32, "f32"), (BF16, "bf16"), (F16, "f16")):
        a = o.fill((5, 7), tag, seed=11, stream=0, dist="uniform")
        b = o.fill((7, 3), tag, seed=11, stream=1, dist="uniform")
        for acc, accname in ((ACC_NATIVE, "native"), (ACC_F64, "f64")):
            st, c = o.matmul(a, b, tag, acc=acc, nthreads=1)
            assert st == 0
            fx["matmul"].append({"dtype": name, "acc": accname, "seed": 11, "a_shape": [5, 7], "b_shape": [7, 3],
                                 "out_hex": [float(v).hex() for v in c.reshape(-1)]})
    with open(os.path.join(HERE, "oracle_fixtures.json"), "w") as f:
        json.dump(fx, f, indent=1)
    print("wrote oracle_fixtures.json")


if __name__ == "__main__":
    main()
