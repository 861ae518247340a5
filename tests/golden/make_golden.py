"""Generates tests/golden/known_answers.npz from the C oracle.

The reference (Rust) cannot be built or imported offline, so these vectors come from the oracle's
restatement of it; they pin the oracle against accidental change and give the GPU tests fixed
inputs and outputs that need no oracle at run time.  Run from the repository root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import oracle as O  # noqa: E402
from xn_b200 import synth  # noqa: E402
from xn_b200.dtypes import GgmlDType as D  # noqa: E402


def main():
    O.build()
    out = {}
    n, k, m = 24, 512, 5
    x = synth.make_activation(m, k, seed=7, tensor_id=77)
    x[1, 256:512] = 0.0          # an all-zero Q8_K block / Q8_0 blocks
    x[2, 3] = x[2, 9] = 4.5      # a tie in |x| for the Q8_K argmax (first wins)
    x[2, 9] = -4.5
    x[3, :] *= 1e-3
    out["x"] = x
    out["act_q8_0"] = O.from_float(O.Q8_0, x)
    out["act_q8k"] = O.from_float(O.Q8K, x)
    for dt in (D.Q4_0, D.Q8_0, D.Q4K, D.Q6K):
        w = synth.make_weight(dt, n, k, seed=7, tensor_id=int(dt))
        out[f"w_{dt.name}"] = w
        out[f"deq_{dt.name}"] = O.to_float(dt, w, n * k)
        out[f"y_{dt.name}"] = O.matmul(dt, x, w, n, threads=1)
    # weights produced by the reference's own quantizers from a dense matrix (from_linear path)
    dense = synth.make_activation(n, k, seed=7, tensor_id=99) * np.float32(0.05)
    out["dense"] = dense
    for dt in (D.Q4_0, D.Q8_0, D.Q4K, D.Q6K):
        out[f"wq_{dt.name}"] = O.from_float(dt, dense)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_answers.npz"), **out)
    print("wrote known_answers.npz:", {k_: v.shape for k_, v in out.items()})


if __name__ == "__main__":
    main()
