"""Generate the convolutional golden fixtures (tests/golden/conv_*.npz) from the compiled
reference.

    python tests/golden/make_golden_conv.py

Needs oracle/_ref/libdeepity_ref.so (python oracle/build_ref.py, which needs the reference
checkout).  The cases live in tests/conv_common.py (CONV_CASES), from which the seeded inputs
are regenerated bit for bit; a fixture stores the energy of every train step, the prediction
after training and every layer's z, e, W, b after the last step (sums and sums of squares for
the benchmark-shaped case).
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from conv_common import CONV_CASES, run_conv_reference  # noqa: E402

if __name__ == "__main__":
    for name, case in CONV_CASES.items():
        out = run_conv_reference(case)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, "energies", out["energies"])
