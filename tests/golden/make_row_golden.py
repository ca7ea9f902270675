"""Generate tests/golden/row_reference.npz from the reference's own NumPy statement of the
32-lane FP32 row schedule (tools/ascend/tests/test_row_reference.py:7-28: reduce_row, softmax, rms).

Run once where the reference checkout is available:
    python tests/golden/make_row_golden.py /path/to/rust-ascend
Only outputs are stored; inputs are regenerated from the seeds below by `row_case_inputs`.
"""
import importlib.util
import os
import sys

import numpy as np

SHAPES = [(1, 32), (3, 96), (7, 256), (2, 1024), (3, 4096)]


def row_case_inputs(rows, width):
    rng = np.random.default_rng(1000 + 7 * rows + width)
    x = rng.normal(size=(rows, width)).astype(np.float32)
    big = (rng.normal(size=(rows, width)) * 3 + 1000).astype(np.float32)
    w = rng.uniform(0.5, 1.5, size=width).astype(np.float32)
    return x, big, w


def main(reference_root):
    path = os.path.join(reference_root, "tools/ascend/tests/test_row_reference.py")
    spec = importlib.util.spec_from_file_location("row_reference", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    out = {}
    for rows, width in SHAPES:
        x, big, w = row_case_inputs(rows, width)
        key = f"{rows}x{width}"
        out[f"sum_{key}"] = ref.reduce_row(x)
        out[f"max_{key}"] = ref.reduce_row(x, True)
        out[f"softmax_{key}"] = ref.softmax(big)
        out[f"logsoftmax_{key}"] = ref.softmax(big, True)
        y, r = ref.rms(x, w)  # the reference helper fixes eps = 1e-5
        out[f"rms_y_{key}"] = y
        out[f"rms_rstd_{key}"] = r
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "row_reference.npz"), **out)


if __name__ == "__main__":
    main(sys.argv[1])
