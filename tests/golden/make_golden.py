"""Regenerates tests/golden/reference_fixture.npz from the reference's own golden file.

The reference checks itself against PyTorch through
crates/weta/tests/fixtures/reference.safetensors (written by its scripts/make_fixtures.py,
consumed by crates/weta/tests/reference.rs at 1e-9).  This script copies those 63 tensors,
unchanged, into an .npz so the oracle can be pinned to them on machines where the reference
checkout is absent.  Run from the repository root:

    python tests/golden/make_golden.py /path/to/weta
"""
import os
import sys

import numpy as np
from safetensors.numpy import load_file


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/weta")
    root = sys.argv[1]
    src = os.path.join(root, "crates/weta/tests/fixtures/reference.safetensors")
    tensors = load_file(src)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_fixture.npz")
    np.savez_compressed(out, **tensors)
    print(f"wrote {len(tensors)} tensors to {out}")


if __name__ == "__main__":
    main()
