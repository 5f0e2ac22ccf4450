"""Produce the code-book JSON files of this directory with the reference's solver.

    python turboquant_b200/codebooks/make_codebooks.py /path/to/reference

The code books are data: Lloyd-Max centroids and bucket boundaries for the
coordinate distribution of a random point on the unit sphere in d dimensions
(reference codebook.py:68-143).  For every (d, bits) that the reference ships
as JSON the shipped values are taken; the others are computed by the
reference's solver in a scratch directory, because the reference would
otherwise write them into its own package directory (codebook.py:158-170).
Both sides of every parity test must use the same constants to the bit,
which is why the files are generated once and committed.
"""

import json
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
DIMS = (64, 128, 256)
BITS = (1, 2, 3, 4)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import turboquant.codebook as ref_codebook

    scratch = tempfile.mkdtemp(prefix="tq_codebooks_")
    for f in os.listdir(ref_codebook._CODEBOOK_DIR):
        if f.endswith(".json"):
            shutil.copy(os.path.join(ref_codebook._CODEBOOK_DIR, f), scratch)
    ref_codebook._CODEBOOK_DIR = scratch
    for d in DIMS:
        for b in BITS:
            cb = ref_codebook.get_codebook(d, b)
            with open(os.path.join(HERE, f"codebook_d{d}_b{b}.json"), "w") as fh:
                json.dump(cb, fh, indent=2)
    shutil.rmtree(scratch, ignore_errors=True)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python " + os.path.basename(__file__) + " <path to a checkout of the reference (0xSero/turboquant)>")
    main(sys.argv[1])
