"""Recipe for oracle/_ref: places the reference's own dense implementation beside the oracle.  TEST INFRASTRUCTURE ONLY.

The reference's CPU path for stick-breaking attention is one pure-PyTorch file,
``stickbreaking_attention/sb_ref.py`` (function ``stickbreaking``, lines 8-25).  It needs no compilation; this
script takes it, unmodified, from the reference checkout into ``oracle/_ref/`` (a git-ignored directory, so the
file never enters this repository's history) where the benchmark's CPU arm can import it on a machine that has no
reference checkout.

    python oracle/build_ref.py [path-to-reference-checkout]

``ref_drive.py`` (committed, beside this file) drives the copied function per sequence the way the reference's own
tests do (tests/test_varlen.py:11-43 of the reference).
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build_ref(reference_root="/root/reference"):
    """Returns the path of oracle/_ref/sb_ref.py, or None when no reference checkout is present and no earlier
    copy exists."""
    src = os.path.join(reference_root, "stickbreaking_attention", "sb_ref.py")
    dst = os.path.join(OUT, "sb_ref.py")
    if os.path.isfile(src):
        os.makedirs(OUT, exist_ok=True)
        shutil.copyfile(src, dst)
    return dst if os.path.isfile(dst) else None


if __name__ == "__main__":
    print(build_ref(*sys.argv[1:2]))
