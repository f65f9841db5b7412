"""Recipe for ``oracle/_ref/``: the reference's own CPU implementation, used as checker and CPU baseline.

    python oracle/install_ref.py /path/to/reference/checkout

The reference's CPU path is one pure-torch file, ``HRDPLR/naive.py`` (``hrdplr_naive``,
``HRDPLR/naive.py:76-263``): there is nothing to compile, so "building" it means placing that file,
unmodified, where ``oracle.ref_naive`` finds it.  ``oracle/_ref/`` is listed in ``.gitignore`` -- the
reference's source never enters this repository's history -- but it travels with the working tree to
the machine the benchmark runs on.  TEST INFRASTRUCTURE ONLY: the shipped operator never touches it.

Returns 0 and prints the destination when the file was placed, 1 when the checkout has no
``HRDPLR/naive.py``.
"""
import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def install(ref_root: str) -> str:
    src = os.path.join(ref_root, "HRDPLR", "naive.py")
    if not os.path.isfile(src):
        raise FileNotFoundError(src)
    os.makedirs(DEST, exist_ok=True)
    dst = os.path.join(DEST, "naive.py")
    shutil.copyfile(src, dst)
    with open(dst, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(DEST, "SOURCE.txt"), "w") as f:
        f.write(f"HRDPLR/naive.py of the reference checkout, unmodified\nsha256 {digest}\n")
    return dst


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    try:
        print(install(sys.argv[1]))
    except FileNotFoundError as e:
        print(f"not found: {e}", file=sys.stderr)
        sys.exit(1)
