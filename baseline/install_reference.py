"""Places the reference files whose call sites the drop-in tests exercise under baseline/_ref/.

    python baseline/install_reference.py <reference checkout>      (or set HILS_REFERENCE_ROOT)

The reference has no build target for its Python sources, so `pip install --target baseline/_ref` does not apply;
this copies the two modules that bind the ops by import (their relative paths kept).  baseline/_ref/ is git-ignored:
nothing of the reference enters the history.  tests/test_gpu_reference_callsites.py looks for the files under
$HILS_REFERENCE_ROOT and baseline/_ref/, in that order, and skips when neither has them.
"""
import os
import shutil
import sys

FILES = ["models/FlashHiLS/hils_attention.py", "models/NaiveBSA/naive_bsa_kernel.py"]


def main():
    src = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HILS_REFERENCE_ROOT")
    if not src:
        raise SystemExit("usage: python baseline/install_reference.py <reference checkout>  (or set HILS_REFERENCE_ROOT)")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    for f in FILES:
        os.makedirs(os.path.dirname(os.path.join(dst, f)), exist_ok=True)
        shutil.copyfile(os.path.join(src, f), os.path.join(dst, f))
        print("copied", f)


if __name__ == "__main__":
    main()
