"""Places the reference's own implementation of the hot path beside the oracle, UNMODIFIED, as ``oracle/_ref/``.

    python oracle/make_ref.py <path to a checkout of the reference project>

``oracle/_ref/`` is a build output: it is ignored by git (nothing of the reference enters the history) and is only
used as a checker and as the timed CPU baseline -- by the tests, by the smoke entry and by the CPU legs of bench.py.
The product package never imports it.  The files are copied byte for byte; ``load()`` imports them from there.
"""
import importlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
# the forward being replaced, the quantiser and wrapper classes it uses, and the weight-only NVFP4 module
FILES = ["utils/__init__.py", "utils/quant_utils.py", "utils/hadamard_utils.py", "dirotq_fused_unrotation.py",
         "dirotq_fused_unrotation_fast.py", "speedup/weight_only_nvfp4.py"]


def make(ref_root: str) -> str:
    for rel in FILES:
        src = os.path.join(ref_root, rel)
        dst = os.path.join(DEST, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if os.path.exists(src):
            shutil.copyfile(src, dst)
        elif rel.endswith("__init__.py"):
            open(dst, "a").close()
        else:
            raise FileNotFoundError(src)
    return DEST


def available() -> bool:
    return all(os.path.exists(os.path.join(DEST, rel)) for rel in FILES if not rel.endswith("__init__.py"))


def load():
    """(utils.quant_utils, dirotq_fused_unrotation, dirotq_fused_unrotation_fast) imported from oracle/_ref."""
    if not available():
        raise RuntimeError("oracle/_ref is not populated: run `python oracle/make_ref.py <reference checkout>`")
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    qu = importlib.import_module("utils.quant_utils")
    slow = importlib.import_module("dirotq_fused_unrotation")
    fast = importlib.import_module("dirotq_fused_unrotation_fast")
    return qu, slow, fast


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit(__doc__)
    print(make(sys.argv[1]))
