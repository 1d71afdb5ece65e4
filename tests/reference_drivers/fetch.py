"""Puts the reference's own driver scripts where the drop-in test can run them unmodified.

    python tests/reference_drivers/fetch.py [reference_root]

Copies test/torch_test.py, test/bench.py and test/util.py of the reference checkout (the directory given on the
command line or in DQMOE_REFERENCE_ROOT; REFERENCE_ROOT below otherwise) into baseline/_ref/test/ at the root of this
repository. That folder is ignored by git,
so the scripts never enter this repository's history; tests/test_gpu_reference_drivers.py runs
torch_test.py from there as a child process with dqmoe_b200/dropin on PYTHONPATH, so that its
`import moe_test` resolves to the drop-in module, as the reference's develop.sh:12-15 arranges for its own
extension. Nothing is edited: the copies are byte-identical (checked by size and digest after the copy).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import sys

FILES = ("torch_test.py", "bench.py", "util.py")
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
DEST = os.path.join(ROOT, "baseline", "_ref", "test")
REFERENCE_ROOT = os.environ.get("DQMOE_REFERENCE_ROOT", "/root/reference")


def _digest(path: str) -> str:
    with open(path, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def fetch(reference_root: str = REFERENCE_ROOT) -> bool:
    """True when the three scripts are in place (copied now or earlier); False without a reference checkout."""
    src_dir = os.path.join(reference_root, "test")
    if not all(os.path.exists(os.path.join(src_dir, f)) for f in FILES):
        return all(os.path.exists(os.path.join(DEST, f)) for f in FILES)
    os.makedirs(DEST, exist_ok=True)
    for f in FILES:
        src, dst = os.path.join(src_dir, f), os.path.join(DEST, f)
        shutil.copyfile(src, dst)
        if _digest(src) != _digest(dst):
            raise RuntimeError(f"copy of {src} differs from its source")
    return True


if __name__ == "__main__":
    ok = fetch(sys.argv[1] if len(sys.argv) > 1 else REFERENCE_ROOT)
    print(DEST if ok else "no reference checkout found")
