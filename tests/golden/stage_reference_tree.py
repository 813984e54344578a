"""Stage a working copy of the reference's Python packages for the drop-in test.

    python tests/golden/stage_reference_tree.py /path/to/reference

copies deserve_worker/ and deserve_utils/ (Python files only, unmodified) into
baseline/_ref/ at the repository root. That directory is git-ignored: the copy is
a test fixture of this machine, not part of the repository.
tests/test_gpu_dropin_reference.py runs the reference's own caller code from
there against this package, and is skipped where the copy is absent. The
reference's packages cannot be pip-installed into a target directory: its
deserve_worker/pyproject.toml declares `py-modules = []` and no packages, so
an install carries no code.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent


def main(ref_root: str) -> None:
    src_root, dst_root = Path(ref_root), ROOT / "baseline" / "_ref"
    n = 0
    for pkg in ("deserve_worker", "deserve_utils"):
        for src in (src_root / pkg).rglob("*.py"):
            dst = dst_root / src.relative_to(src_root)
            dst.parent.mkdir(parents=True, exist_ok=True)
            shutil.copyfile(src, dst)
            n += 1
    print(f"staged {n} files under {dst_root}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/stage_reference_tree.py /path/to/reference")
    main(sys.argv[1])
