"""Install the UMA-QMoE reference's own Python package under ``oracle/_ref/`` (test infrastructure).

    python oracle/make_ref.py [--reference /path/to/reference/checkout]

The reference is pure Python (one package, ``src/uma_qmoe``; its build back end only copies that
directory into a wheel), so "installing" it is placing that package directory where
``sys.path.insert(0, "oracle/_ref")`` finds it.  ``oracle/_ref/`` is listed in ``.gitignore``: nothing of
the reference enters this repository's history, but the directory travels with the working tree to the
machine the benchmark runs on, where ``bench.py --impl reference`` and the ``cpu_baseline`` leg time the
reference's CPU correctness path (``torch.ops.uma_qmoe.moe_forward(..., performance_mode=False)``,
``src/uma_qmoe/custom_op.py:301-340``) itself instead of this repository's restatement of it.

Only ``tests/``, ``__graft_entry__`` and ``bench.py`` may use what this script installs; the product
package never imports it.
"""

from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def install(reference: Path) -> Path:
    package = reference / "src" / "uma_qmoe"
    if not (package / "custom_op.py").exists():
        raise FileNotFoundError(f"{package} is not the reference's package directory")
    dest = TARGET / "uma_qmoe"
    if dest.exists():
        shutil.rmtree(dest)
    TARGET.mkdir(parents=True, exist_ok=True)
    shutil.copytree(package, dest, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    (TARGET / "INSTALLED_FROM.txt").write_text(f"{package}\n")
    return dest


def available() -> bool:
    return (TARGET / "uma_qmoe" / "custom_op.py").exists()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="checkout of the reference project")
    args = ap.parse_args()
    if args.reference is None:
        sys.exit("pass --reference <checkout of zihaomu/UMA-QMoE>")
    print(install(Path(args.reference)))
