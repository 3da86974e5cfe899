#!/usr/bin/env python3
"""Recipe for ``oracle/_ref/``: the reference project's own NumPy evaluator, importable on a box without the checkout.

    python oracle/make_ref.py --reference <checkout of luogantt/General-AI-Compiler>

TEST INFRASTRUCTURE ONLY.  The reference's CPU path for multi-scale deformable
attention is pure Python + NumPy (``src/gac/core/ops.py:787-851`` behind
``evaluate_op`` :854, driven by ``reference_run`` in
``src/gac/validation/reference.py:32-38``).  This script takes the four modules
that path consists of, unmodified, from a checkout and places them under
``oracle/_ref/gac/`` -- a directory that is never committed (``.gitignore``) --
so that the benchmark's CPU arm and the parity tests can run the reference's
OWN code where no checkout exists.  The two package ``__init__`` files it
writes are empty: the reference's top-level ``__init__`` only installs legacy
import aliases that this path does not use.

Nothing in the shipped package imports ``oracle/_ref``.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
# module path inside the reference's src/ -> same path under oracle/_ref/
MODULES = ("gac/core/errors.py", "gac/core/ir.py", "gac/core/ops.py", "gac/validation/reference.py")
PACKAGES = ("gac", "gac/core", "gac/validation")


def make_ref(reference: Path, dest: Path = DEST) -> Path:
    src = Path(reference) / "src"
    missing = [m for m in MODULES if not (src / m).is_file()]
    if missing:
        raise FileNotFoundError(f"{src} does not hold {missing}")
    for pkg in PACKAGES:
        (dest / pkg).mkdir(parents=True, exist_ok=True)
        (dest / pkg / "__init__.py").write_text("")
    digests = {}
    for module in MODULES:
        shutil.copyfile(src / module, dest / module)
        digests[module] = hashlib.sha256((dest / module).read_bytes()).hexdigest()
    (dest / "MANIFEST.json").write_text(json.dumps({"modules": digests}, indent=1, sort_keys=True) + "\n")
    return dest


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--reference", default=os.environ.get("GAC_REFERENCE"), required="GAC_REFERENCE" not in os.environ,
                    help="checkout of the reference project; default: $GAC_REFERENCE")
    args = ap.parse_args()
    print(make_ref(Path(args.reference)))


if __name__ == "__main__":
    sys.exit(main())
