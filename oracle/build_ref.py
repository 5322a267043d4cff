"""Recipe that places the reference's own pure-Python recurrence under ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY (the checker and the timed CPU baseline; never the product path).

The reference implementation of this path (0z5a/flashrnn) is three torch-only modules:
``flashrnn/flashrnn2/torch_backend.py`` (``flashrnn_torch``), ``reference.py`` (``recurrence``) and
``state_contract.py``. They need no build; this script copies them, unmodified, from a checkout of the
reference into ``oracle/_ref/flashrnn2_ref/`` so that they can be imported without the rest of the
reference package (whose ``__init__`` pulls in its CUDA JIT machinery). ``oracle/_ref/`` is a build
output: it is not tracked by git and nothing in the product imports it.

    python oracle/build_ref.py [path-to-reference-checkout]
"""

from __future__ import annotations

import hashlib
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "flashrnn2_ref"
FILES = ("torch_backend.py", "reference.py", "state_contract.py")
DEFAULT_CHECKOUT = Path("/root/reference")


def build_ref(checkout: Path = DEFAULT_CHECKOUT) -> bool:
    """Copy the modules; returns False (and changes nothing) when the checkout is absent."""
    src = Path(checkout) / "flashrnn" / "flashrnn2"
    if not all((src / f).exists() for f in FILES):
        return False
    OUT.mkdir(parents=True, exist_ok=True)
    (OUT.parent / "__init__.py").write_text("")
    (OUT / "__init__.py").write_text('"""Unmodified copy of the reference modules listed in SOURCES.txt."""\n')
    lines = []
    for f in FILES:
        shutil.copyfile(src / f, OUT / f)
        lines.append(f"{hashlib.sha256((OUT / f).read_bytes()).hexdigest()}  flashrnn/flashrnn2/{f}")
    (OUT / "SOURCES.txt").write_text("\n".join(lines) + "\n")
    return True


def load_reference():
    """Return the reference's ``flashrnn_torch`` from ``oracle/_ref`` or None when it was not built."""
    if not (OUT / "torch_backend.py").exists():
        return None
    root = str(HERE.parent)
    if root not in sys.path:
        sys.path.insert(0, root)
    from oracle._ref.flashrnn2_ref.torch_backend import flashrnn_torch

    return flashrnn_torch


if __name__ == "__main__":
    ok = build_ref(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    print("oracle/_ref built" if ok else "reference checkout not found: nothing built")
