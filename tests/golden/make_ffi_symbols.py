"""Generates tests/golden/ffi_symbols.txt: every `wst_*` function the engine's Rust
crate declares in crates/whetstone-kernels/src/ffi.rs, one per line, sorted -- the
symbols a library that replaces the engine's kernel library must export.

    python tests/golden/make_ffi_symbols.py <path of the reference checkout>

(default: the directory ``reference`` beside this repository).  The checkout cannot
travel with this repository, so the list is committed; tests/test_dropin_link.py
checks the linked drop-in library against it.
"""

from __future__ import annotations

import re
import sys
from pathlib import Path


def main() -> None:
    here = Path(__file__).resolve().parent
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else here.parents[2] / "reference"
    text = (root / "crates" / "whetstone-kernels" / "src" / "ffi.rs").read_text()
    names = sorted(set(re.findall(r"\bfn\s+(wst_[a-z0-9_]+)\s*\(", text)))
    (here / "ffi_symbols.txt").write_text("\n".join(names) + "\n")
    print(f"{len(names)} symbols")


if __name__ == "__main__":
    main()
