"""Recipe for oracle/_ref: a byte-for-byte copy of the reference's model.py.

TEST INFRASTRUCTURE ONLY. The reference is one pure-Python file with nothing to
compile, so "building" it means placing the unmodified file where the GPU box
can import it: oracle/_ref/ is git-ignored (the copy never enters the history)
but travels with the working tree. The copy gives

  - the CPU arm of bench.py the reference's own classes (model.MOE,
    model.py:192-276) instead of the restatement in moe_oracle.py, and
  - the decoder test and bench the reference's own LLM (model.py:322-372) to
    swap the new block into.

    python oracle/make_ref.py [/path/to/GemmaLLM]

Without an argument the reference checkout is looked for next to this
repository or where $MOE_REFERENCE_DIR points. Where none is found nothing is
written and an existing copy is kept.
"""
from __future__ import annotations

import hashlib
import importlib.util
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF_OUT = HERE / "_ref"
MODULE_NAME = "gemmallm_reference_model"


def reference_dir(arg: str | None = None) -> Path | None:
    for cand in (arg, os.environ.get("MOE_REFERENCE_DIR"), HERE.parent.parent / "reference"):
        if cand and Path(cand, "model.py").exists():
            return Path(cand)
    return None


def make(arg: str | None = None) -> Path | None:
    """Copy model.py into oracle/_ref/ and record its SHA-256. Returns the copy's
    path, or None when there is no reference checkout here."""
    src_dir = reference_dir(arg)
    if src_dir is None:
        return REF_OUT / "model.py" if (REF_OUT / "model.py").exists() else None
    data = (src_dir / "model.py").read_bytes()
    REF_OUT.mkdir(exist_ok=True)
    dst = REF_OUT / "model.py"
    if not dst.exists() or dst.read_bytes() != data:
        dst.write_bytes(data)
    (REF_OUT / "SOURCE.txt").write_text(
        f"model.py: unmodified copy of the reference's model.py\nsha256 {hashlib.sha256(data).hexdigest()}\n")
    return dst


def available() -> bool:
    return (REF_OUT / "model.py").exists()


def load():
    """Import oracle/_ref/model.py (the reference's module, unmodified) under a private
    module name. Raises FileNotFoundError when the copy is absent."""
    if MODULE_NAME in sys.modules:
        return sys.modules[MODULE_NAME]
    path = REF_OUT / "model.py"
    if not path.exists():
        raise FileNotFoundError(f"{path} is missing: run oracle/make_ref.py where the reference is checked out")
    spec = importlib.util.spec_from_file_location(MODULE_NAME, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[MODULE_NAME] = mod
    try:
        spec.loader.exec_module(mod)
    except Exception:
        del sys.modules[MODULE_NAME]
        raise
    return mod


if __name__ == "__main__":
    out = make(sys.argv[1] if len(sys.argv) > 1 else None)
    print(out if out else "no reference checkout found; nothing written")
