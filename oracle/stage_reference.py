"""Stage the UNMODIFIED reference implementation (skywong14/htree) under oracle/_ref/.  TEST INFRASTRUCTURE ONLY.

    python oracle/stage_reference.py [path-to-reference-checkout]

The reference is pure Python + Triton JIT: there is nothing to compile, so "building" it for a machine that has no
checkout means placing byte-identical copies of the files of the operator's path (src/parallel.py, src/backward.py,
src/naive.py) and of its NSA comparison baseline (ref_nsa/) in oracle/_ref/, which version control ignores.  Nothing
is edited; MANIFEST.json records the SHA-256 of every staged file so that a run can state which bytes it executed.
Only tests and the baseline legs of the benchmark load these files (through oracle/ref_triton.py); the product
package never does.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
# the checkout: $HTREE_REFERENCE, else a directory named "reference" beside this repository
DEFAULT_SOURCE = os.environ.get("HTREE_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
FILES = ["src/parallel.py", "src/backward.py", "src/naive.py",
         "ref_nsa/__init__.py", "ref_nsa/nsa_parallel.py", "ref_nsa/nsa_compression.py", "ref_nsa/nsa_utils.py"]


def _sha(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def stage(source: str = DEFAULT_SOURCE, dest: str = DEST) -> bool:
    """Copy the files when `source` exists; returns whether oracle/_ref/ is populated afterwards."""
    manifest = os.path.join(dest, "MANIFEST.json")
    if not os.path.isdir(source):
        return os.path.exists(manifest)
    sums = {}
    for rel in FILES:
        src = os.path.join(source, rel)
        if not os.path.exists(src):
            continue
        dst = os.path.join(dest, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if not os.path.exists(dst) or _sha(dst) != _sha(src):
            shutil.copyfile(src, dst)
            os.chmod(dst, 0o644)
        sums[rel] = _sha(dst)
    with open(manifest, "w") as f:
        json.dump({"files": sums}, f, indent=1, sort_keys=True)
    return True


def verify(dest: str = DEST) -> bool:
    """True iff every staged file still has the digest recorded when it was copied."""
    manifest = os.path.join(dest, "MANIFEST.json")
    if not os.path.exists(manifest):
        return False
    with open(manifest) as f:
        sums = json.load(f)["files"]
    return all(os.path.exists(os.path.join(dest, rel)) and _sha(os.path.join(dest, rel)) == s for rel, s in sums.items())


if __name__ == "__main__":
    ok = stage(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_SOURCE)
    print("oracle/_ref staged" if ok else "no reference checkout found; oracle/_ref left empty")
