"""Builds ``oracle/_ref``: the reference project's own Python, byte-compiled (TEST INFRASTRUCTURE).

    python oracle/build_ref.py /path/to/ml-flashpoint

Every ``*.py`` under ``<reference root>/src/ml_flashpoint`` is compiled where it lies with
``py_compile`` and only the resulting sourceless bytecode is kept, packed into one archive,
``oracle/_ref/reference_bytecode.zip``, that mirrors the package tree (Python imports sourceless
``.pyc`` files straight from a zip on ``sys.path``). No reference source is copied. ``oracle/_ref``
is a build output: it is ignored by git and rebuilt from a reference checkout by this recipe.

The two compiled extension modules of the reference (``buffer_object_ext``, ``transfer_service_ext``)
cannot be built offline (their CMake build fetches abseil and googletest); ``ref_arm.py`` registers
stand-ins for them, so every line that moves or formats checkpoint bytes is the reference's own.

``manifest.json`` records the interpreter's bytecode magic, the torch version and the SHA-256 of
every source file compiled, so that a stale or foreign build is recognised at load time.
"""

from __future__ import annotations

import hashlib
import importlib.util
import json
import os
import py_compile
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# a checkout of the reference project next to this repository, unless MLF_REFERENCE_ROOT names another place
DEFAULT_REFERENCE_ROOT = os.environ.get("MLF_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def reference_available(ref_root: str = DEFAULT_REFERENCE_ROOT) -> bool:
    return os.path.isfile(os.path.join(ref_root, "src", "ml_flashpoint", "__init__.py"))


def _sources(ref_root: str):
    base = os.path.join(ref_root, "src", "ml_flashpoint")
    for folder, _, files in sorted(os.walk(base)):
        for name in sorted(files):
            if name.endswith(".py"):
                path = os.path.join(folder, name)
                yield path, os.path.relpath(path, os.path.join(ref_root, "src"))


def _sha(path: str) -> str:
    with open(path, "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def is_current(ref_root: str = DEFAULT_REFERENCE_ROOT) -> bool:
    """True when ``oracle/_ref`` was built by this interpreter from exactly these sources."""
    try:
        with open(os.path.join(OUT, "manifest.json")) as f:
            manifest = json.load(f)
    except (OSError, ValueError):
        return False
    if manifest.get("magic") != importlib.util.MAGIC_NUMBER.hex():
        return False
    want = {rel: _sha(path) for path, rel in _sources(ref_root)}
    return want == manifest.get("sources")


ARCHIVE = os.path.join(OUT, "reference_bytecode.zip")


def build(ref_root: str = DEFAULT_REFERENCE_ROOT, force: bool = False) -> str:
    import tempfile
    import zipfile

    if not reference_available(ref_root):
        raise FileNotFoundError(f"no reference checkout at {ref_root} (expected src/ml_flashpoint/__init__.py)")
    if not force and is_current(ref_root) and os.path.isfile(ARCHIVE):
        return OUT
    shutil.rmtree(OUT, ignore_errors=True)
    os.makedirs(OUT)
    hashes = {}
    src_root = os.path.join(ref_root, "src")
    with tempfile.TemporaryDirectory() as scratch, zipfile.ZipFile(ARCHIVE, "w", zipfile.ZIP_STORED) as archive:
        # directories that hold only compiled extensions are still packages the Python side imports
        # from (namespace packages): every directory of the tree gets an entry, Python or not
        for folder, _, _ in sorted(os.walk(os.path.join(src_root, "ml_flashpoint"))):
            archive.writestr(zipfile.ZipInfo(os.path.relpath(folder, src_root) + "/"), b"")
        for path, rel in _sources(ref_root):
            compiled = os.path.join(scratch, "module.pyc")
            py_compile.compile(
                path,
                cfile=compiled,
                dfile=os.path.join("<reference>", rel),
                doraise=True,
                invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH,
            )
            archive.write(compiled, rel + "c")  # pkg/mod.py -> pkg/mod.pyc, importable without the source
            hashes[rel] = _sha(path)
    import torch

    manifest = {
        "what": "byte-compiled reference package (ml_flashpoint), no sources",
        "archive": os.path.basename(ARCHIVE),
        "magic": importlib.util.MAGIC_NUMBER.hex(),
        "python": sys.version.split()[0],
        "torch": torch.__version__,
        "sources": hashes,
    }
    with open(os.path.join(OUT, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    return OUT


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else DEFAULT_REFERENCE_ROOT
    print(build(root, force=True))
