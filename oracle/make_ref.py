"""Puts the reference project's own CPU oracles next to the port, for timing and cross-checks.

    python oracle/make_ref.py --reference /path/to/reference/checkout

The reference's CPU implementation of the path is four pure-torch files under its reference/ folder
(fixed_route_attention.py, grouped_reference.py, decode_reference.py, merge_reference.py).  This recipe
copies them, unmodified, from the checkout into oracle/_ref/reference/, a folder that version control
ignores: nothing of the reference is ever committed here.  The benchmark's CPU arm imports them from
there when they are present (and says kind = "reference"), and falls back to the numpy port in
oracle/moba_oracle.py when they are not (kind = "port").

The reference's decode side (src/moba_opt/kv_cache.py, prepared_decode.py, cache_layout.py and the
Triton kernels ops/paged_decode.py, ops/prepared_decode.py) needs only torch and triton, unlike its
prefill side.  The same recipe copies those five files, unmodified, into oracle/_ref/moba_opt_decode/;
`load_ref_decode` imports them as a package of their own (the reference's package __init__ is left out,
because it imports the prefill side).  On a GPU they give the reference's own decode results for the
same inputs: a cross-check for the tests and a same-machine baseline for the benchmark's decode leg.
"""
import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
FILES = ("__init__.py", "fixed_route_attention.py", "grouped_reference.py", "decode_reference.py", "merge_reference.py")
DECODE_FILES = ("kv_cache.py", "prepared_decode.py", "cache_layout.py", "ops/paged_decode.py", "ops/prepared_decode.py")
DECODE_PACKAGE = "moba_opt_decode"


def make_ref(reference_root, out_dir=HERE / "_ref"):
    """Returns the folder that holds the copies, or None when the checkout is not there."""
    src = Path(reference_root) / "reference"
    if not all((src / name).exists() for name in FILES):
        return None
    dst = Path(out_dir) / "reference"
    dst.mkdir(parents=True, exist_ok=True)
    for name in FILES:
        shutil.copyfile(src / name, dst / name)
    pkg = Path(reference_root) / "src" / "moba_opt"
    if all((pkg / name).exists() for name in DECODE_FILES):
        out = Path(out_dir) / DECODE_PACKAGE
        (out / "ops").mkdir(parents=True, exist_ok=True)
        for name in DECODE_FILES:
            shutil.copyfile(pkg / name, out / name)
    return dst


def load_ref(out_dir=HERE / "_ref"):
    """(grouped_reference, decode_reference) imported from oracle/_ref, or None when make_ref has not run."""
    root = Path(out_dir)
    if not all((root / "reference" / name).exists() for name in FILES):
        return None
    sys.path.insert(0, str(root))
    try:
        sys.modules.pop("reference", None)
        from reference.decode_reference import decode_reference
        from reference.grouped_reference import grouped_reference
    finally:
        sys.path.remove(str(root))
    return grouped_reference, decode_reference


def load_ref_decode(out_dir=HERE / "_ref"):
    """The reference's decode modules (kv_cache with PagedKVCache / ContiguousKVCache, prepared_decode) imported from
    oracle/_ref as the package `moba_opt_decode`, or None when make_ref has not copied them or triton is missing."""
    import importlib
    import importlib.util
    import types
    root = Path(out_dir) / DECODE_PACKAGE
    if not all((root / name).exists() for name in DECODE_FILES) or importlib.util.find_spec("triton") is None:
        return None
    if DECODE_PACKAGE not in sys.modules:
        for name, path in ((DECODE_PACKAGE, root), (DECODE_PACKAGE + ".ops", root / "ops")):
            pkg = types.ModuleType(name)
            pkg.__path__ = [str(path)]          # a package without an __init__: submodules import each other relatively
            sys.modules[name] = pkg
    return importlib.import_module(DECODE_PACKAGE + ".kv_cache"), importlib.import_module(DECODE_PACKAGE + ".prepared_decode")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    print(make_ref(ap.parse_args().reference))
