"""Puts the reference project's own CPU oracles next to the port, for timing and cross-checks.

    python oracle/make_ref.py --reference /path/to/reference/checkout

The reference's CPU implementation of the path is four pure-torch files under its reference/ folder
(fixed_route_attention.py, grouped_reference.py, decode_reference.py, merge_reference.py).  This recipe
copies them, unmodified, from the checkout into oracle/_ref/reference/, a folder that version control
ignores: nothing of the reference is ever committed here.  The benchmark's CPU arm imports them from
there when they are present (and says kind = "reference"), and falls back to the numpy port in
oracle/moba_oracle.py when they are not (kind = "port").
"""
import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
FILES = ("__init__.py", "fixed_route_attention.py", "grouped_reference.py", "decode_reference.py", "merge_reference.py")


def make_ref(reference_root, out_dir=HERE / "_ref"):
    """Returns the folder that holds the copies, or None when the checkout is not there."""
    src = Path(reference_root) / "reference"
    if not all((src / name).exists() for name in FILES):
        return None
    dst = Path(out_dir) / "reference"
    dst.mkdir(parents=True, exist_ok=True)
    for name in FILES:
        shutil.copyfile(src / name, dst / name)
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


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    print(make_ref(ap.parse_args().reference))
