"""Recipe for ``oracle/_ref``: the reference's own Python package, placed where the CPU baseline arm of
``bench.py`` can import it on a machine that has no reference checkout.

    python oracle/make_ref.py [--reference /path/to/segment-anything-fast]

TEST / MEASUREMENT INFRASTRUCTURE ONLY.  The reference is a pure-Python project, so "building" it means making
its package directory importable: this script copies ``<reference>/segment_anything_fast`` (unmodified) to
``oracle/_ref/segment_anything_fast``.  ``oracle/_ref/`` is listed in ``.gitignore`` and never committed; nothing
under ``segment_anything_fast_b200/`` imports it.  ``bench.py --impl reference`` (and the ``cpu_baseline`` leg of
the default run) import it with ``SEGMENT_ANYTHING_FAST_USE_FLASH_4=0``, i.e. the reference's own CPU path
(SDPA composite, flash_4.py:347-348,368-370), and time ``sam_model_registry['vit_h']().image_encoder``.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
# where the reference checkout sits on the build machine: $SAMB_REFERENCE_DIR, else ~/reference
DEFAULT_REFERENCE = os.environ.get("SAMB_REFERENCE_DIR", os.path.join(os.path.expanduser("~"), "reference"))


def make_ref(reference: str = DEFAULT_REFERENCE, quiet: bool = False) -> bool:
    """Returns True when ``oracle/_ref/segment_anything_fast`` exists afterwards."""
    src = os.path.join(reference, "segment_anything_fast")
    dst = os.path.join(REF_DIR, "segment_anything_fast")
    if not os.path.isdir(src):
        if not quiet:
            print(f"no reference package at {src}; leaving {REF_DIR} as it is")
        return os.path.isdir(dst)
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    if not quiet:
        print(f"copied {src} -> {dst}")
    return True


def import_ref():
    """Import the reference package from ``oracle/_ref`` (CPU path).  Raises ImportError when it is not there."""
    if not os.path.isdir(os.path.join(REF_DIR, "segment_anything_fast")):
        raise ImportError("oracle/_ref/segment_anything_fast is missing (run oracle/make_ref.py where the reference checkout is)")
    os.environ["SEGMENT_ANYTHING_FAST_USE_FLASH_4"] = "0"
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import segment_anything_fast
    return segment_anything_fast


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ok = make_ref(ap.parse_args().reference)
    sys.exit(0 if ok else 1)
