"""Put the UNMODIFIED reference packages next to the oracle so that they travel with a snapshot of this tree.

    python oracle/make_ref.py [/path/to/the/reference/checkout]      # default: $HQMQ_REFERENCE_CHECKOUT

The reference (kswain98/hqmq) is pure Python: its ``hqmq`` and ``src`` packages are installed, file for file,
under ``oracle/_ref/`` (git-ignored: nothing of it enters the history of this repository).  ``bench.py`` times
them as the CPU baseline and as the incumbent GPU kernel when the directory exists, and says so when it does
not.  Test infrastructure only: nothing under ``hqmq_b200/`` imports it.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PACKAGES = ("hqmq", "src")
# where a checkout of the reference lives on the build host (overridable; absent on the machines that only run)
CHECKOUT = os.environ.get("HQMQ_REFERENCE_CHECKOUT", os.path.join(os.sep, "root", "reference"))


def checkout_present(ref_root: str = CHECKOUT) -> bool:
    return all(os.path.isdir(os.path.join(ref_root, p)) for p in PACKAGES)


def install(ref_root: str = CHECKOUT) -> str:
    if not all(os.path.isdir(os.path.join(ref_root, p)) for p in PACKAGES):
        raise FileNotFoundError(f"no reference checkout at {ref_root}")
    os.makedirs(DEST, exist_ok=True)
    for p in PACKAGES:
        dst = os.path.join(DEST, p)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(ref_root, p), dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DEST


def available() -> bool:
    return all(os.path.isfile(os.path.join(DEST, p, "__init__.py")) for p in PACKAGES)


def import_reference():
    """The reference's public package (``hqmq``), imported from oracle/_ref."""
    if not available():
        raise ImportError("oracle/_ref is absent: run `python oracle/make_ref.py` where the reference checkout exists")
    if DEST not in sys.path:
        sys.path.insert(0, DEST)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")       # the reference's hqmq_padded.py has an invalid escape in a docstring
        import hqmq
    return hqmq


if __name__ == "__main__":
    print(install(sys.argv[1] if len(sys.argv) > 1 else CHECKOUT))
