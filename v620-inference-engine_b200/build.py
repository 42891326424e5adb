"""Build every native component in-tree: ``python -m qwb200.build [--force] [--verbose]``."""
import argparse
import sys

from .ops import lib as qlib


def build_all(force: bool = False, verbose: bool = False) -> None:
    path = qlib.build(force=force, verbose=verbose)
    print("built", path)
    print("built", qlib.build(force=force, verbose=verbose, checked=True))
    try:
        from .native import build as nbuild
        nbuild.build(force=force, verbose=verbose)
    except ImportError:
        pass


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    sys.exit(0)
