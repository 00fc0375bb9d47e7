"""python -m ninfer_fusion_b200.eval run SUITE.yaml --out DIR"""
import argparse
import json
import sys

from .coordinator import run_suite


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ninfer_fusion_b200.eval")
    sub = ap.add_subparsers(dest="cmd", required=True)
    r = sub.add_parser("run", help="run every job of a suite")
    r.add_argument("suite")
    r.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    print(json.dumps(run_suite(a.suite, a.out), indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
