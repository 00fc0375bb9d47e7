"""python -m ninfer_fusion_b200.archkit adapt MODEL_ID config.json | matrix --model ID | import PATH"""
from __future__ import annotations

import argparse
import json
import sys

from ..models.config import get_config
from . import adapt_config, budget_matrix, geometry_gates


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="archkit")
    sub = ap.add_subparsers(dest="cmd", required=True)
    a = sub.add_parser("adapt", help="config.json -> package description and the capability gate's verdict")
    a.add_argument("model_id"); a.add_argument("config")
    a.add_argument("--world", type=int, default=1); a.add_argument("--weights", default="bf16")
    m = sub.add_parser("matrix", help="GPU budget matrix of a registered model")
    m.add_argument("--model", default="qwen3.6-27b"); m.add_argument("--world", type=int, default=1)
    m.add_argument("--batch", type=int, default=1)
    i = sub.add_parser("import", help="what is this path, can it be served, what fits on which GPU, how to start it")
    i.add_argument("path")
    i.add_argument("--gpu", default="b200"); i.add_argument("--context", type=int, default=32768)
    i.add_argument("--lanes", type=int, default=8); i.add_argument("--world", type=int, default=1)
    args = ap.parse_args(argv)
    if args.cmd == "import":
        from .model_import import advise
        out = advise(args.path, args.gpu, args.context, args.lanes, args.world)
        print(json.dumps(out, indent=1))
        return 0 if str(out.get("verdict", "")).startswith(("servable", "convert first")) else 1
    if args.cmd == "adapt":
        with open(args.config, encoding="utf-8") as f:
            desc = adapt_config(args.model_id, json.load(f))
        desc["gates"] = geometry_gates(desc, args.world, args.weights)
        table = desc.pop("layer_table")
        print(json.dumps(desc))
        print(json.dumps({"layer_table": table}))
        return 0 if desc["servable"] and not desc["gates"] else 1
    for row in budget_matrix(get_config(args.model), args.world, args.batch):
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    sys.exit(main())
