"""``python -m fairseq2_b200.assets list|show NAME`` (cf. fairseq2 ``assets/cli.py:26-219``)."""
from __future__ import annotations

import argparse
import sys

from fairseq2_b200.assets.store import AssetNotFoundError, get_asset_store
from fairseq2_b200.utils.yaml import dump_yaml


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="fairseq2_b200.assets")
    sub = ap.add_subparsers(dest="cmd", required=True)
    ls = sub.add_parser("list", help="list asset names")
    ls.add_argument("--kind", choices=["model", "tokenizer", "dataset", "all"], default="all")
    sh = sub.add_parser("show", help="show an asset card")
    sh.add_argument("name")
    args = ap.parse_args(argv)
    store = get_asset_store()
    if args.cmd == "list":
        for n in store.retrieve_names():
            card = store.retrieve_card(n)
            kind = "model" if card.has_field("model_family") else "tokenizer" if card.has_field("tokenizer_family") \
                else "dataset" if card.has_field("dataset_family") else "other"
            if args.kind in ("all", kind):
                print(f"{kind:10s} {n}")
        return 0
    try:
        card = store.retrieve_card(args.name)
    except AssetNotFoundError as ex:
        print(str(ex), file=sys.stderr)
        return 1
    md = {k: v for k, v in card.flatten().items() if not k.startswith("__")}
    print(dump_yaml(md), end="")
    return 0
