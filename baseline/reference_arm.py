"""Runs the unmodified reference (installed under ``baseline/_ref``) on the
headline configuration and prints the same JSON line as ``bench.py``."""
from __future__ import annotations

import json
from argparse import Namespace


def run_reference_arm(args: Namespace) -> None:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}), flush=True)
