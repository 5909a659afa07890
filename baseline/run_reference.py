"""Reference arm of bench.py (filled in by the baseline harness)."""
import json
import os


def run_reference(args) -> dict:
    if int(os.environ.get("RANK", "0")) != 0:
        return {}
    return {"impl": "reference", "unavailable": "reference harness not built yet"}
