"""Reference arm of the benchmark: the unmodified reference package from ``baseline/_ref``."""
import json
import os
import sys


def run(args) -> None:
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    rank = int(os.environ.get("RANK", 0))
    if not os.path.isdir(os.path.join(ref, "autoparallel")):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}))
        return
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}))
