"""Generates tests/golden/failure_golden.json: what the REFERENCE library (oracle/_ref) returns,
call by call, on the hostile artifacts and adapters of failure_cases.py.

    python tests/golden/make_failure_golden.py
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
from oracle import harness as H  # noqa: E402
import failure_cases as F  # noqa: E402


def main():
    lib = H.ref()
    assert lib is not None, "build oracle/_ref first (make -C oracle ref)"
    rec = F.all_records(lib)
    json.dump(rec, open(os.path.join(HERE, "failure_golden.json"), "w"), indent=1)
    for k, v in rec.items():
        print(k, [(r[0], r[1]) for r in v])


if __name__ == "__main__":
    main()
