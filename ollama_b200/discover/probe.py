"""Probe child: prints one JSON line ``{"devices": [...]}`` describing the CUDA devices it can see."""
from __future__ import annotations

import json
import sys


def main() -> int:
    try:
        from .devices import probe_in_process
        devs = [d.to_json() for d in probe_in_process()]
    except Exception as e:  # the parent treats any failure as "no usable GPU"
        print(json.dumps({"devices": [], "error": str(e)}))
        return 0
    print(json.dumps({"devices": devs}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
