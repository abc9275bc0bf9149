"""Probe child.  Without arguments: prints one JSON line ``{"devices": [...]}`` describing the CUDA devices it can see.
``--validate``: the parent made exactly one device visible; create a context on it, allocate, compute, read back, and print
``{"ok": true, "free_memory": N}`` - or ``{"ok": false, "error": ...}``; a crash or a hang is the parent's answer too."""
from __future__ import annotations

import json
import sys


def validate() -> dict:
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 1:
        return {"ok": False, "error": "no CUDA device visible"}
    major, _ = torch.cuda.get_device_capability(0)
    if major < 10:
        return {"ok": False, "error": f"compute capability {major}.x is older than sm_100"}
    x = torch.arange(1024, device="cuda:0", dtype=torch.float32)
    total = float((x * 2).sum().item())                 # a context, an allocation, a kernel and a copy back
    if total != 1023.0 * 1024.0:
        return {"ok": False, "error": f"device arithmetic is wrong ({total})"}
    free, _ = torch.cuda.mem_get_info(0)
    return {"ok": True, "free_memory": int(free)}


def main(argv: list[str] | None = None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    try:
        if "--validate" in argv:
            print(json.dumps(validate()))
            return 0
        from .devices import probe_in_process
        devs = [d.to_json() for d in probe_in_process()]
    except Exception as e:  # the parent treats any failure as "no usable GPU"
        print(json.dumps({"devices": [], "ok": False, "error": str(e)}))
        return 0
    print(json.dumps({"devices": devs}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
