"""GPU discovery and memory accounting types.

``DeviceInfo`` carries what the scheduler needs (id, name, compute capability, total / free memory,
driver) -- the fields of the reference's ``ml.DeviceInfo`` (ml/device.go:277-331).  Discovery itself
runs in a child process (``python -m ollama_b200.discover.probe`` or the C++ ``devquery`` helper) so
that a driver fault cannot take the server down, which is the reason the reference probes through
short-lived children as well (discover/native_probe.go:19-23, 69-106).  Free memory reported to the
scheduler is the minimum of what the driver reports and what the loaded runners account for
(discover/runner.go:266-367).

Discovery has two passes, like the reference's (discover/runner.go:128-180).  The first lists what the driver
enumerates without creating a context.  The second starts one more child per listed device, with only that device
visible, which creates a context on it and runs a few device operations; a device whose child crashes, hangs or reports
an error is dropped, so that a GPU that enumerates but cannot run (fallen off the bus, an unsupported driver pairing,
held exclusively by another process) never reaches the scheduler.  ``devices_env`` builds the environment that makes a
runner's children see exactly the devices chosen for them (ml/device.go:631-660); ``flash_attention_supported`` is the
predicate of ml/device.go:569-600 for the one family this engine targets.
"""
from __future__ import annotations

import concurrent.futures as cf
import json
import logging
import os
import subprocess
import sys
from dataclasses import asdict, dataclass
from typing import Callable

log = logging.getLogger("ollama_b200.discover")

GPU_OVERHEAD_DEFAULT = 457 << 20     # bytes reserved per device on top of OLLAMA_GPU_OVERHEAD (ml/device.go:359-364)


@dataclass
class DeviceInfo:
    id: str = "0"
    index: int = 0
    library: str = "cuda"
    name: str = ""
    compute_major: int = 0
    compute_minor: int = 0
    total_memory: int = 0
    free_memory: int = 0
    driver: str = ""
    pci_id: str = ""
    integrated: bool = False

    @property
    def compute(self) -> str:
        return f"{self.compute_major}.{self.compute_minor}"

    def to_json(self) -> dict:
        return asdict(self)


@dataclass
class SystemInfo:
    total_memory: int = 0
    free_memory: int = 0
    threads: int = 0


def system_info() -> SystemInfo:
    try:
        import psutil
        vm = psutil.virtual_memory()
        return SystemInfo(int(vm.total), int(vm.available), os.cpu_count() or 1)
    except Exception:
        return SystemInfo(0, 0, os.cpu_count() or 1)


def probe_in_process() -> list[DeviceInfo]:
    """Enumerate CUDA devices through torch (used inside the probe child)."""
    import torch
    out: list[DeviceInfo] = []
    if not torch.cuda.is_available():
        return out
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        out.append(DeviceInfo(id=f"GPU-{i}", index=i, name=p.name, compute_major=p.major, compute_minor=p.minor,
                              total_memory=int(total), free_memory=int(free), driver=str(torch.version.cuda or ""),
                              pci_id=getattr(p, "pci_bus_id", "") and f"{p.pci_bus_id:02x}" or "", integrated=bool(getattr(p, "is_integrated", 0))))
    return out


def _run_child(cmd: list[str], env: dict[str, str], timeout: float) -> dict | None:
    """One probe child: its last stdout line as JSON, or None when it failed, crashed or ran out of time."""
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
        if r.returncode != 0:
            return None
        return json.loads(r.stdout.strip().splitlines()[-1])
    except (subprocess.TimeoutExpired, OSError, ValueError, IndexError, TypeError):
        return None


def devices_env(devs: list[DeviceInfo], base: dict[str, str] | None = None) -> dict[str, str]:
    """Environment in which a child process sees exactly ``devs``, in this order (ml/device.go:631-660): the driver-level
    selector is set to their ids (UUIDs where known, else indices), the enumeration order is pinned to the bus order the
    indices refer to.  An empty list hides every GPU."""
    env = dict(os.environ if base is None else base)
    outer = [x.strip() for x in env.get("CUDA_VISIBLE_DEVICES", "").split(",") if x.strip()]

    def selector(d: DeviceInfo) -> str:
        if d.id.startswith("GPU-") and len(d.id) > 8:
            return d.id                                # a UUID names the device whatever is visible now
        # an index counts within what this process sees: translate it through the selector already in force
        return outer[d.index] if d.index < len(outer) else str(d.index)

    ids = [selector(d) for d in devs]
    env["CUDA_VISIBLE_DEVICES"] = ",".join(ids) if devs else "-1"
    env["CUDA_DEVICE_ORDER"] = "PCI_BUS_ID"
    return env


def flash_attention_supported(devs: list[DeviceInfo]) -> bool:
    """ml/device.go:569-600: every selected device has to support the fused attention kernels; for this engine that means
    the sm_100 family its kernels are compiled for.  No devices (CPU execution) counts as supported."""
    return all(d.library == "cpu" or (d.library == "cuda" and d.compute_major >= 10) for d in devs)


def validate_devices(devs: list[DeviceInfo], timeout: float = 30.0, run_child: Callable[[list[str], dict[str, str], float], dict | None] = _run_child,
                     base_env: dict[str, str] | None = None) -> list[DeviceInfo]:
    """Second pass: one child per device, all at once, each seeing only its device; keep the devices whose child answered
    ``{"ok": true}``.  Free memory reported by a child that did answer replaces the first pass's figure."""
    if not devs:
        return []
    cmd = [sys.executable, "-m", "ollama_b200.discover.probe", "--validate"]

    def check(d: DeviceInfo) -> DeviceInfo | None:
        env = devices_env([d], base_env)
        env["PYTHONPATH"] = os.pathsep.join(sys.path)
        ans = run_child(cmd, env, timeout)
        if not ans or not ans.get("ok"):
            log.warning("dropping GPU %s (%s): it did not initialise (%s)", d.id, d.name, (ans or {}).get("error", "no answer"))
            return None
        if ans.get("free_memory"):
            d.free_memory = int(ans["free_memory"])
        return d

    with cf.ThreadPoolExecutor(max_workers=len(devs)) as ex:
        return [d for d in ex.map(check, devs) if d is not None]


def gpu_devices(timeout: float = 30.0, validate: bool | None = None) -> list[DeviceInfo]:
    """Run the probe child and parse its JSON; an unresponsive or crashing probe means "no GPUs".  ``validate`` (default: on
    unless ``B200_DISCOVERY_VALIDATE=0``) adds the second pass on the first call of a process; later calls only refresh the
    memory figures of devices that passed."""
    native = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "native", "devquery")
    cmds = ([[native]] if os.path.exists(native) else []) + [[sys.executable, "-m", "ollama_b200.discover.probe"]]
    if validate is None:
        validate = os.environ.get("B200_DISCOVERY_VALIDATE", "1") != "0"
    for cmd in cmds:
        data = _run_child(cmd, {**os.environ, "PYTHONPATH": os.pathsep.join(sys.path)}, timeout)
        if data is None:
            continue
        try:
            devs = filter_devices([DeviceInfo(**d) for d in data.get("devices", [])])
        except TypeError:
            continue
        if validate and devs:
            known = _validated.get("ids")
            if known is None:
                devs = validate_devices(devs, timeout)
                _validated["ids"] = {d.id for d in devs}
            else:
                devs = [d for d in devs if d.id in known]
        return devs
    return []


_validated: dict[str, set[str] | None] = {"ids": None}      # ids that passed the second pass in this process


def filter_devices(devs: list[DeviceInfo]) -> list[DeviceInfo]:
    """Honour CUDA_VISIBLE_DEVICES-style ordering already applied by the driver; drop integrated GPUs and devices older than sm_100."""
    return [d for d in devs if not d.integrated and d.compute_major >= 10]
