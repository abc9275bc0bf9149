"""GPU discovery and memory accounting types.

``DeviceInfo`` carries what the scheduler needs (id, name, compute capability, total / free memory,
driver) -- the fields of the reference's ``ml.DeviceInfo`` (ml/device.go:277-331).  Discovery itself
runs in a child process (``python -m ollama_b200.discover.probe`` or the C++ ``devquery`` helper) so
that a driver fault cannot take the server down, which is the reason the reference probes through
short-lived children as well (discover/native_probe.go:19-23, 69-106).  Free memory reported to the
scheduler is the minimum of what the driver reports and what the loaded runners account for
(discover/runner.go:266-367).
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from dataclasses import asdict, dataclass

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


def gpu_devices(timeout: float = 30.0) -> list[DeviceInfo]:
    """Run the probe child and parse its JSON; an unresponsive or crashing probe means "no GPUs"."""
    native = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "native", "devquery")
    cmds = ([[native]] if os.path.exists(native) else []) + [[sys.executable, "-m", "ollama_b200.discover.probe"]]
    for cmd in cmds:
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout,
                               env={**os.environ, "PYTHONPATH": os.pathsep.join(sys.path)})
            if r.returncode != 0:
                continue
            data = json.loads(r.stdout.strip().splitlines()[-1])
            devs = [DeviceInfo(**d) for d in data.get("devices", [])]
            return filter_devices(devs)
        except (subprocess.TimeoutExpired, OSError, ValueError, IndexError, TypeError):
            continue
    return []


def filter_devices(devs: list[DeviceInfo]) -> list[DeviceInfo]:
    """Honour CUDA_VISIBLE_DEVICES-style ordering already applied by the driver; drop integrated GPUs and devices older than sm_100."""
    return [d for d in devs if not d.integrated and d.compute_major >= 10]
