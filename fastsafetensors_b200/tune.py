"""Reader settings derived from the host: how many worker threads, how much pinned memory, which
I/O path.

Upstream ships this as an example (``examples/tgis_weight.py:19-55``): it reads ``FST_CONFIG``,
``FST_NOGDS``, ``FST_THREADS`` and ``FST_BBUF_SIZE_KB`` and, when ``FST_CONFIG`` is ``auto``
(the default), sets ``nogds`` if ``/run/udev`` is missing, the thread count to the physical cores
of the GPU's NUMA node and the bounce size to the L2 capacity of those cores.  ``auto_config``
here keeps those variables and that return triple.  The policy behind it is the ring reader's:

* threads: the logical CPUs of the GPU's node that this process may run on, divided among the
  ranks of the machine (one process per GPU all read at once), between 2 and 16.  Logical, not
  physical as upstream counts: a worker mostly sleeps in an ``O_DIRECT`` ``pread``, and what a
  cold read needs is requests in flight, not cores.  (From the page cache 8 and 16 workers moved
  the same bytes per second on a 16-vCPU host, 32 fewer: the ring's pinning cost grows with it.)
* pinned memory: two slots per thread of ``DEFAULT_SLOT_KB`` each (windows of that size keep a
  cold ``O_DIRECT`` stream at the device's rate and still pipeline within one file); pinning goes
  through the CUDA driver and is not charged to ``RLIMIT_MEMLOCK``, so that limit is not consulted;
* ``nogds`` is False only where the ``nvidia-fs`` driver and ``/run/udev`` are both present.  It
  is passed on as upstream's flag; the I/O mode stays ``auto`` (ring reader) either way.
"""

from __future__ import annotations

import glob
import os
from dataclasses import dataclass
from typing import Dict, Optional, Set, Tuple

from .common import get_device_numa_node

DEFAULT_SLOT_KB = 4096
MIN_SLOT_KB = 256
MIN_THREADS, MAX_THREADS = 2, 16


def _parse_cpu_list(text: str) -> Set[int]:
    """``"0-3,8,10-11"`` -> {0,1,2,3,8,10,11} (the kernel's cpulist format)."""
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def _read(path: str) -> Optional[str]:
    try:
        with open(path) as f:
            return f.read().strip()
    except OSError:
        return None


def _size_kb(text: Optional[str]) -> int:
    """sysfs cache sizes: ``"2048K"`` or ``"2M"``."""
    if not text:
        return 0
    unit = text[-1].upper()
    try:
        return int(text[:-1]) * {"K": 1, "M": 1024, "G": 1024 * 1024}[unit] if unit in "KMG" else int(text) // 1024
    except ValueError:
        return 0


@dataclass(frozen=True)
class HostTopology:
    """What the tuner looks at, for one NUMA node."""
    node: int
    cpus: Tuple[int, ...]          # logical CPUs of the node this process may run on
    physical_cores: int            # distinct (package, core) pairs among them
    l2_kb: int                     # capacity of the distinct L2 caches serving them

    @classmethod
    def probe(cls, node: Optional[int], sysfs: str = "/sys", allowed: Optional[Set[int]] = None) -> "HostTopology":
        if allowed is None:
            try:
                allowed = set(os.sched_getaffinity(0))
            except (AttributeError, OSError):
                allowed = None
        node_cpus: Optional[Set[int]] = None
        if node is not None and node >= 0:
            text = _read(f"{sysfs}/devices/system/node/node{node}/cpulist")
            if text:
                node_cpus = _parse_cpu_list(text)
        if node_cpus is None:   # no NUMA information: every CPU the system lists
            node_cpus = set()
            for d in glob.glob(f"{sysfs}/devices/system/cpu/cpu[0-9]*"):
                try:
                    node_cpus.add(int(os.path.basename(d)[3:]))
                except ValueError:
                    pass
            if not node_cpus:
                node_cpus = set(range(os.cpu_count() or 1))
        cpus = sorted(node_cpus & allowed) if allowed else sorted(node_cpus)
        if not cpus:            # affinity excludes the node: run where we are allowed to
            cpus = sorted(allowed or node_cpus)
        cores: Set[Tuple[str, str]] = set()
        caches: Dict[str, int] = {}
        for c in cpus:
            base = f"{sysfs}/devices/system/cpu/cpu{c}"
            core = _read(f"{base}/topology/core_id")
            pkg = _read(f"{base}/topology/physical_package_id") or "0"
            cores.add((pkg, core if core is not None else f"cpu{c}"))
            for idx in glob.glob(f"{base}/cache/index[0-9]*"):
                if _read(f"{idx}/level") != "2":
                    continue
                shared = _read(f"{idx}/shared_cpu_list") or str(c)
                caches.setdefault(shared, _size_kb(_read(f"{idx}/size")))
        return cls(node if node is not None else -1, tuple(cpus), len(cores), sum(caches.values()))


@dataclass(frozen=True)
class ReaderSettings:
    nogds: bool
    max_threads: int
    bbuf_size_kb: int
    slot_kb: int
    io_mode: str                   # always "auto": cuFile has to be asked for by name
    numa_node: int

    def loader_kwargs(self) -> Dict[str, object]:
        """Keyword arguments for ``SafeTensorsFileLoader`` / ``ParallelLoader``."""
        return {"nogds": self.nogds, "max_threads": self.max_threads, "bbuf_size_kb": self.bbuf_size_kb,
                "slot_kb": self.slot_kb, "io_mode": self.io_mode}


def gds_usable(sysfs_run: str = "/run/udev", proc_modules: str = "/proc/modules") -> bool:
    """cuFile can reach the device directly only with the nvidia-fs driver loaded; libcufile also
    needs the udev database to map files to block devices."""
    mods = _read(proc_modules) or ""
    return os.path.isdir(sysfs_run) and any(line.split(" ", 1)[0] == "nvidia_fs" for line in mods.splitlines())


def suggest(device_index: Optional[int] = None, local_world: Optional[int] = None, sysfs: str = "/sys",
            topology: Optional[HostTopology] = None, gds: Optional[bool] = None) -> ReaderSettings:
    """Settings for one loader process that feeds GPU ``device_index``.

    ``local_world``: loader processes on this machine that read at the same time (default: the
    launcher's ``LOCAL_WORLD_SIZE``, else 1)."""
    node = get_device_numa_node(device_index) if device_index is not None else None
    topo = topology or HostTopology.probe(node, sysfs)
    if local_world is None:
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", "1") or 1)
    threads = max(MIN_THREADS, min(MAX_THREADS, (len(topo.cpus) or 1) // max(1, local_world)))
    slot_kb = DEFAULT_SLOT_KB
    use_gds = gds_usable() if gds is None else gds
    return ReaderSettings(nogds=not use_gds, max_threads=threads, bbuf_size_kb=threads * 2 * slot_kb,
                          slot_kb=slot_kb, io_mode="auto", numa_node=topo.node)


def auto_config(device_index: Optional[int] = None) -> Tuple[bool, int, int]:
    """``(nogds, max_copier_threads, bbuf_size_kb_total)`` from the environment, as upstream's
    example computes it: explicit values from ``FST_NOGDS`` / ``FST_THREADS`` /
    ``FST_BBUF_SIZE_KB`` unless ``FST_CONFIG`` is ``auto`` (default), in which case the host
    decides (``suggest``)."""
    nogds = os.environ.get("FST_NOGDS") == "1"
    threads = int(os.environ.get("FST_THREADS", "16"))
    bbuf_kb = int(os.environ.get("FST_BBUF_SIZE_KB", "163840"))
    if os.environ.get("FST_CONFIG", "auto") == "auto":
        try:
            s = suggest(device_index)
        except Exception as e:  # noqa: BLE001 - a tuner must not stop a load
            print(f"Failed to auto-configure fastsafetensors_b200. reason: {e}")
        else:
            nogds, threads, bbuf_kb = s.nogds, s.max_threads, s.bbuf_size_kb
    return nogds, threads, bbuf_kb

