"""Benchmark of the safetensors -> HBM tensor-parallel load path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--config NAME]

Workload (synthetic values, the shapes of the benchmark configurations):

* N = 1: the Llama-2-13B-shaped checkpoint (3 files, 26.03 GB, fp16 weights and fp32 norms, odd
  header lengths so that every window goes through the realign kernel): the largest
  configuration that fits one GPU.  The single rank owns every file and packs the shards of all
  4 tensor-parallel ranks (what the owner of a file does before the exchange).
* N > 1: the first 8 of the 30 files of the Llama-3-70B-shaped checkpoint (37.6 GB of 141 GB:
  what fits the boxes' disk), owned round-robin, tensor parallelism N-way, shards exchanged over
  NVLink.  ``--config`` / ``--files`` select any other configuration.

One JSON line is printed by rank 0:

* ``value``    GB/s of tensor data turned into shards per second with the file images already
               resident in memory (gather kernel + exchange), CUDA events, max over ranks;
* ``e2e``      the same checkpoint from files on disk to shards in HBM through the public loader
               API, page cache dropped before every step (cold reads), wall clock between device
               synchronisations, max over ranks; ``e2e_warm``: files in the page cache;
* ``storage_read`` cold O_DIRECT read rate of the same files with the loader's own request
               pattern, measured before, between and after the cold steps;
* ``roofline`` the gather kernel against the measured HBM copy bandwidth;
* ``parity``   a sample of the shards compared byte for byte with regenerated tensor data;
* ``reference_cuda`` upstream's own CUDA path (``device=cuda:r``, NCCL) on the same files at this N;
* ``cpu_baseline`` upstream fastsafetensors (CPU, gloo ranks) on a bounded sample (N = 1 only).

``--impl reference`` runs upstream's own CPU path (built into ``oracle/_ref``) on the same files
and reports the same two quantities: ``value`` = file images resident in host memory -> shards
(upstream's shuffle phase), ``e2e`` = cold files -> shards.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from collections import OrderedDict

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GB = 1e9
L2_BYTES = 126 * (1 << 20)
METRIC = ("safetensors->HBM tensor-parallel load: GB/s of tensor data sharded with file images "
          "resident (value), files on disk -> shards (e2e)")
# bytes of cold reading an arm spends on timed end-to-end steps (bounds the step count)
E2E_COLD_BYTES = 200e9


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--config", default=None,
                    help="gpt2-small | llama3-8b | llama2-13b | llama3-70b | mixtral-8x7b "
                         "(default: llama2-13b on one GPU, llama3-70b otherwise)")
    ap.add_argument("--files", type=int, default=0,
                    help="keep only the first F files of the checkpoint (default: all, 8 for llama3-70b)")
    ap.add_argument("--scale", default="full", choices=("full", "tiny"))
    ap.add_argument("--dir", default=os.environ.get("FST_BENCH_DIR", "/tmp/fst_bench"))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true")
    ap.add_argument("--warm-only", action="store_true", help="skip the cold end-to-end phase and the storage roofline")
    ap.add_argument("--e2e-steps", type=int, default=0, help="cold end-to-end steps (default: by checkpoint size)")
    ap.add_argument("--threads", type=int, default=int(os.environ.get("FST_BENCH_THREADS", 0)),
                    help="reader threads per rank (default: host CPUs / ranks, between 2 and 16)")
    ap.add_argument("--transport", default=os.environ.get("FST_B200_TRANSPORT", "auto"),
                    choices=("auto", "nccl", "peer"),
                    help="N > 1: all_to_all over NCCL, gather-kernel stores into peer arenas, or the "
                         "library's own choice")
    ap.add_argument("--ref-settings", default="best", choices=("best", "defaults", "tuned"),
                    help="--impl reference: upstream's library defaults, the rule of its perf tool, or "
                         "whichever of the two is faster in one untimed step each")
    ap.add_argument("--ref-budget", type=float, default=330.0,
                    help="--impl reference: seconds the resident phase may take before its steps are cut "
                         "to the first files of the checkpoint")
    ap.add_argument("--layers", type=int, default=0,
                    help="keep only the first L transformer layers (small case for profiler captures)")
    ap.add_argument("--other-kernels-only", action="store_true",
                    help="only the stand-alone timing of the realign and convert kernels (for profiler captures)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="only the device-resident phase (for profiler captures)")
    return ap.parse_args()


def dist_env():
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)),
            int(os.environ.get("WORLD_SIZE", 1)))


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if x > 0.5 * max(mx or [1])] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------
# workload (shared by both arms; nothing here touches the loader under test)
# ------------------------------------------------------------------------------------------
def plan_for(spec, tp: int) -> "OrderedDict[str, tuple]":
    return OrderedDict((t.name, (t.action[0], t.action[1] % tp) if t.action[0] == "push" else t.action)
                       for t in spec.tensors)


def read_into_page_cache(paths) -> None:
    """Buffered sequential read of every file, so that a following phase finds them cached
    (nothing to do for files on a memory file system)."""
    for p in paths:
        if os.path.realpath(p).startswith("/dev/shm/"):
            continue
        with open(p, "rb", buffering=0) as f:
            while f.read(64 << 20):
                pass


class Workload:
    """Files, tensors and plan of one run.  ``--layers L`` cuts the checkpoint to its first L
    layers, ``--files F`` to the tensors of its first F files (file boundaries stay those of the
    whole checkpoint)."""

    def __init__(self, args, world: int, n_files: int = 0):
        """``n_files`` > 0: the file count another rank has decided on (see ``_fit_to_disk``)."""
        import re

        from tests import synth

        name = args.config or ("llama2-13b" if world == 1 else "llama3-70b")
        spec = synth.config(name, args.scale)
        if args.layers > 0:
            def keep(tname: str) -> bool:
                m = re.search(r"(?:layers|h)\.(\d+)\.", tname)
                return m is None or int(m.group(1)) < args.layers
            spec.tensors = [t for t in spec.tensors if keep(t.name)]
            spec.name = f"{spec.name}-first{args.layers}layers"
        self.spec = spec
        self.groups = synth.partition(spec)
        self.total_files = len(self.groups)
        self.dir = os.path.join(args.dir, spec.name)
        self.disk_note = ""
        if n_files > 0:
            self.n_files = n_files
        else:
            want = args.files or (8 if name == "llama3-70b" and args.scale == "full" else self.total_files)
            self.n_files = max(1, min(want, self.total_files))
            self.disk_note = self._fit_to_disk(args.dir, world)
        self.tp = spec.tp if world == 1 else world
        self.indices = [i for g in self.groups[: self.n_files] for i in g]   # tensor indices in the kept files
        self.tensors = [spec.tensors[i] for i in self.indices]
        self.data_bytes = sum(t.nbytes for t in self.tensors)
        full = plan_for(spec, self.tp)
        self.plan = OrderedDict((t.name, full[t.name]) for t in self.tensors)
        self.paths = sorted(os.path.join(self.dir, synth.file_name(spec, k, self.total_files))
                            for k in range(self.n_files))
        subset = "" if self.n_files == self.total_files else \
            f" (first {self.n_files} of its {self.total_files} files)"
        self.label = (f"{spec.name} ({args.scale}){subset}: {len(self.tensors)} tensors, "
                      f"{self.n_files} files, {self.data_bytes} data bytes, tensor-parallel {self.tp}-way")

    def _fit_to_disk(self, top: str, world: int) -> str:
        """Make sure the files that still have to be written fit the disk: remove this
        benchmark's other checkpoints first, then keep fewer files (never fewer than one per
        rank).  Returns a note for the log, empty if nothing had to be done."""
        import shutil

        from tests import synth

        def missing_bytes(n_files: int) -> int:
            need = 0
            for k in range(n_files):
                size = sum(self.spec.tensors[i].nbytes for i in self.groups[k]) + (1 << 20)
                path = os.path.join(self.dir, synth.file_name(self.spec, k, self.total_files))
                if not (os.path.exists(path) and os.path.getsize(path) >= size - (1 << 20)):
                    need += size
            return need

        os.makedirs(top, exist_ok=True)
        margin = 2 << 30
        note = ""
        if missing_bytes(self.n_files) + margin > shutil.disk_usage(top).free:
            for other in sorted(os.listdir(top)):
                if other != self.spec.name and os.path.isdir(os.path.join(top, other)):
                    shutil.rmtree(os.path.join(top, other), ignore_errors=True)
                    note += f"removed {other}; "
        while self.n_files > max(1, world) and missing_bytes(self.n_files) + margin > shutil.disk_usage(top).free:
            self.n_files -= 1
            note += f"cut to {self.n_files} files (disk); "
        return note

    def config_block(self) -> dict:
        """The ``config`` object: identical in both arms."""
        return {"workload": self.label, "tp": self.tp, "files": self.n_files, "data_bytes": self.data_bytes,
                "l2": f"every step moves far more than L2 ({L2_BYTES} B); no flush between steps"}

    def write(self, rank: int, barrier) -> None:
        from tests import synth

        if rank == 0:
            t0 = time.time()
            synth.write_checkpoint(self.spec, self.dir, fsync=True, only_files=range(self.n_files))
            sys.stderr.write(f"[bench] checkpoint {self.label} in {self.dir} ({time.time() - t0:.1f} s) "
                             f"{self.disk_note}\n")
        barrier()

    def e2e_steps(self, args) -> int:
        if args.e2e_steps > 0:
            return args.e2e_steps
        return int(max(2, min(args.steps, round(E2E_COLD_BYTES / max(self.data_bytes, 1)))))


def host_threads(args, world: int) -> int:
    if args.threads > 0:
        return args.threads
    # one thread per core of the rank's share of the host (four ranks on 32 cores measured 44.9
    # GB/s warm with 8 threads each and 42.6 GB/s with 4)
    return int(max(2, min(16, (os.cpu_count() or 16) // max(1, world))))


# ------------------------------------------------------------------------------------------
# parity inside the bench: a sample of the produced shards against regenerated tensor bytes
# ------------------------------------------------------------------------------------------
def expected_shard(tensor, raw, action, dst: int, tp: int):
    """Bytes rank ``dst`` must hold for ``tensor`` (numpy): block ``dst`` of ceil(n/tp) on the
    split dimension, the whole tensor for replicated and pushed ones."""
    import numpy as np

    from tests import synth

    if action[0] != "shard":
        return raw
    item = synth._ITEMSIZE[tensor.dtype]
    dim = action[1]
    a = raw.reshape(*tensor.shape, item)
    block = -(-tensor.shape[dim] // tp)
    sl = [slice(None)] * len(tensor.shape)
    sl[dim] = slice(dst * block, (dst + 1) * block)
    return np.ascontiguousarray(a[tuple(sl)]).reshape(-1)


def parity_sample(wl: Workload, want: int = 40, max_bytes: int = 600 << 20):
    """Deterministic sample of positions in ``wl.tensors``: the first tensor of every kind of
    action (dim 0, dim 1, replicated, pushed) and an even stride over the rest."""
    first, rest = {}, []
    for pos, t in enumerate(wl.tensors):
        if t.nbytes > max_bytes:
            continue
        kind = wl.plan[t.name][:2] if wl.plan[t.name][0] == "shard" else wl.plan[t.name][:1]
        if kind not in first:
            first[kind] = pos
        else:
            rest.append(pos)
    stride = max(1, len(rest) // max(1, want - len(first)))
    return sorted(set(first.values()) | set(rest[::stride][: want]))


def check_parity(wl: Workload, get_result, dsts) -> dict:
    """``get_result(name, dst)`` -> torch tensor (or None where ``dst`` does not get the tensor).
    Compares SHA-256 of the produced bytes with the regenerated ones for every ``dst`` in ``dsts``."""
    import torch

    from tests import synth

    checked, bad, kinds = 0, [], set()
    for pos in parity_sample(wl):
        t = wl.tensors[pos]
        action = wl.plan[t.name]
        raw = synth.expected_bytes(wl.spec, wl.indices[pos])
        for dst in dsts:
            got = get_result(t.name, dst)
            if action[0] == "push" and action[1] != dst:
                if got is not None:
                    bad.append(f"{t.name}@{dst}: present on a rank it was not pushed to")
                continue
            if got is None:
                bad.append(f"{t.name}@{dst}: missing")
                continue
            have = got.contiguous().reshape(-1).view(torch.uint8).cpu().numpy()
            exp = expected_shard(t, raw, action, dst, wl.tp)
            if hashlib.sha256(have.tobytes()).digest() != hashlib.sha256(exp.tobytes()).digest():
                bad.append(f"{t.name}@{dst}: bytes differ")
            checked += 1
            kinds.add(action[0] + (str(action[1]) if action[0] == "shard" else ""))
    return {"checked": checked, "ok": not bad, "kinds": sorted(kinds), "mismatches": bad[:5]}


# ------------------------------------------------------------------------------------------
# this repository's arm
# ------------------------------------------------------------------------------------------
def b200_arm(args) -> dict:
    import torch
    import torch.distributed as dist

    import fastsafetensors_b200 as fst
    from fastsafetensors_b200 import cpp
    from fastsafetensors_b200.batch import PeerArenaUnavailable, PeerShardExchange, ShardExchange
    from fastsafetensors_b200.file_buffer import resolve_transport
    from tests import synth

    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the b200 arm has no CPU substitute")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    pg = None
    if world > 1:
        import datetime

        # no all-reduce of any size is on the path; NVLS buys nothing here and a rank that leaves
        # early while bound to a multicast object can disturb its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device(device),
                                timeout=datetime.timedelta(seconds=900))
        pg = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks(obj) -> list:
        if world == 1:
            return [obj]
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def note(msg: str) -> None:
        if rank == 0:
            sys.stderr.write(f"[bench] {time.strftime('%H:%M:%S')} {msg}\n")
            sys.stderr.flush()

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    if args.other_kernels_only:
        return {"other_kernels": other_kernels(device, peak)} if rank == 0 else {}

    # rank 0 looks at the disk and decides how many files the run keeps; the others follow
    decided = [Workload(args, world).n_files if rank == 0 else 0]
    if world > 1:
        dist.broadcast_object_list(decided, src=0)
    wl = Workload(args, world, n_files=decided[0])
    tp, plan, paths, data_bytes = wl.tp, wl.plan, wl.paths, wl.data_bytes
    wl.write(rank, barrier)
    owners = synth.owners(paths, world)
    threads = host_threads(args, world)

    def open_loader():
        return fst.SafeTensorsFileLoader(pg if pg is not None else fst.SingleGroup(), torch.device(device),
                                         nogds=True, max_threads=threads)

    # "auto" is the library's rule, and NCCL on all ranks together if peer mapping is refused
    may_fall_back = False
    if world > 1:
        want = resolve_transport(args.transport, world, fst.Device.from_str(device))
        may_fall_back = want == "auto"
        args.transport = "nccl" if want == "nccl" else "peer"

    def make_exchange(fb):
        if world > 1 and args.transport == "peer":
            try:
                return PeerShardExchange(fb, plan, tp, rank)
            except PeerArenaUnavailable as e:     # every rank gets it at the same call
                if not may_fall_back:
                    raise
                note(f"peer arenas unavailable ({e}); NCCL all-to-all instead")
                args.transport = "nccl"
        return ShardExchange(fb, plan, tp, rank if world > 1 else 0, local=(world == 1))

    # ---------------------------------------------------------------- device-resident phase
    note(f"{wl.label}; {threads} reader threads per rank")
    note("device-resident phase: loading images")
    loader = open_loader()
    loader.add_filenames(owners)
    fb = loader.copy_files_to_device()
    ex = make_exchange(fb)
    stream = torch.cuda.current_stream()
    warmup = max(3, args.warmup)
    # clocks are sampled every 200 ms from here to the end of the timed region; the warm-up runs
    # for at least 1.5 s so that the short timed region is bracketed by samples taken under load
    sampler = ClockSampler(local_rank) if rank == 0 else None
    # every rank must run the same number of steps (each step ends in a collective when N > 1):
    # time the first warm-up steps, then agree on how many more fill the 1.5 s
    t_w = time.perf_counter()
    for _ in range(warmup):
        ex.run()
    torch.cuda.synchronize()
    per_step = (time.perf_counter() - t_w) / warmup
    extra = 0 if args.kernel_only else int(max_over_ranks(min(2000.0, 1.5 / max(per_step, 1e-6))))
    for i in range(extra):
        ex.run()
        if i % 8 == 7:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    barrier()
    m0 = cpp.get_cpp_metrics()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_events = []
    torch.cuda.synchronize()
    barrier()
    start.record(stream)
    for _ in range(args.steps):
        ex.run(timing=kernel_events)     # an event pair around every gather launch
    stop.record(stream)
    torch.cuda.synchronize()
    barrier()
    m1 = cpp.get_cpp_metrics()
    resident_ms = max_over_ranks(start.elapsed_time(stop)) / args.steps
    kernel_ms_total = sum(a.elapsed_time(b) for a, b in kernel_events)
    n_launch = len(kernel_events)
    launches_timed = m1.kernel_launches - m0.kernel_launches
    payload_per_step = ex.payload_bytes                      # bytes this rank's kernel moves per step
    # the roofline entry is the kernel over the timed launches: algorithmic bytes of a launch =
    # 2 x its payload (read once, written once); per launch, the average over the launches of a step
    launches_per_step = max(1, n_launch // max(1, args.steps))
    alg_bytes_per_launch = 2.0 * payload_per_step / launches_per_step
    kernel_ms = kernel_ms_total / max(1, n_launch)           # average launch duration
    achieved = alg_bytes_per_launch / (kernel_ms * 1e-3) / GB if kernel_ms > 0 else 0.0
    clocks = sampler.stop() if sampler else None
    egress = ex.egress_bytes if world > 1 else 0

    # parity: a sample of what the timed steps produced, against regenerated tensor bytes
    note("parity sample")
    if world == 1:
        per_dst = ex.results()
        parity = check_parity(wl, lambda n, d: (per_dst[d][n].get_raw() if n in per_dst[d] else None), range(tp))
        per_dst = None
    else:
        mine = ex.results()
        parity = check_parity(wl, lambda n, d: (mine[n].get_raw() if n in mine else None), [rank])
        mine = None
        every = all_ranks(parity)
        parity = {"checked": sum(p["checked"] for p in every), "ok": all(p["ok"] for p in every),
                  "kinds": sorted(set(k for p in every for k in p["kinds"])),
                  "mismatches": [m for p in every for m in p["mismatches"]][:5]}
    parity["what"] = "SHA-256 of result bytes (device -> host) against regenerated tensor data, after the timed steps"
    # a light device -> host read of the result
    check = int(ex.recv[:: max(1, ex.recv.numel() // 4096)].to(torch.int64).sum().item())
    if isinstance(ex, PeerShardExchange):
        ex.close()          # collective: the ranks unmap each other's arenas
    del ex
    fb.close()
    loader.close()
    torch.cuda.empty_cache()

    result = {
        "metric": METRIC,
        "value": round(data_bytes / (resident_ms * 1e-3) / GB, 2),
        "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(resident_ms, 4),
        "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": wl.config_block(),
        "notes": {
            "value_phase": "file images resident in HBM -> gather kernel (+ exchange)",
            "how": ("one rank packs the shards of all destinations" if world == 1 else
                    "files owned round-robin, " + ("chunked NCCL all-to-all overlapped with the gather launches"
                                                   if args.transport == "nccl"
                                                   else "gather kernel stores into peer arenas (NVLink)")),
            "payload_bytes_per_rank_and_step": int(payload_per_step),
            "reader_threads_per_rank": threads,
        },
        "gpu_launches": int(launches_timed),
        "roofline": {
            "bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            "peak_source": peak_src,
            "kernel": "fst_gather_kernel", "launches": n_launch,
            "avg_launch_ms": round(kernel_ms, 4),
            "algorithmic_bytes_per_launch": int(alg_bytes_per_launch),
        },
        "clocks": clocks,
        "parity": parity,
        "result_checksum": check,
    }
    if world > 1 and args.transport == "peer":
        # most of this kernel's stores land in other GPUs' HBM; the recorded ratio is of local copies
        result["roofline"].update({"traffic": None, "traffic_source": "peer stores: no local-DRAM figure recorded",
                                   "bound_note": "NVLink-bound, see nvlink"})
    else:
        result["roofline"].update(recorded_traffic(alg_bytes_per_launch))
    if world > 1:
        peer_ref = measure_peer_copy(barrier, max_over_ranks) if not args.kernel_only else None
        egress_max = max(all_ranks(egress))
        rate = egress_max / (resident_ms * 1e-3) / GB
        # every byte a rank sends crosses NVLink once; with the step time this is the per-GPU
        # egress rate the exchange sustains
        result["nvlink"] = {"transport": args.transport, "egress_bytes_per_rank_and_step": int(egress_max),
                            "egress_gbs_per_gpu": round(rate, 1),
                            "peer_copy_gbs_measured": peer_ref,
                            "frac_of_peer_copy": round(rate / peer_ref, 3) if peer_ref else None,
                            "note": "egress of the rank that sends most over the whole step (gather "
                                    "launches + exchange); the reference is one 1 GiB device-to-device "
                                    "copy to the neighbouring GPU, all ranks at once, slowest rank"}
        if args.transport == "peer":
            # fused pack + transfer: the step cannot be faster than the slower of moving this
            # rank's payload through HBM and pushing its remote part through NVLink
            link = peer_ref or 770.0
            target_ms = max(2.0 * payload_per_step / (peak * GB), egress / (link * GB)) * 1e3
            result["nvlink"]["fused_kernel"] = {"target_ms": round(target_ms, 4),
                                                "achieved_ms": round(kernel_ms, 4),
                                                "frac": round(target_ms / kernel_ms, 4) if kernel_ms else None}

    # ---------------------------------------------------------------- end to end (public API)
    e2e_parity = {}

    def e2e_step(check: bool = False):
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        ld = open_loader()
        ld.add_filenames(owners)
        t1 = time.perf_counter()
        buf = ld.copy_files_to_device(wait=False)     # reads queued; files are waited for in order
        if world == 1:
            got = buf.shard_locally(plan, tp)
            probe = next(iter(got[-1].values())).get_raw()
        else:
            got = buf.exchange(plan, transport=args.transport)
            probe = next(iter(got.values())).get_raw()
        t2 = time.perf_counter()
        head = probe.reshape(-1)[:1024].cpu()      # device -> host read of the result
        torch.cuda.synchronize()
        t3 = time.perf_counter()
        barrier()
        t4 = time.perf_counter()
        if check:        # outside the timed region: the shards this step produced, against regenerated data
            if world == 1:
                p = check_parity(wl, lambda n, d: (got[d][n].get_raw() if n in got[d] else None), range(tp))
            else:
                p = check_parity(wl, lambda n, d: (got[n].get_raw() if n in got else None), [rank])
            every = all_ranks(p)
            e2e_parity.update({"checked": sum(q["checked"] for q in every), "ok": all(q["ok"] for q in every),
                               "mismatches": [m for q in every for m in q["mismatches"]][:5]})
        del got, probe
        buf.close()
        ld.close()
        return (max_over_ranks(t4 - t0), int(head.numel() * head.element_size()),
                {"open_and_headers": t1 - t0, "read_pack_exchange_queued": t2 - t1, "device_drain": t3 - t2,
                 "wait_for_other_ranks": t4 - t3, "total": t4 - t0})

    def cold_read_pass() -> float:
        """One pass of the storage roofline: every rank reads the files it owns, all submitted at
        once (the loader's pattern), O_DIRECT, into host memory; GB/s over all ranks."""
        if rank == 0:
            synth.drop_page_cache(paths)
        barrier()
        dt = max_over_ranks(read_files_direct(owners[rank], threads))
        return sum(os.path.getsize(p) for p in paths) / dt / GB

    def e2e_phase(cold: bool, steps: int, warmup_steps: int, passes_at=()):
        times, d2h, parts, passes = [], 0, [], []
        read_ns = 0
        for i in range(warmup_steps + steps):
            if i - warmup_steps in passes_at:
                passes.append(round(cold_read_pass(), 3))
            if cold:
                if rank == 0:
                    synth.drop_page_cache(paths)
                barrier()
            r0 = cpp.get_cpp_metrics().read_ns
            dt, d2h, part = e2e_step(check=(not cold and i == warmup_steps + steps - 1))
            if i >= warmup_steps:
                times.append(dt)
                parts.append(part)
                read_ns += cpp.get_cpp_metrics().read_ns - r0
            torch.cuda.empty_cache()
        if steps in passes_at:
            passes.append(round(cold_read_pass(), 3))
        mean = sum(times) / len(times)
        read_s = read_ns / 1e9 / len(times)
        mine = {k: round(sum(p[k] for p in parts) / len(parts), 4) for k in parts[0]}
        mine["pread_thread_seconds"] = round(read_s, 3)
        mine["rank"] = rank
        slowest = max(all_ranks(mine), key=lambda p: p["total"] - p["wait_for_other_ranks"])
        return {"value": round(data_bytes / mean / GB, 3), "unit": "GB/s",
                "h2d_bytes_per_step": int(data_bytes), "d2h_bytes_per_step": d2h,
                "s_per_step": round(mean, 4), "steps": steps, "warmup": warmup_steps,
                "s_per_step_min_max": [round(min(times), 4), round(max(times), 4)],
                "page_cache": "dropped before every step" if cold else "warm",
                "slowest_rank_phases_s": slowest}, passes

    note(f"device-resident phase done: {resident_ms:.3f} ms per step")
    if rank == 0 and not args.kernel_only:
        result["other_kernels"] = other_kernels(device, peak)
    if not args.no_e2e and not args.kernel_only:
        cold_steps = wl.e2e_steps(args)
        if not args.warm_only:
            note(f"end-to-end phase, cold ({cold_steps} steps, storage read passes before, between and after)")
            mA = cpp.get_cpp_metrics()
            result["e2e"], passes = e2e_phase(True, cold_steps, 1, passes_at=(0, cold_steps // 2, cold_steps))
            mB = cpp.get_cpp_metrics()
            result["e2e"]["io"] = {"direct_requests": mB.direct_io_requests - mA.direct_io_requests,
                                   "buffered_requests": mB.buffered_io_requests - mA.buffered_io_requests}
            result["storage_read"] = {
                "cold_direct_gbs_max": max(passes), "cold_direct_gbs_median": statistics.median(passes),
                "passes_gbs": passes, "threads_per_rank": threads, "block": "4 MiB",
                "reading_ranks": sum(1 for r in owners if owners[r]),
                "tool": "native reader, O_DIRECT, all owned files submitted at once, host destination "
                        "(fio is not installed); passes before, between and after the cold steps"}
            result["e2e"]["frac_of_storage_read"] = round(result["e2e"]["value"] / max(passes), 3)
            result["e2e"]["frac_of_storage_read_median"] = round(
                result["e2e"]["value"] / statistics.median(passes), 3)
        note("end-to-end phase, warm")
        if rank == 0:
            read_into_page_cache(paths)
        barrier()
        mC = cpp.get_cpp_metrics()
        result["e2e_warm"], _ = e2e_phase(False, min(args.steps, 3), 2)
        mD = cpp.get_cpp_metrics()
        result["e2e_warm"]["io"] = {"direct_requests": mD.direct_io_requests - mC.direct_io_requests,
                                    "buffered_requests": mD.buffered_io_requests - mC.buffered_io_requests}
        # the shards of the last end-to-end step were checked too (files -> deferred reads ->
        # pipelined pack and exchange), not only those of the resident phase
        parity["e2e_checked"] = e2e_parity.get("checked", 0)
        parity["checked"] += e2e_parity.get("checked", 0)
        if not e2e_parity.get("ok", True):
            parity["ok"] = False
            parity["mismatches"] = (parity["mismatches"] + ["e2e: " + m for m in e2e_parity["mismatches"]])[:5]
    if not parity["ok"]:
        note(f"PARITY FAILURE: {parity['mismatches']}")
    # ---------------------------------------------------------------- upstream's CUDA path, same N
    if not args.no_reference_cuda and not args.kernel_only and not args.no_e2e:
        note("upstream's CUDA path on the same files")
        result["reference_cuda"] = reference_cuda_phase(wl, owners, pg, rank, world, device, barrier,
                                                        max_over_ranks, result if rank == 0 else None)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.kernel_only:
        note("cpu baseline (upstream on the host cores, bounded sample)")
        result["cpu_baseline"] = cpu_baseline(wl)
    return result if rank == 0 else {"parity_ok": parity["ok"]}


KERNEL_SOURCE = os.path.join(ROOT, "fastsafetensors_b200", "csrc", "fst_kernels.cu")
DEVICE_CODE_END = "// Host side: argument checks"


def gather_device_code_hash() -> str:
    """SHA-256 (16 hex digits) of the device code of the gather and realign kernels: the kernel
    source file up to the comment that opens its host side."""
    text = open(KERNEL_SOURCE, encoding="utf-8").read()
    return hashlib.sha256(text[: text.index(DEVICE_CODE_END)].encode()).hexdigest()[:16]


def recorded_traffic(alg_bytes_per_launch: float) -> dict:
    """DRAM traffic of a gather launch from the recorded profiler capture: the ratio of dram
    read+write bytes to algorithmic bytes measured on a small case of this kernel, kept in
    ``profiles/fst_gather_kernel_traffic.json`` with a hash of the kernel's device code.  Traffic
    grows in proportion to the units processed, so the ratio scales to a full launch.  If the
    device code has changed since the capture the figure is marked as a constant."""
    path = os.path.join(ROOT, "profiles", "fst_gather_kernel_traffic.json")
    try:
        rec = json.load(open(path))
        current = gather_device_code_hash()
        ratio = float(rec["dram_bytes_per_algorithmic_byte"])
    except (OSError, ValueError, KeyError):
        return {"traffic": None, "traffic_source": "no recorded capture"}
    fresh = current == rec.get("device_code_sha256_16")
    return {"traffic": int(ratio * alg_bytes_per_launch),
            "traffic_source": ("profiler capture of a small case x units processed"
                               if fresh else "constant: the kernel's device code changed after the recorded capture"),
            "traffic_ratio": ratio}


def measure_peer_copy(barrier, max_over_ranks):
    """GB/s of one device-to-device copy of 1 GiB from this GPU to its neighbour (best of 5),
    all ranks at once; the slowest rank's figure: the NVLink reference the exchange is held
    against."""
    import torch

    n = 1 << 30
    try:
        me = torch.cuda.current_device()
        src = torch.empty(n, dtype=torch.uint8, device=f"cuda:{me}")
        dst = torch.empty(n, dtype=torch.uint8, device=f"cuda:{(me + 1) % torch.cuda.device_count()}")
        best = 0.0
        for i in range(7):
            torch.cuda.synchronize()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            dst.copy_(src, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            if i >= 2:
                best = max(best, n / (a.elapsed_time(b) * 1e-3) / GB)
        del src, dst
        torch.cuda.empty_cache()
        return round(-max_over_ranks(-best), 1)
    except Exception as e:  # noqa: BLE001
        sys.stderr.write(f"[bench] peer copy measurement failed: {e}\n")
        max_over_ranks(0.0)
        return None


_read_scratch = None


def read_files_direct(my_paths, threads: int) -> float:
    """Seconds to read ``my_paths`` cold with the loader's reader settings (O_DIRECT, 4 MiB
    windows, two slots per thread), everything submitted before the first wait and in the
    loader's order (file after file).  The bytes are thrown away: every request is a 256 MiB
    piece of a file and all of them land in one 256 MiB host buffer that was touched beforehand,
    so neither page faults nor a multi-gigabyte destination are part of the figure."""
    global _read_scratch
    import numpy as np

    from fastsafetensors_b200 import _native as nat
    from fastsafetensors_b200 import cpp

    if not my_paths:
        return 0.0
    piece = 256 << 20
    if _read_scratch is None:
        _read_scratch = np.empty(piece, dtype=np.uint8)
        _read_scratch.fill(0)
    buf = cpp.gds_device_buffer(_read_scratch.ctypes.data, _read_scratch.size, False)
    reader = cpp.Reader(-1, threads, 4 << 20, 2, io_mode=nat.IO_DIRECT)
    t0 = time.perf_counter()
    reqs = []
    for p in my_paths:
        size = os.path.getsize(p) // 4096 * 4096
        for off in range(0, size, piece):
            reqs.append(reader.submit(p, off, min(piece, size - off), buf, 0))
    for r in reqs:
        reader.wait(r)
    dt = time.perf_counter() - t0
    reader.close()
    return dt


def other_kernels(device: str, peak: float) -> dict:
    """The path's other two kernels, timed alone with CUDA events on 1 GiB inputs (larger than
    L2): fst_realign with the source 9 bytes off a 16-byte boundary (an odd header), and
    fst_convert F32 -> BF16.  Algorithmic bytes: 2 x payload, and 4 + 2 bytes per element."""
    import torch

    from fastsafetensors_b200 import _native as nat

    n = 1 << 30
    stream = torch.cuda.current_stream()
    out = {}

    def timed(launch, alg_bytes):
        for _ in range(3):
            launch()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        a.record(stream)
        for _ in range(reps):
            launch()
        b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        gbs = alg_bytes / (ms * 1e-3) / GB
        return {"avg_launch_ms": round(ms, 4), "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                "frac": round(gbs / peak, 4), "algorithmic_bytes_per_launch": int(alg_bytes)}

    src = torch.empty(n + 64, dtype=torch.uint8, device=device)
    dst = torch.empty(n + 64, dtype=torch.uint8, device=device)
    out["fst_realign_kernel"] = timed(
        lambda: nat.realign(dst.data_ptr(), src.data_ptr() + 9, n, stream.cuda_stream), 2.0 * n)
    f32 = src[: n].view(torch.float32)
    bf16 = dst[: n // 2].view(torch.bfloat16)
    ops = [(f32.data_ptr(), bf16.data_ptr(), f32.numel(), nat.DT_CODES["F32"], nat.DT_CODES["BF16"])]
    out["fst_convert_kernel"] = timed(lambda: nat.convert(ops, stream.cuda_stream), 1.5 * n)
    # column split with short segments: a [524288, 2048]-byte matrix (1 GiB) split 8 ways on its
    # inner dimension, i.e. 256-byte row segments (what an 8-bit or 4-bit checkpoint gives)
    rows, width, seg = n // 2048, 2048, 256
    cols = [(src.data_ptr() + r * seg, dst.data_ptr() + r * rows * seg, rows, seg, width, seg) for r in range(8)]
    out["fst_gather_kernel_256B_segments"] = timed(
        lambda: nat.gather(cols, stream.cuda_stream, (src.data_ptr(), n), (dst.data_ptr(), n)), 2.0 * n)
    # the same split with every source 3 bytes off (funnel-shift path), and one flat misaligned copy
    off = [(c[0] + 3,) + c[1:] for c in cols]
    out["fst_gather_kernel_256B_segments_shifted"] = timed(
        lambda: nat.gather(off, stream.cuda_stream, (src.data_ptr(), n + 64), (dst.data_ptr(), n)), 2.0 * n)
    flat = [(src.data_ptr() + 5, dst.data_ptr(), 1, n, 0, 0)]
    out["fst_gather_kernel_flat_shifted"] = timed(
        lambda: nat.gather(flat, stream.cuda_stream, (src.data_ptr(), n + 64), (dst.data_ptr(), n)), 2.0 * n)
    del src, dst
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------
# upstream's CUDA path, timed inside the same ranks on the same files
# ------------------------------------------------------------------------------------------
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
REFERENCE_CUDA_LIMIT_S = 300.0


def reference_cuda_phase(wl: Workload, owners, pg, rank, world, device, barrier, max_over_ranks,
                         line_so_far) -> dict:
    """Upstream's loader with ``device=cuda:r`` and ``nogds=True`` (buffered pread + synchronous
    cudaMemcpy per chunk), the checkpoint's plan served tensor by tensor through
    ``get_sharded`` / ``get_tensor`` / ``push_tensor`` (tensor_factory.py:58-192: with N > 1 one
    NCCL scatter or broadcast and one device synchronisation per tensor; with one rank upstream
    returns whole tensors, so N = 1 times the load alone).  One cold and one warm end-to-end step
    and the time of the shuffle phase alone.

    A watchdog ends the process (after rank 0 has printed the line it has so far) if upstream's
    code does not come back within the limit."""
    import torch

    from tests import synth

    if not os.path.exists(os.path.join(REF_DIR, "fastsafetensors", "__init__.py")):
        return {"unavailable": "oracle/_ref is not built (oracle/build_ref.sh)"}

    def give_up():
        if line_so_far is not None:
            line_so_far["reference_cuda"] = {"unavailable": f"upstream's CUDA path did not finish within "
                                                            f"{REFERENCE_CUDA_LIMIT_S:.0f} s"}
            emit(line_so_far)
        os._exit(0)

    dog = threading.Timer(REFERENCE_CUDA_LIMIT_S, give_up)
    dog.daemon = True
    dog.start()
    try:
        sys.path.insert(0, REF_DIR)
        import fastsafetensors as ref

        out = {}
        for label, cold in (("cold", True), ("warm", False)):
            if cold and rank == 0:
                synth.drop_page_cache(wl.paths)
            torch.cuda.synchronize()
            barrier()
            t0 = time.perf_counter()
            loader = ref.SafeTensorsFileLoader(pg if pg is not None else ref.SingleGroup(), device, nogds=True)
            loader.add_filenames(owners)
            fb = loader.copy_files_to_device()
            torch.cuda.synchronize()
            t1 = time.perf_counter()
            keep = []
            for name, action in wl.plan.items():
                if action[0] == "shard":
                    keep.append(fb.get_sharded(name, action[1]))
                elif action[0] == "replicate":
                    keep.append(fb.get_tensor(name))
                else:
                    keep.append(fb.push_tensor(name, action[1]))
            torch.cuda.synchronize()
            barrier()
            t2 = time.perf_counter()
            total, shuffle = max_over_ranks(t2 - t0), max_over_ranks(t2 - t1)
            out[label] = {"e2e_gbs": round(wl.data_bytes / total / GB, 3), "s_per_step": round(total, 3),
                          "shuffle_phase_s": round(shuffle, 4),
                          "shuffle_phase_gbs": round(wl.data_bytes / shuffle / GB, 2)}
            del keep
            fb.close()
            loader.close()
            torch.cuda.empty_cache()
        out["what"] = (f"upstream fastsafetensors 0.3.2 (oracle/_ref), device cuda:r, nogds, {world} rank(s) over "
                       f"NCCL, library defaults; files -> HBM, then every tensor of the plan"
                       + (" (one rank: upstream hands out whole tensors, no sharding)" if world == 1 else ""))
        return out
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {e}"}
    finally:
        dog.cancel()
        if REF_DIR in sys.path:
            sys.path.remove(REF_DIR)


# ------------------------------------------------------------------------------------------
# upstream's CPU path (the checker's build in oracle/_ref), timed on the host cores
# ------------------------------------------------------------------------------------------
def _numa_nodes() -> int:
    import glob

    return max(1, len(glob.glob("/sys/devices/system/node/node[0-9]*")))


def _host_cores_and_l2_kb():
    """Physical cores and their summed L2 capacity in KiB, from sysfs (what upstream's perf tool
    reads, perf/fastsafetensors_perf/perf.py:345-365); (None, None) if unreadable."""
    import glob

    cores, l2_kb = set(), 0
    try:
        for cpudir in glob.glob("/sys/devices/system/cpu/cpu[0-9]*"):
            if not os.path.exists(f"{cpudir}/topology/core_id"):
                continue
            size = open(f"{cpudir}/cache/index2/size").read().strip()
            if not size.endswith("K"):
                return None, None
            core = (open(f"{cpudir}/topology/physical_package_id").read().strip(),
                    open(f"{cpudir}/topology/core_id").read().strip())
            if core not in cores:
                cores.add(core)
                l2_kb += int(size[:-1])
    except (OSError, ValueError):
        return None, None
    return (len(cores) or None), (l2_kb or None)


def _reference_settings(kind: str, paths, world: int):
    """Keyword arguments for upstream's loader and for its ``copy_files_to_device``.

    ``defaults``: what a caller that passes nothing gets (vLLM does): 16 threads, a 16 MiB bounce
    buffer and a 16 GiB block, i.e. ONE read request, hence one thread, per file.
    ``tuned``: the rule of upstream's own benchmark tool (perf/fastsafetensors_perf/perf.py,
    get_auto_config): threads = physical cores, bounce = their L2 capacity, block = checkpoint
    bytes / ranks / threads rounded up to the bounce size, so that every thread has a block."""
    if kind == "defaults":
        return {}, {}
    cores, l2_kb = _host_cores_and_l2_kb()
    threads = max(1, cores or os.cpu_count() or 1)
    bbuf_kb = l2_kb or 16 * 1024
    block = max(1, sum(os.path.getsize(p) for p in paths) // world // threads)
    unit = bbuf_kb * 1024
    if block % unit:
        block += unit - block % unit
    return {"max_threads": threads, "bbuf_size_kb": bbuf_kb}, {"max_copy_block_size": block}


def _reference_rank(rank: int, world: int, paths, plan_items, phases, port: int, out_path: str,
                    settings: str = "defaults") -> None:
    """One gloo rank running UPSTREAM's loader on device "cpu": files owned round-robin, every
    tensor requested by the plan (get_sharded / get_tensor / push_tensor).  ``settings``:
    ``defaults``, ``tuned`` or ``best`` (one untimed step with each, the faster one is timed).

    Phases, each ``(label, kind, steps, warmup, budget_s)``:
    ``kind == "e2e_cold" / "e2e_warm"``: loader construction -> copy_files_to_device -> every
    tensor of the plan, page cache dropped before the step or not;
    ``kind == "resident"``: the images are loaded once, untimed, and kept (auto_mem_delete off);
    a step is every tensor of the plan from the resident images -- upstream's shuffle phase
    (perf.py:609-637, t2 -> t3).  If the first step shows that the steps would not fit
    ``budget_s``, the phase goes on with the first files only and says so."""
    sys.path.insert(0, REF_DIR)
    import torch
    import torch.distributed as dist

    import fastsafetensors as ref
    from tests import synth

    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    pg = None
    if world > 1:
        # an explicit tcp:// rendezvous of our own: drop what a launcher (torchrun) left in the
        # environment, or every rank would wait as a client of the launcher's store
        for key in [k for k in os.environ if k.startswith("TORCHELASTIC_")]:
            os.environ.pop(key)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world)
        pg = dist.group.WORLD

    def barrier():
        if world > 1:
            dist.barrier()

    def agreed(value):
        """Rank 0's value on every rank."""
        box = [value]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        return box[0]

    def serve_plan(fb):
        present = set(fb.key_to_rank_lidx)
        keep = []
        for name, action in plan_items:
            if name not in present:
                continue
            if action[0] == "shard":
                keep.append(fb.get_sharded(name, action[1]))
            elif action[0] == "replicate":
                keep.append(fb.get_tensor(name))
            else:
                keep.append(fb.push_tensor(name, action[1]))
        return keep

    def open_and_copy(kind: str, use):
        loader_kw, copy_kw = _reference_settings(kind, use, world)
        loader = ref.SafeTensorsFileLoader(pg if pg is not None else ref.SingleGroup(), "cpu", nogds=True,
                                           **loader_kw)
        loader.add_filenames(synth.owners(use, world))
        fb = loader.copy_files_to_device(**copy_kw)
        nbytes = sum(m.size_bytes - m.header_length for m, _ in loader.meta.values())
        return loader, fb, nbytes

    def e2e_step(kind: str, n_files: int, cold: bool):
        use = sorted(paths)[:n_files]
        if cold and rank == 0:
            synth.drop_page_cache(use)
        barrier()
        t0 = time.perf_counter()
        loader, fb, nbytes = open_and_copy(kind, use)
        keep = serve_plan(fb)
        barrier()
        dt = time.perf_counter() - t0
        del keep
        fb.close()
        loader.close()
        return dt, nbytes

    results = {}
    chosen = None if settings == "best" else settings
    tried = {}
    for label, kind, steps, warmup, budget_s in phases:
        n_files = len(paths)
        if kind in ("e2e_cold", "e2e_warm"):
            cold = kind == "e2e_cold"
            if chosen is None:
                # one untimed step with each setting over the whole checkpoint; they double as warm-up
                trial = {}
                for k in ("defaults", "tuned"):
                    trial[k] = e2e_step(k, n_files, cold)
                    tried[k] = round(trial[k][1] / trial[k][0] / GB, 3)
                chosen = agreed(max(tried, key=tried.get))
                if steps == 0:      # the trial of the faster setting is the sample
                    results[label] = {"seconds": [trial[chosen][0]], "bytes": [trial[chosen][1]], "files": n_files}
                    continue
            else:
                for _ in range(warmup):
                    e2e_step(chosen, n_files, cold)
            samples = [e2e_step(chosen, n_files, cold) for _ in range(steps)]
            results[label] = {"seconds": [s_[0] for s_ in samples], "bytes": [s_[1] for s_ in samples],
                              "files": n_files}
            continue
        # resident phase
        use_kind = chosen or "tuned"
        secs, nb = [], 0
        while True:
            loader, fb, nb = open_and_copy(use_kind, sorted(paths)[:n_files])
            fb.auto_mem_delete = False          # keep the images: every step starts from them
            barrier()
            t0 = time.perf_counter()
            keep = serve_plan(fb)
            barrier()
            first = time.perf_counter() - t0
            del keep
            fit = agreed(first * (steps + warmup) <= budget_s or n_files == 1)
            if fit:
                break
            fb.close()
            loader.close()
            n_files = agreed(max(1, min(n_files - 1, int(n_files * budget_s / (first * (steps + warmup))))))
        for i in range(max(0, warmup - 1) + steps):
            barrier()
            t0 = time.perf_counter()
            keep = serve_plan(fb)
            barrier()
            dt = time.perf_counter() - t0
            del keep
            if i >= max(0, warmup - 1):
                secs.append(dt)
        fb.close()
        loader.close()
        results[label] = {"seconds": secs, "bytes": [nb] * len(secs), "files": n_files}
    results["settings"] = {"used": chosen, "tried_gbs": tried,
                           "kwargs": [dict(d) for d in _reference_settings(chosen or "tuned", sorted(paths), world)]}
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)
    if world > 1:
        dist.destroy_process_group()


def run_reference(wl: Workload, paths, phases, timeout_s: float = 900.0, settings: str = "defaults") -> dict:
    import socket
    import tempfile

    import torch.multiprocessing as mp

    if not os.path.exists(os.path.join(REF_DIR, "fastsafetensors", "__init__.py")):
        raise FileNotFoundError("oracle/_ref is missing (build it with oracle/build_ref.sh)")
    plan_items = list(wl.plan.items())
    tp = wl.tp
    with tempfile.TemporaryDirectory() as tmp:
        out_path = os.path.join(tmp, "times.json")
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:   # a port that is free now
            sock.bind(("127.0.0.1", 0))
            port = sock.getsockname()[1]
        if tp == 1:
            _reference_rank(0, 1, paths, plan_items, phases, port, out_path, settings)
        else:
            ctx = mp.start_processes(_reference_rank, args=(tp, paths, plan_items, phases, port, out_path, settings),
                                     nprocs=tp, join=False, start_method="spawn")
            deadline = time.time() + timeout_s
            while not ctx.join(timeout=5):
                if time.time() > deadline:
                    for p in ctx.processes:
                        p.kill()
                    raise TimeoutError(f"upstream CPU run exceeded {timeout_s} s")
        return json.load(open(out_path))


def cpu_baseline(wl: Workload) -> dict:
    """Upstream on the host cores on a bounded sample: the first file of the checkpoint, loaded
    cold from disk to the shards of all ranks, once with each of upstream's two settings."""
    sample = wl.paths[:1]
    try:
        t = run_reference(wl, sample, [("cold", "e2e_cold", 0, 0, 1e9)], timeout_s=300.0, settings="best")
    except Exception as e:  # noqa: BLE001
        return {"value": None, "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
                "sample": f"failed: {type(e).__name__}: {e}"}
    cold, nbytes = t["cold"]["seconds"][0], t["cold"]["bytes"][0]
    return {"value": round(nbytes / cold / GB, 3), "unit": "GB/s", "cores": os.cpu_count(),
            "kind": "reference",
            "sample": f"upstream fastsafetensors 0.3.2, device cpu, nogds, {wl.tp} gloo ranks, the first file of "
                      f"the {wl.spec.name} checkpoint ({nbytes} data bytes) from disk to shards with the page "
                      f"cache dropped ({cold:.2f} s); the faster of library defaults (one request per file) "
                      f"and the rule of upstream's perf tool (a block per thread), cold GB/s: "
                      f"{t['settings']['tried_gbs']}, used: {t['settings']['used']} {t['settings']['kwargs']}",
            "settings": t["settings"], "numa_nodes": _numa_nodes()}


def reference_arm(args) -> dict:
    rank, _, world = dist_env()
    if rank != 0:
        return {}
    wl = Workload(args, world)
    wl.write(0, lambda: None)
    warmup = max(3, args.warmup)
    cold_steps = wl.e2e_steps(args)
    phases = [("cold", "e2e_cold", cold_steps, 1, 1e9), ("warm", "e2e_warm", min(args.steps, 3), 1, 1e9),
              ("resident", "resident", args.steps, warmup, args.ref_budget)]
    if args.no_e2e:
        phases = phases[2:]
    try:
        t = run_reference(wl, wl.paths, phases, timeout_s=800.0, settings=args.ref_settings)
    except Exception as e:  # noqa: BLE001
        if args.ref_settings == "defaults":
            raise
        sys.stderr.write(f"[bench] reference arm with settings {args.ref_settings!r} failed "
                         f"({type(e).__name__}: {e}); running upstream's defaults\n")
        t = run_reference(wl, wl.paths, phases, timeout_s=800.0, settings="defaults")

    def rate(ph):
        return sum(ph["bytes"]) / sum(ph["seconds"]) / GB

    res = t["resident"]
    res_s = sum(res["seconds"]) / len(res["seconds"])
    v = round(rate(res), 3)
    whole = res["files"] == len(wl.paths)
    used = f"settings {t['settings']['used']} {t['settings']['kwargs']}"
    sample = (f"upstream fastsafetensors 0.3.2 (oracle/_ref), device cpu, nogds, {wl.tp} gloo ranks on "
              f"{os.cpu_count()} cores; file images resident in host memory -> every tensor of the plan through "
              f"get_sharded / get_tensor / push_tensor (upstream's shuffle phase), "
              + ("whole checkpoint per step" if whole else
                 f"first {res['files']} of {len(wl.paths)} files per step (the whole checkpoint would not fit "
                 f"{args.ref_budget:.0f} s)") + f"; {used}")
    out = {
        "impl": "reference",
        "metric": METRIC,
        "value": v, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(res_s * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": wl.config_block(),
        "notes": {"value_phase": "file images resident in host memory -> shards in host memory "
                                 "(upstream's shuffle phase, gloo)",
                  "whole_checkpoint_per_step": whole},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": os.cpu_count(), "kind": "reference",
                         "sample": sample, "numa_nodes": _numa_nodes(), "settings": t["settings"]},
        "gpu_launches": 0,
    }
    if "cold" in t:
        cold = t["cold"]
        out["e2e"] = {"value": round(rate(cold), 3), "unit": "GB/s", "h2d_bytes_per_step": 0,
                      "d2h_bytes_per_step": 0, "steps": len(cold["seconds"]), "warmup": 1,
                      "s_per_step": round(sum(cold["seconds"]) / len(cold["seconds"]), 3),
                      "page_cache": "dropped before every step",
                      "what": "files on disk -> shards in host memory, whole checkpoint per step; "
                              f"cold GB/s of one untimed step with each of upstream's settings: "
                              f"{t['settings']['tried_gbs']}; {used}"}
        out["e2e_warm"] = {"value": round(rate(t["warm"]), 3), "unit": "GB/s", "steps": len(t["warm"]["seconds"])}
    else:
        out["e2e"] = {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    return out


_json_fd = None


def emit(line: dict) -> None:
    os.write(_json_fd, (json.dumps(line) + "\n").encode())


def main() -> None:
    global _json_fd
    args = parse_args()
    # stdout carries the one JSON line and nothing else: libraries that print to file
    # descriptor 1 (NCCL's version banner, for one) are sent to stderr for the whole run
    sys.stdout.flush()
    _json_fd = os.dup(1)
    os.dup2(2, 1)
    out = reference_arm(args) if args.impl == "reference" else b200_arm(args)
    sys.stdout.flush()
    parity_ok = True
    if out:
        parity_ok = out.get("parity", {}).get("ok", out.get("parity_ok", True))
        if "parity_ok" not in out:
            emit(out)
    os.close(_json_fd)
    if not parity_ok:
        sys.exit(3)


if __name__ == "__main__":
    main()
