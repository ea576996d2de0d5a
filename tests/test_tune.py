"""Reader settings from the host topology (a fake sysfs tree) and from upstream's environment
variables (examples/tgis_weight.py:19-55)."""

import pytest

from fastsafetensors_b200 import tune


def make_sysfs(root, nodes, smt=2, l2_kb=2048):
    """nodes: list of lists of logical cpu ids; consecutive groups of `smt` cpus share a core and
    an L2."""
    for n, cpus in enumerate(nodes):
        d = root / "devices/system/node" / f"node{n}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(",".join(str(c) for c in cpus) + "\n")
        for i, c in enumerate(cpus):
            base = root / "devices/system/cpu" / f"cpu{c}"
            (base / "topology").mkdir(parents=True)
            (base / "topology/core_id").write_text(f"{i // smt}\n")
            (base / "topology/physical_package_id").write_text(f"{n}\n")
            sib = cpus[(i // smt) * smt:(i // smt) * smt + smt]
            for idx, (level, size) in enumerate([("1", "48K"), ("1", "32K"), ("2", f"{l2_kb}K"), ("3", "32M")]):
                cd = base / "cache" / f"index{idx}"
                cd.mkdir(parents=True)
                (cd / "level").write_text(level + "\n")
                (cd / "size").write_text(size + "\n")
                (cd / "shared_cpu_list").write_text(",".join(str(s) for s in sib) + "\n")
    return str(root)


def test_cpu_list_parsing():
    assert tune._parse_cpu_list("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert tune._parse_cpu_list("") == set()
    assert tune._size_kb("2048K") == 2048 and tune._size_kb("2M") == 2048 and tune._size_kb(None) == 0


def test_topology_counts_cores_and_distinct_l2(tmp_path):
    sysfs = make_sysfs(tmp_path, [list(range(0, 32)), list(range(32, 64))])
    t = tune.HostTopology.probe(1, sysfs, allowed=set(range(64)))
    assert t.node == 1 and t.cpus == tuple(range(32, 64))
    assert t.physical_cores == 16
    assert t.l2_kb == 16 * 2048          # one L2 per core, not per hyperthread
    # affinity narrows it
    t = tune.HostTopology.probe(1, sysfs, allowed={32, 33, 34, 0})
    assert t.cpus == (32, 33, 34) and t.physical_cores == 2
    # affinity outside the node: run where allowed
    t = tune.HostTopology.probe(1, sysfs, allowed={0, 1})
    assert t.cpus == (0, 1)
    # unknown node: all CPUs listed
    t = tune.HostTopology.probe(None, sysfs, allowed=set(range(64)))
    assert len(t.cpus) == 64 and t.node == -1


def test_suggest_divides_cpus_among_local_ranks(tmp_path):
    sysfs = make_sysfs(tmp_path, [list(range(64))])
    topo = tune.HostTopology.probe(0, sysfs, allowed=set(range(64)))
    s = tune.suggest(None, local_world=1, topology=topo, gds=False)
    assert (s.max_threads, s.slot_kb, s.nogds, s.io_mode) == (16, 4096, True, "auto")
    assert s.bbuf_size_kb == 16 * 2 * 4096
    assert tune.suggest(None, local_world=8, topology=topo, gds=False).max_threads == 8
    assert tune.suggest(None, local_world=64, topology=topo, gds=False).max_threads == 2
    s = tune.suggest(None, local_world=8, topology=topo, gds=True)
    assert s.nogds is False and s.io_mode == "auto"
    kw = s.loader_kwargs()
    assert set(kw) == {"nogds", "max_threads", "bbuf_size_kb", "slot_kb", "io_mode"}


def test_gds_usable_needs_driver_and_udev(tmp_path):
    mods = tmp_path / "modules"
    mods.write_text("nvidia_uvm 1 0 - Live 0x0\nnvidia 2 1 nvidia_uvm, Live 0x0\n")
    udev = tmp_path / "udev"
    udev.mkdir()
    assert not tune.gds_usable(str(udev), str(mods))
    mods.write_text("nvidia_fs 1 0 - Live 0x0\nnvidia 2 1 - Live 0x0\n")
    assert tune.gds_usable(str(udev), str(mods))
    assert not tune.gds_usable(str(tmp_path / "missing"), str(mods))


def test_auto_config_env(monkeypatch):
    for k in ("FST_CONFIG", "FST_NOGDS", "FST_THREADS", "FST_BBUF_SIZE_KB", "LOCAL_WORLD_SIZE"):
        monkeypatch.delenv(k, raising=False)
    monkeypatch.setenv("FST_CONFIG", "manual")
    assert tune.auto_config(None) == (False, 16, 163840)
    monkeypatch.setenv("FST_NOGDS", "1")
    monkeypatch.setenv("FST_THREADS", "4")
    monkeypatch.setenv("FST_BBUF_SIZE_KB", "8192")
    assert tune.auto_config(None) == (True, 4, 8192)
    monkeypatch.setenv("FST_CONFIG", "auto")
    nogds, threads, bbuf = tune.auto_config(None)
    assert 2 <= threads <= 16 and bbuf == threads * 2 * 4096
    assert nogds == (not tune.gds_usable())


def test_settings_drive_a_loader(tmp_path):
    import numpy as np
    import torch
    from safetensors.torch import save_file

    import fastsafetensors_b200 as fst

    path = str(tmp_path / "a.safetensors")
    raw = (np.arange(4096) % 251).astype(np.uint8)
    save_file({"t": torch.from_numpy(raw.copy())}, path)
    s = tune.suggest(None, local_world=4, gds=False)
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cpu", **s.loader_kwargs())
    loader.add_filenames({0: [path]})
    fb = loader.copy_files_to_device()
    assert np.array_equal(fb.get_tensor("t").numpy(), raw)
    fb.close()
    loader.close()


@pytest.mark.gpu
def test_suggested_settings_load_onto_the_gpu(tmp_path):
    """The tuner asks the native library for the device's NUMA node; whatever it answers, the
    suggested settings must load a file onto the device byte for byte."""
    import numpy as np
    import torch
    from safetensors.torch import save_file

    import fastsafetensors_b200 as fst

    s = tune.suggest(0)
    assert 2 <= s.max_threads <= 16 and s.bbuf_size_kb == s.max_threads * 2 * s.slot_kb
    path = str(tmp_path / "g.safetensors")
    raw = np.random.default_rng(5).integers(0, 256, (3 << 20) + 17, dtype=np.uint8)
    save_file({"t": torch.from_numpy(raw.copy())}, path)
    loader = fst.SafeTensorsFileLoader(fst.SingleGroup(), "cuda:0", **s.loader_kwargs())
    loader.add_filenames({0: [path]})
    fb = loader.copy_files_to_device()
    assert np.array_equal(fb.get_tensor("t").cpu().numpy(), raw)
    fb.close()
    loader.close()
