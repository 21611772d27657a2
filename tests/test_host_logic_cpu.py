"""Host-side logic that needs no GPU: argument parsing, initialisers, buffer layout, and the
2-rank data-parallel identity (gloo) the multi-GPU trainer relies on."""
import math
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from minitensor_b200 import mlp, nn


def test_pair_parsing():
    assert nn._pair(2, "stride") == (2, 2)
    assert nn._pair((1, 3), "stride") == (1, 3)
    with pytest.raises(ValueError):
        nn._pair((1, 2, 3), "stride")
    with pytest.raises(ValueError):
        nn._pair("1", "stride")


def test_init_bounds_follow_reference():
    rng = np.random.default_rng(0)
    w = nn.xavier_uniform((128, 784), rng=rng)          # sqrt(6 / (fan_in + fan_out))
    assert w.dtype == np.float32 and np.abs(w).max() <= math.sqrt(6.0 / (784 + 128))
    w = nn.he_uniform((128, 784), rng=rng)              # sqrt(6 / fan_in)
    assert np.abs(w).max() <= math.sqrt(6.0 / 784) and np.abs(w).max() > 0.9 * math.sqrt(6.0 / 784)
    w = nn.he_uniform((64, 64, 3, 3), rng=rng)          # conv: fan_in = C_in * kH * kW
    assert np.abs(w).max() <= math.sqrt(6.0 / 576)


def test_normal_initialisers_follow_reference():
    """he_normal: std sqrt(2 / fan_in) (engine/src/nn/init.rs:432-443), the large conv config's weights;
    xavier_normal: std sqrt(2 / (fan_in + fan_out)); fans of vectors and scalars as calculate_fan_in_fan_out."""
    rng = np.random.default_rng(1)
    w = nn.he_normal((64, 64, 3, 3), rng=rng)
    assert w.dtype == np.float32 and w.shape == (64, 64, 3, 3)
    assert abs(float(w.std()) / math.sqrt(2.0 / 576) - 1.0) < 0.02 and abs(float(w.mean())) < 3e-3
    w = nn.he_normal((512, 2048), rng=rng)
    assert abs(float(w.std()) / math.sqrt(2.0 / 2048) - 1.0) < 0.01
    w = nn.xavier_normal((300, 500), rng=rng)
    assert abs(float(w.std()) / math.sqrt(2.0 / 800) - 1.0) < 0.02
    assert nn._fans(()) == (1, 1) and nn._fans((7,)) == (7, 7) and nn._fans((3, 5)) == (5, 3)
    assert nn._fans((8, 4, 3, 3)) == (36, 72)
    w = nn.init_tensor("lecun_uniform", (10, 48), rng=rng)
    assert np.abs(w).max() <= math.sqrt(3.0 / 48)
    assert (nn.init_tensor(("constant", 0.1), (4,)) == np.float32(0.1)).all()
    u = nn.init_tensor(("uniform", -2.0, 3.0), (1000,), rng=rng)
    assert u.min() >= -2.0 and u.max() <= 3.0 and u.max() > 2.5
    g = nn.init_tensor(("normal", 5.0, 0.5), (20000,), rng=rng)
    assert abs(float(g.mean()) - 5.0) < 0.02 and abs(float(g.std()) - 0.5) < 0.02
    with pytest.raises(ValueError):
        nn.init_tensor("orthogonal", (3, 3))


def test_flat_layout_and_flops():
    dims = [8192, 4096, 4096, 4096, 1000]
    w_off, b_off, total = mlp.mlp_layout(dims)
    assert total == 71_218_152                      # parameter count of the large MLP config
    assert w_off[0] == 0 and b_off[0] == 8192 * 4096 and w_off[1] == b_off[0] + 4096
    assert mlp.mlp_flops_per_sample(dims) == 360_120_320
    assert mlp.mlp_flops_per_sample([784, 128, 10]) == 3 * 2 * (784 * 128 + 128 * 10) - 2 * 784 * 128
    assert mlp.shard_rows(65536, 8, 3) == (3 * 8192, 4 * 8192)
    with pytest.raises(ValueError):
        mlp.shard_rows(10, 4, 0)


def _dp_worker(rank, world, port, dims, x, labels, params, out):
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = mlp.shard_rows(x.shape[0], world, rank)
    p = params.copy()
    m, v = np.zeros_like(p), np.zeros_like(p)
    # gradients of the local-shard mean loss (the Adam update inside is discarded)
    _, g = oracle.mlp_train_step(dims, x[lo:hi], labels[lo:hi], p, m, v, 0.0, 0.9, 0.999, 1e-8, 1, want_grads=True)
    t = torch.from_numpy(g)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)        # what MLPTrainer does per layer slice
    t *= 1.0 / world                                # what its Adam launch applies as grad_scale
    if rank == 0:
        out.put(t.numpy().copy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_average_equals_full_batch():
    """Row-sharding + all-reduce(sum) / world reproduces the full-batch mean-loss gradient."""
    import oracle
    oracle.build()
    rng = np.random.default_rng(3)
    dims = [12, 9, 5]
    x = rng.standard_normal((16, 12)).astype(np.float32)
    labels = rng.integers(0, 5, 16)
    _, _, total = mlp.mlp_layout(dims)
    params = (rng.standard_normal(total) * 0.3).astype(np.float32)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 500)
    procs = [ctx.Process(target=_dp_worker, args=(r, 2, port, dims, x, labels, params, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    p = params.copy()
    _, full = oracle.mlp_train_step(dims, x, labels, p, np.zeros_like(p), np.zeros_like(p), 0.0, 0.9, 0.999, 1e-8, 1,
                                    want_grads=True)
    np.testing.assert_allclose(got, full, rtol=1e-5, atol=1e-6)


def test_host_binding_follows_nvml_and_never_raises(monkeypatch):
    """hostmem.bind_host_to_gpu: with no NVML answer it returns None and leaves the affinity alone; with an NVML that
    names a subset of the allowed CPUs as local to the GPU (a fake module here) the process is bound to that subset."""
    import os
    import sys
    import types
    from minitensor_b200 import hostmem
    before = os.sched_getaffinity(0)
    try:
        assert hostmem.bind_host_to_gpu(0) is None or isinstance(hostmem.bind_host_to_gpu(0), dict)
        os.sched_setaffinity(0, before)
        if len(before) < 2:
            return
        want = sorted(before)[: len(before) // 2]
        words = [0] * ((max(before) // 64) + 1)
        for c in want:
            words[c // 64] |= 1 << (c % 64)
        fake = types.SimpleNamespace(
            nvmlInit=lambda: None, nvmlShutdown=lambda: None,
            nvmlDeviceGetCpuAffinity=lambda handle, n: (words + [0] * n)[:max(n, len(words))])
        monkeypatch.setitem(sys.modules, "pynvml", fake)
        monkeypatch.setattr(hostmem, "_nvml_handle", lambda nvml, index: object())
        info = hostmem.bind_host_to_gpu(0)
        assert info == {"cpus": len(want), "first": want[0], "last": want[-1]}
        assert os.sched_getaffinity(0) == set(want)
        # a mask that names every allowed CPU (one node) changes nothing
        os.sched_setaffinity(0, before)
        for c in before:
            words[c // 64] |= 1 << (c % 64)
        assert hostmem.bind_host_to_gpu(0) is None
        assert os.sched_getaffinity(0) == before
    finally:
        os.sched_setaffinity(0, before)


def test_traffic_records_are_folded_from_ncu_csv(tmp_path, monkeypatch):
    """bench.record_traffic: the long CSV form ncu writes with --csv --log-file (one row per launch and metric,
    units in their own column) becomes a per-launch mean in profiles/dram_traffic.json; expressions joined by
    ' + ' record the sum of their means (a call made of a tensor kernel and its fix-up)."""
    import json
    import bench
    (tmp_path / "profiles").mkdir()
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    rows = ['"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size",'
            '"Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"']
    def add(i, kernel, name, unit, value):
        rows.append(f'"{i}","1","python","box","{kernel}","1","7","(256, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","{name}","{unit}","{value}"')
    add(0, "void mtb::gemm_split_umma2_kernel<64, 3>(A)", "dram__bytes_read.sum", "Mbyte", "300")
    add(0, "void mtb::gemm_split_umma2_kernel<64, 3>(A)", "dram__bytes_write.sum", "Mbyte", "40")
    add(0, "void mtb::gemm_split_umma2_kernel<64, 3>(A)", "gpu__time_duration.sum", "us", "270")
    add(1, "mtb::tail_fixup_kernel(G)", "dram__bytes_read.sum", "Kbyte", "9,000")
    add(1, "mtb::tail_fixup_kernel(G)", "dram__bytes_write.sum", "byte", "11000000")
    add(2, "void mtb::gemm_split_umma2_kernel<64, 3>(A)", "dram__bytes_read.sum", "Mbyte", "320")
    add(2, "void mtb::gemm_split_umma2_kernel<64, 3>(A)", "dram__bytes_write.sum", "Mbyte", "40")
    csv_path = tmp_path / "list.csv"
    csv_path.write_text("==PROF== banner line\n" + "\n".join(rows) + "\n")
    rec = bench.record_traffic(str(csv_path), "k.only", "gemm_split_umma2", "ncu ... cmd")
    assert rec["launches_captured"] == 2 and abs(rec["dram_bytes_per_launch"] - 350e6) < 1
    rec = bench.record_traffic(str(csv_path), "k.call", "gemm_split_umma2 + tail_fixup", "ncu ... cmd")
    assert abs(rec["dram_bytes_per_launch"] - (350e6 + 20e6)) < 1 and rec["launches_captured"] == 3
    data = json.load(open(tmp_path / "profiles" / "dram_traffic.json"))
    assert set(data) == {"k.only", "k.call"} and data["k.call"]["command"] == "ncu ... cmd"
    with pytest.raises(SystemExit):
        bench.record_traffic(str(csv_path), "k.none", "no_such_kernel", "cmd")
