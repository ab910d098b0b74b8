"""The benchmark's command-line contract where no GPU is present: the reference arm answers with its one-line
``unavailable`` record and exit code 0, the options the drivers pass are accepted, and the torch-2.11 shims for the
reference package install the names they promise."""
import json
import subprocess
import sys

import pytest
import torch


def test_reference_arm_reports_unavailable_without_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    p = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-500:]
    rec = json.loads(p.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec and "\n" not in rec["unavailable"]


def test_benchmark_options():
    sys.argv, saved = ["bench.py", "--gpus", "4", "--steps", "7", "--warmup", "3", "--deterministic", "--watchdog", "0"], sys.argv
    try:
        import bench

        args = bench.parse()
    finally:
        sys.argv = saved
    assert (args.gpus, args.steps, args.warmup, args.impl) == (4, 7, 3, "ours")
    assert args.deterministic and args.watchdog == 0 and args.seq_len == 8192 and args.local_batch == 1
    assert args.placement == "shard" and args.layers == 32


def test_compat_shims_install_the_promised_names():
    """``baseline/compat.py`` gives torch 2.11 the names the reference package imports (plain PyTorch equivalents)."""
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp

    from baseline import compat

    compat.install()
    assert hasattr(dcp, "CheckpointableTensor")
    assert callable(dist.all_gather_single) and callable(dist.reduce_scatter_single)
    assert hasattr(dist, "_spmd_no_typecheck") and hasattr(dist, "_is_spmd_types_available")
    assert hasattr(torch.ops.fsdp, "_all_gather_copy_out_") and hasattr(torch.ops.fsdp, "chunk_cat_mixed_dtype")
    assert hasattr(torch.Tensor, "_has_grad_dtype_override")
    # the copy-out shim scatters a gathered [world, row] buffer into per-parameter outputs: rank-major rows for
    # dim-0 shards, interleaved back along the leading dimension for an inner-dim shard
    src = torch.arange(12.0).view(2, 6)                      # world 2, row = [2 | 4] elements
    outs = [torch.zeros(4), torch.zeros(8)]
    torch.ops.fsdp._all_gather_copy_out_(outs, src, [2, 4], [1, 1], 2)
    assert torch.equal(outs[0].view(2, 2), src[:, :2]) and torch.equal(outs[1].view(2, 4), src[:, 2:])
    inner = [torch.zeros(2, 4)]                              # a [2, 4] parameter sharded on dim 1: 2 leading rows
    torch.ops.fsdp._all_gather_copy_out_(inner, src[:, 2:].contiguous(), [4], [2], 2)
    want = torch.stack([src[r, 2:].view(2, 2) for r in range(2)], dim=1).reshape(2, 4)
    assert torch.equal(inner[0], want)
    compat.install()                                  # installing twice is harmless


def test_clock_sampler_reads_clocks_and_throttle_reasons_from_a_fake_nvml(monkeypatch):
    """The benchmark only reads the GPU's state (clocks, throttle reasons) while the timed region runs; against a fake
    NVML module: the median SM clock, the maximum clock, the reasons decoded from the bit mask, the physical index taken
    from CUDA_VISIBLE_DEVICES, and no call that would change a setting."""
    import sys
    import time
    import types

    calls = []
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    fake.nvmlInit = lambda: calls.append("init")
    fake.nvmlDeviceGetHandleByIndex = lambda i: calls.append(("handle", i)) or f"gpu{i}"
    seq = iter([1300.0, 1400.0, 1350.0] + [1350.0] * 1000)
    fake.nvmlDeviceGetClockInfo = lambda h, kind: next(seq)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965.0
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4 | 0x1      # power cap + "gpu idle" (not a reported reason)

    def forbidden(*a, **k):
        raise AssertionError("the benchmark must not change a GPU setting")

    for name in ("nvmlDeviceSetApplicationsClocks", "nvmlDeviceSetGpuLockedClocks", "nvmlDeviceResetGpuLockedClocks",
                 "nvmlDeviceSetPowerManagementLimit", "nvmlDeviceSetPersistenceMode"):
        setattr(fake, name, forbidden)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "5,6")
    import bench

    s = bench.ClockSampler(1)
    assert ("handle", 6) in calls                                            # local index 1 is physical GPU 6
    s.start()
    time.sleep(0.35)
    rec = s.stop()
    assert rec["source"] == "nvml" and rec["samples"] >= 3
    assert rec["sm_mhz"] == 1350.0 and rec["sm_max_mhz"] == 1965.0
    assert rec["reasons"] == ["sw_power_cap"]
