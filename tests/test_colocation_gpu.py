"""End to end on one GPU: profile both clients, run HP solo and the HP/BE pair under the scheduler
through benchmarking/launch_jobs.py with the capture library preloaded."""
import os

import pytest

pytestmark = pytest.mark.gpu


def test_profile_then_colocate(built, tmp_path):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from orion_b200 import experiments as E
    out = str(tmp_path)
    env = {"ORION_GATE_TIMEOUT_S": 15}
    hp = E.profile_client("resnet50_hp", os.path.join(out, "profiles"), timeout=240)
    be = E.profile_client("resnet50_be", os.path.join(out, "profiles"), timeout=240)
    assert hp[3] == 53 + 3 + 1, "prepared ResNet-50 inference: 53 convolutions, 3 other kernels, 1 channel padding of the image"
    assert be[3] > 400
    with open(hp[2]) as f:
        assert f.readline().strip() == "Name,Profile,Memory_footprint,SM_usage,Duration"
        rows = [l.rstrip("\n").split(",") for l in f]
    assert all(len(r) == 5 for r in rows)
    # every implicit-GEMM launch announces its class from its arithmetic intensity: deep layers compute-bound (1),
    # the shallow 1x1 layers and the stem memory-bound (0); none is left unknown
    igemm = [r for r in rows if "igemm" in r[0]]
    assert len(igemm) == 54 and all(r[1] in ("0", "1") for r in igemm)
    assert sum(1 for r in igemm if r[1] == "1") >= 40
    assert all(r[1] == "0" for r in rows if "pool" in r[0] or "pad_channels" in r[0])

    solo = E.run_launch_jobs([E.client_entry("resnet50_hp", hp, 130, rps=80)], os.path.join(out, "solo"), extra_env=env, timeout=180)
    hp_solo = solo["clients"][0]
    assert hp_solo["iterations"] == 130 and 0 < hp_solo["p50_latency"] < 50
    assert solo["scheduler"]["stats"]["join_timeouts"] == 0

    pair = [E.client_entry("resnet50_be", be, 100000), E.client_entry("resnet50_hp", hp, 130, rps=80)]
    depth = int(0.025 * hp_solo["p50_latency"] * 1e6)
    trace = os.path.join(out, "pair.obs")
    co = E.run_launch_jobs(pair, os.path.join(out, "pair"), depth=depth, extra_env=dict(env, ORION_RECORD_OBS=trace), timeout=240)
    be_c, hp_c = co["clients"]
    assert hp_c["iterations"] == 130
    assert be_c["iterations"] >= 11 and be_c["samples_per_s"] > 0
    st = co["scheduler"]["stats"]
    assert st["hp_submits"] > 0 and st["be_submits"] > 0 and st["join_timeouts"] == 0
    assert co["scheduler"]["own_launches"] > 130 * 50
    assert hp_c["p99_latency"] < 20 * hp_solo["p99_latency"]

    # The decisions this run took on the GPU, checked against the compiled reference scheduler fed the same queue heads,
    # event-query answers, clock reads and stop acknowledgements (oracle/ref_driver.cpp, observation mode).
    import json
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref = os.path.join(root, "oracle", "_ref", "ref_replay")
    assert os.path.exists(trace)
    if os.path.exists(ref):
        r = subprocess.run([ref, "--observations", trace, os.path.join(root, "oracle", "_ref")], capture_output=True, text=True,
                           timeout=300)
        rep = json.loads(r.stdout.strip().splitlines()[-1])
        assert r.returncode == 0 and rep["matched"] is True, rep
        assert rep["decisions"] > 130 * 50
        if not rep["truncated"] and st["forced_iter_ends"] == 0:
            assert rep["decisions"] >= st["hp_submits"] + st["be_submits"]


def test_best_effort_stream_inside_a_green_context_partition(built, tmp_path):
    """ORION_BE_SM_QUOTA=64: the scheduler creates the best-effort client's stream inside a green context that owns 64 SMs
    (the hardware keeps that client's kernels off the other 84), reports the partition it got, and the pair still runs to
    completion with every op scheduled."""
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device")
    from orion_b200 import experiments as E
    out = str(tmp_path)
    env = {"ORION_GATE_TIMEOUT_S": 15, "ORION_BE_SM_QUOTA": 64}
    hp = E.profile_client("resnet50_hp", os.path.join(out, "profiles"), timeout=240)
    be = E.profile_client("resnet50_be", os.path.join(out, "profiles"), timeout=240)
    pair = [E.client_entry("resnet50_be", be, 100000), E.client_entry("resnet50_hp", hp, 100, rps=80)]
    co = E.run_launch_jobs(pair, os.path.join(out, "pair"), depth=34000, extra_env=env, timeout=240)
    be_c, hp_c = co["clients"]
    st = co["scheduler"]["stats"]
    assert st["green_be_sms"] == 64, "the driver granted a partition of another size (granularity is 8 SMs on B200)"
    assert hp_c["iterations"] == 100 and be_c["iterations"] >= 11
    assert st["join_timeouts"] == 0 and st["forced_iter_ends"] == 0
