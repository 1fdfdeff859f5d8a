"""The N > 1 path of bench.py on the host: independent replicas, one process each, that meet only in a gloo barrier and one
gather of their per-rank records; rank 0 alone aggregates and prints.  Runs as two gloo ranks on the CPU (no GPU work: the
records are synthetic), plus the pure helpers the aggregation relies on."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RANK_SCRIPT = textwrap.dedent('''
    import json, os, sys
    sys.path.insert(0, %(root)r)
    import torch.distributed as dist
    import bench
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cores = bench.rank_cores(rank, world)
    # what a replica reports: rank 1 is the slower, noisier one
    local = {"be_sps": 1600.0 + 50 * rank, "be_sps_e2e": 1500.0 + 40 * rank, "be_solo_sps": 2100.0,
             "hp_p99": 2.7 + 0.3 * rank, "hp_solo_p99": 2.5, "timed_s": 25.0 + rank, "cores": cores, "rank": rank}
    dist.barrier()
    gathered = [None] * world
    dist.all_gather_object(gathered, local)
    if rank == 0:
        worst, value, e2e_value, step_time, solo_sum = bench.aggregate_ranks(gathered)
        print(json.dumps({"worst_rank": worst["rank"], "value": value, "e2e": e2e_value, "step_time": step_time, "solo": solo_sum,
                          "cores": [g["cores"] for g in gathered]}))
    dist.destroy_process_group()
''')


def test_two_replicas_gather_on_rank0_and_share_no_core(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(RANK_SCRIPT % {"root": ROOT})
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29653",
                   OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env))
    outs = [p.communicate(timeout=180) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1][-2000:] for o in outs]
    assert outs[1][0].strip() == ""                         # only rank 0 prints
    r = json.loads(outs[0][0].strip().splitlines()[-1])
    assert r["worst_rank"] == 1                             # latency ratio 3.0 / 2.5 against 2.7 / 2.5
    assert r["value"] == 1600.0 + 1650.0 and r["e2e"] == 1500.0 + 1540.0 and r["solo"] == 4200.0
    assert r["step_time"] == 26.0                           # the longest rank's timed region
    a, b = r["cores"]
    if a is not None and b is not None:                     # enough cores to give each replica three or more
        assert len(a) == len(b) >= 3 and not set(a) & set(b)


def test_window_rate_and_paired_bootstrap():
    sys.path.insert(0, ROOT)
    import bench
    # 11 iteration ends 0.1 s apart, window covers ends 2..8 -> 6 intervals of batch 32 in 0.6 s
    be = {"iteration_end_times": [0.1 * i for i in range(11)], "batchsize": 32, "samples_per_s": 1.0}
    rate, n = bench.be_rate_in_window(be, 0.15, 0.85)
    assert n == 7 and abs(rate - 6 * 32 / 0.6) < 1e-6
    assert bench.be_rate_in_window(be, 5.0, 6.0) == (1.0, 0)      # nothing inside: falls back to the client's own figure
    # identical latency lists: the ratio and its interval are exactly one
    lat = [1.0 + 0.01 * (i % 17) for i in range(400)]
    lo, hi = bench.paired_bootstrap_p99_ratio(lat, lat)
    assert lo == hi == 1.0
    lo, hi = bench.paired_bootstrap_p99_ratio([1.2 * v for v in lat], lat)
    assert abs(lo - 1.2) < 1e-9 and abs(hi - 1.2) < 1e-9
