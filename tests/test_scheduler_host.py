"""Live scheduler + capture library on the host: client threads queue ops through the
lock-free rings, the scheduler thread grants them (ORION_FAKE_GPU=1: every event is
complete at once).  Each scenario runs in a child process because the libraries keep
process-wide state."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DRIVER = textwrap.dedent('''
    import ctypes, json, sys, threading, time
    sys.path.insert(0, %(root)r)
    from src.scheduler_frontend import PyScheduler
    cap = ctypes.CDLL(%(root)r + "/orion_b200/lib/liborion_capture.so", mode=ctypes.RTLD_GLOBAL)
    sched = ctypes.CDLL(%(root)r + "/orion_b200/lib/liborion_sched.so")
    cap.stop.restype = ctypes.c_bool
    cfg = json.loads(sys.argv[1])
    N = len(cfg["clients"])
    barriers = [threading.Barrier(N + 1)]
    done = [0] * N
    wrong = []
    quotas = [set() for _ in range(N)]
    def client(i):
        c = cfg["clients"][i]
        barriers[0].wait()
        it = 0
        while it < c["iters"]:
            for t in (c.get("first_ops") if it == 0 and c.get("first_ops") else c["ops"]):
                got = cap.orion_capture_op(t)
                if got != i: wrong.append((i, got))
                if t == 0: quotas[i].add(cap.orion_capture_last_quota())
            cap.block(it)
            for t in c.get("after", []):
                cap.orion_capture_op(t)
            it += 1
            done[i] = it
            if it == 1 or it == 10: barriers[0].wait()
            if cap.stop(): break
        barriers[0].wait()
    ths = [threading.Thread(target=client, args=(i,)) for i in range(N)]
    for t in ths: t.start()
    ps = PyScheduler(sched, N)
    st = threading.Thread(target=ps.run_scheduler, args=(
        barriers, [t.native_id for t in ths], ["m"] * N, [c["profile"] for c in cfg["clients"]], [None] * N,
        [c["num_kernels"] for c in cfg["clients"]], [None] * N, [c["iters"] for c in cfg["clients"]], True, True,
        cfg.get("reef", False), cfg.get("sequential", False), cfg.get("depth", 160000), cfg.get("hp_limit", 1), cfg.get("update_start", 1),
        [c["train"] for c in cfg["clients"]]))
    t0 = time.time(); st.start()
    for t in ths: t.join()
    st.join()
    print(json.dumps({"done": done, "wrong": wrong, "stats": ps.stats(), "secs": time.time() - t0,
                      "hp_samples": len(ps.durations_ms(N - 1)), "quotas": [sorted(q) for q in quotas]}))
''')


def _run(cfg, env_extra=None, timeout=120, expect_failure=False):
    env = dict(os.environ, ORION_FAKE_GPU="1", ORION_GATE_TIMEOUT_S="5")
    env.update(env_extra or {})
    out = subprocess.run([sys.executable, "-c", DRIVER % {"root": ROOT}, json.dumps(cfg)], capture_output=True, text=True,
                         timeout=timeout, env=env)
    if expect_failure:
        assert out.returncode != 0
        return out.stderr
    assert out.returncode == 0, out.stderr[-3000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


def _profile(tmp_path, name, rows):
    p = tmp_path / name
    p.write_text("Name,Profile,Memory_footprint,SM_usage,Duration\n" + "".join("k,%d,0,%d,%d\n" % r for r in rows))
    return str(p)


def test_pair_runs_to_completion_and_best_effort_is_stopped(built, tmp_path):
    be = _profile(tmp_path, "be", [(1, 40, 9000), (0, 200, 5000), (-1, 30, 3000)] * 10)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000), (0, 20, 2000)] * 6)
    r = _run({"clients": [{"profile": be, "num_kernels": 30, "iters": 100000, "train": True, "ops": [1] + [0] * 30},
                          {"profile": hp, "num_kernels": 12, "iters": 60, "train": False, "ops": [1] + [0] * 12, "after": [1]}],
              "depth": 20000})
    assert r["done"][1] == 60 and 10 <= r["done"][0] < 100000
    assert not r["wrong"]
    s = r["stats"]
    assert s["hp_submits"] == 60 * 14 - 1 or s["hp_submits"] >= 60 * 13          # 12 kernels + copies per request
    assert s["be_submits"] >= 10 * 31 and s["join_timeouts"] == 0 and s["forced_iter_ends"] == 0
    assert r["hp_samples"] == 60


def test_single_client_and_reef_policy(built, tmp_path):
    p = _profile(tmp_path, "p", [(1, 10, 1000)] * 5)
    r = _run({"clients": [{"profile": p, "num_kernels": 5, "iters": 15, "train": False, "ops": [0] * 5}]})
    assert r["done"] == [15] and r["stats"]["hp_submits"] == 75
    be = _profile(tmp_path, "be", [(1, 100, 500)] * 4)
    r = _run({"reef": True, "depth": 3, "clients": [{"profile": be, "num_kernels": 4, "iters": 100000, "train": True, "ops": [0] * 4},
                                                     {"profile": p, "num_kernels": 5, "iters": 30, "train": False, "ops": [0] * 5}]})
    assert r["done"][1] == 30 and r["done"][0] >= 10


def test_profile_longer_than_the_op_stream_does_not_deadlock(built, tmp_path):
    """The client issues 4 ops per request, the profile announces 6: the scheduler closes the
    request when the client is already waiting for it (the reference would hang here)."""
    p = _profile(tmp_path, "p", [(1, 10, 1000)] * 6)
    r = _run({"clients": [{"profile": p, "num_kernels": 6, "iters": 14, "train": False, "ops": [0] * 4}]})
    assert r["done"] == [14]
    assert r["stats"]["forced_iter_ends"] == 14


def test_profile_shorter_than_the_op_stream_keeps_running(built, tmp_path):
    p = _profile(tmp_path, "p", [(1, 10, 1000)] * 3)
    r = _run({"clients": [{"profile": p, "num_kernels": 3, "iters": 13, "train": False, "ops": [0] * 5}]}, timeout=180)
    assert r["done"] == [13]


def test_first_request_longer_than_its_profile_degrades_instead_of_stalling(built, tmp_path):
    """An inference client whose first request launches one-time work (here 40 ops) under a profile that only describes the
    steady state (5 rows): the scheduler closes eight "iterations" inside that first request and moves through its phases ahead
    of the client.  The client must come through: it waits out one grant timeout per scheduler pause, runs the rest of the
    pause unscheduled, and every request completes."""
    import time
    p = _profile(tmp_path, "p", [(1, 10, 1000)] * 5)
    t0 = time.time()
    r = _run({"clients": [{"profile": p, "num_kernels": 5, "iters": 16, "train": False, "ops": [0] * 5, "first_ops": [0] * 40}]},
             env_extra={"ORION_GATE_TIMEOUT_S": "2"}, timeout=170)
    assert r["done"] == [16]
    assert time.time() - t0 < 120


def test_recorded_run_replays_identically_through_policy_core_and_oracles(built, tmp_path):
    """ORION_RECORD_SCRIPT: the live scheduler writes its measured phase as an arrival script.  The same
    script must give one decision log whether it is replayed by the product's policy core, by the Python
    restatement, or (where it was compiled) by the reference scheduler itself."""
    import hashlib
    from oracle import policy_oracle
    be = _profile(tmp_path, "be", [(1, 40, 9000), (0, 200, 5000), (-1, 30, 3000)] * 8)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000), (0, 20, 2000)] * 5)
    script = tmp_path / "recorded.script"
    r = _run({"clients": [{"profile": be, "num_kernels": 24, "iters": 100000, "train": True, "ops": [1] + [0] * 24},
                          {"profile": hp, "num_kernels": 10, "iters": 40, "train": False, "ops": [1] + [0] * 10}],
              "depth": 20000}, env_extra={"ORION_RECORD_SCRIPT": str(script)})
    assert r["done"][1] == 40 and script.exists()
    text = script.read_text()
    assert text.startswith("orion_script 1") and "nclients 2" in text
    log = tmp_path / "product.log"
    out = subprocess.run([built["orion_replay"], str(script), "--log", str(log)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    product = log.read_bytes()
    assert product.count(b"\nS ") > 100
    assert policy_oracle.run_script(str(script)).encode() == product
    ref = os.path.join(ROOT, "oracle", "_ref", "ref_replay")
    if os.path.exists(ref):
        ref_log = tmp_path / "ref.log"
        out = subprocess.run([ref, str(script), os.path.join(ROOT, "oracle", "_ref"), str(ref_log)], capture_output=True, text=True,
                             timeout=300)
        assert out.returncode == 0, out.stderr
        assert hashlib.sha256(ref_log.read_bytes()).hexdigest() == hashlib.sha256(product).hexdigest()


def test_more_kernels_announced_than_profile_rows_ends_the_run_with_a_message(built, tmp_path):
    """The policy indexes the profile with the op counter; a profile shorter than num_kernels (or empty) would be read
    past its end.  setup() refuses it."""
    p = _profile(tmp_path, "p", [(1, 10, 1000)] * 3)
    err = _run({"clients": [{"profile": p, "num_kernels": 5, "iters": 12, "train": False, "ops": [0] * 5}]}, expect_failure=True)
    assert "announces 5 kernels" in err and "3 rows" in err
    empty = _profile(tmp_path, "empty", [])
    err = _run({"clients": [{"profile": empty, "num_kernels": 1, "iters": 12, "train": False, "ops": [0]}]}, expect_failure=True)
    assert "0 rows" in err


def test_more_compute_ops_than_events_in_one_iteration_aborts(built, tmp_path):
    """30000 events exist per client (reference utils_sched.cpp:150); op 30001 of one iteration must not index past them."""
    n = 30001
    p = _profile(tmp_path, "big", [(1, 10, 1000)] * n)
    err = _run({"clients": [{"profile": p, "num_kernels": n, "iters": 12, "train": False, "ops": [0] * n}]}, expect_failure=True,
               timeout=300)
    assert "events per client" in err


def test_best_effort_grants_carry_the_sm_quota_left_by_the_high_priority_op(built, tmp_path):
    """148 SMs; the high-priority ops need 60 and 20 SMs.  A best-effort kernel granted while a high-priority request is in
    flight gets 148 - need rounded down to the partition granularity of 8 (88 or 128); with no request in flight it gets the
    whole device minus the configured reserve (148 - 16 -> 128).  The high-priority client's grants carry no quota."""
    be = _profile(tmp_path, "be", [(1, 40, 9000), (0, 200, 5000), (-1, 30, 3000)] * 10)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000), (0, 20, 2000)] * 6)
    cfg = {"clients": [{"profile": be, "num_kernels": 30, "iters": 100000, "train": True, "ops": [1] + [0] * 30},
                       {"profile": hp, "num_kernels": 12, "iters": 300, "train": False, "ops": [1] + [0] * 12}],
           "depth": 20000}
    r = _run(cfg, env_extra={"ORION_MAX_SMS": "148", "ORION_HP_RESERVE_SMS": "16"})
    assert r["quotas"][1] == [0]
    assert set(r["quotas"][0]) <= {0, 88, 128} and 128 in r["quotas"][0]
    assert r["stats"]["quota_grants"] > 0 and r["stats"]["quota_ctas_sum"] >= 88 * r["stats"]["quota_grants"]
    r = _run(cfg, env_extra={"ORION_MAX_SMS": "148", "ORION_SM_QUOTA": "0"})
    assert r["quotas"] == [[0], [0]] and r["stats"]["quota_grants"] == 0


def test_elastic_kernels_are_cut_to_the_quota_and_others_are_not(built):
    cap = ctypes_lib(built["liborion_capture.so"])
    k1, k2 = 0x7f0000001230, 0x7f0000004560
    assert cap.orion_capture_mark_elastic(k1, 4) == 0
    assert cap.orion_capture_clamp_grid(k1, 592, 88) == 352      # 88 SMs x 4 resident CTAs
    assert cap.orion_capture_clamp_grid(k1, 100, 88) == 100      # already narrower
    assert cap.orion_capture_clamp_grid(k1, 592, 0) == 592       # no quota
    assert cap.orion_capture_clamp_grid(k2, 592, 88) == 592      # not declared elastic
    assert cap.orion_capture_mark_elastic(k1, 1) == 0            # re-declaring changes the factor
    assert cap.orion_capture_clamp_grid(k1, 148, 88) == 88


def ctypes_lib(path):
    import ctypes
    lib = ctypes.CDLL(path)
    lib.orion_capture_mark_elastic.argtypes = [ctypes.c_void_p, ctypes.c_int]
    lib.orion_capture_clamp_grid.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_int]
    lib.orion_capture_clamp_grid.restype = ctypes.c_uint
    return lib


def test_two_best_effort_clients_share_the_device_with_one_high_priority_client(built, tmp_path):
    """Three live clients (the reference's benchmarking/multi_client_example.json has this shape): both best-effort clients
    make progress round-robin, each is stopped when the high-priority client is done, every op reaches the client that
    queued it."""
    be = _profile(tmp_path, "be", [(1, 40, 9000), (0, 60, 5000), (-1, 30, 3000)] * 6)
    be2 = _profile(tmp_path, "be2", [(0, 20, 4000), (1, 50, 7000)] * 10)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000), (0, 20, 2000)] * 6)
    r = _run({"clients": [{"profile": be, "num_kernels": 18, "iters": 100000, "train": True, "ops": [1] + [0] * 18},
                          {"profile": be2, "num_kernels": 20, "iters": 100000, "train": True, "ops": [0] * 20},
                          {"profile": hp, "num_kernels": 12, "iters": 80, "train": False, "ops": [1] + [0] * 12}],
              "depth": 30000}, env_extra={"ORION_MAX_SMS": "148"})
    assert r["done"][2] == 80 and not r["wrong"]
    assert 10 <= r["done"][0] < 100000 and 10 <= r["done"][1] < 100000
    assert r["stats"]["be_submits"] >= 10 * (19 + 20) and r["stats"]["join_timeouts"] == 0 and r["stats"]["forced_iter_ends"] == 0
    assert r["quotas"][2] == [0]


def test_high_priority_training_client_runs_the_update_phase_rule(built, tmp_path):
    """The high-priority client trains (reference scheduler_eval.cpp:338,427-445): best-effort ops are also admitted once
    the high-priority iteration has reached its update phase (op index >= update_start) and the op before it has completed,
    if they need no more than the SM threshold, which is bisected every ten iterations against the tolerated iteration time."""
    be = _profile(tmp_path, "be", [(1, 20, 9000), (0, 30, 5000)] * 8)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000)] * 8 + [(0, 10, 2000)] * 6)
    r = _run({"clients": [{"profile": be, "num_kernels": 16, "iters": 100000, "train": True, "ops": [0] * 16},
                          {"profile": hp, "num_kernels": 14, "iters": 45, "train": True, "ops": [1] + [0] * 14}],
              "depth": 20000, "hp_limit": 1000, "update_start": 8}, env_extra={"ORION_MAX_SMS": "148"})
    assert r["done"][1] == 45 and not r["wrong"]
    assert r["done"][0] >= 10
    assert r["stats"]["queries"] > 0 and r["stats"]["join_timeouts"] == 0
    assert r["hp_samples"] == 45


REF_REPLAY = os.path.join(ROOT, "oracle", "_ref", "ref_replay")


def _check_observations(trace, expect_match=True):
    """Feeds an observation trace to the compiled reference scheduler (oracle/ref_driver.cpp, second mode)."""
    out = subprocess.run([REF_REPLAY, "--observations", str(trace), os.path.join(ROOT, "oracle", "_ref")], capture_output=True,
                         text=True, timeout=300)
    line = out.stdout.strip().splitlines()[-1] if out.stdout.strip() else "{}"
    rep = json.loads(line)
    if expect_match:
        assert out.returncode == 0 and rep.get("matched") is True, (out.returncode, line, out.stderr[-2000:])
    return out.returncode, rep


def _live_scenarios(tmp_path):
    be = _profile(tmp_path, "be", [(1, 40, 9000), (0, 200, 5000), (-1, 30, 3000)] * 8)
    be2 = _profile(tmp_path, "be2", [(0, 20, 4000), (1, 50, 7000)] * 10)
    hp = _profile(tmp_path, "hp", [(1, 60, 8000), (0, 20, 2000)] * 5)
    hpt = _profile(tmp_path, "hpt", [(1, 60, 8000)] * 8 + [(0, 10, 2000)] * 6)
    bes = _profile(tmp_path, "bes", [(1, 20, 9000), (0, 30, 5000)] * 8)
    pair = [{"profile": be, "num_kernels": 24, "iters": 100000, "train": True, "ops": [1] + [0] * 24, "after": [2]},
            {"profile": hp, "num_kernels": 10, "iters": 60, "train": False, "ops": [1] + [0] * 10}]
    return {
        "pair": ({"clients": pair, "depth": 20000}, {}),
        "pair_tight_threshold": ({"clients": pair, "depth": 6000}, {"ORION_MAX_SMS": "148"}),
        "reef": ({"clients": pair, "depth": 12, "reef": True}, {}),
        "two_best_effort": ({"clients": [
            {"profile": be, "num_kernels": 24, "iters": 100000, "train": True, "ops": [1] + [0] * 24},
            {"profile": be2, "num_kernels": 20, "iters": 100000, "train": True, "ops": [0] * 20},
            {"profile": hp, "num_kernels": 10, "iters": 60, "train": False, "ops": [1] + [0] * 10}], "depth": 30000},
            {"ORION_MAX_SMS": "148"}),
        "hp_training": ({"clients": [
            {"profile": bes, "num_kernels": 16, "iters": 100000, "train": True, "ops": [0] * 16},
            {"profile": hpt, "num_kernels": 14, "iters": 45, "train": True, "ops": [1] + [0] * 14}],
            "depth": 20000, "hp_limit": 1000, "update_start": 8}, {"ORION_MAX_SMS": "148"}),
        "single": ({"clients": [{"profile": hp, "num_kernels": 10, "iters": 30, "train": False, "ops": [1] + [0] * 10}]}, {}),
        # the reference's unfinished temporal-sharing policy releases only warm-up requests and malloc records: 12 iterations
        # of each client are all it ever lets through, so the run is kept inside them
        "sequential": ({"clients": [
            {"profile": be, "num_kernels": 24, "iters": 10, "train": True, "ops": [1] + [0] * 24},
            {"profile": hp, "num_kernels": 10, "iters": 10, "train": False, "ops": [1] + [0] * 10}], "sequential": True}, {}),
    }


import pytest


@pytest.mark.skipif(not os.path.exists(REF_REPLAY), reason="the reference scheduler was not compiled on this machine")
@pytest.mark.parametrize("name", ["pair", "pair_tight_threshold", "reef", "two_best_effort", "hp_training", "single", "sequential"])
def test_live_decisions_are_the_reference_schedulers_on_the_same_observations(built, tmp_path, name):
    """ORION_RECORD_OBS: the live scheduler writes every answer it got (queue heads, event queries, clock reads, stop
    acknowledgements) and every decision it took.  The compiled reference scheduler, handed the same answers at the same
    calls, must release the same ops on the same streams with the same events, close the same requests and stop the same
    clients (src/scheduler/scheduler_eval.cpp:238-487 against the live run itself, not against a re-simulation)."""
    cfg, env = _live_scenarios(tmp_path)[name]
    trace = tmp_path / "trace.obs"
    r = _run(cfg, env_extra=dict(env, ORION_RECORD_OBS=str(trace)))
    assert not r["wrong"] and r["stats"]["forced_iter_ends"] == 0
    rc, rep = _check_observations(trace)
    live = (r["stats"]["hp_submits"] + r["stats"]["be_submits"]
            if not cfg.get("reef") and not cfg.get("sequential") and len(cfg["clients"]) > 1 else None)
    assert rep["decisions"] > 100 and not rep["truncated"] and rep["phase"] == 3
    if live is not None:
        assert rep["decisions"] == live
    assert rep["requests_closed"] >= sum(min(c["iters"], 10) for c in cfg["clients"])


@pytest.mark.skipif(not os.path.exists(REF_REPLAY), reason="the reference scheduler was not compiled on this machine")
def test_a_tampered_observation_trace_is_reported(built, tmp_path):
    """The checker must notice a decision the reference would not have taken: move one release of the measured phase to
    the other stream, drop one, and cut a trace short without the `truncated` mark."""
    import re
    cfg, env = _live_scenarios(tmp_path)["pair"]
    trace = tmp_path / "trace.obs"
    _run(cfg, env_extra=dict(env, ORION_RECORD_OBS=str(trace)))
    text = trace.read_text()
    _check_observations(trace)
    body = text.split("\nphase 0 ", 1)
    assert len(body) == 2
    m = list(re.finditer(r" S0:0:0:0:(\d+)", body[1]))[5]
    for bad_tail in (body[1][:m.start()] + " S0:0:1:0:" + m.group(1) + body[1][m.end():],     # other stream
                     body[1][:m.start()] + body[1][m.end():],                                 # release missing
                     body[1][:m.start()].rsplit("\n", 1)[0] + "\nendphase\n"):               # live run "stopped" early
        bad = tmp_path / "bad.obs"
        bad.write_text(body[0] + "\nphase 0 " + bad_tail)
        rc, rep = _check_observations(bad, expect_match=False)
        assert rc == 3 and rep["matched"] is False, rep


@pytest.mark.skipif(not os.path.exists(REF_REPLAY), reason="the reference scheduler was not compiled on this machine")
def test_a_trace_cut_by_the_recording_limit_is_compared_up_to_the_cut(built, tmp_path):
    cfg, env = _live_scenarios(tmp_path)["pair"]
    trace = tmp_path / "trace.obs"
    _run(cfg, env_extra=dict(env, ORION_RECORD_OBS=str(trace), ORION_RECORD_OBS_MAX_LINES="700"))
    assert trace.read_text().rstrip().endswith("truncated")
    rc, rep = _check_observations(trace)
    assert rep["truncated"] and rep["decisions"] > 100


def test_two_threads_of_one_client_take_turns_on_its_ring(built, tmp_path):
    """A helper thread registered to the best-effort client queues ops while the client's own thread does: every op of both is
    granted exactly once and the scheduler's count matches (the ring has one producer at a time)."""
    code = textwrap.dedent('''
        import ctypes, json, sys, threading
        sys.path.insert(0, %(root)r)
        from src.scheduler_frontend import PyScheduler
        cap = ctypes.CDLL(%(root)r + "/orion_b200/lib/liborion_capture.so", mode=ctypes.RTLD_GLOBAL)
        sched = ctypes.CDLL(%(root)r + "/orion_b200/lib/liborion_sched.so")
        cap.stop.restype = ctypes.c_bool
        prof = sys.argv[1]
        N, ITERS, OPS = 1, 30, 40
        barriers = [threading.Barrier(N + 1)]
        got = {"main": 0, "helper": 0, "wrong": 0}
        go = threading.Event(); done_iter = threading.Event()
        def helper():
            cap.orion_capture_register_thread(0)
            while True:
                go.wait(); go.clear()
                if got.get("quit"): return
                for _ in range(OPS // 2):
                    r = cap.orion_capture_op(0)
                    got["helper"] += 1
                    if r != 0: got["wrong"] += 1
                done_iter.set()
        def client():
            barriers[0].wait()
            h = threading.Thread(target=helper); h.start()
            for it in range(ITERS):
                go.set()
                for _ in range(OPS // 2):
                    r = cap.orion_capture_op(0)
                    got["main"] += 1
                    if r != 0: got["wrong"] += 1
                done_iter.wait(); done_iter.clear()
                cap.block(it)
                if it == 0 or it == 9: barriers[0].wait()
            got["quit"] = True; go.set(); h.join()
            barriers[0].wait()
        th = threading.Thread(target=client); th.start()
        ps = PyScheduler(sched, N)
        st = threading.Thread(target=ps.run_scheduler, args=(barriers, [th.native_id], ["m"], [prof], [None], [OPS], [None], [ITERS],
                                                             True, True, False, False, 160000, 1, 1, [True]))
        st.start(); th.join(); st.join()
        print(json.dumps({"got": {k: v for k, v in got.items() if k != "quit"}, "stats": ps.stats()}))
    ''')
    prof = _profile(tmp_path, "p", [(1, 40, 9000)] * 40)
    out = subprocess.run([sys.executable, "-c", code % {"root": ROOT}, prof], capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, ORION_FAKE_GPU="1", ORION_GATE_TIMEOUT_S="5"))
    assert out.returncode == 0, out.stderr[-3000:]
    r = json.loads(out.stdout.strip().splitlines()[-1])
    assert r["got"] == {"main": 30 * 20, "helper": 30 * 20, "wrong": 0}
    assert r["stats"]["hp_submits"] + r["stats"]["be_submits"] >= 30 * 40 and r["stats"]["join_timeouts"] == 0
