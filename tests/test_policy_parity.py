"""Decision parity of the scheduling policy.

Golden logs in tests/golden/ were produced by the reference's own scheduler sources
(compiled unmodified, driven by oracle/ref_driver.cpp); tests/golden/make_golden.py
regenerates them.  Every case must be reproduced bit for bit by
  * the product's policy core (orion_replay), and
  * the Python restatement in oracle/policy_oracle.py.
"""
import gzip
import hashlib
import json
import os
import subprocess

import pytest

from oracle import policy_oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")
with open(os.path.join(GOLD, "policy_index.json")) as f:
    INDEX = json.load(f)
CASES = sorted(INDEX)


def _first_diff(a, b):
    la, lb = a.splitlines(), b.splitlines()
    for i, (x, y) in enumerate(zip(la, lb)):
        if x != y:
            return "line %d: got %r want %r" % (i + 1, x, y)
    return "length %d vs %d" % (len(la), len(lb))


def _decisions(text):
    return "".join(l for l in text.splitlines(True) if not l.startswith("Q"))


@pytest.mark.parametrize("case", CASES)
def test_product_policy_matches_reference_log(case, built, tmp_path):
    log = tmp_path / "log.txt"
    out = subprocess.run([built["orion_replay"], os.path.join(GOLD, case + ".script"), "--log", str(log)], capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    info = json.loads(out.stdout.strip().splitlines()[-1])
    data = log.read_bytes()
    want_dec = gzip.open(os.path.join(GOLD, case + ".decisions.gz"), "rb").read().decode()
    assert _decisions(data.decode()) == want_dec, _first_diff(_decisions(data.decode()), want_dec)
    assert hashlib.sha256(data).hexdigest() == INDEX[case]["sha256"]      # includes every event query and its answer
    assert info["decisions"] == INDEX[case]["decisions"]
    assert info["log_fnv1a"] == INDEX[case]["log_fnv1a"]


@pytest.mark.parametrize("case", CASES)
def test_python_oracle_matches_reference_log(case):
    text = policy_oracle.run_script(os.path.join(GOLD, case + ".script"))
    want_dec = gzip.open(os.path.join(GOLD, case + ".decisions.gz"), "rb").read().decode()
    assert _decisions(text) == want_dec, _first_diff(_decisions(text), want_dec)
    assert hashlib.sha256(text.encode()).hexdigest() == INDEX[case]["sha256"]


def test_golden_cases_cover_all_policies():
    algos = set()
    for case in CASES:
        with open(os.path.join(GOLD, case + ".script")) as f:
            for line in f:
                if line.startswith("algo"):
                    algos.add(line.split()[1])
    assert algos == {"orion", "reef", "sequential"}
    assert any("hp_train" in c for c in CASES) and any("single" in c for c in CASES)


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ref_replay")),
                    reason="reference scheduler not compiled here (make -C oracle ref)")
@pytest.mark.parametrize("case", ["pair_open", "hp_train", "reef_pair", "three_clients"])
def test_reference_scheduler_still_produces_the_committed_logs(case, tmp_path):
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    log = tmp_path / "ref.txt"
    out = subprocess.run([os.path.join(ref_dir, "ref_replay"), os.path.join(GOLD, case + ".script"), ref_dir, str(log)],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert hashlib.sha256(log.read_bytes()).hexdigest() == INDEX[case]["sha256"]


def test_unsupported_record_type_aborts_the_policy(built, tmp_path):
    """The reference aborts on record types its replay switch does not know (utils_sched.cpp:514-516)."""
    prof = tmp_path / "p.profile"
    prof.write_text("Name,Profile,Memory_footprint,SM_usage,Duration\nk,1,0,10,1000\n")
    script = tmp_path / "bad.script"
    script.write_text("orion_script 1\nalgo orion\ndepth 1000 hp_limit 1 update_start 1 max_sms 80\nnclients 1\n"
                      "client 0\n train 0 num_iters 12 think 0\n profile p.profile 1\n ops 1 5 0 1\n gaps closed\nend\n"
                      "phases 1 0 0\n")
    out = subprocess.run([built["orion_replay"], str(script)], capture_output=True, text=True, timeout=60)
    assert out.returncode == 2


# ---------------------------------------------------------------------------------------------- traces of live runs
with open(os.path.join(GOLD, "live_index.json")) as _f:
    LIVE = json.load(_f)


@pytest.mark.parametrize("case", sorted(LIVE))
def test_policy_core_reproduces_the_decisions_of_recorded_live_runs(case, built):
    """tests/golden/live_*.obs: observation traces of live runs (queue heads, event answers, clock reads, stop acknowledgements in;
    releases, closed requests, stop requests out).  The compiled reference scheduler, fed each trace, took exactly the recorded
    decisions (counts in live_index.json, written by tests/golden/make_live_observations.py); the product's policy core fed the
    same trace must take them too, to the last token."""
    out = subprocess.run([built["orion_replay"], "--observations", os.path.join(GOLD, case + ".obs")], capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    rep = json.loads(out.stdout.strip().splitlines()[-1])
    want = LIVE[case]
    assert rep["matched"] is True and not rep["truncated"]
    assert (rep["decisions"], rep["requests_closed"], rep["polls"], rep["phase"]) == (want["decisions"], want["requests_closed"],
                                                                                      want["polls"], want["phase"])


@pytest.mark.skipif(not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ref_replay")),
                    reason="reference scheduler not compiled here (make -C oracle ref)")
@pytest.mark.parametrize("case", sorted(LIVE))
def test_reference_scheduler_still_agrees_with_the_recorded_live_runs(case):
    ref_dir = os.path.join(ROOT, "oracle", "_ref")
    out = subprocess.run([os.path.join(ref_dir, "ref_replay"), "--observations", os.path.join(GOLD, case + ".obs"), ref_dir],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    rep = json.loads(out.stdout.strip().splitlines()[-1])
    assert rep["matched"] is True and {k: rep[k] for k in LIVE[case]} == LIVE[case]


def test_policy_core_notices_a_decision_that_is_not_its_own(built, tmp_path):
    """A release moved to the other stream in a recorded trace is a mismatch for the product's replay as well (exit 3)."""
    import re
    import shutil
    for f in os.listdir(GOLD):
        if f.startswith("live_pair."):
            shutil.copy(os.path.join(GOLD, f), tmp_path / f)
    text = (tmp_path / "live_pair.obs").read_text()
    head, tail = text.split("\nphase 0 ", 1)
    m = list(re.finditer(r" S0:0:0:0:(\d+)", tail))[3]
    (tmp_path / "live_pair.obs").write_text(head + "\nphase 0 " + tail[:m.start()] + " S0:0:1:0:" + m.group(1) + tail[m.end():])
    out = subprocess.run([built["orion_replay"], "--observations", str(tmp_path / "live_pair.obs")], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 3 and json.loads(out.stdout.strip().splitlines()[-1])["matched"] is False
