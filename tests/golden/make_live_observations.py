"""Generates the observation-trace fixtures tests/golden/live_*.obs: live runs of the scheduler and the capture library on the
host (ORION_FAKE_GPU=1: client threads queue ops through the rings, every event completes at once), recorded with
ORION_RECORD_OBS.  A trace holds every answer the policy got and every decision it took; its profile files are copied beside
it and named relative to it.  live_index.json keeps, per trace, the verdict and the counts of the compiled reference scheduler
fed the trace (oracle/_ref/ref_replay --observations), which `tests/test_policy_parity.py` checks against the product's replay.

    python tests/golden/make_live_observations.py        # needs orion_b200/lib/*.so and oracle/_ref (make -C oracle)

Timing decides how the live polls interleave, so a regenerated trace differs from the committed one; both are valid inputs.
"""
import json
import os
import pathlib
import re
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "tests"))

SCENARIOS = ["pair", "two_best_effort", "hp_training", "reef"]


def main():
    import test_scheduler_host as T
    ref = os.path.join(ROOT, "oracle", "_ref", "ref_replay")
    index = {}
    for name in SCENARIOS:
        tmp = pathlib.Path(tempfile.mkdtemp(prefix="orion_live_"))
        cfg, env = T._live_scenarios(tmp)[name]
        trace = tmp / "trace.obs"
        T._run(cfg, env_extra=dict(env, ORION_RECORD_OBS=str(trace)))
        text = trace.read_text()
        # profiles beside the trace, named relative to it
        paths = set(re.findall(r" profile (\S+) ", text) + re.findall(r"^setup_change \d+ (\S+) ", text, re.M))
        for path in sorted(paths, key=len, reverse=True):   # longest first: one path may be the prefix of another
            dst = "live_%s.%s.profile" % (name, os.path.basename(path))
            shutil.copy(path, os.path.join(HERE, dst))
            text = text.replace(path + " ", dst + " ")
        out = os.path.join(HERE, "live_%s.obs" % name)
        with open(out, "w") as f:
            f.write(text)
        r = subprocess.run([ref, "--observations", out, os.path.join(ROOT, "oracle", "_ref")], capture_output=True, text=True, timeout=300)
        rep = json.loads(r.stdout.strip().splitlines()[-1])
        assert r.returncode == 0 and rep["matched"], rep
        index["live_" + name] = {k: rep[k] for k in ("matched", "decisions", "requests_closed", "polls", "phase")}
        shutil.rmtree(tmp, ignore_errors=True)
        print(name, index["live_" + name], os.path.getsize(out), "bytes")
    with open(os.path.join(HERE, "live_index.json"), "w") as f:
        json.dump(index, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
