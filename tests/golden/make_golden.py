"""Generate the policy golden fixtures.

Writes, for a fixed list of seeded cases, a synthetic per-kernel profile file, an
arrival script, and the decision log that the *reference scheduler itself*
(oracle/_ref/ref_replay, built by `make -C oracle ref` from the reference
checkout) produces for it.  Only this script needs the reference; the tests read
the committed files.

    python tests/golden/make_golden.py            # regenerate everything
    python tests/golden/make_golden.py --check    # verify the committed logs instead
    python tests/golden/make_golden.py --import-recorded <recorded.script> [--name c2_recorded] [--iters 60]
        # adopt an arrival script the live scheduler recorded on a GPU (ORION_RECORD_SCRIPT) as a further case: its
        # profile files (real per-kernel profiles of that run) are copied next to it, the run is cut to --iters
        # requests per client, and the reference scheduler's log for it is committed like the others

Profiles are synthetic rows in the model_kernels format (same five columns, value
ranges modelled on profiled convolution / batch-norm / elementwise kernels: SM
need 1..4000, duration 2..900 us); they are not copies of any profiled model.
"""
import argparse
import gzip
import hashlib
import json
import os
import random
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")

KERNEL, MEMCPY, MALLOC, FREE, MEMSET = 0, 1, 2, 3, 4
COMPUTE_TYPES = [0, 0, 0, 0, 6, 7, 9, 12, 13, 14, 15, 16]
NAMES = ["Conv", "BatchNorm", "void at::native::vectorized_elementwise_kernel",
         "void at::native::reduce_kernel", "volta_sgemm_128x64_tn", "void at::native::elementwise_kernel"]


def make_profile(rng, n, big_frac, max_sm, dur_lo=2000, dur_hi=900000):
    rows = []
    for _ in range(n):
        name = rng.choice(NAMES)
        prof = rng.choice([1, 1, 0, 0, -1])
        if rng.random() < big_frac:
            sm = rng.randint(max_sm + 1, 4000)
        else:
            sm = rng.randint(1, max_sm)
        dur = rng.choice([rng.randint(dur_lo, dur_hi), rng.randint(dur_lo, dur_lo * 10)])
        if rng.random() < 0.1:
            dur = dur + 0.5
        rows.append((name, prof, 0, sm, dur))
    return rows


def write_profile(path, rows):
    with open(path, "w") as f:
        f.write("Name,Profile,Memory_footprint,SM_usage,Duration\n")
        for r in rows:
            f.write("%s,%d,%d,%d,%s\n" % r)


def make_ops(rng, rows, memop_frac, gap_hi, tick_ns):
    """One op per profile row plus sprinkled memory ops (which have no row)."""
    ops = []
    for r in rows:
        while rng.random() < memop_frac:
            ops.append((rng.choice([MEMCPY, MALLOC, FREE, MEMSET]), rng.randint(0, gap_hi), rng.randint(0, 30)))
        dur = max(1, int(float(r[4]) / tick_ns * rng.uniform(0.5, 1.5)))
        ops.append((rng.choice(COMPUTE_TYPES), rng.randint(0, gap_hi), dur))
    if rng.random() < 0.5:
        ops.append((MEMCPY, rng.randint(0, gap_hi), rng.randint(0, 30)))
    return ops


def fmt_ops(key, ops):
    return "  %s %d %s\n" % (key, len(ops), " ".join("%d %d %d" % o for o in ops))


def build_case(name, seed, out_dir, algo="orion", nclients=2, hp_train=False, be_rows=60, hp_rows=25,
               be_iters=40, hp_iters=40, depth=160000, max_sms=80, open_loop=False, big_frac=0.3,
               memop_frac=0.05, gap_hi=6, two_profiles=True, update_start=1, hp_limit=1, think=20,
               warm=(1, 10)):
    rng = random.Random(seed)
    tick_ns = 1000.0
    lines = ["orion_script 1\n", "algo %s\n" % algo,
             "depth %d hp_limit %d update_start %d max_sms %d\n" % (depth, hp_limit, update_start, max_sms),
             "nclients %d\n" % nclients]
    for c in range(nclients):
        is_hp = c == nclients - 1
        train = hp_train if is_hp else True
        nrows = hp_rows if is_hp else be_rows
        rows = make_profile(rng, nrows, big_frac if not is_hp else 0.2, max_sms)
        p1 = "%s.c%d.profile" % (name, c)
        write_profile(os.path.join(out_dir, p1), rows)
        lines.append("client %d\n" % c)
        iters = hp_iters if is_hp else be_iters
        lines.append("  train %d num_iters %d think %d\n" % (1 if train else 0, iters, think))
        if train and two_profiles and nclients > 1:
            rows0 = rows[: max(3, (2 * nrows) // 3)]
            p0 = "%s.c%d.first.profile" % (name, c)
            write_profile(os.path.join(out_dir, p0), rows0)
            lines.append("  profile %s %d\n" % (p0, len(rows0)))
            lines.append("  profile2 %s %d\n" % (p1, len(rows)))
            lines.append(fmt_ops("ops0", make_ops(rng, rows0, memop_frac, gap_hi, tick_ns)))
        else:
            lines.append("  profile %s %d\n" % (p1, len(rows)))
        lines.append(fmt_ops("ops", make_ops(rng, rows, memop_frac, gap_hi, tick_ns)))
        if open_loop and is_hp:
            mean = sum(float(r[4]) for r in rows) / tick_ns * 1.5
            gaps = [int(rng.expovariate(1.0 / mean)) for _ in range(iters)]
            lines.append("  gaps open %s\n" % " ".join(map(str, gaps)))
        else:
            lines.append("  gaps closed\n")
        lines.append("end\n")
    lines.append("phases 3 1 %d 1 %d 0 0\n" % warm)
    with open(os.path.join(out_dir, name + ".script"), "w") as f:
        f.writelines(lines)


CASES = [
    dict(name="pair_closed", seed=1),
    dict(name="pair_open", seed=2, open_loop=True, hp_iters=60, be_iters=200),
    dict(name="pair_small_depth", seed=3, depth=3000, open_loop=True, hp_iters=50, be_iters=100),
    dict(name="pair_sm148", seed=4, max_sms=148, depth=100000, open_loop=True, hp_iters=50, be_iters=100),
    dict(name="pair_nomem", seed=5, memop_frac=0.0, big_frac=0.0, hp_iters=30, be_iters=30),
    dict(name="three_clients", seed=6, nclients=3, open_loop=True, hp_iters=40, be_iters=60, depth=20000),
    dict(name="four_clients", seed=7, nclients=4, hp_iters=30, be_iters=30, depth=50000, be_rows=30),
    dict(name="single_client", seed=8, nclients=1, hp_iters=25, two_profiles=False),
    dict(name="hp_train", seed=9, hp_train=True, hp_rows=40, update_start=25, hp_limit=12, hp_iters=45,
         be_iters=80, depth=40000, big_frac=0.1),
    dict(name="hp_train_tight", seed=10, hp_train=True, hp_rows=30, update_start=20, hp_limit=2, hp_iters=35,
         be_iters=60, depth=10000, big_frac=0.05, two_profiles=False),
    dict(name="reef_pair", seed=11, algo="reef", depth=12, open_loop=True, hp_iters=40, be_iters=80),
    dict(name="reef_three", seed=12, algo="reef", depth=3, nclients=3, hp_iters=30, be_iters=40),
    dict(name="reef_single", seed=13, algo="reef", nclients=1, hp_iters=15, two_profiles=False),
    dict(name="seq_warm_only", seed=14, algo="sequential", hp_iters=10, be_iters=10, warm=(1, 10)),
    dict(name="be_starved", seed=15, big_frac=0.9, hp_iters=40, be_iters=40, think=0, gap_hi=0),
    dict(name="long_gaps", seed=16, gap_hi=200, think=500, hp_iters=30, be_iters=30, depth=500000),
]


def run_ref(script, log):
    exe = os.path.join(REF_DIR, "ref_replay")
    out = subprocess.run([exe, script, REF_DIR, log], capture_output=True, text=True, timeout=600)
    if out.returncode != 0:
        raise RuntimeError("ref_replay failed on %s: %s" % (script, out.stderr[-2000:]))
    return json.loads(out.stdout.strip().splitlines()[-1])


# Cases recorded from live runs on a GPU (see --import-recorded); their scripts and profiles are committed as they are.
RECORDED = ["c2_recorded"]


def import_recorded(src, name, iters):
    """Copy a recorded arrival script into this directory as case `name`: profile paths become local copies, every client
    runs `iters` requests (the open-loop gap list is cut to match)."""
    out, client = [], -1
    for line in open(src):
        tok = line.split()
        if tok[:1] == ["client"]:
            client = int(tok[1])
        if tok[:1] == ["profile"]:
            local = "%s.c%d.profile" % (name, client)
            with open(tok[1]) as f, open(os.path.join(HERE, local), "w") as g:
                g.write(f.read())
            line = "  profile %s %s\n" % (local, tok[2])
        elif tok[:1] == ["train"]:
            tok[tok.index("num_iters") + 1] = str(iters)
            line = "  " + " ".join(tok) + "\n"
        elif tok[:2] == ["gaps", "open"]:
            gaps = tok[2:2 + iters]
            gaps += ["0"] * (iters - len(gaps))
            line = "  gaps open " + " ".join(gaps) + "\n"
        out.append(line)
    with open(os.path.join(HERE, name + ".script"), "w") as f:
        f.writelines(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--import-recorded", default="")
    ap.add_argument("--name", default="c2_recorded")
    ap.add_argument("--iters", type=int, default=60)
    args = ap.parse_args()
    if not os.path.exists(os.path.join(REF_DIR, "ref_replay")):
        sys.exit("build the reference first: make -C oracle ref")
    if args.import_recorded:
        import_recorded(args.import_recorded, args.name, args.iters)
    index = {}
    tmp = os.path.join(HERE, "_tmp.log")
    recorded = [dict(name=n, recorded=True) for n in RECORDED if os.path.exists(os.path.join(HERE, n + ".script"))]
    for case in CASES + recorded:
        kw = dict(case)
        name = kw.pop("name")
        if not args.check and not kw.pop("recorded", False):
            build_case(name, out_dir=HERE, **kw)
        script = os.path.join(HERE, name + ".script")
        info = run_ref(script, tmp)
        data = open(tmp, "rb").read()
        # The full log is pinned by its sha256; the committed file keeps every line
        # except the event queries (which dominate the volume) for readable diffs.
        decisions = b"".join(l for l in data.splitlines(True) if not l.startswith(b"Q"))
        gz = os.path.join(HERE, name + ".decisions.gz")
        if args.check:
            want = gzip.open(gz, "rb").read()
            old = json.load(open(os.path.join(HERE, "policy_index.json")))[name]["sha256"]
            ok = want == decisions and old == hashlib.sha256(data).hexdigest()
            print("%-18s %s" % (name, "ok" if ok else "MISMATCH"))
            if not ok:
                sys.exit(1)
        else:
            with open(gz, "wb") as raw, gzip.GzipFile(fileobj=raw, mode="wb", mtime=0) as f:
                f.write(decisions)
        index[name] = dict(decisions=info["decisions"], queries=info["queries"], iters_done=info["iters_done"],
                           log_fnv1a=info["log_fnv1a"], sha256=hashlib.sha256(data).hexdigest())
        print(name, index[name])
    os.remove(tmp)
    if not args.check:
        with open(os.path.join(HERE, "policy_index.json"), "w") as f:
            json.dump(index, f, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
