"""Profile-file loader: same parsing rules as the reference's populate_kernel_info
(reference src/scheduler/scheduler_eval.cpp:498-526)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import policy_oracle


def _load(lib, path, cap=4096):
    prof = (ctypes.c_int * cap)()
    sm = (ctypes.c_int * cap)()
    dur = (ctypes.c_float * cap)()
    n = lib.orion_load_profile(str(path).encode(), prof, sm, dur, cap)
    return n, list(prof[:max(n, 0)]), list(sm[:max(n, 0)]), list(dur[:max(n, 0)])


@pytest.fixture(scope="module")
def sched(built):
    lib = ctypes.CDLL(built["liborion_sched.so"])
    lib.orion_load_profile.restype = ctypes.c_int
    return lib


def test_header_is_skipped_and_fields_parse_like_stoi_stof(sched, tmp_path):
    p = tmp_path / "a"
    p.write_text("Name,Profile,Memory_footprint,SM_usage,Duration\n"
                 "Conv,1,0,98,100480\n"
                 "void at::native::vectorized_elementwise_kernel,0,0,392,32512.5\n"
                 "x,-1,7,12abc,16777217\n")
    n, prof, sm, dur = _load(sched, p)
    assert n == 3 and prof == [1, 0, -1] and sm == [98, 392, 12]
    assert dur[0] == 100480.0 and dur[1] == 32512.5
    assert dur[2] == float(np.float32(16777217))          # durations are floats: > 2^24 loses integer precision
    rows = policy_oracle.load_profile(str(p))
    assert [r[1] for r in rows] == prof and [r[3] for r in rows] == sm and [float(r[4]) for r in rows] == dur


def test_empty_profile_and_missing_file(sched, tmp_path):
    p = tmp_path / "empty"
    p.write_text("Name,Profile,Memory_footprint,SM_usage,Duration\n")
    assert _load(sched, p)[0] == 0
    assert _load(sched, tmp_path / "nope")[0] == -1


def test_short_row_is_reported_not_read_out_of_bounds(sched, tmp_path):
    p = tmp_path / "bad"
    p.write_text("Name,Profile,Memory_footprint,SM_usage,Duration\nConv,1,0\n")
    assert _load(sched, p)[0] == -1


def test_golden_profiles_load_identically_in_oracle_and_product(sched, golden_dir):
    import glob
    import os
    files = sorted(glob.glob(os.path.join(golden_dir, "*.profile")))
    assert files
    for path in files[:8]:
        n, prof, sm, dur = _load(sched, path)
        rows = policy_oracle.load_profile(path)
        assert n == len(rows)
        assert prof == [r[1] for r in rows] and sm == [r[3] for r in rows]
        assert dur == [float(r[4]) for r in rows]


# ---------------------------------------------------------------------------------------------- ncu exports -> profile file
import pytest

PIPE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ncu_pipeline")


@pytest.mark.parametrize("model_type", ["vision", "bert", "transformer"])
def test_profile_from_ncu_exports_equals_the_reference_scripts(model_type, tmp_path):
    """tests/golden/ncu_pipeline/: two synthetic ncu exports and what the reference's own four post-processing scripts made of
    them (tests/golden/make_profile_pipeline_golden.py).  orion_b200/profile_from_ncu.py with the reference's device defaults
    must write the same profile file, byte for byte: SM need, class (including unknown), grouping into Conv / BatchNorm rows,
    dropped rows, names, durations."""
    from orion_b200 import profile_from_ncu as P
    out = tmp_path / "profile"
    n = P.convert(PIPE, str(out), model_type=model_type, device="v100")
    want = open(os.path.join(PIPE, "model_kernels_" + model_type)).read()
    assert out.read_text() == want
    assert n == want.count("\n") - 1


def test_profile_from_ncu_intermediate_columns_match_the_reference():
    """SM need and class of every kernel against the reference's intermediate file (before rows are grouped and dropped)."""
    import csv
    from orion_b200 import profile_from_ncu as P
    kernels = P.process_ncu(os.path.join(PIPE, "output_ncu.csv"))
    raw = list(csv.DictReader(open(os.path.join(PIPE, "raw_ncu.csv"), newline="")))
    ref = list(csv.DictReader(open(os.path.join(PIPE, "output_ncu_sms_roofline.csv"), newline="")))
    assert len(kernels) == len(raw) == len(ref) == 16
    lim = P.DEVICES["v100"]
    for k, r, want in zip(kernels, raw, ref):
        assert k["name"] == want["Kernel_Name"]
        assert P.sm_needed(k, lim["max_threads_sm"], lim["max_shmem_sm"]) == int(want["SM_needed"])
        assert P.roofline_class(k, r, lim["ai_threshold"]) == int(want["Roofline_prof"])
    classes = {int(w["Roofline_prof"]) for w in ref}
    assert classes == {-1, 0, 1}                                    # the fixtures reach all three outcomes of the class rule


def test_profile_from_ncu_b200_limits_and_scheduler_loader(tmp_path):
    """With a B200's limits (228 KB of shared memory per SM) shared-memory-bound kernels need fewer SMs than on the V100 table,
    and the file loads through the scheduler's own profile parser."""
    from orion_b200 import profile_from_ncu as P
    out = tmp_path / "b200"
    n = P.convert(PIPE, str(out), model_type="vision", device="b200")
    rows = [l.split(",") for l in out.read_text().strip().splitlines()[1:]]
    ref = [l.split(",") for l in open(os.path.join(PIPE, "model_kernels_vision")).read().strip().splitlines()[1:]]
    assert n == len(rows) == len(ref)
    assert all(int(a[3]) <= int(b[3]) for a, b in zip(rows, ref)) and any(int(a[3]) < int(b[3]) for a, b in zip(rows, ref))


# ---------------------------------------------------------------------------------------------- shipped client configurations
def test_example_configurations_are_consistent_with_the_committed_profiles():
    """benchmarking/configs/*.json: the client lists of configurations 2-5 and a three-client example, in the reference's schema
    (benchmarking/multi_client_example.json).  Every profile they name exists beside them, `num_kernels` is its row count (the
    scheduler refuses anything larger), the high-priority client is the last entry, and training clients carry the profile of
    their first iteration and that of the steady state, and so do the inference clients (their first request re-lays filters)."""
    import glob
    import json
    cfg_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarking", "configs")
    files = sorted(glob.glob(os.path.join(cfg_dir, "*.json")))
    assert len(files) >= 5
    for path in files:
        cfg = json.load(open(path))
        assert len(cfg) >= 2
        for i, c in enumerate(cfg):
            assert set(c) >= {"arch", "kernel_file", "num_kernels", "num_iters", "args"}
            assert set(c["args"]) >= {"batchsize", "rps", "uniform", "dummy_data", "train"}    # vision clients add model_name
            # every client's first request / iteration launches one-time work (lazy initialisation, filter re-layout), so each
            # entry names the profile of the first iteration and the steady-state one that replaces it (setup_change)
            pairs = [(c["kernel_file"], c["num_kernels"]), (c["additional_kernel_file"], c["additional_num_kernels"])]
            assert c["num_kernels"] >= c["additional_num_kernels"]
            for rel, n in pairs:
                prof = os.path.normpath(os.path.join(cfg_dir, rel))
                with open(prof) as f:
                    lines = f.read().strip().splitlines()
                assert lines[0] == "Name,Profile,Memory_footprint,SM_usage,Duration"
                assert len(lines) - 1 == n, (os.path.basename(path), rel)
            assert c["args"]["train"] == (i < len(cfg) - 1)     # best-effort training clients first, the inference client last
