"""Profile-file loader: same parsing rules as the reference's populate_kernel_info
(reference src/scheduler/scheduler_eval.cpp:498-526)."""
import ctypes

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
