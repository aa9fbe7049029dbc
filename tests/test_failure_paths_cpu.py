"""Failure paths that need no GPU: NCCL calls that fail are injected on the host, by pointing the
library's NCCL binding ($VOLTA_B200_NCCL_LIB) at a stand-in whose calls return NCCL error codes.
Each case runs in a child process, because the binding is resolved once per process."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FAKE_SRC = os.path.join(os.path.dirname(__file__), "fakes", "fake_nccl.c")

CHILD = r"""
import ctypes as C, sys
sys.path.insert(0, %r)
from volta_b200 import load_library
lib = load_library()
uid = (C.c_uint8 * 128)()
rc = lib.volta_b200_dp_unique_id(C.byref(uid))
print("uid", rc, lib.volta_b200_last_error(None).decode() if rc else "")
if rc == 0:
    rc = lib.volta_b200_dp_check(bytes(uid), int(sys.argv[1]), int(sys.argv[2]), None, int(sys.argv[3]), None)
    print("check", rc, lib.volta_b200_last_error(None).decode() if rc else "")
""" % ROOT


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("fake") / "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", out, FAKE_SRC], check=True)
    return out


def run_child(fake, world, rank, count, **env):
    e = dict(os.environ, VOLTA_B200_NCCL_LIB=fake, **{k: str(v) for k, v in env.items()})
    r = subprocess.run([sys.executable, "-c", CHILD, str(world), str(rank), str(count)], env=e, capture_output=True,
                       text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    out = {}
    for ln in r.stdout.splitlines():          # "<call> <return code> <message>"
        parts = (ln.split(" ", 2) + ["", ""])[:3]
        out[parts[0]] = (parts[1], parts[2])
    return out


def test_healthy_stand_in_bootstraps_and_reduces(fake_nccl):
    out = run_child(fake_nccl, 2, 1, 0)
    assert out["uid"][0] == "0" and out["check"][0] == "0"


def test_system_error_from_comm_init_is_reported_with_nccls_message(fake_nccl):
    out = run_child(fake_nccl, 2, 0, 0, FAKE_NCCL_FAIL="init")
    assert out["check"][0] == "4"                                  # VB200_ERR_NCCL
    assert "ncclCommInitRank failed: unhandled system error" in out["check"][1]


def test_rank_count_mismatch_is_refused(fake_nccl):
    out = run_child(fake_nccl, 4, 0, 0, FAKE_NCCL_WORLD=2)
    assert out["check"][0] == "4" and "invalid argument" in out["check"][1]


def test_failing_all_reduce_is_reported(fake_nccl):
    out = run_child(fake_nccl, 2, 0, 64, FAKE_NCCL_FAIL="allreduce", FAKE_NCCL_CODE=6)
    # count > 0 needs a buffer: a null one is an argument error, caught before NCCL is called
    assert out["check"][0] == "1"
    e = dict(os.environ, VOLTA_B200_NCCL_LIB=fake_nccl, FAKE_NCCL_FAIL="allreduce", FAKE_NCCL_CODE="6")
    child = CHILD.replace("None, int(sys.argv[3])", "C.cast(C.create_string_buffer(256), C.c_void_p), int(sys.argv[3])")
    r = subprocess.run([sys.executable, "-c", child, "2", "0", "64"], env=e, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("check")][0]
    assert line.split()[1] == "4" and "ncclAllReduce failed: remote process exited" in line


def test_failing_unique_id_is_reported(fake_nccl):
    out = run_child(fake_nccl, 2, 0, 0, FAKE_NCCL_FAIL="uid", FAKE_NCCL_CODE=3)
    assert out["uid"][0] == "4" and "ncclGetUniqueId failed: internal error" in out["uid"][1]


def test_missing_library_file_is_an_error_not_a_crash(tmp_path):
    out = run_child(str(tmp_path / "nowhere.so"), 2, 0, 0)
    assert out["uid"][0] == "4" and "VOLTA_B200_NCCL_LIB" in out["uid"][1]
