"""Failure paths of the NCCL layer, made on the host (no GPU, no second rank): a peer that never joins must end
tesserae_nccl_comm_init_deadline with an error inside its time limit and an aborted communicator; a peer that
joins late must not; tesserae_nccl_comm_abort must reach ncclCommAbort.  The failing calls come from a stand-in
libnccl (tests/helpers/fake_nccl.c) that the test compiles with gcc and the library loads by path."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

HERE = Path(__file__).resolve().parent


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory):
    out = tmp_path_factory.mktemp("fake_nccl") / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-Wall", "-o", str(out), str(HERE / "helpers" / "fake_nccl.c")], check=True)
    return out


def _run(fake, scenario):
    env = {k: v for k, v in os.environ.items() if k not in ("TESSERAE_NCCL_LIB", "FAKE_NCCL_READY_AFTER_MS")}
    r = subprocess.run([sys.executable, str(HERE / "helpers" / "nccl_deadline_worker.py"), str(fake), scenario],
                       capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_rank_that_never_joins_times_out_and_is_aborted(fake_nccl):
    res = _run(fake_nccl, "never_joins")
    assert res["rc"] != 0
    assert "did not join" in res["message"] and "300 ms" in res["message"], res
    assert 0.25 <= res["seconds"] <= 5.0, res          # gave up at the deadline, not at once and not never
    assert res["comm"] in (None, 0)                    # no handle is handed out
    assert res["aborts"] == 1                          # the half-made communicator was given up


def test_rank_that_joins_late_is_waited_for(fake_nccl):
    res = _run(fake_nccl, "joins_late")
    assert res["rc"] == 0 and res["comm_set"] and res["aborts"] == 0, res
    assert 0.05 <= res["seconds"] <= 4.0, res
    assert res["reduce_scatter_rc"] == 0, res          # an "in progress" answer is settled inside the wrapper
    assert res["abort_rc"] == 0 and res["aborts_after"] == 1 and res["abort_null_rc"] == 0, res


def test_missing_library_message_names_the_path_tried():
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from tesserae_b200 import _native as N\n"
            "rc = N.lib().tesserae_nccl_load(b'/nonexistent/libnccl_nowhere.so')\n"
            "print(rc, N.last_error())\n") % str(HERE.parent)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split()[0] != "0" and "/nonexistent/libnccl_nowhere.so" in r.stdout
