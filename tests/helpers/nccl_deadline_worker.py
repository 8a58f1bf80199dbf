"""Child process of tests/test_nccl_failure_cpu.py: drives the communicator failure paths of the C ABI against
the stand-in NCCL (tests/helpers/fake_nccl.c).  A process of its own because the library binds one NCCL for
its lifetime.  Prints one RESULT line of JSON."""
import ctypes as C
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from tesserae_b200 import _native as N  # noqa: E402

fake_path, scenario = sys.argv[1], sys.argv[2]
lib = N.lib()
N.check(lib.tesserae_nccl_load(fake_path.encode()), "nccl_load")
fake = C.CDLL(fake_path)
uid = C.create_string_buffer(128)
N.check(lib.tesserae_nccl_unique_id(uid), "unique_id")
comm = C.c_void_p(1)
out = {"scenario": scenario}
if scenario == "never_joins":
    os.environ.pop("FAKE_NCCL_READY_AFTER_MS", None)
    t0 = time.perf_counter()
    rc = lib.tesserae_nccl_comm_init_deadline(C.byref(comm), 2, 0, uid, 300)
    out.update(rc=rc, seconds=time.perf_counter() - t0, message=N.last_error(), comm=comm.value,
               aborts=fake.fake_nccl_counter(0))
elif scenario == "joins_late":
    os.environ["FAKE_NCCL_READY_AFTER_MS"] = "60"
    t0 = time.perf_counter()
    rc = lib.tesserae_nccl_comm_init_deadline(C.byref(comm), 2, 0, uid, 5000)
    out.update(rc=rc, seconds=time.perf_counter() - t0, comm_set=bool(comm.value), aborts=fake.fake_nccl_counter(0))
    x = C.create_string_buffer(64)
    out["reduce_scatter_rc"] = lib.tesserae_nccl_reduce_scatter_f32(comm, x, x, 4, None)   # "in progress", then settles
    out["abort_rc"] = lib.tesserae_nccl_comm_abort(comm)
    out["aborts_after"] = fake.fake_nccl_counter(0)
    out["abort_null_rc"] = lib.tesserae_nccl_comm_abort(None)
print("RESULT " + json.dumps(out), flush=True)
