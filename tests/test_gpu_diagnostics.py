"""GPU: the diagnostics build of the library (libgradb_diag.so, csrc/gradb_diag.h), run in a child process so that
the product library is what every other test loads.

* a bounded device-side wait is made to run out (the attention kernel polls a few times for a tile whose copy was
  left out): the kernel records its code and returns, the call reports GRADB_ERR_DEVICE_WAIT, nothing faults, and
  the same session decodes correctly afterwards;
* a device-side index check catches an id that was planted in the history behind the host checks;
* outputs hold no NaN or Inf; the single-sequence kernel's stage trace is recorded."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
DIAG = ROOT / "grad.cpp_b200" / "libgradb_diag.so"

SCRIPT = textwrap.dedent('''
    import sys
    import numpy as np
    sys.path.insert(0, sys.argv[1] + "/tests"); sys.path.insert(0, sys.argv[1])
    from conftest import load_package, GOLDEN_MODELS
    g = load_package()
    from grad_cpp_b200 import checkpoint as ck
    from oracle.oracle import Port
    dims, seed, std, perturb = GOLDEN_MODELS["hs64_modern"]
    dm = ck.ModelDims(*dims)
    path = sys.argv[2] + "/m.bin"
    ck.write_synthetic(path, dm, seed, std, perturb)
    port = Port(); om = port.load(path)
    m = g.GPTModel.load(path)
    rng = np.random.default_rng(3)
    prompts = [rng.integers(0, dm.vocab, n).astype(np.int32) for n in (9, 5, 12)]
    greedy = g.Sampling(1, 1.0, 1.2, 0, 1.0)
    want = [port.generate(om, p, 8, greedy=True, penalty=1.2) for p in prompts]

    s = g.BatchSession(m, 3)
    assert all(np.array_equal(a, b) for a, b in zip(s.generate(prompts, greedy, 8), want))
    assert s.diag_count_nonfinite(3) == 0
    print("baseline ok")

    # 1. a wait that runs out: four polls for a tile that never comes
    s.diag_attention_wait(4, 0)
    try:
        s.prefill(prompts)
        print("FAIL: no error")
    except g.binding.GradbError as e:
        print("wait expired:", e.status, e)
        assert e.status == g.binding.ERR_DEVICE_WAIT and "code 301" in str(e)
    s.diag_attention_wait(0, -1)
    out = s.generate(prompts, greedy, 8)          # the same session, afterwards
    assert all(np.array_equal(a, b) for a, b in zip(out, want)), "session did not recover"
    # and inside the on-device loop (graph launches)
    s.diag_attention_wait(4, 0)
    try:
        s.generate(prompts, greedy, 8)
        print("FAIL: no error in the loop")
    except g.binding.GradbError as e:
        assert e.status == g.binding.ERR_DEVICE_WAIT
    s.diag_attention_wait(0, -1)
    assert all(np.array_equal(a, b) for a, b in zip(s.generate(prompts, greedy, 8), want))
    print("recovered ok")

    # 2. an id outside the vocabulary, planted behind the host-side checks, is caught by the device-side check
    s.reset()
    lg = s.prefill(prompts)
    s.diag_poke_history(1, 2, dm.vocab + 7)
    try:
        s.select(greedy, n_seq=3)
        s.step(np.array([1, 1, 1], np.int32))
        print("FAIL: index check silent")
    except g.binding.GradbError as e:
        print("index check:", e.status, e)
        assert e.status == g.binding.ERR_INVALID and "index check" in str(e)
    for bad in ([dm.vocab], [-1]):
        try:
            s.set_history(0, bad)
            print("FAIL: history accepted", bad)
        except IndexError:
            pass
    assert all(np.array_equal(a, b) for a, b in zip(s.generate(prompts, greedy, 8), want))

    # 3. stage trace of the single-sequence kernel
    one = g.BatchSession(m, 1)
    one.prefill([prompts[0]])
    one.step([3])
    tr = one.stage_trace()
    assert len(tr) > 4 * dm.layers and np.all(np.diff(tr.astype(np.int64)) >= 0), len(tr)
    print("trace stamps", len(tr))
    print("ALL OK")
''')


def test_diagnostics_build_wait_expiry_index_checks_and_trace(tmp_path):
    if not DIAG.exists():
        pytest.skip("diagnostics library not built")
    env = dict(os.environ, GRADB_LIB=str(DIAG), GRADB_B1_TRACE="1")
    out = subprocess.run([sys.executable, "-c", SCRIPT, str(ROOT), str(tmp_path)], env=env, capture_output=True,
                         text=True, timeout=600)
    print(out.stdout)
    assert out.returncode == 0 and "ALL OK" in out.stdout and "FAIL" not in out.stdout, out.stdout + out.stderr[-3000:]


def test_product_library_has_no_diagnostic_entry_points(pkg):
    import ctypes
    L = ctypes.CDLL(str(ROOT / "grad.cpp_b200" / "libgradb.so"))
    for name in ("gradb_session_stage_trace", "gradb_diag_attention_wait", "gradb_diag_poke_history"):
        assert not hasattr(L, name), name
