"""Memory-safety check without a memory checker: the kernel test-suite once more against the bounds-check build.

libingot_cuda_check.so is the same library compiled with -DINGOT_BOUNDS_CHECK: every offset a kernel computes into
the KV cache, the split scratch, the query or the output is compared with its buffer's extent before the access,
and a violation raises bit 8 of the status word instead of touching memory. The parity tests assert a clear status
word after every call, so running them against this build shows that no kernel ever computes an out-of-range
offset on any shape the suite covers. A second test proves that the checks are live, by telling the kernels that
the cache is shorter than it is (accesses are flagged and skipped; nothing leaves a buffer, nothing faults).
"""
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from helpers import D, H, HKV
from ingot_b200 import workloads as W

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECK_LIB = os.path.join(ROOT, "inference-agent_b200", "libingot_cuda_check.so")
IN_CHILD = "INGOT_BOUNDS_CHILD"


def _is_check_build():
    import ingot_b200 as ib
    return ib.lib().ingot_build_flags() == b"bounds-check"


def test_kernel_suite_passes_on_the_bounds_check_build():
    if os.environ.get(IN_CHILD):
        pytest.skip("already inside the bounds-check run")
    if not os.path.exists(CHECK_LIB):
        pytest.skip("libingot_cuda_check.so not built")
    env = dict(os.environ, INGOT_CUDA_LIB=CHECK_LIB, **{IN_CHILD: "1"})
    files = ["test_gpu_rope_append.py", "test_gpu_decode.py", "test_gpu_prefill.py", "test_gpu_layers_api.py",
             "test_gpu_bounds_build.py"]
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"] +
                       [os.path.join(ROOT, "tests", f) for f in files], env=env, cwd=ROOT, stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:]
    assert " passed" in r.stdout and "checks are live: ok" in r.stdout, r.stdout[-3000:]


def test_the_checks_are_live(capsys):
    """Only meaningful on the bounds-check build (it runs inside the child process of the test above)."""
    if not _is_check_build():
        pytest.skip("production build: the range checks are compiled out")
    import torch
    import ingot_b200 as ib
    n_keys = 2048
    rng = np.random.default_rng(31)
    wl = W.Decode(rng.standard_normal((1, H, D), dtype=np.float32),
                  [rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)],
                  [rng.standard_normal((n_keys, HKV, D), dtype=np.float32).astype(np.float16)], np.array([n_keys], dtype=np.int32))
    want = helpers.oracle_decode(wl)
    out, kv = helpers.gpu_decode(wl)
    helpers.assert_parity(out.cpu().numpy(), want, "decode on the bounds-check build")
    q = helpers.to_dev(wl.q)
    # Pretend each layer of the cache ends after its very first row: every other row is now "out of range".
    assert ib.lib().ingot_kv_test_shrink_extent(kv.handle, D) == 0
    ib.attn_decode(kv, 0, q, max_seq_len=n_keys)
    torch.cuda.synchronize()
    assert kv.status() & 8, "the range checks did not fire"
    kr = rng.standard_normal((1, HKV, D), dtype=np.float32)
    ib.rope_kv_append(kv, 0, None, helpers.to_dev(kr), helpers.to_dev(kr), helpers.to_dev(helpers.inv_freq()), n_keys - 1)
    torch.cuda.synchronize()
    assert kv.status() & 8, "the append kernel's range check did not fire"
    # Real extent back: clean status, correct result (the skipped append left the cache as it was).
    assert ib.lib().ingot_kv_test_shrink_extent(kv.handle, 0) == 0
    again = ib.attn_decode(kv, 0, q, max_seq_len=n_keys)
    torch.cuda.synchronize()
    assert kv.status() == 0
    helpers.assert_parity(again.cpu().numpy(), want, "decode after the shrunken-extent calls")
    with capsys.disabled():
        print("checks are live: ok")
