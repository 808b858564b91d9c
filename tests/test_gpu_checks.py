"""The checked build (libmechta_kv_checks.so: every cache buffer between canary bytes) under the parity tests.

The library is chosen once per process (MKV_LIB_PATH), so the cases run in child processes: a slice of the parity
suite with the guards verified at every cache close, and the check itself against a guard touched from the host."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKS = os.path.join(ROOT, "mechta_b200", "libmechta_kv_checks.so")


def _env():
    # brings the checked library up to date with the sources (a no-op when it is)
    r = subprocess.run(["make", "-C", os.path.join(ROOT, "mechta_b200", "csrc"), "checks"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return dict(os.environ, MKV_LIB_PATH=CHECKS)


def test_parity_slice_leaves_every_guard_intact():
    """Append, rollback, verify at tile edges and at full size, the fused step, ring caches, shards, ragged batches,
    prefill and snapshot/restore on both formats: KvCache.close() raises if a canary byte changed."""
    sel = ("append or truncate or verify_edges or full_size or fused_step or ring or shards or ragged_batch_of or "
           "prefill_over_cache or snapshot_restore")
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_kv.py"), "-q", "-x", "-m", "gpu", "-k", sel],
                       env=_env(), cwd=ROOT, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


def test_a_touched_guard_is_reported():
    code = (
        "import torch\n"
        "from mechta_b200 import _lib, kv\n"
        "assert _lib.lib().mkv_checks_enabled() == 1\n"
        "torch.cuda.set_device(0)\n"
        "ctx = kv.KvContext(0, torch.cuda.current_stream())\n"
        "c = kv.KvCache(ctx, kv.KvFormat.F32, 2, 4096)\n"
        "assert c.check_guards() == 0\n"
        "_lib.check(_lib.lib().mkv_checks_touch_guard(c._h))\n"
        "assert c.check_guards() == 3, c.check_guards()\n"
        "try:\n"
        "    c.close()\n"
        "except _lib.MkvError as e:\n"
        "    print('reported:', e)\n"
        "else:\n"
        "    raise SystemExit('close() did not report the touched guard')\n"
        "ctx.close()\n")
    r = subprocess.run([sys.executable, "-c", code], env=_env(), cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "reported:" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_the_shipped_library_has_no_guards(tmp_path):
    import torch
    from mechta_b200 import _lib, kv
    if _lib.lib().mkv_checks_enabled():
        pytest.skip("this process runs the checked build")
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    c = kv.KvCache(ctx, kv.KvFormat.F16, 1, 4096)
    assert c.check_guards() == 0
    assert _lib.lib().mkv_checks_touch_guard(c._h) != 0  # MKV_ERR_UNSUPPORTED: there is no guard to touch
    c.close()
    ctx.close()
