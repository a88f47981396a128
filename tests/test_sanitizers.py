"""Host runtime under AddressSanitizer + UBSan and under ThreadSanitizer: the native self tests
(proxy thread, FIFO, bootstrap sockets, plugin loader, schedules, tuner) linked into a plain
executable by `make asan` / `make tsan`.  Stands in for device-side race detection, which is not
available here."""
import shutil
import subprocess

import pytest

from mp_util import ROOT


@pytest.mark.parametrize("target", ["asan", "tsan"])
def test_native_selftests_under_sanitizer(target):
    if shutil.which("make") is None:
        pytest.skip("no make")
    p = subprocess.run(["make", "-C", ROOT, "-j", "8", target], capture_output=True, text=True, timeout=1500)
    out = p.stdout + p.stderr
    if "cannot find -lasan" in out or "cannot find -ltsan" in out or "cannot find -lubsan" in out:
        pytest.skip("sanitizer runtime not installed")
    assert p.returncode == 0, out[-3000:]
    assert "FAILED" not in out and "ERROR: AddressSanitizer" not in out and "WARNING: ThreadSanitizer" not in out
    assert "runtime error:" not in out  # UBSan
    assert out.count(" ok") >= 13
