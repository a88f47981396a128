"""Native (C++) unit tests of the host runtime, one pytest case per self test.  The tests live in
tests/native/selftest.cc and are built into tests/native/libuccl_selftest.so (test-only code, not
part of libuccl.so); this file drives them through ctypes."""
import ctypes
import os

import pytest

import unified_ccl_b200 as u

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_LIB = ctypes.CDLL(os.path.join(ROOT, "tests", "native", "libuccl_selftest.so"))
_LIB.ucclSelfTestName.restype = ctypes.c_char_p
_LIB.ucclSelfTestName.argtypes = [ctypes.c_int]
_LIB.ucclSelfTestRun.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_size_t]
NAMES = [_LIB.ucclSelfTestName(i).decode() for i in range(_LIB.ucclSelfTestCount())]


def _run(name):
    report = ctypes.create_string_buffer(8192)
    rc = _LIB.ucclSelfTestRun(name.encode(), report, len(report))
    return rc, report.value.decode(errors="replace")


def test_selftests_exist():
    assert {"proxy_in_order", "proxy_immediate_completion", "proxy_errors", "ll128_codec", "ring_schedule", "tuner",
            "plugin_loader", "socket_loopback", "topology", "conversions", "config", "api_rules"} <= set(NAMES)


@pytest.mark.parametrize("name", NAMES)
def test_selftest(name, monkeypatch):
    plugin = os.path.join(ROOT, "plugins", "sample", "libuccl-net-sample.so")
    if os.path.exists(plugin):
        monkeypatch.setenv("UCCL_SELFTEST_PLUGIN", plugin)
    rc, report = _run(name)
    assert rc == 0, report


def test_unknown_selftest():
    rc, report = _run("does_not_exist")
    assert rc == 2 and "no such" in report


def test_version_and_errors():
    assert u._C.get_version() == 100
    assert u._C.get_error_string(0) == "no error"
    assert "invalid argument" in u._C.get_error_string(3)
