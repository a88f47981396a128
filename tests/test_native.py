"""Native (C++) unit tests of the host runtime, one pytest case per self test."""
import os

import pytest

import unified_ccl_b200 as u

NAMES = u._C.selftest_names()
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_selftests_exist():
    assert {"proxy_in_order", "proxy_immediate_completion", "proxy_errors", "ll128_codec", "ring_schedule", "tuner",
            "plugin_loader", "socket_loopback", "topology", "conversions", "config", "api_rules"} <= set(NAMES)


@pytest.mark.parametrize("name", NAMES)
def test_selftest(name, monkeypatch):
    plugin = os.path.join(ROOT, "plugins", "sample", "libuccl-net-sample.so")
    if os.path.exists(plugin):
        monkeypatch.setenv("UCCL_SELFTEST_PLUGIN", plugin)
    rc, report = u._C.selftest_run(name)
    assert rc == 0, report


def test_unknown_selftest():
    rc, report = u._C.selftest_run("does_not_exist")
    assert rc == 2 and "no such" in report


def test_version_and_errors():
    assert u._C.get_version() == 100
    assert u._C.get_error_string(0) == "no error"
    assert "invalid argument" in u._C.get_error_string(3)
