"""`make install PREFIX=...` puts the library, the public headers, the sample plugin and the tuning
tables where a C or C++ program expects them (the reference installs libuccl.so and its headers,
src/CMakeLists.txt:79-90); a client built against the installed copy alone must run."""
import os
import shutil
import subprocess

import pytest

from mp_util import ROOT


def test_make_install_and_link_a_client(tmp_path):
    if shutil.which("make") is None or shutil.which("g++") is None:
        pytest.skip("no make / g++")
    prefix = tmp_path / "prefix"
    p = subprocess.run(["make", "-C", ROOT, "install", "PREFIX=" + str(prefix)], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    for rel in ("lib/libuccl.so", "include/uccl.h", "include/uccl_net.h", "include/uccl_device.cuh", "include/uccl_noalloc.h",
                "lib/libuccl-net-sample.so"):
        assert (prefix / rel).exists(), rel
    assert any(f.endswith(".json") for f in os.listdir(prefix / "share" / "uccl" / "tuning"))
    exe = tmp_path / "client"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-O1", "-I" + str(prefix / "include"), "-I" + cuda + "/include",
           os.path.join(ROOT, "tests", "native", "c_api_client.cc"), "-o", str(exe), "-L" + str(prefix / "lib"), "-luccl",
           "-Wl,-rpath," + str(prefix / "lib"), "-L" + cuda + "/lib64", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    env = dict(os.environ, UCCL_BACKEND="cpu", UCCL_BOOTSTRAP_IFNAME="lo")
    p = subprocess.run([str(exe), "initall", "2"], env=env, capture_output=True, timeout=120)
    assert p.returncode == 0 and p.stdout.count(b"ok") == 2, (p.stdout[-500:], p.stderr[-1500:])
