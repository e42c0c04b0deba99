"""The C++ policy core under AddressSanitizer + UBSan and the rank control plane under
ThreadSanitizer: the core's own CPU tests are re-run in a child interpreter that loads the
instrumented build (``ORINFER_CORE_LIB``) with the sanitizer runtime preloaded.  A report from
either tool fails the child (``halt_on_error`` / non-zero exit code)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _runtime(name):
    out = subprocess.run(["gcc", f"-print-file-name={name}"], capture_output=True, text=True)
    path = out.stdout.strip()
    return path if os.path.isabs(path) and os.path.exists(path) else None


def _run(sanitizer, runtime, tests, extra_env):
    from orinfer_b200.ops import build
    lib = build.build_core(sanitizer)
    env = dict(os.environ, ORINFER_CORE_LIB=str(lib), LD_PRELOAD=runtime,
               PYTHONPATH=ROOT, **extra_env)
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", *tests]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)


def test_policy_core_is_clean_under_asan_and_ubsan():
    runtime = _runtime("libasan.so")
    if runtime is None:
        pytest.skip("no AddressSanitizer runtime in this toolchain")
    res = _run("asan", runtime,
               ["tests/test_sampling_core.py", "tests/test_prefix_cache.py",
                "tests/test_policy_core.py", "tests/test_weight_io.py",
                "tests/test_host_rows.py", "tests/test_transfers.py", "tests/test_properties.py"],
               {"ASAN_OPTIONS": "detect_leaks=0:halt_on_error=1:exitcode=97",
                "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1"})
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0, tail
    assert "ERROR: AddressSanitizer" not in tail and "runtime error:" not in tail
    assert " passed" in res.stdout


def test_rank_control_plane_is_clean_under_tsan():
    runtime = _runtime("libtsan.so")
    if runtime is None:
        pytest.skip("no ThreadSanitizer runtime in this toolchain")
    res = _run("tsan", runtime, ["tests/test_team.py"],
               {"TSAN_OPTIONS": "halt_on_error=1:exitcode=98:report_signal_unsafe=0"})
    tail = (res.stdout + res.stderr)[-3000:]
    if "unexpected memory mapping" in tail or "FATAL: ThreadSanitizer" in tail:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this container")
    assert res.returncode == 0, tail
    assert "WARNING: ThreadSanitizer" not in tail
    assert " passed" in res.stdout
