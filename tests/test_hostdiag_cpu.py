"""The two front doors that need neither a GPU nor torch: they must run as plain scripts, say which paths they
tested, open real artifacts with the container's rules, and exit 0 / 3 / 2."""
import os
import subprocess
import sys

import pytest

from ninfer_fusion_b200 import cli

SCRIPT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ninfer_fusion_b200", "hostdiag.py")


def _run(*args):
    # -X importtime would be noisy; instead the script itself is asked not to have torch loaded
    code = ("import runpy, sys; sys.argv = ['hostdiag'] + %r\n"
            "try:\n    runpy.run_path(%r, run_name='__main__')\nexcept SystemExit as e:\n    rc = e.code\n"
            "assert 'torch' not in sys.modules, 'hostdiag imported torch'\nsys.exit(rc)\n") % (list(args), SCRIPT)
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60)


def test_cufree_reports_tested_paths_without_torch():
    r = _run("cufree")
    assert r.returncode == 0, r.stderr
    assert "/dev/nvidiactl" in r.stdout and "libcuda.so.1" in r.stdout and "_C.so" in r.stdout
    assert "cannot tell whether a GPU works" in r.stdout


def test_hostpath_opens_a_real_artifact_and_refuses_a_foreign_file(tmp_path):
    path = tmp_path / "tiny.ninfer"
    assert cli.main(["make-artifact", "--model", "tiny-dense", "--out", str(path)]) == 0
    ok = _run("hostpath", str(path))
    assert ok.returncode == 0, ok.stdout + ok.stderr
    assert "registry gate: accepted" in ok.stdout and "content_tokens_emitted: 0" in ok.stdout
    other = tmp_path / "other.bin"
    other.write_bytes(b"not an artifact at all")
    bad = _run("hostpath", str(path), str(other))
    assert bad.returncode == 3 and "refused: not a version-2 .ninfer file" in bad.stdout
    assert _run().returncode == 2
