"""The package installs with pip and imports from the installed copy with no path edits
(counterpart of the reference's `pip install -e .`, setup.py:122-176 / pyproject.toml:1-12)."""
import os
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def test_pip_install_then_import_from_site_packages(tmp_path):
    site = tmp_path / "site"
    r = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
                        "--quiet", "--target", str(site), str(REPO / "ascend-ops_b200")],
                       capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert (site / "ascend910a_extras" / "lib" / "libb200ops.so").exists()
    code = ("import ascend910a_extras, ascend910a_extras.ops as ops, moe_decode_layer, moe_parallel;"
            "from ascend910a_extras import cabi;"
            "assert cabi.load().b200ops_version() >= 200;"
            "print(ascend910a_extras.__file__)")
    env = {k: v for k, v in os.environ.items() if k != "PYTHONPATH"}
    env["PYTHONPATH"] = str(site)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(tmp_path), env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert str(site) in r.stdout  # the installed copy, not the source tree
