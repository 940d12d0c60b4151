"""The wheel holds the package and the prebuilt sm_100a library (no JIT step at import)."""
import os
import subprocess
import sys
import zipfile

from conftest import PKG_DIR


def test_wheel_contains_the_native_library(tmp_path):
    cmd = [sys.executable, "setup.py", "-q", "egg_info", "--egg-base", str(tmp_path),
           "build", "--build-base", str(tmp_path / "b"), "bdist_wheel", "-d", str(tmp_path / "dist")]
    subprocess.run(cmd, cwd=PKG_DIR, check=True, capture_output=True, timeout=900)
    wheels = os.listdir(tmp_path / "dist")
    assert len(wheels) == 1 and wheels[0].startswith("accelerated_scan_b200-") and "py3-none-linux" in wheels[0]
    names = zipfile.ZipFile(tmp_path / "dist" / wheels[0]).namelist()
    for member in ("__init__.py", "_native.py", "warp.py", "complex.py", "sharded.py", "stateful.py", "libascan_b200.so"):
        assert "accelerated_scan/" + member in names
