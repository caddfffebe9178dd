"""The example scripts run to completion on CPU and leave a clean exit status (the rank threads of a collected model are
joined before the interpreter shuts down)."""
import os
import subprocess
import sys

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script", ["train_and_save.py", "memory_efficient_loading.py", "generate.py"])
def test_example_runs(script):
    proc = subprocess.run([sys.executable, os.path.join(REPO, "examples", script)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "terminate called" not in proc.stderr
