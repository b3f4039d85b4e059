"""The seeded random call sequences of tests/cdnn_failures.py on the reference CPU engine alone: the harness side of
the GPU test (tests/test_failure_paths_gpu.py) that needs no GPU.  One child process, as for the GPU cases."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_random_programs_run_on_the_reference_engine_and_depend_on_their_seed_only():
    if not (ROOT / "neoml_b200" / "lib" / "host" / "libcdnn_host.so").exists():
        pytest.skip("hosted NeoML libraries not built (they need a NeoML checkout)")
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "cdnn_failures.py"), "random_program_cpu"], capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, f"{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    row = json.loads(r.stdout.strip().splitlines()[-1])
    assert all(row["classes"].values()), row
    assert row["largest_value"] < 1e4, row   # the programs keep their values bounded (tanh after the growing steps)
