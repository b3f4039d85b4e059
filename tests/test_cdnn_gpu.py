"""The five benchmark configurations as NeoML CDnn graphs on the B200 engine, reached through NeoML's own factory
(CreateGpuMathEngine of the hosted libNeoMathEngine.so), against the same graphs on NeoML's CPU engine.

Each case runs tests/cdnn_parity.py in a process of its own: the hosted NeoMathEngine library and the oracle's
reference build carry the same soname and must not meet in one process.  "full" is the configuration's stated size.

Tolerance: gate (norm-wise max relative error) < 1e-4 for the default 3xTF32 arithmetic, < 1e-2 for the TF32 opt-in;
arg-max indices bit-exact.
"""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HOSTED = ROOT / "neoml_b200" / "lib" / "host" / "libcdnn_host.so"

pytestmark = pytest.mark.gpu


def run_parity(config: str, scale: str, flags: int = 0, threads: int = 16) -> dict:
    if not HOSTED.exists():
        pytest.skip("hosted NeoML libraries not built (make -C neoml_b200/host needs a NeoML checkout)")
    r = subprocess.run([sys.executable, str(ROOT / "tests" / "cdnn_parity.py"), "--config", config, "--scale", scale,
                        "--flags", str(flags), "--cpu-threads", str(threads)], capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, f"cdnn_parity failed:\n{r.stdout[-2000:]}\n{r.stderr[-4000:]}"
    row = json.loads(r.stdout.strip().splitlines()[-1])
    print(json.dumps(row))
    return row


def check(row: dict, tol: float) -> None:
    assert "B200" in row["gpu_engine"], row["gpu_engine"]
    for key, value in row.items():
        if key.endswith("_gate"):
            assert value < tol, f"{key} = {value:.3e} (bar {tol:g}) in {row['what']}"
        if key.endswith("_finite"):
            assert value, f"{key}: non-finite output in {row['what']}"


CONFIGS = ["1", "2", "3", "4", "4ones", "4causal", "5a", "5b", "5c"]


@pytest.mark.parametrize("config", CONFIGS)
def test_small_cdnn_matches_cpu_engine(config):
    row = run_parity(config, "small", threads=4)
    check(row, 1e-4)
    if config == "3":
        assert row["argmax_mismatches"] == 0


@pytest.mark.parametrize("config", CONFIGS)
def test_full_size_cdnn_matches_cpu_engine(config):
    row = run_parity(config, "full")
    check(row, 1e-4)
    if config == "3":
        assert row["argmax_mismatches"] == 0, f"{row['argmax_mismatches']} of {row['argmax_count']} arg-max indices differ"


@pytest.mark.parametrize("config", ["1", "3", "4", "5a"])
def test_tf32_opt_in_small(config):
    row = run_parity(config, "small", flags=2, threads=4)   # GpuMathEngineCublasUseTensorCoresTF32Flag
    check(row, 1e-2)
