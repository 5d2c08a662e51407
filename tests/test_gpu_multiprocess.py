"""Real multi-GPU runs: one process per GPU over NVLink, every algorithm
(including NVLS multimem when the driver grants a multicast object) against a
CPU oracle gathered through gloo.  Skipped on a single-GPU machine, where
tests/test_gpu_emulated_collectives.py covers the same kernels."""
import json
import os
import subprocess
import sys

import pytest

from conftest import gpu_count

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_world(world, tmp_path, nvls=True):
    out = tmp_path / f"report_{world}.json"
    env = dict(os.environ, PENNY_TEST_NVLS="1" if nvls else "0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + world),
           os.path.join(ROOT, "tests", "_mp_worker.py"), str(out)]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    return json.loads(out.read_text())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_all_collectives(world, tmp_path):
    if gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    rep = run_world(world, tmp_path)
    assert rep["failures"] == [], "\n".join(rep["failures"][:20])
    assert rep["checked"] > 100
