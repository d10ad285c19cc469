"""Expert parallelism on real GPUs: a gpt_oss-style model whose experts are spread over 2 (4, 8 when present) GPUs of one
node, every rank decoding its own sequence with an all-to-all dispatch and combine per layer, produces on every rank the tokens
and logits of the same model held whole on one GPU.  One process per GPU under torchrun; skipped with fewer GPUs."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_ep_matches_single_gpu(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                        "--master-addr", "127.0.0.1", "--master-port", "29655", os.path.join(ROOT, "tests", "ep_worker.py"),
                        "small_oss", "21", "16"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert f"EP{world} OK" in r.stdout
