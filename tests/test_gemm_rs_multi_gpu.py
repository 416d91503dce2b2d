"""GEMM + reduce-scatter on 2 or more GPUs (skipped on a single-GPU box): child processes under torchrun."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, provider, protocol):
    env = dict(os.environ, FTB_SYMM_PROVIDER=provider, FTB_RS_PROTOCOL=protocol, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "tests", "_gemm_rs_worker.py")]
    r = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    print(r.stdout[-4000:])
    assert r.returncode == 0


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("provider,protocol", [("auto", "auto"), ("auto", "pull"), ("auto", "staged"), ("auto", "push"),
                                               ("cuda_ipc", "push"), ("cuda_ipc", "staged"), ("auto", "copy"), ("cuda_ipc", "copy")])
def test_gemm_rs_matches_oracle(provider, protocol):
    """auto/auto = the copy-engine exchange at two ranks, from four ranks on the fused kernel with the pull protocol
    (in-switch reduction) when the box offers NVSwitch multicast, else push; cuda_ipc/staged = the staged protocol with plain peer loads.  The worker also runs
    the FP8 form, which is always staged, in every combination."""
    _run(min(torch.cuda.device_count(), 8), provider, protocol)
