"""Multi-GPU: the tensor-parallel stack (NCCL all-reduce after the row-parallel linears) against
the NumPy chain, one process per GPU.  Needs at least two GPUs; single-GPU boxes skip it."""
import os
import subprocess
import sys

import pytest

import ullm_cuda as U

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    return U.backend_probe().device_count


@pytest.mark.parametrize("enc,m,mode", [("fp8", 1, "push"), ("aq4", 4, "push"), ("fp8", 8, "nccl"), ("fp8", 24, "push"),
                                        ("fp8", 1, "push-cluster"), ("aq4", 2, "push-cluster"), ("fp8", 3, "push-block")])
def test_tensor_parallel_stack(enc, m, mode):
    n = _gpus()
    if n < 2:
        pytest.skip("needs two GPUs")
    world = 8 if n >= 8 else (4 if n >= 4 else 2)  # every GPU of the box: 2, 4 or 8 ranks
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29581", WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), enc, str(m), mode],
                              env=dict(env, RANK=str(r), LOCAL_RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=600)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timeout")
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
