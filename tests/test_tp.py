"""The shard axis: host helpers as gloo ranks on CPU, the model on 2 GPUs."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(nproc, env_extra, timeout):
    env = dict(os.environ, **env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(HERE, "tp_worker.py")]
    p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0 and "TP_OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def test_shard_axis_host_helpers_on_two_cpu_ranks():
    import __graft_entry__ as ge
    ge.build()
    _run(2, {"MTJ_TP_CPU": "1"}, 300)


def test_a_rank_that_leaves_between_calls_is_noticed_on_the_host():
    _run(3, {"MTJ_TP_CPU": "2"}, 120)


@pytest.mark.gpu
@pytest.mark.parametrize("mp,chunk_pipeline,push_reduce", [(2, "0", "0"), (2, "1", "0"), (2, "0", "1"), (4, "0", "0"),
                                                            (4, "1", "1"), (8, "0", "0"), (8, "1", "1")])
def test_tensor_parallel_generate_matches_oracle(mp, chunk_pipeline, push_reduce):
    """chunk_pipeline = "1": prefill / eval run as chunk pairs whose all-reduce overlaps the other chunk's layer.
    push_reduce = "1": the batched decode step's all-reduce is the push kernel fused with the split-K reduction
    and the LayerNorm instead of the three-kernel chain."""
    import torch
    if torch.cuda.device_count() < mp:
        pytest.skip(f"needs {mp} GPUs")
    _run(mp, {"NCCL_DEBUG": "WARN", "MTJ_TP_PIPE": chunk_pipeline, "MTJ_TP_PUSH": push_reduce}, 240)
