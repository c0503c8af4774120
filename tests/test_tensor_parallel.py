"""Tensor-parallel rollout on two gloo ranks: row-parallel linear, TP engine vs single-rank engine, weight sync."""
import os
import subprocess
import sys

import pytest


def _port() -> str:
    """A port that is free now: other jobs may share the machine, fixed port numbers collide."""
    from siirl_b200.execution.scheduler.launch import find_free_port
    return str(find_free_port())


def test_tensor_parallel_two_cpu_ranks():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, TP_DEVICE="cpu", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", _port(), os.path.join(here, "tp_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "TP_OK" in out.stdout


def test_expert_parallel_two_cpu_ranks():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, EP_DEVICE="cpu", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", _port(), os.path.join(here, "ep_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "EP_OK" in out.stdout


def test_tensor_parallel_training_matches_the_whole_model():
    import os
    import subprocess
    import sys

    from siirl_b200.execution.scheduler.launch import find_free_port
    here = os.path.dirname(os.path.abspath(__file__))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(find_free_port()), os.path.join(here, "tp_train_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2"))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "TP_TRAIN_OK" in out.stdout


@pytest.mark.parametrize("virtual,extra", [(1, 0), (2, 0), (2, 2)])
def test_pipeline_1f1b_schedule_matches_the_whole_model(virtual, extra):
    """Three stages under 1F1B with asynchronous sends (five micro-batches), and under the interleaved schedule with
    two model chunks per stage (six micro-batches; eight, i.e. a group that does not fill the pipeline): per-stage
    gradients equal the whole model's."""
    from siirl_b200.execution.scheduler.launch import find_free_port
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr",
           "127.0.0.1", "--master-port", str(find_free_port()), os.path.join(os.path.dirname(__file__), "pp_worker.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, OMP_NUM_THREADS="1", PP_VIRTUAL=str(virtual), PP_EXTRA=str(extra)))
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "PP_1F1B_OK" in out.stdout
