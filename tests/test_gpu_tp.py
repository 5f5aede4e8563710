"""Tensor-parallel parity and failure detection on 2+ GPUs (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    import torch

    return torch.cuda.device_count()


def _run(mode, world, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "tp_worker.py"), mode]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.parametrize("mode", ["parity", "parity2"])
def test_tp2_tokens_match_oracle(mode):
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(mode, 2, 29611)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 2, r.stdout[-2000:]


def test_tp2_lfm2_conv_layers_split_by_channel():
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run("parity_lfm2", 2, 29619)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 2, r.stdout[-2000:]


@pytest.mark.parametrize("mode", ["prompt", "prompt_lfm2"])
def test_tp2_chunked_prompt_sums_partial_rows_across_ranks(mode):
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(mode, 2, 29623)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 2, r.stdout[-2000:]


def test_tp4_lfm2_conv_layers_split_by_channel():
    if _gpus() < 4:
        pytest.skip("needs 4 GPUs")
    r = _run("parity_lfm2", 4, 29621)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 4, r.stdout[-2000:]


def test_tp4_tokens_match_oracle():
    if _gpus() < 4:
        pytest.skip("needs 4 GPUs")
    r = _run("parity", 4, 29613)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 4


def test_tp8_tokens_match_oracle():
    if _gpus() < 8:
        pytest.skip("needs 8 GPUs")
    r = _run("parity", 8, 29617)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("TP_OK") == 8


def test_missing_rank_is_reported_not_hung():
    if _gpus() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run("timeout", 2, 29615)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_TIMEOUT_OK" in r.stdout
