"""Tensor-parallel decode stack on two GPUs: NCCL all-reduce and the library's own peer-memory
exchange against the unsharded CPU oracle.  Needs 2 GPUs (skipped otherwise); ranks are separate
processes, one per GPU, NVLS off."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_stack_matches_unsharded_oracle(tmp_path):
    import test_tp_gloo as T
    import tp_worker as W
    from ferric_b200 import synth
    from ferric_b200.stack import TPPlan, layer_shards

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "tp2.npz")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), "2", str(port), out])
             for r in range(2)]
    for p in procs:
        assert p.wait(timeout=300) == 0
    got = np.load(out)
    T.HID, T.NFF, T.QOUT, T.KV = W.HID, W.NFF, W.QOUT, W.KV
    plan1 = TPPlan.make(1, 0, W.HID, W.NFF, W.QOUT, W.KV)
    h = synth.activations(W.B, W.HID, seed=5)
    for l in range(W.LAYERS):
        h = T.layer_forward(plan1, layer_shards(plan1, T.full_layer(100 + 10 * l)), h, lambda a: None)
    tol = 1e-4 + 1e-3 * np.abs(h).max()
    assert np.abs(got["nccl"] - h).max() <= tol
    assert np.abs(got["fused"] - h).max() <= tol
    assert np.array_equal(got["fused"], got["fused_replay"])       # graph replay == eager
    assert np.array_equal(got["nccl"], got["nccl_replay"])
