"""GGUF file -> device matrices -> products: the loaders' qm / qm_cat contract (crates/ferric-llama/src/qwen35.rs:366-402)
through ferric_cuda_qmatrix_from_gguf, against the same bytes handed to from_bytes directly and against the oracle."""
import numpy as np
import pytest
import torch

import gguf_writer as W
from ferric_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F():
    import ferric_b200
    return ferric_b200


@pytest.fixture(scope="module")
def ctx(F):
    c = F.Context(0)
    yield c
    c.close()


def test_qm_and_qm_cat(F, ctx):
    rng = np.random.default_rng(0)
    hidden = 512
    q = synth.q4k_blocks(rng, 96 * hidden // 256)
    k = synth.q4k_blocks(rng, 32 * hidden // 256)
    v = synth.q4k_blocks(rng, 32 * hidden // 256)
    down = synth.q6k_blocks(rng, hidden * 768 // 256)
    head = synth.q8_0_blocks(rng, 40 * hidden // 32)
    gate = synth.q5k_blocks(rng, 64 * hidden // 256)
    data = W.build([("general.architecture", W.STR, "qwen3")],
                   [("blk.0.attn_q.weight", [hidden, 96], 12, q.tobytes()), ("blk.0.attn_k.weight", [hidden, 32], 12, k.tobytes()),
                    ("blk.0.attn_v.weight", [hidden, 32], 12, v.tobytes()), ("blk.0.ffn_down.weight", [768, hidden], 14, down.tobytes()),
                    ("output.weight", [hidden, 40], 8, head.tobytes()), ("blk.0.ffn_gate.weight", [hidden, 64], 13, gate.tobytes()),
                    ("blk.0.attn_norm.weight", [hidden], 0, np.ones(hidden, np.float32).tobytes())])
    g = F.Gguf.parse(data)
    x = synth.activations(3, hidden, seed=1)
    xd = torch.from_numpy(x).cuda()

    qkv = g.qmatrix(ctx, "blk.0.attn_q.weight", "blk.0.attn_k.weight", "blk.0.attn_v.weight")     # qm_cat
    assert (qkv.rows(), qkv.cols(), qkv.ggml_type()) == (160, hidden, 12)
    ref = O.matmul_q(np.concatenate([q, k, v]), 12, 160, hidden, x)
    got = qkv.matmul(xd).cpu().numpy()
    assert (np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref)).all()
    direct = F.QMatrix.from_bytes(ctx, np.concatenate([q, k, v]), 12, 160, hidden)
    assert np.array_equal(direct.matmul(xd).cpu().numpy(), got)                                   # same bytes, same result

    d = g.qmatrix(ctx, "blk.0.ffn_down.weight")                                                   # qm: dims [in, out]
    assert (d.rows(), d.cols(), d.ggml_type()) == (hidden, 768, 14)
    xf = synth.activations(2, 768, seed=2)
    ref = O.matmul_q(down, 14, hidden, 768, xf)
    got = d.matmul(torch.from_numpy(xf).cuda()).cpu().numpy()
    assert (np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref)).all()

    g5 = g.qmatrix(ctx, "blk.0.ffn_gate.weight")                                                  # Q5_K (some Q4_K_M files mix it in)
    assert (g5.rows(), g5.cols(), g5.ggml_type()) == (64, hidden, 13)
    ref = O.matmul_q(gate.reshape(-1), 13, 64, hidden, x)
    got = g5.matmul(xd).cpu().numpy()
    assert (np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref)).all()
    g5.close()

    h = g.qmatrix(ctx, "output.weight")
    assert (h.rows(), h.cols(), h.ggml_type()) == (40, hidden, 8)

    with pytest.raises(F.FerricError, match="mixed quant formats"):
        g.qmatrix(ctx, "blk.0.attn_q.weight", "output.weight")
    with pytest.raises(F.FerricError, match="input dim differs"):
        _mismatch(F, ctx)
    with pytest.raises(F.FerricError, match="no tensor"):
        g.qmatrix(ctx, "blk.9.attn_q.weight")
    with pytest.raises(F.FerricError) as e:
        g.qmatrix(ctx, "blk.0.attn_norm.weight")                                                  # F32: no packed kernel, and 1-D
    assert e.value.status in (2, 3)
    for m in (qkv, direct, d, h):
        m.close()
    g.close()


def _mismatch(F, ctx):
    rng = np.random.default_rng(1)
    a = synth.q6k_blocks(rng, 16 * 256 // 256)
    b = synth.q6k_blocks(rng, 16 * 512 // 256)
    g = F.Gguf.parse(W.build([], [("a", [256, 16], 14, a.tobytes()), ("b", [512, 16], 14, b.tobytes())]))
    try:
        g.qmatrix(ctx, "a", "b")
    finally:
        g.close()
