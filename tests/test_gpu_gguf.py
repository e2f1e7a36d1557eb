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


def test_proj_fused_and_split(F, ctx):
    """Proj::load / matmul / gate_up_swiglu (crates/ferric-llama/src/qwen3.rs:192-228): q|k|v with V in Q6_K beside
    Q4_K Q and K -- the mix real Q4_K_M files carry -- loads as a Split projection and its product equals the
    reference's matmul-per-part-and-concatenate on the oracle; same formats load Fused; gate|up goes through the fused
    SwiGLU kernel when it is one matrix and through matmul + swiglu when it is not, with the same result."""
    rng = np.random.default_rng(3)
    hidden, nq, nkv, n_ff = 512, 96, 32, 64
    q = synth.q4k_blocks(rng, nq * hidden // 256)
    k = synth.q4k_blocks(rng, nkv * hidden // 256)
    v6 = synth.q6k_blocks(rng, nkv * hidden // 256)
    v4 = synth.q4k_blocks(rng, nkv * hidden // 256)
    gate = synth.q4k_blocks(rng, n_ff * hidden // 256)
    up4 = synth.q4k_blocks(rng, n_ff * hidden // 256)
    up6 = synth.q6k_blocks(rng, n_ff * hidden // 256)
    v8 = synth.q8_0_blocks(rng, nkv * hidden // 32)
    g = F.Gguf.parse(W.build([], [("q", [hidden, nq], 12, q.tobytes()), ("k", [hidden, nkv], 12, k.tobytes()),
                                  ("v6", [hidden, nkv], 14, v6.tobytes()), ("v4", [hidden, nkv], 12, v4.tobytes()),
                                  ("v8", [hidden, nkv], 8, v8.tobytes()),
                                  ("gate", [hidden, n_ff], 12, gate.tobytes()), ("up4", [hidden, n_ff], 12, up4.tobytes()),
                                  ("up6", [hidden, n_ff], 14, up6.tobytes())]))
    tol = lambda got, ref: (np.abs(got - ref) <= 1e-4 + 1e-3 * np.abs(ref)).all()
    for m in (1, 3, 20):                                            # 20 rows: the tensor-core decode kernel on the Q4_K parts
        x = synth.activations(m, hidden, seed=m)
        xd = torch.from_numpy(x).cuda()
        split = g.proj(ctx, "q", "k", "v6")
        assert not split.fused() and split.part_types() == [12, 12, 14] and (split.rows(), split.cols()) == (nq + 2 * nkv, hidden)
        ref = np.concatenate([O.matmul_q(q, 12, nq, hidden, x), O.matmul_q(k, 12, nkv, hidden, x), O.matmul_q(v6, 14, nkv, hidden, x)], axis=1)
        assert tol(split.matmul(xd).cpu().numpy(), ref)
        three = g.proj(ctx, "q", "v8", "v6")                        # a part without a prepared form between two that have one
        ref3 = np.concatenate([O.matmul_q(q, 12, nq, hidden, x), O.matmul_q(v8, 8, nkv, hidden, x), O.matmul_q(v6, 14, nkv, hidden, x)], axis=1)
        assert tol(three.matmul(xd).cpu().numpy(), ref3)
        fused = g.proj(ctx, "q", "k", "v4")
        assert fused.fused() and fused.part_types() == [12]
        reff = O.matmul_q(np.concatenate([q, k, v4]), 12, nq + 2 * nkv, hidden, x)
        assert tol(fused.matmul(xd).cpu().numpy(), reff)
        gu_f, gu_s = g.proj(ctx, "gate", "up4"), g.proj(ctx, "gate", "up6")
        assert gu_f.fused() and not gu_s.fused()
        ref_f = O.swiglu(O.matmul_q(np.concatenate([gate, up4]), 12, 2 * n_ff, hidden, x), n_ff)
        ref_s = O.swiglu(np.concatenate([O.matmul_q(gate, 12, n_ff, hidden, x), O.matmul_q(up6, 14, n_ff, hidden, x)], axis=1), n_ff)
        assert tol(gu_f.gate_up_swiglu(xd, n_ff).cpu().numpy(), ref_f)
        assert tol(gu_s.gate_up_swiglu(xd, n_ff).cpu().numpy(), ref_s)
        with pytest.raises(F.FerricError) as e:
            gu_s.gate_up_swiglu(xd, n_ff + 16)
        assert e.value.status == 3
        for p in (split, three, fused, gu_f, gu_s):
            p.close()
    single = g.proj(ctx, "q")
    assert single.fused() and single.rows() == nq
    single.close()
    with pytest.raises(F.FerricError, match="no tensor"):
        g.proj(ctx, "q", "nope")
    # a projection over matrices built by hand
    parts = [F.QMatrix.from_bytes(ctx, q, 12, nq, hidden), F.QMatrix.from_bytes(ctx, v6, 14, nkv, hidden)]
    p = F.Proj.from_parts(ctx, parts)
    x = synth.activations(2, hidden, seed=9)
    ref = np.concatenate([O.matmul_q(q, 12, nq, hidden, x), O.matmul_q(v6, 14, nkv, hidden, x)], axis=1)
    assert tol(p.matmul(torch.from_numpy(x).cuda()).cpu().numpy(), ref)
    p.close()
    g.close()
