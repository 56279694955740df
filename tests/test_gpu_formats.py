"""GPU parity tests of the block formats beyond q4_0 / q4_K: q8_0, q6_K, q5_K, q3_K matrices and tables, bf16 / f16 / f32
tables (decode contract: src/quant.c:184-274 of the reference; its device paths: src/cuda/model-cuda-i8.cu:141-196,645-746)."""
import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu

TOL = 1e-2


def _random_blocks(s, rng, t, n):
    if t == s.Q8_0:
        raw = rng.integers(0, 256, size=(n // 32, 34), dtype=np.uint8)
        raw[:, 1] &= 0x3F                                   # keep the f16 scale finite and small
        return raw.reshape(-1)
    raw = s.random_k_blocks(rng, n, t).reshape(-1, s.BLOCK_BYTES[t][1])
    return raw.reshape(-1)


@pytest.mark.parametrize("tname", ["Q8_0", "Q6_K", "Q5_K", "Q3_K"])
def test_dequant_bit_exact_all_byte_patterns(lg, port_built, tname):
    """Every packed byte uniform random: the device decode equals the host decode (itself pinned bit-exact to the compiled
    reference) to the last bit."""
    from oracle.pyref import PortOracle
    s = synth_module()
    t = getattr(s, tname)
    tp, _ = model_files("tiny")
    rng = np.random.default_rng(60 + t)
    rows, k = 24, 1024
    raw = _random_blocks(s, rng, t, rows * k)
    o = PortOracle(tp, None, 64)
    want = o.dequant(t, raw, rows * k).reshape(rows, k)
    o.close()
    got = lg.dequant(t, raw, rows, k)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("tname", ["F16", "BF16", "F32"])
def test_dense_table_rows_bit_exact(lg, tname):
    s = synth_module()
    rng = np.random.default_rng(70)
    x = (rng.standard_normal((8, 256)) * 3).astype(np.float32)
    if tname == "F16":
        raw, want = x.astype(np.float16).view(np.uint8), x.astype(np.float16).astype(np.float32)
    elif tname == "BF16":
        bits = (x.view(np.uint32) >> 16).astype(np.uint16)
        raw, want = bits.view(np.uint8), (bits.astype(np.uint32) << 16).view(np.float32)
    else:
        raw, want = x.view(np.uint8), x
    got = lg.dequant(getattr(s, tname), raw.reshape(-1), 8, 256)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("tname", ["Q8_0", "Q6_K", "Q5_K", "Q3_K"])
@pytest.mark.parametrize("m,k,M", [(64, 256, 1), (528, 1024, 4), (1040, 3840 if False else 3840 - 3840 % 256, 8), (96, 512, 5)])
def test_gemv_matches_f64_on_decoded_weights(lg, port_built, tname, m, k, M):
    from oracle.pyref import PortOracle
    s = synth_module()
    t = getattr(s, tname)
    tp, _ = model_files("tiny")
    rng = np.random.default_rng(m + k + M + t)
    if t == s.Q8_0:
        raw = s.quantize_q8_0(rng.standard_normal(m * k).astype(np.float32) * 0.02)
    else:
        raw = s.random_k_blocks(rng, m * k, t)
    o = PortOracle(tp, None, 64)
    w = o.dequant(t, raw, m * k).reshape(m, k).astype(np.float64)
    o.close()
    x = (rng.standard_normal((M, k)) * np.exp(rng.standard_normal((M, k)))).astype(np.float32)
    want = x.astype(np.float64) @ w.T
    got = lg.gemv(t, raw, m, k, x)
    assert np.abs(got - want).max() / np.abs(want).max() < 2e-4
    if k >= 512:
        got2 = lg.gemv(t, raw, m, k, x, kslices=2)
        assert np.abs(got2 - want).max() / np.abs(want).max() < 2e-4
    # a row of a block carries the bits of the same row run alone
    alone = lg.gemv(t, raw, m, k, x[M - 1:M])
    assert np.array_equal(alone[0].view(np.uint32), got[M - 1].view(np.uint32))


def test_mixed_format_model_teacher_forced_and_streams(lg, port_built):
    """A model whose tensors use every format at once, with a head holding dense matrices: logits against the oracle token
    by token, after a prompt pass, and speculative == plain streams with the head drafting."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files("mixed")
    o = PortOracle(tp, None, 512, True, 4)
    stream = s.prompt_ids(60, o.n_vocab, seed=71)
    worst = 0.0
    with lg.Session(tp, None, 512) as g:
        o.prefill(stream[:20], 0); g.prefill(stream[:20], 0)
        for i in range(20, 60):
            want, got = o.forward(int(stream[i]), i), g.forward(int(stream[i]), i)
            worst = max(worst, float(np.abs(got - want).max() / (want.max() - want.min())))
    o.close()
    print(f"mixed formats: worst err/range {worst:.2e}")
    assert worst <= TOL
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        assert g.head
        prompt = s.prompt_ids(40, g.n_vocab, seed=72)          # 40 tokens: the prompt pass of a non-q4 model takes the 8-token path
        plain, _ = g.generate(prompt, 48, 0)
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        a, st = g.generate(prompt, 48, 1)                       # the head (f16 / bf16 / q8_0 tensors) drafts on the device
        assert np.array_equal(a, plain) and st[0] > 0
        assert g.draft(int(plain[0]), 41) >= 0
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        b, _ = g.generate_device(prompt, 48, 2, s.replay_drafts(plain, g.n_vocab, 0.6))
        assert np.array_equal(b[:48], plain)
