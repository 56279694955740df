"""GPU parity tests of the wide (prompt) matmul -- q4 weights expanded to f16 in the kernel,
tcgen05.mma with f32 accumulation -- called through the C ABI."""
import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu


def _oracle():
    from oracle.pyref import PortOracle
    tp, _ = model_files("tiny")
    return PortOracle(tp, None, 64, False, 4)


def _weights(s, rng, wtype, m, k):
    o = _oracle()
    if wtype == "q4_0":
        raw, t = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32) * 0.02), s.Q4_0
    else:
        raw, t = s.random_q4_K(rng, m * k), s.Q4_K
    w = o.dequant(t, raw, m * k).reshape(m, k)
    o.close()
    return raw, t, w


@pytest.mark.parametrize("wtype,m,k", [("q4_0", 128, 64), ("q4_0", 256, 256), ("q4_0", 1024, 3840), ("q4_0", 80, 15360),
                                        ("q4_K", 512, 1024), ("q4_K", 48, 15360)])
@pytest.mark.parametrize("n", [1, 40, 64, 100, 129, 256])
def test_prefill_matmul_matches_oracle(lg, port_built, wtype, m, k, n):
    s = synth_module()
    rng = np.random.default_rng(m + k + n)
    raw, t, w = _weights(s, rng, wtype, m, k)
    x = rng.standard_normal((n, k)).astype(np.float32)
    got = lg.prefill_matmul(t, raw, m, k, x)
    # the kernel's operands: x rounded to f16, weights rounded to f16; f32 accumulation
    x16 = x.astype(np.float16).astype(np.float64)
    want = (w.astype(np.float64) @ x16.T).T
    scale = np.abs(want).max()
    err = np.abs(got - want).max() / scale
    # q4_0: d*(q-8) rounded once to f16 (2^-11 relative per weight); q4_K: two f16 products and an f16 fma
    assert err < (1e-3 if wtype == "q4_0" else 4e-3), err


def test_prefill_matmul_q4_0_weights_are_the_f16_rounding_of_the_exact_value(lg, port_built):
    """With one-hot activations the matmul returns single weights: each equals f16(d * (q - 8))."""
    s = synth_module()
    rng = np.random.default_rng(11)
    m, k = 128, 256
    raw, t, w = _weights(s, rng, "q4_0", m, k)
    x = np.zeros((k, k), dtype=np.float32)
    x[np.arange(k), np.arange(k)] = 1.0
    got = lg.prefill_matmul(t, raw, m, k, x)          # got[c][r] = W[r][c]
    want = w.astype(np.float16).astype(np.float32)
    assert np.array_equal(got.T.view(np.uint32), want.view(np.uint32))


def test_prefill_matmul_columns_are_independent(lg):
    """A token's result does not depend on how many other tokens share the block."""
    s = synth_module()
    rng = np.random.default_rng(12)
    m, k = 256, 1024
    raw = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32) * 0.02)
    x = rng.standard_normal((200, k)).astype(np.float32)
    full = lg.prefill_matmul(s.Q4_0, raw, m, k, x)
    part = lg.prefill_matmul(s.Q4_0, raw, m, k, x[:30])
    assert np.array_equal(full[:30].view(np.uint32), part.view(np.uint32))


@pytest.mark.parametrize("wtype", ["q4_0", "q4_K"])
def test_prefill_matmul_geglu_epilogue(lg, port_built, wtype):
    s = synth_module()
    rng = np.random.default_rng(13)
    m, k, n = 192, 512, 77
    raw_g, t, wg = _weights(s, rng, wtype, m, k)
    raw_u, _, wu = _weights(s, rng, wtype, m, k)
    x = rng.standard_normal((n, k)).astype(np.float32)
    got = lg.prefill_matmul(t, raw_g, m, k, x, raw_up=raw_u)
    x16 = x.astype(np.float16).astype(np.float64)
    g = (wg.astype(np.float64) @ x16.T).T
    u = (wu.astype(np.float64) @ x16.T).T
    gelu = 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    want = gelu * u
    assert np.abs(got - want).max() / np.abs(want).max() < 5e-3      # f16 output + f16 weights


# ---- the wide prompt pass through the model API ------------------------------------------------

@pytest.mark.parametrize("name,n", [("mid", 300), ("mid_k", 300), ("mid", 37)])
def test_wide_prefill_matches_oracle(lg, port_built, name, n):
    """model_prefill of n tokens (blocks of up to 256 on the tcgen05 path + a narrow tail): cache rows and the
    logits of the following step against the CPU oracle."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files(name)
    o = PortOracle(tp, None, 512, True, 4)
    toks = s.prompt_ids(n + 4, o.n_vocab, seed=21)
    o.prefill(toks[:n], 0)
    with lg.Session(tp, None, 512) as g:
        g.prefill(toks[:n], 0)
        kv_dim = 2 * 256
        for layer in range(o.n_layer if hasattr(o, "n_layer") else 3):
            for pos in sorted({max(0, n - 60), n - 33, n - 9, n - 1}):
                ko, vo = o.kv_row(layer, pos, kv_dim)
                kg, vg = g.kv_row(layer, pos, kv_dim)
                assert np.abs(kg - ko).max() < 1e-2 * max(1.0, np.abs(ko).max()), (layer, pos)
                assert np.abs(vg - vo).max() < 1e-2 * max(1.0, np.abs(vo).max()), (layer, pos)
        for i in range(n, n + 4):
            want, got = o.forward(int(toks[i]), i), g.forward(int(toks[i]), i)
            assert np.abs(got - want).max() / (want.max() - want.min()) <= 1e-2
    o.close()


def test_wide_prefill_then_mtp_equals_plain(lg):
    """After a wide prompt pass the speculative stream is still byte-identical to plain greedy decoding."""
    s = synth_module()
    tp, _ = model_files("mid")
    with lg.Session(tp, None, 1024, mtp_n=4) as g:
        prompt = s.prompt_ids(200, g.n_vocab, seed=22)
        plain, _ = g.generate_device(prompt, 96, 0)
    with lg.Session(tp, None, 1024, mtp_n=4) as g:
        rp = s.replay_drafts(plain, g.n_vocab, 0.7)
        mtp, _ = g.generate_device(prompt, 96, 2, rp)
    assert np.array_equal(plain[:96], mtp[:96])


@pytest.mark.parametrize("name,n", [("mid", 100), ("tiny", 70), ("mid", 13)])
def test_mixed_prefill_matches_oracle(lg, port_built, name, n):
    """model_prefill_mixed / model_prefill_embd: media positions take an embedding row as it is (wide blocks and the
    narrow 8-token tail both), then the next steps' logits against the CPU oracle."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files(name)
    o = PortOracle(tp, None, 256, True, 4)
    rng = np.random.default_rng(41)
    toks = s.prompt_ids(n + 3, o.n_vocab, seed=23)
    n_rows = 9
    rows = (rng.standard_normal((n_rows, o.n_embd)) * 2.0).astype(np.float32)
    ids = toks[:n].astype(np.int32).copy()
    where = rng.choice(n, size=n_rows, replace=False)
    where[0] = n - 1                                     # one media position in the narrow tail
    for r, w in enumerate(where):
        ids[w] = -(r + 1)
    o.prefill_mixed(rows, ids, 0)
    with lg.Session(tp, None, 256) as g:
        g.prefill_mixed(rows, ids, 0)
        for i in range(n, n + 3):
            want, got = o.forward(int(toks[i]), i), g.forward(int(toks[i]), i)
            assert np.abs(got - want).max() / (want.max() - want.min()) <= 1e-2
    o.close()


def test_embd_prefill_matches_oracle(lg, port_built):
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files("mid")
    o = PortOracle(tp, None, 256, True, 4)
    rng = np.random.default_rng(42)
    n = 45
    rows = (rng.standard_normal((n, o.n_embd)) * 2.0).astype(np.float32)
    o.prefill_mixed(rows, -(np.arange(n, dtype=np.int32) + 1), 0)
    toks = s.prompt_ids(3, o.n_vocab, seed=24)
    with lg.Session(tp, None, 256) as g:
        g.prefill_embd(rows, 0)
        for i in range(3):
            want, got = o.forward(int(toks[i]), n + i), g.forward(int(toks[i]), n + i)
            assert np.abs(got - want).max() / (want.max() - want.min()) <= 1e-2
    o.close()
