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
