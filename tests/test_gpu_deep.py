"""GPU parity tests of the long-context span attention kernel (G tiles of 64 keys per CTA, online softmax),
forced on at small cache lengths so the CPU oracle can follow."""
import importlib

import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu

TOL = 1e-2


@pytest.fixture
def deep(lg):
    lg.set_attn_deep(128, 3)            # spans of 3 x 64 keys on every full-attention layer
    yield lg
    lg.set_attn_deep(4096, 0)


@pytest.mark.parametrize("name", ["mid", "var"])
def test_span_attention_logits_match_oracle(deep, port_built, name):
    """Teacher-forced logits deep enough for several spans, against the CPU oracle."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files(name)
    n = 600
    o = PortOracle(tp, None, 1024, True, 4)
    toks = s.prompt_ids(n + 6, o.n_vocab, seed=51)
    o.prefill(toks[:n], 0)
    with deep.Session(tp, None, 1024) as g:
        g.prefill(toks[:n], 0)
        for i in range(n, n + 6):
            want, got = o.forward(int(toks[i]), i), g.forward(int(toks[i]), i)
            assert np.abs(got - want).max() / (want.max() - want.min()) <= TOL
    o.close()


@pytest.mark.parametrize("n", [2, 4, 5, 8])
def test_span_attention_mtp_stream_equals_plain(deep, n):
    """A row's result does not depend on the verify width: speculative == plain, byte for byte, across span borders."""
    s = synth_module()
    tp, _ = model_files("mid")
    n_gen = 420                                           # crosses several 192-key span borders
    with deep.Session(tp, None, 1024, mtp_n=n) as g:
        prompt = s.prompt_ids(150, g.n_vocab, seed=52)
        plain, _ = g.generate_device(prompt, n_gen, 0)
    for p in (0.0, 0.7, 1.0):
        with deep.Session(tp, None, 1024, mtp_n=n) as g:
            rp = s.replay_drafts(plain, g.n_vocab, p)
            mtp, _ = g.generate_device(prompt, n_gen, 2, rp)
        assert np.array_equal(plain[:n_gen], mtp[:n_gen]), (n, p)


def test_span_attention_equals_tile_attention_stream(lg):
    """Same greedy stream with and without the span kernel (the two decompositions agree to rounding; on this
    well-conditioned model the argmax never flips over 300 tokens)."""
    s = synth_module()
    tp, _ = model_files("mid")
    with lg.Session(tp, None, 1024) as g:
        prompt = s.prompt_ids(150, g.n_vocab, seed=53)
        a, _ = g.generate_device(prompt, 300, 0)
    lg.set_attn_deep(128, 2)
    try:
        with lg.Session(tp, None, 1024) as g:
            b, _ = g.generate_device(prompt, 300, 0)
    finally:
        lg.set_attn_deep(4096, 0)
    same = int((a[:300] == b[:300]).sum())
    print(f"span vs tile kernel: {same}/300 tokens equal")
    first_diff = int(np.argmax(a[:300] != b[:300])) if same < 300 else 300
    assert first_diff >= 50                      # free-running streams may part ways late; early divergence would be a bug
