"""GPU parity tests of the whole decode / verify / draft path through the model C API."""
import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu

TOL = 1e-2          # max-abs logit error allowed, as a fraction of that step's logit range


def _teacher_forced(lg, name, n_prompt, n_steps, max_seq=2048, use_spec=False):
    """Feed the oracle's own greedy stream to both sides; return per-step (err/range, margins, argmax eq)."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files(name)
    o = PortOracle(tp, None, max_seq, True, 4)
    prompt = s.prompt_ids(n_prompt, o.n_vocab, seed=1)
    gen, _ = o.generate(prompt, n_steps, 0)
    o.close()
    stream = np.concatenate([prompt, gen])
    o = PortOracle(tp, None, max_seq, True, 4)
    rows = []
    with lg.Session(tp, None, max_seq) as g:
        for i, t in enumerate(stream[:-1]):
            want = o.forward(int(t), i)
            got = g.forward(int(t), i)
            rng_ = float(want.max() - want.min())
            top2 = np.partition(want, -2)[-2:]
            rows.append((float(np.abs(got - want).max()) / rng_, float(top2[1] - top2[0]) / rng_,
                         int(got.argmax() == want.argmax())))
    o.close()
    return np.array(rows)


@pytest.mark.parametrize("name", ["tiny", "tiny_cond", "var", "mid", "mid_k"])
def test_teacher_forced_logits_within_tolerance(lg, port_built, name):
    r = _teacher_forced(lg, name, 24, 40)
    err, margin, same = r[:, 0], r[:, 1], r[:, 2]
    print(f"{name}: max err/range {err.max():.2e}, mean {err.mean():.2e}, argmax equal {int(same.sum())}/{len(same)}")
    assert err.max() <= TOL, err.max()
    # the argmax must agree wherever the oracle's top-1/top-2 margin exceeds twice the measured error
    clear = margin > 2 * err.max()
    assert np.all(same[clear] == 1)


def test_golden_teacher_forced_logits(lg, golden):
    """Against logits recorded from the compiled reference backend (all-f16 cache)."""
    tp, _ = model_files("tiny")
    stream = np.concatenate([golden["prompt"], golden["plain_f16"]])
    steps = list(golden["tf_steps"])
    with lg.Session(tp, None, 512) as g:
        g.prefill(stream[:63], 0)
        worst = 0.0
        k = 0
        for i in range(63, 191):
            if i in steps:
                got = g.forward(int(stream[i]), i)
                want = golden["tf_logits_f16"][k]; k += 1
                worst = max(worst, float(np.abs(got - want).max() / (want.max() - want.min())))
            else:
                g.forward(int(stream[i]), i, want_logits=False)
    print(f"golden teacher-forced: worst err/range {worst:.2e}")
    assert worst <= TOL


def test_kv_rows_match_oracle(lg, port_built):
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files("tiny_cond")
    o = PortOracle(tp, None, 256, True, 4)
    toks = s.prompt_ids(20, o.n_vocab, seed=4)
    with lg.Session(tp, None, 256) as g:
        g.prefill(toks, 0)                       # blocks of 8 + a ragged tail of 4
        o.prefill(toks, 0)
        for layer in range(4):
            for pos in (0, 7, 8, 19):
                ko, vo = o.kv_row(layer, pos, 64)
                kg, vg = g.kv_row(layer, pos, 64)
                assert np.abs(kg - ko).max() < 5e-3 * max(1.0, np.abs(ko).max())
                assert np.abs(vg - vo).max() < 5e-3 * max(1.0, np.abs(vo).max())
                # stored values are exactly representable in f16
                assert np.array_equal(kg.astype(np.float16).astype(np.float32), kg)
    o.close()


def test_argmax_ties_pick_lowest_index(lg):
    tp, _ = model_files("zero")
    with lg.Session(tp, None, 64) as g:
        assert g.next(17, 0) == 0
        assert g.next(0, 1) == 0
        lgts = g.forward(5, 2)
        assert np.all(lgts == 0.0)


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8])
def test_spec_accept_semantics(lg, n):
    """adv = 1 + run of out[j-1] == toks[j]; out[j] equals the plain greedy successor."""
    s = synth_module()
    tp, _ = model_files("tiny_cond")
    prompt = s.prompt_ids(16, 4096, seed=6)
    with lg.Session(tp, None, 512, mtp_n=n) as g:
        plain, _ = g.generate(prompt, 40, 0)
    for bad_at in list(range(1, n)) + [None]:
        with lg.Session(tp, None, 512, mtp_n=n) as g:
            g.prefill(prompt[:-1], 0)
            best = g.next(int(prompt[-1]), 15)
            assert best == plain[0]
            toks = [int(plain[j]) for j in range(n)]            # all drafts right
            if bad_at is not None:
                toks[bad_at] = (toks[bad_at] + 1) % 4096
            adv, out = g.spec(toks, 16)
            want_adv = n if bad_at is None else bad_at
            assert adv == want_adv, (bad_at, adv)
            for j in range(adv):
                assert out[j] == plain[j + 1]


@pytest.mark.parametrize("name", ["tiny", "mid"])
@pytest.mark.parametrize("n", [2, 4, 8])
def test_mtp_stream_equals_plain_stream(lg, name, n):
    """E5/E6: replayed drafts at any acceptance rate, host-driven or device-resident, twice."""
    s = synth_module()
    tp, hp = model_files(name)
    with lg.Session(tp, None, 2048, mtp_n=n) as g:
        V = g.n_vocab
        prompt = s.prompt_ids(32, V, seed=8)
        plain, _ = g.generate(prompt, 96, 0)
    with lg.Session(tp, None, 2048, mtp_n=n) as g:
        again, _ = g.generate(prompt, 96, 0)
        assert np.array_equal(plain, again)                                # run twice
    with lg.Session(tp, None, 2048, mtp_n=n) as g:
        dev, _ = g.generate_device(prompt, 96, 0)
        assert np.array_equal(plain, dev[:96])
    for p in (0.0, 0.5, 0.8, 1.0):
        rp = s.replay_drafts(plain, V, p)
        with lg.Session(tp, None, 2048, mtp_n=n) as g:
            a, (nd, na) = g.generate(prompt, 96, 2, rp)
            assert np.array_equal(a, plain), (p, "host")
            if p == 1.0:
                assert na == nd
            if p == 0.0:
                assert na == 0
        with lg.Session(tp, None, 2048, mtp_n=n) as g:
            b, (nd2, na2) = g.generate_device(prompt, 96, 2, rp)
            assert np.array_equal(b[:96], plain), (p, "device")


@pytest.mark.parametrize("name", ["tiny", "var", "mid"])
def test_draft_head_rounds_equal_plain(lg, name):
    """The real draft head (random init: accepts almost nothing) never changes the output."""
    s = synth_module()
    tp, hp = model_files(name)
    with lg.Session(tp, hp, 1024) as g:
        prompt = s.prompt_ids(24, g.n_vocab, seed=9)
        plain, _ = g.generate(prompt, 48, 0)
    with lg.Session(tp, hp, 1024) as g:
        host, st = g.generate(prompt, 48, 1)
        assert np.array_equal(host, plain)
    with lg.Session(tp, hp, 1024) as g:
        dev, st2 = g.generate_device(prompt, 48, 1)
        assert np.array_equal(dev[:48], plain)
        assert st2[0] >= st[0] > 0


def test_draft_tokens_match_oracle_where_margin_allows(lg, port_built):
    """Device draft head vs the host draft of the oracle, teacher-forced on the oracle's stream."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files("tiny_cond")
    o = PortOracle(tp, hp, 512, True, 4)
    prompt = s.prompt_ids(24, 4096, seed=12)
    gen, _ = o.generate(prompt, 24, 0)
    o.close()
    stream = np.concatenate([prompt, gen])
    o = PortOracle(tp, hp, 512, True, 4)
    same = 0
    with lg.Session(tp, hp, 512) as g:
        for i in range(len(stream) - 1):
            want = o.forward(int(stream[i]), i)
            got = g.next(int(stream[i]), i)
            top2 = np.partition(want, -2)[-2:]
            if top2[1] - top2[0] > 2e-2 * (want.max() - want.min()):      # a clear margin: the greedy successor must agree
                assert got == int(want.argmax()), i
            if i >= 8:
                same += int(g.draft(int(stream[i + 1]), i + 1) == o.draft(int(stream[i + 1]), i + 1))
    o.close()
    total = len(stream) - 1 - 8
    print(f"draft tokens equal to the oracle's: {same}/{total}")
    assert same >= total * 0.8


def test_ring_wraps_without_corruption(lg, port_built):
    """Generate past the ring length of the sliding-window layers (window 64 + spare)."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files("mid")
    n = 1150                                      # ring rows = 64 + 1024
    with lg.Session(tp, None, 1400, mtp_n=4) as g:
        prompt = s.prompt_ids(8, g.n_vocab, seed=13)
        plain, _ = g.generate_device(prompt, n, 0)
    with lg.Session(tp, None, 1400, mtp_n=4) as g:
        rp = s.replay_drafts(plain, g.n_vocab, 0.7)
        mtp, _ = g.generate_device(prompt, n, 2, rp)
    assert np.array_equal(plain[:n], mtp[:n])
    # the oracle, teacher-forced near the end, still agrees on the logits
    o = PortOracle(tp, None, 1400, True, 4)
    stream = np.concatenate([prompt, plain])
    o.prefill(stream[:1100], 0)
    with lg.Session(tp, None, 1400) as g:
        g.prefill(stream[:1100], 0)
        for i in range(1100, 1110):
            want, got = o.forward(int(stream[i]), i), g.forward(int(stream[i]), i)
            assert np.abs(got - want).max() / (want.max() - want.min()) <= TOL
    o.close()


def test_prefix_save_restore(lg):
    s = synth_module()
    tp, _ = model_files("tiny")
    import ctypes as C
    with lg.Session(tp, None, 512) as g:
        L = g.L
        L.kvcache_save_prefix.argtypes = [C.c_void_p, C.c_int]
        L.kvcache_restore_prefix.argtypes = [C.c_void_p, C.c_int]
        toks = s.prompt_ids(40, 4096, seed=14)
        g.prefill(toks[:20], 0)
        L.kvcache_save_prefix(g.kv, 20)
        a = [g.next(int(t), 20 + i) for i, t in enumerate(toks[20:30])]
        g.prefill(toks[30:], 0)                                   # clobber rows 0..9
        L.kvcache_restore_prefix(g.kv, 20)
        b = [g.next(int(t), 20 + i) for i, t in enumerate(toks[20:30])]
        assert a == b
