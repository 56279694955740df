"""GPU tests of how the serving loop of the reference uses the backend around the speculative step:
the sampling hook (`model_pick`, src/run.c:83, src/cuda/mtp-kernel.cuh:103-111), plain and speculative
steps mixed in one session (the `-think` interleave, src/run.c:549-553), a head the device cannot run
(drafting off, decoding on: src/cuda/mtp-kernel.cuh:263-267,331-337) and the position guard."""
import ctypes as C

import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu

PICK_T = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_float), C.c_int)


class _Hook:
    """Installs a Python function as the library's `model_pick` for the duration of a with-block."""

    def __init__(self, lib, fn):
        self.slot = C.c_void_p.in_dll(lib, "model_pick")
        self.rows = []

        def cb(ptr, n):
            row = np.ctypeslib.as_array(ptr, shape=(n,)).copy()
            self.rows.append(row)
            return int(fn(row))
        self.cb = PICK_T(cb)

    def __enter__(self):
        self.slot.value = C.cast(self.cb, C.c_void_p).value
        return self

    def __exit__(self, *a):
        self.slot.value = None


def test_model_pick_rows_are_the_logits_and_its_choice_is_returned(lg, port_built):
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, _ = model_files("tiny_cond")
    prompt = s.prompt_ids(12, 4096, seed=41)
    second = lambda row: int(np.argsort(row, kind="stable")[-2])
    with lg.Session(tp, None, 256, mtp_n=4) as g:
        g.prefill(prompt[:-1], 0)
        greedy = g.next(int(prompt[-1]), 11)
        with _Hook(g.L, second) as h:
            picked = g.next(int(prompt[-1]), 11)
            assert len(h.rows) == 1
        o = PortOracle(tp, None, 256, True, 4)
        o.prefill(prompt[:-1], 0)
        want = o.forward(int(prompt[-1]), 11)
        o.close()
        row = h.rows[0]
        # the hook saw the soft-capped logits row of that step, and the call returned the hook's token
        assert np.abs(row - want).max() <= 1e-2 * (want.max() - want.min())
        assert int(row.argmax()) == greedy and picked == second(row) and picked != greedy
        # a verify block: out[j] is the hook's choice on row j, adv counts the run of out[j-1] == toks[j]
        toks = np.array([int(prompt[-1]), picked, 7, 9], dtype=np.int32)
        with _Hook(g.L, second) as h:
            adv, out = g.spec(toks, 11)
            assert len(h.rows) == 4
        assert out[0] == picked and [int(x) for x in out] == [second(r) for r in h.rows]
        want_adv = 1
        while want_adv < 4 and out[want_adv - 1] == toks[want_adv]:
            want_adv += 1
        assert adv == want_adv and adv >= 2
        # with the hook gone the greedy path is back
        assert g.next(int(prompt[-1]), 11) == greedy


def test_plain_and_speculative_steps_interleave_in_one_session(lg):
    s = synth_module()
    tp, _ = model_files("mid")
    with lg.Session(tp, None, 1024, mtp_n=4) as g:
        V = g.n_vocab
        prompt = s.prompt_ids(20, V, seed=42)
        plain, _ = g.generate(prompt, 80, 0)
    rp = s.replay_drafts(plain, V, 0.6)
    with lg.Session(tp, None, 1024, mtp_n=4) as g:
        g.prefill(prompt[:-1], 0)
        best, pos, got = g.next(int(prompt[-1]), 19), 20, []
        got.append(best)
        n_done = 1
        for seg, (mode, rounds) in enumerate([(2, 3), (0, 5), (2, 4), (0, 2), (2, 50)]):
            toks, st = g.rounds_host(best, pos, n_done, 80, rounds, mode, rp)
            got.extend(int(t) for t in toks)
            n_done += len(toks)
            best, pos = st["best"], st["pos"]
            if n_done >= 80:
                break
        assert got[:80] == [int(t) for t in plain[:80]]


def test_head_the_device_cannot_run_turns_drafting_off(lg):
    s = synth_module()
    tp, hp = model_files("mid_oddhead")
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        assert g.head                                   # the host accepted the file
        prompt = s.prompt_ids(16, g.n_vocab, seed=43)
        plain, _ = g.generate(prompt, 24, 0)
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        g.prefill(prompt[:-1], 0)
        first = g.next(int(prompt[-1]), 15)
        assert g.draft(first, 16) == -1                 # unusable on the device: -1, no exit
        assert g.draft(first, 16) == -1                 # and it stays off
        assert g.draft_chain(first, 17) == -1
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        out, st = g.generate(prompt, 24, 1)             # the caller pads the slots; the stream is unchanged
        assert np.array_equal(out, plain)
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        with pytest.raises(RuntimeError):
            g.generate_device(prompt, 24, 1)            # device-resident rounds need a head: refused, not crashed
        assert g.next(int(prompt[-1]), 15) == first


def test_rounds_that_could_leave_the_cache_are_refused(lg):
    s = synth_module()
    tp, _ = model_files("tiny")
    with lg.Session(tp, None, 64, mtp_n=4) as g:
        prompt = s.prompt_ids(8, 4096, seed=44)
        g.prefill(prompt[:-1], 0)
        first = g.next(int(prompt[-1]), 7)
        g.set_replay(np.zeros(256, dtype=np.int32))
        g.rounds_begin(first, 8, 1)
        assert g.rounds_enqueue(4, 2, 14, use_head=False) == 0        # 8 + 14 * 4 = 64 rows: fits
        _, st = g.rounds_collect(1, 0)
        assert st["pos"] <= 64
        left = (64 - st["pos"]) // 4
        assert g.rounds_enqueue(4, 2, left + 1, use_head=False) == -2  # one round too many
        assert g.rounds_enqueue(4, 2, left, use_head=False) == 0
        g.rounds_collect(1, 0)
        out = np.zeros(8, dtype=np.int32)
        toks = np.zeros(4, dtype=np.int32)
        assert g.L.lgs_spec(g.h, toks, 62, out) == -2                   # rows 62..65 of a 64-row cache


def test_blocking_calls_wait_once_per_round(lg):
    """mtp_draft runs the whole round ahead; the chained drafts and the verify that follow are answered from its record."""
    s = synth_module()
    tp, hp = model_files("mid")
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        V = g.n_vocab
        prompt = s.prompt_ids(20, V, seed=45)
        plain, _ = g.generate(prompt, 60, 0)
    rp = s.replay_drafts(plain, V, 0.7)
    for mode in (1, 3):                                   # the head's own drafts; the head's cost with replayed drafts
        with lg.Session(tp, hp, 1024, mtp_n=4) as g:
            g.prefill(prompt[:-1], 0)
            best = g.next(int(prompt[-1]), 19)
            before = g.host_syncs()
            toks, st = g.rounds_host(best, 20, 1, 60, 12, mode, rp if mode == 3 else None)
            waits = g.host_syncs() - before
            assert waits == 12, (mode, waits)              # one wait per round, not one per call (4 per round)
            got = [best] + [int(t) for t in toks]
            assert got == [int(t) for t in plain[:len(got)]], mode
            if mode == 3:
                assert st["n_accept"] > 0                   # the replayed drafts, not the random head's, were verified


def test_caller_that_verifies_other_tokens_than_drafted_gets_its_own_answer(lg):
    s = synth_module()
    tp, hp = model_files("mid")
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        V = g.n_vocab
        prompt = s.prompt_ids(16, V, seed=46)
        plain, _ = g.generate(prompt, 24, 0)
    with lg.Session(tp, hp, 512, mtp_n=4) as g:
        g.prefill(prompt[:-1], 0)
        best = g.next(int(prompt[-1]), 15)
        assert best == plain[0]
        d1 = g.draft(best, 16)                              # the whole round ran on the head's drafts
        assert d1 >= 0
        # the caller ignores them and verifies the true continuation with one wrong token in slot 2
        toks = np.array([best, plain[1], (plain[2] + 1) % V, plain[3]], dtype=np.int32)
        adv, out = g.spec(toks, 16)
        assert adv == 2 and out[0] == plain[1] and out[1] == plain[2]
        # a chained draft asked for another token than the recorded one still answers (synchronously), and the verify of
        # the true continuation after it is right
        best2, pos2 = int(out[1]), 18
        d = g.draft(best2, pos2)
        other = (d + 1) % V
        assert g.draft_chain(other, pos2 + 1) >= 0
        toks = np.array([best2, plain[3], plain[4], plain[5]], dtype=np.int32)
        adv, out = g.spec(toks, pos2)
        assert adv == 4 and [int(x) for x in out] == [int(x) for x in plain[3:7]]


def test_a_wait_that_runs_out_reports_and_returns(lg):
    """Every device-side wait in this library is bounded: when nothing completes the barrier, the kernel gives up after its
    limit, raises a status bit the host reads, and returns -- the context stays usable (no trap, no hang)."""
    s = synth_module()
    tp, _ = model_files("tiny")
    with lg.Session(tp, None, 64) as g:
        before = g.next(5, 0)
        assert g.L.lg_debug_bounded_wait(g.model, 1024) == 1      # LG_ERR_MBAR_TIMEOUT: the wait ran out and said so
        assert g.L.lg_debug_bounded_wait(g.model, 0) == -1        # bad argument, no launch
        assert g.next(5, 0) == before                              # the engine and the context still work


def test_low_confidence_drafts_are_called_off_and_the_output_does_not_change(lg):
    """Variable draft length: with the margin threshold out of reach every round drafts once and skips the two chained
    drafts; with the threshold off none is skipped.  The emitted stream is the plain greedy one in every case."""
    s = synth_module()
    tp, hp = model_files("mid")
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        prompt = s.prompt_ids(20, g.n_vocab, seed=47)
        plain, _ = g.generate(prompt, 48, 0)
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        g.set_draft_margin(1e30)
        dev, st = g.generate_device(prompt, 48, 1)
        assert np.array_equal(dev[:48], plain)
        rounds = st[0] // 3
        assert rounds > 0 and g.drafts_skipped() == 2 * rounds
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        g.set_draft_margin(0.0)
        dev, st = g.generate_device(prompt, 48, 1)
        assert np.array_equal(dev[:48], plain) and g.drafts_skipped() == 0
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        g.set_draft_margin(1e30)
        host, _ = g.generate(prompt, 48, 1)                     # the blocking calls see the padded slots and still agree
        assert np.array_equal(host, plain)
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        # a finite threshold: some rounds stop early, some do not -- the stream still does not move
        g.set_draft_margin(0.05)
        dev, st = g.generate_device(prompt, 48, 1)
        assert np.array_equal(dev[:48], plain)
