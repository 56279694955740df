"""The reference's own host half (src/gguf.c, quant.c, model.c, mtp.c, unmodified) driving this repository's CUDA backend
on a GPU: oracle/_ref/libref_b200_n4.so is those sources + the test shim + lg_engine.o (`make -C oracle dropin`)."""
import os

import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO = os.path.join(ROOT, "oracle", "_ref", "libref_b200_n4.so")


def _session(target, head, max_seq):
    from oracle import pyref

    class RefHostOnB200(pyref._Oracle):
        prefix = "ref_"
        fresh_copy = True          # the backend keeps one engine per loaded image, like the reference's file-scope state

        def __init__(self):
            super().__init__(SO, target, head, max_seq, False)
    return RefHostOnB200()


@pytest.mark.skipif(not os.path.exists(SO), reason="drop-in artefact not built (needs the reference tree at build time)")
@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_reference_host_code_on_this_backend_plain_equals_mtp_equals_own_host(lg, name):
    s = synth_module()
    tp, hp = model_files(name)
    with lg.Session(tp, hp, 1024, mtp_n=4) as g:
        prompt = s.prompt_ids(24, g.n_vocab, seed=51)
        own, _ = g.generate(prompt, 48, 0)                       # this repository's host code on the same backend
        V = g.n_vocab
    o = _session(tp, hp, 1024)
    assert o.mtp_n == 4 and o._f("has_head")(o.h) == 1           # the reference's mtp_open accepted the head file
    plain, _ = o.generate(prompt, 48, 0)                         # its model_prefill / model_forward_next loop
    o.close()
    o = _session(tp, hp, 1024)
    mtp, st = o.generate(prompt, 48, 1)                          # its mtp_draft / mtp_draft_chain / model_forward_spec rounds
    o.close()
    o = _session(tp, hp, 1024)
    rep, st2 = o.generate(prompt, 48, 2, s.replay_drafts(plain, V, 0.6))
    o.close()
    assert np.array_equal(plain, own)
    assert np.array_equal(mtp, plain) and st[0] > 0
    assert np.array_equal(rep, plain) and st2[1] > 0
