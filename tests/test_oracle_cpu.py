"""CPU tests: the oracle against the reference's golden vectors, the host C, the C ABI surface."""
import hashlib
import os
import re

import numpy as np
import pytest

from tests.conftest import ROOT, has_ref, model_files, synth_module


def _sha(p):
    return hashlib.sha256(open(p, "rb").read()).hexdigest()


def test_generator_is_reproducible(golden):
    tp, hp = model_files("tiny")
    assert _sha(tp) == str(golden["sha_target"])
    assert _sha(hp) == str(golden["sha_head"])


@pytest.mark.skipif(not has_ref(4), reason="compiled reference backend not present")
@pytest.mark.parametrize("tname", ["Q8_0", "Q6_K", "Q5_K", "Q3_K", "Q4_K", "Q4_0"])
def test_port_decode_bit_exact_vs_compiled_reference_on_random_blocks(port_built, tname):
    """All byte patterns (f16 scale fields kept finite): the host decode this repository ships equals the reference's."""
    from oracle.pyref import PortOracle, RefOracle
    s = synth_module()
    t = getattr(s, tname)
    tp, _ = model_files("tiny")
    blk, nbytes = s.BLOCK_BYTES[t]
    rng = np.random.default_rng(80 + t)
    raw = rng.integers(0, 256, size=(3000, nbytes), dtype=np.uint8)
    for col in {s.Q8_0: [0], s.Q6_K: [208], s.Q5_K: [0, 2], s.Q3_K: [108], s.Q4_K: [0, 2], s.Q4_0: [0]}[t]:
        raw[:, col + 1] &= 0xBF                              # clear one exponent bit: no inf / nan scales
    a, b = RefOracle(tp, None, 64), PortOracle(tp, None, 64)
    ya, yb = a.dequant(t, raw.reshape(-1), 3000 * blk), b.dequant(t, raw.reshape(-1), 3000 * blk)
    a.close(); b.close()
    assert np.array_equal(ya.view(np.uint32), yb.view(np.uint32))


def test_port_dequant_matches_reference_kat(golden, port_built):
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files("tiny")
    o = PortOracle(tp, None, 64, False, 4)
    a = o.dequant(s.Q4_0, golden["kat_q4_0_raw"], 2048)
    b = o.dequant(s.Q4_K, golden["kat_q4_K_raw"], 2048)
    o.close()
    assert np.array_equal(a.view(np.uint32), golden["kat_q4_0_out"].view(np.uint32))
    assert np.array_equal(b.view(np.uint32), golden["kat_q4_K_out"].view(np.uint32))
    # third opinion: the numpy decoder of the generator
    assert np.array_equal(s.dequantize_q4_0(golden["kat_q4_0_raw"]), golden["kat_q4_0_out"])


@pytest.mark.parametrize("f16", [False, True])
def test_port_stream_matches_reference_golden(golden, port_built, f16):
    from oracle.pyref import PortOracle
    tp, hp = model_files("tiny")
    o = PortOracle(tp, hp, 512, f16, 4)
    g, _ = o.generate(golden["prompt"], 128, 0)
    o.close()
    assert np.array_equal(g, golden["plain_f16" if f16 else "plain_f32"])


def test_port_mtp_equals_plain_and_golden(golden, port_built):
    from oracle.pyref import PortOracle
    tp, hp = model_files("tiny")
    o = PortOracle(tp, hp, 512, False, 4)
    g, stats = o.generate(golden["prompt"], 128, 1)
    o.close()
    assert np.array_equal(g, golden["mtp_f32"]) and np.array_equal(g, golden["plain_f32"])
    assert stats[0] > 0


def test_port_teacher_forced_logits_and_drafts_bit_exact(golden, port_built):
    from oracle.pyref import PortOracle
    tp, hp = model_files("tiny")
    stream = np.concatenate([golden["prompt"], golden["plain_f16"]])
    o = PortOracle(tp, hp, 512, True, 4)
    steps = list(golden["tf_steps"])
    got, drafts = [], []
    for i, t in enumerate(stream[:191]):
        lg = o.forward(int(t), i)
        if i in steps:
            got.append(lg)
        if 64 <= i < 96:
            drafts.append(o.draft(int(stream[i + 1]), i + 1))
    o.close()
    assert np.array_equal(np.stack(got).view(np.uint32), golden["tf_logits_f16"].view(np.uint32))
    assert np.array_equal(np.array(drafts), golden["drafts_f16"])


@pytest.mark.skipif(not has_ref(4), reason="compiled reference backend not present")
@pytest.mark.parametrize("name", ["var", "mid", "mid_k", "mixed", "hd512"])
def test_port_bit_exact_vs_compiled_reference(port_built, name):
    """Every optional branch (softcap, output scale, rope divisors, V=K, KV sharing, q4_K, hd 256; q8_0 / q6_K / q5_K / q3_K
    matrices with f16 / bf16 head tensors; full-attention layers of head size 512)."""
    from oracle.pyref import PortOracle, RefOracle
    s = synth_module()
    tp, hp = model_files(name)
    a, b = RefOracle(tp, hp, 256, True, 4), PortOracle(tp, hp, 256, True, 4)
    toks = s.prompt_ids(12, a.n_vocab, seed=3)
    for i, t in enumerate(toks):
        la, lb = a.forward(int(t), i), b.forward(int(t), i)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)), (name, i)
        if hp and i > 0:
            assert a.draft(int(t), i + 1) == b.draft(int(t), i + 1)
    ga, _ = a.generate(toks, 24, 1 if hp else 0)
    gb, _ = b.generate(toks, 24, 1 if hp else 0)
    a.close(); b.close()
    assert np.array_equal(ga, gb)


@pytest.mark.skipif(not has_ref(4), reason="compiled reference backend not present")
@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_port_mixed_prefill_bit_exact_vs_compiled_reference(port_built, name):
    """Media positions (embedding rows in place of token ids; token 0's per-layer row on models that have one)."""
    from oracle.pyref import PortOracle, RefOracle
    s = synth_module()
    tp, _ = model_files(name)
    a, b = RefOracle(tp, None, 128, True, 4), PortOracle(tp, None, 128, True, 4)
    rng = np.random.default_rng(31)
    toks = s.prompt_ids(14, a.n_vocab, seed=5)
    rows = rng.standard_normal((3, a.n_embd)).astype(np.float32)
    ids = toks.astype(np.int32).copy()
    ids[[2, 3, 9]] = [-1, -3, -2]                       # rows 0, 2, 1
    a.prefill_mixed(rows, ids[:13], 0); b.prefill_mixed(rows, ids[:13], 0)
    la, lb = a.forward(int(toks[13]), 13), b.forward(int(toks[13]), 13)
    a.close(); b.close()
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))


def test_replay_rounds_equal_plain_on_oracle(port_built):
    """Oracle-replayed drafts at any acceptance rate never change the stream; adv counts follow p."""
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files("tiny")
    prompt = s.prompt_ids(16, 4096, seed=2)
    o = PortOracle(tp, None, 256, True, 4)
    plain, _ = o.generate(prompt, 40, 0)
    o.close()
    for p, lo, hi in ((0.0, 0, 0), (1.0, 1, 1), (0.5, 0.1, 0.9)):
        o = PortOracle(tp, None, 256, True, 4)
        g, (nd, na) = o.generate(prompt, 40, 2, s.replay_drafts(plain, 4096, p))
        o.close()
        assert np.array_equal(g, plain)
        # replay[i] is the draft for stream index i; a fully correct table accepts every draft
        assert lo <= (na / nd if p not in (0.0, 1.0) else round(na / nd, 6)) <= hi or p == 0.5


def test_host_rejects_bad_heads_and_files(port_built, tmp_path):
    from oracle.pyref import PortOracle
    s = synth_module()
    tp, hp = model_files("tiny")
    # a head built for a different backbone width must be refused (target keeps running headless)
    import dataclasses
    other = dataclasses.replace(s.TINY, n_embd=512)
    bad = str(tmp_path / "bad_head.gguf")
    s.write_head(bad, s.TINY_HEAD, other, seed=1)
    o = PortOracle(tp, bad, 64, False, 4)
    assert o._f("has_head")(o.h) == 0
    o.close()
    # a target file is not a head
    o = PortOracle(tp, tp, 64, False, 4)
    assert o._f("has_head")(o.h) == 0
    o.close()
    # truncated / non-GGUF files fail to open
    junk = tmp_path / "junk.gguf"
    junk.write_bytes(open(tp, "rb").read()[:1000])
    with pytest.raises(RuntimeError):
        PortOracle(str(junk), None, 64, False, 4)
    junk.write_bytes(b"NOPE" + bytes(100))
    with pytest.raises(RuntimeError):
        PortOracle(str(junk), None, 64, False, 4)


def test_library_exports_every_declared_symbol(lg):
    """The C-ABI library loads without a GPU and exports everything include/lg_b200.h declares."""
    L = lg.load()
    text = open(os.path.join(ROOT, "include", "lg_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = set(re.findall(r"\b((?:lg_|model_|kvcache_|mtp_)\w+)\s*(?:\(|;)", text))
    assert declared and declared == set(lg.ABI_SYMBOLS), declared ^ set(lg.ABI_SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def test_weight_byte_formula():
    s = synth_module()
    assert s.B12.weight_bytes() == 6_617_825_280
    assert s.E4B.weight_bytes() == 2_521_202_688
    assert s.TINY.weight_bytes() == 2_838_528
