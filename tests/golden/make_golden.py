"""Generate tests/golden/tiny_golden.npz from the UNMODIFIED reference CPU backend.

Run where the reference tree is mounted and `make -C oracle ref` has built oracle/_ref:

    python tests/golden/make_golden.py

Contents (all from the tiny benchmark configuration, seed 0, 64-token prompt seed 1):
  sha_target / sha_head : sha256 of the generated GGUF files (guards generator drift)
  prompt                : the 64 prompt ids
  plain_f32 / plain_f16 : 128 greedy tokens, reference `run` semantics, f32 rings / all-f16 cache
  mtp_f32               : the same through MTP rounds of width 4 (must equal plain_f32)
  tf_logits_f16         : teacher-forced logits (all-f16 cache) at stream steps tf_steps
  drafts_f16            : host draft-head token after each of the first 32 generated tokens
  kat_q4_0_raw/_out, kat_q4_K_raw/_out : random blocks and their reference decode
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests.conftest import model_files, synth_module  # noqa: E402
from oracle.pyref import RefOracle  # noqa: E402


def sha(path):
    return hashlib.sha256(open(path, "rb").read()).hexdigest()


def main():
    s = synth_module()
    tp, hp = model_files("tiny")
    prompt = s.prompt_ids(64, s.TINY.n_vocab, seed=1)
    out = dict(sha_target=sha(tp), sha_head=sha(hp), prompt=prompt)
    for tag, f16 in (("f32", False), ("f16", True)):
        o = RefOracle(tp, hp, 512, f16, 4)
        out[f"plain_{tag}"], _ = o.generate(prompt, 128, 0)
        o.close()
    o = RefOracle(tp, hp, 512, False, 4)
    out["mtp_f32"], _ = o.generate(prompt, 128, 1)
    o.close()
    # teacher-forced on the f16 stream: logits at selected steps, draft tokens
    stream = np.concatenate([prompt, out["plain_f16"]])
    o = RefOracle(tp, hp, 512, True, 4)
    steps = [63, 64, 65, 80, 100, 127, 150, 190]
    logits, drafts = [], []
    for i, t in enumerate(stream[:191]):
        lg = o.forward(int(t), i)
        if i in steps:
            logits.append(lg)
        if 64 <= i < 96:
            drafts.append(o.draft(int(stream[i + 1]), i + 1))
    out["tf_steps"] = np.array(steps, dtype=np.int32)
    out["tf_logits_f16"] = np.stack(logits)
    out["drafts_f16"] = np.array(drafts, dtype=np.int32)
    rng = np.random.default_rng(11)
    raw0 = s.quantize_q4_0(rng.standard_normal(32 * 64).astype(np.float32))
    rawk = s.random_q4_K(rng, 256 * 8)
    out["kat_q4_0_raw"], out["kat_q4_0_out"] = raw0, o.dequant(s.Q4_0, raw0, 32 * 64)
    out["kat_q4_K_raw"], out["kat_q4_K_out"] = rawk, o.dequant(s.Q4_K, rawk, 256 * 8)
    o.close()
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "tiny_golden.npz"), **out)
    print({k: (v.shape if hasattr(v, "shape") else v) for k, v in out.items()})


if __name__ == "__main__":
    main()
