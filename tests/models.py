"""Named, seeded test models (shapes small enough for the CPU oracle to finish in seconds)."""
import dataclasses
import os

from tests.conftest import synth_module


def shapes():
    s = synth_module()
    tiny = s.TINY
    return {
        # the benchmark plan's tiny configuration (4 layers, hd 64, PLE 64) and its 1-block head
        "tiny": (tiny, s.TINY_HEAD, 0, 1),
        # same, q-norm weight hd^-0.5: a well-conditioned twin for end-to-end logit gates
        "tiny_cond": (dataclasses.replace(tiny, q_norm_scale=64 ** -0.5), s.TINY_HEAD, 0, 1),
        # every optional branch: softcap, layer_output_scale, rope_freqs, V = K projection, KV sharing
        "var": (dataclasses.replace(tiny, n_layer=8, shared_kv_layers=4, softcap=30.0, layer_output_scale=True,
                                    rope_freqs=True, drop_attn_v=True, q_norm_scale=64 ** -0.5),
                dataclasses.replace(s.TINY_HEAD, softcap=20.0, layer_output_scale=True, n_layer=2), 3, 4),
        # head size 256 with grouped queries, short window (ring wraps early), no PLE
        "mid": (s.TargetShape(n_layer=6, n_embd=512, n_head=8, n_head_kv=2, head_dim=256, n_ff=2048, n_vocab=8192,
                              window=64, local_per_global=2, ple=0, q_norm_scale=256 ** -0.5),
                s.HeadShape(n_layer=2, n_inner=256, n_head=8, n_ff=512), 5, 6),
        # q4_K weights (super-blocks of 256)
        "mid_k": (s.TargetShape(n_layer=3, n_embd=512, n_head=8, n_head_kv=2, head_dim=256, n_ff=2048, n_vocab=8192,
                                window=64, local_per_global=2, ple=0, q_norm_scale=256 ** -0.5, wtype=s.Q4_K),
                  None, 7, 8),
        # --- layer cuts of the benchmark shapes (2 layers: one sliding-window, one full-attention; vocab cut to 32768) ---
        # 12B-class shape, q4_0, norms = 1 as the benchmark files have them
        "b12_cut": (dataclasses.replace(s.B12, n_layer=2, n_vocab=32768), None, 20, 21),
        # its well-conditioned twin (q-norm weight hd^-0.5) with a 1-block head of the benchmark head's width
        "b12_cut_cond": (dataclasses.replace(s.B12, n_layer=2, n_vocab=32768, q_norm_scale=256 ** -0.5),
                         dataclasses.replace(s.B12_HEAD, n_layer=1), 20, 21),
        # the same shape in q4_K
        "b12k_cut": (dataclasses.replace(s.B12, n_layer=2, n_vocab=32768, wtype=s.Q4_K), None, 22, 23),
        "b12k_cut_cond": (dataclasses.replace(s.B12, n_layer=2, n_vocab=32768, wtype=s.Q4_K, q_norm_scale=256 ** -0.5),
                          None, 22, 23),
        # E4B-class shape: per-layer embeddings of width 256 together with head size 256, 8 / 2 heads
        "e4b_cut": (dataclasses.replace(s.E4B, n_layer=2, n_vocab=32768), None, 24, 25),
        "e4b_cut_cond": (dataclasses.replace(s.E4B, n_layer=2, n_vocab=32768, q_norm_scale=256 ** -0.5),
                         dataclasses.replace(s.E4B_HEAD, n_layer=1), 24, 25),
        # full-attention layers with head size 512 beside sliding-window layers of 256 (real Gemma-4 geometry)
        "hd512": (s.TargetShape(n_layer=4, n_embd=512, n_head=4, n_head_kv=2, head_dim=256, head_dim_global=512, n_ff=1024,
                                n_vocab=4096, window=64, local_per_global=1, ple=0, q_norm_scale=256 ** -0.5),
                  None, 26, 27),
        # a head whose 3 query heads the target's 2 KV heads do not divide: the device must turn drafting off, not exit
        "mid_oddhead": (s.TargetShape(n_layer=6, n_embd=512, n_head=8, n_head_kv=2, head_dim=256, n_ff=2048, n_vocab=8192,
                                      window=64, local_per_global=2, ple=0, q_norm_scale=256 ** -0.5),
                        s.HeadShape(n_layer=1, n_inner=256, n_head=3, n_ff=512), 5, 11),
        # every block format the reference reads in one model: q6_K embeddings / head and o-projection, q8_0 queries, q5_K
        # keys, values, gate and up, q3_K down-projection, a q6_K per-layer table; the head file carries an f16 and a bf16
        # matrix beside q8_0 ones (dense matrices are accepted in a draft head only)
        "mixed": (dataclasses.replace(tiny, q_norm_scale=64 ** -0.5,
                                      wtypes={"token_embd.weight": s.Q6_K, "attn_q.weight": s.Q8_0, "attn_k.weight": s.Q5_K,
                                              "attn_v.weight": s.Q5_K, "attn_output.weight": s.Q6_K, "ffn_gate.weight": s.Q5_K,
                                              "ffn_up.weight": s.Q5_K, "ffn_down.weight": s.Q3_K, "inp_gate.weight": s.Q8_0,
                                              "per_layer_token_embd.weight": s.Q6_K, "per_layer_model_proj.weight": s.Q6_K}),
                  dataclasses.replace(s.TINY_HEAD, wtypes={"pre_projection.weight": s.F16, "post_projection.weight": s.BF16,
                                                           "attn_q.weight": s.Q8_0, "ffn_down.weight": s.Q8_0}), 30, 31),
        # all-zero weights: every logit ties at 0, the argmax must be index 0
        "zero": (dataclasses.replace(tiny, sigma=0.0, ple=0), None, 9, 10),
    }


def build(name: str, cache: str):
    s = synth_module()
    target, head, seed_t, seed_h = shapes()[name]
    tp = s.cached(cache, f"{name}.gguf", s.write_target, target, seed_t)
    hp = s.cached(cache, f"{name}_head.gguf", s.write_head, head, target, seed_h) if head is not None else None
    return tp, hp
