"""Seeded synthetic Gemma-4-architecture GGUF files (target models and draft heads).

Real checkpoints are not available offline, so every test and benchmark runs on
random-init files with the shapes of the configurations named in the benchmark
plan.  The file bytes are the ground truth for both sides of every parity check
(the oracle and the CUDA backend read the same file), so the q4_0 encoder here
only has to be *a* valid encoder, not ggml's.

What the loaders on the other side expect (reference: src/gguf.c:249-386 container,
src/model.c:67-189 target keys and per-layer geometry from tensor shapes,
src/mtp.c:124-233 draft-head keys and tensors):

* container: GGUF v3, little endian, data section aligned to `general.alignment`;
* tensor dims[0] is the contraction length k, dims[1] the row count m, a row is
  k/32 consecutive 18-byte q4_0 blocks (or k/256 144-byte q4_K super-blocks);
* `n_vocab` is the length of the `tokenizer.ggml.tokens` string array.

Small files are generated with numpy (bit-reproducible on any host); the large
benchmark files can be generated on the GPU with torch (`device="cuda"`), which
is seconds instead of minutes but only reproducible on the same GPU type.
"""
from __future__ import annotations

import hashlib
import os
import struct
from dataclasses import dataclass, field, asdict
from typing import Dict, List, Optional

import numpy as np

# ggml tensor type ids (reference: include/quant.h:13-24)
F32, F16, Q4_0, Q8_0, Q3_K, Q4_K, Q5_K, Q6_K, BF16 = 0, 1, 2, 8, 11, 12, 13, 14, 30
BLOCK_BYTES = {Q4_0: (32, 18), Q8_0: (32, 34), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
# gguf metadata value types (reference: include/gguf.h:17-32)
T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR = 4, 5, 6, 7, 8, 9


# ----------------------------------------------------------------------------
# block encoders
# ----------------------------------------------------------------------------

def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    """Encode float32 values (size % 32 == 0) as q4_0 blocks; returns uint8 bytes.

    Per 32 values: d = f16(amax/7); q = clamp(rint(x/d) + 8, 0, 15); byte j holds
    element j in the low nibble and element j+16 in the high nibble; block = f16 d
    then 16 bytes (layout: reference src/quant.c:83-86, decode :276-285).
    """
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    amax = np.abs(x).max(axis=1)
    d16 = (amax / np.float32(7.0)).astype(np.float16)
    d = d16.astype(np.float32)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, 1), np.float32(0.0)).astype(np.float32)
    q = np.clip(np.rint(x * inv[:, None]) + 8, 0, 15).astype(np.uint8)
    packed = (q[:, :16] | (q[:, 16:] << 4)).astype(np.uint8)
    out = np.empty((x.shape[0], 18), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = packed
    return out.reshape(-1)


def dequantize_q4_0(raw: np.ndarray) -> np.ndarray:
    """numpy decode of q4_0 bytes (used by tests as a third opinion)."""
    b = np.frombuffer(raw, dtype=np.uint8).reshape(-1, 18)
    d = b[:, :2].copy().view(np.float16).astype(np.float32)
    lo = (b[:, 2:] & 0xF).astype(np.int32) - 8
    hi = (b[:, 2:] >> 4).astype(np.int32) - 8
    return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)


def random_q4_K(rng: np.random.Generator, n_elems: int) -> np.ndarray:
    """Random q4_K super-blocks (256 values, 144 bytes) with weights of magnitude <~ 0.1.

    d ~ U(0.5,1.5)e-4 and dmin ~ 7.5 d give roughly zero-mean weights:
    y = d*sc*q - dmin*m with sc, m uniform 6-bit and q uniform 4-bit
    (layout and decode: reference src/quant.c:56-61,155-182).
    """
    nb = n_elems // 256
    out = np.empty((nb, 144), dtype=np.uint8)
    d = (rng.uniform(0.5e-4, 1.5e-4, nb)).astype(np.float32)
    dmin = (d * 7.5 * rng.uniform(0.9, 1.1, nb)).astype(np.float32)
    out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out[:, 4:] = rng.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    return out.reshape(-1)


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """Encode float32 values as q8_0 blocks: per 32 values d = f16(amax/127), q = rint(x/d) as int8 (layout: reference
    src/quant.c:78-81)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    d16 = (np.abs(x).max(axis=1) / np.float32(127.0)).astype(np.float16)
    d = d16.astype(np.float32)
    inv = np.where(d > 0, np.float32(1.0) / np.where(d > 0, d, 1), np.float32(0.0)).astype(np.float32)
    q = np.clip(np.rint(x * inv[:, None]), -127, 127).astype(np.int8)
    out = np.empty((x.shape[0], 34), dtype=np.uint8)
    out[:, 0:2] = d16.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.reshape(-1)


def random_k_blocks(rng: np.random.Generator, n_elems: int, wtype: int) -> np.ndarray:
    """Random q6_K / q5_K / q3_K super-blocks with weights of magnitude <~ 0.1: every packed byte uniform, the f16
    super-block scales drawn so that d * (largest integer scale) * (largest q) stays small (layouts: reference
    src/quant.c:48-78; decode :184-274)."""
    blk, nbytes = BLOCK_BYTES[wtype]
    nb = n_elems // blk
    out = rng.integers(0, 256, size=(nb, nbytes), dtype=np.uint8)
    if wtype == Q6_K:        # |q| <= 32, |scale| <= 128
        d = rng.uniform(1.0e-5, 2.5e-5, nb).astype(np.float16)
        out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    elif wtype == Q3_K:      # |q| <= 4, |scale| <= 32
        d = rng.uniform(4.0e-4, 8.0e-4, nb).astype(np.float16)
        out[:, 108:110] = d.view(np.uint8).reshape(-1, 2)
    elif wtype == Q5_K:      # q <= 31, scale <= 63; dmin ~ 15.5 d centres the weights
        d = rng.uniform(2.5e-5, 7.5e-5, nb).astype(np.float32)
        dmin = (d * 15.5 * rng.uniform(0.9, 1.1, nb)).astype(np.float32)
        out[:, 0:2] = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
        out[:, 2:4] = dmin.astype(np.float16).view(np.uint8).reshape(-1, 2)
    else:
        raise ValueError(wtype)
    return out.reshape(-1)


def _torch_q4_0(x):
    """Same encoder as quantize_q4_0 on a torch tensor (any device); returns uint8 tensor."""
    import torch
    x = x.reshape(-1, 32).float()
    amax = x.abs().amax(dim=1)
    d16 = (amax / 7.0).to(torch.float16)
    d = d16.float()
    inv = torch.where(d > 0, 1.0 / torch.where(d > 0, d, torch.ones_like(d)), torch.zeros_like(d))
    q = (torch.round(x * inv[:, None]) + 8).clamp_(0, 15).to(torch.uint8)
    packed = q[:, :16] | (q[:, 16:] << 4)
    out = torch.empty((x.shape[0], 18), dtype=torch.uint8, device=x.device)
    out[:, 0:2] = d16.view(torch.uint8).reshape(-1, 2)
    out[:, 2:] = packed
    return out.reshape(-1)


# ----------------------------------------------------------------------------
# container writer
# ----------------------------------------------------------------------------

def _s(b: str) -> bytes:
    e = b.encode("utf-8")
    return struct.pack("<Q", len(e)) + e


class GGUFWriter:
    """Two-pass streaming writer: declare metadata and tensor shapes, then stream payloads."""

    ALIGN = 32

    def __init__(self, path: str):
        self.path = path
        self.kv: List[bytes] = []
        self.tensors: List[dict] = []

    # -- metadata
    def add_u32(self, k, v): self.kv.append(_s(k) + struct.pack("<II", T_U32, v))
    def add_f32(self, k, v): self.kv.append(_s(k) + struct.pack("<If", T_F32, v))
    def add_str(self, k, v): self.kv.append(_s(k) + struct.pack("<I", T_STR) + _s(v))

    def add_arr_i32(self, k, vals):
        self.kv.append(_s(k) + struct.pack("<IIQ", T_ARR, T_I32, len(vals)) +
                       np.asarray(vals, dtype="<i4").tobytes())

    def add_arr_bool(self, k, vals):
        self.kv.append(_s(k) + struct.pack("<IIQ", T_ARR, T_BOOL, len(vals)) +
                       np.asarray(vals, dtype=np.uint8).tobytes())

    def add_arr_str(self, k, vals):
        body = b"".join(_s(v) for v in vals)
        self.kv.append(_s(k) + struct.pack("<IIQ", T_ARR, T_STR, len(vals)) + body)

    # -- tensors
    @staticmethod
    def nbytes(ttype: int, dims) -> int:
        n = int(np.prod(dims))
        if ttype in BLOCK_BYTES:
            return n // BLOCK_BYTES[ttype][0] * BLOCK_BYTES[ttype][1]
        return {F32: 4 * n, F16: 2 * n, BF16: 2 * n}[ttype]

    def declare(self, name: str, dims, ttype: int, producer):
        """producer() -> bytes-like (numpy uint8 array or bytes) of exactly nbytes."""
        self.tensors.append(dict(name=name, dims=list(dims), type=ttype, producer=producer))

    def write(self) -> str:
        """Stream the file; returns the sha256 of its bytes."""
        off = 0
        for t in self.tensors:
            t["offset"] = off
            off += (self.nbytes(t["type"], t["dims"]) + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        head = struct.pack("<4sIQQ", b"GGUF", 3, len(self.tensors), len(self.kv)) + b"".join(self.kv)
        for t in self.tensors:
            head += _s(t["name"]) + struct.pack("<I", len(t["dims"]))
            head += struct.pack("<%dQ" % len(t["dims"]), *t["dims"])
            head += struct.pack("<IQ", t["type"], t["offset"])
        pad = (-len(head)) % self.ALIGN
        sha = hashlib.sha256()
        with open(self.path, "wb") as f:
            for chunk in (head, b"\0" * pad):
                f.write(chunk); sha.update(chunk)
            for t in self.tensors:
                raw = t["producer"]()
                raw = raw.tobytes() if hasattr(raw, "tobytes") else bytes(raw)
                want = self.nbytes(t["type"], t["dims"])
                if len(raw) != want:
                    raise ValueError(f"{t['name']}: {len(raw)} bytes, expected {want}")
                tail = b"\0" * ((-want) % self.ALIGN)
                f.write(raw); f.write(tail)
                sha.update(raw); sha.update(tail)
        return sha.hexdigest()


# ----------------------------------------------------------------------------
# model shapes
# ----------------------------------------------------------------------------

@dataclass
class TargetShape:
    n_layer: int
    n_embd: int
    n_head: int
    n_head_kv: int
    head_dim: int
    n_ff: int
    n_vocab: int
    window: int
    local_per_global: int            # k in "k:1 local:global", anchored so the last layer is global
    ple: int = 0
    n_ctx: int = 131072
    rope_base: float = 1e6
    rope_base_swa: float = 1e4
    eps: float = 1e-6
    softcap: float = 0.0
    shared_kv_layers: int = 0
    # branch-exercising options (off in the benchmark files)
    layer_output_scale: bool = False
    rope_freqs: bool = False
    drop_attn_v: bool = False
    q_norm_scale: Optional[float] = None   # "conditioned twin": attn_q_norm.weight = this constant
    wtype: int = Q4_0
    sigma: float = 0.02
    head_dim_global: Optional[int] = None  # head size of the full-attention layers when it differs (Gemma-4: 512 vs 256)
    # per-tensor formats: tensor-name suffix (e.g. "ffn_down.weight", "token_embd.weight") -> ggml type, overriding wtype
    wtypes: Dict[str, int] = field(default_factory=dict)

    def hd(self, l: int) -> int:
        return self.head_dim if (self.is_local(l) or self.head_dim_global is None) else self.head_dim_global

    def is_local(self, l: int) -> bool:
        return (self.n_layer - 1 - l) % (self.local_per_global + 1) != 0

    def weight_bytes(self) -> int:
        """Algorithmic bytes of quantized weights one decode/verify step streams."""
        ne, H, Hkv, hd, L = self.n_embd, self.n_head, self.n_head_kv, self.head_dim, self.n_layer
        total = self.n_vocab * ne + ne * self.ple * L
        for l in range(L):
            hd = self.hd(l)
            total += ne * H * hd + 2 * ne * Hkv * hd + H * hd * ne + 3 * ne * self.n_ff + 2 * ne * self.ple
        return int(total * 0.5625)


@dataclass
class HeadShape:
    n_layer: int
    n_inner: int
    n_head: int
    n_ff: int
    eps: float = 1e-6
    softcap: float = 0.0
    layer_output_scale: bool = False
    with_post: bool = True
    sigma: float = 0.02
    wtypes: Dict[str, int] = field(default_factory=dict)    # tensor-name suffix -> ggml type (default q4_0)


# Shapes of the benchmark configurations.
TINY = TargetShape(n_layer=4, n_embd=256, n_head=4, n_head_kv=1, head_dim=64, n_ff=1024, n_vocab=4096,
                   window=128, local_per_global=3, ple=64)
TINY_HEAD = HeadShape(n_layer=1, n_inner=256, n_head=4, n_ff=1024)
E4B = TargetShape(n_layer=35, n_embd=2048, n_head=8, n_head_kv=2, head_dim=256, n_ff=16384,
                  n_vocab=262144, window=512, local_per_global=5, ple=256)
E4B_HEAD = HeadShape(n_layer=4, n_inner=256, n_head=8, n_ff=2048)
B12 = TargetShape(n_layer=48, n_embd=3840, n_head=16, n_head_kv=8, head_dim=256, n_ff=15360,
                  n_vocab=262144, window=1024, local_per_global=5, ple=0)
B12_HEAD = HeadShape(n_layer=4, n_inner=1024, n_head=16, n_ff=4096)


class _Gen:
    """Weight source: numpy (host, portable) or torch (device, fast)."""

    def __init__(self, seed: int, device: str = "cpu"):
        self.device = device
        self.rng = np.random.default_rng(seed)
        if device != "cpu":
            import torch
            self.tgen = torch.Generator(device=device)
            self.tgen.manual_seed(seed)

    def weight(self, n: int, sigma: float, wtype: int):
        if wtype == Q4_K:
            return random_q4_K(self.rng, n)
        if wtype in (Q6_K, Q5_K, Q3_K):
            return random_k_blocks(self.rng, n, wtype)
        if self.device == "cpu" or wtype in (Q8_0, F16, BF16):
            x = self.rng.standard_normal(n, dtype=np.float32) * np.float32(sigma)
            if wtype == Q8_0:
                return quantize_q8_0(x)
            if wtype == F16:
                return x.astype(np.float16).view(np.uint8)
            if wtype == BF16:
                return (x.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
            return quantize_q4_0(x) if wtype == Q4_0 else x.view(np.uint8)
        import torch
        out = []
        step = 1 << 28                         # bound device temporaries to ~1 GiB of f32
        for s in range(0, n, step):
            x = torch.randn(min(step, n - s), generator=self.tgen, device=self.device) * sigma
            out.append(_torch_q4_0(x).cpu().numpy() if wtype == Q4_0 else x.cpu().numpy().view(np.uint8))
        return np.concatenate(out) if len(out) > 1 else out[0]


def _ones(n, v=1.0):
    return lambda: np.full(n, v, dtype=np.float32).view(np.uint8)


def write_target(path: str, s: TargetShape, seed: int = 0, device: str = "cpu") -> str:
    """Write a target model; returns the file's sha256."""
    g = _Gen(seed, device)
    w = GGUFWriter(path)
    a = "gemma4"
    w.add_str("general.architecture", a)
    w.add_u32("general.alignment", GGUFWriter.ALIGN)
    w.add_u32(f"{a}.block_count", s.n_layer)
    w.add_u32(f"{a}.embedding_length", s.n_embd)
    w.add_u32(f"{a}.attention.head_count", s.n_head)
    w.add_u32(f"{a}.attention.head_count_kv", s.n_head_kv)
    w.add_arr_i32(f"{a}.feed_forward_length", [s.n_ff] * s.n_layer)
    w.add_u32(f"{a}.context_length", s.n_ctx)
    w.add_u32(f"{a}.attention.sliding_window", s.window)
    w.add_u32(f"{a}.embedding_length_per_layer_input", s.ple)
    w.add_f32(f"{a}.attention.layer_norm_rms_epsilon", s.eps)
    w.add_f32(f"{a}.rope.freq_base", s.rope_base)
    w.add_f32(f"{a}.rope.freq_base_swa", s.rope_base_swa)
    w.add_f32(f"{a}.final_logit_softcapping", s.softcap)
    w.add_u32(f"{a}.attention.key_length", s.head_dim_global or s.head_dim)
    w.add_u32(f"{a}.attention.key_length_swa", s.head_dim)
    w.add_u32(f"{a}.attention.shared_kv_layers", s.shared_kv_layers)
    w.add_arr_bool(f"{a}.attention.sliding_window_pattern", [s.is_local(l) for l in range(s.n_layer)])
    w.add_arr_str("tokenizer.ggml.tokens", [f"<{i}>" for i in range(s.n_vocab)])

    def qw(name, k, m, wtype=None):
        wt = s.wtype if wtype is None else wtype
        for suffix, t in s.wtypes.items():
            if name.endswith(suffix):
                wt = t
        if wt in (Q4_K, Q6_K, Q5_K, Q3_K) and k % 256:
            wt = Q4_0                           # super-blocks need k % 256 == 0
        w.declare(name, [k, m], wt, lambda: g.weight(k * m, s.sigma, wt))

    ne, H, Hkv, L = s.n_embd, s.n_head, s.n_head_kv, s.n_layer
    n_own = L - s.shared_kv_layers
    qw("token_embd.weight", ne, s.n_vocab)
    w.declare("output_norm.weight", [ne], F32, _ones(ne))
    if s.rope_freqs:
        hg = s.head_dim_global or s.head_dim
        rf = np.linspace(1.0, 8.0, hg // 2, dtype=np.float32)
        w.declare("rope_freqs.weight", [hg // 2], F32, lambda: rf.view(np.uint8))
    if s.ple:
        # gather-only table: always q4_0 so its row length need not be a multiple of 256
        qw("per_layer_token_embd.weight", s.ple * L, s.n_vocab, Q4_0)
        qw("per_layer_model_proj.weight", ne, s.ple * L)
        w.declare("per_layer_proj_norm.weight", [s.ple], F32, _ones(s.ple))
    for l in range(L):
        p = f"blk.{l}."
        hd = s.hd(l)
        w.declare(p + "attn_norm.weight", [ne], F32, _ones(ne))
        qw(p + "attn_q.weight", ne, H * hd)
        if l < n_own:
            qw(p + "attn_k.weight", ne, Hkv * hd)
            if not s.drop_attn_v:
                qw(p + "attn_v.weight", ne, Hkv * hd)
        qs = 1.0 if s.q_norm_scale is None else s.q_norm_scale * (s.head_dim / hd) ** 0.5   # hd^-0.5 per layer kind
        w.declare(p + "attn_q_norm.weight", [hd], F32, _ones(hd, qs))
        w.declare(p + "attn_k_norm.weight", [hd], F32, _ones(hd))
        qw(p + "attn_output.weight", H * hd, ne)
        w.declare(p + "post_attention_norm.weight", [ne], F32, _ones(ne))
        w.declare(p + "ffn_norm.weight", [ne], F32, _ones(ne))
        qw(p + "ffn_gate.weight", ne, s.n_ff)
        qw(p + "ffn_up.weight", ne, s.n_ff)
        qw(p + "ffn_down.weight", s.n_ff, ne)
        w.declare(p + "post_ffw_norm.weight", [ne], F32, _ones(ne))
        if s.ple:
            qw(p + "inp_gate.weight", ne, s.ple)
            qw(p + "proj.weight", s.ple, ne)
            w.declare(p + "post_norm.weight", [ne], F32, _ones(ne))
        if s.layer_output_scale:
            w.declare(p + "layer_output_scale.weight", [1], F32, _ones(1, 0.5 + 0.25 * (l % 3)))
    return w.write()


def write_head(path: str, h: HeadShape, t: TargetShape, seed: int = 1, device: str = "cpu",
               arch: str = "gemma4-assistant") -> str:
    """Write a draft head matched to target shape `t`; returns the file's sha256."""
    g = _Gen(seed, device)
    w = GGUFWriter(path)
    w.add_str("general.architecture", arch)
    w.add_u32("general.alignment", GGUFWriter.ALIGN)
    w.add_u32(f"{arch}.block_count", h.n_layer)
    w.add_u32(f"{arch}.embedding_length", h.n_inner)
    w.add_u32(f"{arch}.embedding_length_out", t.n_embd)
    w.add_u32(f"{arch}.attention.head_count", h.n_head)
    w.add_u32(f"{arch}.feed_forward_length", h.n_ff)
    w.add_f32(f"{arch}.attention.layer_norm_rms_epsilon", h.eps)
    w.add_f32(f"{arch}.rope.freq_base", t.rope_base)
    w.add_f32(f"{arch}.rope.freq_base_swa", t.rope_base_swa)
    w.add_f32(f"{arch}.final_logit_softcapping", h.softcap)

    def qw(name, k, m):
        wt = Q4_0
        for suffix, t in h.wtypes.items():
            if name.endswith(suffix):
                wt = t
        w.declare(name, [k, m], wt, lambda: g.weight(k * m, h.sigma, wt))

    ni, hd = h.n_inner, t.head_dim
    qw("nextn.pre_projection.weight", 2 * t.n_embd, ni)
    if h.with_post:
        qw("nextn.post_projection.weight", ni, t.n_embd)
    qw("token_embd.weight", ni, t.n_vocab)
    w.declare("output_norm.weight", [ni], F32, _ones(ni))
    for l in range(h.n_layer):
        p = f"blk.{l}."
        for n in ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm"):
            w.declare(p + n + ".weight", [ni], F32, _ones(ni))
        w.declare(p + "attn_q_norm.weight", [hd], F32, _ones(hd))
        qw(p + "attn_q.weight", ni, h.n_head * hd)
        qw(p + "attn_output.weight", h.n_head * hd, ni)
        qw(p + "ffn_gate.weight", ni, h.n_ff)
        qw(p + "ffn_up.weight", ni, h.n_ff)
        qw(p + "ffn_down.weight", h.n_ff, ni)
        if h.layer_output_scale:
            w.declare(p + "layer_output_scale.weight", [1], F32, _ones(1, 0.75))
    return w.write()


def prompt_ids(n: int, n_vocab: int, seed: int = 1) -> np.ndarray:
    """Uniform-random prompt token ids."""
    return np.random.default_rng(seed).integers(0, n_vocab, n).astype(np.int32)


def replay_drafts(greedy: np.ndarray, n_vocab: int, p: float, seed: int = 7) -> np.ndarray:
    """Oracle-replayed drafts: the draft offered for stream index i equals the recorded greedy
    token greedy[i] with probability p, else (greedy[i]+1) mod n_vocab."""
    rng = np.random.default_rng(seed)
    hit = rng.random(len(greedy)) < p
    return np.where(hit, greedy, (greedy + 1) % n_vocab).astype(np.int32)


def cached(path_dir: str, name: str, writer, *args, **kw) -> str:
    """Write `name` under path_dir unless it already exists; returns the path."""
    os.makedirs(path_dir, exist_ok=True)
    path = os.path.join(path_dir, name)
    if not os.path.exists(path):
        tmp = path + ".tmp%d" % os.getpid()
        writer(tmp, *args, **kw)
        os.replace(tmp, path)
    return path
