"""ctypes binding of liblg_b200.so -- the sm_100a backend of the little-gemma speculative-decode
step.  The library is the product; this module only loads it and exposes a `Session` whose
methods map one-to-one onto the C model API (model_forward, model_forward_next, model_prefill,
model_forward_spec, mtp_draft, ...).

There is no CPU path: importing works without a GPU (so symbols can be inspected), but every
compute call needs the CUDA library and a B200.  A missing library raises immediately.

The directory name has a hyphen: import it with
    importlib.import_module("little-gemma_b200")
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblg_b200.so")

_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")

# every symbol include/lg_b200.h declares
ABI_SYMBOLS = [
    "model_kv_host", "kvcache_init", "kvcache_free", "kvcache_save_prefix", "kvcache_restore_prefix",
    "model_forward", "model_forward_next", "model_prefill", "model_prefill_embd", "model_prefill_mixed",
    "model_prefill_reserve", "model_forward_spec", "mtp_draft_device", "mtp_draft_chain_device", "mtp_free_device",
    "lg_forward_spec_n", "lg_set_replay", "lg_rounds_begin", "lg_rounds_enqueue", "lg_rounds_collect",
    "lg_set_round_width", "lg_set_replay_origin", "lg_host_syncs", "lg_set_draft_margin", "lg_drafts_skipped", "lg_weight_bytes", "lg_round_launches", "lg_last_hidden", "lg_kv_row", "lg_stream", "lg_engine_release",
    "lg_bench_matmul_pass", "lg_bench_prefill_pass", "lg_set_attn_deep", "lg_flash_decode_noalloc",
    "lg_debug_bounded_wait", "lg_debug_stamps", "lg_debug_clear_stamps", "lg_matmul_resid_host",
    "lg_dequant_host", "lg_gemv_host", "lg_flash_decode_host", "lg_flash_decode_cluster_host", "lg_prefill_matmul_host",
]

_lib = None


def load() -> C.CDLL:
    """Load liblg_b200.so (built by build.py); raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `python little-gemma_b200/build.py` (needs nvcc). "
                          "There is no fallback path.")
    L = C.CDLL(LIB_PATH)
    L.lgs_open.restype = C.c_void_p
    L.lgs_open.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int]
    L.lgs_close.argtypes = [C.c_void_p]
    for n in ("lgs_n_vocab", "lgs_n_embd", "lgs_n_layer", "lgs_has_head"):
        getattr(L, n).argtypes = [C.c_void_p]; getattr(L, n).restype = C.c_int
    for n in ("lgs_model", "lgs_kv", "lgs_head"):
        getattr(L, n).argtypes = [C.c_void_p]; getattr(L, n).restype = C.c_void_p
    L.lgs_set_mtp_n.argtypes = [C.c_void_p, C.c_int]
    L.lgs_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.lgs_last_hidden.argtypes = [C.c_void_p, _f32p]
    L.lgs_next.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lgs_next.restype = C.c_int
    L.lgs_prefill.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int]
    L.lgs_prefill_mixed.argtypes = [C.c_void_p, _f32p, _i32p, C.c_int, C.c_int]
    L.lgs_prefill_embd.argtypes = [C.c_void_p, _f32p, C.c_int, C.c_int]
    L.lgs_spec.argtypes = [C.c_void_p, _i32p, C.c_int, _i32p]; L.lgs_spec.restype = C.c_int
    L.lgs_draft.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lgs_draft.restype = C.c_int
    L.lgs_draft_chain.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lgs_draft_chain.restype = C.c_int
    L.lgs_kv_row.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]; L.lgs_kv_row.restype = C.c_int
    L.lgs_generate.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, _i32p, C.c_int, C.c_void_p, C.c_int, _i32p]
    L.lgs_generate.restype = C.c_int
    L.lgs_generate_device.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, _i32p, C.c_int, C.c_void_p, C.c_int, _i32p]
    L.lgs_generate_device.restype = C.c_int
    L.lg_dequant_host.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p]; L.lg_dequant_host.restype = C.c_int
    L.lg_gemv_host.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int, _f32p]
    L.lg_gemv_host.restype = C.c_int
    L.lg_matmul_resid_host.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p, _f32p, C.c_float, C.c_void_p, C.c_float, _f32p]
    L.lg_matmul_resid_host.restype = C.c_int
    L.lg_prefill_matmul_host.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
    L.lg_prefill_matmul_host.restype = C.c_int
    L.lg_flash_decode_host.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_int, _f32p]
    L.lg_flash_decode_host.restype = C.c_int
    L.lg_flash_decode_cluster_host.argtypes = L.lg_flash_decode_host.argtypes
    L.lg_flash_decode_cluster_host.restype = C.c_int
    L.lg_flash_decode_noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.lg_flash_decode_noalloc.restype = C.c_int
    L.lg_set_replay.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    L.lg_rounds_begin.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    L.lg_rounds_enqueue.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    L.lg_rounds_enqueue.restype = C.c_int
    L.lg_rounds_collect.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, _i32p]
    L.lg_rounds_collect.restype = C.c_int
    L.lg_weight_bytes.argtypes = [C.c_void_p]; L.lg_weight_bytes.restype = C.c_longlong
    L.lg_round_launches.argtypes = [C.c_void_p]; L.lg_round_launches.restype = C.c_longlong
    L.lg_stream.argtypes = [C.c_void_p]; L.lg_stream.restype = C.c_void_p
    L.lg_bench_matmul_pass.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lg_bench_matmul_pass.restype = C.c_int
    L.lg_set_attn_deep.argtypes = [C.c_int, C.c_int]; L.lg_set_attn_deep.restype = None
    L.lg_bench_prefill_pass.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lg_bench_prefill_pass.restype = C.c_int
    L.lgs_rounds_host.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _i32p, C.c_int, C.c_void_p, C.c_int, _i32p]
    L.lgs_rounds_host.restype = C.c_int
    L.lg_set_draft_margin.argtypes = [C.c_void_p, C.c_float]; L.lg_set_draft_margin.restype = None
    L.lg_drafts_skipped.argtypes = [C.c_void_p]; L.lg_drafts_skipped.restype = C.c_longlong
    L.lg_debug_bounded_wait.argtypes = [C.c_void_p, C.c_int]; L.lg_debug_bounded_wait.restype = C.c_int
    L.lgs_host_syncs.argtypes = [C.c_void_p]; L.lgs_host_syncs.restype = C.c_longlong
    L.lg_set_round_width.argtypes = [C.c_int]; L.lg_set_round_width.restype = None
    L.lg_set_replay_origin.argtypes = [C.c_void_p, C.c_int, C.c_int]; L.lg_set_replay_origin.restype = None
    _lib = L
    return L


def dequant(ggml_type: int, raw: np.ndarray, n_rows: int, k: int) -> np.ndarray:
    """Decode file-format blocks on the GPU (bit-exact to the reference decode)."""
    L = load()
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.empty((n_rows, k), dtype=np.float32)
    rc = L.lg_dequant_host(ggml_type, raw.ctypes.data_as(C.c_void_p), n_rows, k, out.reshape(-1))
    if rc:
        raise ValueError(f"lg_dequant_host failed ({rc})")
    return out


def gemv(ggml_type: int, raw: np.ndarray, m: int, k: int, x: np.ndarray, kslices: int = 0) -> np.ndarray:
    """y[tok] = W x[tok] through the production matmul kernel; x is [M, k] f32, M <= 8."""
    L = load()
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    M = x.shape[0]
    y = np.empty((M, m), dtype=np.float32)
    rc = L.lg_gemv_host(ggml_type, raw.ctypes.data_as(C.c_void_p), m, k, x.reshape(-1), M, kslices, y.reshape(-1))
    if rc:
        raise ValueError(f"lg_gemv_host failed ({rc})")
    return y


def matmul_resid(ggml_type: int, raw: np.ndarray, m: int, k: int, act: np.ndarray, xres: np.ndarray, add_w: np.ndarray,
                 out_scale: float, norm_w, eps: float):
    """The decode step's chain o = W act; x' = (x + rmsnorm(o) add_w) out_scale; y = rmsnorm(x') norm_w (norm_w None: y = x')
    through the production kernels (matmul with complete rows + norm sums, residual kernel).  Returns (x', y, cluster_used)."""
    L = load()
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    act = np.ascontiguousarray(act, dtype=np.float32)
    x = np.array(xres, dtype=np.float32, order="C", copy=True)
    aw = np.ascontiguousarray(add_w, dtype=np.float32)
    nw = None if norm_w is None else np.ascontiguousarray(norm_w, dtype=np.float32)
    M = act.shape[0]
    y = np.empty((M, m), dtype=np.float32)
    rc = L.lg_matmul_resid_host(ggml_type, raw.ctypes.data_as(C.c_void_p), m, k, act.reshape(-1), M, x.reshape(-1), aw, out_scale,
                                None if nw is None else nw.ctypes.data_as(C.c_void_p), eps, y.reshape(-1))
    if rc < 0:
        raise ValueError(f"lg_matmul_resid_host failed ({rc})")
    return x, y, bool(rc)


def prefill_matmul(ggml_type: int, raw: np.ndarray, m: int, k: int, x: np.ndarray, raw_up: np.ndarray = None) -> np.ndarray:
    """y[tok] = W x[tok] for up to 256 rows of x at once through the wide tcgen05 matmul (x rounded to f16).
    With raw_up, raw/raw_up are a gate/up pair and y = gelu_tanh(gate x) * (up x), rounded to f16."""
    L = load()
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[0]
    y = np.empty((n, m), dtype=np.float32)
    up = None
    if raw_up is not None:
        raw_up = np.ascontiguousarray(raw_up, dtype=np.uint8)
        up = raw_up.ctypes.data_as(C.c_void_p)
    rc = L.lg_prefill_matmul_host(ggml_type, raw.ctypes.data_as(C.c_void_p), up, m, k, x.reshape(-1), n, y.reshape(-1))
    if rc:
        raise ValueError(f"lg_prefill_matmul_host failed ({rc})")
    return y


def set_attn_deep(min_seq: int = 4096, force_g: int = 0) -> None:
    """Caches of at least min_seq rows use the span attention kernel on full-attention layers (force_g > 0 fixes the
    tiles per span).  Call before opening the Session it should apply to."""
    load().lg_set_attn_deep(min_seq, force_g)


def flash_decode(q: np.ndarray, k: np.ndarray, v: np.ndarray, n_head_kv: int, window: int, pos: int,
                 cluster: bool = False) -> np.ndarray:
    """q [M, H, hd]; k, v [seq, Hkv*hd] (rounded to f16 on upload); query j sits at pos + j.
    cluster=True runs the cluster-merged kernel (raises if the case has more key tiles than a cluster holds)."""
    L = load()
    q = np.ascontiguousarray(q, dtype=np.float32); k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    M, H, hd = q.shape
    out = np.empty_like(q)
    fn = L.lg_flash_decode_cluster_host if cluster else L.lg_flash_decode_host
    rc = fn(q.reshape(-1), k.reshape(-1), v.reshape(-1), M, H, n_head_kv, hd, k.shape[0], window, pos, out.reshape(-1))
    if rc:
        raise ValueError(f"lg_flash_decode_host failed ({rc})")
    return out


def flash_decode_noalloc(d_q: int, d_k: int, d_v: int, M: int, H: int, n_head_kv: int, hd: int, seq: int, window: int,
                         pos: int, d_out: int, stream: int = 0) -> int:
    """The allocation-free flash-decode entry point: every argument named d_* is a raw device address
    (q f32 [M,H,hd]; k, v f16 [seq, Hkv*hd]; out f32 [M,H,hd]).  Enqueues on `stream` and returns the
    library's status code (0 = launched)."""
    return int(load().lg_flash_decode_noalloc(d_q, d_k, d_v, M, H, n_head_kv, hd, seq, window, pos, d_out, stream))


class Session:
    """One loaded target model (+ optional draft head) with its KV cache on the GPU."""

    def __init__(self, target: str, head: str | None = None, max_seq: int = 4096, mtp_n: int = 4):
        self.L = load()
        self.h = self.L.lgs_open(target.encode(), (head or "").encode(), max_seq, 1)
        if not self.h:
            raise RuntimeError(f"cannot open {target}")
        self.n_vocab = self.L.lgs_n_vocab(self.h)
        self.n_embd = self.L.lgs_n_embd(self.h)
        self.n_layer = self.L.lgs_n_layer(self.h)
        self.mtp_n = mtp_n
        self.L.lgs_set_mtp_n(self.h, mtp_n)
        self.model = self.L.lgs_model(self.h)
        self.kv = self.L.lgs_kv(self.h)
        self.head = self.L.lgs_head(self.h)

    def close(self):
        if self.h:
            self.L.lgs_close(self.h)
            self.h = None

    def __enter__(self): return self
    def __exit__(self, *a): self.close()

    def forward(self, tok: int, pos: int, want_logits: bool = True):
        if not want_logits:
            self.L.lgs_forward(self.h, tok, pos, None)
            return None
        out = np.empty(self.n_vocab, dtype=np.float32)
        self.L.lgs_forward(self.h, tok, pos, out.ctypes.data_as(C.c_void_p))
        return out

    def last_hidden(self) -> np.ndarray:
        out = np.empty(self.n_embd, dtype=np.float32)
        self.L.lgs_last_hidden(self.h, out)
        return out

    def next(self, tok: int, pos: int) -> int:
        return self.L.lgs_next(self.h, tok, pos)

    def prefill(self, toks, pos0: int = 0):
        toks = np.ascontiguousarray(toks, dtype=np.int32)
        self.L.lgs_prefill(self.h, toks, len(toks), pos0)

    def prefill_mixed(self, rows, ids, pos0: int = 0):
        """model_prefill_mixed: ids[i] >= 0 is a token id, ids[i] < 0 names embedding row -ids[i]-1 of `rows` [n_rows, n_embd]."""
        rows = np.ascontiguousarray(rows, dtype=np.float32).reshape(-1)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        self.L.lgs_prefill_mixed(self.h, rows, ids, len(ids), pos0)

    def prefill_embd(self, rows, pos0: int = 0):
        """model_prefill_embd: every position is an embedding row."""
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        self.L.lgs_prefill_embd(self.h, rows.reshape(-1), rows.shape[0], pos0)

    def spec(self, toks, pos: int):
        toks = np.ascontiguousarray(toks, dtype=np.int32)
        assert len(toks) == self.mtp_n
        out = np.zeros(8, dtype=np.int32)
        adv = self.L.lgs_spec(self.h, toks, pos, out)
        return adv, out[:self.mtp_n]

    def draft(self, tok: int, pos: int) -> int:
        return self.L.lgs_draft(self.h, tok, pos)

    def draft_chain(self, tok: int, pos: int) -> int:
        return self.L.lgs_draft_chain(self.h, tok, pos)

    def kv_row(self, layer: int, pos: int, kv_dim: int):
        k = np.empty(kv_dim, dtype=np.float32); v = np.empty(kv_dim, dtype=np.float32)
        d = self.L.lgs_kv_row(self.h, layer, pos, k, v)
        return (k[:d], v[:d]) if d else (None, None)

    def generate(self, prompt, n_gen: int, mode: int = 0, replay=None):
        """Host-driven generation through the reference-shaped blocking calls."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(n_gen + 8, dtype=np.int32); stats = np.zeros(2, dtype=np.int32)
        rp, nr = None, 0
        if replay is not None:
            replay = np.ascontiguousarray(replay, dtype=np.int32)
            rp, nr = replay.ctypes.data_as(C.c_void_p), len(replay)
        n = self.L.lgs_generate(self.h, prompt, len(prompt), n_gen, out, mode, rp, nr, stats)
        return out[:n], (int(stats[0]), int(stats[1]))

    def generate_device(self, prompt, n_gen: int, mode: int = 0, replay=None):
        """Device-resident rounds: one host synchronisation for the whole generation."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(n_gen + 8, dtype=np.int32); stats = np.zeros(2, dtype=np.int32)
        rp, nr = None, 0
        if replay is not None:
            replay = np.ascontiguousarray(np.concatenate([replay, np.zeros(8, np.int32)]), dtype=np.int32)
            rp, nr = replay.ctypes.data_as(C.c_void_p), len(replay)
        n = self.L.lgs_generate_device(self.h, prompt, len(prompt), n_gen, out, mode, rp, nr, stats)
        if n < 0:
            raise RuntimeError("device rounds unavailable (no draft head?)")
        return out[:n], (int(stats[0]), int(stats[1]))

    def rounds_host(self, best: int, pos: int, n_emitted: int, n_gen: int, n_rounds: int, mode: int, replay=None):
        """Host-driven rounds from a given state; returns (tokens[n_emitted:], stats dict)."""
        out = np.zeros(n_gen + 8, dtype=np.int32); stats = np.zeros(4, dtype=np.int32)
        rp, nr = None, 0
        if replay is not None:
            replay = np.ascontiguousarray(replay, dtype=np.int32)
            rp, nr = replay.ctypes.data_as(C.c_void_p), len(replay)
        g = self.L.lgs_rounds_host(self.h, best, pos, n_emitted, n_gen, n_rounds, out, mode, rp, nr, stats)
        return out[n_emitted:g], dict(n_draft=int(stats[0]), n_accept=int(stats[1]), pos=int(stats[2]), best=int(stats[3]))

    def matmul_pass(self, n: int, classes: int = 0) -> int:
        """Enqueue the weight matmuls of one verify step (classes: 1 qkv, 2 o, 4 gate/up, 8 down, 16 head, 32 PLE)."""
        return int(self.L.lg_bench_matmul_pass(self.model, n, classes))

    def prefill_pass(self, n: int, classes: int = 0) -> int:
        """Enqueue the kernels of one wide prompt block of n tokens (classes as in matmul_pass; default the matmuls)."""
        return int(self.L.lg_bench_prefill_pass(self.model, n, classes))

    # device-resident rounds, raw
    def rounds_begin(self, first: int, pos: int, n_emitted: int = 1):
        self.L.lg_rounds_begin(self.model, first, pos, n_emitted)

    def set_replay(self, replay):
        replay = np.ascontiguousarray(replay, dtype=np.int32)
        self.L.lg_set_replay(self.model, replay.ctypes.data_as(C.c_void_p), len(replay))

    def rounds_enqueue(self, n: int, mode: int, n_rounds: int, use_head: bool = True) -> int:
        return self.L.lg_rounds_enqueue(self.model, self.kv, self.head if use_head else None, n, mode, n_rounds)

    def rounds_collect(self, from_: int = 1, cap: int = 0):
        stats = np.zeros(4, dtype=np.int32)
        toks = np.zeros(max(cap, 1), dtype=np.int32)
        n = self.L.lg_rounds_collect(self.model, toks.ctypes.data_as(C.c_void_p), from_, cap, stats)
        return toks[:n], dict(pos=int(stats[0]), n_emitted=int(stats[1]), n_draft=int(stats[2]), n_accept=int(stats[3]))

    def set_draft_margin(self, margin: float) -> None:
        """Call off a round's remaining drafts when a draft's best logit leads the runner-up by less than `margin` (0 = off)."""
        self.L.lg_set_draft_margin(self.model, float(margin))

    def drafts_skipped(self) -> int:
        return int(self.L.lg_drafts_skipped(self.model))

    def host_syncs(self) -> int:
        """Blocking device-to-host waits the reference-shaped calls of this session have made so far."""
        return int(self.L.lgs_host_syncs(self.h))

    def weight_bytes(self) -> int:
        return int(self.L.lg_weight_bytes(self.model))

    def round_launches(self) -> int:
        return int(self.L.lg_round_launches(self.model))

    def stream(self) -> int:
        return int(self.L.lg_stream(self.model) or 0)
