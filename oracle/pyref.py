"""ctypes faces of the two CPU checkers. TEST INFRASTRUCTURE ONLY.

`RefOracle`  -- oracle/_ref/libref_cpu_n<N>.so: the unmodified reference CPU backend
                (built by `make -C oracle ref` where the reference tree is mounted).
`PortOracle` -- oracle/liblg_oracle.so: this repository's own C restatement.
Both expose the same methods so tests can run either against the CUDA backend.
"""
from __future__ import annotations

import ctypes as C
import os
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def ref_lib_path(n: int) -> str:
    return os.path.join(HERE, "_ref", f"libref_cpu_n{n}.so")


def port_lib_path() -> str:
    return os.path.join(HERE, "liblg_oracle.so")


class _Oracle:
    prefix = ""
    fresh_copy = False

    def __init__(self, lib_path: str, target: str, head: str | None, max_seq: int, kv_f16_all: bool):
        if not os.path.exists(lib_path):
            raise FileNotFoundError(lib_path)
        if self.fresh_copy:
            # The reference keeps per-process statics sized by the first model it sees (its greedy
            # pick buffer, src/cpu/model-cpu.c:466-470), so every session gets its own image.
            import shutil, tempfile
            fd, tmp = tempfile.mkstemp(suffix=".so", prefix="libref_")
            os.close(fd)
            shutil.copyfile(lib_path, tmp)
            self.lib = L = C.CDLL(tmp)
            os.unlink(tmp)
        else:
            self.lib = L = C.CDLL(lib_path)
        p = self.prefix
        f = lambda name: getattr(L, p + name)
        f("open").restype = C.c_void_p
        f("open").argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int]
        f("close").argtypes = [C.c_void_p]
        for n in ("n_vocab", "n_embd", "has_head"):
            f(n).argtypes = [C.c_void_p]; f(n).restype = C.c_int
        f("forward").argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p]; f("forward").restype = None
        f("last_hidden").argtypes = [C.c_void_p, _f32p]; f("last_hidden").restype = None
        f("next").argtypes = [C.c_void_p, C.c_int, C.c_int]; f("next").restype = C.c_int
        f("prefill").argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int]; f("prefill").restype = None
        f("prefill_mixed").argtypes = [C.c_void_p, _f32p, _i32p, C.c_int, C.c_int]; f("prefill_mixed").restype = None
        f("spec").argtypes = [C.c_void_p, _i32p, C.c_int, _i32p]; f("spec").restype = C.c_int
        f("draft").argtypes = [C.c_void_p, C.c_int, C.c_int]; f("draft").restype = C.c_int
        f("kv_row").argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, _f32p]; f("kv_row").restype = C.c_int
        f("dequant").argtypes = [C.c_uint, C.c_void_p, _f32p, C.c_longlong]; f("dequant").restype = C.c_int
        f("generate").argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, _i32p, C.c_int, C.c_void_p, _i32p]
        f("generate").restype = C.c_int
        f("mtp_n").restype = C.c_int
        f("set_threads").argtypes = [C.c_int]; f("set_threads").restype = C.c_int
        self._f = f
        self.h = f("open")(target.encode(), (head or "").encode(), max_seq, int(kv_f16_all))
        if not self.h:
            raise RuntimeError(f"oracle could not open {target}")
        self.n_vocab = f("n_vocab")(self.h)
        self.n_embd = f("n_embd")(self.h)
        self.mtp_n = f("mtp_n")()

    def close(self):
        if self.h:
            self._f("close")(self.h)
            self.h = None

    def set_threads(self, n: int) -> int:
        """Ask the checker's OpenMP runtime for n threads (0: leave as is); returns the count it will use."""
        return int(self._f("set_threads")(n))

    def forward(self, tok: int, pos: int) -> np.ndarray:
        out = np.empty(self.n_vocab, dtype=np.float32)
        self._f("forward")(self.h, tok, pos, out)
        return out

    def last_hidden(self) -> np.ndarray:
        out = np.empty(self.n_embd, dtype=np.float32)
        self._f("last_hidden")(self.h, out)
        return out

    def next(self, tok: int, pos: int) -> int:
        return self._f("next")(self.h, tok, pos)

    def prefill(self, toks, pos0: int = 0):
        toks = np.ascontiguousarray(toks, dtype=np.int32)
        self._f("prefill")(self.h, toks, len(toks), pos0)

    def prefill_mixed(self, rows, ids, pos0: int = 0):
        """ids[i] >= 0: token id; ids[i] < 0: embedding row -ids[i]-1 of `rows` [n_rows, n_embd] (a media position)."""
        rows = np.ascontiguousarray(rows, dtype=np.float32).reshape(-1)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        self._f("prefill_mixed")(self.h, rows, ids, len(ids), pos0)

    def spec(self, toks, pos: int):
        toks = np.ascontiguousarray(toks, dtype=np.int32)
        assert len(toks) == self.mtp_n
        out = np.zeros(self.mtp_n, dtype=np.int32)
        adv = self._f("spec")(self.h, toks, pos, out)
        return adv, out

    def draft(self, tok: int, pos: int) -> int:
        return self._f("draft")(self.h, tok, pos)

    def kv_row(self, layer: int, pos: int, kv_dim: int):
        k = np.empty(kv_dim, dtype=np.float32); v = np.empty(kv_dim, dtype=np.float32)
        d = self._f("kv_row")(self.h, layer, pos, k, v)
        return (k[:d], v[:d]) if d else (None, None)

    def dequant(self, ggml_type: int, raw: np.ndarray, n: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        rc = self._f("dequant")(ggml_type, raw.ctypes.data_as(C.c_void_p), out, n)
        if rc != 0:
            raise ValueError("unsupported type")
        return out

    def generate(self, prompt, n_gen: int, mode: int = 0, replay=None):
        """mode 0 plain, 1 MTP with the loaded head, 2 MTP with replayed drafts."""
        prompt = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.zeros(n_gen, dtype=np.int32)
        stats = np.zeros(2, dtype=np.int32)
        rp = None
        if replay is not None:
            replay = np.ascontiguousarray(np.concatenate([replay, np.zeros(self.mtp_n, np.int32)]), dtype=np.int32)
            rp = replay.ctypes.data_as(C.c_void_p)
        n = self._f("generate")(self.h, prompt, len(prompt), n_gen, out, mode, rp, stats)
        return out[:n], (int(stats[0]), int(stats[1]))


class RefOracle(_Oracle):
    prefix = "ref_"
    fresh_copy = True

    def __init__(self, target, head=None, max_seq=4096, kv_f16_all=False, mtp_n=4):
        super().__init__(ref_lib_path(mtp_n), target, head, max_seq, kv_f16_all)


class PortOracle(_Oracle):
    prefix = "orc_"

    def __init__(self, target, head=None, max_seq=4096, kv_f16_all=False, mtp_n=4):
        super().__init__(port_lib_path(), target, head, max_seq, kv_f16_all)
        self.lib.orc_set_mtp_n.argtypes = [C.c_void_p, C.c_int]
        self.lib.orc_set_mtp_n(self.h, mtp_n)
        self.mtp_n = mtp_n
