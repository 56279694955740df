"""The drop-in claim, checked against the reference's own host code (no GPU needed).

`make -C oracle dropin` links this repository's CUDA backend object with the UNMODIFIED host sources of
cortexist/little-gemma -- the whole CLI (src/run.c + gguf.c quant.c model.c tokenizer.c media.c mtp.c + the media GPU
stub) exactly as its CMakeLists.txt links a backend (CMakeLists.txt:42-45,77-78), LG_MTP_N=3 -- and, for the GPU test,
the reference's host half plus the test shim as a shared object.  A link that succeeds has found every backend symbol
the host imports exactly once and every host symbol the backend imports.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")
_REF_TREE = subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "print-ref"], capture_output=True, text=True).stdout.strip()
HAVE_REFERENCE = bool(_REF_TREE) and os.path.isdir(os.path.join(_REF_TREE, "src"))

BACKEND_SYMBOLS = ["model_kv_host", "kvcache_init", "kvcache_free", "kvcache_save_prefix", "kvcache_restore_prefix",
                   "model_forward", "model_forward_next", "model_prefill", "model_prefill_embd", "model_prefill_mixed",
                   "model_prefill_reserve", "model_forward_spec", "mtp_draft_device", "mtp_draft_chain_device",
                   "mtp_free_device"]


def _defined(path, dynamic):
    out = subprocess.check_output(["nm", "--defined-only"] + (["-D"] if dynamic else []) + [path], text=True)
    return {line.split()[-1] for line in out.splitlines() if line.strip()}


@pytest.fixture(scope="module")
def artefacts():
    if HAVE_REFERENCE:
        subprocess.check_call(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "dropin"])   # up to date: a no-op
    exe, so = os.path.join(REF, "run-b200"), os.path.join(REF, "libref_b200_n4.so")
    if not (os.path.exists(exe) and os.path.exists(so)):
        pytest.skip("the reference tree is not mounted here and no prebuilt drop-in artefacts travelled")
    return exe, so


def test_reference_cli_links_against_this_backend(artefacts):
    exe, _ = artefacts
    syms = _defined(exe, dynamic=False)
    assert "main" in syms and "mtp_open" in syms and "load_gguf" in syms          # the reference's host code is in there
    for s in BACKEND_SYMBOLS:
        assert s in syms, s                                                        # and every backend symbol resolved
    undefined = subprocess.check_output(["nm", "-u", exe], text=True)
    for s in BACKEND_SYMBOLS + ["model_pick", "gguf_find_tensor", "ggml_nbytes"]:
        assert f" {s}\n" not in undefined, s


def test_reference_host_half_links_into_a_shared_object(artefacts):
    _, so = artefacts
    syms = _defined(so, dynamic=True)
    for s in ["ref_open", "ref_generate", "ref_spec", "ref_draft"] + BACKEND_SYMBOLS:
        assert s in syms, s
