"""The allocation-free flash-decode entry point against the regular one and against an f64 reference.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has
already run everything else.  It must pass alone in a fresh process and after the other tests.

Who needs it: callers that may not allocate device memory -- code running inside a stream capture,
a serving loop whose memory layout was fixed at start-up, or a host whose allocator owns the whole
GPU.  They hand over device pointers for inputs and outputs; the kernel's scratch (per-tile partial
results and counters) sits in a 4 MiB array built into the library.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(rng, M, H, Hkv, hd, seq):
    q = (rng.standard_normal((M, H, hd)) * 0.3).astype(np.float32)
    k = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    v = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    return q, k, v


def test_no_alloc_flash_decode_matches_regular_entry_point_twice(lg):
    import torch
    rng = np.random.default_rng(21)
    # two calls in a row with different shapes and positions: the second one meets the first one's
    # leftovers in the shared scratch array
    cases = [(4, 8, 2, 256, 700, 256, 600), (2, 4, 1, 64, 300, 0, 290)]
    for (M, H, Hkv, hd, seq, window, pos) in cases:
        q, k, v = _case(rng, M, H, Hkv, hd, seq)
        want = lg.flash_decode(q, k, v, Hkv, window, pos)            # existing entry point (allocates)
        dq = torch.from_numpy(q).cuda()
        dk = torch.from_numpy(k).cuda().to(torch.float16).contiguous()
        dv = torch.from_numpy(v).cuda().to(torch.float16).contiguous()
        out = torch.zeros((M, H, hd), dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        rc = lg.flash_decode_noalloc(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), M, H, Hkv, hd, seq, window, pos,
                                     out.data_ptr(), 0)
        assert rc == 0
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max())
        # and against plain f64 attention over the f16-rounded cache, so a fault shared by both entry points shows
        from tests.test_gpu_kernels import _attn_ref
        ref = _attn_ref(q, k, v, Hkv, window, pos)
        assert np.abs(got - ref).max() < 2e-4 * max(1.0, np.abs(ref).max())


def test_no_alloc_rejects_oversized_requests(lg):
    import torch
    # 8 rows x 64 heads x 512 dims over a 60,000-position cache cannot fit a 4 MiB scratch
    buf = torch.zeros(16, device="cuda")
    rc = lg.flash_decode_noalloc(buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), 8, 64, 64, 512, 60000, 0, 59000,
                                 buf.data_ptr(), 0)
    assert rc == -4
    assert lg.flash_decode_noalloc(0, 0, 0, 1, 1, 1, 64, 16, 0, 0, 0, 0) == -1


def test_no_alloc_rejects_misaligned_pointers_without_launching(lg):
    import torch
    # K / V rows are fetched 16 bytes at a time: a view that starts at an odd element must be turned away on the host
    q = torch.zeros((1, 1, 64), dtype=torch.float32, device="cuda")
    kv = torch.zeros(16 * 64 + 8, dtype=torch.float16, device="cuda")
    out = torch.zeros((1, 1, 64), dtype=torch.float32, device="cuda")
    ok = lg.flash_decode_noalloc(q.data_ptr(), kv.data_ptr(), kv.data_ptr(), 1, 1, 1, 64, 16, 0, 3, out.data_ptr(), 0)
    assert ok == 0
    torch.cuda.synchronize()
    off = kv[1:].data_ptr()                              # 2 bytes into the buffer
    assert lg.flash_decode_noalloc(q.data_ptr(), off, kv.data_ptr(), 1, 1, 1, 64, 16, 0, 3, out.data_ptr(), 0) == -1
    assert lg.flash_decode_noalloc(q.data_ptr(), kv.data_ptr(), off, 1, 1, 1, 64, 16, 0, 3, out.data_ptr(), 0) == -1
    assert lg.flash_decode_noalloc(q.data_ptr() + 2, kv.data_ptr(), kv.data_ptr(), 1, 1, 1, 64, 16, 0, 3, out.data_ptr(), 0) == -1
    torch.cuda.synchronize()
