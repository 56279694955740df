"""GPU parity tests of the individual kernels, called through the C ABI."""
import numpy as np
import pytest

from tests.conftest import model_files, synth_module

pytestmark = pytest.mark.gpu


def _oracle():
    from oracle.pyref import PortOracle
    tp, _ = model_files("tiny")
    return PortOracle(tp, None, 64, False, 4)


# ---- E1: q4 decode is bit-exact ---------------------------------------------------------

def test_dequant_bit_exact_golden(lg, golden):
    s = synth_module()
    a = lg.dequant(s.Q4_0, golden["kat_q4_0_raw"], 1, 2048).reshape(-1)
    b = lg.dequant(s.Q4_K, golden["kat_q4_K_raw"], 1, 2048).reshape(-1)
    assert np.array_equal(a.view(np.uint32), golden["kat_q4_0_out"].view(np.uint32))
    assert np.array_equal(b.view(np.uint32), golden["kat_q4_K_out"].view(np.uint32))


@pytest.mark.parametrize("wtype", ["q4_0", "q4_K"])
def test_dequant_bit_exact_random_blocks(lg, port_built, wtype):
    s = synth_module()
    rng = np.random.default_rng(5)
    o = _oracle()
    if wtype == "q4_0":
        # all byte patterns incl. subnormal / negative / huge f16 scales (inf and nan scales excluded)
        raw = rng.integers(0, 256, size=(4096, 18), dtype=np.uint8)
        raw[:, 1] = np.where((raw[:, 1] & 0x7C) == 0x7C, raw[:, 1] & 0x83, raw[:, 1])
        t, n = s.Q4_0, 4096 * 32
    else:
        raw = rng.integers(0, 256, size=(512, 144), dtype=np.uint8)
        for c in (1, 3):
            raw[:, c] = np.where((raw[:, c] & 0x7C) == 0x7C, raw[:, c] & 0x83, raw[:, c])
        t, n = s.Q4_K, 512 * 256
    want = o.dequant(t, raw.reshape(-1), n)
    o.close()
    got = lg.dequant(t, raw.reshape(-1), 8, n // 8).reshape(-1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# ---- the small-M matmul ------------------------------------------------------------------

def _ref_matvec(w_f32, x):
    return (w_f32.astype(np.float64) @ x.astype(np.float64).T).T


@pytest.mark.parametrize("wtype,m,k", [("q4_0", 256, 256), ("q4_0", 1024, 3840), ("q4_0", 80, 15360),
                                        ("q4_0", 4096, 64), ("q4_K", 512, 1024), ("q4_K", 48, 15360)])
@pytest.mark.parametrize("M", [1, 4, 5, 8])
def test_gemv_matches_oracle(lg, port_built, wtype, m, k, M):
    s = synth_module()
    rng = np.random.default_rng(m + k + M)
    o = _oracle()
    if wtype == "q4_0":
        raw, t = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32) * 0.02), s.Q4_0
    else:
        raw, t = s.random_q4_K(rng, m * k), s.Q4_K
    w = o.dequant(t, raw, m * k).reshape(m, k)
    o.close()
    # heavy-tailed activations: per-group scales must cope with a few large entries
    x = (rng.standard_normal((M, k)) * np.exp(rng.standard_normal((M, k)))).astype(np.float32)
    want = _ref_matvec(w, x)
    got = lg.gemv(t, raw, m, k, x)
    scale = np.abs(want).max()
    err = np.abs(got - want).max() / scale
    assert err < 2e-4, err                     # 16-bit activations: ~1e-5 typical
    # k-sliced partial sums add up to the same thing (within f32 re-association)
    if k >= 512:
        got2 = lg.gemv(t, raw, m, k, x, kslices=2)
        assert np.abs(got2 - want).max() / scale < 2e-4


def _resid_ref(w, act, x, add_w, out_scale, norm_w, eps):
    """f64 statement of the chain: o = W act; x' = (x + rmsnorm(o) add_w) out_scale; y = rmsnorm(x') norm_w."""
    o = act.astype(np.float64) @ w.astype(np.float64).T
    s1 = 1.0 / np.sqrt((o * o).mean(axis=1, keepdims=True) + eps)
    xn = (x.astype(np.float64) + o * s1 * add_w.astype(np.float64)) * out_scale
    if norm_w is None:
        return xn, xn
    s2 = 1.0 / np.sqrt((xn * xn).mean(axis=1, keepdims=True) + eps)
    return xn, xn * s2 * norm_w.astype(np.float64)


@pytest.mark.parametrize("m,k,want_cluster", [(3840, 4096, False), (3840, 15360, True), (2048, 256, None), (2048, 16384, True), (256, 512, None)])
@pytest.mark.parametrize("M", [1, 4, 5, 8])
def test_matmul_with_sums_and_residual_kernel_match_f64(lg, port_built, m, k, want_cluster, M):
    """The o / down / PLE projections of the benchmark shapes through the sums epilogue (k slices reduced inside a cluster
    where the plan has them) and the residual kernel: the new residual row and the next norm's row against f64, with a
    residual stream that carries outliers (the second norm's mean square comes from partial sums, not from a pass over the row)."""
    s = synth_module()
    rng = np.random.default_rng(m + k + M)
    o = _oracle()
    raw = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32) * 0.02)
    w = o.dequant(s.Q4_0, raw, m * k).reshape(m, k)
    o.close()
    act = (rng.standard_normal((M, k)) * np.exp(rng.standard_normal((M, k)))).astype(np.float32)
    x = (rng.standard_normal((M, m)) * np.exp(1.5 * rng.standard_normal((M, m)))).astype(np.float32)
    x[:, 7] *= 300.0                                        # one massive channel, as residual streams have
    add_w = (1.0 + 0.3 * rng.standard_normal(m)).astype(np.float32)
    norm_w = (1.0 + 0.3 * rng.standard_normal(m)).astype(np.float32)
    eps = 1e-6
    for out_scale, nw in ((1.0, norm_w), (0.37, norm_w), (1.0, None)):
        xn, y, used_cluster = lg.matmul_resid(s.Q4_0, raw, m, k, act, x, add_w, out_scale, nw, eps)
        want_x, want_y = _resid_ref(w, act, x, add_w, out_scale, nw, eps)
        if want_cluster is not None:
            assert used_cluster == want_cluster
        ex = np.abs(xn - want_x).max() / np.abs(want_x).max()
        ey = np.abs(y - want_y).max() / np.abs(want_y).max()
        assert ex < 2e-4 and ey < 2e-4, (ex, ey)
        # rows do not depend on the block's width: the row run alone carries the same bits
        if M > 1:
            xa, ya, _ = lg.matmul_resid(s.Q4_0, raw, m, k, act[M - 1:M], x[M - 1:M], add_w, out_scale, nw, eps)
            assert np.array_equal(xa[0].view(np.uint32), xn[M - 1].view(np.uint32))
            assert np.array_equal(ya[0].view(np.uint32), y[M - 1].view(np.uint32))


def test_gemv_column_is_independent_of_block_width(lg):
    """Row j of an M-wide block is bit-identical to the same row run alone (MTP == plain)."""
    s = synth_module()
    rng = np.random.default_rng(3)
    m, k = 512, 3840
    raw = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32) * 0.02)
    x = rng.standard_normal((8, k)).astype(np.float32)
    full = lg.gemv(s.Q4_0, raw, m, k, x)
    for j in (0, 3, 4, 7):
        alone = lg.gemv(s.Q4_0, raw, m, k, x[j:j + 1])
        assert np.array_equal(alone[0].view(np.uint32), full[j].view(np.uint32))
    four = lg.gemv(s.Q4_0, raw, m, k, x[:4])
    assert np.array_equal(four.view(np.uint32), full[:4].view(np.uint32))


def test_gemv_zero_and_ragged(lg):
    s = synth_module()
    rng = np.random.default_rng(9)
    m, k = 40, 128                               # rows not a multiple of 16
    raw = s.quantize_q4_0(rng.standard_normal(m * k).astype(np.float32))
    x = np.zeros((2, k), dtype=np.float32)
    x[1] = rng.standard_normal(k)
    got = lg.gemv(s.Q4_0, raw, m, k, x)
    assert np.all(got[0] == 0)
    want = _ref_matvec(s.dequantize_q4_0(raw).reshape(m, k), x)
    assert np.abs(got - want).max() / np.abs(want).max() < 2e-4


# ---- split-KV flash-decode ---------------------------------------------------------------

def _attn_ref(q, k, v, Hkv, window, pos):
    M, H, hd = q.shape
    seq = k.shape[0]
    k16 = k.astype(np.float16).astype(np.float64); v16 = v.astype(np.float16).astype(np.float64)
    out = np.zeros_like(q, dtype=np.float64)
    for j in range(M):
        p = pos + j
        lo = max(0, p - window + 1) if window > 0 else 0
        rows = [t % seq for t in range(lo, p + 1)]
        for h in range(H):
            c = (h // (H // Hkv)) * hd
            kk, vv = k16[rows, c:c + hd], v16[rows, c:c + hd]
            sc = kk @ q[j, h].astype(np.float64)
            w = np.exp(sc - sc.max()); w /= w.sum()
            out[j, h] = w @ vv
    return out


@pytest.mark.parametrize("H,Hkv,hd", [(4, 1, 64), (8, 2, 256), (16, 8, 256)])
@pytest.mark.parametrize("M,window,seq,pos", [(1, 0, 512, 0), (4, 0, 512, 200), (4, 128, 200, 130), (8, 128, 200, 1000),
                                               (8, 128, 256, 1000), (5, 64, 160, 63), (4, 0, 300, 296)])
@pytest.mark.parametrize("cluster", [False, True])
def test_flash_decode_matches_reference(lg, H, Hkv, hd, M, window, seq, pos, cluster):
    rng = np.random.default_rng(H * hd + M + pos)
    q = (rng.standard_normal((M, H, hd)) * 0.3).astype(np.float32)
    k = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    v = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    want = _attn_ref(q, k, v, Hkv, window, pos)
    if cluster and pos + M > seq and seq % 128:
        pytest.skip("the cluster kernel needs a ring of whole key tiles (the engine allocates such rings)")
    got = lg.flash_decode(q, k, v, Hkv, window, pos, cluster=cluster)
    assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("H,Hkv,hd,M,window,seq,pos", [(16, 8, 256, 4, 1024, 2048, 1500), (16, 8, 256, 4, 0, 2400, 2300),
                                                         (8, 2, 256, 4, 0, 4000, 3990), (16, 8, 256, 4, 1024, 2048, 5000), (8, 2, 256, 8, 512, 1536, 1029),
                                                         (4, 2, 512, 4, 0, 900, 700), (16, 8, 256, 1, 0, 1800, 1799)])
def test_flash_decode_cluster_full_clusters(lg, H, Hkv, hd, M, window, seq, pos):
    """Benchmark-shaped cases: 10 tiles of a 1024-key window in a cluster of 16, head size 512, a 15-tile full-attention row."""
    rng = np.random.default_rng(hd + M + pos)
    q = (rng.standard_normal((M, H, hd)) * 0.3).astype(np.float32)
    k = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    v = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    want = _attn_ref(q, k, v, Hkv, window, pos)
    got = lg.flash_decode(q, k, v, Hkv, window, pos, cluster=True)
    assert np.abs(got - want).max() < 2e-4 * max(1.0, np.abs(want).max())


def test_flash_decode_cluster_refuses_what_does_not_fit(lg):
    rng = np.random.default_rng(5)
    q = np.zeros((1, 4, 64), np.float32); k = np.zeros((9000, 64), np.float32)
    with pytest.raises(ValueError):
        lg.flash_decode(q, k, k, 1, 0, 8900, cluster=True)          # 71 tiles of 128 keys: more than 4 per CTA of a cluster of 16


def test_flash_decode_row_equals_single_query(lg):
    """A query at position p gives bit-identical output as row 2 of a block at p-2 or alone at p."""
    rng = np.random.default_rng(1)
    H, Hkv, hd, seq = 8, 2, 256, 1200
    k = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    v = rng.standard_normal((seq, Hkv * hd)).astype(np.float32)
    q = (rng.standard_normal((4, H, hd)) * 0.3).astype(np.float32)
    for cluster in (False, True):
        for window in (0, 256):
            blk = lg.flash_decode(q, k, v, Hkv, window, 700, cluster=cluster)
            one = lg.flash_decode(q[2:3], k, v, Hkv, window, 702, cluster=cluster)
            assert np.array_equal(blk[2].view(np.uint32), one[0].view(np.uint32))
        # the window's first key crosses a tile boundary between the block's first row and row 2: the block then starts
        # one tile earlier than the single query does, and the row's bits must not notice
        if cluster:
            # full attention over more tiles than the cluster has CTAs: each CTA folds several tiles together
            rng2 = np.random.default_rng(2)
            k2 = rng2.standard_normal((2600, Hkv * hd)).astype(np.float32); v2 = rng2.standard_normal((2600, Hkv * hd)).astype(np.float32)
            blk = lg.flash_decode(q, k2, v2, Hkv, 0, 2300, cluster=True)
            one = lg.flash_decode(q[3:4], k2, v2, Hkv, 0, 2303, cluster=True)  # row 3 sits in the next tile (2303 // 128 = 17, 2300 // 128 = 17)
            assert np.array_equal(blk[3].view(np.uint32), one[0].view(np.uint32))
            blk = lg.flash_decode(q, k2, v2, Hkv, 0, 2302, cluster=True)       # rows 2302, 2303 | 2304, 2305: the block spans a tile border
            one = lg.flash_decode(q[1:2], k2, v2, Hkv, 0, 2303, cluster=True)
            assert np.array_equal(blk[1].view(np.uint32), one[0].view(np.uint32))
        blk = lg.flash_decode(q, k, v, Hkv, 300, 682, cluster=cluster)        # rows at 682..685: windows start at 383..386
        one = lg.flash_decode(q[2:3], k, v, Hkv, 300, 684, cluster=cluster)   # 383 is in tile 2, 385 in tile 3
        assert np.array_equal(blk[2].view(np.uint32), one[0].view(np.uint32))
