"""FLASH_ATTN_EXT on the GPU vs the CPU oracle, through the C ABI (-m gpu).

Tolerance asked of F16-KV attention: 1e-3 relative per output element.  The decode-shaped
kernels reproduce the CPU arithmetic (exact score dots, the f16 accumulator's rounding order,
the host libm's expf), so the comparison below is made bit for bit wherever no softcap / ALiBi
function (tanhf, powf) is involved, and at 1e-3 otherwise.
"""
import numpy as np
import pytest

import b200
import orc
from conftest import bits_equal
from test_oracle_flash_attn import case_names, load_case

pytestmark = pytest.mark.gpu
REL_TOL = 1e-3


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


def rel_err(got, want):
    return np.abs(got - want) / np.maximum(np.abs(want), 1e-30)


def synth_case(H, Hkv, D, T, n_kv, seed, causal=True):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((H, T, D)).astype(np.float32)
    k = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    v = rng.standard_normal((Hkv, n_kv, D)).astype(np.float16).view(np.uint16)
    mask = None
    if causal:
        # row t sees positions <= t + (n_kv - T); f16 0 / -inf like the reference's kq_mask
        off = n_kv - T
        m = np.where(np.arange(n_kv)[None, :] <= np.arange(T)[:, None] + off, 0.0, -np.inf).astype(np.float16)
        mask = m.view(np.uint16)
    return q, k, v, mask


def test_reference_dump_cases_below_64_rows(dev, golden):
    """The one_chunk cases of the reference's dump, sinks and the GQA decode shape included."""
    g = golden("flash_attn")
    seen = 0
    for c in case_names(g):
        d = load_case(g, c)
        if d["T"] >= 64 or d["q"].shape[2] not in (64, 128) or d["v"].shape[2] not in (64, 128):
            continue
        kv = dev.KvCacheView(d["k"], d["v"])
        got = dev.flash_attn(d["q"], kv, d["mask"], d["scale"], sinks=d["sinks"], max_bias=d["max_bias"],
                             softcap=d["softcap"])
        assert bits_equal(got, d["dst"]), c
        seen += 1
    assert seen >= 2


def test_split_kv_probe(dev, golden):
    """The reference's own 1-row runs over 600 positions, 1 and 8 threads (chunks)."""
    g = golden("flash_attn_probe")
    checked = 0
    for p in sorted({k.split("/")[0] for k in g.files}):
        dk, dv, h, hkv, t, skv = (int(x) for x in g[p + "/geom"])
        scale = float(g[p + "/knobs"][0])
        q = g[p + "/q"].reshape(h, t, dk)
        kv = dev.KvCacheView(g[p + "/k"].reshape(hkv, skv, dk), g[p + "/v"].reshape(hkv, skv, dv))
        mask = g[p + "/mask"].reshape(t, skv)
        for r in sorted(x for x in g.files if x.startswith(p + "/rec/")):
            tag, tt, nth = (int(x) for x in r.split("/")[2:])
            if tag == 1:
                got = dev.flash_attn(q[:, tt:tt + 1], kv, mask[tt:tt + 1], scale, n_chunks=nth)
            elif tag == 0:
                got = dev.flash_attn(q, kv, mask, scale, n_chunks=nth)
            else:
                got = dev.flash_attn(q[:, 1:], kv, mask[1:], scale)
            assert bits_equal(got.ravel(), g[r]), r
            checked += 1
    assert checked == 16


@pytest.mark.parametrize("n_kv", [512, 4096, 32768])
@pytest.mark.parametrize("n_chunks", [8, 16])
def test_decode_gqa_head_dim_128(dev, n_kv, n_chunks):
    """BASELINE shape: D 128, 32 query heads over 8 KV heads, one query row, causal mask."""
    q, k, v, mask = synth_case(32, 8, 128, 1, n_kv, seed=n_kv)
    want, path = orc.flash_attn(q, k, v, mask, 1.0 / np.sqrt(128.0), n_chunks=n_chunks)
    assert path == orc.FA_SPLIT_KV
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 1.0 / np.sqrt(128.0), n_chunks=n_chunks)
    assert rel_err(got, want).max() <= REL_TOL
    assert bits_equal(got, want)


@pytest.mark.parametrize("shape", [(5, 300), (16, 1024), (63, 200), (1, 511), (2, 700)], ids=str)
def test_one_chunk_rows(dev, shape):
    """Fewer than 64 query rows that do not qualify for split-KV: whole-range scan per row."""
    T, n_kv = shape
    q, k, v, mask = synth_case(8, 2, 128, T, n_kv, seed=T * 1000 + n_kv)
    want, path = orc.flash_attn(q, k, v, mask, 0.0883883)
    assert path == orc.FA_ONE_CHUNK
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 0.0883883)
    assert bits_equal(got, want)


def test_fully_masked_rows_and_padded_cache(dev):
    """Positions past the used cells are masked -inf (the cache pads n_kv to 256); a row whose
    mask is all -inf gives zeros."""
    q, k, v, _ = synth_case(4, 2, 64, 3, 256, seed=5, causal=False)
    m = np.full((3, 256), -np.inf, dtype=np.float16)
    m[0, :10] = 0.0
    m[1, :200] = 0.0
    mask = m.view(np.uint16)
    want, _ = orc.flash_attn(q, k, v, mask, 0.125)
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 0.125)
    assert bits_equal(got, want)
    assert not got[2].any()


def test_reference_dump_cases_tiled(dev, golden):
    """The 64-row-or-more cases of the reference's dump: plain, ragged KV tail, DV != DK, no mask,
    sinks (bit-exact); softcap and ALiBi go through tanhf / powf and are held to the tolerance."""
    g = golden("flash_attn")
    seen = 0
    for c in case_names(g):
        d = load_case(g, c)
        if d["T"] < 64 or d["q"].shape[2] not in (64, 128) or d["v"].shape[2] not in (64, 128):
            continue
        kv = dev.KvCacheView(d["k"], d["v"])
        got = dev.flash_attn(d["q"], kv, d["mask"], d["scale"], sinks=d["sinks"], max_bias=d["max_bias"],
                             softcap=d["softcap"])
        if d["softcap"] == 0.0 and d["max_bias"] == 0.0:
            assert bits_equal(got, d["dst"]), c
        else:
            scale = np.abs(d["dst"]).max(axis=-1, keepdims=True)
            assert (np.abs(got - d["dst"]) <= REL_TOL * scale).all(), c
        seen += 1
    assert seen >= 8


@pytest.mark.parametrize("shape", [(512, 512), (512, 4096), (100, 300), (64, 64)], ids=str)
def test_prefill_gqa_head_dim_128(dev, shape):
    """BASELINE shape (D 128, 32 heads over 8 KV heads, causal) through the tiled path."""
    T, n_kv = shape
    q, k, v, mask = synth_case(32, 8, 128, T, n_kv, seed=T + n_kv)
    want, path = orc.flash_attn(q, k, v, mask, 1.0 / np.sqrt(128.0))
    assert path == orc.FA_TILED
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 1.0 / np.sqrt(128.0))
    assert rel_err(got, want).max() <= REL_TOL
    assert bits_equal(got, want)


def test_softcap_and_sinks_within_tolerance(dev):
    q, k, v, mask = synth_case(8, 2, 64, 4, 333, seed=77)
    sinks = np.random.default_rng(3).standard_normal(8).astype(np.float32)
    want, _ = orc.flash_attn(q, k, v, mask, 0.125, sinks=sinks, softcap=15.0)
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 0.125, sinks=sinks, softcap=15.0)
    scale = np.abs(want).max(axis=-1, keepdims=True)
    assert (np.abs(got - want) <= REL_TOL * scale).all()


@pytest.mark.parametrize("D", [128, 64])
def test_rows_over_a_cache_shared_by_sixteen_sequences(dev, D):
    """batched decode over the unified cache: 16 rows, each seeing only its own sequence's cells (blocks of prompt
    cells, then interleaved generated ones) among 3072; one row sees nothing"""
    T, n_kv = 16, 3072
    q, k, v, _ = synth_case(8, 2, D, T, n_kv, seed=77, causal=False)
    m = np.full((T, n_kv), -np.inf, dtype=np.float16)
    for t in range(T):
        m[t, t * 128:(t + 1) * 128] = 0.0            # the sequence's prompt cells
        m[t, 2048 + t:2048 + 16 * 40:16] = 0.0        # its generated tokens, one cell in sixteen
    m[5, :] = -np.inf
    mask = m.view(np.uint16)
    want, _ = orc.flash_attn(q, k, v, mask, 0.0883883)
    got = dev.flash_attn(q, dev.KvCacheView(k, v), mask, 0.0883883)
    assert bits_equal(got, want)
    assert not got[:, 5].any() if got.shape[1] == T else not got[5].any()


def test_head_per_cta_kernel_passes_the_same_cases():
    """the CTA-per-head split-KV kernel is selected by B200_FA_DECODE_HEAD=1, read once per process: run this
    file's other tests in a child with it set"""
    import os
    import subprocess
    import sys
    if os.environ.get("B200_FA_DECODE_HEAD") == "1":
        pytest.skip("already the child")
    env = dict(os.environ, B200_FA_DECODE_HEAD="1")
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider"], env=env,
                       capture_output=True, text=True, timeout=1800)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
