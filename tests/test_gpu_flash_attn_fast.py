"""FLASH_ATTN_EXT in the library's fast numerics mode (f32 accumulation, no ordered f16 chain) against the CPU
oracle and against a float64 evaluation of softmax(q k^T scale + mask) v (-m gpu).

Tolerance asked of F16-KV attention: 1e-3, applied per output row relative to the row's largest magnitude (an
element near zero has no meaningful relative error of its own).  Three distances are measured and printed for
every case: GPU - CPU, GPU - f64 and CPU - f64.  The CPU path itself sits 2e-3 (512 cached positions) to 1.6e-2
(32768) away from f64: with F16 values it keeps its accumulator in f16 and rounds it once per position
(crates/ggml/src/flash_attn.rs:583-641; the reference's own test allows 1e-2 there, :1631-1636).  No kernel that
computes the function accurately can therefore be within 1e-3 of the CPU's bits at those lengths; what is
required here is that the fast kernel is within 1e-3 of f64, and no further from f64 than the CPU path is, which
bounds its distance from the CPU by the CPU's own error.  (The exact kernels of the other test files reproduce
the CPU's bits, f16 chain included.)"""
import numpy as np
import pytest

import b200
import orc
from test_gpu_flash_attn import synth_case

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.fixture(scope="module")
def dev():
    mod = b200.load()
    assert mod.device_count() > 0
    mod.set_device(0)
    return mod


def ref64(q, k, v, mask, scale):
    """q f32 [H, T, D]; k, v f16 bits [Hkv, n_kv, D]; mask f16 bits [T, n_kv] -> f64 [T, H, D]"""
    H, T, D = q.shape
    G = H // k.shape[0]
    kf, vf = k.view(np.float16).astype(np.float64), v.view(np.float16).astype(np.float64)
    m = np.zeros((T, k.shape[1])) if mask is None else mask.view(np.float16).astype(np.float64)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        s = q[h].astype(np.float64) @ kf[h // G].T * scale + m
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        out[:, h] = (p / p.sum(axis=1, keepdims=True)) @ vf[h // G]
    return out


def row_rel(a, b):
    """largest |a - b| per output row over the row's largest |b|"""
    return float((np.abs(a - b).max(axis=-1) / np.maximum(np.abs(b).max(axis=-1), 1e-30)).max())


def run_fast(dev, q, k, v, mask, scale, **kw):
    """mode 1: the fast kernel wherever it applies (the numerics policy alone sends only single query rows to it)"""
    return dev.flash_attn(q, dev.KvCacheView(k, v), mask, scale, mode=1, **kw)


def test_fast_policy_takes_rows_below_a_prompt_batch(dev, monkeypatch):
    """under the fast numerics policy fewer than 64 query rows take the tensor-core decode kernel (not the CPU's bits,
    within the tolerance of f64); with that kernel switched off a single row takes the f32 CUDA-core kernel and several
    rows keep the exact kernels"""
    scale = 1.0 / np.sqrt(128.0)
    dev.set_numerics(dev.FAST)
    try:
        q1, k1, v1, mask1 = synth_case(8, 2, 128, 1, 768, seed=9)
        cpu1, _ = orc.flash_attn(q1, k1, v1, mask1, scale, n_chunks=8)
        q3, k3, v3, mask3 = synth_case(8, 2, 128, 3, 300, seed=10)
        cpu3, _ = orc.flash_attn(q3, k3, v3, mask3, scale)
        got = dev.flash_attn(q1, dev.KvCacheView(k1, v1), mask1, scale, n_chunks=8)
        assert not np.array_equal(got.view(np.uint32), cpu1.view(np.uint32)) and row_rel(got, ref64(q1, k1, v1, mask1, scale)) <= TOL
        got = dev.flash_attn(q3, dev.KvCacheView(k3, v3), mask3, scale)
        assert not np.array_equal(got.view(np.uint32), cpu3.view(np.uint32)) and row_rel(got, ref64(q3, k3, v3, mask3, scale)) <= TOL
        monkeypatch.setenv("B200_FA_DECODE_MMA", "0")
        got = dev.flash_attn(q1, dev.KvCacheView(k1, v1), mask1, scale, n_chunks=8)
        assert not np.array_equal(got.view(np.uint32), cpu1.view(np.uint32)) and row_rel(got, ref64(q1, k1, v1, mask1, scale)) <= 1e-5
        got = dev.flash_attn(q3, dev.KvCacheView(k3, v3), mask3, scale)
        assert np.array_equal(got.view(np.uint32), cpu3.view(np.uint32))
    finally:
        dev.set_numerics(dev.EXACT)


@pytest.mark.parametrize("kernel", ["mma", "cuda-core"])
@pytest.mark.parametrize("n_kv", [512, 768, 4096, 32768])
def test_decode_one_row_gqa_128(dev, n_kv, kernel, monkeypatch):
    """the benchmark's decode shape: 32 query heads on 8 KV heads of 128, one query row, causal mask; the tensor-core
    decode kernel (csrc/flash_attn_decode_mma.cu) and the CUDA-core one (csrc/flash_attn_fast.cu)"""
    monkeypatch.setenv("B200_FA_DECODE_MMA", "1" if kernel == "mma" else "0")
    scale = 1.0 / np.sqrt(128.0)
    q, k, v, mask = synth_case(32, 8, 128, 1, n_kv, seed=n_kv + 1)
    cpu, _ = orc.flash_attn(q, k, v, mask, scale, n_chunks=8)
    want = ref64(q, k, v, mask, scale)
    got = run_fast(dev, q, k, v, mask, scale)
    d_gc, d_g64, d_c64 = row_rel(got, cpu), row_rel(got, want), row_rel(cpu, want)
    print(f"decode n_kv={n_kv}: GPU-CPU {d_gc:.2e}  GPU-f64 {d_g64:.2e}  CPU-f64 {d_c64:.2e}")
    assert d_g64 <= TOL
    assert d_g64 <= max(d_c64, 1e-5)
    assert d_gc <= 1.05 * (d_c64 + d_g64) + 1e-6


@pytest.mark.parametrize("kernel", ["mma", "cuda-core"])
@pytest.mark.parametrize("shape", [(16, 3072, 128), (5, 300, 64), (2, 700, 128), (63, 200, 128), (33, 9000, 128)], ids=str)
def test_few_rows_with_ragged_masks(dev, shape, kernel, monkeypatch):
    """several rows, each with its own visible cells (batched decode over a shared cache), a row that sees nothing,
    a context that is not a multiple of the tile"""
    monkeypatch.setenv("B200_FA_DECODE_MMA", "0" if kernel == "cuda-core" else "1")
    T, n_kv, D = shape
    q, k, v, _ = synth_case(8, 2, D, T, n_kv, seed=T * 7 + n_kv, causal=False)
    rng = np.random.default_rng(T)
    m = np.full((T, n_kv), -np.inf, dtype=np.float16)
    for t in range(T):
        lo = int(rng.integers(0, n_kv // 2))
        m[t, lo:lo + max(1, n_kv // (T + 1))] = 0.0
        m[t, n_kv - 1 - t % 3] = 0.0
    if T > 2:
        m[2, :] = -np.inf
    mask = m.view(np.uint16)
    scale = 1.0 / np.sqrt(float(D))
    cpu, _ = orc.flash_attn(q, k, v, mask, scale)
    got = run_fast(dev, q, k, v, mask, scale)
    if T > 2:
        assert not got[2].any() and not cpu[2].any()
    live = [t for t in range(T) if not (T > 2 and t == 2)]
    with np.errstate(invalid="ignore"):
        want = ref64(q, k, v, mask, scale)
    d_gc, d_g64, d_c64 = row_rel(got[live], cpu[live]), row_rel(got[live], want[live]), row_rel(cpu[live], want[live])
    print(f"rows {shape}: GPU-CPU {d_gc:.2e}  GPU-f64 {d_g64:.2e}  CPU-f64 {d_c64:.2e}")
    assert d_g64 <= TOL and d_g64 <= max(d_c64, 1e-5)


@pytest.mark.parametrize("heads", [(4, 4), (8, 4), (16, 2), (16, 1), (12, 4), (32, 8)], ids=str)
@pytest.mark.parametrize("shape", [(1, 1000, 128, True), (7, 650, 64, True), (1, 333, 128, False), (4, 64, 64, False)], ids=str)
def test_decode_kernel_head_groupings(dev, heads, shape):
    """1, 2, 4, 8 and 16 query heads per KV head (row blocks of whole tokens; three heads per KV head do not tile a block
    of 16 rows and take the CUDA-core kernel), head sizes 128 and 64, with a causal mask and with none, a cache
    shorter than two tiles"""
    H, Hkv = heads
    T, n_kv, D, causal = shape
    q, k, v, mask = synth_case(H, Hkv, D, T, n_kv, seed=H * 100 + T, causal=causal)
    scale = 1.0 / np.sqrt(float(D))
    cpu, _ = orc.flash_attn(q, k, v, mask, scale)
    want = ref64(q, k, v, mask, scale)
    got = run_fast(dev, q, k, v, mask, scale)
    d_g64, d_c64 = row_rel(got, want), row_rel(cpu, want)
    print(f"heads {heads} {shape}: GPU-f64 {d_g64:.2e}  CPU-f64 {d_c64:.2e}")
    assert dev.kernel_error() == 0
    assert d_g64 <= TOL and d_g64 <= max(d_c64, 1e-5)


def test_unsupported_variants_fall_back_to_the_exact_kernels(dev):
    """sinks and softcap are not in the fast kernel: the call still succeeds and gives the exact path's bits"""
    q, k, v, mask = synth_case(8, 2, 64, 1, 600, seed=5)
    sinks = np.random.default_rng(3).standard_normal(8).astype(np.float32)
    want, _ = orc.flash_attn(q, k, v, mask, 0.125, sinks=sinks, n_chunks=8)
    got = run_fast(dev, q, k, v, mask, 0.125, sinks=sinks, n_chunks=8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


# ---- prompt batches: the tensor-core kernel (csrc/flash_attn_prefill.cu) ---------------------------------------------
PREFILL = [
    # (H, Hkv, D, T, n_kv, causal)
    (8, 2, 128, 64, 64, True),        # one tile, one row block per KV head
    (8, 2, 128, 100, 1000, True),     # ragged rows, ragged last tile
    (32, 8, 128, 512, 512, True),     # the prompt shape of the 8B model: half of every tile row is the causal future
    (32, 8, 128, 128, 4096, True),    # a long cache in front of the batch
    (6, 2, 64, 70, 333, True),        # three heads per KV head (a row block starts in the middle of a token), head size 64
    (4, 4, 64, 65, 129, True),        # one head per KV head: 64 mask rows per row block
    (8, 2, 128, 96, 777, False),      # no mask at all
]


@pytest.mark.parametrize("kernel", ["tcgen05", "mma.sync"])
@pytest.mark.parametrize("shape", PREFILL, ids=str)
def test_prompt_batches(dev, shape, kernel, monkeypatch):
    """the mma.sync kernel is the default; head size 128 with two or more heads per KV head also has a tcgen05 kernel,
    taken when B200_FA_PREFILL_TC=1 (read per call)"""
    H, Hkv, D, T, n_kv, causal = shape
    if kernel == "tcgen05":
        if D != 128 or H == Hkv:
            pytest.skip("no tcgen05 form for this shape")
        monkeypatch.setenv("B200_FA_PREFILL_TC", "1")
    q, k, v, mask = synth_case(H, Hkv, D, T, n_kv, seed=sum(shape[:5]), causal=causal)
    scale = 1.0 / np.sqrt(float(D))
    want = ref64(q, k, v, mask, scale)
    got = run_fast(dev, q, k, v, mask, scale)
    d_g64 = row_rel(got, want)
    # the same function with q rounded to f16 first, as the CPU path (and this kernel) rounds it: flash_attn.rs:433
    d_g64q = row_rel(got, ref64(q.astype(np.float16).astype(np.float32), k, v, mask, scale))
    line = f"prompt {shape} {kernel}: GPU-f64 {d_g64:.2e}  GPU-f64(q16) {d_g64q:.2e}"
    if T * n_kv * H <= 8 * 100 * 1000:   # the CPU restatement is a scalar loop: small cases only
        cpu, _ = orc.flash_attn(q, k, v, mask, scale)
        d_gc, d_c64 = row_rel(got, cpu), row_rel(cpu, want)
        line += f"  GPU-CPU {d_gc:.2e}  CPU-f64 {d_c64:.2e}"
        assert d_gc <= 1.05 * (d_c64 + d_g64) + 1e-6
    print(line)
    assert d_g64 <= TOL


def test_prompt_batch_with_holes_and_blind_rows(dev):
    """a mask that is not causal: windows per token, a token that sees nothing, whole tiles nobody sees"""
    H, Hkv, D, T, n_kv = 8, 2, 128, 130, 1500
    q, k, v, _ = synth_case(H, Hkv, D, T, n_kv, seed=77, causal=False)
    rng = np.random.default_rng(5)
    m = np.full((T, n_kv), -np.inf, dtype=np.float16)
    for t in range(T):
        lo = int(rng.integers(0, 700))
        m[t, lo:lo + 1 + int(rng.integers(0, 200))] = 0.0
        m[t, 1400 + t % 7] = 0.0            # positions 900..1399 stay hidden from everyone: skipped tiles
    m[17, :] = -np.inf
    mask = m.view(np.uint16)
    scale = 1.0 / np.sqrt(float(D))
    got = run_fast(dev, q, k, v, mask, scale)
    assert not got[17].any()
    live = [t for t in range(T) if t != 17]
    with np.errstate(invalid="ignore"):
        want = ref64(q, k, v, mask, scale)
    assert row_rel(got[live], want[live]) <= TOL


def test_prompt_batches_follow_the_numerics_policy(dev):
    """mode 0: the exact tiled kernel (the CPU's bits) under the exact policy, the tensor-core kernel under the fast one"""
    q, k, v, mask = synth_case(8, 2, 128, 64, 256, seed=31)
    scale = 1.0 / np.sqrt(128.0)
    cpu, _ = orc.flash_attn(q, k, v, mask, scale)
    kv = dev.KvCacheView(k, v)
    assert np.array_equal(dev.flash_attn(q, kv, mask, scale).view(np.uint32), cpu.view(np.uint32))
    dev.set_numerics(dev.FAST)
    try:
        got = dev.flash_attn(q, kv, mask, scale)
    finally:
        dev.set_numerics(dev.EXACT)
    assert not np.array_equal(got.view(np.uint32), cpu.view(np.uint32))
    assert row_rel(got, ref64(q, k, v, mask, scale)) <= TOL
