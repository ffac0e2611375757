"""Each kernel alone against a plain fp32 (or float64) restatement of the same op, at sizes other
than the engine's: widths and vocabularies that are no power of two, head sizes in steps of 16,
odd group counts, rows that straddle tiles, pages in scrambled order.  Where random inputs would
hide a fault (one far key among hundreds, a window's edge) the inputs are made so that it shows.
"""
import math

import numpy as np
import pytest
import torch

from tests.plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from gophonic_b200 import ops
    return ops


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(device=DEV, dtype=dtype)


def close(got: torch.Tensor, ref: torch.Tensor, tol: float):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-30)
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def tol_of(dtype):
    return 2e-5 if dtype == torch.float32 else 1.2e-2


# ---- embedding, norm, activation ----------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_gather(ops, dtype):
    table = rnd(333, 72, dtype=dtype)
    ids = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty((5, 72), dtype=torch.float32, device=DEV)
    ops.embed_gather(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [16, 80, 1000, 4100])
def test_add_rmsnorm(ops, dtype, n):
    rows, eps = 7, 3e-5
    h, delta, w = rnd(rows, n, seed=1), rnd(rows, n, seed=2), 1 + 0.1 * rnd(n, seed=3)
    ref_h = h.double() + delta.double()
    ref = ref_h / torch.sqrt((ref_h * ref_h).mean(-1, keepdim=True) + eps) * w.double()
    h1, out = h.clone(), torch.empty((rows, n), dtype=dtype, device=DEV)
    ops.add_rmsnorm(h1, delta, w, eps, out)
    close(h1, ref_h, 1e-6)
    close(out, ref, tol_of(dtype))
    # without an addend the residual is left alone
    h2, out2 = h.clone(), torch.empty((rows, n), dtype=dtype, device=DEV)
    ops.add_rmsnorm(h2, None, w, eps, out2)
    assert torch.equal(h2, h)
    close(out2, h.double() / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps) * w.double(), tol_of(dtype))
    # gathered rows: normalise h[idx] + delta[idx], residual untouched
    idx = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    h3, out3 = h.clone(), torch.empty((3, n), dtype=dtype, device=DEV)
    ops.add_rmsnorm(h3, delta, w, eps, out3, idx)
    assert torch.equal(h3, h)
    close(out3, ref[idx.long()], tol_of(dtype))
    # a row's result does not depend on the other rows
    out4 = torch.empty((1, n), dtype=dtype, device=DEV)
    ops.add_rmsnorm(h[2:3].clone(), delta[2:3].clone(), w, eps, out4)
    assert torch.equal(out4[0], out[2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter", [8, 136, 1000])
def test_swiglu(ops, dtype, inter):
    gu = rnd(5, 2 * inter, dtype=dtype, scale=3.0)
    out = torch.empty((5, inter), dtype=dtype, device=DEV)
    ops.swiglu(gu, out)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    close(out, g / (1 + torch.exp(-g)) * u, 1e-6 if dtype == torch.float32 else 5e-3)
    big = torch.tensor([[-100.0, 100.0, 0.0, -20.0, 1.0, 1.0, 1.0, 1.0]], device=DEV)
    o = torch.empty((1, 4), device=DEV)
    ops.swiglu(big, o)
    assert torch.isfinite(o).all() and o[0, 1] == 100.0 and abs(o[0, 0].item()) < 1e-30


@pytest.mark.parametrize("M", [1, 8, 9, 33, 64, 100, 128, 300])
@pytest.mark.parametrize("inter,K", [(8, 64), (136, 80), (1000, 96), (12288 // 8, 512), (4096, 2048), (9600, 1024)])  # the last two: K slices
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_with_swiglu_epilogue(ops, M, inter, K, out_dtype):
    """gate/up rows interleaved in blocks of eight; the few-row kernel applies silu(gate) * up itself,
    and the stand-alone kernel reads the same interleaved layout."""
    gate, up = rnd(inter, K, dtype=torch.bfloat16, scale=0.2, seed=1), rnd(inter, K, dtype=torch.bfloat16, scale=0.2, seed=2)
    w = torch.stack([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    x = rnd(M, K, dtype=torch.bfloat16, seed=3)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    ref = g / (1 + torch.exp(-g)) * u
    assert ops.gemm_swiglu_accepts(x, w)
    algos = ["auto"] + (["skinny"] if M <= 64 else ["tc5", "tc5_pair"]) + (["tc5_decode"] if M <= ops.TC5_DECODE_MAX_ROWS else [])
    for algo in algos:
        out = torch.full((M, inter), float("nan"), dtype=out_dtype, device=DEV)
        ops.gemm_swiglu(x, w, out, algo=algo)
        close(out, ref, 2e-5 if out_dtype == torch.float32 else 6e-3)
    assert ops.tc5_status() == 0
    gu = torch.empty((M, 2 * inter), dtype=torch.bfloat16, device=DEV)
    ops.gemm(x, w, gu)
    out2 = torch.empty((M, inter), dtype=torch.bfloat16, device=DEV)
    ops.swiglu(gu, out2, True)
    close(out2, ref, 1.2e-2)


# ---- few-row products with the norm and the residual add folded in ---------------------------
# up to 8 rows the fragment-streaming kernel, 9 to 64 the tcgen05 decode kernel (alone and in clusters of K slices)
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K,count", [(64, 64, 1), (1000, 96, 5), (6144, 4096, 256), (136, 2048, 128), (40, 520, 33), (24576, 512, 7), (33024, 64, 3),
                                       (5120, 8192, 40)])   # the last one is large enough for the tcgen05 decode kernel at every row count
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_that_applies_the_rows_norm_factors_from_statistics(ops, M, N, K, count, out_dtype):
    """out = rmsnorm(h) w^T where the rows arrive as bf16(h * norm weight) and each row's sum of
    squares as ``count`` partial sums (here: of uneven column blocks): the kernel adds them up and
    multiplies its finished sums by 1 / sqrt(mean + eps)."""
    eps = 2e-6
    h, nw = rnd(M, K, scale=3.0, seed=1), 1 + 0.1 * rnd(K, seed=2)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=3)
    edges = torch.linspace(0, K, count + 1).round().long().tolist()
    stats = torch.full((max(M, 8), max(count, 8) + 3), float("nan"), device=DEV)
    for c in range(count):
        stats[:M, c] = (h[:, edges[c]:edges[c + 1]].double() ** 2).sum(-1).float()
    x = (h * nw).to(torch.bfloat16)
    rs = 1.0 / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    ref = rs * (x.double() @ w.double().T)
    assert ops.gemm_scaled_accepts(x, w)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    ops.gemm_scaled(x, eps, stats, count, w, out)
    close(out, ref, 2e-5 if out_dtype == torch.float32 else 6e-3)
    # against the norm itself: the rows were rounded to bfloat16 before instead of after the factor
    exact = (h.double() * rs * nw.double()) @ w.double().T
    close(out, exact, 1.2e-2)
    if 1 < M <= 8:   # a row's result does not depend on the other rows
        one = torch.empty((1, N), dtype=out_dtype, device=DEV)
        ops.gemm_scaled(x[M - 1:].contiguous(), eps, stats[M - 1:].contiguous(), count, w, one)
        assert torch.equal(one[0], out[M - 1])
    elif M > 8:      # nor on where among them it stands (another row count may mean another kernel)
        back = torch.empty_like(out)
        ops.gemm_scaled(x.flip(0).contiguous(), eps, stats[:M].flip(0).contiguous(), count, w, back)
        assert torch.equal(back.flip(0), out)


@pytest.mark.parametrize("M", [1, 5, 8, 12, 40, 64])
@pytest.mark.parametrize("inter,K", [(8, 64), (136, 80), (12288 // 8, 512), (12288, 1024), (16512, 64)])
def test_gemm_that_applies_the_rows_norm_factors_with_the_swiglu_epilogue(ops, M, inter, K):
    eps = 1e-6
    gate, up = rnd(inter, K, dtype=torch.bfloat16, scale=0.2, seed=1), rnd(inter, K, dtype=torch.bfloat16, scale=0.2, seed=2)
    w = torch.stack([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    h, nw = rnd(M, K, scale=2.0, seed=3), 1 + 0.1 * rnd(K, seed=4)
    stats = torch.zeros((max(M, 8), 8), device=DEV)
    stats[:M, 0] = (h.double() ** 2).sum(-1).float()
    x = (h * nw).to(torch.bfloat16)
    rs = 1.0 / torch.sqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    g, u = rs * (x.double() @ gate.double().T), rs * (x.double() @ up.double().T)
    out = torch.full((M, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_scaled(x, eps, stats, 1, w, out, swiglu=True)
    close(out, g / (1 + torch.exp(-g)) * u, 6e-3)


@pytest.mark.parametrize("M", [1, 4, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(64, 64), (1000, 96), (4096, 12288), (4096, 4096), (40, 520), (5120, 1024), (19200, 128), (5120, 8192)])
def test_gemm_that_adds_into_the_residual_and_prepares_the_next_norm(ops, M, N, K):
    """h += x w^T in the product's own epilogue: the bits of the product into a buffer and a float32
    add; partial sums of squares of the new residual, one per block of columns (16 wide up to 8
    rows, 128 wide above); and the new rows times the next norm's weight, rounded to bfloat16."""
    x, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    h0, nw = rnd(M, N, seed=3), 1 + 0.1 * rnd(N, seed=4)
    prod = torch.empty((M, N), dtype=torch.float32, device=DEV)
    algo = ops.gemm_algo(M, N, K)        # few rows: the fragment-streaming kernel, unless the product is large
    assert algo == ("skinny" if M <= 8 and (N, K) != (5120, 8192) else "tc5_decode")
    ops.gemm(x, w, prod, algo=algo)
    h = h0.clone()
    room = ops.fold_capacity(N)
    stats = torch.full((max(M, 8), room + 2), float("nan"), device=DEV)
    nxt = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    assert ops.gemm_residual_accepts(x, w, h)
    count = ops.gemm_residual(x, w, h, stats, nw, nxt)
    block = 16 if algo == "skinny" else 128
    assert count == (N + block - 1) // block
    assert torch.equal(h, h0 + prod)
    close(h, h0.double() + x.double() @ w.double().T, 2e-5)
    assert torch.equal(nxt, (h * nw).to(torch.bfloat16))
    pad = torch.zeros((M, count * block), dtype=torch.float64, device=DEV)
    pad[:, :N] = h.double()
    want = (pad ** 2).view(M, count, block).sum(-1)
    assert (stats[:M, :count].double() - want).abs().max() <= 1e-5 * want.abs().max()
    assert torch.isnan(stats[M:]).all() and torch.isnan(stats[:, count:]).all()      # nothing else is written
    # without a next norm only the residual and the statistics are written
    h2, stats2 = h0.clone(), torch.zeros((max(M, 8), room), device=DEV)
    assert ops.gemm_residual(x, w, h2, stats2) == count
    assert torch.equal(h2, h) and torch.equal(stats2[:M, :count], stats[:M, :count])
    with pytest.raises(ops.KernelError):
        ops.gemm_residual(rnd(65, K, dtype=torch.bfloat16), w, torch.zeros((65, N), device=DEV), torch.zeros((65, room), device=DEV))
    with pytest.raises(ops.KernelError, match="without a tensor"):
        ops.gemm_residual(x, w, h2, stats2, nw, None)


def test_embedding_leaves_row_statistics_and_prepares_the_first_norm(ops):
    table = rnd(333, 72, dtype=torch.bfloat16)
    ids = torch.tensor([0, 332, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty((5, 72), dtype=torch.float32, device=DEV)
    stats = torch.full((8, 9), float("nan"), device=DEV)
    nw = 1 + 0.1 * rnd(72, seed=4)
    nxt = torch.empty((5, 72), dtype=torch.bfloat16, device=DEV)
    ops.embed_gather(table, ids, out, stats, nw, nxt)
    assert torch.equal(out, table[ids.long()].float())
    assert torch.equal(nxt, (out * nw).to(torch.bfloat16))
    want = (out.double() ** 2).sum(-1)
    assert (stats[:5, 0].double() - want).abs().max() <= 1e-6 * want.max() and torch.isnan(stats[:, 1:]).all()


# ---- matrix products ----------------------------------------------------------------------
SHAPES = [(1, 64, 64), (3, 1000, 96), (17, 136, 80), (64, 333, 160), (65, 192, 96), (130, 520, 264), (257, 96, 4104)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("combo", ["fff", "bbf", "bbb", "bfb", "fbf"])
def test_gemm_simt(ops, M, N, K, combo):
    dt = {"f": torch.float32, "b": torch.bfloat16}
    a, w = rnd(M, K, dtype=dt[combo[0]], seed=1), rnd(N, K, dtype=dt[combo[1]], scale=0.1, seed=2)
    out = torch.empty((M, N), dtype=dt[combo[2]], device=DEV)
    ops.gemm_simt(a, w, out)
    close(out, a.double() @ w.double().T, 2e-5 if combo[2] == "f" else 6e-3)


def test_gemm_simt_rows_do_not_depend_on_the_batch(ops):
    a, w = rnd(70, 200, seed=4), rnd(150, 200, seed=5)
    full = torch.empty((70, 150), device=DEV)
    ops.gemm_simt(a, w, full)
    one = torch.empty((1, 150), device=DEV)
    ops.gemm_simt(a[67:68].contiguous(), w, one)
    assert torch.equal(one[0], full[67])


@pytest.mark.parametrize("algo", ["skinny", "tc5", "tc5_pair", "tc5_decode"])
@pytest.mark.parametrize("M,N,K", SHAPES + [(8, 4096, 1024), (64, 1536, 2048), (100, 1536, 2048), (128, 200, 8200), (256, 4096, 520),
                                            (300, 1000, 512), (2048, 512, 1024), (48, 19200, 1024)])   # the last: more tiles than SMs
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tensor_core_kernels(ops, algo, M, N, K, out_dtype):
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    if (algo == "skinny" and M > 64) or (algo == "tc5_decode" and M > ops.TC5_DECODE_MAX_ROWS):
        with pytest.raises(ops.KernelError):
            ops.gemm(a, w, out, algo=algo)
        return
    if algo in ("tc5", "tc5_pair") and not ops.tc5_accepts(a, w, out):
        with pytest.raises(ops.KernelError):
            ops.gemm(a, w, out, algo=algo)
        return
    ops.gemm(a, w, out, algo=algo)
    if algo.startswith("tc5"):
        assert ops.tc5_status() == 0, "a tcgen05 kernel gave up waiting on a barrier"
    close(out, a.double() @ w.double().T, 2e-5 if out_dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("M,N,K", [(192, 96, 64), (300, 1000, 512), (2048, 520, 1032), (257, 96, 4104)])
def test_gemm_adds_into_the_residual(ops, M, N, K):
    """out += a w^T in the epilogue: the same bits as the product into a buffer and a float32 add."""
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    h = rnd(M, N, seed=3)
    assert ops.gemm_add_accepts(a, w, h)
    prod = torch.empty((M, N), dtype=torch.float32, device=DEV)
    ops.gemm(a, w, prod, algo="tc5_pair")
    want = h + prod
    ops.gemm_add(a, w, h)
    assert ops.tc5_status() == 0
    assert torch.equal(h, want)
    close(h, rnd(M, N, seed=3).double() + a.double() @ w.double().T, 2e-5)
    small = rnd(8, K, dtype=torch.bfloat16, seed=4)
    assert not ops.gemm_add_accepts(small, w, torch.empty((8, N), device=DEV))


# Sizes of a full-size layer: every CTA of the persistent kernels computes several tiles one after
# the other (768 tiles of 256 x 256 on 74 pairs, 1536 of 128 x 256 on 148 CTAs), so both tensor-memory
# accumulators are handed back more than once, the stage ring runs on across tiles and the staging
# buffers of the reducing epilogue are used again; one ragged size whose last tiles hang over.
FULL_SIZE = [(2048, 24576, 4096), (2048, 4096, 12288), (2048, 6144, 4096), (150, 24576, 4096), (1000, 5000, 4104)]


def _close_wide(got: torch.Tensor, ref: torch.Tensor, tol: float):
    """As ``close``, on the device (the products are hundreds of megabytes), and naming the first
    bad element: its tile says which round of the tile loop went wrong."""
    err = (got.double() - ref).abs()
    scale = ref.abs().max().item()
    worst = err.max().item() / scale
    if not worst < tol:
        at = int(torch.nonzero(err.flatten() >= tol * scale)[0])
        r, c = divmod(at, ref.shape[1])
        raise AssertionError(f"relative error {worst:.3e} >= {tol}; first bad element ({r}, {c}), "
                             f"tile of 256 x 256 ({r // 256}, {c // 256})")
    assert torch.isfinite(got).all()


@pytest.mark.parametrize("M,N,K", FULL_SIZE)
def test_gemm_tiled_kernels_walk_many_tiles_per_cta(ops, M, N, K):
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    ref = a.double() @ w.double().T
    for algo in ("tc5", "tc5_pair"):
        for out_dtype in (torch.float32, torch.bfloat16):
            out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
            ops.gemm(a, w, out, algo=algo)
            assert ops.tc5_status() == 0, "a tcgen05 kernel gave up waiting on a barrier"
            _close_wide(out, ref, 2e-5 if out_dtype == torch.float32 else 6e-3)
    # the epilogue that adds into the fp32 residual: the bits of product-then-add, and the float64 sum
    h0 = rnd(M, N, seed=3)
    if not ops.gemm_add_accepts(a, w, h0):
        assert M < ops.TC5_PAIR_MIN_ROWS   # only prompt-sized steps add in the epilogue
        return
    prod = torch.empty((M, N), dtype=torch.float32, device=DEV)
    ops.gemm(a, w, prod, algo="tc5_pair")
    h = h0.clone()
    ops.gemm_add(a, w, h)
    assert ops.tc5_status() == 0
    assert torch.equal(h, h0 + prod)
    _close_wide(h, h0.double() + ref, 2e-5)
    # twice in a row into the same residual, as two layers do
    ops.gemm_add(a, w, h)
    assert torch.equal(h, (h0 + prod) + prod)


@pytest.mark.parametrize("M,inter,K", [(2048, 12288, 4096), (150, 12288, 4096), (1000, 2504, 4104)])
def test_gemm_swiglu_tiled_kernels_walk_many_tiles_per_cta(ops, M, inter, K):
    gate, up = rnd(inter, K, dtype=torch.bfloat16, scale=0.05, seed=1), rnd(inter, K, dtype=torch.bfloat16, scale=0.05, seed=2)
    w = torch.stack([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous()
    x = rnd(M, K, dtype=torch.bfloat16, seed=3)
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    ref = g / (1 + torch.exp(-g)) * u
    for algo in ("tc5", "tc5_pair", "auto"):
        for out_dtype in (torch.float32, torch.bfloat16):
            out = torch.full((M, inter), float("nan"), dtype=out_dtype, device=DEV)
            ops.gemm_swiglu(x, w, out, algo=algo)
            assert ops.tc5_status() == 0
            _close_wide(out, ref, 2e-5 if out_dtype == torch.float32 else 6e-3)


def test_gemm_dispatch_never_puts_float32_on_tensor_cores(ops):
    a, w = rnd(4, 64), rnd(8, 64)
    out = torch.empty((4, 8), device=DEV)
    assert ops.gemm(a, w, out) == "simt"
    a16 = a.to(torch.bfloat16)
    assert ops.gemm(a16, w, out) == "simt"  # a weight stored in 32-bit stays on the fp32 kernel
    with pytest.raises(ops.KernelError):
        ops.gemm_simt(a.cpu(), w, out)


# ---- fused per-head norm + rotation + cache write ------------------------------------------
def paged(n_pages, kvh, d, dtype, seed):
    k = rnd(n_pages, kvh, 64, d, dtype=dtype, seed=seed)
    v = rnd(n_pages, kvh, 64, d, dtype=dtype, seed=seed + 1)
    return k, v


def gather_kv(plane, table_row, length):
    """[length, kvh, d] of one sequence out of the paged plane."""
    pages = plane[table_row[: (length + 63) // 64].long()]          # [p, kvh, 64, d]
    return pages.permute(0, 2, 1, 3).reshape(-1, plane.shape[1], plane.shape[3])[:length]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d,rot,qk_norm", [(4, 2, 16, 16, True), (5, 1, 48, 48, True), (6, 3, 32, 16, True),
                                                    (2, 2, 128, 128, False), (3, 1, 80, 0, True), (5, 2, 128, 128, True), (2, 1, 128, 64, True)])
@pytest.mark.parametrize("lens", [[3, 70, 1], [3, 300, 1]])   # rows per sequence in this step; many rows: the prompt kernels
def test_qk_norm_rope_kv_write(ops, dtype, heads, kvh, d, rot, qk_norm, lens):
    eps, theta = 2e-6, 5000.0
    past = [0, 60, 130]         # tokens already cached
    slots = [2, 0, 5]
    rows = sum(lens)
    max_pages = (max(p + n for p, n in zip(past, lens)) + 63) // 64 + 1
    n_pages = 3 * max_pages + 4
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1)).to(torch.int32)
    table = torch.zeros((6, max_pages), dtype=torch.int32)
    for i, s in enumerate(slots):
        table[s] = perm[i * max_pages:(i + 1) * max_pages]
    table = table.to(DEV)
    k_plane, v_plane = paged(n_pages, kvh, d, dtype, 3)
    k0, v0 = k_plane.clone(), v_plane.clone()
    qkv = rnd(rows, (heads + 2 * kvh) * d, dtype=dtype, seed=9)
    qkv0 = qkv.clone()
    qw, kw = (1 + 0.1 * rnd(d, seed=5), 1 + 0.1 * rnd(d, seed=6)) if qk_norm else (None, None)
    row_pos = torch.tensor(sum(([p + j for j in range(n)] for n, p in zip(lens, past)), []), dtype=torch.int32, device=DEV)
    row_seq = torch.tensor(sum(([i] * n for i, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    cos = sin = None
    if rot:
        c, s = P.rope_tables(np.arange(512), rot, theta)
        cos, sin = (torch.tensor(x, dtype=torch.float32, device=DEV) for x in (c, s))
    ops.qk_norm_rope_kv_write(qkv, heads, kvh, d, qw, kw, eps, cos, sin, rot, row_pos, row_seq, seq_slot,
                              table, k_plane, v_plane, True)
    # reference in float64 from the inputs
    x = qkv0.double().cpu().numpy()
    q = x[:, :heads * d].reshape(rows, heads, d)
    k = x[:, heads * d:(heads + kvh) * d].reshape(rows, kvh, d)
    v = x[:, (heads + kvh) * d:].reshape(rows, kvh, d)
    if qk_norm:
        q, k = P.rms_norm(q, qw.double().cpu().numpy(), eps), P.rms_norm(k, kw.double().cpu().numpy(), eps)
    if rot:
        c, s = P.rope_tables(row_pos.cpu().numpy(), rot, theta)
        q, k = P.apply_rope(q, c, s), P.apply_rope(k, c, s)
    tol = tol_of(dtype)
    close(qkv[:, :heads * d], torch.tensor(q.reshape(rows, -1)), tol)
    assert torch.equal(qkv[:, heads * d:], qkv0[:, heads * d:])  # k and v columns of the buffer are not changed
    r = 0
    touched = torch.zeros(n_pages, 64, dtype=torch.bool)
    for i, (n, p0, slot) in enumerate(zip(lens, past, slots)):
        kk = gather_kv(k_plane, table[slot], p0 + n)[p0:]
        vv = gather_kv(v_plane, table[slot], p0 + n)[p0:]
        close(kk, torch.tensor(k[r:r + n]), tol)
        assert torch.equal(vv, qkv0[r:r + n, (heads + kvh) * d:].reshape(n, kvh, d))
        for pos in range(p0, p0 + n):
            touched[table[slot, pos // 64].item(), pos % 64] = True
        r += n
    # nothing else in the planes moved
    keep = ~touched.to(DEV)
    assert torch.equal(k_plane.permute(0, 2, 1, 3)[keep], k0.permute(0, 2, 1, 3)[keep])
    assert torch.equal(v_plane.permute(0, 2, 1, 3)[keep], v0.permute(0, 2, 1, 3)[keep])
    # a run that reads another run's cache writes nothing
    qkv2, k2, v2 = qkv0.clone(), k0.clone(), v0.clone()
    ops.qk_norm_rope_kv_write(qkv2, heads, kvh, d, qw, kw, eps, cos, sin, rot, row_pos, row_seq, seq_slot,
                              table, k2, v2, False)
    assert torch.equal(k2, k0) and torch.equal(v2, v0) and torch.equal(qkv2[:, :heads * d], qkv[:, :heads * d])


# ---- attention ------------------------------------------------------------------------------
def attention_reference(q, k_plane, v_plane, table, slots, q_lens, kv_lens, heads, kvh, d, scale, window):
    """float64, one sequence at a time, from the paged planes."""
    out = []
    r = 0
    for slot, ql, kl in zip(slots, q_lens, kv_lens):
        k = gather_kv(k_plane, table[slot], kl).double().cpu().numpy()
        v = gather_kv(v_plane, table[slot], kl).double().cpu().numpy()
        qq = q[r:r + ql].double().cpu().numpy().reshape(ql, heads, d)
        # rows are the last ql positions of kl keys: pad queries in front and take the tail
        full_q = np.zeros((kl, heads, d))
        full_q[kl - ql:] = qq
        out.append(P.causal_attention(full_q, k, v, scale, window)[kl - ql:].reshape(ql, heads * d))
        r += ql
    return torch.tensor(np.concatenate(out, 0))


def attention_case(ops, dtype, heads, kvh, d, q_lens, kv_lens, window=0, splits=1, algo="auto", seed=0, craft=None):
    nseq = len(q_lens)
    max_pages = (max(kv_lens) + 63) // 64
    n_pages = nseq * max_pages + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).to(torch.int32)
    slots = list(range(nseq - 1, -1, -1))
    table = torch.zeros((nseq, max_pages), dtype=torch.int32)
    for i, s in enumerate(slots):
        table[s] = perm[i * max_pages:(i + 1) * max_pages]
    table = table.to(DEV)
    k_plane, v_plane = paged(n_pages, kvh, d, dtype, seed + 1)
    rows = sum(q_lens)
    stride = heads * d + 24
    qbuf = rnd(rows, stride, dtype=dtype, seed=seed + 2)
    q = qbuf[:, :heads * d]
    if craft is not None:
        craft(q, k_plane, v_plane, table, slots)
    out = torch.full((rows, heads * d), float("nan"), dtype=dtype, device=DEV)
    starts = np.concatenate([[0], np.cumsum(q_lens)[:-1]])
    mk = lambda x: torch.tensor(list(x), dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    scratch = None
    if splits > 1:
        scratch = torch.empty(ops.attention_scratch_floats(nseq, heads, d, splits), dtype=torch.float32, device=DEV)
    used = ops.attention(q, out, k_plane, v_plane, table, mk(slots), mk(starts), mk(q_lens), mk(kv_lens), nseq,
                         max(q_lens), heads, kvh, d, scale, window, splits, scratch, algo=algo)
    ref = attention_reference(q, k_plane, v_plane, table, slots, q_lens, kv_lens, heads, kvh, d, scale, window)
    return out, ref, used


GEOMS = [(4, 2, 16), (6, 3, 32), (5, 1, 48), (8, 8, 64), (7, 1, 80), (4, 1, 96), (2, 1, 112), (32, 8, 128), (20, 1, 32),
         (2, 2, 256)]


KINDS = [(torch.float32, "simt"), (torch.bfloat16, "simt"), (torch.bfloat16, "auto")]


@pytest.mark.parametrize("dtype,algo", KINDS)
@pytest.mark.parametrize("heads,kvh,d", GEOMS)
def test_attention_prompts(ops, dtype, algo, heads, kvh, d):
    """Whole prompts, prompts that continue a cached prefix, and a single row, in one batch."""
    out, ref, used = attention_case(ops, dtype, heads, kvh, d, q_lens=[70, 5, 1, 33], kv_lens=[70, 69, 130, 33], algo=algo)
    close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)
    if algo == "auto":
        assert used == ("prefill_tc5" if d == 128 else "prefill_mma")
    out, ref, _ = attention_case(ops, dtype, heads, kvh, d, q_lens=[200, 130], kv_lens=[200, 333], algo=algo, seed=3)
    close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)
    assert ops.tc5_status() == 0


@pytest.mark.parametrize("algo", ["prefill_tc5", "prefill_mma"])
@pytest.mark.parametrize("heads,kvh", [(4, 1), (3, 3), (32, 8)])
def test_attention_prompts_head_dim_128_both_tensor_core_kernels(ops, algo, heads, kvh):
    """The tcgen05 kernel (tiles of 128 rows, two pages a step) and the mma.sync kernel on the same
    cases: lengths around the tile and page sizes, prompts that continue a cached prefix, a window."""
    for q_lens, kv_lens, window in (([128], [128], 0), ([129, 1, 64], [129, 300, 64], 0), ([257, 100], [257, 612], 0),
                                    ([300], [700], 150), ([65], [65], 7)):
        out, ref, used = attention_case(ops, torch.bfloat16, heads, kvh, 128, q_lens, kv_lens, window=window, algo=algo, seed=11)
        assert used == algo
        close(out, ref, 1.2e-2)
    assert ops.tc5_status() == 0


def test_attention_long_prompt_starts_its_ctas_kv_head_by_kv_head(ops):
    """A prompt whose keys and values (all kv heads) pass 48 MB makes the tcgen05 kernel start its CTAs
    one kv head after the other; the mma.sync kernel, which has no such order, must agree with it."""
    heads, kvh, d, n = 32, 16, 128, 6200          # 6200 * 16 * 512 bytes = 50.8 MB
    pages = (n + 63) // 64
    k_plane, v_plane = paged(pages, kvh, d, torch.bfloat16, 5)
    table = torch.randperm(pages, generator=torch.Generator().manual_seed(2)).to(torch.int32).reshape(1, pages).to(DEV)
    q = rnd(n, heads * d, dtype=torch.bfloat16, seed=6)
    mk = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    outs = {}
    for algo in ("prefill_tc5", "prefill_mma"):
        out = torch.full((n, heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        used = ops.attention(q, out, k_plane, v_plane, table, mk([0]), mk([0]), mk([n]), mk([n]), 1, n, heads, kvh, d,
                             d ** -0.5, 0, 1, None, algo=algo)
        assert used == algo
        outs[algo] = out.float()
    assert ops.tc5_status() == 0
    assert torch.isfinite(outs["prefill_tc5"]).all()
    err = (outs["prefill_tc5"] - outs["prefill_mma"]).abs().max() / outs["prefill_mma"].abs().max()
    assert err < 1.2e-2, float(err)


@pytest.mark.parametrize("dtype,algo", KINDS)
@pytest.mark.parametrize("heads,kvh,d", GEOMS)
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_attention_single_tokens(ops, dtype, algo, heads, kvh, d, splits):
    out, ref, used = attention_case(ops, dtype, heads, kvh, d, q_lens=[1, 1, 1, 1, 1], kv_lens=[1, 64, 65, 700, 333],
                                    splits=splits, algo=algo)
    close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)
    if algo == "auto":
        assert used == "decode_mma"


@pytest.mark.parametrize("heads,kvh,d,rot", [(4, 2, 16, 16), (5, 1, 48, 32), (32, 8, 128, 128), (8, 2, 128, 64), (20, 1, 32, 0), (2, 2, 256, 256),
                                              (40, 2, 64, 64), (6, 3, 112, 112)])
@pytest.mark.parametrize("splits", [1, 3, 8])
@pytest.mark.parametrize("normed,write,window", [(True, True, 0), (False, True, 0), (True, False, 0), (True, True, 100)])
def test_single_token_attention_that_rotates_and_stores_the_token_itself(ops, heads, kvh, d, rot, splits, normed, write, window):
    """One kernel instead of two: the queries are normed and rotated by the attention kernel, the
    token's own key and value come from the q/k/v row and are stored in the cache.  The output and
    the cache afterwards are the bits the two kernels one after the other give; a run that does not
    write the cache (it reads another run's) finds the key of its position there."""
    kv_lens = [1, 64, 65, 700, 333, 128]
    nseq = len(kv_lens)
    assert ops.attention_decode_rope_accepts(torch.bfloat16, d, rot, 1)
    max_pages = (max(kv_lens) + 63) // 64
    n_pages = nseq * max_pages + 2
    table = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(5))[:nseq * max_pages].to(torch.int32).reshape(nseq, max_pages).to(DEV)
    k0, v0 = paged(n_pages, kvh, d, torch.bfloat16, 11)
    qkv0 = rnd(nseq, (heads + 2 * kvh) * d, dtype=torch.bfloat16, seed=12)
    qw, kw = (1 + 0.1 * rnd(d, seed=13), 1 + 0.1 * rnd(d, seed=14)) if normed else (None, None)
    cos = torch.cos(rnd(800, max(rot // 2, 1), seed=15)) if rot else None
    sin = torch.sin(rnd(800, max(rot // 2, 1), seed=15)) if rot else None
    mk = lambda x: torch.tensor(list(x), dtype=torch.int32, device=DEV)
    pos, seqs, slots = mk([n - 1 for n in kv_lens]), mk(range(nseq)), mk(range(nseq))
    scratch = torch.empty(ops.attention_scratch_floats(nseq, heads, d, splits), dtype=torch.float32, device=DEV) if splits > 1 else None
    results = []
    for fused in (False, True):
        qkv, k, v = qkv0.clone(), k0.clone(), v0.clone()
        out = torch.full((nseq, heads * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        rope_args = (heads, kvh, d, qw, kw, 1e-6, cos, sin, rot, pos, seqs, slots, table, k, v, write)
        attn_args = (k, v, table, slots, mk(range(nseq)), mk([1] * nseq), mk(kv_lens), nseq, 1, heads, kvh, d, d ** -0.5, window, splits, scratch)
        if fused:
            ops.attention_decode_rope(qkv, out, rope_args, attn_args)
            assert torch.equal(qkv, qkv0)          # the rows stay as the product left them
        else:
            ops.qk_norm_rope_kv_write(qkv, *rope_args)
            ops.attention(qkv[:, :heads * d], out, *attn_args, algo="decode_mma")
        results.append((out, k, v))
    (out_a, k_a, v_a), (out_b, k_b, v_b) = results
    assert torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
    assert torch.equal(out_a, out_b)
    assert torch.equal(k_a, k0) != write and torch.equal(v_a, v0) != write


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kvh,d", [(8, 2, 24), (3, 1, 40), (2, 2, 6)])
def test_attention_head_sizes_that_are_no_multiple_of_16(ops, dtype, heads, kvh, d):
    """Even head sizes between the steps of 16 (the reference's own test shape has 24) run on the
    CUDA-core kernel in both dtypes: prompts, continued prompts, single tokens with key splits."""
    out, ref, used = attention_case(ops, dtype, heads, kvh, d, q_lens=[70, 5, 1, 33], kv_lens=[70, 69, 130, 33])
    assert used == "simt"
    close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)
    for splits in (1, 3):
        out, ref, used = attention_case(ops, dtype, heads, kvh, d, q_lens=[1, 1, 1], kv_lens=[1, 700, 65], splits=splits)
        assert used == "simt"
        close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)


def test_attention_head_sizes_without_a_tensor_core_kernel_fall_back(ops):
    out, ref, used = attention_case(ops, torch.bfloat16, 2, 1, 144, q_lens=[40, 1], kv_lens=[40, 90])
    assert used == "simt"
    close(out, ref, 1.2e-2)
    with pytest.raises(ops.KernelError, match="head_dim 144"):
        attention_case(ops, torch.bfloat16, 2, 1, 144, q_lens=[40], kv_lens=[40], algo="prefill_mma")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("algo", ["simt", "auto"])
@pytest.mark.parametrize("heads,kvh,d", [(4, 2, 64), (8, 2, 128), (8, 2, 24)])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype, algo, heads, kvh, d):
    """One query and one key 500 positions back are scaled so that key takes all the weight: the
    output must be that key's value, for a prompt row and for a single-token row.  At head_dim 128
    the prompt runs on the tcgen05 kernel and the single tokens on the mma.sync one; head_dim 24
    has no tensor-core kernel."""
    far = 37

    def craft(q, k_plane, v_plane, table, slots):
        for seq, slot in enumerate(slots):
            page, off = table[slot, far // 64].item(), far % 64
            k_plane[page, :, off] = 0
            k_plane[page, :, off, 3] = 30.0
        q[:] = q * 0.05
        q[:, 3::d] = 30.0
    for q_lens, kv_lens, splits in (([520], [520], 1), ([1, 1], [538, 100], 1), ([1, 1], [538, 100], 4)):
        out, ref, _ = attention_case(ops, dtype, heads, kvh, d, q_lens, kv_lens, splits=splits, algo=algo, craft=craft)
        close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)
        # the last row of the first sequence sits > 480 keys after the far key and still returns its value
        assert ref[q_lens[0] - 1].abs().max() > 0


@pytest.mark.parametrize("dtype,algo", KINDS)
def test_attention_window_edge(ops, dtype, algo):
    """With a window of w the key at distance w - 1 is the last one seen: a dominant key placed
    exactly there is found, one step further it is not."""
    heads, kvh, d, w = 2, 1, 32, 70
    for dist, q_lens, kv_lens in ((w - 1, [1], [200]), (w, [1], [200]), (w - 1, [90], [200]), (w, [90], [200])):
        target = kv_lens[0] - 1 - dist

        def craft(q, k_plane, v_plane, table, slots):
            page, off = table[slots[0], target // 64].item(), target % 64
            k_plane[page, :, off] = 0
            k_plane[page, :, off, 5] = 40.0
            q[:] = q * 0.05
            q[:, 5::d] = 40.0
        out, ref, _ = attention_case(ops, dtype, heads, kvh, d, q_lens, kv_lens, window=w, craft=craft, algo=algo)
        close(out, ref, 1e-5 if dtype == torch.float32 else 1.2e-2)


@pytest.mark.parametrize("algo", ["prefill_tc5", "prefill_mma", "simt"])
def test_attention_rescales_its_running_output_by_a_real_factor(ops, algo):
    """The tcgen05 kernel rescales O only when a row's maximum outgrew the scale in use by more than
    2^8.  Random scores never do that after the first page, so the inputs are made to: key A (second
    page) lifts the maximum by 2^7.3, just under the threshold (no rescale, probabilities up to 158
    rounded to bfloat16); key B (fourth page) lifts it by 2^8.5 over the scale in use, so O and the row
    sum are multiplied by 2^-8.5, after which the old keys, A and B each hold about a third of the
    weight: a factor that is wrong, or applied to only one of O and the sum, moves the output by
    tens of per cent.  Every other row has a weak query and keeps its scale, so a warp holds rows
    that rescale beside rows that multiply by one.  A second prompt continues a cached prefix."""
    heads, kvh, d = 4, 2, 128
    pos_a, pos_b = 100, 200
    unit = (1.0 / math.sqrt(d)) * 1.4426950408889634          # one raw score in the kernel's base-2 units

    def craft(q, k_plane, v_plane, table, slots):
        k_plane.mul_(0.25)
        k_plane[..., 3] = 0      # ordinary keys score within a few hundredths of zero
        for slot in slots:
            for pos, lift in ((pos_a, 7.5), (pos_b, 8.7)):
                page, off = table[slot, pos // 64].item(), pos % 64
                k_plane[page, :, off] = 0
                k_plane[page, :, off, 3] = lift / (8.0 * unit)
        q.mul_(0.05)
        q[0::2, 3::d] = 8.0      # strong rows: scores of A and B stand 7.5 and 8.7 above the rest
        q[1::2, 3::d] = 0.5      # weak rows: nothing grows
    out, ref, used = attention_case(ops, torch.bfloat16, heads, kvh, d, q_lens=[300, 70], kv_lens=[300, 400], algo=algo,
                                    seed=5, craft=craft)
    assert used == algo and ops.tc5_status() == 0
    close(out, ref, 1.2e-2)
    # the case is what it claims: on a strong row past B, neither B nor the keys before it are negligible
    assert ref[298].abs().max() > 0


def test_attention_refuses_what_it_cannot_take(ops):
    with pytest.raises(ops.KernelError, match="head_dim"):
        attention_case(ops, torch.float32, 2, 1, 272, [3], [3])
    with pytest.raises(ops.KernelError, match="single-token"):
        attention_case(ops, torch.float32, 2, 1, 32, [3], [3], splits=2)


# ---- selection --------------------------------------------------------------------------------
def test_argmax_first_maximum_nan_and_ties(ops):
    V = 151936
    x = rnd(6, V)
    x[0, 777] = x[0, 123456] = 50.0           # tie: the lower index
    x[1, 5] = float("nan")
    x[1, 9000] = 60.0
    x[2] = float("nan")                        # all NaN: index 0
    x[3, V - 1] = 70.0
    x[4] = -float("inf")
    x[5, 0] = 80.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(x, out)
    assert out.tolist() == [777, 9000, 0, V - 1, 0, 0]
    ref = [P.argmax_first(r) for r in x.cpu().numpy()]
    assert out.tolist() == ref


@pytest.mark.parametrize("V,wide", [(23, False), (1000, False), (151936, False), (151936, True), (20000, True)])
def test_sampler_matches_the_plain_sampler(ops, V, wide):
    """``wide``: with scratch, rows of a wide vocabulary are selected by many CTAs (histogram,
    gather, sort); without, one CTA scans each row.  Both follow the plain sampler."""
    rows = 12
    logits = rnd(rows, V, scale=2.0, seed=V)
    logits[3, : min(V, 40)] = 1.5           # many ties at the threshold
    logits[6, 100:6000] = 9.0               # thousands of equal logits on top: the candidate list overflows
    scratch = torch.zeros(ops.sample_scratch_bytes(rows, V), dtype=torch.uint8, device=DEV) if wide else None
    assert (scratch is None) or scratch.numel() > 0
    temps = [0.8, 1.0, 0.0, 0.7, 1.3, 0.5, 1.0, 1.0, 2.0, 0.9, 1.0, 0.3]
    ks = [20, 0, 5, 10, 1, 2000, 50, 3, 0, 7, 1024, 2]
    ps = [0.0, 0.9, 0.5, 0.0, 0.0, 0.95, 1.0, 0.5, 0.2, 0.0, 0.99, 0.0]
    for draw0 in (0, 17):
        seeds = [1000 + i for i in range(rows)]
        draws = [draw0 + i for i in range(rows)]
        mk = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        draws_dev = mk(draws, torch.int64)
        ops.sample(logits, mk(temps, torch.float32), mk(ks, torch.int32), mk(ps, torch.float32),
                   mk(seeds, torch.int64), draws_dev, out, scratch=scratch, advance=wide)
        if wide:  # the kernel advanced the counters of the rows it sampled, not of the greedy one
            assert draws_dev.tolist() == [d + (1 if temps[i] > 0 else 0) for i, d in enumerate(draws)]
        host = logits.cpu().numpy()
        for r in range(rows):
            tok, cand, probs = P.sample_token(host[r], temps[r], ks[r], ps[r], seeds[r], draws[r])
            got = out[r].item()
            if got != tok:
                # expf on the device and exp on the host may differ in the last place: the draw may
                # then fall on the other side of a boundary between neighbouring candidates
                assert cand is not None and got in cand
                i, j = cand.index(got), cand.index(tok)
                assert abs(i - j) == 1, (r, got, tok)


def test_sampler_distribution_and_batch_independence(ops):
    V = 300
    base = torch.full((V,), -30.0)
    base[[7, 100, 250]] = torch.tensor([math.log(5.0), math.log(3.0), math.log(2.0)])
    n = 4000
    logits = base.repeat(n, 1).to(DEV)
    mk = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(logits, mk([1.0] * n, torch.float32), mk([3] * n, torch.int32), mk([0.0] * n, torch.float32),
               mk([42] * n, torch.int64), mk(list(range(n)), torch.int64), out)
    counts = torch.bincount(out.long().cpu(), minlength=V).double() / n
    assert set(torch.nonzero(counts).flatten().tolist()) <= {7, 100, 250}      # never outside top-k
    assert abs(counts[7] - 0.5) < 0.035 and abs(counts[100] - 0.3) < 0.035 and abs(counts[250] - 0.2) < 0.035
    # equal (seed, draw) -> equal token, whatever else is in the batch
    one = torch.empty(1, dtype=torch.int32, device=DEV)
    for i in (0, 1234, 3999):
        ops.sample(logits[:1], mk([1.0], torch.float32), mk([3], torch.int32), mk([0.0], torch.float32),
                   mk([42], torch.int64), mk([i], torch.int64), one)
        assert one.item() == out[i].item()


def test_sampler_rows_take_their_options_by_index(ops):
    """opt_row: logits row i uses entry opt_row[i] of the option tables, as a batch whose shorter
    requests have ended does."""
    V = 40000
    logits = rnd(3, V, scale=2.0, seed=3)
    mk = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)
    temps, ks, ps = mk([0.0, 0.9, 0.0, 0.0, 0.7, 1.1], torch.float32), mk([0, 30, 0, 0, 0, 5], torch.int32), mk([0, 0.9, 0, 0, 0.5, 0], torch.float32)
    seeds, draws = mk([0, 11, 0, 0, 12, 13], torch.int64), mk([0, 4, 0, 0, 9, 2], torch.int64)
    opt_row = mk([5, 1, 4], torch.int32)
    out, ref = torch.empty(3, dtype=torch.int32, device=DEV), torch.empty(3, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(ops.sample_scratch_bytes(3, V), dtype=torch.uint8, device=DEV)
    ops.sample(logits, temps, ks, ps, seeds, draws.clone(), out, opt_row=opt_row, scratch=scratch)
    pick = opt_row.long()
    ops.sample(logits, temps[pick], ks[pick], ps[pick], seeds[pick], draws[pick], ref)
    assert out.tolist() == ref.tolist()


def test_presence_penalty_and_seen_bitmap(ops):
    V, rows = 70, 3
    logits = torch.zeros((rows, V), device=DEV)
    seen = torch.zeros((4, 3), dtype=torch.int32, device=DEV)
    seen_row = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    toks = torch.tensor([5, 69, 33], dtype=torch.int32, device=DEV)
    ops.mark_seen(toks, V, seen, seen_row)
    ops.mark_seen(torch.tensor([64, 69, 33], dtype=torch.int32, device=DEV), V, seen, seen_row)
    pres = torch.tensor([1.5, 0.0, 2.0], device=DEV)
    ops.presence_penalty(logits, seen, seen_row, pres)
    want = torch.zeros((rows, V))
    want[0, 5] = want[0, 64] = -1.5
    want[2, 33] = -2.0      # marked twice, penalised once; row 1 has no penalty
    assert torch.equal(logits.cpu(), want)
