"""Each kernel alone against a plain PyTorch float64/float32 reference of the same op, at sizes other
than the tiny models': odd head counts, widths and vocabularies that are no power of two, head sizes in
steps of 16."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from nano_vllm_cpp_b200.csrc import ops as o
    return o


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, rel, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    bound = rel * max(1e-6, float(want.abs().max()))
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: max error {err:.3g} > {bound:.3g}"


# ------------------------------------------------------------------------------- embedding, norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(dtype):
    o = ops()
    table = rnd(1000, 72, dtype=dtype)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    err = o.ErrorFlag(DEV)
    o.embedding(ids, table, out, err)
    err.check("embedding")
    assert torch.equal(out, table[ids.long()].float())
    bad = torch.tensor([3, 1000], dtype=torch.int32, device=DEV)
    o.embedding(bad, table, out[:2], err)
    with pytest.raises(o.KernelError, match="bad index"):
        err.check("embedding")


@pytest.mark.parametrize("H", [64, 200, 2048, 3000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(H, out_dtype):
    o = ops()
    x, br, w = rnd(7, H), rnd(7, H, seed=1), rnd(H, seed=2) + 1
    x0 = x.clone()
    out = torch.empty(7, H, dtype=out_dtype, device=DEV)
    out32 = torch.empty(7, H, device=DEV)
    o.add_rmsnorm(x, br, w, 1e-5, out, out32)
    s = (x0.double() + br.double())
    want = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + 1e-5) * w.double()
    close(x, s, 1e-7, "residual")
    close(out32, want, 1e-6, "norm f32")
    close(out, want, 1e-6 if out_dtype == torch.float32 else 2 ** -8, "norm out")
    y = x.clone()
    o.add_rmsnorm(y, None, w, 1e-5, out)        # no branch: x unchanged
    assert torch.equal(y, x)


# ------------------------------------------------------------------------------- plain product
@pytest.mark.parametrize("M,N,K", [(1, 5, 7), (3, 130, 100), (70, 64, 16), (129, 200, 333)])
@pytest.mark.parametrize("ta,tw", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                   (torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_gemm_plain(M, N, K, ta, tw):
    o = ops()
    a, w, b = rnd(M, K, dtype=ta), rnd(N, K, dtype=tw, seed=1), rnd(N, seed=2)
    out = torch.empty(M, N, device=DEV)
    o.gemm_plain(a, w, out, bias=b)
    close(out, a.double() @ w.double().T + b.double(), 2e-6, "gemm")
    w2 = rnd(2 * N, K, dtype=tw, seed=3)
    o.gemm_plain(a, w2, out, swiglu=True)
    g, u = a.double() @ w2[:N].double().T, a.double() @ w2[N:].double().T
    close(out, g / (1 + torch.exp(-g)) * u, 2e-6, "swiglu")
    rows = torch.randint(0, M, (9,), dtype=torch.int32).to(DEV)
    out9 = torch.empty(9, N, device=DEV)
    o.gemm_plain(a, w, out9, a_rows=rows)
    close(out9, a[rows.long()].double() @ w.double().T, 2e-6, "gather")


def test_gemm_plain_rows_do_not_depend_on_the_batch():
    o = ops()
    a, w = rnd(100, 300), rnd(77, 300, seed=1)
    full = torch.empty(100, 77, device=DEV)
    o.gemm_plain(a, w, full)
    one = torch.empty(1, 77, device=DEV)
    for r in (0, 63, 64, 99):
        o.gemm_plain(a[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])         # bit for bit


# ------------------------------------------------------------------------------- tensor-core product
def tc_case(M, N, K, swiglu, bias, out_dtype, splits=None, seed=0):
    o = ops()
    a = rnd(M, K, dtype=torch.bfloat16, seed=seed)
    w = rnd(2 * N if swiglu else N, K, dtype=torch.bfloat16, scale=0.5, seed=seed + 1)
    b = rnd(N, seed=seed + 2) if bias else None
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
    assert o.gemm_fast_usable(a, w, out, bias=b, swiglu=swiglu)
    err = o.ErrorFlag(DEV)
    o.gemm_fast(a, w, out, bias=b, swiglu=swiglu, err=err, splits=splits)
    err.check("tc_gemm")
    if swiglu:
        g, u = a.double() @ w[:N].double().T, a.double() @ w[N:].double().T
        want = g / (1 + torch.exp(-g)) * u
    else:
        want = a.double() @ w.double().T
    if b is not None:
        want = want + b.double()
    close(out, want, 2e-5 if out_dtype == torch.float32 else 2 ** -8, f"tc {M}x{N}x{K} swiglu={swiglu}")
    # and against the plain kernel on the same operands
    ref = torch.empty(M, N, dtype=torch.float32, device=DEV)
    o.gemm_plain(a, w, ref, bias=b, swiglu=swiglu)
    close(out, ref, 2e-5 if out_dtype == torch.float32 else 2 ** -8, "tc vs plain")


def test_tc_gemm_smallest():
    tc_case(1, 128, 64, False, False, torch.float32)


@pytest.mark.parametrize("M,N,K", [(5, 200, 72), (16, 256, 512), (17, 130, 1000), (100, 384, 264), (300, 136, 2048),
                                   (513, 640, 136)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_tc_gemm_shapes(M, N, K, swiglu):
    tc_case(M, N, K, swiglu, True, torch.float32)
    tc_case(M, N, K, swiglu, False, torch.bfloat16, seed=5)


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_tc_gemm_split_k(splits):
    tc_case(8, 256, 2048, False, True, torch.float32, splits=splits)
    tc_case(3, 200, 1160, True, False, torch.bfloat16, splits=splits)


@pytest.mark.parametrize("T,E,K", [(5, 6, 3), (64, 8, 2), (300, 60, 4), (1, 60, 4)])
def test_tc_gemm_grouped(T, E, K):
    """Both grouped products of an expert layer against the plain grouped kernel and float64."""
    o = ops()
    H, I = 136, 72
    g = torch.Generator().manual_seed(T)
    x = rnd(T, H, dtype=torch.bfloat16)
    w1 = rnd(E, 2 * I, H, dtype=torch.bfloat16, scale=0.3, seed=1)
    w2 = rnd(E, H, I, dtype=torch.bfloat16, scale=0.3, seed=2)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    err = o.ErrorFlag(DEV)
    res = {}
    for fast in (True, False):
        tile = o.grouped_token_tile(T * K, E) if fast else o.gemm_plain_tile_m()
        al = o.MoeAlignment(T * K, E, tile, DEV)
        o.moe_align(idx, K, al, err)
        act = torch.empty(T * K, I, dtype=torch.bfloat16, device=DEV)
        y = torch.empty(T * K, H, dtype=torch.float32, device=DEV)
        if fast:
            o.gemm_fast_grouped(x, w1, act, al, a_rows=al.sorted_token, swiglu=True, err=err)
            o.gemm_fast_grouped(act, w2, y, al, err=err)
        else:
            o.gemm_plain(x, w1, act, a_rows=al.sorted_token, swiglu=True, M=T * K, tiles=al.tiles)
            o.gemm_plain(act, w2, y, M=T * K, tiles=al.tiles)
        err.check("grouped")
        res[fast] = y[al.pair_pos.long()].reshape(T, K, H)       # back to (row, k) order
    want = torch.zeros(T, K, H, dtype=torch.float64)
    for t in range(T):
        for k in range(K):
            e = int(idx[t, k])
            gg, uu = x[t].double().cpu() @ w1[e, :I].double().cpu().T, x[t].double().cpu() @ w1[e, I:].double().cpu().T
            a = (gg / (1 + torch.exp(-gg)) * uu).to(torch.bfloat16).double()
            want[t, k] = a @ w2[e].double().cpu().T
    close(res[False], want, 2e-2, "plain grouped")
    close(res[True], want, 2e-2, "tc grouped")
    close(res[True], res[False], 2e-2, "tc vs plain grouped")
