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


# ------------------------------------------------------------------------------- random weights
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,mean,std", [(1, 0.0, 0.02), (4099, 0.0, 0.05), (5_000_003, 0.0, 0.02), (3584, 1.0, 0.1)])
def test_random_fill_has_the_bits_of_the_host_rule(dtype, n, mean, std):
    """A tensor drawn on the device equals the one numpy draws on the host, bit for bit."""
    from nano_vllm_cpp_b200.weights.random_values import host_values, tensor_key
    key = tensor_key(9, f"some.tensor.{n}")
    out = torch.empty(n, dtype=dtype, device=DEV)
    ops().random_fill(out, key, mean, std)
    want = torch.from_numpy(host_values(key, n, mean, std)).to(dtype)
    assert torch.equal(out.cpu(), want)


def test_random_source_draws_the_same_model_on_both_devices():
    from nano_vllm_cpp_b200.config.registry import get_architecture
    from nano_vllm_cpp_b200.parts import Model
    from nano_vllm_cpp_b200.weights import RandomSource
    import helpers
    arch = get_architecture("Qwen2MoeForCausalLM")
    specs = Model(arch.build_model(arch.config_from_dict(helpers.CASES["B"]["config"]))).tensor_specs()
    host = RandomSource(specs, 3, 0.05, 0.1, "cpu", torch.bfloat16)
    dev = RandomSource(specs, 3, 0.05, 0.1, DEV, torch.bfloat16)
    for name in specs:
        assert torch.equal(dev.stored(name).cpu(), host.stored(name)), name


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
    # the branch as a sum not yet taken: gate * dense + sum_r weight[t, r] * rows[index[t, r]]
    for R, with_dense in ((3, True), (8, False), (1, True)):
        rows, weight = rnd(50, H, seed=3), rnd(7, R, seed=4)
        index = torch.randint(0, 50, (7, R), generator=torch.Generator().manual_seed(5), dtype=torch.int32).to(DEV)
        dense, gate = (rnd(7, H, seed=6), rnd(7, 3, seed=7)) if with_dense else (None, None)
        x1 = x0.clone()
        o.add_rmsnorm(x1, None, w, 1e-5, out, out32, mix=(rows, index, weight, dense, None if gate is None else gate[:, 1:2]))
        s = (weight.double()[:, :, None] * rows.double()[index.long()]).sum(1)
        if with_dense:
            s = s + torch.sigmoid(gate[:, 1].double())[:, None] * dense.double()
        s = s + x0.double()
        want = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + 1e-5) * w.double()
        close(x1, s, 2e-6, "residual after mix")
        close(out32, want, 2e-6, "norm after mix")


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


def test_tc_gemm_short_last_wave():
    """More tiles than CTAs and a last wave for less than half of them: its tiles are cut into token parts."""
    tc_case(2048, 6144, 264, False, True, torch.bfloat16)        # 192 tiles of 256 x 256 on 148 CTAs
    tc_case(1024, 5120, 136, False, False, torch.float32)        # 160 tiles: twelve left over, four parts each


@pytest.mark.parametrize("splits", [2, 3, 7])
def test_tc_gemm_split_k(splits):
    tc_case(8, 256, 2048, False, True, torch.float32, splits=splits)
    tc_case(3, 200, 1160, True, False, torch.bfloat16, splits=splits)


@pytest.mark.parametrize("T,E,K,H,I", [(5, 6, 3, 136, 72), (64, 8, 2, 136, 72), (300, 60, 4, 136, 72), (1, 60, 4, 136, 72),
                                       (700, 6, 3, 136, 72), (130, 3, 2, 136, 72),
                                       (1, 9, 4, 1032, 520), (4, 5, 3, 2048, 1408)])     # few pairs, long K: K is split
def test_tc_gemm_grouped(T, E, K, H, I):
    """Both grouped products of an expert layer against the plain grouped kernel and float64."""
    o = ops()
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
            # the same with tiles taken from a counter (twice: the counter sets itself back), also on a capped grid
            counter = torch.zeros(2, dtype=torch.int32, device=DEV)
            for cap in (0, 3):
                act2, y2 = torch.full_like(act, float("nan")), torch.full_like(y, float("nan"))
                o.gemm_fast_grouped(x, w1, act2, al, a_rows=al.sorted_token, swiglu=True, err=err, counter=counter[0:1],
                                    max_ctas=cap)
                o.gemm_fast_grouped(act2, w2, y2, al, err=err, tiles_ready=True, counter=counter[1:2], max_ctas=cap)
                err.check("grouped, by counter")
                assert counter.tolist() == [0, 0]
                if T * K <= o.GROUPED_SPLIT_MAX_PAIRS and H >= 512:     # the product by position split K: other sums
                    close(act2, act, 1e-2, "by counter vs split K")
                    close(y2, y, 1e-2, "by counter vs split K")
                else:
                    assert torch.equal(act2, act) and torch.equal(y2, y)
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


@pytest.mark.parametrize("T,E,K,C", [(5, 6, 3, 2), (1, 60, 4, 4), (40, 7, 2, 3), (64, 9, 1, 1)])
def test_always_on_experts_run_before_the_routing(T, E, K, C):
    """C experts that every row visits sit in row order behind the routed pairs and get no tiles from the routing;
    a fixed tile list runs them straight from the unsorted rows (here on a second stream, before the routing is
    launched), the routed experts follow, and both fill the same buffers.  Against float64."""
    o = ops()
    H, I, KT = 136, 72, K + C
    x = rnd(T, H, dtype=torch.bfloat16)
    w1 = rnd(E + C, 2 * I, H, dtype=torch.bfloat16, scale=0.3, seed=1)
    w2 = rnd(E + C, H, I, dtype=torch.bfloat16, scale=0.3, seed=2)
    logits, gate = rnd(T, E, scale=2.0, seed=3), rnd(T, seed=4)
    err = o.ErrorFlag(DEV)
    al = o.MoeAlignment(T * KT, E + C, o.grouped_token_tile(T * KT, E + C), DEV)
    st = o.StaticTiles(T, K, E, C, DEV)
    idx = torch.empty(T, KT, dtype=torch.int32, device=DEV)
    score = torch.empty(T, KT, device=DEV)
    act = torch.full((T * KT, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    y = torch.full((T * KT, H), float("nan"), dtype=torch.float32, device=DEV)
    main, side = torch.cuda.current_stream(), torch.cuda.Stream()
    fork, join = torch.cuda.Event(), torch.cuda.Event()
    fork.record(main)
    side.wait_event(fork)
    with torch.cuda.stream(side):
        o.gemm_fast_grouped(x, w1, act, al, swiglu=True, err=err, tiles=st, tiles_ready=True, x_rows=st.x_rows)
        o.gemm_fast_grouped(act, w2, y, al, err=err, tiles=st, tiles_ready=True)
        join.record(side)
    o.moe_route_small(logits, K, False, C, gate, idx, score, al, err, static=True)
    xs = o.permute_rows(x, al.sorted_token, T * K)
    o.gemm_fast_grouped(xs, w1, act, al, swiglu=True, err=err, tiles_ready=True)
    o.gemm_fast_grouped(act, w2, y, al, err=err, tiles_ready=True)
    main.wait_event(join)
    err.check("grouped")
    pos = al.pair_pos.cpu().view(T, KT)
    for t in range(T):
        assert idx[t, K:].tolist() == list(range(E, E + C))
        assert pos[t, K:].tolist() == [T * K + c * T + t for c in range(C)]
        assert all(0 <= int(q) < T * K for q in pos[t, :K])
    nt = int(al.num_tiles)
    assert all(int(e) < E for e in al.tile_expert[:nt])
    assert sum(int(r) for r in al.tile_rows[:nt]) == T * K
    got = y[al.pair_pos.long()].reshape(T, KT, H)
    want = torch.zeros(T, KT, H, dtype=torch.float64)
    xd, w1d, w2d = x.double().cpu(), w1.double().cpu(), w2.double().cpu()
    for t in range(T):
        for k in range(KT):
            e = int(idx[t, k])
            gg, uu = xd[t] @ w1d[e, :I].T, xd[t] @ w1d[e, I:].T
            want[t, k] = (gg / (1 + torch.exp(-gg)) * uu).to(torch.bfloat16).double() @ w2d[e].T
    close(got, want, 2e-2, "always-on and routed experts")


# ------------------------------------------------------------------------------- small products, router
# ------------------------------------------------------------------------------- products of a handful of rows
@pytest.mark.parametrize("R,N,K", [(1, 5, 32), (1, 6144, 2048), (2, 130, 288), (3, 2048, 1408), (5, 61, 544), (8, 200, 3584),
                                   (8, 4, 64), (7, 1000, 96), (4, 33, 20480), (9, 130, 288), (16, 2048, 2048), (17, 61, 544),
                                   (31, 6144, 2048), (32, 40, 96), (25, 200, 3584)])
@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_skinny_gemm_dense(R, N, K, swiglu, out_dtype):
    o = ops()
    if swiglu and R > 8:                                                  # SwiGLU: eight rows at most, refused beyond
        a = rnd(R, K, dtype=torch.bfloat16, seed=1)
        w = rnd(2 * N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
        assert not o.skinny_usable(a, w, R, True)
        with pytest.raises(o.KernelError):
            o.skinny_gemm(a, w, torch.empty((R, N), dtype=out_dtype, device=DEV), swiglu=True)
        return
    a = rnd(R + 2, K, dtype=torch.bfloat16, seed=1)                       # two more rows than are used
    w = rnd(2 * N if swiglu else N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    bias = None if swiglu else rnd(N, seed=3)
    out = torch.full((R + 2, N), float("nan"), dtype=out_dtype, device=DEV)
    err = o.ErrorFlag(DEV)
    o.skinny_gemm(a, w, out, bias=bias, swiglu=swiglu, rows=R, err=err)
    err.check("skinny")
    y = a[:R].double() @ w.double().T
    want = (y[:, :N] / (1 + torch.exp(-y[:, :N])) * y[:, N:]) if swiglu else y + bias.double()
    close(out[:R], want, 2e-5 if out_dtype == torch.float32 else 1e-2, "skinny dense")
    assert bool(torch.isnan(out[R:].float()).all())                       # rows beyond R are not touched
    # a row's result does not depend on how many rows ride along
    if R > 1:
        one = torch.empty((1, N), dtype=out_dtype, device=DEV)
        o.skinny_gemm(a[R - 1:R], w, one, bias=bias, swiglu=swiglu, rows=1)
        assert torch.equal(one[0], out[R - 1])
    # sizes it does not take are refused, not guessed at
    assert not o.skinny_usable(a[:, :K - 8], w[:, :K - 8].contiguous(), R) and not o.skinny_usable(a, w, 33)
    assert not o.skinny_usable(a, w, 9, True)
    with pytest.raises(o.KernelError):
        o.skinny_gemm(a[:, :K - 8].contiguous(), w[:, :K - 8].contiguous(), out, swiglu=swiglu, rows=R)


@pytest.mark.parametrize("T,N,K", [(1, 1, 64), (8, 60, 2048), (33, 7, 100), (5, 64, 3000), (1030, 61, 520), (1025, 9, 2050),
                                   (300, 61, 2048), (600, 61, 1032), (2100, 5, 264), (520, 65, 3584), (9, 3, 3076)])
@pytest.mark.parametrize("tw", [torch.float32, torch.bfloat16])
def test_rowdot(T, N, K, tw):
    o = ops()
    a, w = rnd(T, K), rnd(N, K, dtype=tw, seed=1)
    out = torch.empty(T, N, device=DEV)
    o.rowdot(a, w, out)
    close(out, a.double() @ w.double().T, 2e-6, "rowdot")
    wide = torch.empty(T, N, device=DEV)
    o.rowdot(a, w, wide, wide=True)                  # the many-rows kernel: same values up to rounding
    close(wide, a.double() @ w.double().T, 2e-6, "rowdot wide")
    if T >= 4:                                       # ... and a row's value does not depend on how many rows a block takes
        part = torch.empty(T // 4, N, device=DEV)
        o.rowdot(a[:T // 4].contiguous(), w, part, wide=True)
        assert torch.equal(part, wide[:T // 4])
    one = torch.empty(1, N, device=DEV)
    o.rowdot(a[T - 1:T].contiguous(), w, one)
    assert torch.equal(one[0], out[T - 1])          # a row does not depend on the batch


@pytest.mark.parametrize("T,E,K,renorm", [(9, 60, 4, False), (4, 6, 3, True), (130, 8, 2, True), (3, 100, 8, False)])
def test_router_topk(T, E, K, renorm):
    o = ops()
    logits = rnd(T, E, scale=2.0)
    logits[0, :] = 0.5                                # an exact tie: the lowest indices win
    idx = torch.empty(T, K, dtype=torch.int32, device=DEV)
    sc = torch.empty(T, K, device=DEV)
    o.router_topk(logits, K, renorm, idx, sc)
    p = torch.softmax(logits.double(), -1).cpu()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(p[t, e]), e))[:K]
        assert idx[t].tolist() == order
        w = p[t, order]
        if renorm:
            w = w / w.sum()
        close(sc[t], w, 1e-6, "router weights")
    assert idx[0].tolist() == list(range(K))


def test_moe_align_and_combine():
    o = ops()
    T, K, E, H = 37, 3, 10, 72
    g = torch.Generator().manual_seed(3)
    idx = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).to(torch.int32).to(DEV)
    err = o.ErrorFlag(DEV)
    al = o.MoeAlignment(T * K, E, 16, DEV)
    o.moe_align(idx, K, al, err)
    err.check("align")
    counts = torch.bincount(idx.flatten().long().cpu(), minlength=E)
    assert al.counts.cpu().tolist() == counts.tolist()
    assert al.offsets.cpu().tolist() == [0] + torch.cumsum(counts, 0).tolist()
    pos = al.pair_pos.cpu().long()
    assert sorted(pos.tolist()) == list(range(T * K))                 # a permutation
    assert al.sorted_token.cpu()[pos].tolist() == [i // K for i in range(T * K)]
    off = al.offsets.cpu()
    for i in range(T * K):                                            # every pair sits in its expert's segment
        e = int(idx.flatten()[i])
        assert off[e] <= pos[i] < off[e + 1]
    nt = int(al.num_tiles)
    assert nt == sum((int(c) + 15) // 16 for c in counts)
    covered = []
    for i in range(nt):
        e, r0, r = int(al.tile_expert[i]), int(al.tile_row0[i]), int(al.tile_rows[i])
        assert off[e] <= r0 and r0 + r <= off[e + 1] and 1 <= r <= 16
        covered += list(range(r0, r0 + r))
    assert sorted(covered) == list(range(T * K))
    y, score, sh, gl = rnd(T * K, H), rnd(T, K, seed=1).abs(), rnd(T, H, seed=2), rnd(T, seed=3)
    out = torch.empty(T, H, device=DEV)
    o.moe_combine(y, al.pair_pos, score, sh, gl, out)
    want = torch.sigmoid(gl.double())[:, None] * sh.double()
    yy = y.double()[al.pair_pos.long()].reshape(T, K, H)
    want = want + (score.double()[:, :, None] * yy).sum(1)
    close(out, want, 2e-6, "combine")
    o.moe_combine(y, al.pair_pos, score, None, None, out)
    close(out, (score.double()[:, :, None] * yy).sum(1), 2e-6, "combine without shared expert")
    # the last experts' tiles spread through the list: the same tiles in another order
    def tiles(a):
        m = int(a.num_tiles)
        return [(int(a.tile_expert[i]), int(a.tile_row0[i]), int(a.tile_rows[i])) for i in range(m)]
    plain_order = tiles(al)
    o.moe_align(idx, K, al, err, spread_last=3)
    err.check("align")
    spread = tiles(al)
    assert sorted(spread) == sorted(plain_order) and spread != plain_order
    tail = [i for i, t3 in enumerate(spread) if t3[0] >= E - 3]
    others = [t3 for t3 in spread if t3[0] < E - 3]
    assert others == [t3 for t3 in plain_order if t3[0] < E - 3]          # each kind keeps its own order
    assert tail[0] < len(spread) // 2 and all(b - a >= 2 for a, b in zip(tail, tail[1:])) or len(tail) * 2 > len(spread)
    bad = idx.clone()
    bad[5, 1] = E
    o.moe_align(bad, K, al, err)
    with pytest.raises(o.KernelError):
        err.check("align")


# ------------------------------------------------------------------------------- rotary + cache write, attention
def paged_setup(lens, Hkv, D, page, dtype, seed=0, shuffle=True):
    """Random keys/values for requests of the given lengths, scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum((n + page - 1) // page for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    max_blocks = max((n + page - 1) // page for n in lens) + 1
    bt = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    kc = torch.zeros(n_pages, Hkv, page, D, dtype=dtype)
    vc = torch.zeros_like(kc)
    ks, vs = [], []
    for i, n in enumerate(lens):
        k = (torch.randn(n, Hkv, D, generator=g)).to(dtype)
        v = (torch.randn(n, Hkv, D, generator=g)).to(dtype)
        ks.append(k), vs.append(v)
        for b in range((n + page - 1) // page):
            p = perm.pop()
            bt[i, b] = p
            seg = slice(b * page, min(n, (b + 1) * page))
            kc[p, :, :seg.stop - seg.start] = k[seg].transpose(0, 1)
            vc[p, :, :seg.stop - seg.start] = v[seg].transpose(0, 1)
    return kc.to(DEV), vc.to(DEV), bt.to(DEV), ks, vs


def attention_reference(q, k, v, pos, scale, window):
    """q: [Hq, D] at position pos; k, v: [n, Hkv, D] -> [Hq, D] in float64."""
    Hq, Hkv = q.shape[0], k.shape[1]
    lo = max(0, pos + 1 - window) if window > 0 else 0
    out = torch.zeros(Hq, q.shape[1], dtype=torch.float64)
    for h in range(Hq):
        kh = h // (Hq // Hkv)
        s = (k[lo:pos + 1, kh].double() @ q[h].double()) * scale
        out[h] = torch.softmax(s, 0) @ v[lo:pos + 1, kh].double()
    return out


@pytest.mark.parametrize("Hq,Hkv,D,page", [(3, 1, 32, 16), (4, 4, 16, 16), (6, 2, 48, 32), (14, 2, 128, 16), (2, 1, 256, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 20])
def test_attention_plain_and_decode(Hq, Hkv, D, page, dtype, window):
    o = ops()
    lens = [1, 16, 17, 200, 333]
    kc, vc, bt, ks, vs = paged_setup(lens, Hkv, D, page, dtype, seed=D)
    T = len(lens)
    width = (Hq + 2 * Hkv) * D
    qkv = rnd(T, width, dtype=dtype, seed=7)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    row_entry = torch.arange(T, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    want = torch.stack([attention_reference(qkv[i, :Hq * D].reshape(Hq, D).cpu(), ks[i], vs[i], lens[i] - 1, scale, window)
                        for i in range(T)]).reshape(T, Hq * D)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    out = torch.empty(T, Hq * D, dtype=dtype, device=DEV)
    o.paged_attention_plain(qkv, kc, vc, bt, row_entry, pos, scale, window, out, Hq, Hkv, D)
    close(out, want, tol, "plain attention")
    out2 = torch.full_like(out, float("nan"))
    o.attention_decode(qkv, kc, vc, bt, row_entry, pos, scale, window, out2, Hq, Hkv, D, max(lens))
    close(out2, want, tol, "decode attention")
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)        # a subset of the rows, in another order
    out3 = torch.zeros_like(out)
    o.attention_decode(qkv, kc, vc, bt, row_entry, pos, scale, window, out3, Hq, Hkv, D, 4096, rows=rows)
    close(out3[[0, 3]], want[[0, 3]], tol, "decode attention on a row subset")
    assert float(out3[[1, 2, 4]].abs().max()) == 0.0


@pytest.mark.parametrize("D,window", [(128, 0), (64, 6000), (128, 70)])
def test_attention_decode_long_context(D, window):
    """Contexts of tens of thousands of keys (more splits, more pages than the kernel caches per block) beside
    a short one, grouped queries, against float64."""
    o = ops()
    Hq, Hkv, page = 8, 2, 16
    lens = [20000, 5, 33000]
    kc, vc, bt, ks, vs = paged_setup(lens, Hkv, D, page, torch.bfloat16, seed=D + window)
    T = len(lens)
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, seed=9)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    row_entry = torch.arange(T, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    want = torch.stack([attention_reference(qkv[i, :Hq * D].reshape(Hq, D).cpu(), ks[i], vs[i], lens[i] - 1, scale, window)
                        for i in range(T)]).reshape(T, Hq * D)
    out = torch.full((T, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = o.ErrorFlag(DEV)
    o.attention_decode(qkv, kc, vc, bt, row_entry, pos, scale, window, out, Hq, Hkv, D, max(lens), err=err)
    err.check("decode attention")
    close(out, want, 1.5e-2, "decode attention, long context")


@pytest.mark.parametrize("kernel", ["plain", "decode"])
def test_attention_finds_one_far_key(kernel):
    """Among 700 keys one far key matches the query; its value must dominate the output.  With a window
    that excludes it, it must not."""
    o = ops()
    Hq = Hkv = 2
    D, page, n, far = 64, 16, 700, 37
    kc, vc, bt, ks, vs = paged_setup([n], Hkv, D, page, torch.bfloat16, seed=1)
    q = torch.zeros(1, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16)
    key = ks[0][far, 1].float()
    q[0, D:2 * D] = (key / key.norm() * 40).to(torch.bfloat16)        # head 1 looks for that key
    q = q.to(DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    ent = torch.zeros(1, dtype=torch.int32, device=DEV)
    for window, hit in ((0, True), (n - far, True), (n - far - 1, False)):
        out = torch.empty(1, Hq * D, dtype=torch.bfloat16, device=DEV)
        if kernel == "plain":
            o.paged_attention_plain(q, kc, vc, bt, ent, pos, 1.0, window, out, Hq, Hkv, D)
        else:
            o.attention_decode(q, kc, vc, bt, ent, pos, 1.0, window, out, Hq, Hkv, D, n)
        want = attention_reference(q[0, :Hq * D].reshape(Hq, D).cpu(), ks[0], vs[0], n - 1, 1.0, window)
        close(out[0], want.reshape(-1), 1.5e-2, f"window {window}")
        near = float((out[0, D:].float().cpu() - vs[0][far, 1].float()).abs().max())
        assert (near < 0.1) == hit


@pytest.mark.parametrize("Hq,Hkv,D,rot", [(3, 1, 32, 32), (4, 2, 16, 16), (2, 2, 48, 32), (2, 1, 128, 128)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_store(Hq, Hkv, D, rot, dtype):
    o = ops()
    page, T = 16, 6
    positions = [0, 1, 15, 16, 100, 4095]
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=dtype)
    orig = qkv.clone()
    inv = torch.tensor([1.0 / (10000.0 ** (2.0 * i / rot)) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV)
    n_pages = 4096 // page + 1
    kc = torch.zeros(n_pages, Hkv, page, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    bt = torch.arange(n_pages, dtype=torch.int32).flip(0).reshape(1, -1).to(DEV).contiguous()   # page i -> n_pages-1-i
    ent = torch.zeros(T, dtype=torch.int32, device=DEV)
    err = o.ErrorFlag(DEV)
    o.rope_store(qkv, torch.tensor(positions, dtype=torch.int32, device=DEV), inv, rot, kc, vc, bt, ent, Hq, Hkv, D,
                 True, err)
    err.check("rope")

    def rotate(x, p):
        x = x.double()
        ang = (torch.tensor(float(p), dtype=torch.float32) * inv.cpu()).double()
        c, s = torch.cos(ang), torch.sin(ang)
        x1, x2 = x[..., :rot // 2], x[..., rot // 2:rot]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rot:]], -1)

    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    for i, p in enumerate(positions):
        heads = orig[i].reshape(Hq + 2 * Hkv, D).cpu()
        close(qkv[i, :Hq * D].reshape(Hq, D), rotate(heads[:Hq], p), tol, "q")
        page_id = n_pages - 1 - p // page
        close(kc[page_id, :, p % page], rotate(heads[Hq:Hq + Hkv], p), tol, "k")
        assert torch.equal(vc[page_id, :, p % page].cpu(), heads[Hq + Hkv:])
    assert torch.equal(qkv[:, Hq * D:], orig[:, Hq * D:])           # k and v stay as they were in the buffer
    bt[0, 0] = -1                                                      # the page of position 4095 is missing
    o.rope_store(qkv, torch.tensor(positions, dtype=torch.int32, device=DEV), inv, rot, kc, vc, bt, ent, Hq, Hkv, D,
                 True, err)
    with pytest.raises(o.KernelError):
        err.check("rope")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_store_with_coordinates_per_pair(dtype):
    """Pairs turned by other numbers than the row's place in its sequence: every row has three coordinates and every
    pair names the one it is turned by; the cache slot still comes from the place in the sequence."""
    o = ops()
    Hq, Hkv, D, rot, page, T = 3, 1, 32, 24, 16, 5
    positions = [0, 3, 17, 40, 41]
    coords = torch.tensor([[0, 0, 0], [3, 1, 2], [17, 5, 0], [9, 7, 7], [40, 2, 300]], dtype=torch.int32)
    axis = torch.tensor([0, 0, 1, 2, 1, 2, 0, 1, 2, 2, 1, 0], dtype=torch.int32)          # rot / 2 = 12 pairs
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=dtype)
    orig = qkv.clone()
    inv = torch.tensor([1.0 / (50.0 ** (2.0 * i / rot)) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV)
    n_pages = 4
    kc = torch.zeros(n_pages, Hkv, page, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    bt = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=DEV)
    ent = torch.zeros(T, dtype=torch.int32, device=DEV)
    err = o.ErrorFlag(DEV)
    o.rope_store(qkv, torch.tensor(positions, dtype=torch.int32, device=DEV), inv, rot, kc, vc, bt, ent, Hq, Hkv, D,
                 True, err, rot_positions=coords.to(DEV), pair_axis=axis.to(DEV))
    err.check("rope")
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    for i, p in enumerate(positions):
        heads = orig[i].reshape(Hq + 2 * Hkv, D).cpu().double()
        ang = (coords[i][axis.long()].float() * inv.cpu()).double()
        c, sn = torch.cos(ang), torch.sin(ang)
        x1, x2 = heads[:, :rot // 2], heads[:, rot // 2:rot]
        want = torch.cat([x1 * c - x2 * sn, x2 * c + x1 * sn, heads[:, rot:]], -1)
        close(qkv[i, :Hq * D].reshape(Hq, D), want[:Hq], tol, "q")
        page_id = int(bt[0, p // page])
        close(kc[page_id, :, p % page], want[Hq:Hq + Hkv], tol, "k")
        assert torch.equal(vc[page_id, :, p % page].cpu().double(), heads[Hq + Hkv:])
    # one coordinate per row and no table of axes: the same as positions of their own
    a, b = orig.clone(), orig.clone()
    other = torch.tensor([7, 7, 0, 100, 3], dtype=torch.int32, device=DEV)
    o.rope_store(a, torch.tensor(positions, dtype=torch.int32, device=DEV), inv, rot, kc, vc, bt, ent, Hq, Hkv, D,
                 False, err, rot_positions=other)
    o.rope_store(b, other, inv, rot, kc, vc, bt, ent, Hq, Hkv, D, False, err)
    assert torch.equal(a, b)
    with pytest.raises(o.KernelError):
        o.rope_store(a, other, inv, rot, kc, vc, bt, ent, Hq, Hkv, D, False, err, pair_axis=axis.to(DEV))


@pytest.mark.parametrize("D,window,ctx,new", [(128, 0, 0, 1100), (64, 300, 500, 700), (128, 0, 16000, 900), (128, 5000, 0, 17000)])
def test_attention_prefill_tc_long(D, window, ctx, new):
    """Long portions on the tcgen05 kernel against the mma.sync kernel on the same cache: many row tiles, a
    window that gives early blocks of keys to nobody, and more pages than the kernel keeps in shared memory."""
    o = ops()
    Hq, Hkv, page = 2, 1, 16
    n = ctx + new
    kc, vc, bt, ks, vs = paged_setup([n], Hkv, D, page, torch.bfloat16, seed=3)
    qkv = rnd(new, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, seed=4)
    cu = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    p0 = torch.tensor([ctx], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    outs = []
    for kernel in ("auto", "mma"):
        out = torch.full((new, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        err = o.ErrorFlag(DEV)
        o.attention_prefill(qkv, kc, vc, bt, cu, p0, (new + 63) // 64, scale, window, out, Hq, Hkv, D, err=err,
                            kernel=kernel)
        err.check("prefill attention")
        outs.append(out)
    close(outs[0], outs[1], 1.5e-2, "tcgen05 vs mma.sync")
    # row by row, each with its own largest value as the scale: a row that averages thousands of keys is small
    # beside row 0, which sees one, and must not pass on the strength of that
    a, b = outs[0].double(), outs[1].double()
    scale_of_row = b.abs().max(dim=-1, keepdim=True).values.clamp_min(1e-6)
    worst = float(((a - b).abs() / scale_of_row).max())
    assert worst <= 4e-2, f"a row differs from the mma.sync kernel by {worst:.3g} of its own largest value"
    for r in (0, new // 2, new - 1):                     # and a few rows against float64
        want = attention_reference(qkv[r, :Hq * D].reshape(Hq, D).cpu(), ks[0], vs[0], ctx + r, scale, window)
        close(outs[0][r], want.reshape(-1), 1.5e-2, f"row {r}")


@pytest.mark.parametrize("kernel", ["auto", "mma"])
@pytest.mark.parametrize("where", ["window edge", "beyond the shared-memory table", "first page of a continued portion"])
def test_attention_prefill_finds_one_far_key(kernel, where):
    """One query row in the middle of a row tile matches one key among thousands; that key's value must dominate
    the row's output, on the tcgen05 kernel and on the mma.sync kernel: at the two sides of a window's edge, in a
    page beyond the first 1,024 entries of the block table (the part the kernel keeps in shared memory), and in the
    first page of a portion that continues a cached prefix."""
    o = ops()
    Hq = Hkv = 2
    D, page = 64, 16
    if where == "window edge":
        ctx, new, row, window = 600, 300, 170, 400           # the row sits at position 770 and sees keys 371..770
        fars = [(371, True), (370, False)]
    elif where == "beyond the shared-memory table":
        ctx, new, row, window = 16900, 200, 77, 0            # pages 1,024 and later hold keys from 16,384 on
        fars = [(16500, True), (16385, True)]
    else:
        ctx, new, row, window = 130, 200, 90, 0              # the portion starts in the middle of page 8
        fars = [(130, True), (128, True)]
    n = ctx + new
    kc, vc, bt, ks, vs = paged_setup([n], Hkv, D, page, torch.bfloat16, seed=5)
    cu = torch.tensor([0, new], dtype=torch.int32, device=DEV)
    p0 = torch.tensor([ctx], dtype=torch.int32, device=DEV)
    for far, hit in fars:
        qkv = rnd(new, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, seed=6)
        key = ks[0][far, 1].float()
        qkv[row, D:2 * D] = (key / key.norm() * 40).to(torch.bfloat16).to(DEV)      # head 1 of that row looks for the key
        out = torch.full((new, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        err = o.ErrorFlag(DEV)
        o.attention_prefill(qkv, kc, vc, bt, cu, p0, (new + 63) // 64, 1.0, window, out, Hq, Hkv, D, err=err, kernel=kernel)
        err.check("prefill attention")
        want = attention_reference(qkv[row, :Hq * D].reshape(Hq, D).cpu(), ks[0], vs[0], ctx + row, 1.0, window)
        close(out[row], want.reshape(-1), 1.5e-2, f"{where}: key {far}")
        near = float((out[row, D:].float().cpu() - vs[0][far, 1].float()).abs().max())
        assert (near < 0.1) == hit, f"{where}: key {far} should {'dominate' if hit else 'be out of sight'} ({near:.3g})"
        other = attention_reference(qkv[row - 1, :Hq * D].reshape(Hq, D).cpu(), ks[0], vs[0], ctx + row - 1, 1.0, window)
        close(out[row - 1], other.reshape(-1), 1.5e-2, f"{where}: the row before")


@pytest.mark.parametrize("D,page", [(64, 16), (128, 16), (48, 32)])
@pytest.mark.parametrize("window", [0, 50])
def test_mixed_step_sends_single_rows_and_portions_to_their_kernels(D, page, window):
    """A step that holds single rows beside portions: the prefill kernel skips entries of one row (min_rows = 2),
    the decode kernel takes exactly those rows; together they fill every row of the output and equal the plain
    kernel.  The single rows come first, last and in between."""
    o = ops()
    Hq, Hkv = 4, 2
    ctx_len = [300, 0, 75, 1000, 31, 5]
    new = [1, 70, 1, 150, 2, 1]
    lens = [c + n for c, n in zip(ctx_len, new)]
    kc, vc, bt, ks, vs = paged_setup(lens, Hkv, D, page, torch.bfloat16, seed=D + window)
    T = sum(new)
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, seed=12)
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    pos = torch.tensor([c + i for c, n in zip(ctx_len, new) for i in range(n)], dtype=torch.int32, device=DEV)
    row_entry = torch.tensor([e for e, n in enumerate(new) for _ in range(n)], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ref = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    o.paged_attention_plain(qkv, kc, vc, bt, row_entry, pos, scale, window, ref, Hq, Hkv, D)
    out = torch.full_like(ref, float("nan"))
    singles = torch.tensor([cu[e] for e, n in enumerate(new) if n == 1], dtype=torch.int32, device=DEV)
    err = o.ErrorFlag(DEV)
    o.attention_decode(qkv, kc, vc, bt, row_entry, pos, scale, window, out, Hq, Hkv, D, 1001, rows=singles, err=err)
    assert int(torch.isnan(out.float()).any(dim=-1).sum()) == T - 3          # only the three single rows are written
    tiles = sum((n + 63) // 64 for n in new if n >= 2)
    o.attention_prefill(qkv, kc, vc, bt, torch.tensor(cu, dtype=torch.int32, device=DEV),
                        torch.tensor(ctx_len, dtype=torch.int32, device=DEV), tiles, scale, window, out, Hq, Hkv, D,
                        err=err, min_rows=2)
    err.check("mixed step")
    close(out, ref, 1.5e-2, "decode rows + portions vs plain")
    a, b = out.double(), ref.double()
    worst = float(((a - b).abs() / b.abs().max(dim=-1, keepdim=True).values.clamp_min(1e-6)).max())
    assert worst <= 4e-2


@pytest.mark.parametrize("Hq,Hkv,D,page", [(3, 1, 32, 16), (4, 4, 16, 16), (6, 2, 48, 32), (4, 2, 128, 16), (2, 1, 256, 16),
                                           (5, 5, 80, 16), (3, 3, 64, 16), (6, 2, 64, 32), (2, 1, 128, 64), (7, 1, 64, 64),
                                           (2, 2, 128, 32)])
@pytest.mark.parametrize("window", [0, 20, 100])
def test_attention_prefill_against_plain(Hq, Hkv, D, page, window):
    """Portions of several requests in one batch: a whole prompt, a portion that continues a cached
    prefix, a single decode row, a two-row portion, a portion longer than two tiles."""
    o = ops()
    ctx_len = [0, 130, 75, 31, 5]        # tokens already in the cache
    new = [70, 40, 1, 2, 150]            # rows of this step
    lens = [c + n for c, n in zip(ctx_len, new)]
    kc, vc, bt, ks, vs = paged_setup(lens, Hkv, D, page, torch.bfloat16, seed=D + window)
    T = sum(new)
    qkv = rnd(T, (Hq + 2 * Hkv) * D, dtype=torch.bfloat16, seed=11)
    cu = [0]
    for n in new:
        cu.append(cu[-1] + n)
    pos = torch.tensor([c + i for c, n in zip(ctx_len, new) for i in range(n)], dtype=torch.int32, device=DEV)
    row_entry = torch.tensor([e for e, n in enumerate(new) for _ in range(n)], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    ref = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    o.paged_attention_plain(qkv, kc, vc, bt, row_entry, pos, scale, window, ref, Hq, Hkv, D)
    out = torch.full_like(ref, float("nan"))
    tiles = sum((n + 63) // 64 for n in new)
    o.attention_prefill(qkv, kc, vc, bt, torch.tensor(cu, dtype=torch.int32, device=DEV),
                        torch.tensor(ctx_len, dtype=torch.int32, device=DEV), tiles, scale, window, out, Hq, Hkv, D)
    close(out, ref, 1.5e-2, "prefill vs plain")
    # and a few rows against float64
    for r in (0, 69, 70, 109, 110, 112, T - 1):
        e = int(row_entry[r])
        want = attention_reference(qkv[r, :Hq * D].reshape(Hq, D).cpu(), ks[e], vs[e], int(pos[r]), scale, window)
        close(out[r], want.reshape(-1), 1.5e-2, f"row {r}")


def test_block_tables_are_put_together_on_the_device():
    """``sync_block_tables``: a step's tables come from the tables kept by state slot, after the rows that travel
    with the step have been taken in; what lies beyond an entry's pages is left alone."""
    from nano_vllm_cpp_b200.csrc import ops
    g = torch.Generator().manual_seed(3)
    slots, max_blocks = 7, 2100                   # more than one chunk of the kernel's walk along a table
    kept = torch.randint(0, 5000, (slots, max_blocks), generator=g, dtype=torch.int32)
    step = torch.full((slots, max_blocks), -7, dtype=torch.int32)
    entry_slot = torch.tensor([4, 0, 6, 2], dtype=torch.int32)
    lens = torch.tensor([2100, 3, 0, 1500], dtype=torch.int32)
    src = torch.tensor([1, -1, -1, 0], dtype=torch.int32)
    rows = torch.randint(5000, 9000, (2, max_blocks), generator=g, dtype=torch.int32)
    want_kept, want_step = kept.clone(), step.clone()
    for e in range(4):
        s, n = int(entry_slot[e]), int(lens[e])
        if src[e] >= 0:
            want_kept[s, :n] = rows[int(src[e]), :n]
        want_step[e, :n] = want_kept[s, :n]
    d = [t.to(DEV) for t in (src, lens, rows, entry_slot, kept, step)]
    ops.sync_block_tables(*d, 4)
    assert torch.equal(d[4].cpu(), want_kept) and torch.equal(d[5].cpu(), want_step)
    ops.sync_block_tables(*d, 4)                   # the same step again changes nothing
    assert torch.equal(d[4].cpu(), want_kept) and torch.equal(d[5].cpu(), want_step)
