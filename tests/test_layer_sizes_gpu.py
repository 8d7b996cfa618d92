"""The engine at the layer sizes of the benchmark shapes against the plain implementation.

Two layers of the Qwen1.5-MoE-A2.7B and of the Qwen2-57B-A14B sizes (sixty or sixty-four experts, a shared expert
of four or eight expert widths, widths of 2,048 and 3,584, seven query heads per kv head, head size 128), a small
vocabulary, random weights.  The weights are a function of (seed, tensor name, element index), so the plain
implementation gets exactly the model that the engine draws for itself: it takes each tensor, drawn by the same
rule, as float64 when it needs it and runs its formulas on the GPU in float64 (the tiny models' tests run the same
functions on the CPU).

Requests of 1 to 1,024 tokens are run whole, with the last 32 tokens one by one, in portions of changing size
down to two tokens, and mixed (up to four live requests, portions beside single rows, on a pool so small that
pages are used again).  Every position's logits are compared: float32 within 1e-5, and bit for bit between the
schedules; bfloat16 within the tolerance of the other tests.

A bfloat16 run may rightly send a token to another expert than the float64 run does when the token sits on the
edge between two experts (its K-th and (K+1)-th router logits nearly equal): such a row then differs by more than
rounding.  With 64 experts that happens to a row in a hundred or so.  A row may therefore exceed the tolerance
only if the plain implementation's router margin of that row is small in some layer (``helpers.EDGE_MARGIN``).
"""
import json
import os

import pytest
import torch

import plain_model
from helpers import TOL, Replay, EDGE_MARGIN, MAX_EDGE_SHARE

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=2, decoder_sparse_step=1,
            mlp_only_layers=[], norm_topk_prob=False, vocab_size=1000, rope_theta=1000000.0, rms_norm_eps=1e-6,
            max_position_embeddings=8192, use_sliding_window=False, tie_word_embeddings=False, qkv_bias=True)
SHAPES = {
    # Qwen1.5-MoE-A2.7B layer sizes
    "a2.7b": dict(BASE, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, head_dim=128, num_experts=60,
                  num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
                  intermediate_size=5632),
    # Qwen2-57B-A14B layer sizes
    "57b": dict(BASE, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128, num_experts=64,
                num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
                intermediate_size=18944),
}
SEED, STD, NORM_STD = 5, 0.02, 0.1
LENGTHS = {"a": 1024, "b": 1, "c": 200, "d": 77, "e": 333, "f": 16, "g": 64}
POOL_TOKENS = 1536      # a + c + d + e's start are live together; all seven need 1,715: pages are used again

# the mixed schedule: per step [(request, tokens)], then the requests that end after it
MIXED = [
    ([("a", 500), ("b", 1)], ["b"]),
    ([("a", 500), ("c", 100), ("d", 2)], []),
    ([("a", 23), ("c", 99), ("d", 68)], []),
    ([("a", 1), ("c", 1), ("d", 7), ("e", 50)], ["a", "c", "d"]),
    ([("e", 1), ("f", 16)], ["f"]),
    ([("e", 281), ("g", 62)], []),
    ([("e", 1), ("g", 2)], ["e", "g"]),
]


class DrawnWeights:
    """name -> float64 tensor on the GPU, drawn when asked for by the random-weights rule."""

    def __init__(self, cfg):
        from nano_vllm_cpp_b200.config.registry import get_architecture
        from nano_vllm_cpp_b200.parts import Model
        from nano_vllm_cpp_b200.weights import RandomSource
        arch = get_architecture(cfg["architectures"][0])
        self.specs = Model(arch.build_model(arch.config_from_dict(cfg))).tensor_specs()
        self.source = RandomSource(self.specs, SEED, STD, NORM_STD, "cuda", torch.bfloat16)

    def __contains__(self, name):
        return name in self.specs

    def __getitem__(self, name):
        return self.source.stored(name).double()


def request_ids(rid):
    g = torch.Generator().manual_seed(100 + ord(rid))
    return torch.randint(0, BASE["vocab_size"], (LENGTHS[rid],), generator=g).tolist()


def schedules():
    """name -> list of (parts [(request, tokens)], ends)."""
    whole = [([(r, n)], [r]) for r, n in LENGTHS.items()]
    tail = []
    for r, n in LENGTHS.items():
        head = max(n - 32, 1)
        tail.append(([(r, head)], []))
        tail += [([(r, 1)], []) for _ in range(n - head)]
        tail[-1] = (tail[-1][0], [r])
    portions = []
    sizes = [7, 64, 2, 33, 16, 1, 45, 128, 3, 2, 300, 2, 5]
    for r, n in LENGTHS.items():
        at, k = 0, 0
        while at < n:
            s = min(sizes[k % len(sizes)], n - at)
            if n - at - s == 1:          # never leave a single last token behind: the last portion has two
                s = n - at if s == 1 else s - 1
            portions.append(([(r, s)], []))
            at, k = at + s, k + 1
        portions[-1] = (portions[-1][0], [r])
    return {"whole": whole, "last 32 one by one": tail, "portions": portions, "mixed": MIXED}


def run_schedule(runner, steps):
    """All positions' logits of all requests: {request: float32 [n, V]}."""
    ids = {r: request_ids(r) for r in LENGTHS}
    at = {r: 0 for r in LENGTHS}
    rp = Replay(runner)
    out = {}
    for parts, ends in steps:
        entries = []
        for r, n in parts:
            entries.append((r, ids[r][at[r]:at[r] + n], True))
            at[r] += n
        rp.step(entries)
        for r in ends:
            assert at[r] == LENGTHS[r]
            out[r] = torch.stack([rp.logits[(r, p)] for p in range(LENGTHS[r])])
        rp.step([], end=ends)
    assert sorted(out) == sorted(LENGTHS)
    for pool in runner.manager.pools:
        assert pool.num_free() == pool.num_pages
    return out


@pytest.fixture(scope="module", params=sorted(SHAPES))
def shape(request, tmp_path_factory):
    """(name, config, folder, plain logits and router margins per request)."""
    cfg = SHAPES[request.param]
    folder = str(tmp_path_factory.mktemp(request.param))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    W = DrawnWeights(cfg)
    plain, margin = {}, {}
    for r in LENGTHS:
        ms = []
        plain[r] = plain_model.forward(cfg, W, request_ids(r), margins=ms).cpu()
        assert len(ms) == cfg["num_hidden_layers"]
        margin[r] = torch.stack(ms).min(dim=0).values
    del W
    torch.cuda.empty_cache()
    return request.param, cfg, folder, plain, margin


def make_runner(folder, dtype):
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, max_tokens=POOL_TOKENS, max_requests=4, max_model_len=1024,
                       random_seed=SEED, std=STD, norm_std=NORM_STD)


def test_float32_against_plain_and_bit_equal_between_schedules(shape):
    name, cfg, folder, plain, _ = shape
    runner = make_runner(folder, "float32")
    tol = TOL["float32"]
    first = None
    for sname, steps in schedules().items():
        got = run_schedule(runner, steps)
        for r in LENGTHS:
            want = plain[r]
            assert float(want.abs().max()) > 0.5
            bound = tol["abs"] + tol["rel"] * float(want.abs().max())
            err = float((got[r].double() - want).abs().max())
            assert err <= bound, f"{name} float32 {sname} request {r}: max error {err:.3g} > {bound:.3g}"
        if first is None:
            first = got
        else:
            for r in LENGTHS:
                assert torch.equal(got[r], first[r]), f"{name} float32: {sname} differs from whole in request {r}"
    del runner
    torch.cuda.empty_cache()


def test_bfloat16_against_plain(shape):
    name, cfg, folder, plain, margin = shape
    runner = make_runner(folder, "bfloat16")
    tol = TOL["bfloat16"]
    for sname, steps in schedules().items():
        got = run_schedule(runner, steps)
        edge_rows = rows = 0
        for r in LENGTHS:
            want = plain[r]
            bound = tol["abs"] + tol["rel"] * float(want.abs().max())
            err = (got[r].double() - want).abs().max(dim=-1).values
            off = torch.nonzero(err > bound).reshape(-1).tolist()
            not_edge = [(p, float(err[p]), float(margin[r][p])) for p in off if float(margin[r][p]) >= EDGE_MARGIN]
            assert not not_edge, (f"{name} bfloat16 {sname} request {r}: rows (position, error, router margin) beyond "
                                  f"{bound:.3g} that sit on no edge: {not_edge[:8]}")
            edge_rows += len(off)
            rows += LENGTHS[r]
        assert edge_rows <= MAX_EDGE_SHARE * rows, f"{name} bfloat16 {sname}: {edge_rows} of {rows} rows beyond the tolerance"
    del runner
    torch.cuda.empty_cache()
