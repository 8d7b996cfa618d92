"""The engine at the layer sizes of the benchmark shapes (two layers, a small vocabulary, random weights made on
the device): the float32 run must not depend on how a request is cut into steps, and the bfloat16 run on the
tensor-core kernels must agree with it within the bfloat16 tolerance of the other tests.

The tiny configurations of the other tests reach none of these sizes (sixty or sixty-four experts, a shared
expert of four or eight expert widths, widths of 2,048 and 3,584, seven query heads per kv head), and the plain
CPU implementation is too slow for them, so here the float32 run, which the tiny configurations hold to the
plain implementation, is the reference.

A bfloat16 run may rightly send a token to another expert than the float32 run does when the token sits on the
edge between two experts (its K-th and (K+1)-th router logits nearly equal): such a row then differs by more than
rounding.  With 64 experts that happens to a row in a hundred or so.  The test therefore reads the router's margins
from the float32 run and lets a row exceed the tolerance only if its margin is small in some layer, and only a
few rows in all.
"""
import json
import os

import pytest
import torch

from helpers import TOL, Replay, assert_close

EDGE_MARGIN = 0.03     # router logits (of order one) closer than this: the bfloat16 run may pick either expert
MAX_EDGE_ROWS = 3

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
N = 200            # tokens of the request
WANT = [0, 1, 15, 16, 17, 63, 64, 127, 128, 150] + list(range(N - 33, N))


def run(folder, dtype, cuts, seed):
    """Logits at the wanted positions of one request fed in portions of the given sizes."""
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    runner = ModelRunner(folder, dtype=dtype, max_tokens=1024, max_requests=4, random_seed=seed)
    ids = torch.randint(0, BASE["vocab_size"], (N,), generator=torch.Generator().manual_seed(11)).tolist()
    other = torch.randint(0, BASE["vocab_size"], (40,), generator=torch.Generator().manual_seed(12)).tolist()
    rp = Replay(runner)
    at = 0
    for k, n in enumerate(cuts):
        places = [w - at for w in WANT if at <= w < at + n]
        parts = [("a", ids[at:at + n], places)]
        if k % 2 == 1 and k // 2 < len(other):       # another request's tokens ride along in every second step
            parts.append(("b", other[k // 2:k // 2 + 1], []))
        rp.step(parts)
        at += n
    assert at == N
    rows = torch.stack([rp.logits[("a", w)] for w in WANT])
    runner.close("a")
    del rp, runner
    torch.cuda.empty_cache()
    return rows


def router_margins(folder, cuts, seed, monkeypatch):
    """The float32 run of the whole request with, per position, the smallest gap between the K-th and the
    (K+1)-th router logit over the layers."""
    from nano_vllm_cpp_b200.parts import feedforward
    seen = []
    inner = feedforward.small_linear

    def spy(ctx, h32, w):
        out = inner(ctx, h32, w)
        seen.append(out.detach().float().cpu())
        return out

    monkeypatch.setattr(feedforward, "small_linear", spy)
    rows = run(folder, "float32", cuts, seed)
    monkeypatch.undo()
    return rows, seen


def assert_close_but_for_edges(got, ref, margin_of_row, what):
    tol = TOL["bfloat16"]
    bound = tol["abs"] + tol["rel"] * float(ref.abs().max())
    err = (got.double() - ref.double()).abs().max(-1).values
    off = [i for i in range(len(err)) if float(err[i]) > bound]
    not_edge = [(i, float(err[i]), margin_of_row[i]) for i in off if margin_of_row[i] >= EDGE_MARGIN]
    assert not not_edge, f"{what}: rows (index, error, router margin) beyond {bound:.3g} that sit on no edge: {not_edge}"
    assert len(off) <= MAX_EDGE_ROWS, f"{what}: {len(off)} rows beyond {bound:.3g}"


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_benchmark_layer_sizes(shape, tmp_path, monkeypatch):
    cfg = SHAPES[shape]
    folder = str(tmp_path / shape)
    os.makedirs(folder)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    whole = [N]
    tail = [N - 32] + [1] * 32                                     # the last 32 tokens one by one
    pieces = [7, 64, 2, 33, 16, 1, 45]
    pieces += [N - sum(pieces) - 2, 2]                              # portions of changing size, down to two tokens
    ref, logits = router_margins(folder, whole, 5, monkeypatch)
    assert torch.isfinite(ref).all() and float(ref.abs().max()) > 0.05
    E, K = cfg["num_experts"], cfg["num_experts_per_tok"]
    logits = [x for x in logits if x.shape[1] >= E]                 # (the shared expert's gate may be a call of its own)
    assert len(logits) == cfg["num_hidden_layers"] and all(x.shape[0] == N for x in logits)
    margin = torch.full((N,), float("inf"))
    for x in logits:
        top = torch.sort(x[:, :E], dim=-1, descending=True).values
        margin = torch.minimum(margin, top[:, K - 1] - top[:, K])
    margin_of_row = [float(margin[w]) for w in WANT]
    for name, cuts in (("last 32 one by one", tail), ("portions", pieces)):
        assert_close(run(folder, "float32", cuts, seed=5), ref, "float32", f"{shape} float32 {name}")
    for name, cuts in (("whole", whole), ("last 32 one by one", tail), ("portions", pieces)):
        assert_close_but_for_edges(run(folder, "bfloat16", cuts, seed=5), ref, margin_of_row, f"{shape} bfloat16 {name}")
