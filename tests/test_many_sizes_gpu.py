"""The engine against the plain implementation over a spread of configurations that the two tiny test models and
the benchmark shapes do not reach: head sizes from 16 to 256 in steps of 16, odd numbers of heads and of query heads
per kv head, widths and vocabularies that are no power of two (and widths that are no multiple of 32, which the
kernels for a handful of rows and the TMA-fed kernels refuse, so that the plain kernels take over), every expert
chosen, a single expert chosen, shared experts that are a whole number of expert widths, another number, or absent,
dense layers by either rule, windows that are no multiple of the page, pages of 32 tokens, no projection biases, tied
and untied heads.  Every configuration runs whole, with its last tokens one by one, in portions down to two tokens,
and mixed on a pool so small that pages are used again, in float32 and in bfloat16.
"""
import json
import os
import struct

import numpy as np
import pytest
import torch

import helpers
import plain_model
from helpers import Replay

pytestmark = pytest.mark.gpu


def cfg(**kw):
    base = dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=2, hidden_size=64,
                num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=8, num_experts_per_tok=2,
                moe_intermediate_size=32, shared_expert_intermediate_size=64, intermediate_size=96,
                decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=False, vocab_size=200, rope_theta=10000.0,
                rms_norm_eps=1e-6, max_position_embeddings=512, use_sliding_window=False, sliding_window=0,
                max_window_layers=0, tie_word_embeddings=False, qkv_bias=True)
    base.update(kw)
    return base


# name -> (config, page size)
CONFIGS = {
    "d16_one_kv_head": (cfg(num_attention_heads=5, num_key_value_heads=1, hidden_size=72, vocab_size=131), 16),
    "d32_every_expert": (cfg(head_dim=32, num_attention_heads=3, num_key_value_heads=3, num_experts=5,
                             num_experts_per_tok=5, norm_topk_prob=True, hidden_size=96, moe_intermediate_size=40,
                             shared_expert_intermediate_size=60), 16),
    "d48_one_expert_window20": (cfg(head_dim=48, num_attention_heads=6, num_key_value_heads=2, num_experts=3,
                                    num_experts_per_tok=1, use_sliding_window=True, sliding_window=20, hidden_size=104,
                                    shared_expert_intermediate_size=0, tie_word_embeddings=True, vocab_size=257), 16),
    "d64_seven_per_kv_head_pages32": (cfg(head_dim=64, num_attention_heads=7, num_key_value_heads=1, hidden_size=128,
                                          num_experts=16, num_experts_per_tok=4, moe_intermediate_size=64,
                                          shared_expert_intermediate_size=128, rope_theta=1e6, rms_norm_eps=1e-5), 32),
    "d80_dense_and_sparse": (cfg(head_dim=80, num_attention_heads=2, num_key_value_heads=2, hidden_size=160,
                                 num_hidden_layers=3, decoder_sparse_step=2, mlp_only_layers=[], intermediate_size=136,
                                 moe_intermediate_size=56, shared_expert_intermediate_size=56), 16),
    "d96_window33_second_layer": (cfg(head_dim=96, num_attention_heads=4, num_key_value_heads=4, hidden_size=192,
                                      use_sliding_window=True, sliding_window=33, max_window_layers=1,
                                      num_experts=7, num_experts_per_tok=3, norm_topk_prob=True), 16),
    "d112_no_bias": (cfg(head_dim=112, num_attention_heads=2, num_key_value_heads=1, hidden_size=200, qkv_bias=False,
                         moe_intermediate_size=24, shared_expert_intermediate_size=72, vocab_size=1000), 16),
    "d128_benchmark_like": (cfg(head_dim=128, num_attention_heads=4, num_key_value_heads=4, hidden_size=256,
                                num_experts=12, num_experts_per_tok=4, moe_intermediate_size=96,
                                shared_expert_intermediate_size=384, rope_theta=1e6), 16),
    "d128_grouped_window8": (cfg(head_dim=128, num_attention_heads=8, num_key_value_heads=2, hidden_size=224,
                                 use_sliding_window=True, sliding_window=8, num_experts=6, num_experts_per_tok=2,
                                 moe_intermediate_size=64, shared_expert_intermediate_size=96, mlp_only_layers=[0]), 16),
    "d256": (cfg(head_dim=256, num_attention_heads=2, num_key_value_heads=1, hidden_size=96, tie_word_embeddings=True,
                 vocab_size=50), 16),
    "d192_only_dense_layers": (cfg(head_dim=192, num_attention_heads=1, num_key_value_heads=1, hidden_size=64,
                                   num_experts=0, num_experts_per_tok=0, moe_intermediate_size=0,
                                   shared_expert_intermediate_size=0, intermediate_size=72), 16),
}


def bf16_bits(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write_model(c, out_dir, seed):
    """config.json + model.safetensors (BF16), names and shapes written out here from the configuration format."""
    H, V, D = c["hidden_size"], c["vocab_size"], c["head_dim"]
    q, kv = c["num_attention_heads"] * D, c["num_key_value_heads"] * D
    names = [("model.embed_tokens.weight", (V, H), "w")]
    for l in range(c["num_hidden_layers"]):
        p = f"model.layers.{l}."
        names += [(p + "input_layernorm.weight", (H,), "n"), (p + "post_attention_layernorm.weight", (H,), "n"),
                  (p + "self_attn.q_proj.weight", (q, H), "w"), (p + "self_attn.k_proj.weight", (kv, H), "w"),
                  (p + "self_attn.v_proj.weight", (kv, H), "w"), (p + "self_attn.o_proj.weight", (H, q), "w")]
        if c["qkv_bias"]:
            names += [(p + "self_attn.q_proj.bias", (q,), "w"), (p + "self_attn.k_proj.bias", (kv,), "w"),
                      (p + "self_attn.v_proj.bias", (kv,), "w")]
        if plain_model.layer_is_sparse(c, l):
            I, SI, E = c["moe_intermediate_size"], c["shared_expert_intermediate_size"], c["num_experts"]
            names.append((p + "mlp.gate.weight", (E, H), "w"))
            for e in range(E):
                names += [(f"{p}mlp.experts.{e}.gate_proj.weight", (I, H), "w"), (f"{p}mlp.experts.{e}.up_proj.weight", (I, H), "w"),
                          (f"{p}mlp.experts.{e}.down_proj.weight", (H, I), "w")]
            if SI > 0:
                names += [(p + "mlp.shared_expert.gate_proj.weight", (SI, H), "w"), (p + "mlp.shared_expert.up_proj.weight", (SI, H), "w"),
                          (p + "mlp.shared_expert.down_proj.weight", (H, SI), "w"), (p + "mlp.shared_expert_gate.weight", (1, H), "w")]
        else:
            I = c["intermediate_size"]
            names += [(p + "mlp.gate_proj.weight", (I, H), "w"), (p + "mlp.up_proj.weight", (I, H), "w"),
                      (p + "mlp.down_proj.weight", (H, I), "w")]
    names.append(("model.norm.weight", (H,), "n"))
    if not c["tie_word_embeddings"]:
        names.append(("lm_head.weight", (V, H), "w"))
    rs = np.random.RandomState(seed)
    header, blobs, off = {}, [], 0
    for name, shape, kind in names:
        z = rs.standard_normal(shape)
        raw = bf16_bits(z * 0.06 if kind == "w" else 1.0 + z * 0.1).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(c, f)
    return out_dir


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("many_sizes")
    return {name: write_model(c, str(root / name), seed=40 + i) for i, (name, (c, _)) in enumerate(CONFIGS.items())}


def ids_of(name, rid, n):
    rs = np.random.RandomState(sum(map(ord, name)) * 7 + ord(rid) * 31 + n)
    return [int(t) for t in rs.randint(0, CONFIGS[name][0]["vocab_size"], size=n)]


LENGTHS = {"a": 61, "b": 1, "c": 34, "d": 17, "e": 50}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_cut_at_many_sizes(name, dtype, folders):
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    c, page = CONFIGS[name]
    mdir = folders[name]
    ids = {r: ids_of(name, r, n) for r, n in LENGTHS.items()}
    runner = ModelRunner(mdir, dtype=dtype, page_size=page, max_tokens=160, max_requests=4)

    def check(rp, what, rids):
        for r in rids:
            rp.compare(r, ids[r], mdir, dtype, f"{name} {dtype} {what}")

    # whole
    rp = Replay(runner)
    for r in ("a", "b", "c"):
        rp.step([(r, ids[r], True)])
        check(rp, "whole", [r])
        rp.step([], end=[r])
    # the last tokens one by one, two requests side by side
    rp = Replay(runner)
    rp.step([("a", ids["a"][:41], True), ("d", ids["d"][:3], True)])
    for t in range(20):
        parts = [("a", ids["a"][41 + t:42 + t], True)]
        if 3 + t < 17:
            parts.append(("d", ids["d"][3 + t:4 + t], True))
        rp.step(parts)
    check(rp, "one by one", ["a", "d"])
    rp.step([], end=["a", "d"])
    # portions of changing size, down to two tokens
    rp = Replay(runner)
    at = 0
    for n in (7, 2, 16, 1, 3, 19, 2, 9, 2):
        rp.step([("a", ids["a"][at:at + n], True)])
        at += n
    assert at == 61
    check(rp, "portions", ["a"])
    rp.step([], end=["a"])
    # mixed: up to four live requests on 160 tokens of pool for 163 tokens in all (pages are used again)
    rp = Replay(runner)
    rp.step([("a", ids["a"][:30], True), ("b", ids["b"], True)], end=["b"])
    rp.step([("a", ids["a"][30:31], True), ("c", ids["c"][:20], True), ("d", ids["d"][:2], True)])
    rp.step([("a", ids["a"][31:60], True), ("c", ids["c"][20:21], True), ("d", ids["d"][2:], True)], end=["d"])
    rp.step([("a", ids["a"][60:], True), ("c", ids["c"][21:], True), ("e", ids["e"][:9], True)], end=["a", "c"])
    rp.step([("e", ids["e"][9:48], True)])
    rp.step([("e", ids["e"][48:49], True)])
    rp.step([("e", ids["e"][49:], True)], end=["e"])
    check(rp, "mixed", ["a", "b", "c", "d", "e"])
    for pool in runner.manager.pools:
        assert pool.num_free() == pool.num_pages


def test_sizes_that_no_kernel_takes_are_refused(tmp_path):
    """A head size that is no multiple of 16, or beyond 256, is an error at load time, not a wrong result."""
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    for D in (24, 272):
        c = cfg(head_dim=D, num_attention_heads=2, num_key_value_heads=1)
        mdir = write_model(c, str(tmp_path / f"d{D}"), seed=1)
        with pytest.raises(Exception, match="head_dim"):
            ModelRunner(mdir, dtype="bfloat16", max_tokens=64, max_requests=2)


def random_schedule(rng, lengths, page, pool_tokens, max_live=4):
    """Steps [(parts [(request, tokens)], ends)] that feed every request whole, in portions of random sizes (single
    tokens and pairs among them), with up to ``max_live`` requests live and never more tokens held (each request's
    count rounded up to whole pages) than the pool has."""
    left = dict(lengths)
    fed = {r: 0 for r in lengths}
    waiting, live, steps = list(lengths), [], []
    pages = lambda n: (n + page - 1) // page

    def reserved():                      # what the live requests will hold when they are whole
        return sum(pages(lengths[r]) for r in live) * page

    while waiting or live:
        while waiting and len(live) < max_live and rng.random() < 0.7:
            r = waiting[0]
            if reserved() + pages(lengths[r]) * page > pool_tokens:  # room for the whole request, so nobody gets stuck
                break
            live.append(waiting.pop(0))
        if not live:
            live.append(waiting.pop(0))
        parts, ends = [], []
        for r in list(live):
            if rng.random() < 0.25 and len(live) > 1:
                continue                                   # the request sits this step out
            n = min(left[r], rng.choice([1, 1, 2, 2, 3, 5, 7, 16, 17, 31, 64]))
            if left[r] - n == 1 and rng.random() < 0.5:
                n += 1
            parts.append((r, n))
        if not parts:
            continue
        for r, n in parts:
            fed[r] += n
            left[r] -= n
            if left[r] == 0:
                ends.append(r)
                live.remove(r)
        steps.append((parts, ends))
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["d16_one_kv_head", "d64_seven_per_kv_head_pages32", "d96_window33_second_layer",
                                  "d128_benchmark_like"])
def test_random_schedules(name, dtype, folders):
    """Five random ways of cutting and mixing six requests, on a pool that holds less than half of their tokens."""
    import random
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    c, page = CONFIGS[name]
    mdir = folders[name]
    lengths = {"a": 90, "b": 1, "c": 47, "d": 2, "e": 64, "f": 33}
    ids = {r: ids_of(name, r, n) for r, n in lengths.items()}
    pool = 224
    runner = ModelRunner(mdir, dtype=dtype, page_size=page, max_tokens=pool, max_requests=4)
    for seed in range(5):
        rng = random.Random(1000 * seed + len(name))
        order = list(lengths)
        rng.shuffle(order)
        steps = random_schedule(rng, {r: lengths[r] for r in order}, page, pool)
        rp = Replay(runner)
        at = {r: 0 for r in lengths}
        done = {}
        for parts, ends in steps:
            rp.step([(r, ids[r][at[r]:at[r] + n], True) for r, n in parts])
            for r, n in parts:
                at[r] += n
            for r in ends:
                rp.compare(r, ids[r], mdir, dtype, f"{name} {dtype} random schedule {seed}")
                done[r] = True
            rp.step([], end=ends)
        assert sorted(done) == sorted(lengths)
        for p in runner.manager.pools:
            assert p.num_free() == p.num_pages
