"""The plain implementation against the reference's own CPU forward pass (recorded output of
tools/ref_top5.cpp, see tests/golden/make_golden.py): top-5 ids and logits of the last position
and the routed experts and weights of the last token."""
import json
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402
import plain_model  # noqa: E402

with open(os.path.join(HERE, "golden", "ref_top5.json")) as f:
    GOLD = json.load(f)


@pytest.mark.parametrize("key", sorted(GOLD))
def test_plain_matches_reference_cpu(key, tmp_path):
    cname, _ = key.split("/")
    mdir = make_golden.tiny_model(make_golden.CASES[cname], str(tmp_path / cname))
    cfg, W = plain_model.read_folder(mdir)
    g = GOLD[key]
    logits = plain_model.forward(cfg, W, g["ids"])[-1]
    top = torch.topk(logits, 5)
    assert [int(i) for i in top.indices] == [t[0] for t in g["top5"]]
    for v, (_, want) in zip(top.values, g["top5"]):
        assert abs(float(v) - want) <= 6e-4          # the reference prints three decimals
    # routing of the last token in every sparse layer
    eps = cfg["rms_norm_eps"]
    x = plain_model.embedding(W["model.embed_tokens.weight"], g["ids"])
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = plain_model.rms_norm(x, W[p + "input_layernorm.weight"], eps)
        x = x + plain_model.attention_layer(h, W, p + "self_attn.", cfg, l, list(range(len(g["ids"]))))
        h = plain_model.rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)
        if plain_model.layer_is_sparse(cfg, l):
            idx, w = plain_model.route(h, W[p + "mlp.gate.weight"], cfg["num_experts_per_tok"], cfg["norm_topk_prob"])
            want = g["routes"][str(l)]
            assert [int(i) for i in idx[-1]] == [r[0] for r in want]
            for a, r in zip(w[-1], want):
                assert abs(float(a) - r[1]) <= 6e-5  # four decimals
            x = x + plain_model.sparse_mlp(h, W, p + "mlp.", cfg)
        else:
            assert str(l) not in g["routes"]
            x = x + plain_model.dense_mlp(h, W, p + "mlp.")


def test_plain_samplers_match_the_reference_cpu():
    """plain_model.sample and plain_model.sample_row against the recorded choices of the reference's own
    ``Sampler::sample`` and ``sample_row`` (include/nanovllm/sampler.hpp, see tests/golden/make_golden_sampler.py)
    for the same rows, parameters and uniform numbers."""
    import make_golden_sampler
    with open(os.path.join(HERE, "golden", "ref_sample_row.json")) as f:
        gold = json.load(f)
    rows = make_golden_sampler.rows()
    first = make_golden_sampler.first_rows()
    assert len(rows) == len(gold["sample_row"]) and len(first) == len(gold["sample"])
    for i, ((logits, temp, _), g) in enumerate(zip(first, gold["sample"])):      # Sampler::sample, sampler.hpp:10-34
        assert plain_model.sample(logits, temp, g["u"]) == g["token"], f"first sampler, case {i}"
    for i, ((logits, temp, top_p, pen, window, recent, _), g) in enumerate(zip(rows, gold["sample_row"])):
        got = plain_model.sample_row(logits, temp, top_p, g["u"], recent, pen, window)
        assert got == g["token"], f"case {i}: temperature {temp}, top_p {top_p}, penalty {pen}, window {window}"
