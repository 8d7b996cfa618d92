"""Shared pieces of the tests: the two tiny configurations, model folders in temporary places,
plain-implementation logits, and a replay driver over the engine's step function."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402
import plain_model  # noqa: E402

CASES = dict(make_golden.CASES)
# A third configuration, for the kernels that only head sizes 64 and 128 reach (tensor-core attention for prompts
# and for decoding) inside the whole engine: grouped queries, a window on the second layer, a shared expert that
# is a whole number of expert widths (so that it runs as extra experts on the fast path), sizes no power of two.
CASES["C"] = dict(
    config=dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=2,
                hidden_size=136, num_attention_heads=4, num_key_value_heads=2, head_dim=64, num_experts=5,
                num_experts_per_tok=2, moe_intermediate_size=40, shared_expert_intermediate_size=80,
                intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True,
                vocab_size=300, rope_theta=10000.0, rms_norm_eps=1e-6, max_position_embeddings=512,
                use_sliding_window=True, sliding_window=48, max_window_layers=1, tie_word_embeddings=False,
                qkv_bias=True, hidden_act="silu"),
    seed=4, std=0.03, norm_std=0.1, prompts={})

# C without its window: one group of layers, so that requests can share pages of a common prefix, with the head size
# that the tensor-core attention kernels take.
CASES["D"] = dict(config=dict(CASES["C"]["config"], use_sliding_window=False), seed=6, std=0.03, norm_std=0.1, prompts={})
# A with weights four times as large: in A itself (weights N(0, 0.02), width 64) the branches of a layer are tiny
# beside the path from the embedding to the head, so a fault inside a layer could hide under the bfloat16 tolerance;
# here every layer's branch weighs as much as what it is added to.
CASES["A8"] = dict(config=dict(CASES["A"]["config"]), seed=8, std=0.08, norm_std=0.1, prompts={})

# Tolerances, fixed before the first GPU run.  float32: sums of at most a few hundred float32
# products against float64 -> 1e-5 absolute on logits of order one.  bfloat16: activations are
# rounded to 8 bits of mantissa (2^-9 relative) a few times per layer; over the layers of the
# tiny models that gives errors of the order of one percent of the largest logit.
TOL = {"float32": dict(abs=1e-5, rel=1e-5), "bfloat16": dict(abs=2e-2, rel=3e-2)}


def model_folder(case_name, tmp_path_factory_or_dir):
    d = tmp_path_factory_or_dir
    if hasattr(d, "mktemp"):
        d = str(d.mktemp(f"model_{case_name}"))
    return make_golden.tiny_model(CASES[case_name], os.path.join(str(d), case_name))


def prompt(case_name, n, salt=0):
    rs = np.random.RandomState(7000 + ord(case_name[0]) * 131 + n * 17 + salt)
    return [int(x) for x in rs.randint(0, CASES[case_name]["config"]["vocab_size"], size=n)]


# A bfloat16 run may rightly send a token to another expert than the float64 run does when the token sits on the
# edge between two experts: its K-th and (K+1)-th router logits closer than this fraction of the spread of its
# router logits (bfloat16 activations carry errors of about one percent).  Such a row then differs by more than
# rounding; the comparisons below let a bfloat16 row exceed the tolerance only if it is such a row, and only a few.
EDGE_MARGIN = 0.01
MAX_EDGE_SHARE = 0.1        # (with a dozen experts and two sparse layers about one row in fifteen has such a margin)

_plain_cache = {}


def _plain(mdir, ids):
    key = (mdir, tuple(ids))
    if key not in _plain_cache:
        if mdir not in _plain_cache:
            _plain_cache[mdir] = plain_model.read_folder(mdir)
        cfg, W = _plain_cache[mdir]
        ms = []
        logits = plain_model.forward(cfg, W, list(ids), margins=ms)
        margin = torch.stack(ms).min(dim=0).values if ms else torch.full((len(ids),), float("inf"), dtype=torch.float64)
        _plain_cache[key] = (logits, margin)
    return _plain_cache[key]


def plain_logits(mdir, ids):
    """float64 logits [T, V] of the plain implementation for one whole sequence (cached)."""
    return _plain(mdir, ids)[0]


def plain_margins(mdir, ids):
    """Per position, the smallest router margin over the sparse layers (see ``plain_model.route``)."""
    return _plain(mdir, ids)[1]


def assert_rows_close(got, want, margin, dtype, what=""):
    """``assert_close`` row by row; in bfloat16 a row may exceed the bound if it sits on a router edge
    (``margin`` below EDGE_MARGIN), and only a few rows may."""
    got = torch.as_tensor(got, dtype=torch.float64).cpu()
    want = torch.as_tensor(want, dtype=torch.float64).cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = TOL[dtype]
    bound = tol["abs"] + tol["rel"] * float(want.abs().max())
    err = (got - want).abs().max(dim=-1).values
    off = torch.nonzero(err > bound).reshape(-1).tolist()
    if dtype != "bfloat16":
        assert not off, f"{what}: rows {off[:8]} differ by more than {bound:.3g}; max {float(err.max()):.3g}"
        return
    plain_rows = [(r, float(err[r]), float(margin[r])) for r in off if float(margin[r]) >= EDGE_MARGIN]
    assert not plain_rows, (f"{what}: rows (row, error, router margin) beyond {bound:.3g} that sit on no router edge: "
                            f"{plain_rows[:8]}")
    assert len(off) <= max(2, MAX_EDGE_SHARE * len(err)), f"{what}: {len(off)} of {len(err)} rows beyond {bound:.3g}"


def assert_close(got, want, dtype, what=""):
    got = torch.as_tensor(got, dtype=torch.float64).cpu()
    want = torch.as_tensor(want, dtype=torch.float64).cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    tol = TOL[dtype]
    bound = tol["abs"] + tol["rel"] * want.abs().max()
    err = (got - want).abs()
    if not bool((err <= bound).all()):
        bad = torch.nonzero(err > bound)
        first = bad[0].tolist()
        raise AssertionError(f"{what}: {len(bad)} of {err.numel()} values differ by more than {float(bound):.3g}; "
                             f"max {float(err.max()):.3g}; first at {first}: got {float(got[tuple(first)]):.6g}, "
                             f"want {float(want[tuple(first)]):.6g}")


class Replay:
    """Drives ModelRunner.step with a schedule and collects logits per (request, position)."""

    def __init__(self, runner):
        from nano_vllm_cpp_b200.engine.batch import StepEntry
        self.runner, self.StepEntry = runner, StepEntry
        self.fed = {}          # rid -> tokens fed so far
        self.logits = {}       # (rid, position) -> float32 row

    def step(self, parts, end=()):
        """parts: list of (rid, tokens, want_all or list of places)."""
        entries = []
        for rid, toks, want in parts:
            places = list(range(len(toks))) if want is True else list(want)
            entries.append(self.StepEntry(rid, list(toks), places))
        out = self.runner.step(entries).float().cpu()
        r = 0
        for e in entries:
            if e.rid not in self.fed:      # a new request under an id used before: forget the old rows
                for key in [k for k in self.logits if k[0] == e.rid]:
                    del self.logits[key]
            base = self.fed.get(e.rid, 0)
            for w in e.want:
                self.logits[(e.rid, base + w)] = out[r]
                r += 1
            self.fed[e.rid] = base + len(e.tokens)
        for rid in end:
            self.runner.close(rid)
            self.fed.pop(rid, None)
        self.runner.manager.check()

    def compare(self, rid, ids, mdir, dtype, what):
        want = plain_logits(mdir, ids)
        pos = sorted(p for (r, p) in self.logits if r == rid)
        assert pos, f"{what}: no logits were collected for {rid}"
        got = torch.stack([self.logits[(rid, p)] for p in pos])
        assert_rows_close(got, want[pos], plain_margins(mdir, ids)[pos], dtype, f"{what} request {rid}")


def assert_greedy_follows_plain(mdir, prompt_ids, tokens, dtype, what=""):
    """``tokens`` were generated greedily by the engine from ``prompt_ids``.  Every token must be the plain
    implementation's choice for its prefix, up to the first position where the plain logits leave the choice open
    within the dtype's tolerance (their two largest values closer than twice the bound, since both may move): from
    there on the two runs may rightly follow different sequences.  Returns the number of tokens that were held."""
    cfg, W = _plain_cache.setdefault(mdir, plain_model.read_folder(mdir))
    tol = TOL[dtype]
    ids = list(prompt_ids)
    for k, tok in enumerate(tokens):
        logits = plain_model.forward(cfg, W, ids)[-1]
        top = torch.topk(logits, 2)
        bound = tol["abs"] + tol["rel"] * float(logits.abs().max())
        if int(top.indices[0]) != int(tok):
            gap = float(top.values[0] - logits[int(tok)])
            assert gap <= 2 * bound, (f"{what}: token {k} is {tok}, the plain implementation takes {int(top.indices[0])} "
                                      f"with a lead of {gap:.3g} over it (tolerance {2 * bound:.3g})")
            return k
        ids.append(int(tok))
    return len(tokens)
