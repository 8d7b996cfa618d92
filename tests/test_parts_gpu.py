"""The parts of a layer one by one against the plain implementation, at sizes of their own; the
order list (a layer run twice, a call that reads another call's cache); and a toy mixer with a
per-request state that is defined here, registered, built from a config.json and stepped through the
engine without any change to the package."""
import json
import math
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda"


def ctx_for(dtype):
    from nano_vllm_cpp_b200.csrc import ops
    from nano_vllm_cpp_b200.parts import RunContext
    return RunContext(device=torch.device(DEV), act_dtype=dtype, err=ops.ErrorFlag(DEV), page_size=16)


class DictFetch:
    """Hands a part its tensors from a dict of float64 CPU tensors, in the run's storage types."""

    def __init__(self, tensors, dtype):
        self.t, self.dtype = tensors, dtype

    def __call__(self, name):
        t = self.t[name]
        return t.to(torch.float32 if t.dim() == 1 else self.dtype).to(DEV)

    def has(self, name):
        return name in self.t


def rand_tensors(specs, seed, std=0.1, dtype=torch.bfloat16):
    """Random values already rounded to bfloat16, as float64 (so both runs and the plain code see the same)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, s in specs.items():
        t = torch.randn(s.shape, generator=g) * std
        if s.init == "ones":
            t = t + 1.0
        out[name] = t.to(torch.bfloat16).double()
    return out


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, rel, what):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max())
    bound = rel * max(1e-3, float(want.abs().max()))
    assert err <= bound, f"{what}: max error {err:.3g} > {bound:.3g}"


# ------------------------------------------------------------------------------- parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    H = 200
    part = build_part("norm", PartSpec("rmsnorm", dict(size=H, eps=1e-5)))
    W = rand_tensors(part.tensor_specs(), 1)
    part.load(DictFetch(W, dtype), ctx_for(dtype))
    x = torch.randn(9, H, generator=torch.Generator().manual_seed(2))
    br = torch.randn(9, H, generator=torch.Generator().manual_seed(3))
    xd = x.to(DEV)
    out, out32 = part.forward(xd, br.to(DEV), want_f32=True)
    want = pm.rms_norm(x.double() + br.double(), W["weight"], 1e-5)
    close(xd, x.double() + br.double(), 1e-6, "stream")
    close(out32, want, 2e-6, "float32 copy")
    close(out, want, tol(dtype) if dtype == torch.bfloat16 else 2e-6, "normalised rows")
    assert out.dtype == dtype


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_swiglu_part(dtype):
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    H, I = 136, 200
    part = build_part("feed_forward", PartSpec("dense_swiglu", dict(hidden_size=H, intermediate_size=I)))
    W = rand_tensors(part.tensor_specs(), 4)
    part.load(DictFetch(W, dtype), ctx_for(dtype))
    h = (torch.randn(21, H, generator=torch.Generator().manual_seed(5))).to(torch.bfloat16)
    out = part.forward(h.to(dtype).to(DEV), None, None)
    want = pm.dense_mlp(h.double(), W, "")
    assert out.dtype == torch.float32
    close(out, want, tol(dtype), "dense mlp")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,K,renorm,SI", [(10, 3, True, 72), (5, 5, False, 0), (60, 4, False, 264)])
def test_sparse_moe_part(dtype, E, K, renorm, SI):
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    H, I = 136, 56
    part = build_part("feed_forward", PartSpec("sparse_moe_swiglu", dict(
        hidden_size=H, num_experts=E, top_k=K, intermediate_size=I, shared_intermediate_size=SI, renormalize=renorm)))
    W = rand_tensors(part.tensor_specs(), 6, std=0.2)
    ctx = ctx_for(dtype)
    part.load(DictFetch(W, dtype), ctx)
    h = (torch.randn(37, H, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16)
    hd = h.to(dtype).to(DEV)
    mix = part.forward(hd, h.float().to(DEV), None)      # the experts' outputs, not yet summed
    ctx.err.check("moe")
    out = mix.sum()
    cfg = dict(num_experts=E, num_experts_per_tok=K, norm_topk_prob=renorm, shared_expert_intermediate_size=SI,
               moe_intermediate_size=I)
    want = pm.sparse_mlp(h.double(), W, "", cfg)
    close(out, want, tol(dtype), "sparse mlp")
    # the stacked layout of the expert tensors gives the same layer
    stacked = {k: v for k, v in W.items() if not k.startswith("experts.")}
    stacked["experts.gate_up_proj"] = torch.stack([torch.cat([W[f"experts.{e}.gate_proj.weight"], W[f"experts.{e}.up_proj.weight"]]) for e in range(E)])
    stacked["experts.down_proj"] = torch.stack([W[f"experts.{e}.down_proj.weight"] for e in range(E)])
    part2 = build_part("feed_forward", PartSpec("sparse_moe_swiglu", dict(
        hidden_size=H, num_experts=E, top_k=K, intermediate_size=I, shared_intermediate_size=SI, renormalize=renorm)))
    assert set(part2.tensor_specs(lambda n: n in stacked)) == set(stacked)
    part2.load(DictFetch(stacked, dtype), ctx)
    assert torch.equal(part2.forward(hd, h.float().to(DEV), None).sum(), out)
    # the norm that takes the branch sums the mix itself: the same rows as the sum followed by the norm
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=H, eps=1e-6)))
    norm.load(DictFetch({"weight": torch.linspace(0.5, 1.5, H)}, dtype), ctx)
    x1 = torch.randn(37, H, generator=torch.Generator().manual_seed(8)).to(DEV)
    x2 = x1.clone()
    y1, _ = norm.forward(x1, mix)
    y2, _ = norm.forward(x2, out)
    close(x1, x2, 1e-6, "residual after mix")
    close(y1.float(), y2.float(), 1e-6 if dtype == torch.float32 else 2 ** -7, "norm after mix")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv,D,window,bias", [(6, 2, 32, 0, True), (3, 3, 48, 10, False), (5, 1, 16, 33, True)])
def test_attention_part_in_portions(dtype, Hq, Hkv, D, window, bias):
    """Two requests; the first runs whole, the second in a portion, then both get one more row."""
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    from nano_vllm_cpp_b200.cache import DeviceCache
    H = 72
    part = build_part("mixer", PartSpec("paged_attention", dict(
        hidden_size=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, bias=bias, window=window,
        position=PartSpec("rotary_neox", dict(rotary_dim=D, theta=5000.0)))))
    W = rand_tensors(part.tensor_specs(), 8, std=0.15)
    ctx = ctx_for(dtype)
    part.load(DictFetch(W, dtype), ctx)
    cache = DeviceCache([part.cache_spec()], 16, 4, DEV, dtype)
    cache.allocate(16)
    g = torch.Generator().manual_seed(9)
    xa = torch.randn(40, H, generator=g).to(torch.bfloat16)
    xb = torch.randn(50, H, generator=g).to(torch.bfloat16)
    cfg = dict(num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D, rope_theta=5000.0,
               use_sliding_window=window > 0, sliding_window=window, max_window_layers=0)
    want_a = pm.attention_layer(xa.double(), W, "", cfg, 0, list(range(40)))
    want_b = pm.attention_layer(xb.double(), W, "", cfg, 0, list(range(50)))
    # step 1: a whole minus one row (39 rows), b's first 20 rows.  Pages: a -> 0..2, b -> 3..6
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo
    from batch_builder import build_batch
    ta, tb = [0, 1, 2], [3, 4, 5, 6]

    def run(parts):
        ses, infos, tabs, rows, row0 = [], [], [], [], 0
        for slot, (x, table, p0, n) in enumerate(parts):
            ses.append(StepEntry(slot, [0] * n, []))
            infos.append(EntryInfo(slot, slot, p0, n, row0))
            tabs.append(table)
            rows.append(x[p0:p0 + n])
            row0 += n
        batch = build_batch(ses, infos, [tabs], 8, DEV)
        out = part.forward(torch.cat(rows).to(dtype).to(DEV), batch, cache.view(0))
        ctx.err.check("attention")
        return out

    o1 = run([(xa, ta, 0, 39), (xb, tb, 0, 20)])
    close(o1[:39], want_a[:39], tol(dtype), "a rows 0..38")
    close(o1[39:], want_b[:20], tol(dtype), "b rows 0..19")
    o2 = run([(xa, ta, 39, 1), (xb, tb, 20, 29)])
    close(o2[:1], want_a[39:], tol(dtype), "a row 39")
    close(o2[1:], want_b[20:49], tol(dtype), "b rows 20..48")
    o3 = run([(xb, tb, 49, 1)])
    close(o3, want_b[49:], tol(dtype), "b row 49 (decode kernel in bfloat16)")


def test_part_constructors_refuse_what_the_kernels_cannot_take():
    from nano_vllm_cpp_b200.parts import build_part, PartSpec
    pos = PartSpec("none", {})
    with pytest.raises(ValueError, match="head_dim"):
        build_part("mixer", PartSpec("paged_attention", dict(hidden_size=64, num_heads=2, num_kv_heads=2, head_dim=24, bias=False, position=pos)))
    with pytest.raises(ValueError, match="head_dim"):
        build_part("mixer", PartSpec("paged_attention", dict(hidden_size=64, num_heads=2, num_kv_heads=2, head_dim=512, bias=False, position=pos)))
    with pytest.raises(ValueError, match="multiple"):
        build_part("mixer", PartSpec("paged_attention", dict(hidden_size=64, num_heads=3, num_kv_heads=2, head_dim=16, bias=False, position=pos)))
    with pytest.raises(ValueError, match="top_k"):
        build_part("feed_forward", PartSpec("sparse_moe_swiglu", dict(hidden_size=64, num_experts=4, top_k=5, intermediate_size=8)))
    with pytest.raises(KeyError, match="no mixer part"):
        build_part("mixer", PartSpec("does_not_exist", {}))


# ------------------------------------------------------------------------------- the order list
def plain_with_order(cfg, W, ids, order):
    """plain_model.forward with an explicit list of (layer, cache_of) calls: a call with cache_of reads the
    keys and values that the named earlier call made and makes none of its own."""
    T = len(ids)
    eps = cfg["rms_norm_eps"]
    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], pm.head_dim(cfg)
    kv = {}
    for ci, (l, cache_of) in enumerate(order):
        p = f"model.layers.{l}."
        h = pm.rms_norm(x, W[p + "input_layernorm.weight"], eps)
        proj = lambda n, heads: (h @ W[p + f"self_attn.{n}.weight"].T + W[p + f"self_attn.{n}.bias"]).reshape(T, heads, D)
        q = pm.rope_neox(proj("q_proj", Hq), list(range(T)), cfg["rope_theta"])
        if cache_of is None:
            kv[ci] = (pm.rope_neox(proj("k_proj", Hkv), list(range(T)), cfg["rope_theta"]), proj("v_proj", Hkv))
            k, v = kv[ci]
        else:
            k, v = kv[cache_of]
        a = pm.causal_attention(q, k, v, 1.0 / np.sqrt(D), pm.layer_window(cfg, l))
        x = x + a.reshape(T, Hq * D) @ W[p + "self_attn.o_proj.weight"].T
        h = pm.rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)
        x = x + (pm.sparse_mlp(h, W, p + "mlp.", cfg) if pm.layer_is_sparse(cfg, l) else pm.dense_mlp(h, W, p + "mlp."))
    return pm.rms_norm(x, W["model.norm.weight"], eps) @ W["lm_head.weight"].T


def test_order_list_repeats_a_layer_and_shares_a_cache(tmp_path):
    from nano_vllm_cpp_b200.config import register_architecture, Qwen2MoeConfig
    from nano_vllm_cpp_b200.models.qwen2_moe import build_spec
    from nano_vllm_cpp_b200.parts import LayerCall
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    order = [(0, None), (1, None), (1, None), (0, 0)]

    def build(cfg):
        spec = build_spec(cfg)
        spec.order = [LayerCall(l, c) for l, c in order]
        return spec

    register_architecture("ToyOrderForCausalLM", Qwen2MoeConfig.from_dict, build)
    mdir = helpers.model_folder("A", str(tmp_path))
    cfg = json.load(open(os.path.join(mdir, "config.json")))
    cfg["architectures"] = ["ToyOrderForCausalLM"]
    json.dump(cfg, open(os.path.join(mdir, "config.json"), "w"))
    pcfg, W = pm.read_folder(mdir)
    ids = helpers.prompt("A", 45, salt=30)
    want = plain_with_order(pcfg, W, ids, order)
    runner = ModelRunner(mdir, dtype="float32", max_tokens=128)
    assert len(runner.cache.views) == 4 and runner.cache.views[3].k is runner.cache.views[0].k
    assert runner.cache.views[2].k is not runner.cache.views[1].k and not runner.cache.views[3].write
    rp = helpers.Replay(runner)
    for a, b in ((0, 20), (20, 22), (22, 44), (44, 45)):
        rp.step([("o", ids[a:b], True)])
    got = torch.stack([rp.logits[("o", p)] for p in range(45)])
    helpers.assert_close(got, want, "float32", "order list")


# ------------------------------------------------------------------------------- a toy mixer with state
@dataclass
class ToyConfig:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    rms_norm_eps: float
    decay: float

    @classmethod
    def from_dict(cls, d):
        return cls(d["vocab_size"], d["hidden_size"], d["num_hidden_layers"], d["intermediate_size"],
                   d["rms_norm_eps"], d["decay"])


def define_toy():
    """A mixer that keeps one vector per request: s_t = decay * s_{t-1} + h_t, out_t = W s_t."""
    from nano_vllm_cpp_b200.parts import Mixer, TensorSpec, StateCacheSpec, PartSpec, LayerSpec, ModelSpec, register_part
    from nano_vllm_cpp_b200.config import register_architecture

    class DecayingSum(Mixer):
        graph_safe = False                      # walks the entries on the host

        def __init__(self, hidden_size, decay):
            self.hidden, self.decay = hidden_size, decay

        def tensor_specs(self, available=None):
            return {"mix.weight": TensorSpec((self.hidden, self.hidden))}

        def load(self, fetch, ctx):
            self.ctx = ctx
            self.w = fetch("mix.weight").float()

        def cache_spec(self):
            return StateCacheSpec((self.hidden,), torch.float32)

        def forward(self, h, batch, cache):
            out = torch.empty((batch.T, self.hidden), dtype=torch.float32, device=h.device)
            for e in batch.entries:
                s = cache.state[e.slot]
                for r in range(e.row0, e.row0 + e.length):
                    s = self.decay * s + h[r].float()
                    out[r] = self.w @ s
                cache.state[e.slot] = s
            return out

    register_part("mixer", "toy_decaying_sum", DecayingSum)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))

        def layer():
            return LayerSpec(
                norm1=norm, mixer=PartSpec("toy_decaying_sum", dict(hidden_size=cfg.hidden_size, decay=cfg.decay)),
                norm2=norm, feed_forward=PartSpec("dense_swiglu", dict(hidden_size=cfg.hidden_size,
                                                                       intermediate_size=cfg.intermediate_size)),
                names={"norm1": "ln1.", "mixer": "toy.", "norm2": "ln2.", "feed_forward": "mlp."})

        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                         layers=[layer() for _ in range(cfg.num_hidden_layers)], final_norm=norm,
                         tie_word_embeddings=True, init_std=0.1)

    register_architecture("ToyStateForCausalLM", ToyConfig.from_dict, build)


def toy_plain(cfg, W, ids):
    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = pm.rms_norm(x, W[p + "ln1.weight"], cfg["rms_norm_eps"])
        s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
        out = []
        for t in range(len(ids)):
            s = cfg["decay"] * s + h[t]
            out.append(W[p + "toy.mix.weight"] @ s)
        x = x + torch.stack(out)
        h = pm.rms_norm(x, W[p + "ln2.weight"], cfg["rms_norm_eps"])
        x = x + pm.dense_mlp(h, W, p + "mlp.")
    return pm.rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"]) @ W["model.embed_tokens.weight"].T


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from nano_vllm_cpp_b200.weights import write_model_folder
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    define_toy()
    cfg = dict(architectures=["ToyStateForCausalLM"], vocab_size=90, hidden_size=40, num_hidden_layers=2,
               intermediate_size=56, rms_norm_eps=1e-5, decay=0.9)
    mdir = write_model_folder(cfg, str(tmp_path / "toy"), seed=3, norm_std=0.1, dtype="float32")
    _, W = pm.read_folder(mdir)
    runner = ModelRunner(mdir, dtype="float32", max_tokens=64, max_requests=2)
    assert [v.kind for v in runner.cache.views] == ["state", "state"] and not runner.cuda_graphs
    g = np.random.RandomState(0)
    ids = {r: [int(t) for t in g.randint(0, 90, size=n)] for r, n in (("a", 23), ("b", 9), ("c", 12))}
    rp = helpers.Replay(runner)
    rp.step([("a", ids["a"][:10], True), ("b", ids["b"][:2], True)])
    rp.step([("a", ids["a"][10:11], True), ("b", ids["b"][2:], True)], end=["b"])
    rp.step([("a", ids["a"][11:], True), ("c", ids["c"], True)])      # c takes b's slot: its state starts from zero
    for r in ids:
        got = torch.stack([rp.logits[(r, p)] for p in range(len(ids[r]))])
        helpers.assert_close(got, toy_plain(cfg, W, ids[r]), "float32", f"toy request {r}")


def define_toy_hybrid():
    """The state mixer in layer 0 and paged attention in layer 1: a model whose requests hold a state slot *and*
    pages, so that the engine's scheduler can run out of pages and preempt it."""
    from nano_vllm_cpp_b200.parts import PartSpec, LayerSpec, ModelSpec
    from nano_vllm_cpp_b200.config import register_architecture
    define_toy()

    def build(cfg):
        H = cfg["hidden_size"]
        norm = PartSpec("rmsnorm", dict(size=H, eps=cfg["rms_norm_eps"]))
        mlp = PartSpec("dense_swiglu", dict(hidden_size=H, intermediate_size=cfg["intermediate_size"]))
        attn = PartSpec("paged_attention", dict(
            hidden_size=H, num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
            head_dim=cfg["head_dim"], bias=False,
            position=PartSpec("rotary_neox", dict(rotary_dim=cfg["head_dim"], theta=cfg["rope_theta"]))))
        names = {"norm1": "ln1.", "norm2": "ln2.", "feed_forward": "mlp."}
        layers = [LayerSpec(norm1=norm, mixer=PartSpec("toy_decaying_sum", dict(hidden_size=H, decay=cfg["decay"])),
                            norm2=norm, feed_forward=mlp, names=dict(names, mixer="toy.")),
                  LayerSpec(norm1=norm, mixer=attn, norm2=norm, feed_forward=mlp, names=dict(names, mixer="self_attn."))]
        return ModelSpec(vocab_size=cfg["vocab_size"], hidden_size=H, layers=layers, final_norm=norm,
                         tie_word_embeddings=True, init_std=0.1)

    register_architecture("ToyHybridForCausalLM", dict, build)


def toy_hybrid_plain(cfg, W, ids):
    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    eps = cfg["rms_norm_eps"]
    p = "model.layers.0."
    h = pm.rms_norm(x, W[p + "ln1.weight"], eps)
    s = torch.zeros(cfg["hidden_size"], dtype=torch.float64)
    out = []
    for t in range(len(ids)):
        s = cfg["decay"] * s + h[t]
        out.append(W[p + "toy.mix.weight"] @ s)
    x = x + torch.stack(out)
    x = x + pm.dense_mlp(pm.rms_norm(x, W[p + "ln2.weight"], eps), W, p + "mlp.")
    p = "model.layers.1."
    h = pm.rms_norm(x, W[p + "ln1.weight"], eps)
    x = x + pm.attention_layer(h, W, p + "self_attn.", cfg, 1, list(range(len(ids))))
    x = x + pm.dense_mlp(pm.rms_norm(x, W[p + "ln2.weight"], eps), W, p + "mlp.")
    return pm.rms_norm(x, W["model.norm.weight"], eps) @ W["model.embed_tokens.weight"].T


def test_toy_state_through_the_engine(tmp_path):
    """The state of a request starts from zero whoever held its slot before, also after a preemption, and a model
    with a state never shares prefix pages: two requests one after the other on the only slot, two prompts with 32
    common tokens under an engine that was asked for prefix sharing, and a pool so small that requests are
    preempted.  Greedy tokens equal the plain restatement's."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    from nano_vllm_cpp_b200.weights import write_model_folder
    define_toy_hybrid()
    cfg = dict(architectures=["ToyHybridForCausalLM"], vocab_size=90, hidden_size=40, num_hidden_layers=2,
               intermediate_size=56, rms_norm_eps=1e-5, decay=0.9, num_attention_heads=2, num_key_value_heads=1,
               head_dim=16, rope_theta=10000.0)
    mdir = write_model_folder(cfg, str(tmp_path / "hybrid"), seed=5, norm_std=0.1, dtype="float32")
    _, W = pm.read_folder(mdir)

    def plain_greedy(ids, n):
        ids = list(ids)
        for _ in range(n):
            ids.append(int(torch.argmax(toy_hybrid_plain(cfg, W, ids)[-1])))
        return ids[-n:]

    g = np.random.RandomState(1)
    common = [int(t) for t in g.randint(0, 90, size=32)]
    prompts = [common + [int(t) for t in g.randint(0, 90, size=n)] for n in (3, 9)] + [[int(t) for t in g.randint(0, 90, size=20)]]
    want = [plain_greedy(p, 12) for p in prompts]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    # one slot: every request takes over the slot of the one before it
    eng = LLMEngine(mdir, max_model_len=128, num_kv_blocks=16, dtype="float32", max_num_seqs=1, enable_prefix_caching=True)
    assert not eng.runner.manager.prefix_caching and eng.runner.cache.has_state
    assert [o["token_ids"] for o in eng.generate(prompts, sp)] == want
    # all live together; the second prompt must not adopt the first's pages
    eng = LLMEngine(mdir, max_model_len=128, num_kv_blocks=16, dtype="float32", max_num_seqs=4, enable_prefix_caching=True)
    assert [o["token_ids"] for o in eng.generate(prompts, sp)] == want
    # 8 pages = 128 tokens for 44 + 53 + 32 at the end: somebody is preempted and starts again from zero
    eng = LLMEngine(mdir, max_model_len=128, num_kv_blocks=8, dtype="float32", max_num_seqs=4)
    assert [o["token_ids"] for o in eng.generate(prompts, sp)] == want
    assert eng.scheduler.num_preemptions > 0
    assert eng.runner.manager.free_slots() == 4


def test_a_model_without_pages_has_no_pool(tmp_path):
    """The toy model whose mixers keep only a state: no page pool is made, however much memory is free, and the
    engine admits requests by state slots."""
    from nano_vllm_cpp_b200 import LLMEngine, SamplingParams
    from nano_vllm_cpp_b200.weights import write_model_folder
    define_toy()
    cfg = dict(architectures=["ToyStateForCausalLM"], vocab_size=90, hidden_size=40, num_hidden_layers=2,
               intermediate_size=56, rms_norm_eps=1e-5, decay=0.9)
    mdir = write_model_folder(cfg, str(tmp_path / "toy"), seed=3, norm_std=0.1, dtype="float32")
    _, W = pm.read_folder(mdir)
    eng = LLMEngine(mdir, max_model_len=64, num_kv_blocks=0, dtype="float32", max_num_seqs=2)
    assert eng.runner.manager.pools == [] and eng.runner.num_pages == 0
    g = np.random.RandomState(2)
    prompts = [[int(t) for t in g.randint(0, 90, size=n)] for n in (5, 11, 8)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        ids = list(p)
        for _ in range(6):
            ids.append(int(torch.argmax(toy_plain(cfg, W, ids)[-1])))
        assert o["token_ids"] == ids[len(p):]


# ------------------------------------------------------------------------------- two more toy parts: a position encoding and a routing feed-forward
@dataclass
class Toy2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float

    @classmethod
    def from_dict(cls, d):
        return cls(*(d[k] for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_heads", "head_dim",
                                   "intermediate_size", "rms_norm_eps")))


def define_toy2():
    """A position encoding whose frequencies are a tensor of the model (and that turns only half of a head), and a
    feed-forward that sends a row to one of two SwiGLU experts by the sign of a learned projection."""
    from nano_vllm_cpp_b200.parts import (FeedForward, PositionEncoding, TensorSpec, PartSpec, LayerSpec, ModelSpec,
                                          register_part)
    from nano_vllm_cpp_b200.parts.linear import linear
    from nano_vllm_cpp_b200.config import register_architecture

    class LearnedFrequencies(PositionEncoding):
        def __init__(self, rotary_dim):
            self.rotary_dim = rotary_dim

        def tensor_specs(self, available=None):
            return {"freq": TensorSpec((self.rotary_dim // 2,), kind="vector")}

        def load(self, fetch, ctx):
            self.ctx = ctx
            self._inv = fetch("freq").float().contiguous()

        def inv_freq(self):
            return self._inv

    class SignSwitch(FeedForward):
        graph_safe = False                      # gathers rows by a mask on the host side of the stream

        def __init__(self, hidden_size, intermediate_size):
            self.hidden, self.inter = hidden_size, intermediate_size

        def tensor_specs(self, available=None):
            s = {"switch.weight": TensorSpec((1, self.hidden))}
            for e in (0, 1):
                s[f"e{e}.gate_up.weight"] = TensorSpec((2 * self.inter, self.hidden))
                s[f"e{e}.down.weight"] = TensorSpec((self.hidden, self.inter))
            return s

        def load(self, fetch, ctx):
            self.ctx = ctx
            self.sw = fetch("switch.weight").float()
            self.w = [(fetch(f"e{e}.gate_up.weight"), fetch(f"e{e}.down.weight")) for e in (0, 1)]

        def forward(self, h, h32, batch):
            side = (h.float() @ self.sw.T).flatten() < 0
            out = torch.zeros((h.shape[0], self.hidden), dtype=torch.float32, device=h.device)
            for e in (0, 1):
                rows = torch.nonzero(side == bool(e)).flatten()
                if rows.numel():
                    x = h.index_select(0, rows).contiguous()
                    act = linear(self.ctx, x, self.w[e][0], self.ctx.act_dtype, swiglu=True)
                    out.index_copy_(0, rows, linear(self.ctx, act, self.w[e][1], torch.float32))
            return out

    register_part("position", "toy_learned_frequencies", LearnedFrequencies)
    register_part("feed_forward", "toy_sign_switch", SignSwitch)

    def build(cfg):
        norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))
        att = PartSpec("paged_attention", dict(
            hidden_size=cfg.hidden_size, num_heads=cfg.num_heads, num_kv_heads=cfg.num_heads, head_dim=cfg.head_dim,
            bias=False, position=PartSpec("toy_learned_frequencies", dict(rotary_dim=cfg.head_dim // 2))))
        ff = PartSpec("toy_sign_switch", dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size))
        layers = [LayerSpec(norm1=norm, mixer=att, norm2=norm, feed_forward=ff) for _ in range(cfg.num_hidden_layers)]
        return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers, final_norm=norm,
                         tie_word_embeddings=True, init_std=0.1)

    register_architecture("ToySwitchForCausalLM", Toy2Config.from_dict, build)


def toy2_plain(cfg, W, ids):
    T, Hh, D, R = len(ids), cfg["num_heads"], cfg["head_dim"], cfg["head_dim"] // 2
    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    pos = torch.arange(T, dtype=torch.float64)
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        h = pm.rms_norm(x, W[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q, k, v = (h @ W[p + f"self_attn.{n}_proj.weight"].double().T for n in "qkv")
        ang = pos[:, None] * W[p + "self_attn.freq"].double()[None, :]          # [T, R/2]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

        def turn(t):
            t = t.reshape(T, Hh, D).clone()
            a, b = t[..., :R // 2].clone(), t[..., R // 2:R].clone()
            t[..., :R // 2], t[..., R // 2:R] = a * c - b * s, b * c + a * s
            return t

        q, k, v = turn(q), turn(k), v.reshape(T, Hh, D)
        sc = torch.einsum("thd,uhd->htu", q, k) / math.sqrt(D)
        sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        att = torch.einsum("htu,uhd->thd", torch.softmax(sc, -1), v).reshape(T, Hh * D)
        x = x + att @ W[p + "self_attn.o_proj.weight"].double().T
        h = pm.rms_norm(x, W[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        side = (h @ W[p + "mlp.switch.weight"].double().T).flatten() < 0
        out = torch.zeros_like(x)
        for e in (0, 1):
            gu = h @ W[p + f"mlp.e{e}.gate_up.weight"].double().T
            I = gu.shape[1] // 2
            y = (gu[:, :I] / (1 + torch.exp(-gu[:, :I])) * gu[:, I:]) @ W[p + f"mlp.e{e}.down.weight"].double().T
            out[side == bool(e)] = y[side == bool(e)]
        x = x + out
    return pm.rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"]) @ W["model.embed_tokens.weight"].double().T


def test_toy_position_encoding_and_routing_feed_forward(tmp_path):
    """Another position encoding and a feed-forward with routing of its own, registered from outside the package,
    in a model that is built, loaded and stepped (whole, and cut into a portion and single tokens)."""
    from nano_vllm_cpp_b200.weights import write_model_folder
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    define_toy2()
    cfg = dict(architectures=["ToySwitchForCausalLM"], vocab_size=70, hidden_size=48, num_hidden_layers=2, num_heads=3,
               head_dim=16, intermediate_size=40, rms_norm_eps=1e-5)
    mdir = write_model_folder(cfg, str(tmp_path / "toy2"), seed=5, norm_std=0.1, dtype="float32")
    _, W = pm.read_folder(mdir)
    runner = ModelRunner(mdir, dtype="float32", max_tokens=64, max_requests=2)
    ids = [int(t) for t in np.random.RandomState(1).randint(0, 70, size=21)]
    want = toy2_plain(cfg, W, ids)
    rp = helpers.Replay(runner)
    rp.step([("w", ids, True)], end=["w"])
    rp.step([("c", ids[:13], True)])
    for t in range(13, 21):
        rp.step([("c", ids[t:t + 1], True)])
    for r in ("w", "c"):
        got = torch.stack([rp.logits[(r, p)] for p in range(len(ids))])
        helpers.assert_close(got, want, "float32", f"toy switch request {r}")


# ------------------------------------------------------------------------------- a position encoding with two coordinates
def define_toy_grid_position():
    """A position encoding that turns half of its pairs by the row's place in the sequence and the other half by a
    second coordinate of the row (here the place divided by four, as if the tokens were laid out in rows of four):
    it gives the rotation kernel the coordinates of every row and says which pair follows which."""
    from nano_vllm_cpp_b200.parts import PositionEncoding, PartSpec, LayerSpec, ModelSpec, register_part
    from nano_vllm_cpp_b200.config import register_architecture

    class GridRotary(PositionEncoding):
        def __init__(self, rotary_dim, theta):
            self.rotary_dim, self.theta = rotary_dim, theta

        def load(self, fetch, ctx):
            half = self.rotary_dim // 2
            inv = [1.0 / (self.theta ** ((2.0 * (i % (half // 2))) / half)) for i in range(half)]
            self._inv = torch.tensor(inv, dtype=torch.float64).float().to(ctx.device)
            self._axis = torch.tensor([i // (half // 2) for i in range(half)], dtype=torch.int32, device=ctx.device)

        def inv_freq(self):
            return self._inv

        def rotation_positions(self, batch):
            pos = batch.positions
            return torch.stack([pos, pos // 4], dim=1).contiguous()

        def pair_axis(self):
            return self._axis

    register_part("position", "toy_grid_rotary", GridRotary)

    def build(cfg):
        H = cfg["hidden_size"]
        norm = PartSpec("rmsnorm", dict(size=H, eps=cfg["rms_norm_eps"]))
        att = PartSpec("paged_attention", dict(
            hidden_size=H, num_heads=cfg["num_heads"], num_kv_heads=cfg["num_kv_heads"], head_dim=cfg["head_dim"],
            bias=False, position=PartSpec("toy_grid_rotary", dict(rotary_dim=cfg["head_dim"], theta=cfg["theta"]))))
        mlp = PartSpec("dense_swiglu", dict(hidden_size=H, intermediate_size=cfg["intermediate_size"]))
        layers = [LayerSpec(norm1=norm, mixer=att, norm2=norm, feed_forward=mlp) for _ in range(2)]
        return ModelSpec(vocab_size=cfg["vocab_size"], hidden_size=H, layers=layers, final_norm=norm,
                         tie_word_embeddings=True, init_std=0.1)

    register_architecture("ToyGridForCausalLM", dict, build)


def toy_grid_plain(cfg, W, ids):
    T, Hq, Hkv, D = len(ids), cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    half = D // 2
    inv = torch.tensor([1.0 / (cfg["theta"] ** ((2.0 * (i % (half // 2))) / half)) for i in range(half)],
                       dtype=torch.float64).float().double()
    pos = torch.arange(T)
    coord = torch.stack([pos, pos // 4], 1)
    axis = torch.tensor([i // (half // 2) for i in range(half)])
    ang = (coord[:, axis].float() * inv.float()).double()                     # [T, half], the product in float32
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def turn(x):                                                              # [T, heads, D]
        x1, x2 = x[..., :half], x[..., half:]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)

    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    for l in range(2):
        p = f"model.layers.{l}."
        h = pm.rms_norm(x, W[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
        q, k, v = (h @ W[p + f"self_attn.{n}_proj.weight"].double().T for n in "qkv")
        q, k, v = turn(q.reshape(T, Hq, D)), turn(k.reshape(T, Hkv, D)), v.reshape(T, Hkv, D)
        out = torch.zeros(T, Hq, D, dtype=torch.float64)
        for hh in range(Hq):
            sc = (q[:, hh] @ k[:, hh // (Hq // Hkv)].T) / (D ** 0.5)
            sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
            out[:, hh] = torch.softmax(sc, -1) @ v[:, hh // (Hq // Hkv)]
        x = x + out.reshape(T, Hq * D) @ W[p + "self_attn.o_proj.weight"].double().T
        h = pm.rms_norm(x, W[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
        x = x + pm.dense_mlp(h, W, p + "mlp.")
    return pm.rms_norm(x, W["model.norm.weight"], cfg["rms_norm_eps"]) @ W["model.embed_tokens.weight"].double().T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_position_encoding_with_two_coordinates(dtype, tmp_path):
    """A position encoding whose pairs follow two different coordinates of a row, registered from outside the
    package: the model is built, loaded and stepped whole, in portions and one by one, also in a captured step."""
    from nano_vllm_cpp_b200.weights import write_model_folder
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    define_toy_grid_position()
    cfg = dict(architectures=["ToyGridForCausalLM"], vocab_size=80, hidden_size=48, num_heads=4, num_kv_heads=2,
               head_dim=16, intermediate_size=40, rms_norm_eps=1e-5, theta=100.0)
    mdir = write_model_folder(cfg, str(tmp_path / "grid"), seed=11, norm_std=0.1, dtype="bfloat16")
    _, W = pm.read_folder(mdir)
    runner = ModelRunner(mdir, dtype=dtype, max_tokens=128, max_requests=2)
    ids = [int(t) for t in np.random.RandomState(2).randint(0, 80, size=37)]
    want = toy_grid_plain(cfg, W, ids)
    rp = helpers.Replay(runner)
    rp.step([("w", ids, True)], end=["w"])
    rp.step([("c", ids[:9], True)])
    rp.step([("c", ids[9:22], True)])
    for t in range(22, 37):
        rp.step([("c", ids[t:t + 1], True)])
    for r in ("w", "c"):
        got = torch.stack([rp.logits[(r, p)] for p in range(len(ids))])
        helpers.assert_close(got, want, dtype, f"toy grid position, request {r}")


# ------------------------------------------------------------------------------- toy arrangements
def define_toy_arrangements():
    """Two arrangements that the package does not have: a parallel block (one norm feeds the mixer and the
    feed-forward, both outputs are added) and a layer that is a mixer and nothing else."""
    from nano_vllm_cpp_b200.parts import Arrangement, PartSpec, LayerSpec, ModelSpec, register_part
    from nano_vllm_cpp_b200.parts.base import resolve_branch
    from nano_vllm_cpp_b200.config import register_architecture

    class ParallelBlock(Arrangement):
        slots = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}

        def forward(self, x, pending, batch, cache):
            h, h32 = self.norm.forward(x, resolve_branch(self.norm, pending), want_f32=self.feed_forward.wants_f32_input)
            a = self.mixer.forward(h, batch, cache)
            f = self.feed_forward.forward(h, h32, batch)
            return a + f                     # one float32 branch; the next norm adds it to the stream

    class MixerOnly(Arrangement):
        slots = {"norm": "norm", "mixer": "mixer"}

        def forward(self, x, pending, batch, cache):
            h, _ = self.norm.forward(x, resolve_branch(self.norm, pending))
            return self.mixer.forward(h, batch, cache)

    register_part("arrangement", "toy_parallel", ParallelBlock)
    register_part("arrangement", "toy_mixer_only", MixerOnly)

    def build(cfg):
        H = cfg["hidden_size"]
        norm = PartSpec("rmsnorm", dict(size=H, eps=cfg["rms_norm_eps"]))
        mlp = PartSpec("dense_swiglu", dict(hidden_size=H, intermediate_size=cfg["intermediate_size"]))

        def attn(window):
            return PartSpec("paged_attention", dict(
                hidden_size=H, num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                head_dim=cfg["head_dim"], bias=False, window=window,
                position=PartSpec("rotary_neox", dict(rotary_dim=cfg["head_dim"], theta=cfg["rope_theta"]))))

        layers = [LayerSpec("toy_parallel", dict(norm=norm, mixer=attn(0), feed_forward=mlp),
                            names={"norm": "ln.", "mixer": "self_attn.", "feed_forward": "mlp."}),
                  LayerSpec("toy_mixer_only", dict(norm=norm, mixer=attn(cfg["sliding_window"])),
                            names={"norm": "ln.", "mixer": "self_attn."})]
        return ModelSpec(vocab_size=cfg["vocab_size"], hidden_size=H, layers=layers, final_norm=norm,
                         tie_word_embeddings=True, init_std=0.1)

    register_architecture("ToyArrangementsForCausalLM", dict, build)


def toy_arrangements_plain(cfg, W, ids):
    eps, pos = cfg["rms_norm_eps"], list(range(len(ids)))
    x = pm.embedding(W["model.embed_tokens.weight"], ids)
    p = "model.layers.0."
    h = pm.rms_norm(x, W[p + "ln.weight"], eps)
    x = x + pm.attention_layer(h, W, p + "self_attn.", dict(cfg, use_sliding_window=False), 0, pos) + pm.dense_mlp(h, W, p + "mlp.")
    p = "model.layers.1."
    h = pm.rms_norm(x, W[p + "ln.weight"], eps)
    x = x + pm.attention_layer(h, W, p + "self_attn.", dict(cfg, use_sliding_window=True, max_window_layers=0), 1, pos)
    return pm.rms_norm(x, W["model.norm.weight"], eps) @ W["model.embed_tokens.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_arrangements_are_registered_built_and_stepped(dtype, tmp_path):
    """A layer is an arrangement kind plus whatever parts that arrangement names: a parallel block and a layer without
    a feed-forward, defined here, make a model that is loaded, checked against its tensor names and stepped (whole,
    in portions, one by one, two requests at once) without a change to the package."""
    from nano_vllm_cpp_b200.weights import write_model_folder
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    define_toy_arrangements()
    cfg = dict(architectures=["ToyArrangementsForCausalLM"], vocab_size=90, hidden_size=48, intermediate_size=56,
               rms_norm_eps=1e-5, num_attention_heads=3, num_key_value_heads=1, head_dim=16, rope_theta=10000.0,
               sliding_window=20)
    mdir = write_model_folder(cfg, str(tmp_path / "arr"), seed=7, norm_std=0.1, dtype="bfloat16")
    _, W = pm.read_folder(mdir)
    assert sorted(n for n in W if ".layers.1." in n) == sorted(
        "model.layers.1." + n for n in ("ln.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                        "self_attn.v_proj.weight", "self_attn.o_proj.weight"))
    runner = ModelRunner(mdir, dtype=dtype, max_tokens=128, max_requests=2)
    assert len(runner.manager.pools) == 2                 # a group for the full layer, one for the windowed one
    g = np.random.RandomState(4)
    ids = {r: [int(t) for t in g.randint(0, 90, size=n)] for r, n in (("a", 50), ("b", 33))}
    rp = helpers.Replay(runner)
    rp.step([("a", ids["a"][:30], True), ("b", ids["b"][:2], True)])
    rp.step([("a", ids["a"][30:31], True), ("b", ids["b"][2:], True)], end=["b"])
    for t in range(31, 50):
        rp.step([("a", ids["a"][t:t + 1], True)])
    for r in ids:
        got = torch.stack([rp.logits[(r, p)] for p in range(len(ids[r]))])
        helpers.assert_close(got, toy_arrangements_plain(cfg, W, ids[r]), dtype, f"toy arrangements, request {r}")
