"""Generation through the Python entry point and the command line: greedy tokens equal the plain
implementation's, sampled tokens equal the plain sampler's on the engine's logits, a preempted
request resumes with the same tokens, and batch composition does not change a request's tokens."""
import os
import subprocess
import sys

import pytest
import torch

import helpers
from helpers import prompt

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {c: helpers.model_folder(c, tmp_path_factory) for c in ("A", "B", "C", "D")}


def engine(mdir, **kw):
    from nano_vllm_cpp_b200 import LLMEngine
    kw.setdefault("dtype", "float32")
    kw.setdefault("max_num_seqs", 8)
    return LLMEngine(mdir, kw.pop("max_model_len", 128), kw.pop("num_kv_blocks", 64), **kw)


def plain_greedy(mdir, ids, n):
    cfg, W = helpers.plain_model.read_folder(mdir)
    return helpers.plain_model.greedy_generate(cfg, W, ids, n)


@pytest.mark.parametrize("case", ["A", "B"])
def test_greedy_generation_equals_plain(case, folders):
    from nano_vllm_cpp_b200 import SamplingParams
    lengths = {"A": [5, 17, 33], "B": [1, 9, 24]}[case]
    prompts = [prompt(case, n, salt=9) for n in lengths]
    eng = engine(folders[case])
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o["token_ids"] == plain_greedy(folders[case], p, 12)


@pytest.mark.parametrize("case", ["A", "B", "C"])
def test_greedy_generation_in_bfloat16_follows_plain(case, folders):
    """bfloat16 through the scheduler: every greedy token is the plain implementation's choice up to the first
    position where the plain logits leave the choice open within the bfloat16 tolerance; and at least the
    first tokens of every request are held."""
    from nano_vllm_cpp_b200 import SamplingParams
    lengths = {"A": [5, 17, 33], "B": [1, 9, 24], "C": [2, 40, 70]}[case]
    prompts = [prompt(case, n, salt=9) for n in lengths]
    eng = engine(folders[case], dtype="bfloat16")
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    held = [helpers.assert_greedy_follows_plain(folders[case], p, o["token_ids"], "bfloat16", f"{case} prompt {len(p)}")
            for p, o in zip(prompts, outs)]
    assert sum(held) >= 12, f"only {held} tokens could be held to the plain implementation"


# ------------------------------------------------------------------------------- prefix sharing
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "D"])
def test_logits_of_a_request_that_adopts_another_requests_pages(case, dtype, folders):
    """Request 2 shares its first 40 tokens with request 1 and takes over request 1's two full pages instead of
    running those tokens: once while request 1 is live (the pages are held twice), once after request 1 has ended
    (the pages are revived from the free list), once after a stranger has been through the pool in between.  The
    logits of every position that request 2 runs equal the plain implementation's."""
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    mdir = folders[case]
    runner = ModelRunner(mdir, dtype=dtype, max_tokens=192, max_requests=4, prefix_caching=True)
    m = runner.manager
    assert m.prefix_caching
    shared = prompt(case, 40, salt=70)
    one = shared + prompt(case, 9, salt=71)
    two = shared + prompt(case, 21, salt=72)
    three = shared[:32] + prompt(case, 30, salt=73)
    stranger = prompt(case, 100, salt=74)

    def run_whole(rid, ids):
        runner.step([StepEntry(rid, ids, [len(ids) - 1])])
        m.commit(rid, len(ids), ids)                      # hashes the full pages, as the scheduler's bookkeeping does

    def run_adopting(rid, ids, expect_cached):
        runner.open(rid)
        matched = m.match_prefix(ids)
        cached = m.adopt_prefix(rid, matched)
        assert cached == expect_cached
        rest = ids[cached:]
        logits = runner.step([StepEntry(rid, rest, list(range(len(rest))))]).float().cpu()
        m.commit(rid, len(ids), ids)
        want = helpers.plain_logits(mdir, ids)[cached:]
        helpers.assert_rows_close(logits, want, helpers.plain_margins(mdir, ids)[cached:], dtype,
                                  f"{case} {dtype} request {rid} after {cached} adopted tokens")
        m.check()

    run_whole("one", one)
    run_adopting("two", two, 32)                          # pages 0 and 1 of "one", which is still live
    assert m.pools[0].ref_count[m.get("one").tables[0][0]] == 2
    runner.close("one")
    runner.close("two")
    assert m.pools[0].num_free() == m.pools[0].num_pages
    run_adopting("three", three, 32)                      # both owners are gone: the pages come back from the free list
    runner.close("three")
    run_whole("stranger", stranger)                       # 7 of the 12 pages: the hashed pages are at the back, untouched
    runner.close("stranger")
    run_adopting("again", two, 48)                        # the third page that "two" wrote is still there, too
    runner.close("again")
    run_whole("big", prompt(case, 190, salt=75))          # all 12 pages taken: the hashes are forgotten
    runner.close("big")
    run_adopting("fresh", two, 0)
    runner.close("fresh")
    assert m.pools[0].num_free() == m.pools[0].num_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefix_sharing_through_the_entry_point(dtype, folders):
    """Two waves of requests with common prefixes through the engine with prefix sharing on (its default): the
    second wave adopts pages the first wave wrote.  Greedy tokens follow the plain implementation, and in float32
    they equal those of an engine without prefix sharing."""
    from nano_vllm_cpp_b200 import SamplingParams
    case = "D"
    base = prompt(case, 48, salt=80)
    wave1 = [base + prompt(case, 5, salt=81), prompt(case, 20, salt=82)]
    wave2 = [base + prompt(case, 11, salt=83), base[:40] + prompt(case, 3, salt=84), prompt(case, 33, salt=85)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    eng = engine(folders[case], dtype=dtype, max_model_len=256, num_kv_blocks=32)
    assert eng.runner.manager.prefix_caching
    got1 = [o["token_ids"] for o in eng.generate(wave1, sp)]
    free_before = eng.runner.manager.pools[0].num_free()
    started = []
    inner = eng.runner.launch_tokens

    def spy(entries, *a, **k):
        started.extend((e.rid, len(e.tokens)) for e in entries)
        return inner(entries, *a, **k)

    eng.runner.launch_tokens = spy
    got2 = [o["token_ids"] for o in eng.generate(wave2, sp)]
    assert free_before == eng.runner.manager.pools[0].num_pages
    first_portion = {}
    for rid, n in started:
        first_portion.setdefault(rid, n)
    # 48 and 32 of the shared tokens were adopted, not run again
    assert sorted(first_portion.values()) == [len(wave2[1]) - 32, len(wave2[0]) - 48, 33]
    for p, toks in zip(wave1 + wave2, got1 + got2):
        held = helpers.assert_greedy_follows_plain(folders[case], p, toks, dtype, f"prefix sharing {dtype}")
        assert held >= (10 if dtype == "float32" else 3)
    if dtype == "float32":
        plain = engine(folders[case], dtype=dtype, max_model_len=256, num_kv_blocks=32, enable_prefix_caching=False)
        assert [o["token_ids"] for o in plain.generate(wave1 + wave2, sp)] == got1 + got2


def test_temperature_sampling_is_reproducible_and_follows_the_plain_sampler(folders):
    from nano_vllm_cpp_b200 import SamplingParams
    from nano_vllm_cpp_b200.sampling import uniform
    case = "B"
    prompts = [prompt(case, n, salt=10) for n in (1, 9, 24, 40, 70)]
    sps = [SamplingParams(temperature=0.8, max_tokens=24, ignore_eos=True, seed=100 + i) for i in range(5)]
    a = engine(folders[case], max_model_len=128).generate(prompts, sps)
    b = engine(folders[case], max_model_len=128, max_num_batched_tokens=16, max_num_seqs=2).generate(prompts, sps)
    assert [o["token_ids"] for o in a] == [o["token_ids"] for o in b]      # same seeds, other batching
    # every token is the plain sampler's choice on the plain logits of its prefix with the same u
    cfg, W = helpers.plain_model.read_folder(folders[case])
    ids = list(prompts[1])
    for k, tok in enumerate(a[1]["token_ids"][:8]):
        logits = helpers.plain_model.forward(cfg, W, ids)[-1].float().numpy()
        assert helpers.plain_model.sample(logits, 0.8, uniform(101, k)) == tok
        ids.append(tok)


def test_preempted_request_resumes_with_the_same_tokens(folders):
    from nano_vllm_cpp_b200 import SamplingParams
    case = "A"
    prompts = [prompt(case, 20, salt=20 + i) for i in range(3)]
    sp = [SamplingParams(temperature=0.7, max_tokens=30, ignore_eos=True, seed=5 + i) for i in range(3)]
    roomy = engine(folders[case], num_kv_blocks=64)
    want = [o["token_ids"] for o in roomy.generate(prompts, sp)]
    tight = engine(folders[case], num_kv_blocks=8)          # 150 tokens needed at the end, 128 fit
    got = [o["token_ids"] for o in tight.generate(prompts, sp)]
    assert tight.scheduler.num_preemptions > 0
    assert got == want


@pytest.mark.parametrize("case", ["A", "C"])
def test_preemption_in_bfloat16(case, folders):
    """A preempted request runs its prompt and its own tokens again as one portion, where the uninterrupted run
    decoded them one by one: other kernels, so in bfloat16 the logits differ by rounding and a sampled token may
    differ where two candidates are close.  What must hold: everything finishes, every page comes back, and
    the greedy tokens of the tight run follow the plain implementation like those of the roomy run."""
    from nano_vllm_cpp_b200 import SamplingParams
    prompts = [prompt(case, 20, salt=20 + i) for i in range(3)]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    tight = engine(folders[case], dtype="bfloat16", num_kv_blocks=8)
    got = [o["token_ids"] for o in tight.generate(prompts, sp)]
    assert tight.scheduler.num_preemptions > 0
    assert all(len(t) == 30 for t in got)
    assert all(p.num_free() == p.num_pages for p in tight.runner.manager.pools)
    held = [helpers.assert_greedy_follows_plain(folders[case], p, t, "bfloat16", f"preempted {case}") for p, t in zip(prompts, got)]
    assert sum(held) >= 10


def test_steps_queued_ahead_give_the_same_tokens(folders):
    """The engine queues a step before it has read the tokens of the one before (they are fed back on the
    device) and learns of a stop token a step late: every request's tokens equal those of the plain order, with
    prompts beside decoded tokens, stop tokens in mid-run and so few pages that requests are preempted."""
    from nano_vllm_cpp_b200 import SamplingParams
    case = "A"
    prompts = [prompt(case, n, salt=40 + i) for i, n in enumerate((20, 3, 33, 20, 9, 26))]
    sp = [SamplingParams(temperature=0.9, max_tokens=30, ignore_eos=True, seed=50 + i) for i in range(6)]
    free = [o["token_ids"] for o in engine(folders[case], run_ahead=False).generate(prompts, sp)]
    # a stop token that some requests draw in mid-run: the most frequent token among the free runs' middles
    counts = {}
    for toks in free:
        for t in set(toks[5:25]):
            counts[t] = counts.get(t, 0) + 1
    stop = max(counts, key=counts.get)
    sp = [SamplingParams(temperature=0.9, max_tokens=30, seed=50 + i) for i in range(6)]
    want = [t[:t.index(stop) + 1] if stop in t else t for t in free]
    assert any(len(w) < 30 for w in want)
    for kw in (dict(), dict(num_kv_blocks=8, max_num_seqs=4), dict(max_num_batched_tokens=16)):
        plain = engine(folders[case], run_ahead=False, eos=stop, **kw)
        ahead = engine(folders[case], run_ahead=True, eos=stop, **kw)
        a = [o["token_ids"] for o in plain.generate(prompts, sp)]
        b = [o["token_ids"] for o in ahead.generate(prompts, sp)]
        assert a == want and b == want
        if "num_kv_blocks" in kw:
            assert ahead.scheduler.num_preemptions > 0
        assert all(p.num_free() == p.num_pages for p in ahead.runner.manager.pools)
    # bfloat16: the two orders run the same kernels on the same batches, so their tokens are equal exactly
    # (without preemption: a preempted request's second prompt is cut by when its victim was picked)
    for kw in (dict(), dict(max_num_batched_tokens=16)):
        a = [o["token_ids"] for o in engine(folders[case], dtype="bfloat16", run_ahead=False, eos=stop, **kw).generate(prompts, sp)]
        ahead = engine(folders[case], dtype="bfloat16", run_ahead=True, eos=stop, **kw)
        assert [o["token_ids"] for o in ahead.generate(prompts, sp)] == a
        assert all(p.num_free() == p.num_pages for p in ahead.runner.manager.pools)


def test_sample_kernel_against_plain_sampler():
    from nano_vllm_cpp_b200.csrc import ops
    g = torch.Generator().manual_seed(0)
    for V in (5, 384, 1000, 151936):
        R = 6
        logits = (torch.randn(R, V, generator=g) * 3).cuda()
        temps = torch.tensor([0.0, 0.5, 1.0, 2.0, 0.01, 1.3])
        us = torch.tensor([0.3, 0.0, 0.999999, 0.5, 0.7, 0.123], dtype=torch.float64)
        out = torch.empty(R, dtype=torch.int32, device="cuda")
        ops.sample(logits, temps.cuda(), us.cuda(), out)
        want = [helpers.plain_model.sample(logits[r].cpu().numpy(), float(temps[r]), float(us[r])) for r in range(R)]
        assert out.tolist() == want
    tie = torch.zeros(2, 100).cuda()
    tie[0, 7] = tie[0, 50] = 3.0
    out = torch.empty(2, dtype=torch.int32, device="cuda")
    ops.sample(tie, torch.zeros(2).cuda(), torch.zeros(2, dtype=torch.float64).cuda(), out)
    assert out.tolist() == [7, 0]                            # the first largest logit


def nucleus(logits, rows):
    """rows: (temperature, top_p, penalty, u, recent ids) per row -> the kernel's tokens."""
    from nano_vllm_cpp_b200.csrc import ops
    params = torch.tensor([[t, p, pen, u] for t, p, pen, u, _ in rows], dtype=torch.float64).cuda()
    flat, off = [], [0]
    for *_, recent in rows:
        flat += list(recent)
        off.append(len(flat))
    recent = torch.tensor(flat or [0], dtype=torch.int32).cuda()
    out = torch.empty(len(rows), dtype=torch.int32, device="cuda")
    ops.sample_nucleus(logits, params, recent, torch.tensor(off, dtype=torch.int32).cuda(), out)
    return out.tolist()


def test_nucleus_kernel_against_plain_sampler():
    g = torch.Generator().manual_seed(3)
    for V in (2, 5, 384, 1000, 151936):
        rows = [(0.0, 0.9, 1.0, 0.3, []), (0.5, 0.9, 1.0, 0.0, []), (1.0, 0.95, 1.0, 0.999999, []),
                (2.0, 0.5, 1.0, 0.5, []), (0.7, 0.1, 1.0, 0.97, []), (1.3, 1.0, 1.0, 0.9999, []),
                (1.0, 0.9, 1.3, 0.4, [1, 0, 1, V - 1, V + 5, -2]), (0.8, 0.8, 0.5, 0.6, [V // 2] * 3 + [0]),
                (1.0, 0.0, 1.0, 0.75, []), (0.9, 0.3, 1e20, 0.2, list(range(min(V - 1, 40))))]
        logits = (torch.randn(len(rows), V, generator=g) * 3).cuda()
        want = [helpers.plain_model.sample_row(logits[r].cpu().numpy(), t, p, u, recent, pen, 0)
                for r, (t, p, pen, u, recent) in enumerate(rows)]
        assert nucleus(logits, rows) == want, f"V = {V}"
    # equal scores are taken in index order; one dominant token still leaves a nucleus of two
    tie = torch.zeros(4, 100)
    tie[:, 7] = tie[:, 50] = tie[:, 51] = 3.0
    tie[3, 7] = 6.0
    rows = [(1.0, 0.9, 1.0, 0.0, []), (1.0, 0.9, 1.0, 0.5, []), (1.0, 0.9, 1.0, 0.95, []), (1.0, 0.5, 1.0, 0.9999999, [])]
    got = nucleus(tie.cuda(), rows)
    want = [helpers.plain_model.sample_row(tie[r].numpy(), t, p, u, recent, pen, 0) for r, (t, p, pen, u, recent) in enumerate(rows)]
    assert got == want and got[0] == 7 and got[3] == 50


def test_nucleus_sampling_through_the_entry_point(folders):
    """Requests with top_p and a repetition penalty beside a greedy one and a plainly sampled one: every token is the
    plain sampler's choice on the plain logits of its prefix, with the request's own uniform numbers; the other
    requests' tokens are what they are without such neighbours; another batching changes nothing."""
    from nano_vllm_cpp_b200 import SamplingParams
    from nano_vllm_cpp_b200.sampling import uniform
    case = "A"
    prompts = [prompt(case, n, salt=60 + i) for i, n in enumerate((9, 17, 5, 12))]
    sps = [SamplingParams(temperature=0.9, top_p=0.6, max_tokens=14, ignore_eos=True, seed=200),
           SamplingParams(temperature=1.2, top_p=0.9, repetition_penalty=1.5, repetition_window=4, max_tokens=14,
                          ignore_eos=True, seed=201),
           SamplingParams(temperature=0.0, top_p=0.5, repetition_penalty=2.0, max_tokens=14, ignore_eos=True),
           SamplingParams(temperature=0.8, max_tokens=14, ignore_eos=True, seed=203)]
    a = [o["token_ids"] for o in engine(folders[case]).generate(prompts, sps)]
    b = [o["token_ids"] for o in engine(folders[case], max_num_batched_tokens=16, max_num_seqs=2).generate(prompts, sps)]
    assert a == b
    alone = engine(folders[case]).generate(prompts[2:], sps[2:])
    assert [o["token_ids"] for o in alone] == a[2:]
    cfg, W = helpers.plain_model.read_folder(folders[case])
    for i in (0, 1):
        ids, done = list(prompts[i]), []
        for k, tok in enumerate(a[i]):
            logits = helpers.plain_model.forward(cfg, W, ids)[-1].float().numpy()
            want = helpers.plain_model.sample_row(logits, sps[i].temperature, sps[i].top_p, uniform(sps[i].seed, k), done,
                                                  sps[i].repetition_penalty, sps[i].repetition_window)
            assert tok == want, f"request {i}, token {k}"
            ids.append(tok)
            done.append(tok)
    assert a[2] == plain_greedy(folders[case], prompts[2], 14)      # greedy is never penalised


def test_command_line(folders):
    exe = os.path.join(os.path.dirname(helpers.HERE), "bin", "nanovllm")
    ids = prompt("A", 5, salt=9)
    r = subprocess.run([sys.executable, exe, folders["A"], "--tokens", ",".join(map(str, ids)), "--max-tokens", "6",
                        "--temperature", "0", "--dtype", "float32", "--max-model-len", "64", "--num-kv-blocks", "8",
                        "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("token_ids:")][0]
    assert [int(x) for x in line.split()[1:]] == plain_greedy(folders["A"], ids, 6)
    r = subprocess.run([sys.executable, exe, "--bench", folders["A"], "--num-seqs", "3", "--max-tokens", "4",
                        "--max-model-len", "128", "--num-kv-blocks", "32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "PP: 192 tokens" in r.stdout and "decode:" in r.stdout
    r = subprocess.run([sys.executable, exe, folders["A"], "hello"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 2 and "token ids" in r.stderr


def test_command_line_with_a_config_file_and_the_start_up_lines(tmp_path):
    """``--config`` runs random weights of the model a JSON file describes, without a model folder; ``--dtype fp32``
    is the reference's spelling; at start-up the engine says what the weights took and how large the cache pool is."""
    import json
    exe = os.path.join(os.path.dirname(helpers.HERE), "bin", "nanovllm")
    cfg = tmp_path / "tiny.json"
    cfg.write_text(json.dumps(helpers.CASES["B"]["config"]))
    runs = []
    for _ in range(2):
        r = subprocess.run([sys.executable, exe, "--config", str(cfg), "--seed", "3", "--tokens", "5,17,3", "--max-tokens", "5",
                            "--temperature", "0", "--dtype", "fp32", "--max-model-len", "64", "--num-kv-blocks", "8",
                            "--ignore-eos"], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        runs.append([l for l in r.stdout.splitlines() if l.startswith("token_ids:")][0])
        assert "[nanovllm] weights loaded:" in r.stderr and "[nanovllm] cache pool: 8 pages of 16 tokens" in r.stderr
        assert "[nanovllm] workspace:" in r.stderr and "after a step of 128 tokens" in r.stderr      # all 8 pages
    assert runs[0] == runs[1] and len(runs[0].split()) == 6          # the seed fixes the weights


def test_the_start_up_step_sizes_the_workspace(folders):
    """The engine runs the largest step its scheduler can ask for once at start-up; what the allocator holds after
    it serves every later step: prompts that fill the token budget, decoding, sampling, without more device
    memory being taken (captured decode steps keep memory of their own and are left out here)."""
    from nano_vllm_cpp_b200 import SamplingParams
    case = "C"
    prompts = [prompt(case, n, salt=70 + i) for i, n in enumerate((90, 60, 33, 7, 120, 2))]
    sp = [SamplingParams(temperature=0.8 if i % 2 else 0.0, max_tokens=12, ignore_eos=True, seed=i) for i in range(6)]
    grew = {}
    for warm in (True, False):
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        eng = engine(folders[case], dtype="bfloat16", max_model_len=160, num_kv_blocks=48, max_num_batched_tokens=256,
                     cuda_graphs=False, warm_up=warm, log_stats=False)
        assert all(p.num_free() == p.num_pages for p in eng.runner.manager.pools) and eng.runner.manager.free_slots() == 8
        before = torch.cuda.memory_reserved()
        outs = eng.generate(prompts, sp)
        assert all(len(o["token_ids"]) == 12 for o in outs)
        grew[warm] = torch.cuda.memory_reserved() - before
        del eng
    assert grew[True] <= 2 << 20 and grew[True] < grew[False]       # at most one more small segment of the allocator's


def test_kernel_times():
    """``ops.KernelTimes`` books every launch of a step to its kernel class."""
    from nano_vllm_cpp_b200.csrc import ops
    a = torch.randn(4, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(64, 256, device="cuda").to(torch.bfloat16)
    out = torch.empty(4, 64, device="cuda")
    with ops.KernelTimes() as kt:
        for _ in range(3):
            ops.skinny_gemm(a, w, out)
        ops.gemm_plain(a, w, out)
    rows = {r["name"]: r for r in kt.summary()}
    assert rows["skinny_gemm N=64 K=256"]["calls"] == 3 and rows["gemm_plain"]["calls"] == 1
    assert all(r["ms"] > 0 for r in rows.values())
    assert rows["skinny_gemm N=64 K=256"]["bytes"] == 3 * 64 * 256 * 2
    assert not ops.timing()


def test_smoke_entry():
    sys.path.insert(0, os.path.dirname(helpers.HERE))
    import __graft_entry__
    __graft_entry__.smoke()
