"""The engine against the plain implementation, for every way of cutting the work into steps:
whole, last 32 tokens one by one, portions of changing size, and mixed batches on a pool so small
that pages are used again.  Both tiny configurations, float32 and bfloat16."""
import pytest
import torch

import helpers
from helpers import Replay, prompt

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70], "A8": [5, 17, 33, 70], "B": [1, 9, 24, 40, 70], "C": [2, 33, 64, 129, 200]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {c: helpers.model_folder(c, tmp_path_factory) for c in ("A", "A8", "B", "C")}


def make_runner(mdir, dtype, max_tokens, max_requests=4):
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    return ModelRunner(mdir, dtype=dtype, max_tokens=max_tokens, max_requests=max_requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "A8", "B", "C"])
def test_whole(case, dtype, folders):
    runner = make_runner(folders[case], dtype, 256 if case == "C" else 128)
    rp = Replay(runner)
    for n in LENGTHS[case]:
        ids = prompt(case, n)
        rp.step([(f"r{n}", ids, True)], end=[f"r{n}"])
        rp.compare(f"r{n}", ids, folders[case], dtype, f"whole {case} n={n}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "A8", "B", "C"])
def test_last_32_one_by_one(case, dtype, folders):
    runner = make_runner(folders[case], dtype, 128)
    rp = Replay(runner)
    for n in (40, 70, 100):
        ids = prompt(case, n, salt=1)
        head = n - 32
        rp.step([("x", ids[:head], [head - 1])])
        for t in range(head, n):
            rp.step([("x", ids[t:t + 1], [0])])
        rp.compare("x", ids, folders[case], dtype, f"decode {case} n={n}")
        rp.step([], end=["x"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "A8", "B", "C"])
def test_portions_of_changing_size(case, dtype, folders):
    runner = make_runner(folders[case], dtype, 128)
    rp = Replay(runner)
    ids = prompt(case, 101, salt=2)
    sizes = [7, 2, 16, 1, 3, 31, 2, 17, 2, 5, 15]
    assert sum(sizes) == 101
    at = 0
    for s in sizes:
        rp.step([("p", ids[at:at + s], True)])
        at += s
    rp.compare("p", ids, folders[case], dtype, f"portions {case}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "A8", "B", "C"])
def test_mixed_with_page_reuse(case, dtype, folders):
    """Up to four live requests; portions of some beside decode tokens of others; the pool holds 192
    tokens while the requests need 5 x 64 in turn, so finished requests' pages are used again."""
    runner = make_runner(folders[case], dtype, 192)
    rp = Replay(runner)
    L = {"a": 50, "b": 37, "c": 64, "d": 20, "e": 61, "f": 33}
    ids = {r: prompt(case, n, salt=ord(r)) for r, n in L.items()}
    at = {r: 0 for r in L}

    def take(r, n, want=True):
        toks = ids[r][at[r]:at[r] + n]
        at[r] += len(toks)
        return (r, toks, want)

    rp.step([take("a", 30), take("b", 2)])
    rp.step([take("a", 1), take("b", 20), take("c", 7)])
    rp.step([take("a", 1), take("b", 1), take("c", 40)])
    rp.step([take("a", 18), take("b", 14), take("c", 1)], end=["a", "b"])   # a, b finished: 50, 37
    rp.step([take("c", 1), take("d", 20), take("e", 3)], end=["d"])
    rp.step([take("c", 15), take("e", 2), take("f", 30)], end=["c"])
    rp.step([take("e", 56), take("f", 1)])
    rp.step([take("f", 2)], end=["e", "f"])
    for r in L:
        assert at[r] == L[r]
        rp.compare(r, ids[r], folders[case], dtype, f"mixed {case}")
    for pool in runner.manager.pools:
        assert pool.num_free() == pool.num_pages


@pytest.mark.parametrize("case", ["A", "A8", "B", "C"])
def test_float32_logits_are_bit_equal_however_the_work_is_cut(case, folders):
    """The float32 run uses one kernel per operation whatever the batch is, each output a sum in one fixed order:
    a position's logits are the same bits whole, one by one, in portions, beside other requests and on other pages."""
    runner = make_runner(folders[case], "float32", 256)
    ids = prompt(case, 101, salt=11)
    other = prompt(case, 60, salt=12)

    def collect(rp, rid="x"):
        return torch.stack([rp.logits[(rid, p)] for p in range(101)])

    rp = Replay(runner)
    rp.step([("x", ids, True)], end=["x"])
    whole = collect(rp)
    rp = Replay(runner)
    rp.step([("o", other[:20], [])])                          # another request first: x lies on other pages
    rp.step([("x", ids[:69], True), ("o", other[20:21], [])])
    for t in range(69, 101):
        rp.step([("x", ids[t:t + 1], [0])] + ([("o", other[t - 48:t - 47], [])] if t % 2 else []))
    assert torch.equal(collect(rp), whole), "last 32 one by one"
    rp.step([], end=["x", "o"])
    rp = Replay(runner)
    at = 0
    for k, n in enumerate([7, 2, 16, 1, 3, 31, 2, 17, 2, 5, 15]):
        parts = [("x", ids[at:at + n], True)]
        if k % 3 == 0:
            parts.insert(0, ("o", other[k:k + 3], []))
        rp.step(parts)
        at += n
    assert at == 101 and torch.equal(collect(rp), whole), "portions beside another request"
    rp.step([], end=["x", "o"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["B", "C"])
def test_a_repeated_mixed_step_is_captured_and_replayed(case, dtype, folders):
    """A step's shape (rows per entry, wanted places) seen for the second time is captured as a CUDA graph and
    replayed from then on, whatever it holds: here two decoding requests beside a 24-token portion of a third, five
    times over, then the same totals cut otherwise, then portions alone.  The logits are those of a runner that launches every step kernel by kernel
    (float32: bit for bit; bfloat16: the decode kernel cuts the keys of single rows by the longest sequence allowed
    instead of by the step's longest, so rounding differs)."""
    from nano_vllm_cpp_b200.engine.runner import ModelRunner
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    graphs = ModelRunner(folders[case], dtype=dtype, max_tokens=512, max_requests=4)
    plain = ModelRunner(folders[case], dtype=dtype, max_tokens=512, max_requests=4, cuda_graphs=False)
    ids = {r: prompt(case, 260, salt=80 + i) for i, r in enumerate("abc")}
    at = {"a": 0, "b": 0, "c": 0}

    def step(parts):
        entries = []
        for r, n in parts:                                # (which row is wanted changes from step to step: it is data)
            entries.append(StepEntry(r, ids[r][at[r]:at[r] + n], [(at[r] // 5) % n]))
            at[r] += n
        got, want = graphs.step(entries).clone(), plain.step(entries)
        if dtype == "float32":
            assert torch.equal(got, want), parts
        else:
            helpers.assert_close(got, want, dtype, f"captured step {parts}")

    step([("a", 20), ("b", 7)])
    for _ in range(5):
        step([("a", 1), ("b", 1), ("c", 24)])
    mixed = (3, 26, 2, 3, False)                         # entries, rows, single rows, wanted rows, no sampling
    assert mixed in graphs._graphs and not plain._graphs
    step([("a", 24), ("b", 1), ("c", 1)])                # the same totals, the portion first: the same captured step
    assert len(graphs._graphs) == 1
    step([("a", 2), ("b", 1), ("c", 23)])                # one single row and two portions, cut three ways
    step([("a", 12), ("b", 1), ("c", 13)])
    step([("a", 7), ("b", 1), ("c", 18)])
    assert (3, 26, 1, 3, False) in graphs._graphs and len(graphs._graphs) == 2
    for _ in range(3):
        step([("c", 13)])
    assert (1, 13, 0, 1, False) in graphs._graphs
    for _ in range(3):                                   # ... and decode steps as before
        step([("a", 1), ("b", 1), ("c", 1)])
    assert (3, 3, 3, 3, False) in graphs._graphs
    for r in "abc":
        graphs.close(r), plain.close(r)
    graphs.manager.check()


def test_block_tables_travel_only_when_they_change(folders):
    """A request's block table goes to the device when it has changed (a page taken or given back, a new request)
    and stays there otherwise: decode steps inside a page send no table, the logits are those of a runner whose
    tables all travel with every step, and after a step that was prepared but never ran everything travels again."""
    from nano_vllm_cpp_b200.engine.batch import StepEntry
    case = "C"                                     # one group with a window, one without: pages are given back too
    lazy = make_runner(folders[case], "float32", 64 * 4)
    eager = make_runner(folders[case], "float32", 64 * 4)
    ids = {r: prompt(case, 70, salt=60 + r) for r in range(3)}
    sent_bytes = []
    for step in range(40):
        entries = []
        for r in range(3):
            at = 0 if step == 0 else 30 + step - 1          # 30 tokens at once, then one by one
            n = 30 if step == 0 else 1
            entries.append(StepEntry(r, ids[r][at:at + n], [n - 1]))
        eager.manager.invalidate_tables()
        a = lazy.step(entries).clone()
        sent_bytes.append(lazy.last_h2d_bytes)
        b = eager.step(entries)
        assert torch.equal(a, b), step
        assert eager.last_h2d_bytes >= lazy.last_h2d_bytes
    G, S, mb = len(lazy.manager.pools), 3, lazy.max_blocks
    assert G == 2
    # positions 30..68: pages are taken at 32, 48 and 64 and one is given back at 63; the other steps carry no table
    quiet = min(sent_bytes[1:])
    assert sent_bytes.count(quiet) >= 30 and max(sent_bytes[1:]) >= quiet + 4 * S * mb
    # a prepared step that does not run: the next one brings every table again, and the logits stay right
    entries = [StepEntry(r, ids[r][69:70], [0]) for r in range(3)]
    lazy.prepare([StepEntry(0, ids[0][69:70], [0])])
    lazy.manager.invalidate_tables()
    a, b = lazy.step(entries).clone(), eager.step(entries)
    assert torch.equal(a, b) and lazy.last_h2d_bytes >= quiet + 4 * G * S * mb


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, folders):
    """Positions 0, 1, 2 alone, then 150 tokens one by one (beyond several pages and the window)."""
    case = "B"
    runner = make_runner(folders[case], dtype, 192)
    rp = Replay(runner)
    ids = prompt(case, 150, salt=3)
    for t in range(150):
        rp.step([("l", ids[t:t + 1], [0])])
    rp.compare("l", ids, folders[case], dtype, "long decode")


def test_trace_run_program(folders, tmp_path):
    """bin/trace_run as a user starts it: JSON lines in, <step>.f32 files and 'done' lines out."""
    import json, os, subprocess, sys
    import numpy as np
    case, dtype = "A", "float32"
    ids = prompt(case, 40, salt=4)
    ids2 = prompt(case, 9, salt=5)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": ids[:10], "want": [9]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": ids[10:38], "want": []}, {"id": "b", "tokens": ids2, "want": [0, 8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": ids[38:], "want": [0, 1]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    exe = os.path.join(os.path.dirname(helpers.HERE), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", folders[case], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    V = helpers.CASES[case]["config"]["vocab_size"]
    ref_a, ref_b = helpers.plain_logits(folders[case], ids), helpers.plain_logits(folders[case], ids2)
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    s2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    helpers.assert_close(s0, ref_a[[9]], dtype, "step 0")
    helpers.assert_close(s1, ref_b[[0, 8]], dtype, "step 1")
    helpers.assert_close(s2, ref_a[[38, 39]], dtype, "step 2")


def test_bfloat16_run_of_a_model_stored_in_float32(tmp_path):
    """Tensors stored in 32 bits stay float32 in a bfloat16 run (the products then take the plain kernel);
    activations and the cache are bfloat16.  Portions and decode steps against the plain implementation."""
    from nano_vllm_cpp_b200.weights import write_model_folder
    cfg = dict(helpers.CASES["B"]["config"])
    mdir = write_model_folder(cfg, str(tmp_path / "f32"), seed=4, std=0.05, norm_std=0.1, dtype="float32")
    runner = make_runner(mdir, "bfloat16", 128)
    assert runner.model.layers[1].feed_forward.w_gate_up.dtype == torch.float32
    assert runner.cache.views[0].k.dtype == torch.bfloat16
    rp = Replay(runner)
    ids = prompt("B", 60, salt=6)
    rp.step([("m", ids[:25], True)])
    rp.step([("m", ids[25:27], True)])
    for t in range(27, 60):
        rp.step([("m", ids[t:t + 1], [0])])
    rp.compare("m", ids, mdir, "bfloat16", "float32 weights, bfloat16 run")


def test_trace_run_program_bfloat16(folders, tmp_path):
    import json, os, subprocess, sys
    import numpy as np
    case, dtype = "B", "bfloat16"
    ids = prompt(case, 50, salt=8)
    steps = [{"step": 7, "entries": [{"id": 1, "tokens": ids[:18], "want": list(range(18))}], "end": []}]
    steps += [{"step": 8 + i, "entries": [{"id": 1, "tokens": ids[18 + i:19 + i], "want": [0]}], "end": []} for i in range(32)]
    steps[-1]["end"] = [1]
    steps.append({"step": 99, "entries": [], "end": []})
    out = tmp_path / "out"
    exe = os.path.join(os.path.dirname(helpers.HERE), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", folders[case], "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    V = helpers.CASES[case]["config"]["vocab_size"]
    ref = helpers.plain_logits(folders[case], ids)
    helpers.assert_close(np.fromfile(out / "7.f32", dtype="<f4").reshape(-1, V), ref[:18], dtype, "portion")
    got = np.stack([np.fromfile(out / f"{8 + i}.f32", dtype="<f4") for i in range(32)])
    helpers.assert_close(got, ref[18:50], dtype, "decode steps")
    assert not (out / "99.f32").exists()
