"""The cache manager and the scheduler on the host: no page lost, held twice or freed twice under
random orders of requests; windows give pages back; prefix pages are shared; the scheduler's
decisions under a token budget and when pages run out."""
import random

import pytest

from nano_vllm_cpp_b200.cache import BlockPool, CacheManager, NoFreePages, NoFreeSlot, chain_hash
from nano_vllm_cpp_b200.config import SamplingParams
from nano_vllm_cpp_b200.engine.scheduler import Scheduler, SchedulerError
from nano_vllm_cpp_b200.engine.sequence import Sequence


# ------------------------------------------------------------------------------- block pool
def test_pool_order_and_double_release():
    p = BlockPool(4, 16)
    a, b = p.allocate(), p.allocate()
    assert (a, b) == (0, 1)                      # fresh pages come from the front
    p.release(a)
    assert p.allocate() == 2 and p.allocate() == 3 and p.allocate() == 0   # a freed page goes to the back
    with pytest.raises(NoFreePages):
        p.allocate()
    p.release(b)
    with pytest.raises(RuntimeError):
        p.release(b)                             # freed twice
    p.check()


def test_pool_hash_revival():
    p = BlockPool(3, 4)
    a = p.allocate()
    h = chain_hash([1, 2, 3, 4], None)
    p.set_hash(a, h, [1, 2, 3, 4])
    p.release(a)
    assert p.lookup(h, [1, 2, 3, 4]) == a        # a freed page keeps its hash ...
    assert p.lookup(h, [1, 2, 3, 5]) is None
    p.share(a)                                   # ... and can be revived
    assert p.ref_count[a] == 1 and p.num_free() == 2
    p.release(a)
    p.allocate(), p.allocate()
    assert p.allocate() == a and p.lookup(h, [1, 2, 3, 4]) is None   # handed out again: hash forgotten
    assert chain_hash([1, 2], None) != chain_hash([1, 2], 7) != chain_hash([2, 1], 7)


# ------------------------------------------------------------------------------- cache manager
def test_manager_pages_and_slots():
    m = CacheManager([0], 8, 16, max_requests=2)
    m.open("a")
    m.extend("a", 0, 17)
    assert len(m.get("a").tables[0]) == 2
    m.commit("a", 17)
    m.extend("a", 17, 32)
    assert len(m.get("a").tables[0]) == 2        # position 31 still lies in the second page
    m.commit("a", 32)
    m.extend("a", 32, 33)
    assert len(m.get("a").tables[0]) == 3
    with pytest.raises(RuntimeError):
        m.extend("a", 40, 41)                    # rows must continue where the cache ends
    m.open("b")
    with pytest.raises(NoFreeSlot):
        m.open("c")
    assert m.pages_needed("b", 0, 16 * 5) == [5] and m.can_extend("b", 0, 16 * 5)
    assert not m.can_extend("b", 0, 16 * 5 + 1)
    with pytest.raises(NoFreePages):
        m.extend("b", 0, 16 * 5 + 1)
    m.check()
    m.close("a")
    m.close("b")
    m.check()
    assert m.pools[0].num_free() == 8 and m.free_slots() == 2


def test_windowed_group_gives_pages_back():
    m = CacheManager([0, 16], [16, 6], 16, max_requests=1)
    m.open("r")
    n = 0
    for step in [5, 30, 1, 1, 40, 1, 1, 64, 1]:
        m.extend("r", n, n + step)
        n += step
        m.commit("r", n)
        full, win = m.get("r").tables
        assert all(p >= 0 for p in full) and len(full) == (n + 15) // 16
        live = [i for i, p in enumerate(win) if p >= 0]
        # the next row (position n) reads keys n-15 .. n: pages from (n-15)//16 on are still there
        assert all(win[i] >= 0 for i in range(max(0, n - 15) // 16, len(win)))
        m.check()
    m.extend("r", n, n + 1)
    win = m.get("r").tables[1]
    assert sum(1 for p in win if p >= 0) <= 2    # one page of history plus the page being written
    # a portion too long for the windowed pool is refused: its own rows need the pages at once
    m.close("r")
    m.open("s")
    with pytest.raises(NoFreePages):
        m.extend("s", 0, 16 * 6 + 1)
    m.close("s")
    m.check()


def test_random_request_orders_lose_no_page():
    rng = random.Random(0)
    for trial in range(30):
        windows = rng.choice([[0], [0, 16], [0, 8, 32]])
        m = CacheManager(windows, rng.choice([6, 12, 40]), 16, max_requests=4)
        live, next_id = {}, 0
        for _ in range(300):
            op = rng.random()
            if op < 0.25 and len(live) < 4:
                m.open(next_id)
                live[next_id] = 0
                next_id += 1
            elif op < 0.35 and live:
                rid = rng.choice(list(live))
                m.close(rid)
                del live[rid]
            elif live:
                rid = rng.choice(list(live))
                n = rng.choice([1, 1, 1, 2, 7, 16, 33])
                start = live[rid]
                if m.can_extend(rid, start, start + n):
                    m.extend(rid, start, start + n)
                    m.commit(rid, start + n)
                    live[rid] = start + n
                else:
                    with pytest.raises(NoFreePages):
                        m.extend(rid, start, start + n)
            m.check()
        for rid in list(live):
            m.close(rid)
        m.check()
        assert all(p.num_free() == p.num_pages for p in m.pools) and m.free_slots() == 4


def test_prefix_pages_are_shared_and_never_the_last():
    m = CacheManager([0], 16, 4, max_requests=4, prefix_caching=True)
    toks = list(range(100, 111))                 # 11 tokens: two full pages and a part
    m.open("a")
    m.extend("a", 0, 11)
    m.commit("a", 11, toks)
    assert m.get("a").hashed_pages == 2
    matched = m.match_prefix(toks)               # the same prompt again: both full pages hit
    assert [p for p, _ in matched] == m.get("a").tables[0][:2]
    assert len(m.match_prefix(toks[:8])) == 1    # 8 tokens = exactly two pages: the last one is left to run
    assert m.match_prefix([1] + toks[1:]) == []
    m.open("b")
    assert m.adopt_prefix("b", matched) == 8
    m.extend("b", 8, 11)
    assert m.get("b").tables[0][:2] == m.get("a").tables[0][:2] and m.get("b").tables[0][2] != m.get("a").tables[0][2]
    m.check()
    m.close("a")
    m.check()                                    # shared pages stay with b
    m.close("b")
    matched = m.match_prefix(toks)               # both gone, hashes kept: revival
    assert len(matched) == 2 and m.new_pages_for(11, matched) == 3
    m.open("c")
    m.adopt_prefix("c", matched)
    m.check()
    # windows switch prefix sharing off: a hit must be a hit in every group
    assert not CacheManager([0, 16], 8, 4, 2, prefix_caching=True).prefix_caching


# ------------------------------------------------------------------------------- scheduler
def drive(sched, seqs, rng, max_steps=10000, check=None):
    """Runs the scheduler with a stand-in for the model (random tokens); returns per-step records."""
    for s in seqs:
        sched.add(s)
    records = []
    for _ in range(max_steps):
        if sched.is_finished():
            return records
        out = sched.schedule()
        assert out, "an unfinished scheduler must schedule something"
        assert len({s.seq.seq_id for s in out}) == len(out)
        assert sum(s.count for s in out) <= sched.max_num_batched_tokens
        assert len(out) <= sched.max_num_seqs
        for s in out:                               # the runner's view: pages are there for every row
            rc = sched.manager.get(s.seq.seq_id)
            assert rc.num_tokens == s.start
            assert all(len(t) * sched.manager.page_size >= s.start + s.count for t in rc.tables)
            assert s.samples == (s.start + s.count == s.seq.num_tokens)
        sched.manager.check()
        sampled = {s.seq.seq_id: rng.randrange(2, 50) for s in out if s.samples}
        records.append([(s.seq.seq_id, s.start, s.count, s.samples) for s in out])
        sched.postprocess(out, sampled)
        sched.manager.check()
        if check:
            check(out)
    raise AssertionError("the scheduler did not finish")


def make_sched(pages, *, windows=(0,), budget=64, max_seqs=8, prefix=False, chunk=0, max_len=4096, eos=-1):
    m = CacheManager(list(windows), pages, 16, max_requests=max_seqs, prefix_caching=prefix)
    return Scheduler(m, max_num_seqs=max_seqs, max_num_batched_tokens=budget, max_model_len=max_len, eos=eos,
                     prefill_chunk=chunk)


def test_budget_portions_and_mixed_steps():
    rng = random.Random(1)
    sched = make_sched(64, budget=32)
    seqs = [Sequence(list(range(2, 2 + n)), SamplingParams(max_tokens=6, ignore_eos=True)) for n in (70, 5, 40)]
    rec = drive(sched, seqs, rng)
    a = seqs[0].seq_id
    # the 70-token prompt is cut into 32 + 32 + 6; the rest of the third step's budget goes to the next prompt
    assert rec[0] == [(a, 0, 32, False)] and rec[1] == [(a, 32, 32, False)]
    assert rec[2][0] == (a, 64, 6, True) and rec[2][1][:3] == (seqs[1].seq_id, 0, 5)
    # later steps hold decode tokens of running sequences beside prompt portions of waiting ones
    assert any(any(c == 1 and st >= 70 for (_, st, c, _) in step) and any(c > 1 for (_, _, c, _) in step) for step in rec)
    assert all(s.is_finished and s.num_completion_tokens == 6 for s in seqs)
    assert all(p.num_free() == p.num_pages for p in sched.manager.pools)


def test_prefill_chunk_cap():
    sched = make_sched(64, budget=64, chunk=10)
    seq = Sequence(list(range(2, 27)), SamplingParams(max_tokens=1))
    rec = drive(sched, [seq], random.Random(2))
    assert [r[0][2] for r in rec] == [10, 10, 5]


def test_eos_max_tokens_and_max_model_len():
    sched = make_sched(64, eos=7, max_len=12)
    s1 = Sequence([2, 3, 4], SamplingParams(max_tokens=50))
    s2 = Sequence([2, 3, 4], SamplingParams(max_tokens=50, ignore_eos=True))
    sched.add(s1), sched.add(s2)
    out = sched.schedule()
    sched.postprocess(out, {s1.seq_id: 7, s2.seq_id: 7})
    assert s1.is_finished and not s2.is_finished          # the stop token ends s1 only
    while not sched.is_finished():
        out = sched.schedule()
        sched.postprocess(out, {s.seq.seq_id: 9 for s in out})
    assert s2.num_tokens == 12                            # stopped by max_model_len


def test_out_of_pages_preempts_newest_and_everything_finishes():
    rng = random.Random(3)
    # 3 requests x (20 prompt + 30 new) = 150 tokens -> 12 pages needed at the end; the pool has 8
    sched = make_sched(8, budget=64)
    seqs = [Sequence(list(range(2, 22)), SamplingParams(max_tokens=30, ignore_eos=True)) for _ in range(3)]
    rec = drive(sched, seqs, rng)
    assert sched.num_preemptions > 0
    assert seqs[0].num_preemptions == 0                   # the oldest request is never the victim here
    assert all(s.is_finished and s.num_completion_tokens == 30 for s in seqs)
    # a preempted request comes back with prompt and generated tokens as one prefill from position 0
    victim = max(seqs, key=lambda s: s.num_preemptions)
    again = [e for step in rec for e in step if e[0] == victim.seq_id and e[1] == 0]
    assert len(again) >= 2 and again[-1][2] > 20
    assert all(p.num_free() == p.num_pages for p in sched.manager.pools)


def test_random_workloads_with_tight_pools():
    rng = random.Random(4)
    for trial in range(25):
        windows = rng.choice([(0,), (0, 16)])
        sched = make_sched(rng.choice([8, 10, 16]), windows=windows, budget=rng.choice([16, 48, 200]),
                           max_seqs=rng.choice([2, 4, 8]), prefix=rng.random() < 0.5, chunk=rng.choice([0, 0, 7]))
        seqs = []
        for _ in range(rng.randrange(1, 9)):
            n = rng.choice([1, 3, 16, 17, 40, 64])
            base = rng.choice([100, 200])                 # common prefixes on purpose
            seqs.append(Sequence([base + i for i in range(n)], SamplingParams(max_tokens=rng.choice([1, 5, 30]), ignore_eos=True)))
        drive(sched, seqs, rng)
        assert all(s.is_finished for s in seqs)
        assert all(p.num_free() == p.num_pages for p in sched.manager.pools)
        assert sched.manager.free_slots() == sched.max_num_seqs


def drive_late(sched, seqs, rng, stop, max_steps=10000):
    """The order of an engine that queues step k+1 before it has read step k's tokens: the bookkeeping of step k
    runs with stand-ins (negative numbers), step k+1 is decided, then the tokens of step k arrive and are patched
    in; a stop token that arrives so ends its sequence late.  Returns the decisions per step."""
    for s in seqs:
        sched.add(s)
    records = []
    pending = sched.schedule()
    for _ in range(max_steps):
        if pending is None:
            assert sched.is_finished()
            return records
        cur = pending
        records.append([(s.seq.seq_id, s.start, s.count, s.samples) for s in cur])
        rows = [s.seq for s in cur if s.samples]
        before = [q.num_tokens for q in rows]
        finished = sched.postprocess(cur, {q.seq_id: -(r + 1) for r, q in enumerate(rows)})
        places = [n if q.num_tokens == n + 1 else None for q, n in zip(rows, before)]
        sched.manager.check()
        pending = sched.schedule() if not sched.is_finished() else None
        if pending is not None:
            assert pending, "an unfinished scheduler must schedule something"
            for s in pending:                        # the pages are there although the newest token is a stand-in
                rc = sched.manager.get(s.seq.seq_id)
                assert all(len(t) * sched.manager.page_size >= s.start + s.count for t in rc.tables)
        for q, place in zip(rows, places):           # the tokens of `cur` arrive
            if place is None:
                continue
            tok = rng.randrange(2, 50)
            sched.patch(q, place, tok)
            if tok == stop and not q.ignore_eos and not q.is_finished:
                sched.finish_late(q)
                finished.append(q)
        sched.manager.check()
        if pending is not None and not pending and sched.is_finished():
            pending = None
    raise AssertionError("the scheduler did not finish")


def test_tokens_that_arrive_a_step_late():
    rng = random.Random(11)
    for trial in range(25):
        windows = rng.choice([(0,), (0, 16)])
        sched = make_sched(rng.choice([8, 10, 16]), windows=windows, budget=rng.choice([16, 48, 200]),
                           max_seqs=rng.choice([2, 4, 8]), prefix=rng.random() < 0.5, chunk=rng.choice([0, 0, 7]),
                           eos=7)
        seqs = []
        for _ in range(rng.randrange(1, 9)):
            n = rng.choice([1, 3, 16, 17, 40, 64])
            base = rng.choice([100, 200])
            seqs.append(Sequence([base + i for i in range(n)],
                                 SamplingParams(max_tokens=rng.choice([1, 5, 30]), ignore_eos=rng.random() < 0.3)))
        drive_late(sched, seqs, rng, stop=7)
        for q in seqs:
            assert q.is_finished and all(t >= 0 for t in q.token_ids)       # no stand-in is left
            done = q.completion_token_ids
            if not q.ignore_eos and 7 in done:
                assert done.index(7) == len(done) - 1                       # nothing follows the stop token
            else:
                assert len(done) == q.max_tokens
        assert all(p.num_free() == p.num_pages for p in sched.manager.pools)
        assert sched.manager.free_slots() == sched.max_num_seqs


def test_pool_smaller_than_one_request_is_an_error():
    sched = make_sched(2, budget=64)
    sched.add(Sequence(list(range(2, 42)), SamplingParams(max_tokens=4)))
    with pytest.raises(SchedulerError, match="could not make progress"):
        for _ in range(10):
            out = sched.schedule()
            sched.postprocess(out, {s.seq.seq_id: 5 for s in out if s.samples})


def test_prefix_hit_skips_cached_pages():
    sched = make_sched(32, budget=256, prefix=True)
    p = list(range(2, 50))                                # 48 tokens = 3 full pages
    s1 = Sequence(p, SamplingParams(max_tokens=2, ignore_eos=True))
    drive(sched, [s1], random.Random(5))
    s2 = Sequence(p + [60, 61], SamplingParams(max_tokens=2, ignore_eos=True))
    rec = drive(sched, [s2], random.Random(5))
    assert rec[0] == [(s2.seq_id, 48, 2, True)]           # the three cached pages are not run again


def test_a_state_rules_prefix_sharing_out():
    """A layer with a per-request state has seen every token of its request: pages of another request must not
    let a request skip tokens.  So must a window, or a second group."""
    import plain_host
    for cls in (CacheManager, plain_host.CacheManager):
        assert cls([0], 8, 16, 4, prefix_caching=True).prefix_caching
        assert not cls([0], 8, 16, 4, prefix_caching=True, has_state=True).prefix_caching
        assert not cls([16], 8, 16, 4, prefix_caching=True).prefix_caching
        assert not cls([0, 16], 8, 16, 4, prefix_caching=True).prefix_caching
        assert not cls([], 8, 16, 4, prefix_caching=True, has_state=True).prefix_caching
    m = CacheManager([0], 16, 16, 4, prefix_caching=True, has_state=True)
    sched = Scheduler(m, max_num_seqs=4, max_num_batched_tokens=256, max_model_len=4096)
    p = list(range(2, 50))
    drive(sched, [Sequence(p, SamplingParams(max_tokens=2, ignore_eos=True))], random.Random(5))
    s2 = Sequence(p + [60, 61], SamplingParams(max_tokens=2, ignore_eos=True))
    rec = drive(sched, [s2], random.Random(5))
    assert rec[0] == [(s2.seq_id, 0, 50, True)]           # every token runs again


def test_a_model_without_pages_is_admitted_by_state_slots_alone():
    """No paged layer: the manager has no pool; requests hold a slot each, and the scheduler admits while slots
    are free, whatever their lengths."""
    import plain_host
    m = CacheManager([], 0, 16, max_requests=3, has_state=True)
    assert m.pools == [] and m.free_slots() == 3
    sched = Scheduler(m, max_num_seqs=8, max_num_batched_tokens=64, max_model_len=4096)
    seqs = [Sequence(list(range(2, 2 + n)), SamplingParams(max_tokens=5, ignore_eos=True)) for n in (70, 5, 40, 9, 200)]
    rec = drive(sched, seqs, random.Random(3), check=lambda out: None)
    assert all(len(step) <= 3 for step in rec)             # never more live requests than slots
    assert all(len(q.completion_token_ids) == 5 for q in seqs)
    assert m.free_slots() == 3
    # the plain restatement decides the same
    pm = plain_host.CacheManager([], 0, 16, max_requests=3, has_state=True)
    ps = plain_host.Scheduler(pm, max_num_seqs=8, max_num_batched_tokens=64, max_model_len=4096)
    qs = [plain_host.PlainSeq(100 + i, list(range(2, 2 + n)), 5) for i, n in enumerate((70, 5, 40, 9, 200))]
    for q in qs:
        ps.add(q)
    rng, prec = random.Random(3), []
    while not ps.is_finished():
        out = ps.schedule()
        prec.append([(s.start, s.count, s.samples) for s in out])
        ps.postprocess(out, {s.seq.seq_id: rng.randrange(2, 50) for s in out if s.samples})
    assert prec == [[(b, c, d) for _, b, c, d in step] for step in rec]


# ------------------------------------------------------------------------------- native code against its plain restatement
def test_native_host_code_decides_like_the_plain_restatement():
    """The native pool, manager and scheduler against the plain Python classes of tests/plain_host.py: the same
    random workloads, compared step by step (who runs, from where, how many tokens, which pages)."""
    import plain_host as ph
    rng = random.Random(11)
    for trial in range(40):
        windows = rng.choice([(0,), (0, 16), (0, 8, 32)])
        pages = rng.choice([8, 10, 16, 40])
        budget, max_seqs = rng.choice([16, 48, 200]), rng.choice([2, 4, 8])
        prefix, chunk = rng.random() < 0.5, rng.choice([0, 0, 7])
        native = make_sched(pages, windows=windows, budget=budget, max_seqs=max_seqs, prefix=prefix, chunk=chunk, eos=7)
        pm = ph.CacheManager(list(windows), pages, 16, max_requests=max_seqs, prefix_caching=prefix)
        plain = ph.Scheduler(pm, max_num_seqs=max_seqs, max_num_batched_tokens=budget, max_model_len=4096, eos=7,
                             prefill_chunk=chunk)
        pairs = []
        for i in range(rng.randrange(1, 9)):
            n, base = rng.choice([1, 3, 16, 17, 40, 64]), rng.choice([100, 200])
            toks, mt, ig = [base + j for j in range(n)], rng.choice([1, 5, 30]), rng.random() < 0.7
            a = Sequence(toks, SamplingParams(max_tokens=mt, ignore_eos=ig))
            b = ph.PlainSeq(a.seq_id, toks, mt, ig)
            native.add(a), plain.add(b)
            pairs.append((a, b))
        for step in range(5000):
            assert native.is_finished() == plain.is_finished()
            if native.is_finished():
                break
            try:
                out_p = plain.schedule()
            except ph.SchedulerError:
                with pytest.raises(SchedulerError):
                    native.schedule()
                break
            out_n = native.schedule()
            assert [(s.seq.seq_id, s.start, s.count, s.samples) for s in out_n] == \
                   [(s.seq.seq_id, s.start, s.count, s.samples) for s in out_p]
            for s in out_n:            # the same pages in every group
                assert native.manager.get(s.seq.seq_id).tables == pm.get(s.seq.seq_id).tables
            assert [p.num_free() for p in native.manager.pools] == [p.num_free() for p in pm.pools]
            sampled = {s.seq.seq_id: rng.choice([7, 9, 11, 13]) for s in out_n if s.samples}
            fin_n = native.postprocess(out_n, sampled)
            fin_p = plain.postprocess(out_p, sampled)
            assert [q.seq_id for q in fin_n] == [q.seq_id for q in fin_p]
            assert native.num_preemptions == plain.num_preemptions
            native.manager.check()
        for a, b in pairs:
            assert a.token_ids == b.token_ids and a.num_preemptions == b.num_preemptions
            assert a.is_finished == b.is_finished


def test_native_pool_and_hash_against_the_plain_restatement():
    import plain_host as ph
    rng = random.Random(12)
    for _ in range(20):
        toks = [rng.randrange(0, 1 << 20) for _ in range(rng.choice([1, 4, 16]))]
        prefix = rng.choice([None, rng.getrandbits(64)])
        assert chain_hash(toks, prefix) == ph.chain_hash(toks, prefix)
    a, b = BlockPool(6, 4), ph.BlockPool(6, 4)
    held = []
    for _ in range(400):
        op = rng.random()
        if op < 0.45 and a.num_free():
            pa, pb = a.allocate(), b.allocate()
            assert pa == pb
            held.append(pa)
            if rng.random() < 0.5:
                t = [rng.randrange(5) for _ in range(4)]
                h = chain_hash(t, None)
                a.set_hash(pa, h, t), b.set_hash(pb, h, t)
        elif op < 0.8 and held:
            p = held.pop(rng.randrange(len(held)))
            a.release(p), b.release(p)
        else:
            t = [rng.randrange(5) for _ in range(4)]
            h = chain_hash(t, None)
            la, lb = a.lookup(h, t), b.lookup(h, t)
            assert la == lb
            if la is not None and rng.random() < 0.5:
                a.share(la), b.share(lb)
                held.append(la)
        assert a.num_free() == b.num_free()
        assert [a.ref_count[p] for p in range(6)] == b.ref_count
        a.check()


def test_native_step_arrays_match_the_python_builder():
    """The native fill of a step's index arrays against ``build_batch`` on the same requests.  Block tables travel
    only when they have changed: the test keeps the tables by state slot as the device does, takes in what a step
    brings, and holds the result to the manager's own tables."""
    import numpy as np
    from nano_vllm_cpp_b200.engine.batch import StepEntry, EntryInfo, batch_layout
    from batch_builder import build_batch
    rng = random.Random(5)
    sent_total = entries_total = 0
    for trial in range(30):
        windows = rng.choice([(0,), (0, 16)])
        G = len(windows)
        m = CacheManager(list(windows), 64, 16, max_requests=6)
        max_blocks = 12
        live = {}
        device_tables = [dict() for _ in range(G)]          # per group: slot -> the table as the device has it
        last_sent = [dict() for _ in range(G)]              # per group: rid -> the table when it last travelled
        for step in range(8):
            entries = []
            for rid in rng.sample(["a", "b", 3, 4, "e"], rng.randrange(1, 5)):
                if not m.has(rid):
                    m.open(rid)
                    live[rid] = 0
                n = rng.choice([1, 1, 1, 2, 5, 17])
                if live[rid] + n > 150:
                    continue
                toks = [rng.randrange(1000) for _ in range(n)]
                want = sorted(rng.sample(range(n), rng.randrange(0, min(n, 3) + 1)))
                entries.append(StepEntry(rid, toks, want))
            if not entries:
                continue
            sampling = rng.random() < 0.5
            fixed_rows = len(entries) if rng.random() < 0.3 else 0
            S, T = len(entries), sum(len(e.tokens) for e in entries)
            W = sum(len(e.want) for e in entries)
            _, most = batch_layout(S, T, W, G, max_blocks, sampling)
            buf = np.full(most + 7, 12345, dtype=np.int32)
            used, slots, ids, sent = m.prepare_step(entries, max_blocks, 160, sampling, buf, fixed_rows)
            seg, total = batch_layout(S, T, W, G, max_blocks, sampling, None if fixed_rows else sent)
            assert used <= total <= most and (buf[used:] == 12345).all()
            if not fixed_rows:
                assert used == total
            infos, row0 = [], 0
            for e, (slot, pos0) in zip(entries, slots):
                assert (slot, pos0) == (m.get(e.rid).slot, live[e.rid])
                infos.append(EntryInfo(e.rid, slot, pos0, len(e.tokens), row0))
                row0 += len(e.tokens)
            tables = [[m.get(e.rid).tables[g] for e in entries] for g in range(G)]
            ref = build_batch(entries, infos, tables, max_blocks, "cpu")
            for name, t in (("ids", ref.input_ids), ("pos", ref.positions), ("row_entry", ref.row_entry),
                            ("cu", ref.cu_rows), ("pos0", ref.entry_pos0), ("slot", ref.entry_slot),
                            ("want", ref.want_rows)):
                o, n = seg[name]
                assert buf[o:o + n].tolist() == t.tolist(), name
            o, n = seg["single"]
            singles = [i.row0 for i in infos if i.length == 1]
            assert buf[o:o + n].tolist() == singles + [-1] * (S - len(singles))
            assert ref.single_rows.tolist() == singles and ref.n_single == len(singles)
            for g in range(G):
                src = buf[seg[f"tsrc{g}"][0]:][:S].tolist()
                lens = buf[seg[f"tlen{g}"][0]:][:S].tolist()
                rows = buf[seg[f"trows{g}"][0]:]
                assert sorted(x for x in src if x >= 0) == list(range(sent[g]))      # packed, each row used once
                for i, (e, info) in enumerate(zip(entries, infos)):
                    table = list(m.get(e.rid).tables[g])
                    assert lens[i] == len(table)
                    assert (src[i] >= 0) == (last_sent[g].get(e.rid) != table), (trial, step, e.rid)
                    if src[i] >= 0:
                        row = rows[src[i] * max_blocks:(src[i] + 1) * max_blocks].tolist()
                        assert row == table + [-1] * (max_blocks - len(table))
                        device_tables[g][info.slot] = row
                        last_sent[g][e.rid] = table
                    assert device_tables[g][info.slot][:lens[i]] == ref.block_tables[g][i, :lens[i]].tolist()
                sent_total += sent[g]
                entries_total += S
            m.commit_many(ids, [i.pos0 + i.length for i in infos])
            for e in entries:
                live[e.rid] += len(e.tokens)
                assert m.get(e.rid).num_tokens == live[e.rid]
            if rng.random() < 0.15:                      # a request ends; its slot goes to whoever opens next
                gone = rng.choice(sorted(live, key=str))
                m.close(gone)
                del live[gone]
                for g in range(G):
                    last_sent[g].pop(gone, None)
            if rng.random() < 0.1:                       # a prepared step never ran: everything travels again
                m.invalidate_tables()
                for g in range(G):
                    last_sent[g].clear()
        m.check()
    assert 0 < sent_total < entries_total                # some tables stayed at home
    # a step that fails sends nothing and leaves every table still to be sent
    m = CacheManager([0], 4, 16, max_requests=2)
    m.open("p"), m.open("q")
    buf = np.zeros(512, dtype=np.int32)
    with pytest.raises(Exception):
        m.prepare_step([StepEntry("p", [1] * 20, []), StepEntry("q", [1] * 60, [])], 8, 1000, False, buf)
    used, _, ids, sent = m.prepare_step([StepEntry("p", [1] * 20, [])], 8, 1000, False, buf)
    assert sent == [1]
    m.commit_many(ids, [20])
    used, _, ids, sent = m.prepare_step([StepEntry("p", [1], [])], 8, 1000, False, buf)
    assert sent == [0]                                   # position 20 lies in a page that the request holds already
    # errors: a place that is not among the tokens, an entry without tokens, too long a sequence
    m = CacheManager([0], 8, 16, max_requests=2)
    m.open("x")
    buf = np.zeros(256, dtype=np.int32)
    with pytest.raises(ValueError, match="wanted place"):
        m.prepare_step([StepEntry("x", [1, 2], [2])], 4, 100, False, buf)
    with pytest.raises(ValueError, match="exceed"):
        m.prepare_step([StepEntry("x", list(range(40)), [])], 4, 30, False, buf)
    with pytest.raises(NoFreePages):
        m.prepare_step([StepEntry("x", list(range(16 * 9)), [])], 16, 1000, False, np.zeros(1024, dtype=np.int32))


# ------------------------------------------------------------------------------- the reference's block manager
@pytest.mark.parametrize("which", ["native", "plain"])
def test_pages_handed_out_as_the_reference_block_manager_does(which):
    """The scripted life of a few requests of tests/golden/make_golden_blocks.py on this engine's cache manager
    (and on its plain restatement): cached pages on admission, every block table and the number of free pages
    after every line equal what the reference's own BlockManager (src/block_manager.cpp) recorded."""
    import json
    import os
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "golden"))
    import make_golden_blocks as G
    import plain_host
    with open(os.path.join(here, "golden", "ref_block_manager.json")) as f:
        gold = json.load(f)
    cls = CacheManager if which == "native" else plain_host.CacheManager
    m = cls([0], G.PAGES, G.PAGE, max_requests=8, prefix_caching=True)
    tokens = {}
    for line, want in zip(G.SCRIPT, gold):
        op, name = line[0], line[1]
        if op == "admit":
            tokens[name] = list(line[2])
            matched = m.match_prefix(tokens[name])
            assert len(matched) == want["cached_pages"], line
            m.open(name)
            cached = m.adopt_prefix(name, matched)
            m.extend(name, cached, len(tokens[name]))
            m.commit(name, len(tokens[name]), tokens[name])
        elif op == "decode":
            tokens[name].append(line[2])
            n = len(tokens[name])
            m.extend(name, n - 1, n)
            m.commit(name, n, tokens[name])
        else:
            m.close(name)
        m.check()
        assert m.pools[0].num_free() == want["free"], line
        if op != "end":
            assert m.get(name).tables[0] == want["table"], line
