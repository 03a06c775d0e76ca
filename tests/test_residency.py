"""Replica-cache scheduling: which chunk leaves (FIFO, Belady on a trace), gathers ahead of time, and the
module-level residency hooks.  CPU: the schedulers on stand-in chunks, the rest on gloo ranks with the
host-memory shim serving the elx_* ABI (the scheduling logic is all Python)."""
import pytest
import torch
import torch.multiprocessing as mp

import _dist_workers as W
from _util import free_port
from elixir_b200.chunk import FIFOScheduler, PrefetchScheduler


class FakeChunk:
    """What a scheduler needs of a chunk: identity and an order."""

    def __init__(self, chunk_id):
        self.chunk_id = chunk_id

    def __hash__(self):
        return self.chunk_id

    def __eq__(self, other):
        return self.chunk_id == other.chunk_id

    def __lt__(self, other):
        return self.chunk_id < other.chunk_id

    def __repr__(self):
        return f'c{self.chunk_id}'


def test_fifo_releases_in_order_of_becoming_releasable():
    a, b, c, d = (FakeChunk(i) for i in range(4))
    s = FIFOScheduler()
    s.reset()
    assert s.top() is None
    for x in (c, a, b):
        assert s.add(x)
    assert not s.add(c)    # already there: keeps its place
    assert s.top() is c
    assert s.remove(c) and not s.remove(c) and not s.remove(d)
    assert s.top() is a
    s.add(c)    # back of the queue
    s.remove(a)
    assert s.top() is b
    s.remove(b)
    assert s.top() is c
    s.remove(c)
    assert s.top() is None
    s.clear()
    with pytest.raises(AssertionError):
        s.reset()
        s.add(a)
        s.clear()    # a chunk still waiting at the end of the pass


def test_belady_releases_the_chunk_used_furthest_ahead():
    a, b, c = (FakeChunk(i) for i in range(3))
    trace = [[a], [b], [c], [a], [a, b], [c], [b]]
    s = PrefetchScheduler(trace)
    with torch.enable_grad():
        s.reset()
        s.step([a])    # step 0
        assert s.next_use(a) == 3 and s.next_use(b) == 1 and s.next_use(c) == 2
        s.add(a)
        s.step([b])    # step 1
        s.add(b)    # next use of b: 4, of a: 3
        assert s.top() is b
        s.step([c])    # step 2
        s.add(c)    # next use of c: 5
        assert s.top() is c
        assert s.get_next_chunk([c]) is a
        assert list(s.upcoming(exclude=[c])) == [(3, a), (4, b)]
        s.remove(a)
        s.step([a])    # step 3
        s.add(a)    # a again at 4
        assert s.top() is c
        s.remove(c)
        assert s.top() in (a, b) and s.top() is b    # both next used at step 4: the larger id goes
        s.remove(a), s.remove(b)
        s.step([a, b])    # step 4
        s.add(a)    # never used again: 7 = len(trace)
        s.add(b)    # 6
        assert s.next_use(a) == 7 and s.top() is a
        s.step([c])
        s.step([b])
        with pytest.raises(RuntimeError):
            s.step([a])    # the pass is longer than the trace
        s.remove(a), s.remove(b)
        s.current_step = 6
        s.clear()


def test_prefetch_scheduler_learns_the_trace_from_the_first_pass():
    a, b, c = (FakeChunk(i) for i in range(3))
    s = PrefetchScheduler()
    assert s.learning
    with torch.no_grad():    # a pass without gradients is not the training trace
        s.reset()
        s.step([a])
        s.clear()
    assert s.learning
    with torch.enable_grad():
        s.reset()
        for step in ([a], [b, c], [a], [c]):
            s.step(step)
            for x in step:
                s.add(x)
            assert s.top() is a    # FIFO while learning
            assert s.get_next_chunk(step) is None and list(s.upcoming()) == []
        for x in (a, b, c):
            s.remove(x)
        s.clear()
        assert not s.learning and s.total_steps == 4
        s.reset()
        s.step([a])
        assert s.next_use(a) == 2 and s.next_use(b) == 1 and s.next_use(c) == 1
        assert list(s.upcoming(exclude=[a])) == [(1, b), (1, c)]
        s.relearn()
        assert s.learning


@pytest.mark.parametrize('world', [1, 2])
@pytest.mark.parametrize('prefetch', [False, True])
def test_scheduled_residency_equals_everything_resident(world, prefetch):
    mp.spawn(W.residency_worker, args=(world, free_port(), prefetch, 'float32'), nprocs=world)


def test_micro_gpt2_trains_identically_in_both_residency_modes_and_follows_plain_adamw():
    pytest.importorskip('transformers')
    mp.spawn(W.gpt2_worker, args=(1, free_port()), nprocs=1)


def test_an_abandoned_forward_gives_its_blocks_back():
    mp.spawn(W.abandoned_pass_worker, args=(1, free_port()), nprocs=1)


def test_dropping_the_wrapper_frees_model_and_optimizer_state():
    mp.spawn(W.lifetime_worker, args=(1, free_port()), nprocs=1)


def test_fetcher_decisions_on_a_spelled_out_trace():
    mp.spawn(W.fetcher_scenario_worker, args=(1, free_port()), nprocs=1)


@pytest.mark.parametrize('world', [1, 2])
def test_injected_gradients_land_identically_with_a_small_replica_cache(world):
    mp.spawn(W.inject_worker, args=(world, free_port()), nprocs=world)


def _simulate(scheduler, trace, chunks, blocks, check_top=None):
    """Drive a scheduler the way the fetcher does (one chunk per fetch, released right after use) and count the
    fetches that found their chunk absent."""
    resident, misses = set(), 0
    with torch.no_grad():
        scheduler.reset()
        for step, i in enumerate(trace):
            chunk = chunks[i]
            scheduler.remove(chunk)
            scheduler.step([chunk])
            if chunk not in resident:
                misses += 1
                if len(resident) == blocks:
                    victim = scheduler.top()
                    assert victim is not None and victim in resident and victim is not chunk
                    if check_top is not None:
                        check_top(step, victim, resident - {chunk})
                    scheduler.remove(victim)
                    resident.remove(victim)
                resident.add(chunk)
            scheduler.add(chunk)
        for chunk in list(resident):
            scheduler.remove(chunk)
        scheduler.clear()
    return misses


def test_belady_choice_is_the_furthest_next_use_and_never_loses_to_fifo():
    hypothesis = pytest.importorskip('hypothesis')
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.lists(st.integers(0, 5), min_size=1, max_size=40), st.integers(1, 4))
    def run(trace, blocks):
        chunks = [FakeChunk(i) for i in range(6)]

        def brute_force(step, victim, candidates):
            def next_use(c):
                later = [s for s in range(step + 1, len(trace)) if trace[s] == c.chunk_id]
                return later[0] if later else len(trace)
            best = max(candidates, key=lambda c: (next_use(c), c.chunk_id))
            assert victim is best, (trace, blocks, step)

        belady = _simulate(PrefetchScheduler([[chunks[i]] for i in trace]), trace, chunks, blocks, brute_force)
        fifo = _simulate(FIFOScheduler(), trace, chunks, blocks)
        assert belady <= fifo, (trace, blocks, belady, fifo)
        assert belady >= len(set(trace))    # every chunk has to come in at least once

    run()


def test_schedulers_give_up_the_chunks_the_reference_schedulers_give_up():
    """tests/golden/scheduler.json: evictions of the reference's own FIFOScheduler / PrefetchScheduler on 40
    seeded random traces (generated by tests/golden/make_golden.py); ties included, the sequences are equal."""
    import json
    import os
    import sys
    sys.path.insert(0, W.GOLDEN)
    from make_golden import StandIn, drive_scheduler, scheduler_cases
    cases = json.load(open(os.path.join(W.GOLDEN, 'scheduler.json')))
    assert [(c['trace'], c['blocks']) for c in cases] == [(t, b) for t, b in scheduler_cases()]
    evictions = 0
    for case in cases:
        trace, blocks = case['trace'], case['blocks']
        stand_ins = {i: StandIn(i) for i in set(trace)}
        with torch.enable_grad():
            got = drive_scheduler(PrefetchScheduler([[stand_ins[i]] for i in trace]), trace, blocks, step_with_chunks=True)
            assert got == case['prefetch_victims'], (trace, blocks)
            got = drive_scheduler(FIFOScheduler(), trace, blocks, step_with_chunks=True)
            assert got == case['fifo_victims'], (trace, blocks)
        evictions += len(case['prefetch_victims']) + len(case['fifo_victims'])
    assert evictions > 500
