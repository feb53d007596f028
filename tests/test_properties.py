"""Property tests (hypothesis): whatever the order of operations, the cache manager accounts for
every page and slot; however a request's tokens are cut into steps and mixed with another
request's, the logits at a position are those of the whole sequence.  The cutting property runs on
the host with the plain stand-ins of the kernels (``-m "not gpu"``) and on the GPU with the real
ones (``-m gpu``)."""
from __future__ import annotations

import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

import plain_kernels
import plain_llama
import replay_cases as rc
from kvcore_b200.cache import CacheGroupSpec, KVManager


# ---- cache manager ---------------------------------------------------------------------------
OPERATIONS = st.lists(
    st.tuples(st.sampled_from(["start", "grow", "end"]), st.integers(0, 7), st.integers(1, 23)),
    min_size=1, max_size=120,
)


@settings(max_examples=60, deadline=None)
@given(ops=OPERATIONS, windows=st.sampled_from([(None,), (None, 7), (5, None, 9)]),
       num_pages=st.integers(6, 30), page_size=st.sampled_from([2, 4, 8]))
def test_cache_manager_accounts_for_every_page(ops, windows, num_pages, page_size):
    groups = [CacheGroupSpec(i, (i,), 2, 2, 16, w) for i, w in enumerate(windows)]
    kv = KVManager(groups, num_pages=num_pages, page_size=page_size, max_num_seqs=4, max_model_len=64)
    live: dict[str, int] = {}
    for action, which, amount in ops:
        rid = f"r{which}"
        if action == "start" and rid not in live:
            before = kv.num_free_pages()
            if len(live) < 4 and kv.allocate_slots(rid, amount):
                kv.advance(rid, amount)
                live[rid] = amount
            else:
                assert kv.num_free_pages() == before and not kv.has_request(rid)
        elif action == "grow" and rid in live:
            before = kv.num_free_pages()
            if live[rid] + amount <= 64 and kv.allocate_slots(rid, amount):
                kv.advance(rid, amount)
                live[rid] += amount
            else:
                assert kv.num_free_pages() == before      # a refused allocation changes nothing
        elif action == "end" and rid in live:
            kv.free(rid)
            del live[rid]
        kv.check_invariants()
        assert sorted(kv.live_requests()) == sorted(live)
        for request, tokens in live.items():
            assert kv.num_computed(request) == tokens
            for group, window in enumerate(windows):
                held = sum(1 for page in kv.block_ids(request)[group] if page)
                needed = -(-tokens // page_size)
                assert held <= needed
                if window is None:
                    assert held == needed                  # a full group keeps every page
        slots = [kv.state_slot(request) for request in live]
        assert len(set(slots)) == len(slots)
    for request in list(live):
        kv.free(request)
    kv.check_invariants()
    assert kv.num_free_pages() == [num_pages - 1] * len(windows) and kv.slots.num_free == 4
    assert not any(np.any(table) for table in kv.tables)


# ---- cuttings --------------------------------------------------------------------------------
LENGTHS = {"a": 37, "b": 22}
LONG_LENGTHS = {"a": 230, "b": 141}     # several key tiles and row tiles: the serving kernels' shapes


def _model(tmp_path_factory, name, lengths=LENGTHS):
    config = rc.TINY_CONFIGS[name]
    folder = tmp_path_factory.mktemp(f"prop_{name}")
    rc.write_model(folder, config, rc.TINY_SEEDS[name], "bfloat16")
    weights = plain_llama.load_weights(folder)
    requests = {rid: rc.random_tokens(config["vocab_size"], n, 40 + i) for i, (rid, n) in enumerate(lengths.items())}
    reference = {rid: plain_llama.forward_logits(config, weights, tokens).numpy() for rid, tokens in requests.items()}
    return dict(config=config, folder=folder, requests=requests, reference=reference)


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    return _model(tmp_path_factory, "A")


@pytest.fixture(scope="module", params=[("B", LENGTHS), ("D", LONG_LENGTHS)], ids=["B", "D-long"])
def model_gpu(tmp_path_factory, request):
    return _model(tmp_path_factory, *request.param)


def _trace(requests, sizes_a, sizes_b, order):
    """Steps from two lists of portion sizes (cycled until the tokens run out); ``order`` decides
    step by step whether a, b or both bring their next portion."""
    portions = {"a": rc.cut(requests["a"], sizes_a), "b": rc.cut(requests["b"], sizes_b)}
    cursor = {"a": 0, "b": 0}
    steps, turn = [], 0
    while any(cursor[r] < len(portions[r]) for r in portions):
        choice = order[turn % len(order)]
        turn += 1
        chosen = [r for r in ("a", "b") if r in choice and cursor[r] < len(portions[r])]
        if not chosen:
            chosen = [r for r in ("a", "b") if cursor[r] < len(portions[r])][:1]
        entries, ended = [], []
        for rid in chosen:
            portion = portions[rid][cursor[rid]]
            cursor[rid] += 1
            entries.append({"id": rid, "tokens": portion, "want": list(range(len(portion)))})
            if cursor[rid] == len(portions[rid]):
                ended.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def _check_cutting(case, steps, out_dir, dtype, device, tolerance):
    vocab = case["config"]["vocab_size"]
    rc.run_inprocess(case["folder"], dtype, steps, out_dir, rc.peak_tokens(steps), device=device)
    rows = rc.collect(steps, out_dir, vocab)
    assert len(rows) == sum(len(tokens) for tokens in case["requests"].values())
    for (rid, position), row in rows.items():
        reference = case["reference"][rid]
        error = np.abs(row - reference[position]).max() / np.abs(reference).max()
        assert error <= tolerance, f"{rid}: position {position} is off by {error:.3e}"


SIZES = st.lists(st.integers(1, 12), min_size=1, max_size=6)
LONG_SIZES = st.lists(st.one_of(st.integers(1, 12), st.integers(13, 90)), min_size=1, max_size=6)
ORDER = st.lists(st.sampled_from(["a", "b", "ab"]), min_size=1, max_size=5)


@settings(max_examples=12, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(sizes_a=SIZES, sizes_b=SIZES, order=ORDER)
def test_any_cutting_gives_the_logits_of_the_whole_sequence_on_the_host(model_a, tmp_path_factory, monkeypatch,
                                                                        sizes_a, sizes_b, order):
    plain_kernels.install(monkeypatch)
    steps = _trace(model_a["requests"], sizes_a, sizes_b, order)
    _check_cutting(model_a, steps, tmp_path_factory.mktemp("cut"), "float32", "cpu", 2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tolerance", [("float32", 2e-5), ("bfloat16", 2e-2)])
def test_any_cutting_gives_the_logits_of_the_whole_sequence(model_gpu, tmp_path_factory, dtype, tolerance):
    sizes = LONG_SIZES if len(model_gpu["requests"]["a"]) > 100 else SIZES

    @settings(max_examples=10, deadline=None)
    @given(sizes_a=sizes, sizes_b=sizes, order=ORDER)
    def run(sizes_a, sizes_b, order):
        steps = _trace(model_gpu["requests"], sizes_a, sizes_b, order)
        _check_cutting(model_gpu, steps, tmp_path_factory.mktemp("cut"), dtype, "cuda:0", tolerance)

    run()


# ---- scheduler -------------------------------------------------------------------------------
@settings(max_examples=60, deadline=None)
@given(
    arrivals=st.lists(st.tuples(st.integers(0, 6), st.integers(1, 30), st.integers(1, 9)), min_size=1, max_size=10),
    num_pages=st.integers(10, 40), budget=st.integers(2, 24), max_seqs=st.integers(1, 5),
    partial=st.integers(1, 3), prefix=st.booleans(),
)
def test_scheduler_finishes_every_request_within_its_limits(arrivals, num_pages, budget, max_seqs, partial, prefix):
    """Requests of random lengths arriving at random steps, with few pages: every step stays inside
    the token and request limits, a request's tokens are scheduled in order and once, every request
    ends with exactly max_tokens outputs (pre-emption on deadlock), and all pages come back."""
    from kvcore_b200.config import SchedulerConfig
    from kvcore_b200.engine.request import Request
    from kvcore_b200.engine.scheduler import Scheduler
    from kvcore_b200.sampling import SamplingParams

    page_size, max_model_len = 4, 40
    kv = KVManager([CacheGroupSpec(0, (0, 1), 2, 2, 16, None)], num_pages=num_pages, page_size=page_size,
                   max_num_seqs=max_seqs, max_model_len=max_model_len, enable_prefix_caching=prefix)
    sched = Scheduler(SchedulerConfig(max_num_seqs=max_seqs, max_num_scheduled_tokens=budget,
                                      max_num_partial_prefills=partial, max_long_partial_prefills=partial), kv)
    todo = sorted(
        (when, f"r{i}", n, out) for i, (when, n, out) in enumerate(arrivals)
        # a request must fit the model length and, alone, the cache
        if n + out <= max_model_len and -(-(n + out) // page_size) <= num_pages - 1
    )
    expected = {rid: out for _, rid, _, out in todo}
    outputs: dict[str, int] = {}
    finished: set[str] = set()
    step = 0
    while todo or sched.has_unfinished_requests():
        while todo and todo[0][0] <= step:
            _, rid, n, out = todo.pop(0)
            sched.add_request(Request(rid, [1 + (j * 7 + len(rid)) % 5 for j in range(n)],
                                      SamplingParams(max_tokens=out, temperature=0.0)))
        plan = sched.schedule()
        assert plan.total_num_scheduled_tokens <= budget
        assert len(plan.num_scheduled_tokens) <= max_seqs
        assert plan.total_num_scheduled_tokens == sum(plan.num_scheduled_tokens.values())
        sampled = {}
        for rid, n in plan.num_scheduled_tokens.items():
            assert n >= 1 and rid not in finished
            assert not any(kv.pages_needed(rid, n))        # its pages are there before the step
            kv.advance(rid, n)
            sampled[rid] = 3
        update = sched.update_from_outputs(plan, sampled, stop_token_ids=None)
        for out in update.step_outputs:
            if out.sampled_token_id is not None:
                outputs[out.request_id] = outputs.get(out.request_id, 0) + 1
        for done in update.finished_requests:
            finished.add(done.request_id)
            assert len(done.output_token_ids) == expected[done.request_id]
        kv.check_invariants()
        step += 1
        assert step < 2000, "the scheduler makes no progress"
    assert finished == set(expected)
    sched.schedule()                                       # reports the last finished ids
    assert not kv.live_requests()
    kv.check_invariants()


# ---- one step kept in flight -----------------------------------------------------------------
@pytest.fixture(scope="module")
def model_for_engine(tmp_path_factory):
    folder = tmp_path_factory.mktemp("engine_model")
    rc.write_model(folder, rc.TINY_CONFIGS["A"], 3, "float32")
    return folder


@settings(max_examples=10, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])
@given(
    arrivals=st.lists(st.tuples(st.integers(0, 12), st.integers(1, 30), st.integers(1, 9)), min_size=1, max_size=7),
    num_pages=st.integers(12, 40), budget=st.integers(4, 32), max_seqs=st.integers(1, 4),
    stops=st.lists(st.integers(0, 255), min_size=0, max_size=40),
)
def test_keeping_a_step_in_flight_never_changes_what_comes_out(model_for_engine, monkeypatch, arrivals, num_pages,
                                                                 budget, max_seqs, stops):
    """Random arrivals, lengths, limits, stop tokens and few pages (waiting, preemption): the engine
    with a step in flight returns, request by request, the tokens and finish reasons of the engine
    without, and gives every page back."""
    import json

    from kvcore_b200 import (CacheConfig, DeviceConfig, KVCoreConfig, LoadConfig, ModelConfig, SamplingParams,
                             SchedulerConfig)
    from kvcore_b200.engine.llm_engine import LLMEngine

    plain_kernels.install(monkeypatch)
    config = json.loads((model_for_engine / "config.json").read_text())
    config["eos_token_id"] = sorted(set(stops)) or None
    (model_for_engine / "config.json").write_text(json.dumps({k: v for k, v in config.items() if v is not None}))
    requests = [(step, f"r{i}", rc.random_tokens(256, length, 200 + i), max_tokens)
                for i, (step, length, max_tokens) in enumerate(arrivals)]

    def run(run_ahead: bool):
        engine = LLMEngine(KVCoreConfig(
            model_config=ModelConfig(model=str(model_for_engine), dtype="float32", max_model_len=48),
            load_config=LoadConfig(),
            cache_config=CacheConfig(block_size=4, num_gpu_blocks=num_pages),
            scheduler_config=SchedulerConfig(max_num_seqs=max_seqs, max_num_scheduled_tokens=budget,
                                             max_num_partial_prefills=2, max_long_partial_prefills=2,
                                             run_ahead=run_ahead),
            device_config=DeviceConfig(device="cpu"),
        ))
        core = engine.engine_core
        seen: dict[str, list[int]] = {}
        step = 0
        pending = sorted(requests)
        while pending or core.has_unfinished_requests():
            while pending and pending[0][0] <= step:
                _, rid, prompt, max_tokens = pending.pop(0)
                engine.add_request(rid, SamplingParams(max_tokens=max_tokens, temperature=0.0), prompt_token_ids=prompt)
            for out in engine.step().request_outputs:
                if out.sampled_token_id is not None:
                    seen.setdefault(out.request_id, []).append(out.sampled_token_id)
            step += 1
            assert step < 600, "no progress"
        finished = {rid: core.take_finished_output(rid) for _, rid, _, _ in requests}
        kv = core.model_runner.kv_manager
        kv.check_invariants()
        assert not kv.live_requests() and core._in_flight is None and not core.model_runner.requests
        # a preempted request is recomputed, but the tokens it reported stay the tokens it has
        assert {rid: list(f.output_token_ids) for rid, f in finished.items()} == seen
        return {rid: (f.output_token_ids, f.finish_reason) for rid, f in finished.items()}, core.num_steps_run_ahead

    with_ahead, launched = run(True)
    without, none = run(False)
    assert none == 0
    assert with_ahead == without
