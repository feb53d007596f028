"""The scheduler's decisions: portions under a token budget, running before waiting, the limit
on partial prefills, finishing and freeing, and what happens when pages run out."""
from __future__ import annotations

import pytest

from kvcore_b200.cache import CacheGroupSpec, KVManager
from kvcore_b200.config import SchedulerConfig
from kvcore_b200.engine.request import FinishReason, Request, RequestStatus
from kvcore_b200.engine.scheduler import Scheduler
from kvcore_b200.sampling import SamplingParams


def make(num_pages=33, page_size=4, max_model_len=64, prefix_caching=False, **cfg):
    kv = KVManager([CacheGroupSpec(0, (0, 1), 2, 2, 16, None)], num_pages=num_pages, page_size=page_size,
                   max_num_seqs=cfg.get("max_num_seqs", 8), max_model_len=max_model_len,
                   enable_prefix_caching=prefix_caching)
    return Scheduler(SchedulerConfig(**cfg), kv), kv


def request(rid, n, max_tokens=4, **params):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, temperature=0.0, **params))


def run_step(sched, kv, tokens=None, stop=None):
    """schedule + pretend the model ran + update; returns (output, update)."""
    out = sched.schedule()
    sampled = {}
    for rid, n in out.num_scheduled_tokens.items():
        kv.advance(rid, n)
        sampled[rid] = (tokens or {}).get(rid, 7)
    return out, sched.update_from_outputs(out, sampled, stop_token_ids=stop)


def test_chunked_prefill_then_decode_then_finish():
    sched, kv = make(max_num_scheduled_tokens=5, max_num_seqs=4)
    sched.add_request(request("a", 12, max_tokens=2))
    out, upd = run_step(sched, kv)
    assert out.scheduled_new_reqs[0].req_id == "a" and out.num_scheduled_tokens == {"a": 5}
    assert out.scheduled_new_reqs[0].num_computed_tokens == 0
    assert upd.step_outputs[0].sampled_token_id is None  # a middle portion samples nothing
    out, upd = run_step(sched, kv)
    assert out.scheduled_cached_reqs.req_ids == ("a",) and out.scheduled_cached_reqs.new_token_ids == ((6, 7, 8, 9, 10),)
    assert out.scheduled_cached_reqs.num_computed_tokens == (5,)
    out, upd = run_step(sched, kv)
    assert out.num_scheduled_tokens == {"a": 2} and upd.step_outputs[0].sampled_token_id == 7
    out, upd = run_step(sched, kv)  # decode: one token
    assert out.num_scheduled_tokens == {"a": 1} and out.scheduled_cached_reqs.new_token_ids == ((7,),)
    assert upd.finished_requests[0].finish_reason == FinishReason.LENGTH
    assert upd.finished_requests[0].output_token_ids == (7, 7)
    assert not sched.has_unfinished_requests() and kv.num_free_pages() == [32]
    out = sched.schedule()
    assert out.finished_req_ids == frozenset({"a"}) and out.total_num_scheduled_tokens == 0


def test_running_requests_go_first_and_budget_is_shared():
    sched, kv = make(max_num_scheduled_tokens=8, max_num_partial_prefills=4, max_long_partial_prefills=4)
    sched.add_request(request("a", 3))
    sched.add_request(request("b", 20))
    out, _ = run_step(sched, kv)
    assert out.num_scheduled_tokens == {"a": 3, "b": 5}
    out, _ = run_step(sched, kv)  # a decodes (1), b takes the rest of the budget
    assert list(out.num_scheduled_tokens.items()) == [("a", 1), ("b", 7)]


def test_partial_prefill_limit_skips_to_a_later_request():
    sched, kv = make(max_num_scheduled_tokens=6, max_num_partial_prefills=1)
    sched.add_request(request("a", 10))
    sched.add_request(request("b", 10))
    out, _ = run_step(sched, kv)
    assert out.num_scheduled_tokens == {"a": 6}  # one prefill at a time
    out, _ = run_step(sched, kv)
    assert out.num_scheduled_tokens == {"a": 4}
    out, _ = run_step(sched, kv)  # a decodes, b may now start
    assert out.num_scheduled_tokens == {"a": 1, "b": 5}
    assert [r.request_id for r in sched.running] == ["a", "b"]


def test_long_prefill_threshold_caps_a_portion():
    sched, kv = make(max_num_scheduled_tokens=100, long_prefill_token_threshold=4, max_num_partial_prefills=2,
                     max_long_partial_prefills=1)
    sched.add_request(request("a", 10))
    sched.add_request(request("b", 10))
    sched.add_request(request("c", 2))
    out, _ = run_step(sched, kv)
    assert out.num_scheduled_tokens == {"a": 4, "c": 2}  # b is a second long prefill: skipped, c is short


def test_max_num_seqs():
    sched, kv = make(max_num_seqs=2, max_num_scheduled_tokens=100, max_num_partial_prefills=8)
    for rid in "abc":
        sched.add_request(request(rid, 3))
    out, _ = run_step(sched, kv)
    assert set(out.num_scheduled_tokens) == {"a", "b"}


def test_stop_token_and_abort():
    sched, kv = make(max_num_scheduled_tokens=100, max_num_partial_prefills=8)
    sched.add_request(request("a", 3, max_tokens=10))
    sched.add_request(request("b", 3, max_tokens=10))
    _, upd = run_step(sched, kv, tokens={"a": 99, "b": 5}, stop={99})
    assert [f.request_id for f in upd.finished_requests] == ["a"]
    assert upd.finished_requests[0].finish_reason == FinishReason.STOP
    finished = sched.finish_requests("b", RequestStatus.FINISHED_ABORTED)
    assert finished[0].finish_reason == FinishReason.ABORT and kv.num_free_pages() == [32]
    assert not sched.has_unfinished_requests()


def test_admission_checks():
    sched, kv = make(num_pages=5, page_size=4, max_model_len=32)
    with pytest.raises(ValueError, match="never"):
        sched.add_request(request("big", 20))
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add_request(request("long", 32))
    sched.add_request(request("a", 3))
    with pytest.raises(ValueError, match="Duplicate"):
        sched.add_request(request("a", 3))
    with pytest.raises(ValueError):
        Request("empty", [], SamplingParams(max_tokens=1))


def test_generation_stops_at_max_model_len():
    sched, kv = make(max_model_len=6, max_num_scheduled_tokens=100)
    sched.add_request(request("a", 4, max_tokens=50))
    reasons = []
    while sched.has_unfinished_requests():
        _, upd = run_step(sched, kv)
        reasons += [f.finish_reason for f in upd.finished_requests]
    assert reasons == [FinishReason.LENGTH]


def test_waiting_request_waits_when_pages_run_out():
    sched, kv = make(num_pages=6, page_size=4, max_num_scheduled_tokens=100, max_num_partial_prefills=8)
    sched.add_request(request("a", 12, max_tokens=2))  # 3 pages (+1 for the second token)
    sched.add_request(request("b", 12, max_tokens=2))
    out, _ = run_step(sched, kv)
    assert set(out.num_scheduled_tokens) == {"a"}  # b does not fit: it stays queued, untouched
    assert [r.request_id for r in sched.waiting] == ["b"] and not kv.has_request("b")
    run_step(sched, kv)
    assert not kv.has_request("a")  # finished and freed
    out, _ = run_step(sched, kv)
    assert set(out.num_scheduled_tokens) == {"b"}  # on pages that a held before
    kv.check_invariants()


def test_deadlock_preempts_the_youngest_and_recomputes_it():
    sched, kv = make(num_pages=5, page_size=4, max_num_scheduled_tokens=100, max_num_partial_prefills=8)
    sched.add_request(request("a", 7, max_tokens=8))
    sched.add_request(request("b", 7, max_tokens=8))
    run_step(sched, kv)  # both prefilled: 2 pages each, pool empty; both sampled a token
    out, _ = run_step(sched, kv)  # both fit their 8th token in the second page
    assert set(out.num_scheduled_tokens) == {"a", "b"}
    out, _ = run_step(sched, kv)  # token 9 needs a third page each: none free -> preempt b
    assert out.preempted_req_ids == ("b",) and set(out.num_scheduled_tokens) == {"a"}
    assert sched.num_preemptions == 1 and not kv.has_request("b")
    b = sched.requests["b"]
    assert b.status == RequestStatus.PREEMPTED and b.num_computed_tokens == 0 and b.num_output_tokens == 2
    outputs = {}
    guard = 0
    while sched.has_unfinished_requests():
        out, upd = run_step(sched, kv)
        for new in out.scheduled_new_reqs:  # b comes back as a new request carrying all its tokens
            assert new.req_id == "b" and len(new.prompt_token_ids) == 7 + new.num_output_tokens
        for f in upd.finished_requests:
            outputs[f.request_id] = f.output_token_ids
        guard += 1
        assert guard < 50
        kv.check_invariants()
    assert len(outputs["a"]) == 8 and len(outputs["b"]) == 8


def test_no_progress_is_reported_when_preemption_is_off_or_impossible():
    sched, kv = make(num_pages=5, page_size=4, max_num_scheduled_tokens=100, max_num_partial_prefills=8,
                     preempt_on_deadlock=False)
    sched.add_request(request("a", 7, max_tokens=8))
    sched.add_request(request("b", 7, max_tokens=8))
    run_step(sched, kv)
    run_step(sched, kv)
    out = sched.schedule()
    assert out.total_num_scheduled_tokens == 0 and sched.last_no_progress_state is not None
    assert "no progress" in sched.last_no_progress_state.format_message()
    # a lone request that outgrows the whole pool cannot be helped by preemption either
    sched2, kv2 = make(num_pages=3, page_size=4, max_num_scheduled_tokens=100)
    sched2.add_request(request("a", 7, max_tokens=8))
    run_step(sched2, kv2)
    run_step(sched2, kv2)
    out = sched2.schedule()
    assert out.total_num_scheduled_tokens == 0 and sched2.last_no_progress_state.running == ("a",)


def test_a_request_with_a_known_prefix_starts_behind_it():
    sched, kv = make(prefix_caching=True, max_num_scheduled_tokens=64, max_num_partial_prefills=4)
    sched.add_request(request("a", 14, max_tokens=1))
    out, upd = run_step(sched, kv)
    assert out.scheduled_new_reqs[0].num_computed_tokens == 0 and upd.finished_requests
    # same first 14 tokens, then more: 3 full pages (12 tokens) are taken over, even though "a" is gone
    sched.add_request(request("b", 20, max_tokens=2))
    out, _ = run_step(sched, kv)
    new = out.scheduled_new_reqs[0]
    assert new.req_id == "b" and new.num_computed_tokens == 12 and out.num_scheduled_tokens == {"b": 8}
    assert kv.num_prefix_hits == 3
    kv.check_invariants()
    # an identical prompt: everything but its last token's page is taken over; a request may opt out
    sched.add_request(request("c", 20, max_tokens=1))
    sched.add_request(request("d", 20, max_tokens=1, skip_reading_prefix_cache=True))
    out, _ = run_step(sched, kv)
    assert {r.req_id: r.num_computed_tokens for r in out.scheduled_new_reqs} == {"c": 16, "d": 0}
    while sched.has_unfinished_requests():
        run_step(sched, kv)
    kv.check_invariants()
    assert kv.num_free_pages() == [32]


def test_a_preempted_request_finds_its_own_pages_again():
    sched, kv = make(num_pages=9, prefix_caching=True, max_num_scheduled_tokens=64, max_num_partial_prefills=4)
    sched.add_request(request("a", 12, max_tokens=12))
    sched.add_request(request("b", 12, max_tokens=12))
    preempted = 0
    for _ in range(60):
        if not sched.has_unfinished_requests():
            break
        out, _ = run_step(sched, kv)
        preempted += len(out.preempted_req_ids)
        kv.check_invariants()
    assert not sched.has_unfinished_requests() and preempted > 0 and kv.num_prefix_hits > 0


def test_planning_ahead_of_the_tokens_in_flight():
    """schedule_ahead: only a batch in steady decoding is planned before its tokens are read; a
    request that ends by length with the token in flight is left out; one that turns out to have
    stopped has its extra token dropped; no page is lost on the way."""
    sched, kv = make(max_num_scheduled_tokens=8, max_num_seqs=4, max_num_partial_prefills=2)
    sched.add_request(request("a", 10, max_tokens=2))
    sched.add_request(request("b", 3, max_tokens=5))
    first = sched.schedule()                                  # a: 8 of 10 prompt tokens, b waits
    assert first.num_scheduled_tokens == {"a": 8}
    assert sched.schedule_ahead(first) is None                # a request is waiting
    kv.advance("a", 8)
    sched.update_from_outputs(first, {})
    second = sched.schedule()                                 # a's last 2, b's 3: both sample
    assert second.num_scheduled_tokens == {"a": 2, "b": 3}
    for rid, n in second.num_scheduled_tokens.items():
        kv.advance(rid, n)
    third = sched.schedule_ahead(second)                      # planned while `second` runs
    assert third.num_scheduled_tokens == {"a": 1, "b": 1} and third.pending_token_req_ids == {"a", "b"}
    assert third.scheduled_cached_reqs.num_computed_tokens == (10, 3)
    assert third.scheduled_cached_reqs.num_output_tokens == (1, 1)
    assert third.scheduled_cached_reqs.new_token_ids == ((), ())
    sched.update_from_outputs(second, {"a": 7, "b": 7})
    for rid in third.num_scheduled_tokens:
        kv.advance(rid, 1)
    fourth = sched.schedule_ahead(third)
    assert fourth.num_scheduled_tokens == {"b": 1}            # a reaches max_tokens=2 with the token in flight
    kv.advance("b", 1)                                        # `fourth` is launched before `third` is read
    upd = sched.update_from_outputs(third, {"a": 7, "b": 9}, stop_token_ids={9})   # b stops on 9
    assert [(o.request_id, o.finished) for o in upd.step_outputs] == [("a", True), ("b", True)]
    assert [f.output_token_ids for f in upd.finished_requests] == [(7, 7), (7, 9)]
    upd = sched.update_from_outputs(fourth, {"b": 5})         # b's extra token is nobody's
    assert upd.step_outputs == () and not sched.requests
    kv.check_invariants()
    assert kv.num_free_pages() == [32] and not sched.has_unfinished_requests()


def test_planning_ahead_gives_up_where_pages_run_out():
    sched, kv = make(num_pages=5, page_size=4, max_num_scheduled_tokens=16, max_num_seqs=2, max_num_partial_prefills=2)
    sched.add_request(request("a", 8, max_tokens=6))
    sched.add_request(request("b", 8, max_tokens=6))
    first = sched.schedule()
    assert first.num_scheduled_tokens == {"a": 8, "b": 8}     # all four pages are taken
    for rid in first.num_scheduled_tokens:
        kv.advance(rid, 8)
    assert sched.schedule_ahead(first) is None                # the ninth token needs a page nobody has
    kv.check_invariants()


def test_planning_ahead_continues_prompts_and_respects_the_limits():
    """A prompt portion in flight is followed by the next portion (known tokens), beside the token in
    flight of a decoding request; the token budget and the limit on partial prefills hold; a waiting
    request that could be admitted sends the planner back to schedule()."""
    sched, kv = make(num_pages=60, max_num_scheduled_tokens=6, max_num_seqs=2, max_num_partial_prefills=1)
    sched.add_request(request("a", 3, max_tokens=9))
    out, _ = run_step(sched, kv)                               # a: whole prompt, samples
    sched.add_request(request("b", 14, max_tokens=2))
    first = sched.schedule()                                   # a decodes, b: 5 of 14
    assert first.num_scheduled_tokens == {"a": 1, "b": 5}
    for rid, n in first.num_scheduled_tokens.items():
        kv.advance(rid, n)
    sched.add_request(request("c", 2))
    ahead = sched.schedule_ahead(first)                        # c waits, but both seats are taken
    assert ahead.num_scheduled_tokens == {"a": 1, "b": 5} and ahead.pending_token_req_ids == {"a"}
    cached = ahead.scheduled_cached_reqs
    assert cached.new_token_ids == ((), (6, 7, 8, 9, 10)) and cached.num_computed_tokens == (4, 5)
    sched.update_from_outputs(first, {"a": 7})
    for rid, n in ahead.num_scheduled_tokens.items():
        kv.advance(rid, n)
    third = sched.schedule_ahead(ahead)                        # b's last 4 prompt tokens: it will sample
    assert third.num_scheduled_tokens == {"a": 1, "b": 4}
    sched.update_from_outputs(ahead, {"a": 7})
    for rid, n in third.num_scheduled_tokens.items():
        kv.advance(rid, n)
    fourth = sched.schedule_ahead(third)
    assert fourth.num_scheduled_tokens == {"a": 1, "b": 1} and fourth.pending_token_req_ids == {"a", "b"}
    upd = sched.update_from_outputs(third, {"a": 7, "b": 7})
    assert [o.sampled_token_id for o in upd.step_outputs] == [7, 7]
    for rid in fourth.num_scheduled_tokens:
        kv.advance(rid, 1)
    assert sched.schedule_ahead(fourth).num_scheduled_tokens == {"a": 1}   # b ends by length with its token in flight
    kv.check_invariants()
    # with a free seat and a request waiting, admission comes first
    roomy, kv2 = make(num_pages=60, max_num_scheduled_tokens=6, max_num_seqs=3)
    roomy.add_request(request("a", 3, max_tokens=9))
    out = roomy.schedule()
    kv2.advance("a", 3)
    roomy.add_request(request("b", 3))
    assert roomy.schedule_ahead(out) is None
