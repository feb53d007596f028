"""The engine above the step function: greedy generation through the Python entry point,
seeded sampling, generality of the parts (a toy mixer with state of its own, a layer run
twice, a layer reading another layer's cache, a windowed layer beside full ones).

Every test runs twice: on the CPU with the kernels replaced by their plain statements
(host logic only, ``-m "not gpu"``), and on the GPU with the real kernels (``-m gpu``)."""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

import plain_kernels
import plain_llama
import replay_cases as rc

from kvcore_b200 import (
    CacheConfig, DeviceConfig, KVCoreConfig, LoadConfig, ModelConfig, SamplingParams, SchedulerConfig,
)
from kvcore_b200.config import LlamaConfig, register_architecture, unregister_architecture
from kvcore_b200.config.model_spec import ModelSpec, PartSpec, ScheduleEntry
from kvcore_b200.engine.llm_engine import GenerationRequest, LLMEngine
from kvcore_b200.parts import (MIXERS, POSITION_ENCODINGS, FEED_FORWARDS, CacheSpec, Mixer, PositionEncoding, FeedForward,
                               StateSpec, WeightSlot)

BACKENDS = [pytest.param("cpu", id="host"), pytest.param("cuda:0", id="gpu", marks=pytest.mark.gpu)]


@pytest.fixture(params=BACKENDS)
def device(request, monkeypatch):
    if request.param == "cpu":
        plain_kernels.install(monkeypatch)
    return request.param


def engine_config(folder, device, dtype="float32", **overrides):
    sched = dict(max_num_seqs=4, max_num_scheduled_tokens=64, max_num_partial_prefills=4, max_long_partial_prefills=4)
    sched.update(overrides.pop("scheduler", {}))
    return KVCoreConfig(
        model_config=ModelConfig(model=str(folder), dtype=dtype, max_model_len=overrides.pop("max_model_len", 128)),
        load_config=LoadConfig(**overrides.pop("load", {})),
        cache_config=CacheConfig(block_size=overrides.pop("block_size", 16), num_gpu_blocks=overrides.pop("num_gpu_blocks", 40),
                                 enable_prefix_caching=overrides.pop("prefix_caching", False),
                                 debug_fill_freed_pages=overrides.pop("fill_freed_pages", None)),
        scheduler_config=SchedulerConfig(**sched),
        device_config=DeviceConfig(device=device),
    )


@pytest.mark.parametrize("name,lengths,steps,block,budget", [("A", (7, 13), 8, 16, 64), ("B", (5, 19, 40), 12, 8, 6)])
def test_greedy_generation_matches_plain(device, tmp_path, name, lengths, steps, block, budget):
    config = rc.TINY_CONFIGS[name]
    folder = rc.write_model(tmp_path / "m", config, rc.TINY_SEEDS[name], "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompts = [rc.random_tokens(config["vocab_size"], n, 50 + i) for i, n in enumerate(lengths)]
    engine = LLMEngine(engine_config(folder, device, block_size=block, scheduler=dict(max_num_scheduled_tokens=budget)))
    requests = [GenerationRequest(f"r{i}", SamplingParams(max_tokens=steps, temperature=0.0), tuple(p))
                for i, p in enumerate(prompts)]
    outputs = engine.generate(requests)
    assert [o.request_id for o in outputs] == [r.request_id for r in requests]
    for prompt, output in zip(prompts, outputs):
        assert output.finish_reason == "length"
        assert list(output.output_token_ids) == plain_llama.greedy_generate(config, weights, prompt, steps)
    kv = engine.engine_core.model_runner.kv_manager
    kv.check_invariants()
    assert not kv.live_requests() and not engine.engine_core.model_runner.requests


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["D", "E"])
def test_bfloat16_generation_on_serving_shapes_picks_tokens_the_plain_logits_allow(tmp_path, name):
    """Head sizes 128 and 64, prompts of several key tiles, chunked prefill beside decoding, decode
    steps replayed from graphs: the path that serves (TMA decode attention with its rotation, the
    streaming products with norm, activation and residual inside, the tcgen05 prompt attention).
    In bfloat16 a near-tie may fall either way, so every generated token must be one whose plain
    32-bit logit lies within the rounding bound of the largest."""
    config = rc.TINY_CONFIGS[name]
    folder = rc.write_model(tmp_path / "m", config, rc.TINY_SEEDS[name], "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompts = [rc.random_tokens(config["vocab_size"], n, 80 + i) for i, n in enumerate((70, 150, 33, 9))]
    steps = 40
    engine = LLMEngine(engine_config(folder, "cuda:0", dtype="bfloat16", max_model_len=256, num_gpu_blocks=80,
                                     scheduler=dict(max_num_scheduled_tokens=48)))
    outputs = engine.generate([GenerationRequest(f"r{i}", SamplingParams(max_tokens=steps, temperature=0.0), tuple(p))
                               for i, p in enumerate(prompts)])
    runner = engine.engine_core.model_runner
    assert runner.step_function.num_graph_replays > 0
    for prompt, output in zip(prompts, outputs):
        tokens = list(output.output_token_ids)
        assert len(tokens) == steps and output.finish_reason == "length"
        logits = plain_llama.forward_logits(config, weights, prompt + tokens).numpy()
        bound = 2 * 2e-2 * np.abs(logits).max()       # both candidates may be off by the bfloat16 tolerance
        for index, token in enumerate(tokens):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - bound, f"token {index}: {row[token]} against {row.max()}"
    runner.kv_manager.check_invariants()
    assert not runner.kv_manager.live_requests()


@pytest.mark.parametrize("fill", [None, "zero", "poison"])
def test_generation_with_few_pages_and_preemption(device, tmp_path, fill):
    """So few pages that requests wait, are preempted and recomputed: tokens stay the plain ones, also
    when every page that lost its holder is overwritten (zeros, or a large value) before the next step."""
    config = rc.TINY_CONFIGS["A"]
    folder = rc.write_model(tmp_path / "m", config, 0, "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompts = [rc.random_tokens(256, n, 70 + i) for i, n in enumerate((9, 14, 6, 11))]
    engine = LLMEngine(engine_config(folder, device, block_size=4, num_gpu_blocks=14, fill_freed_pages=fill,
                                     scheduler=dict(max_num_scheduled_tokens=16)))
    outputs = engine.generate([dict(request_id=f"r{i}", prompt_token_ids=p,
                                    sampling_params=dict(max_tokens=10, temperature=0.0))
                               for i, p in enumerate(prompts)])
    for prompt, output in zip(prompts, outputs):
        assert list(output.output_token_ids) == plain_llama.greedy_generate(config, weights, prompt, 10)
    assert engine.engine_core.scheduler.num_preemptions > 0
    runner = engine.engine_core.model_runner
    runner.kv_manager.check_invariants()
    if fill is not None:    # every page has been freed at least once by now and was overwritten at the next step
        storage = runner.storage.group_tensors[0]
        written = 0.0 if fill == "zero" else runner.storage.POISON_VALUE
        for group, pages in enumerate(runner.kv_manager.take_released_pages()):
            runner.storage.fill_pages(group, pages, written)
        assert bool((storage[:, :, 1:] == written).all())


def test_generation_with_shared_prefixes_reuses_pages_and_keeps_the_tokens(device, tmp_path):
    """Prompts that begin alike: with prefix reuse their common pages are computed once (also across
    generate() calls, after the first owner is gone), and the tokens are the plain ones."""
    config = rc.TINY_CONFIGS["A"]
    folder = rc.write_model(tmp_path / "m", config, 0, "float32")
    weights = plain_llama.load_weights(folder)
    stem = rc.random_tokens(256, 37, 90)
    prompts = [stem + rc.random_tokens(256, n, 91 + i) for i, n in enumerate((3, 9, 1))] + [stem[:21]]
    engine = LLMEngine(engine_config(folder, device, block_size=4, num_gpu_blocks=60, prefix_caching=True,
                                     scheduler=dict(max_num_scheduled_tokens=24, max_num_partial_prefills=2)))
    kv = engine.engine_core.model_runner.kv_manager
    assert kv.prefix_caching
    expected = [plain_llama.greedy_generate(config, weights, p, 6) for p in prompts]
    for round_ in range(2):
        requests = [GenerationRequest(f"r{round_}-{i}", SamplingParams(max_tokens=6, temperature=0.0), tuple(p))
                    for i, p in enumerate(prompts)]
        outputs = engine.generate(requests)
        assert [list(o.output_token_ids) for o in outputs] == expected
        kv.check_invariants()
        assert not kv.live_requests()
        if round_ == 0:
            first_round_hits = kv.num_prefix_hits
            assert first_round_hits >= 9          # the 36-token stem is 9 pages; later requests take them over
    # the second round found everything but each prompt's last page
    assert kv.num_prefix_hits - first_round_hits >= sum((len(p) - 1) // 4 for p in prompts) - 2


def test_too_small_a_cache_is_an_error(device, tmp_path):
    folder = rc.write_model(tmp_path / "m", rc.TINY_A, 0, "bfloat16")
    engine = LLMEngine(engine_config(folder, device, block_size=4, num_gpu_blocks=4,
                                     scheduler=dict(preempt_on_deadlock=False)))
    with pytest.raises(RuntimeError, match="no scheduling progress"):
        engine.generate([dict(request_id="a", prompt_token_ids=[1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11],
                              sampling_params=dict(max_tokens=8, temperature=0.0))])


def test_stop_token_from_config(device, tmp_path):
    config = dict(rc.TINY_A)
    folder = rc.write_model(tmp_path / "m", config, 0, "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompt = rc.random_tokens(256, 9, 3)
    expected = plain_llama.greedy_generate(config, weights, prompt, 6)
    stored = json.loads((folder / "config.json").read_text())
    stored["eos_token_id"] = [expected[3], 999999]
    (folder / "config.json").write_text(json.dumps(stored))
    out = LLMEngine(engine_config(folder, device)).generate(
        [dict(request_id="a", prompt_token_ids=prompt, sampling_params=dict(max_tokens=6, temperature=0.0))])
    cut = expected.index(expected[3]) + 1
    assert list(out[0].output_token_ids) == expected[:cut] and out[0].finish_reason == "stop"


def test_seeded_sampling_is_reproducible_and_independent_of_the_batch(device, tmp_path):
    config = rc.TINY_CONFIGS["B"]
    folder = rc.write_model(tmp_path / "m", config, 1, "bfloat16")
    prompts = [rc.random_tokens(config["vocab_size"], n, 90 + i) for i, n in enumerate((5, 19, 40))]

    def run(which, budget):
        engine = LLMEngine(engine_config(folder, device, block_size=8, max_model_len=256,
                                         scheduler=dict(max_num_scheduled_tokens=budget)))
        reqs = [dict(request_id=f"r{i}", prompt_token_ids=prompts[i],
                     sampling_params=SamplingParams(max_tokens=12, temperature=0.8, seed=1234 + i, top_k=50, top_p=0.95))
                for i in which]
        return {o.request_id: o.output_token_ids for o in engine.generate(reqs)}

    together = run([0, 1, 2], 6)
    assert together == run([0, 1, 2], 6)
    if device == "cpu":  # bit-equal logits across batchings hold for the plain kernels and the 32-bit GPU path
        assert run([1], 64)["r1"] == together["r1"]
    assert len({tuple(v) for v in together.values()}) == 3
    unseeded = LLMEngine(engine_config(folder, device, block_size=8, max_model_len=256)).generate(
        [dict(request_id="u", prompt_token_ids=prompts[0], sampling_params=dict(max_tokens=4))])
    assert len(unseeded[0].output_token_ids) == 4


def test_the_second_baseline_configuration_as_stated(device, tmp_path):
    """Vocabulary 512, tied, llama3 scaling, pages of 8 tokens; requests of 5, 19 and 40 tokens, at most
    6 tokens a step, 12 tokens each at temperature 0.8 with a seed.  Every logits row the sampler is
    given is the plain implementation's row at that position, and every token is the one the plain
    statement of the sampling rule draws from it."""
    config = rc.TINY_CONFIGS["B8"]
    folder = rc.write_model(tmp_path / "m", config, 1, "bfloat16")
    weights = plain_llama.load_weights(folder)
    prompts = {f"r{i}": rc.random_tokens(512, n, 50 + i) for i, n in enumerate((5, 19, 40))}
    engine = LLMEngine(engine_config(folder, device, block_size=8, num_gpu_blocks=40,
                                     scheduler=dict(max_num_scheduled_tokens=6)))
    runner = engine.engine_core.model_runner
    seen = []
    sample = runner.sampler.sample

    def recording(logits, params, seeds, token_indices):
        tokens = sample(logits, params, seeds, token_indices)
        seen.append((logits.float().cpu().clone(), list(seeds), list(token_indices), tokens.cpu().tolist()))
        return tokens

    runner.sampler.sample = recording
    outputs = engine.generate([GenerationRequest(rid, SamplingParams(max_tokens=12, temperature=0.8, seed=1000 + i), tuple(p))
                               for i, (rid, p) in enumerate(prompts.items())])
    generated = {o.request_id: list(o.output_token_ids) for o in outputs}
    assert all(len(tokens) == 12 for tokens in generated.values())
    assert engine.engine_core.model_runner.step_function.num_steps >= 12 + 7       # 64 prompt tokens in portions of 6
    rows_checked = 0
    for rid, prompt in prompts.items():
        seed = 1000 + int(rid[1:])
        reference = plain_llama.forward_logits(config, weights, prompt + generated[rid]).numpy()
        for index, token in enumerate(generated[rid]):
            want = torch.from_numpy(reference[len(prompt) + index - 1])
            rows = [(logits[row], tokens[row]) for logits, seeds, indices, tokens in seen
                    for row in range(len(seeds)) if seeds[row] == seed and indices[row] == index]
            assert len(rows) == 1, "one sampler call per token of a request"
            got, sampled = rows[0]
            assert sampled == token
            assert float((got - want).abs().max()) <= 2e-5 * float(np.abs(reference).max())
            assert plain_kernels.sample_row(got, 0.8, 512, 1.0, seed, index)[0] == token
            assert plain_kernels.sample_row(want, 0.8, 512, 1.0, seed, index)[0] == token
            rows_checked += 1
    assert rows_checked == 36
    runner.kv_manager.check_invariants()


def test_running_one_step_ahead_changes_no_output(device, tmp_path):
    """With a step kept in flight the engine returns the tokens it returns without: requests that end
    by length, requests that stop on a token (seen a step late, the extra token dropped), seeded
    sampling, requests that arrive while others decode; and every page comes back."""
    config = rc.TINY_CONFIGS["B"]
    folder = rc.write_model(tmp_path / "m", config, 1, "float32")
    weights = plain_llama.load_weights(folder)
    prompts = [rc.random_tokens(config["vocab_size"], n, 40 + i) for i, n in enumerate((5, 19, 33, 8))]
    greedy = [plain_llama.greedy_generate(config, weights, p, 14) for p in prompts]
    stored = json.loads((folder / "config.json").read_text())
    stored["eos_token_id"] = [greedy[1][6], greedy[3][2]]      # requests 1 and 3 stop early
    (folder / "config.json").write_text(json.dumps(stored))
    params = [SamplingParams(max_tokens=14, temperature=0.0), SamplingParams(max_tokens=14, temperature=0.0),
              SamplingParams(max_tokens=9, temperature=0.7, seed=5, top_k=40),
              SamplingParams(max_tokens=14, temperature=0.0)]

    def run(run_ahead):
        engine = LLMEngine(engine_config(folder, device, block_size=8, max_model_len=256, num_gpu_blocks=30,
                                         scheduler=dict(max_num_scheduled_tokens=24, run_ahead=run_ahead)))
        for i in range(3):
            engine.add_request(f"r{i}", params[i], prompt_token_ids=prompts[i])
        steps, outputs = 0, {}
        while engine.engine_core.has_unfinished_requests():
            for out in engine.step().request_outputs:
                if out.sampled_token_id is not None:
                    outputs.setdefault(out.request_id, []).append(out.sampled_token_id)
            steps += 1
            if steps == 7:    # a late arrival: the batch leaves steady decoding, takes it in, settles again
                engine.add_request("r3", params[3], prompt_token_ids=prompts[3])
        core = engine.engine_core
        finished = {r: core.take_finished_output(r) for r in ("r0", "r1", "r2", "r3")}
        kv = core.model_runner.kv_manager
        kv.check_invariants()
        assert not kv.live_requests() and not core.model_runner.requests and core._in_flight is None
        assert {r: list(f.output_token_ids) for r, f in finished.items()} == outputs
        return outputs, {r: f.finish_reason.value for r, f in finished.items()}, core.num_steps_run_ahead

    ahead, ahead_reasons, launched_ahead = run(True)
    plain, plain_reasons, none_ahead = run(False)
    assert launched_ahead > 5 and none_ahead == 0
    assert ahead == plain and ahead_reasons == plain_reasons
    assert ahead["r0"] == greedy[0]
    assert ahead["r1"] == greedy[1][: greedy[1].index(greedy[1][6]) + 1] and ahead_reasons["r1"] == "stop"
    assert ahead_reasons == {"r0": "length", "r1": "stop", "r2": ahead_reasons["r2"], "r3": "stop"}


def test_abort_ends_a_request_and_leaves_the_others_alone(device, tmp_path):
    config = rc.TINY_CONFIGS["A"]
    folder = rc.write_model(tmp_path / "m", config, 0, "float32")
    weights = plain_llama.load_weights(folder)
    prompts = [rc.random_tokens(256, n, 20 + i) for i, n in enumerate((9, 14, 6))]
    engine = LLMEngine(engine_config(folder, device, block_size=4, num_gpu_blocks=40))
    for i, prompt in enumerate(prompts):
        engine.add_request(f"r{i}", SamplingParams(max_tokens=12, temperature=0.0), prompt_token_ids=prompt)
    for _ in range(5):
        engine.step()
    aborted = engine.abort(["r1", "unknown"])
    assert [a.request_id for a in aborted] == ["r1"] and aborted[0].finish_reason == "abort"
    expected = [plain_llama.greedy_generate(config, weights, p, 12) for p in prompts]
    assert list(aborted[0].output_token_ids) == expected[1][: len(aborted[0].output_token_ids)]
    assert 0 < len(aborted[0].output_token_ids) < 12
    for _ in engine.run():
        pass
    core = engine.engine_core
    assert list(core.take_finished_output("r0").output_token_ids) == expected[0]
    assert list(core.take_finished_output("r2").output_token_ids) == expected[2]
    assert core.take_finished_output("r1").finish_reason.value == "abort"
    kv = core.model_runner.kv_manager
    kv.check_invariants()
    assert not kv.live_requests() and not core.model_runner.requests and core._in_flight is None
    engine.add_request("late", SamplingParams(max_tokens=3, temperature=0.0), prompt_token_ids=prompts[0])
    engine.step()
    assert [a.request_id for a in engine.abort()] == ["late"] and not core.has_unfinished_requests()


def test_random_weights_mode_needs_no_weight_file(device, tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(rc.TINY_A))
    engine = LLMEngine(engine_config(tmp_path, device, load=dict(random_weights=True, seed=3)))
    out = engine.generate([dict(request_id="a", prompt_token_ids=[1, 2, 3],
                                sampling_params=dict(max_tokens=3, temperature=0.0))])
    assert len(out[0].output_token_ids) == 3


def test_requests_are_validated(device, tmp_path):
    folder = rc.write_model(tmp_path / "m", rc.TINY_A, 0, "bfloat16")
    engine = LLMEngine(engine_config(folder, device))
    with pytest.raises(ValueError, match="outside"):
        engine.add_request("a", SamplingParams(max_tokens=1), prompt_token_ids=[1, 256])
    with pytest.raises(ValueError, match="prompt_token_ids or messages"):
        engine.add_request("a", SamplingParams(max_tokens=1))
    with pytest.raises(Exception, match="tokenizer"):
        engine.add_request("a", SamplingParams(max_tokens=1), messages=[{"role": "user", "content": "hi"}])


# ---- generality of the parts ------------------------------------------------------------------
class RunningMeanMixer(Mixer):
    """A toy mixer with state of its own: ``y_t = W (s_t / (t+1))`` with ``s_t = s_{t-1} + x_t``,
    where ``s`` lives in the request's state slot between steps.  Written in torch by the test."""

    def __init__(self, *, hidden_size, name, dtype, device):
        self.hidden_size, self.name = hidden_size, name
        self.weight = torch.empty(hidden_size, hidden_size, dtype=dtype, device=device)

    def state_spec(self):
        return StateSpec((self.hidden_size,), torch.float32)

    def weight_slots(self):
        return [WeightSlot(f"{self.name}.weight", self.weight)]

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        start = 0
        for n, context, slot in zip(ctx.host_query_lens, ctx.host_context_lens, ctx.host_state_slots):
            sums = cache.state[slot] + torch.cumsum(x[start:start + n].float(), dim=0)
            counts = torch.arange(context + 1, context + n + 1, device=x.device, dtype=torch.float32)[:, None]
            out[start:start + n] = ((sums / counts) @ self.weight.float().T).to(x.dtype)
            cache.state[slot] = sums[-1]
            start += n
        return out


class LatentMixer(Mixer):
    """A toy mixer whose pages hold ONE plane: a latent vector ``c_t = W_c x_t`` per cached token
    (no keys and values).  ``y_t = W_o sum_s softmax_s(q_t . c_s / sqrt(L)) c_s`` over ``s <= t`` with
    ``q_t = W_q x_t``.  Written in torch by the test, reading and writing its pages through the step's
    block table."""

    def __init__(self, *, hidden_size, latent, name, dtype, device):
        self.latent, self.name = latent, name
        self.w_c = torch.empty(latent, hidden_size, dtype=dtype, device=device)
        self.w_q = torch.empty(latent, hidden_size, dtype=dtype, device=device)
        self.w_o = torch.empty(hidden_size, latent, dtype=dtype, device=device)

    def cache_spec(self):
        return CacheSpec(planes=1, heads=1, width=self.latent)

    def weight_slots(self):
        return [WeightSlot(f"{self.name}.c.weight", self.w_c), WeightSlot(f"{self.name}.q.weight", self.w_q),
                WeightSlot(f"{self.name}.o.weight", self.w_o)]

    def forward(self, x, ctx, cache):
        assert len(cache.planes) == 1 and cache.v is None
        plane, page = cache.planes[0], cache.page_size        # [pages, 1, page, L]
        table = ctx.block_table(cache.group).long()
        latents = x.float() @ self.w_c.float().T
        queries = x.float() @ self.w_q.float().T
        out = torch.empty_like(x)
        start = 0
        for row, (n, context) in enumerate(zip(ctx.host_query_lens, ctx.host_context_lens)):
            positions = torch.arange(context, context + n, device=x.device)
            plane[table[row, positions // page], 0, positions % page] = latents[start:start + n].to(plane.dtype)
            total = context + n
            cached = plane[table[row, : -(-total // page)], 0].reshape(-1, self.latent)[:total].float()
            scores = queries[start:start + n] @ cached.T / self.latent ** 0.5
            visible = torch.arange(total, device=x.device)[None, :] <= positions[:, None]
            weights = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1)
            out[start:start + n] = ((weights @ cached) @ self.w_o.float().T).to(x.dtype)
            start += n
        return out


class OffsetPosition(PositionEncoding):
    """A toy position encoding: adds ``amplitude * sin(position * rate)`` to every q and k entry."""

    def __init__(self, *, rate, amplitude, dtype, device):
        self.rate, self.amplitude = rate, amplitude

    def apply(self, q, k, ctx):
        shift = (torch.sin(ctx.positions.float() * self.rate) * self.amplitude)[:, None, None]
        q.copy_((q.float() + shift).to(q.dtype))
        if k is not None:
            k.copy_((k.float() + shift).to(k.dtype))


class RoutedFeedForward(FeedForward):
    """A toy feed-forward with routing: every token goes to the one expert its router scores
    highest (scores in 32-bit), ``y = p * W_out[e] relu(W_in[e] x)`` with ``p`` the softmax weight of
    that expert.  Written in torch by the test."""

    def __init__(self, *, hidden_size, inter, experts, name, dtype, device):
        self.name, self.experts = name, experts
        self.router = torch.empty(experts, hidden_size, dtype=dtype, device=device)
        self.w_in = torch.empty(experts, inter, hidden_size, dtype=dtype, device=device)
        self.w_out = torch.empty(experts, hidden_size, inter, dtype=dtype, device=device)

    def weight_slots(self):
        slots = [WeightSlot(f"{self.name}.router.weight", self.router)]
        for e in range(self.experts):
            slots += [WeightSlot(f"{self.name}.experts.{e}.in.weight", self.w_in[e]),
                      WeightSlot(f"{self.name}.experts.{e}.out.weight", self.w_out[e])]
        return slots

    def forward(self, x, ctx):
        scores = torch.softmax(x.float() @ self.router.float().T, dim=-1)
        weight, expert = scores.max(dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = (expert == e).nonzero().flatten()
            if rows.numel():
                hidden = torch.relu(x[rows].float() @ self.w_in[e].float().T)
                out[rows] = (weight[rows, None] * (hidden @ self.w_out[e].float().T)).to(x.dtype)
        return out


def toy_spec(raw):
    """Layers: 0 attention (window 9, toy position), 1 running mean, 2 attention (rope) with a
    routed feed-forward, 3 a mixer that caches one latent vector per token.  Schedule: 0, 1, 2, 0 again
    (own cache), then 2 reading the cache of the first run of 2, then 3."""
    base = LlamaConfig.from_dict(raw).to_model_spec()
    layers = list(base.layers)
    layers[0] = type(layers[0])(
        prefix=layers[0].prefix, block=layers[0].block,
        mixer=layers[0].mixer.with_params(sliding_window=9, position=PartSpec("toy_offset", dict(rate=0.37, amplitude=0.5))),
        feed_forward=layers[0].feed_forward, norms=layers[0].norms)
    layers[1] = type(layers[1])(
        prefix=layers[1].prefix, block=layers[1].block,
        mixer=PartSpec("toy_running_mean", dict(hidden_size=raw["hidden_size"], name="model.layers.1.mean")),
        feed_forward=layers[1].feed_forward, norms=layers[1].norms)
    layers[2] = type(layers[2])(
        prefix=layers[2].prefix, block=layers[2].block, mixer=layers[2].mixer,
        feed_forward=PartSpec("toy_routed", dict(hidden_size=raw["hidden_size"], inter=48, experts=3,
                                                 name="model.layers.2.moe")),
        norms=layers[2].norms)
    layers[3] = type(layers[3])(
        prefix=layers[3].prefix, block=layers[3].block,
        mixer=PartSpec("toy_latent", dict(hidden_size=raw["hidden_size"], latent=24, name="model.layers.3.latent")),
        feed_forward=layers[3].feed_forward, norms=layers[3].norms)
    fields = {f: getattr(base, f) for f in base.__dataclass_fields__}
    fields.update(architecture="ToyForCausalLM", layers=tuple(layers),
                  schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(0),
                            ScheduleEntry(2, cache_of=2), ScheduleEntry(3)))
    return ModelSpec(**fields)


def toy_plain_logits(raw, weights, tokens):
    """The toy model, whole sequence, no cache, in plain torch (float64)."""
    import plain_llama as pl

    w = {k: v.double() for k, v in weights.items()}
    ids = torch.as_tensor(tokens)
    n = ids.numel()
    heads, kvh, dim = raw["num_attention_heads"], raw["num_key_value_heads"], pl.head_dim_of(raw)
    eps, positions = raw["rms_norm_eps"], torch.arange(n)
    inv_freq = pl.rope_inv_freq(raw)

    def attention_layer(x, p, kind, borrowed=None):
        q = pl.linear(x, w[f"{p}.self_attn.q_proj.weight"]).view(n, heads, dim)
        k = pl.linear(x, w[f"{p}.self_attn.k_proj.weight"]).view(n, kvh, dim)
        v = pl.linear(x, w[f"{p}.self_attn.v_proj.weight"]).view(n, kvh, dim)
        if kind == "toy":
            shift = (torch.sin(positions.float() * 0.37) * 0.5).double()[:, None, None]
            q, k = q + shift, k + shift
            window = 9
        else:
            q, k = pl.apply_rope(q, k, positions, inv_freq)
            window = None
        if borrowed is not None:
            k, v = borrowed
        a = pl.causal_attention(q, k, v, dim ** -0.5, window).reshape(n, heads * dim)
        return pl.linear(a, w[f"{p}.self_attn.o_proj.weight"]), (k, v)

    def mean_layer(x, p):
        running = torch.cumsum(x.float(), dim=0).double() / torch.arange(1, n + 1).double()[:, None]
        return pl.linear(running, w["model.layers.1.mean.weight"]), None

    def latent_layer(x, p):
        c, q = pl.linear(x, w[f"{p}.latent.c.weight"]), pl.linear(x, w[f"{p}.latent.q.weight"])
        scores = (q @ c.T) / c.shape[1] ** 0.5
        scores = scores.masked_fill(positions[None, :] > positions[:, None], float("-inf"))
        return pl.linear(torch.softmax(scores, dim=-1) @ c, w[f"{p}.latent.o.weight"]), None

    h = pl.embed(ids, w["model.embed_tokens.weight"])
    residual = None
    kept = {}
    for entry, (layer, borrow) in enumerate([(0, None), (1, None), (2, None), (0, None), (2, 2), (3, None)]):
        p = f"model.layers.{layer}"
        residual = h if residual is None else h + residual
        x = pl.rms_norm(residual, w[f"{p}.input_layernorm.weight"], eps)
        if layer == 1:
            a, _ = mean_layer(x, p)
        elif layer == 3:
            a, _ = latent_layer(x, p)
        else:
            a, kept[entry] = attention_layer(x, p, "toy" if layer == 0 else "rope",
                                             None if borrow is None else kept[borrow])
        residual = a + residual
        x = pl.rms_norm(residual, w[f"{p}.post_attention_layernorm.weight"], eps)
        if layer == 2:
            scores = torch.softmax(x @ w[f"{p}.moe.router.weight"].T, dim=-1)
            weight, expert = scores.max(dim=-1)
            h = torch.zeros_like(x)
            for t in range(n):
                e = int(expert[t])
                hidden = torch.relu(w[f"{p}.moe.experts.{e}.in.weight"] @ x[t])
                h[t] = weight[t] * (w[f"{p}.moe.experts.{e}.out.weight"] @ hidden)
        else:
            h = pl.swiglu_mlp(x, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"])
    final = pl.rms_norm(h + residual, w["model.norm.weight"], eps)
    return (final @ w["lm_head.weight"].T).float()


@pytest.fixture
def toy_parts():
    MIXERS.register("toy_running_mean", RunningMeanMixer)
    MIXERS.register("toy_latent", LatentMixer)
    POSITION_ENCODINGS.register("toy_offset", OffsetPosition)
    FEED_FORWARDS.register("toy_routed", RoutedFeedForward)
    register_architecture("ToyForCausalLM", toy_spec)
    yield
    MIXERS.unregister("toy_running_mean")
    MIXERS.unregister("toy_latent")
    POSITION_ENCODINGS.unregister("toy_offset")
    FEED_FORWARDS.unregister("toy_routed")
    unregister_architecture("ToyForCausalLM")


def test_toy_parts_register_build_and_step_without_touching_the_framework(device, toy_parts, tmp_path):
    raw = dict(rc.TINY_A, architectures=["ToyForCausalLM"], num_hidden_layers=4, max_position_embeddings=256)
    folder = rc.write_model(tmp_path / "m", raw, 4, "float32")
    weights = plain_llama.load_weights(folder)
    assert "model.layers.1.mean.weight" in weights and "model.layers.1.self_attn.q_proj.weight" not in weights
    assert "model.layers.2.moe.experts.2.out.weight" in weights and "model.layers.2.mlp.down_proj.weight" not in weights
    assert "model.layers.3.latent.c.weight" in weights and "model.layers.3.self_attn.k_proj.weight" not in weights
    requests = {f"r{i}": rc.random_tokens(256, n, 30 + i) for i, n in enumerate((40, 75, 23, 58, 31))}
    reference = {rid: toy_plain_logits(raw, weights, toks).numpy() for rid, toks in requests.items()}
    for steps in (rc.trace_whole(requests), rc.trace_chunks(requests), rc.trace_mixed(requests, max_live=3, seed=1)):
        out = tmp_path / f"out{len(steps)}"
        step_function, kv = rc.run_inprocess(folder, "float32", steps, out, rc.peak_tokens(steps), device=device)
        rows = rc.collect(steps, out, 256)
        assert len(rows) == sum(len(t) for t in requests.values())
        for (rid, pos), row in rows.items():
            err = np.abs(row - reference[rid][pos]).max() / np.abs(reference[rid]).max()
            assert err < 3e-5, (rid, pos, err)
        # three groups of pages: windowed keys and values (both runs of layer 0), keys and values that
        # stay (layer 2 and its borrower), and the latent mixer's single plane of one vector a token
        assert [g.kind for g in kv.groups] == ["window", "full", "full"]
        assert [len(g.entries) for g in kv.groups] == [2, 1, 1]
        assert [(g.planes, g.heads, g.width) for g in kv.groups] == [(2, 2, 16), (2, 2, 16), (1, 1, 24)]
        assert tuple(step_function.storage.group_tensors[2].shape[:2]) == (1, 1)
        assert len(step_function.storage.state_tensors) == 1


def test_step_entries_fed_from_a_sampler_output(device, tmp_path):
    """The step function's own view of a token that the host has not seen: a placeholder id and the row
    of the sampler output that holds the real one give the logits of the id packed by the host; what
    cannot be right is refused (no output given, more than one token, a row outside the output)."""
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay

    config = rc.TINY_CONFIGS["A"]
    folder = rc.write_model(tmp_path / "m", config, 2, "float32")
    prompts = {"a": rc.random_tokens(256, 11, 1), "b": rc.random_tokens(256, 6, 2)}

    def run(fed):
        step_function, kv = build_replay(str(folder), "float32", 256, device=device)
        for rid, tokens in prompts.items():
            assert kv.allocate_slots(rid, len(tokens))
        step_function.step([StepEntry(rid, tokens, ()) for rid, tokens in prompts.items()])
        sampled = torch.tensor([77, 5, 190], dtype=torch.int32, device=device)
        for rid in prompts:
            assert kv.allocate_slots(rid, 1)
        if fed:
            entries = [StepEntry("a", (0,), (0,), fed_from=2), StepEntry("b", (0,), (0,), fed_from=0)]
            return step_function, kv, step_function.step(entries, sampled).float().cpu()
        entries = [StepEntry("a", (190,), (0,)), StepEntry("b", (77,), (0,))]
        return step_function, kv, step_function.step(entries).float().cpu()

    _, _, from_host = run(False)
    step_function, kv, from_device = run(True)
    assert torch.equal(from_host, from_device)
    sampled = torch.tensor([1, 2], dtype=torch.int32, device=device)
    for rid in prompts:
        assert kv.allocate_slots(rid, 2)
    for entries, feedback in (([StepEntry("a", (0,), (0,), fed_from=0)], None),
                              ([StepEntry("a", (0, 0), (1,), fed_from=0)], sampled),
                              ([StepEntry("a", (0,), (0,), fed_from=2)], sampled)):
        with pytest.raises(ValueError, match="sampler output"):
            step_function.step(entries, feedback)
