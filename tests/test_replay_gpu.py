"""Trace replay on the GPU against the plain implementation, in 32-bit and in bfloat16:
each request alone and whole; most of it in one step and the last 32 tokens one by one;
portions of changing size down to two (and one) tokens; and mixed, up to four live requests
with so few pages that pages are used again.  In 32-bit the cuttings must also agree with
each other bit for bit, because every kernel of that path sums in an order that depends on
the position only."""
from __future__ import annotations

import numpy as np
import pytest

import plain_llama
import replay_cases as rc

pytestmark = pytest.mark.gpu

# largest |difference| allowed, as a fraction of the largest |logit| of the request.
# bfloat16: measured on these models (all configurations, whole / tail / mixed cuttings), the engine
# lies within 4.3e-3 to 7.3e-3 of the 32-bit plain model and within 5.1e-3 to 7.3e-3 of the plain model
# evaluated with bfloat16 roundings in the reference's places, which itself lies 4.4e-3 to 7.4e-3 from
# 32-bit: two bfloat16 evaluations that round in different places (the engine keeps the norm, the
# activation and the residual sum inside its products) differ from each other as much as each does
# from 32-bit, so the rounded oracle allows no tighter bound than the exact one.  The bound on a single
# row is 1.6 times the largest error seen; beside it the median row error and the largest
# root-mean-square error of a row over a trace are bounded at about 1.3 and 1.7 times what was measured
# (3.0e-3 to 3.9e-3, and 1.3e-3 to 2.1e-3): a kernel that is a little wrong everywhere fails those.
TOLERANCE = {"float32": 2e-5, "bfloat16": 1.2e-2}
BF16_MEDIAN_TOLERANCE = 5e-3
BF16_RMS_TOLERANCE = 3.5e-3
LENGTHS = (45, 70, 33, 101, 64, 17, 128)
# the two configurations with serving head sizes also get requests that span several key tiles
LONG_LENGTHS = (45, 300, 33, 161, 64, 17, 520)


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "B8"])
def model_case(request, tmp_path_factory):
    name = request.param
    config = rc.TINY_CONFIGS[name]
    folder = tmp_path_factory.mktemp(f"model_{name}")
    rc.write_model(folder, config, rc.TINY_SEEDS[name], "bfloat16")
    weights = plain_llama.load_weights(folder)
    lengths = LONG_LENGTHS if name in ("D", "E") else LENGTHS
    requests = {f"r{i}": rc.random_tokens(config["vocab_size"], n, 10 + i) for i, n in enumerate(lengths)}
    reference = {rid: plain_llama.forward_logits(config, weights, toks).numpy() for rid, toks in requests.items()}
    return dict(name=name, config=config, folder=folder, requests=requests, reference=reference,
                page_size=rc.TINY_PAGE_SIZES[name])


def _compare(rows, reference, dtype):
    assert rows
    worst = 0.0
    for (rid, pos), row in rows.items():
        ref = reference[rid][pos]
        assert np.isfinite(row).all(), f"non-finite logits for {rid}@{pos}"
        err = np.abs(row - ref).max() / np.abs(reference[rid]).max()
        if err > TOLERANCE[dtype]:
            first = min(p for (r, p), v in rows.items() if r == rid
                        and np.abs(v - reference[rid][p]).max() / np.abs(reference[rid]).max() > TOLERANCE[dtype])
            raise AssertionError(f"{rid}: first wrong position {first} (error {err:.3e} at {pos})")
        worst = max(worst, err)
    if dtype == "bfloat16" and len(rows) >= 50:
        errors = [np.abs(row - reference[rid][pos]).max() / np.abs(reference[rid]).max() for (rid, pos), row in rows.items()]
        rms = [np.sqrt(np.mean((row - reference[rid][pos]) ** 2)) / np.abs(reference[rid]).max()
               for (rid, pos), row in rows.items()]
        assert np.median(errors) <= BF16_MEDIAN_TOLERANCE, f"median row error {np.median(errors):.3e}"
        assert max(rms) <= BF16_RMS_TOLERANCE, f"largest root-mean-square row error {max(rms):.3e}"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_match_plain_implementation(model_case, dtype, tmp_path):
    config, requests = model_case["config"], model_case["requests"]
    vocab = config["vocab_size"]
    expected_rows = sum(len(t) for t in requests.values())
    results = {}
    traces = {
        "whole": rc.trace_whole(requests),
        "tail": rc.trace_decode_tail(requests, tail=32),
        "chunks": rc.trace_chunks(requests),
        "mixed": rc.trace_mixed(requests, max_live=4, seed=3),
    }
    for name, steps in traces.items():
        out = tmp_path / name
        peak = rc.peak_tokens(steps)
        # the mixed trace reuses pages: there every page that lost its holder is overwritten with a
        # large value before the next step, so stale contents that a kernel let through would show
        rc.run_inprocess(model_case["folder"], dtype, steps, out, peak, page_size=model_case["page_size"],
                         fill_freed_pages="poison" if name == "mixed" else None)
        rows = rc.collect(steps, out, vocab)
        assert len(rows) == expected_rows
        _compare(rows, model_case["reference"], dtype)
        results[name] = rows
    if dtype == "float32":
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"
    import kvcore_b200.kernels as K

    assert K.read_status() == 0


def test_pages_are_used_again(model_case, tmp_path):
    """The mixed trace needs more pages over its life than the pool has."""
    steps = rc.trace_mixed(model_case["requests"], max_live=4, seed=3)
    peak = rc.peak_tokens(steps)
    page = model_case["page_size"]
    total = sum(-(-len(t) // page) for t in model_case["requests"].values())
    assert total * page > peak, "the trace would fit without reuse; make it longer"
    step_function, kv = rc.run_inprocess(model_case["folder"], "float32", steps, tmp_path / "o", peak, page_size=page)
    assert kv.pools[0].num_free == kv.pools[0].num_usable


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_case, dtype, tmp_path):
    """The program itself, as a user drives it: a step, its ``done`` line, the next step."""
    if model_case["name"] != "B":
        pytest.skip("one configuration is enough for the subprocess run")
    requests = dict(list(model_case["requests"].items())[:4])
    steps = rc.trace_mixed(requests, max_live=3, seed=5)
    steps.insert(1, {"step": 1000, "entries": [], "end": []})  # a step that brings nothing
    out = tmp_path / "out"
    rc.run_subprocess(model_case["folder"], dtype, steps, out, rc.peak_tokens(steps))
    rows = rc.collect(steps, out, model_case["config"]["vocab_size"])
    assert len(rows) == sum(len(t) for t in requests.values())
    _compare(rows, model_case["reference"], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decode_and_first_tokens(dtype, tmp_path):
    """A prompt of two tokens, then hundreds of single-token steps across many pages; the first
    positions (one and two keys) are compared like the rest."""
    config = rc.TINY_CONFIGS["B"]
    folder = tmp_path / "m"
    rc.write_model(folder, config, 7, "bfloat16")
    weights = plain_llama.load_weights(folder)
    tokens = rc.random_tokens(config["vocab_size"], 400, 21)
    reference = {"long": plain_llama.forward_logits(config, weights, tokens).numpy()}
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": tokens[:2], "want": [0, 1]}], "end": []}]
    for pos in range(2, len(tokens)):
        steps.append({"step": pos, "entries": [{"id": "long", "tokens": [tokens[pos]], "want": [0]}],
                      "end": ["long"] if pos == len(tokens) - 1 else []})
    rc.run_inprocess(folder, dtype, steps, tmp_path / "o", 448)
    rows = rc.collect(steps, tmp_path / "o", config["vocab_size"])
    assert len(rows) == len(tokens)
    _compare(rows, reference, dtype)


def test_far_key_is_seen_through_the_cache(tmp_path):
    """Weights made so that one far key decides the answer: with a strong o/v path a wrong or
    missing page would change the logits far beyond rounding."""
    config = dict(rc.TINY_CONFIGS["A"], max_position_embeddings=1024)
    folder = tmp_path / "m"
    from kvcore_b200.weights import random_state_dict, write_safetensors
    import json

    weights = random_state_dict(config, 3, 0.02, "float32")
    for layer in range(config["num_hidden_layers"]):
        # sharpen attention: larger q/k make single keys stand out among hundreds
        weights[f"model.layers.{layer}.self_attn.q_proj.weight"] *= 12.0
        weights[f"model.layers.{layer}.self_attn.k_proj.weight"] *= 12.0
        weights[f"model.layers.{layer}.self_attn.v_proj.weight"] *= 4.0
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", weights)
    tokens = rc.random_tokens(config["vocab_size"], 600, 5)
    reference = {"r": plain_llama.forward_logits(config, weights, tokens).numpy()}
    requests = {"r": tokens}
    for steps in (rc.trace_chunks(requests, sizes=(200, 3, 150, 2, 97)), rc.trace_decode_tail(requests, 32)):
        out = tmp_path / f"o{len(steps)}"
        rc.run_inprocess(folder, "float32", steps, out, 640)
        _compare(rc.collect(steps, out, config["vocab_size"]), reference, "float32")


def test_replay_refuses_when_pages_run_out(model_case, tmp_path):
    tokens = model_case["requests"]["r3"]
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tokens, "want": [0]}], "end": []}]
    with pytest.raises(RuntimeError, match="no pages"):
        rc.run_inprocess(model_case["folder"], "float32", steps, tmp_path / "o", 64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_graphs_replay_and_match_eager(dtype, tmp_path):
    """Decode-only steps replay a captured CUDA graph: same logits as the eager path, and the
    graph really is replayed (across a change of batch composition and of the table width)."""
    from kvcore_b200.engine.trace_replay import build_replay, replay_stream
    import json

    config = rc.TINY_CONFIGS["B"]
    folder = tmp_path / "m"
    rc.write_model(folder, config, 9, "bfloat16")
    requests = {f"g{i}": rc.random_tokens(config["vocab_size"], n, 40 + i) for i, n in enumerate((150, 90, 60))}
    steps = rc.trace_decode_tail(requests, tail=70)
    mixed = rc.trace_mixed(requests, max_live=3, seed=2, prompt_fraction=0.3)
    for name, trace in (("tail", steps), ("mixed", mixed)):
        results = {}
        for eager in (True, False):
            step_function, kv = build_replay(str(folder), dtype, rc.peak_tokens(trace))
            step_function.use_cuda_graphs = step_function.use_cuda_graphs and not eager
            out = tmp_path / f"{name}_{eager}"
            replay_stream(step_function, kv, [json.dumps(s) for s in trace], out, lambda _: None)
            results[eager] = rc.collect(trace, out, config["vocab_size"])
            if not eager:
                assert step_function.num_graph_replays > 20
                assert len(step_function._graphs) >= (2 if name == "mixed" else 1)
        for key, row in results[True].items():
            if dtype == "float32":
                assert np.array_equal(row, results[False][key]), key
            else:
                assert np.abs(row - results[False][key]).max() < 1e-2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tokens_fed_from_the_device_give_the_logits_of_tokens_from_the_host(dtype, tmp_path):
    """A decode step may take its token ids from a sampler output that the host has not read
    (``StepEntry.fed_from``): same logits as with the ids packed by the host, eagerly, through the
    decode graphs, and beside a portion of a prompt."""
    import torch

    import kvcore_b200.kernels as kernels
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay

    config = rc.TINY_CONFIGS["B"]
    folder = tmp_path / "m"
    rc.write_model(folder, config, 4, "bfloat16")
    vocab = config["vocab_size"]
    prompts = {f"f{i}": rc.random_tokens(vocab, n, 60 + i) for i, n in enumerate((21, 9, 34))}
    late = rc.random_tokens(vocab, 12, 77)
    decoded = [rc.random_tokens(vocab, 3, 80 + step) for step in range(8)]

    def run(fed: bool):
        step_function, kv = build_replay(str(folder), dtype, 512)
        rows = []
        for rid, tokens in prompts.items():
            assert kv.allocate_slots(rid, len(tokens))
        step_function.step([StepEntry(rid, tokens, ()) for rid, tokens in prompts.items()])
        for step, tokens in enumerate(decoded):
            entries = []
            # rows of the "sampler output" in another order than the entries, with a row nobody takes
            feedback = torch.tensor([tokens[2], 1, tokens[0], tokens[1]], dtype=torch.int32, device="cuda:0")
            for (rid, token), row in zip(zip(prompts, tokens), (2, 3, 0)):
                assert kv.allocate_slots(rid, 1)
                entries.append(StepEntry(rid, (0,), (0,), fed_from=row) if fed else StepEntry(rid, (token,), (0,)))
            if step == 5:   # a prompt portion beside the fed tokens
                assert kv.allocate_slots("late", len(late))
                entries.insert(1, StepEntry("late", late, (len(late) - 1,)))
            rows.append(step_function.step(entries, feedback if fed else None).float().cpu())
        assert kernels.read_status() == 0
        return rows, step_function.num_graph_replays

    host_rows, _ = run(False)
    fed_rows, replays = run(True)
    assert replays >= 4
    for a, b in zip(host_rows, fed_rows):
        assert torch.equal(a, b)


def test_decode_step_with_more_work_items_than_block_slots(tmp_path):
    """160 live requests on a model with two kv heads: 320 (request, kv head) items for the 296 block
    slots of the decode attention, so its blocks stay and share the items.  The logits of one decode
    step, eagerly and through a graph, are those of the plain implementation."""
    import torch

    import kvcore_b200.kernels as kernels
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay

    config = rc.TINY_CONFIGS["D"]
    folder = tmp_path / "m"
    rc.write_model(folder, config, 3, "bfloat16")
    weights = plain_llama.load_weights(folder)
    vocab = config["vocab_size"]
    lengths = [40 + (37 * i) % 150 for i in range(160)]
    requests = {f"q{i}": rc.random_tokens(vocab, n + 3, 300 + i) for i, n in enumerate(lengths)}
    step_function, kv = build_replay(str(folder), "bfloat16", 64 * 160 * 4, max_live=160)
    assert kernels.decode_splits_tma(160, 2, 256) * 160 * 2 > 296
    ids = list(requests)
    for begin in range(0, 160, 16):                      # prompts, sixteen requests a step
        entries = []
        for rid, n in zip(ids[begin:begin + 16], lengths[begin:begin + 16]):
            assert kv.allocate_slots(rid, n)
            entries.append(StepEntry(rid, requests[rid][:n], ()))
        step_function.step(entries)
    sample = ids[::23]
    reference = {rid: plain_llama.forward_logits(config, weights, requests[rid]).numpy() for rid in sample}
    for step in range(3):                                # the third step replays the graph captured in the second
        entries = []
        for rid, n in zip(ids, lengths):
            assert kv.allocate_slots(rid, 1)
            entries.append(StepEntry(rid, (requests[rid][n + step],), (0,)))
        logits = step_function.step(entries).float().cpu().numpy()
        assert np.isfinite(logits).all()
        for rid in sample:
            row, want = logits[ids.index(rid)], reference[rid][lengths[ids.index(rid)] + step]
            assert np.abs(row - want).max() <= TOLERANCE["bfloat16"] * np.abs(reference[rid]).max(), (rid, step)
    assert step_function.num_graph_replays >= 1 and kernels.read_status() == 0
