"""The engine at the layer sizes of Llama 3.1 8B (hidden 4096, 32 query and 8 kv heads of 128,
feed-forward 14336, vocabulary 128256, llama3 rope scaling 8 / 8192) with 2 of its 32 layers and
random weights: fewer layers, not smaller ones, so that every kernel runs at the shapes it serves.

The tiny models of the other tests never reach these branches together: the streaming products
with K = 4096 and 14336 and their fused norm, activation and residual, weight tiles shared by
several blocks, the library products above 16 rows, 16-way splits of the decode attention, block
tables hundreds of pages wide, graphs whose bound on the sequence length is far from its true
value, the 32-bit product at N = 128256.  Compared with the plain implementation
(tests/plain_llama.py; formulas of kvcore/model/models/llama3.py:124-142, 182-247) evaluated in
64-bit on the GPU with torch's elementary operations."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_llama
import replay_cases as rc

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
LLAMA31_8B_2L = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=128256, hidden_size=4096,
    intermediate_size=14336, num_hidden_layers=2, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, max_position_embeddings=131072, tie_word_embeddings=False, rms_norm_eps=1e-5,
    rope_theta=500000.0, hidden_act="silu",
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
)
VOCAB = LLAMA31_8B_2L["vocab_size"]
TOLERANCE = {"float32": 2e-5, "bfloat16": 2e-2}   # of the request's largest |logit|, as in test_replay_gpu.py


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    folder = tmp_path_factory.mktemp("llama31_8b_2l")
    rc.write_model(folder, LLAMA31_8B_2L, 5, "bfloat16")
    weights = {name: t.to(DEV) for name, t in plain_llama.load_weights(folder).items()}
    return dict(folder=folder, weights=weights)


def oracle(model, tokens, rows):
    """64-bit logits of the plain implementation at ``rows`` and the largest |logit| among them."""
    with torch.no_grad():
        logits = plain_llama.forward_logits(LLAMA31_8B_2L, model["weights"], tokens, compute=torch.float64,
                                            rows=rows, device=DEV)
    out = logits.float().cpu().numpy()
    del logits
    torch.cuda.empty_cache()
    return {row: out[i] for i, row in enumerate(rows)}, float(np.abs(out).max())


CHUNK_SIZES = (257, 3, 64, 2, 129, 16, 300, 5)


def interesting_positions(length: int) -> set[int]:
    """The first tokens, both sides of the edges of pages (16), key tiles (64, 128, ...) and of the
    portions that CHUNK_SIZES cuts, and the last 34 tokens."""
    keep = {0, 1, 2}
    edges, cursor = [16, 64, 128, 256, 512, 1024], 0
    for size in CHUNK_SIZES:
        cursor += size
        edges.append(cursor)
    for edge in edges:
        keep.update((edge - 1, edge, edge + 1))
    keep.update(range(length - 34, length))
    return {p for p in keep if 0 <= p < length}


def compare(rows, expected, scale, tolerance, what):
    errors = {key: float(np.abs(row - expected[key]).max()) / scale[key[0]] for key, row in rows.items()}
    for key, row in rows.items():
        assert np.isfinite(row).all(), f"{what}: non-finite logits at {key}"
    wrong = sorted(key for key, err in errors.items() if err > tolerance)
    assert not wrong, f"{what}: first wrong position {wrong[0]} (error {errors[wrong[0]]:.3e}), {len(wrong)} in all"
    return max(errors.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cuttings_at_real_layer_sizes(model, dtype, tmp_path):
    """Requests of ~300 and ~1,100 tokens and two short ones: whole, last 32 tokens one by one,
    portions of changing size, and mixed with so few pages that they are used again.  In 32-bit the
    cuttings agree bit for bit."""
    from kvcore_b200.engine.trace_replay import build_replay
    import kvcore_b200.kernels as K

    lengths = dict(r0=301, r1=1103, r2=40, r3=90, r4=150, r5=70)
    requests = {rid: rc.random_tokens(VOCAB, n, 500 + i) for i, (rid, n) in enumerate(lengths.items())}
    keep = {rid: interesting_positions(n) for rid, n in lengths.items()}
    expected, scale = {}, {}
    for rid, tokens in requests.items():
        rows, scale[rid] = oracle(model, tokens, sorted(keep[rid]))
        expected.update({(rid, pos): row for pos, row in rows.items()})
    traces = {
        "whole": rc.trace_whole(requests),
        "tail": rc.trace_decode_tail(requests, tail=32),
        "chunks": rc.trace_chunks(requests, sizes=CHUNK_SIZES),
        "mixed": rc.trace_mixed(requests, max_live=4, seed=11),
    }
    traces = {name: rc.keep_wants(steps, keep) for name, steps in traces.items()}
    pool = max(rc.peak_tokens(steps) for steps in traces.values())
    assert sum(-(-n // 64) * 64 for n in lengths.values()) > pool, "the requests fit all at once: no page is used again"
    step_function, kv = build_replay(str(model["folder"]), dtype, pool, fill_freed_pages="poison")
    results = {}
    for name, steps in traces.items():
        out = tmp_path / name
        rc.run_on(step_function, kv, steps, out)
        rows = rc.collect(steps, out, VOCAB)
        assert set(rows) == set(expected)
        compare(rows, expected, scale, TOLERANCE[dtype], f"{dtype} {name}")
        results[name] = rows
    if dtype == "float32":
        for name in ("tail", "chunks", "mixed"):
            for key, row in results["whole"].items():
                assert np.array_equal(row, results[name][key]), f"{name} differs from whole at {key}"
    else:
        assert step_function.num_graph_replays > 0
    assert K.read_status() == 0


def test_decode_batches_of_1_8_and_64_at_real_layer_sizes(model):
    """bfloat16 decode steps of 64, 8 and 1 requests (three each: eager, captured, replayed): the
    streaming products at up to 16 rows, the library products above, the graphs."""
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay
    import kvcore_b200.kernels as K

    count = 64
    lengths = [20 + (37 * i) % 101 for i in range(count)]
    requests = {f"d{i}": rc.random_tokens(VOCAB, n + 9, 700 + i) for i, n in enumerate(lengths)}
    ids = list(requests)
    step_function, kv = build_replay(str(model["folder"]), "bfloat16", count * 192, max_live=count)
    for begin in range(0, count, 16):
        entries = []
        for rid, n in zip(ids[begin:begin + 16], lengths[begin:begin + 16]):
            assert kv.allocate_slots(rid, n)
            entries.append(StepEntry(rid, requests[rid][:n], ()))
        assert step_function.step(entries) is None
    done = dict(zip(ids, lengths))
    compared = {64: (0, 7, 33, 63), 8: (0, 7), 1: (0,)}
    got: dict[tuple[str, int], np.ndarray] = {}
    for batch in (64, 8, 1):
        replays = step_function.num_graph_replays
        for _ in range(3):
            entries = []
            for rid in ids[:batch]:
                assert kv.allocate_slots(rid, 1)
                entries.append(StepEntry(rid, (requests[rid][done[rid]],), (0,)))
            logits = step_function.step(entries).float().cpu().numpy()
            for index in compared[batch]:
                got[(ids[index], done[ids[index]])] = logits[index]
            for rid in ids[:batch]:
                done[rid] += 1
        assert step_function.num_graph_replays == replays + 2
    assert K.read_status() == 0
    for index in compared[64]:
        rid = ids[index]
        rows = sorted(pos for r, pos in got if r == rid)
        expected, scale = oracle(model, requests[rid][:done[rid]], rows)
        for pos in rows:
            err = float(np.abs(got[(rid, pos)] - expected[pos]).max()) / scale
            assert err <= TOLERANCE["bfloat16"], f"{rid} position {pos}: error {err:.3e}"


def test_decode_on_8192_tokens_of_context_written_by_chunked_prefill(model):
    """Every request holds 8,192 tokens that went through the model in portions of 2,048 (the cache is
    what the prefill kernels wrote, not a random fill); then decode steps of 64, 8 and 1 requests.
    Block tables are 513 pages wide and the decode attention splits each request's keys 16 ways at
    the small batches."""
    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.engine.trace_replay import build_replay
    import kvcore_b200.kernels as K

    count, context, portion = 64, 8192, 2048
    generator = torch.Generator().manual_seed(900)
    tokens = torch.randint(0, VOCAB, (count, context + 9), generator=generator).tolist()
    ids = [f"c{i}" for i in range(count)]
    step_function, kv = build_replay(str(model["folder"]), "bfloat16", count * (context + 64), max_live=count)
    for rid, row in zip(ids, tokens):
        for begin in range(0, context, portion):
            assert kv.allocate_slots(rid, portion)
            assert step_function.step([StepEntry(rid, row[begin:begin + portion], ())]) is None
    assert K.decode_splits_tma(1, 8, context + 16) == 16
    done = {rid: context for rid in ids}
    compared = {64: (0, 5, 63), 8: (0, 5), 1: (0,)}
    got: dict[tuple[int, int], np.ndarray] = {}
    for batch in (64, 8, 1):
        for _ in range(3):
            entries = []
            for index in range(batch):
                assert kv.allocate_slots(ids[index], 1)
                entries.append(StepEntry(ids[index], (tokens[index][done[ids[index]]],), (0,)))
            logits = step_function.step(entries).float().cpu().numpy()
            for index in compared[batch]:
                got[(index, done[ids[index]])] = logits[index]
            for index in range(batch):
                done[ids[index]] += 1
    assert step_function.last_context.table_width >= 513 and step_function.num_graph_replays >= 3
    assert K.read_status() == 0
    for index in compared[64]:
        rows = sorted(pos for i, pos in got if i == index)
        expected, scale = oracle(model, tokens[index][:done[ids[index]]], rows)
        for pos in rows:
            err = float(np.abs(got[(index, pos)] - expected[pos]).max()) / scale
            assert err <= TOLERANCE["bfloat16"], f"request {index} position {pos}: error {err:.3e}"
