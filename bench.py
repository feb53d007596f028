"""Benchmark: decode and prefill throughput of the Llama 3.1 8B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shape llama31_8b|llama32_3b|llama3_70b] [--serve]

Prints one JSON line.  ``value`` is decoded tokens per second at batch 8 with every request
holding ``context_len`` tokens in the cache (a "step" is one decode step of the whole batch,
sampling included), timed on the device with CUDA events around exactly K steps after W
warm-up steps.  ``e2e`` is the same workload through the Python entry point
(``LLMEngine.step``): every step uploads its inputs from pinned host memory and reads the
sampled tokens back.  ``prefill`` times one 2,048-token prompt; ``roofline`` relates the bytes
a decode step must read (every weight once, and the cache of the live requests) to its
time.  ``points`` holds decode at batch 1 and 64, and the same batches at 1,024 tokens of
context.  Weights are 15 GB, so consecutive steps cannot reuse the L2 cache.

``--shape`` runs the same measurements at the layer sizes of Llama 3.2 3B (tied embeddings, 3 query
heads a kv head) or Llama 3 70B (8 query heads a kv head, 2,048 tokens of context, batches 1/8/32);
``--serve`` times continuous batching of 64 requests through ``LLMEngine.generate`` instead and
prints a line of its own.
"""
from __future__ import annotations

import argparse
import gc
import json
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LLAMA_31_8B = dict(
    architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=128256, hidden_size=4096,
    intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, max_position_embeddings=131072, tie_word_embeddings=False, rms_norm_eps=1e-5,
    rope_theta=500000.0, hidden_act="silu",
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
)
LLAMA_32_3B = dict(
    LLAMA_31_8B, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
    tie_word_embeddings=True,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
)
LLAMA_3_70B = dict(
    LLAMA_31_8B, hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
    max_position_embeddings=8192, rope_scaling=None,
)
# name -> (config.json, label, context of the headline decode number, batches of the side points)
SHAPES = {
    "llama31_8b": (LLAMA_31_8B, "Llama-3.1-8B shape", 8192, (1, 64)),
    "llama32_3b": (LLAMA_32_3B, "Llama-3.2-3B shape", 8192, (1, 64)),
    "llama3_70b": (LLAMA_3_70B, "Llama-3-70B shape", 2048, (1, 32)),
}
CONTEXT_LEN = 8192
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            # the prefill is one step timed on its own: the burst figure is its denominator (the same
            # kind of number as the fallback), not the one of a seconds-long loop under the power cap
            return dict(hbm_gbs=float(raw["hbm_gbs"]), bf16_tflops=float(raw["bf16_tflops"]), source="measured")
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed regions run."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.path = Path(tempfile.mkstemp(suffix=".csv")[1])
        self.process = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.path.open("w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self) -> dict:
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 6:
                continue
            try:
                clocks.append(float(fields[0]))
                max_clock = float(fields[1])
            except ValueError:
                continue
            for name, value in zip(names, fields[2:6]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        self.path.unlink(missing_ok=True)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(config: dict, layers: int) -> dict:
    e, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    h, kvh, d = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    per_layer = (h + 2 * kvh) * d * e + e * h * d + 2 * i * e + e * i + 2 * e
    return dict(
        layer_params=per_layer,
        streamed_params=layers * per_layer + v * e + e,  # every matrix once, the head, the final norm
        kv_bytes_per_token=layers * 2 * kvh * d * 2,
        heads=h, head_dim=d, hidden=e, vocab=v,
    )


def build_runner(shape: dict, layers: int, max_seqs: int, max_len: int, num_pages: int, max_tokens: int):
    import torch

    from kvcore_b200 import CacheConfig, DeviceConfig, KVCoreConfig, LoadConfig, ModelConfig, SchedulerConfig
    from kvcore_b200.engine.runner import ModelRunner

    folder = Path(tempfile.mkdtemp(prefix="kvcore_bench_"))
    (folder / "config.json").write_text(json.dumps({k: v for k, v in dict(shape, num_hidden_layers=layers).items() if v is not None}))
    config = KVCoreConfig(
        model_config=ModelConfig(model=str(folder), dtype="bfloat16", max_model_len=max_len),
        load_config=LoadConfig(random_weights=True, seed=0),
        cache_config=CacheConfig(block_size=BLOCK_SIZE, num_gpu_blocks=num_pages),
        scheduler_config=SchedulerConfig(max_num_seqs=max_seqs, max_num_scheduled_tokens=max_tokens,
                                         max_num_partial_prefills=max_seqs, max_long_partial_prefills=max_seqs),
        device_config=DeviceConfig(device="cuda:0"),
    )
    runner = ModelRunner(config)
    for tensor in runner.storage.group_tensors:  # a cache of plausible values, not zeros
        flat = tensor.view(-1)
        chunk = 1 << 28
        for begin in range(0, flat.numel(), chunk):
            flat[begin : begin + chunk].normal_(0.0, 0.5)
    torch.cuda.synchronize()
    return config, runner


def time_decode(runner, batch: int, context: int, steps: int, warmup: int) -> float:
    """Milliseconds per decode step of ``batch`` requests that each hold ``context`` tokens."""
    import torch

    from kvcore_b200.engine.step import StepEntry
    from kvcore_b200.sampling import SamplingParams

    kv = runner.kv_manager
    for rid in kv.live_requests():
        kv.free(rid)
    ids = [f"bench-{i}" for i in range(batch)]
    for rid in ids:
        assert kv.allocate_slots(rid, context), "cache too small for the benchmark batch"
        kv.advance(rid, context)
    generator = torch.Generator().manual_seed(1)
    vocab = runner.model.spec.vocab_size
    tokens = torch.randint(0, vocab, (steps + warmup, batch), generator=generator).tolist()
    params = [SamplingParams(max_tokens=1, temperature=0.0)] * batch
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one_step(index: int) -> None:
        entries = []
        for rid, token in zip(ids, tokens[index]):
            assert kv.allocate_slots(rid, 1)
            entries.append(StepEntry(rid, [token], (0,)))
        logits = runner.step_function.step(entries)
        runner.sampler.sample(logits, params, [0] * batch, [index] * batch)

    for index in range(warmup):
        one_step(index)
    torch.cuda.synchronize()
    start.record()
    for index in range(warmup, warmup + steps):
        one_step(index)
    stop.record()
    torch.cuda.synchronize()
    for rid in ids:
        kv.free(rid)
    return start.elapsed_time(stop) / steps


def time_prefill(runner, tokens: int, repeats: int, warmup: int) -> float:
    import torch

    from kvcore_b200.engine.step import StepEntry

    kv = runner.kv_manager
    generator = torch.Generator().manual_seed(2)
    vocab = runner.model.spec.vocab_size
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0.0
    for index in range(warmup + repeats):
        prompt = torch.randint(0, vocab, (tokens,), generator=generator).tolist()
        assert kv.allocate_slots("prefill", tokens)
        torch.cuda.synchronize()
        start.record()
        runner.step_function.step([StepEntry("prefill", prompt, (tokens - 1,))])
        stop.record()
        torch.cuda.synchronize()
        kv.free("prefill")
        if index >= warmup:
            total += start.elapsed_time(stop)
    return total / repeats


def check_logits(runner, shape: dict, layers: int, batch: int = 8) -> dict:
    """Before anything is timed: the model that is about to be timed, with its own weights, against the
    plain implementation (tests/plain_llama.py, evaluated in 32-bit on the GPU with elementary torch
    operations on the weights read back from the model).  Two requests of 333 and 700 tokens go
    through the step function in portions of 256 beside each other, six short ones beside them, then
    three decode steps of the whole batch (run eagerly, captured, replayed); the logits at the end of
    the prompts and at every decode step of three of the requests are compared."""
    import torch

    sys.path.insert(0, str(ROOT / "tests"))
    import plain_llama

    from kvcore_b200.engine.step import StepEntry
    import kvcore_b200.kernels as K

    kv, step_function = runner.kv_manager, runner.step_function
    for rid in kv.live_requests():
        kv.free(rid)
    vocab = shape["vocab_size"]
    generator = torch.Generator().manual_seed(5)
    lengths = [333, 700] + [50 + 7 * i for i in range(batch - 2)]
    tokens = [torch.randint(0, vocab, (n + 3,), generator=generator).tolist() for n in lengths]
    ids = [f"check-{i}" for i in range(len(lengths))]
    got: dict[tuple[int, int], torch.Tensor] = {}
    done = [0] * len(lengths)
    while any(d < n for d, n in zip(done, lengths)):
        entries, rows = [], []
        for index, (rid, n) in enumerate(zip(ids, lengths)):
            if done[index] >= n:
                continue
            size = min(256, n - done[index])
            assert kv.allocate_slots(rid, size)
            last = done[index] + size == n
            entries.append(StepEntry(rid, tokens[index][done[index]:done[index] + size], (size - 1,) if last else ()))
            if last:
                rows.append((index, n - 1))
            done[index] += size
        logits = step_function.step(entries)
        for row, key in enumerate(rows):
            got[key] = logits[row].float().cpu()
    for _ in range(3):
        entries = []
        for index, rid in enumerate(ids):
            assert kv.allocate_slots(rid, 1)
            entries.append(StepEntry(rid, (tokens[index][done[index]],), (0,)))
        logits = step_function.step(entries).float().cpu()
        for index in range(len(ids)):
            got[(index, done[index])] = logits[index]
            done[index] += 1
    for rid in ids:
        kv.free(rid)
    status = K.read_status()
    if status:
        raise RuntimeError(f"a kernel reported status {status} during the logits check")
    config = {k: v for k, v in dict(shape, num_hidden_layers=layers).items() if v is not None}
    weights = runner.model.state_dict()
    worst = oracle_worst = rms_worst = oracle_rms_worst = 0.0
    checked = 0
    with torch.no_grad():
        for index in (0, 1, batch - 1):
            rows = sorted(pos for i, pos in got if i == index)
            sequence = tokens[index][:done[index]]
            exact = plain_llama.forward_logits(config, weights, sequence, compute=torch.float32, rows=rows,
                                               device="cuda:0").float().cpu()
            rounded = plain_llama.forward_logits(config, weights, sequence, compute=torch.float32, rows=rows,
                                                 device="cuda:0", round_to=torch.bfloat16).float().cpu()
            scale = float(exact.abs().max())
            for row, pos in enumerate(rows):
                mine, theirs = got[(index, pos)] - exact[row], rounded[row] - exact[row]
                worst = max(worst, float(mine.abs().max()) / scale)
                oracle_worst = max(oracle_worst, float(theirs.abs().max()) / scale)
                rms_worst = max(rms_worst, float(mine.pow(2).mean().sqrt()) / scale)
                oracle_rms_worst = max(oracle_rms_worst, float(theirs.pow(2).mean().sqrt()) / scale)
                checked += 1
    del weights
    torch.cuda.empty_cache()
    # What bfloat16 costs grows with depth (random weights: 1.4e-2 of the largest logit at 2 layers,
    # 6e-2 at 32), so the yardstick is the plain implementation itself evaluated with bfloat16
    # roundings in the reference's places: the engine may stray from 32-bit at most 1.5 times as far as
    # that evaluation does in its worst entry, and 1.3 times in the worst row's root mean square
    # (measured: 0.98 to 1.09, and 1.00 to 1.06, at 2 to 32 layers).
    if not (worst <= 1.5 * oracle_worst and rms_worst <= 1.3 * oracle_rms_worst):
        raise RuntimeError(
            f"logits of the benchmark model stray from the plain implementation: worst entry {worst:.3e} of the "
            f"largest logit (a faithful bfloat16 evaluation: {oracle_worst:.3e}), worst row rms {rms_worst:.3e} "
            f"(faithful: {oracle_rms_worst:.3e})")
    return {"logits_checked": True, "logits_max_err": round(worst, 5), "logits_max_err_faithful_bf16": round(oracle_worst, 5),
            "logits_rms_err": round(rms_worst, 5), "logits_rms_err_faithful_bf16": round(oracle_rms_worst, 5),
            "logits_rows_checked": checked}


def time_e2e(config, runner, batch: int, context: int, steps: int, warmup: int) -> dict:
    """Decode steps through ``LLMEngine.step``: host token ids in, sampled token ids out."""
    import torch

    from kvcore_b200.engine.llm_engine import LLMEngine
    from kvcore_b200.sampling import SamplingParams

    for rid in runner.kv_manager.live_requests():
        runner.kv_manager.free(rid)
    engine = LLMEngine(config, model_runner=runner)
    generator = torch.Generator().manual_seed(3)
    vocab = runner.model.spec.vocab_size
    for index in range(batch):
        prompt = torch.randint(0, vocab, (context,), generator=generator).tolist()
        # requests admitted early decode while later ones still prefill: leave room for that
        engine.add_request(f"e2e-{index}", SamplingParams(max_tokens=1_000_000, temperature=0.0),
                           prompt_token_ids=prompt)
    scheduler = engine.engine_core.scheduler
    while any(r.num_computed_tokens < r.num_prompt_tokens for r in scheduler.requests.values()):
        engine.step()  # prefill, untimed
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    used_before = runner.step_function.num_steps
    # (as `timeit` does: no collection of host garbage inside the few timed milliseconds)
    gc.collect()
    gc.disable()
    try:
        begin = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += sum(1 for o in engine.step().request_outputs if o.sampled_token_id is not None)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - begin
    finally:
        gc.enable()
    # with a step kept in flight, one more step than has been read is launched at either end
    assert abs(runner.step_function.num_steps - used_before - steps) <= 1
    assert produced == steps * batch, f"{produced} tokens from {steps} steps of {batch} requests"
    ctx = runner.step_function.last_context
    h2d = 4 * (4 * (batch + 4) + 4 * batch + batch * ctx.table_width) + batch * 6 * 8
    if engine.engine_core.num_steps_run_ahead:
        h2d += 4 * batch   # which row of the sampler output each token id comes from
    engine.engine_core.drain()
    engine.engine_core.scheduler.shutdown()
    runner.remove_requests(list(runner.requests))
    return {"value": produced / elapsed, "unit": "tokens/s", "ms_per_step": 1000.0 * elapsed / steps,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch,
            "steps_launched_ahead": engine.engine_core.num_steps_run_ahead}


def time_serving(shape: dict, layers: int, requests: int, min_prompt: int, max_prompt: int, chunk: int,
                 max_tokens: int) -> dict:
    """Continuous batching through ``LLMEngine.generate``: ``requests`` prompts of seeded random
    lengths in [min_prompt, max_prompt], at most ``chunk`` tokens a step (portions of prompts beside
    the decoding requests), ``max_tokens`` greedy tokens each.  Host wall clock, everything included."""
    import torch

    from kvcore_b200.engine.llm_engine import LLMEngine
    from kvcore_b200.sampling import SamplingParams

    generator = torch.Generator().manual_seed(4)
    lengths = torch.randint(min_prompt, max_prompt + 1, (requests,), generator=generator).tolist()
    max_len = max_prompt + max_tokens
    pages = sum(-(-(n + max_tokens) // BLOCK_SIZE) for n in lengths) + 1
    config, runner = build_runner(shape, layers, requests, max_len, pages, chunk)
    vocab = runner.model.spec.vocab_size
    batch = [dict(request_id=f"serve-{i}", sampling_params=SamplingParams(max_tokens=max_tokens, temperature=0.0),
                  prompt_token_ids=torch.randint(0, vocab, (n,), generator=generator).tolist())
             for i, n in enumerate(lengths)]
    engine = LLMEngine(config, model_runner=runner)
    engine.generate(batch[:2])  # warm-up: kernels loaded, first graphs captured
    for item in batch:
        item["request_id"] += "-timed"
    torch.cuda.synchronize()
    steps_before = runner.step_function.num_steps
    begin = time.perf_counter()
    outputs = engine.generate(batch)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - begin
    generated = sum(len(o.output_token_ids) for o in outputs)
    assert generated == requests * max_tokens, f"{generated} tokens from {requests} requests"
    return {"seconds": round(elapsed, 3), "requests": requests, "prompt_tokens": sum(lengths),
            "generated_tokens": generated, "steps": runner.step_function.num_steps - steps_before,
            "generated_tokens_per_s": round(generated / elapsed, 1),
            "total_tokens_per_s": round((generated + sum(lengths)) / elapsed, 1),
            "chunk": chunk, "prompt_lengths": f"{min_prompt}-{max_prompt}", "max_tokens": max_tokens,
            "steps_launched_ahead": engine.engine_core.num_steps_run_ahead}


def reference_arm(args) -> int:
    """The unmodified reference, run through its own step loop at the headline's shape.

    ``baseline/_ref/kvcore`` is a plain copy of the reference's pure-Python package (its offline pip
    install fails: the build backend, hatchling, is neither installed nor among the offline wheels).
    Nothing of this repository's engine is on the path: the reference's own ``Llama3ForCausalLM`` is
    built from an in-memory ``LlamaConfig`` (transformers serves as the configuration container the
    reference asks for) with N(0, 0.02) bfloat16 weights on the GPU, and driven by the reference's own
    ``EngineCore.step`` (kvcore/engine/engine_core.py:103-149: ``Scheduler.schedule`` ->
    ``ModelRunner.execute_model`` -> ``sample_tokens`` -> ``update_from_outputs``) with its stock CUDA
    attention backend ``triton_paged``.  Only ``EngineCore.__init__`` is bypassed, because it loads a
    tokenizer and a checkpoint folder that do not exist offline; requests are given as token ids.
    Same batch, same context reached by its own chunked prefill (untimed), same steps and warm-up;
    ``value`` from CUDA events, ``e2e`` from the wall clock (the reference reads its tokens back every
    step, so the two nearly coincide).  Anything that goes wrong is reported as ``unavailable`` with
    the error's own text."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "kvcore").is_dir():
        print(json.dumps({"impl": "reference", "unavailable":
                          "baseline/_ref/kvcore is missing (the offline pip install of the reference fails for want "
                          "of its build backend hatchling; a plain copy of its kvcore/ package goes there instead)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU only"}))
        return 0
    try:
        line = _run_reference(args, ref)
    except BaseException as error:  # the arm must print its line whatever happens
        if isinstance(error, KeyboardInterrupt):
            raise
        text = " ".join(f"{type(error).__name__}: {error}".split())[:400]
        line = {"impl": "reference", "unavailable": f"the reference failed while running: {text}"}
    print(json.dumps(line))
    return 0


def _run_reference(args, ref: Path) -> dict:
    sys.path.insert(0, str(ref))
    sys.dont_write_bytecode = True
    import torch
    from transformers.models.llama.configuration_llama import LlamaConfig  # configuration container only

    from kvcore.config import CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SchedulerConfig
    from kvcore.engine.engine_core import EngineCore
    from kvcore.model.model_runner import ModelRunner
    from kvcore.model.models.llama3 import Llama3ForCausalLM
    from kvcore.sched.scheduler import Scheduler
    from kvcore.utils.request import Request
    from kvcore.utils.sampling_params import SamplingParams

    shape, label, shape_context, _ = SHAPES[args.shape]
    layers = args.layers or shape["num_hidden_layers"]
    context = args.context or shape_context
    batch, steps, warmup = args.batch, args.steps, max(args.warmup, 3)
    keys = ("vocab_size", "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads",
            "head_dim", "max_position_embeddings", "tie_word_embeddings", "rms_norm_eps")
    # the reference's rotary layer reads the base only (kvcore/model/layer/rotary_embedding.py:38-49): it has no
    # llama3 frequency scaling, which changes a table of 64 numbers and no cost
    hf = LlamaConfig(**{k: shape[k] for k in keys}, num_hidden_layers=layers,
                     rope_parameters={"rope_type": "default", "rope_theta": shape["rope_theta"]})
    # The reference's Triton kernels form the offset of a cache block as block_id * stride in 32-bit
    # (kvcore/model/attn_backend/triton_paged.py:66-80, 159-165: both factors are 32-bit integers), and
    # all layers share one tensor of blocks: with blocks of 16 tokens x 8 heads x 128 it can address
    # block ids below 2^31 / 16384 = 131,072.  Batch 8 x 8,192 tokens x 32 layers needs ids up to 131,840;
    # run at that size its kernel made an illegal memory access.  The arm therefore never gives it a
    # pool it cannot address: where the stated context does not fit, it runs the largest context (a
    # multiple of 64) that does, and says so in its line.
    block_elems = BLOCK_SIZE * shape["num_key_value_heads"] * shape["head_dim"]
    addressable = (1 << 31) // block_elems - 1                 # largest pool (null block included) whose ids are safe
    extra = steps + warmup + 4
    per_pair = addressable // (layers * batch) - 2             # blocks a (request, layer) pair may use, two to spare
    stated_context = context
    if -(-(context + extra) // BLOCK_SIZE) > per_pair:
        context = (per_pair * BLOCK_SIZE - extra) // 64 * 64
        if context <= 0:
            raise RuntimeError(f"the reference cannot address a cache for batch {batch} at {layers} layers")
    max_len = context + extra + 60
    blocks = min(layers * batch * (-(-(context + extra) // BLOCK_SIZE) + 2) + 1, addressable)
    assert (blocks - 1) * block_elems < (1 << 31)
    config = KVCoreConfig(
        model_config=ModelConfig(model="unused", hf_config=hf, dtype=torch.bfloat16, max_model_len=max_len),
        cache_config=CacheConfig(block_size=BLOCK_SIZE, num_gpu_blocks=blocks, profile_kv_cache=False,
                                 enable_caching=False),
        scheduler_config=SchedulerConfig(max_num_seqs=batch, max_num_scheduled_tokens=PREFILL_TOKENS,
                                         max_num_partial_prefills=batch, max_long_partial_prefills=batch),
        device_config=DeviceConfig(device="cuda:0"),
    )
    backend = config.model_config.attn_backend        # the reference's own choice on a CUDA device
    torch.manual_seed(0)
    previous = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda:0"):
            model = Llama3ForCausalLM(config)
    finally:
        torch.set_default_dtype(previous)
    with torch.no_grad():
        for name, parameter in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                parameter.fill_(1.0)
            else:
                parameter.normal_(0.0, 0.02)
    model.eval()

    core = EngineCore.__new__(EngineCore)      # its __init__ wants a tokenizer and a checkpoint folder
    core.kvcore_config = config
    core.model_runner = ModelRunner(config)
    core.model_runner.model = model
    core.stop_token_ids = set()
    core.finished_outputs = {}
    kv_config = core._build_kv_manager_config()
    core.scheduler = Scheduler(config, kv_config)
    core.model_runner.initialize_kv_cache(kv_config)

    generator = torch.Generator().manual_seed(3)
    for index in range(batch):
        prompt = torch.randint(0, shape["vocab_size"], (context,), generator=generator).tolist()
        core.scheduler.add_request(Request(request_id=f"ref-{index}", prompt_token_ids=prompt,
                                           sampling_params=SamplingParams(max_tokens=1_000_000, temperature=0.0)))

    def sampled(outputs) -> int:
        return sum(1 for o in outputs.request_outputs if o.sampled_token_id is not None)

    prefill_began = time.perf_counter()
    guard = 0
    while sampled(core.step()) < batch:          # its own chunked prefill, untimed
        guard += 1
        if guard > 4 * batch * (-(-context // PREFILL_TOKENS)) + 16:
            raise RuntimeError("the reference did not reach a step in which every request decodes")
    torch.cuda.synchronize()
    prefill_seconds = time.perf_counter() - prefill_began
    for _ in range(warmup):
        assert sampled(core.step()) == batch
    sampler = ClockSampler()
    sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    gc.collect()          # the same for both arms: no collection of host garbage inside the timed steps
    gc.disable()
    try:
        began = time.perf_counter()
        start.record()
        produced = 0
        for _ in range(steps):
            produced += sampled(core.step())
        stop.record()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - began
    finally:
        gc.enable()
    clocks = sampler.stop()
    assert produced == steps * batch, f"{produced} tokens from {steps} steps of {batch} requests"
    ms_step = start.elapsed_time(stop) / steps
    peaks = measured_peaks()
    numbers = model_numbers(shape, layers)
    step_bytes = 2.0 * numbers["streamed_params"] + batch * context * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    return {
        "metric": f"decode tokens/s, {label.replace('-', ' ')}, batch {batch}, bf16",
        "value": round(batch * 1000.0 / ms_step, 2), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "impl": "reference",
        "data": "synthetic: random N(0,0.02) weights, seeded uniform-random token ids, cache written by its own prefill",
        "config": {
            "model": label, "layers": layers, "layers_of_config": shape["num_hidden_layers"],
            "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
            "kv_heads": shape["num_key_value_heads"], "head_dim": shape["head_dim"],
            "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
            "tied_embeddings": shape["tie_word_embeddings"], "global_batch": batch, "seq_len": context,
            "context_len": context, "block_size": BLOCK_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU", "attn_backend": backend, "stated_context_len": stated_context,
            "l2": f"weights of {2e-9 * numbers['streamed_params']:.0f} GB stream every step: inputs larger than L2",
        },
        "same_config": context == stated_context,
        "note": ("" if context == stated_context else
                 f"the reference's Triton kernels address its shared block tensor with 32-bit offsets (block ids below "
                 f"{addressable + 1}); {batch} requests of {stated_context} tokens at {layers} layers need more, and run so "
                 f"its kernel made an illegal memory access, so it is timed at {context} tokens of context, the most it "
                 f"can address: {100.0 * context / stated_context:.1f} % of the cache bytes, the same weights"),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"],
                     "bytes_per_step": int(step_bytes)},
        "clocks": clocks,
        "e2e": {"value": round(produced / elapsed, 2), "unit": "tokens/s", "ms_per_step": round(1000.0 * elapsed / steps, 3),
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "note": "wall clock around the reference's own EngineCore.step, which uploads its step inputs and reads "
                        "the sampled tokens back every step"},
        "reference_prefill_seconds": round(prefill_seconds, 2),
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=32)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--shape", default="llama31_8b", choices=sorted(SHAPES),
                        help="layer sizes of the model; the default is the headline configuration")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both are reported)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=None)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--skip-points", action="store_true", help="only the headline decode number")
    parser.add_argument("--check", action=argparse.BooleanOptionalAction, default=True,
                        help="before timing, compare logits of the model to be timed with the plain implementation")
    parser.add_argument("--only-prefill", action="store_true",
                        help="time the 2,048-token prefill alone and print its line (for profiling)")
    parser.add_argument("--serve", action="store_true",
                        help="continuous batching instead: 64 requests of 128-4,096 random prompt tokens, "
                             "512 tokens a step, 128 generated tokens each, through LLMEngine.generate")
    args = parser.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine is single-GPU by design, --gpus {args.gpus} is not run")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    import kvcore_b200.kernels as K

    shape, label, shape_context, side_batches = SHAPES[args.shape]
    args.layers = args.layers or shape["num_hidden_layers"]
    args.context = args.context or shape_context
    peaks = measured_peaks()
    numbers = model_numbers(shape, args.layers)
    max_batch = args.batch if args.skip_points else max(max(side_batches), args.batch)
    prefill_steps = -(-max(args.context, PREFILL_TOKENS) // PREFILL_TOKENS)
    margin = args.steps + args.warmup + 8 + args.batch * prefill_steps  # e2e: early requests decode during prefill
    max_len = max(args.context, PREFILL_TOKENS) + margin
    pages = max_batch * (-(-max_len // BLOCK_SIZE)) + 1
    if args.serve:
        import kvcore_b200.kernels as K

        result = time_serving(shape, args.layers, 64, 128, 4096, 512, 128)
        status = K.read_status()
        if status:
            raise RuntimeError(f"a kernel reported status {status} during the measurement: the numbers are void")
        print(json.dumps({"metric": f"continuous batching, {label.replace('-', ' ')}, bf16", "impl": "ours",
                          "layers": args.layers, "layers_of_config": shape["num_hidden_layers"], **result}))
        return 0
    config, runner = build_runner(shape, args.layers, max_batch, max_len, pages, max(PREFILL_TOKENS, max_batch))

    if args.only_prefill:
        ms_prefill = time_prefill(runner, PREFILL_TOKENS, repeats=max(1, args.steps), warmup=2)
        print(json.dumps({"prefill_ms": round(ms_prefill, 3), "layers": args.layers,
                          "tokens_per_s": round(PREFILL_TOKENS * 1000.0 / ms_prefill, 1)}))
        return 0
    checked = {"logits_checked": False}
    if args.check:
        # the check reads the weights back and evaluates them in 32-bit beside the model: about three
        # times the weights' bytes on top of what is held already
        free_bytes, _ = torch.cuda.mem_get_info()
        needed = 3 * runner.model.weight_bytes() + (4 << 30)
        if free_bytes >= needed:
            checked = check_logits(runner, shape, args.layers)
        else:
            checked["logits_check_skipped"] = (f"needs {needed / 2**30:.0f} GiB of free device memory for the plain "
                                               f"implementation's copy of the weights, {free_bytes / 2**30:.0f} GiB are free")
    sampler = ClockSampler()
    sampler.start()
    launches_before = K.api.launch_count
    ms_step = time_decode(runner, args.batch, args.context, args.steps, args.warmup)
    launches = (K.api.launch_count - launches_before) * args.steps // (args.steps + args.warmup)
    points = {}
    point_details = {}
    prefill = None
    e2e = None

    def point(name: str, batch: int, context: int) -> None:
        ms = time_decode(runner, batch, context, args.steps, args.warmup)
        step_bytes = 2.0 * numbers["streamed_params"] + batch * context * numbers["kv_bytes_per_token"]
        gbs = step_bytes / (ms * 1e-3) / 1e9
        points[name] = round(batch * 1000.0 / ms, 2)
        point_details[name] = {"batch": batch, "context": context, "ms_per_step": round(ms, 4),
                               "bytes_per_step": int(step_bytes), "achieved_gbs": round(gbs, 1),
                               "frac": round(gbs / peaks["hbm_gbs"], 4)}

    if not args.skip_points:
        for batch in side_batches:
            point(f"decode_b{batch}", batch, args.context)
        # the decode workload as the baseline configuration states it: prompts of 1,024 tokens
        for batch in (side_batches[0], args.batch, side_batches[1]):
            point(f"decode_b{batch}_ctx1024", batch, 1024)
        ms_prefill = time_prefill(runner, PREFILL_TOKENS, repeats=3, warmup=2)
        t, h, d = PREFILL_TOKENS, numbers["heads"], numbers["head_dim"]
        flops = 2.0 * t * (args.layers * (numbers["layer_params"] - 2 * numbers["hidden"])) \
            + args.layers * 4.0 * h * d * (t * (t + 1) / 2) + 2.0 * numbers["hidden"] * numbers["vocab"]
        prefill = {"value": round(t * 1000.0 / ms_prefill, 1), "tokens": t, "ms": round(ms_prefill, 3),
                   "frac": round(flops / (ms_prefill * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                   "tflops": round(flops / (ms_prefill * 1e-3) / 1e12, 1), "peak_tflops": peaks["bf16_tflops"],
                   "of": peaks["source"]}
        e2e = time_e2e(config, runner, args.batch, args.context, args.steps, args.warmup)
        e2e["value"] = round(e2e["value"], 2)
        e2e["ms_per_step"] = round(e2e["ms_per_step"], 3)
    clocks = sampler.stop()
    status = K.read_status()
    if status:
        raise RuntimeError(f"a kernel reported status {status} during the measurement: the numbers are void")

    step_bytes = 2.0 * numbers["streamed_params"] + args.batch * args.context * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    value = args.batch * 1000.0 / ms_step
    line = {
        "metric": f"decode tokens/s, {label.replace('-', ' ')}, batch {args.batch}, bf16",
        "value": round(value, 2),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, seeded uniform-random token ids, random cache contents",
        "impl": "ours",
        "config": {
            "model": label, "layers": args.layers, "layers_of_config": shape["num_hidden_layers"],
            "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
            "kv_heads": shape["num_key_value_heads"], "head_dim": shape["head_dim"],
            "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
            "tied_embeddings": shape["tie_word_embeddings"], "global_batch": args.batch, "seq_len": args.context, "context_len": args.context,
            "block_size": BLOCK_SIZE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "l2": f"weights of {2e-9 * numbers['streamed_params']:.0f} GB stream every step: inputs larger than L2",
        },
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"],
                     "bytes_per_step": int(step_bytes)},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if prefill is not None:
        line["prefill"] = prefill
    if e2e is not None:
        line["e2e"] = e2e
    if points:
        line["points"] = points
        line["point_details"] = point_details
    line.update(checked)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
