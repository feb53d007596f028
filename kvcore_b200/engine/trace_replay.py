"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it asks the model
runner that generation uses for its model, cache manager, cache storage and step function and
calls ``StepFunction.step`` once per input line.  Input (standard input), one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted it writes ``<out>/<step>.f32``: little-endian 32-bit
floats ``[wanted, vocab]`` in the order of the entries and of each ``want``.  After every
step it prints ``done <step>``.  ``--max-tokens`` sizes the page pool, so pages of ended
requests are used again by later ones.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from .. import kernels as K
from ..cache.kv_manager import KVManager
from ..config.engine_config import CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SchedulerConfig
from .runner import ModelRunner
from .step import StepEntry, StepFunction


def build_replay(model_dir: str, dtype: str, max_tokens: int, *, page_size: int = 16,
                 max_live: int = 8, device: str = "cuda:0", fill_freed_pages: str | None = None):
    """The model with a cache pool for ``max_tokens`` tokens, wired by the model runner as for
    generation; returns (step function, kv manager)."""
    if max_tokens <= 0:
        raise ValueError(f"--max-tokens must be positive, got {max_tokens}")
    pages = -(-max_tokens // page_size) + 1  # + the null page
    config = KVCoreConfig(
        model_config=ModelConfig(model=model_dir, dtype=dtype, max_model_len=max_tokens),
        cache_config=CacheConfig(block_size=page_size, num_gpu_blocks=pages,
                                 debug_fill_freed_pages=fill_freed_pages),
        scheduler_config=SchedulerConfig(max_num_seqs=max_live, max_num_scheduled_tokens=max_tokens),
        device_config=DeviceConfig(device=device),
    )
    runner = ModelRunner(config)
    return runner.step_function, runner.kv_manager


def replay_stream(step_function: StepFunction, kv: KVManager, lines, out_dir: Path, report) -> int:
    out_dir.mkdir(parents=True, exist_ok=True)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_id = record["step"]
        entries = []
        for item in record.get("entries", []):
            request_id = str(item["id"])
            tokens = [int(t) for t in item["tokens"]]
            want = [int(w) for w in item.get("want", [])]
            if not kv.allocate_slots(request_id, len(tokens)):
                raise RuntimeError(
                    f"step {step_id}: no pages for {len(tokens)} more tokens of request {request_id!r} "
                    f"(free pages per group: {kv.num_free_pages()}); raise --max-tokens"
                )
            entries.append(StepEntry(request_id, tokens, want))
        if entries:
            logits = step_function.step(entries)
            if logits is not None:
                data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
                K.raise_on_status()      # the step has finished: nothing its kernels reported goes unseen
                data.tofile(out_dir / f"{step_id}.f32")
        for request_id in record.get("end", []):
            kv.free(str(request_id))
        report(f"done {step_id}")
    return 0


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="tokens the cache pool is made for")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--fill-freed-pages", choices=["zero", "poison"], default=None,
                        help="debugging aid: overwrite pages that nobody holds any more before the next step")
    args = parser.parse_args(argv)

    K.ensure_built(verbose=True)
    step_function, kv = build_replay(
        args.model, args.dtype, args.max_tokens, page_size=args.block_size, device=args.device,
        fill_freed_pages=args.fill_freed_pages,
    )

    def report(text: str) -> None:
        sys.stdout.write(text + "\n")
        sys.stdout.flush()

    return replay_stream(step_function, kv, sys.stdin, Path(args.out), report)


if __name__ == "__main__":
    raise SystemExit(main())
