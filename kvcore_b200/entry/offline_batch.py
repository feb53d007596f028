"""Offline batch generation from the command line.

Options keep the names and meanings of the reference's script
(scripts/run_llm_engine_offline_batch.py:127-174): ``--model``, ``--device``, ``--block-size``,
``--max-model-len``, ``--max-num-seqs``, ``--max-num-scheduled-tokens``,
``--max-num-partial-prefills``, ``--max-long-partial-prefills``,
``--long-prefill-token-threshold``, ``--log-level``, ``--log-file``; its output has the same
sections (run metadata, per-request outputs, timing summary).  ``--attn-backend``,
``--revision``, ``--trust-remote-code`` and ``--local-files-only`` are accepted and have
nothing to select here (one CUDA code path, local folders only).  Added: the compute dtype,
seeded random weights, cache sizing, and requests given as token ids (a JSON file, or seeded
random prompts) instead of the reference's built-in chat messages.

    python -m kvcore_b200.entry.offline_batch --model DIR --random-prompts 4:64 --max-tokens 32
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from datetime import datetime
from pathlib import Path

from ..config import CacheConfig, DeviceConfig, KVCoreConfig, LoadConfig, ModelConfig, SchedulerConfig
from ..sampling import SamplingParams
from ..utils.log import configure_logging


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Run offline batch generation through LLMEngine.")
    parser.add_argument("--model", required=True, help="folder with config.json and safetensors weights")
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--dtype", default=None, choices=["bfloat16", "bf16", "float32", "fp32"])
    parser.add_argument("--attn-backend", default=None, help="accepted for compatibility; one CUDA path exists")
    parser.add_argument("--revision", default=None, help="accepted for compatibility; unused")
    parser.add_argument("--trust-remote-code", action="store_true", help="accepted for compatibility; unused")
    parser.add_argument("--local-files-only", action=argparse.BooleanOptionalAction, default=True)
    parser.add_argument("--random-weights", action="store_true", help="ignore weight files; draw N(0, 0.02)")
    parser.add_argument("--seed", type=int, default=0, help="seed of --random-weights")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-gpu-blocks", type=int, default=None)
    parser.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    parser.add_argument("--enable-prefix-caching", action="store_true",
                        help="requests whose prompts begin with the same full pages share them")
    parser.add_argument("--max-model-len", type=int, default=None)
    parser.add_argument("--max-num-seqs", type=int, default=1024)
    parser.add_argument("--max-num-scheduled-tokens", type=int, default=1024)
    parser.add_argument("--max-num-partial-prefills", type=int, default=128)
    parser.add_argument("--max-long-partial-prefills", type=int, default=128)
    parser.add_argument("--long-prefill-token-threshold", type=int, default=0)
    parser.add_argument("--prompt-tokens-file", default=None,
                        help='JSON list of {"request_id", "prompt_token_ids" | "messages", "sampling_params"}')
    parser.add_argument("--random-prompts", default=None, metavar="N:LEN",
                        help="N seeded random prompts of LEN token ids")
    parser.add_argument("--max-tokens", type=int, default=32)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=None)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--sample-seed", type=int, default=None)
    parser.add_argument("--log-level", default="INFO")
    parser.add_argument("--log-file", default=None, help="also write the terminal output to this file")
    return parser.parse_args(argv)


def build_config(args: argparse.Namespace) -> KVCoreConfig:
    return KVCoreConfig(
        model_config=ModelConfig(model=str(Path(args.model).expanduser()), dtype=args.dtype,
                                 max_model_len=args.max_model_len),
        load_config=LoadConfig(random_weights=args.random_weights, seed=args.seed),
        cache_config=CacheConfig(block_size=args.block_size, num_gpu_blocks=args.num_gpu_blocks,
                                 gpu_memory_utilization=args.gpu_memory_utilization,
                                 enable_prefix_caching=args.enable_prefix_caching),
        scheduler_config=SchedulerConfig(
            max_num_seqs=args.max_num_seqs,
            max_num_scheduled_tokens=args.max_num_scheduled_tokens,
            max_num_partial_prefills=args.max_num_partial_prefills,
            max_long_partial_prefills=args.max_long_partial_prefills,
            long_prefill_token_threshold=args.long_prefill_token_threshold,
        ),
        device_config=DeviceConfig(device=args.device),
    )


def build_requests(args: argparse.Namespace, vocab_size: int) -> list[dict]:
    default = dict(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                   top_p=args.top_p, seed=args.sample_seed)
    if args.prompt_tokens_file:
        with open(args.prompt_tokens_file, "r", encoding="utf-8") as handle:
            specs = json.load(handle)
        requests = []
        for index, spec in enumerate(specs):
            params = dict(default)
            params.update(spec.get("sampling_params", {}))
            requests.append(dict(request_id=str(spec.get("request_id", f"offline-{index:03d}")),
                                 prompt_token_ids=spec.get("prompt_token_ids"),
                                 messages=spec.get("messages"),
                                 sampling_params=SamplingParams.from_mapping(params)))
        return requests
    count, length = (int(x) for x in (args.random_prompts or "4:32").split(":"))
    import torch

    generator = torch.Generator().manual_seed(args.seed)
    return [dict(request_id=f"offline-{index:03d}",
                 prompt_token_ids=torch.randint(0, vocab_size, (length,), generator=generator).tolist(),
                 sampling_params=SamplingParams(**default))
            for index in range(count)]


class _Tee:
    def __init__(self, *streams):
        self.streams = streams

    def write(self, data):
        for stream in self.streams:
            stream.write(data)
        return len(data)

    def flush(self):
        for stream in self.streams:
            stream.flush()


def main(argv=None) -> int:
    program_start = time.perf_counter()
    args = parse_args(argv)
    log_handle = None
    stdout = sys.stdout
    if args.log_file:
        path = Path(args.log_file).expanduser()
        path.parent.mkdir(parents=True, exist_ok=True)
        log_handle = path.open("w", encoding="utf-8")
        sys.stdout = _Tee(stdout, log_handle)
    try:
        configure_logging(args.log_level, force=True)
        from ..engine.llm_engine import LLMEngine

        print("=== Run Metadata ===")
        print(f"start_time={datetime.now().astimezone().isoformat(timespec='seconds')}")
        print(f"log_file={args.log_file}")
        print(f"model={Path(args.model).expanduser()}")
        print(f"device={args.device}")
        print(f"max_num_seqs={args.max_num_seqs}")
        print(f"max_num_scheduled_tokens={args.max_num_scheduled_tokens}")
        engine_start = time.perf_counter()
        engine = LLMEngine(build_config(args))
        engine_elapsed = time.perf_counter() - engine_start
        print(f"engine_init_sec={engine_elapsed:.3f}")
        runner = engine.engine_core.model_runner
        print(f"dtype={runner.dtype} num_gpu_blocks={[p.num_pages for p in runner.kv_manager.pools]}")
        requests = build_requests(args, runner.model.spec.vocab_size)
        print("=== Offline Requests ===")
        for request in requests:
            ids = request.get("prompt_token_ids")
            params = request["sampling_params"]
            print(f"{request['request_id']}: prompt_tokens={len(ids) if ids is not None else 'messages'} "
                  f"max_tokens={params.max_tokens} temperature={params.temperature}")
        generate_start = time.perf_counter()
        outputs = engine.generate(requests)
        generate_elapsed = time.perf_counter() - generate_start
        print("\n=== Detokenized Outputs ===")
        produced = 0
        for output in outputs:
            produced += len(output.output_token_ids)
            print(f"\n[{output.request_id}] finish_reason={output.finish_reason}")
            print(f"token_ids={output.output_token_ids}")
            print(output.output_text)
        print("\n=== Timing Summary ===")
        print(f"end_time={datetime.now().astimezone().isoformat(timespec='seconds')}")
        print(f"num_requests={len(requests)}")
        print(f"output_tokens={produced}")
        print(f"engine_init_sec={engine_elapsed:.3f}")
        print(f"generate_sec={generate_elapsed:.3f}")
        print(f"total_elapsed_sec={time.perf_counter() - program_start:.3f}")
        return 0
    finally:
        sys.stdout = stdout
        if log_handle is not None:
            log_handle.close()


if __name__ == "__main__":
    raise SystemExit(main())
