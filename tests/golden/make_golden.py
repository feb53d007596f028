"""Writes tests/golden/reference_logits.{json,safetensors}: logits of the reference's own
model code (Baizx98/KVCore, unmodified, imported from a checkout) on three tiny random Llama
configurations, on the CPU in float32: A and B as the baseline states them, and one with biases on
every projection, full multi-head attention and a logit scale, all of which the reference implements
(kvcore/model/models/llama3.py:62-74, kvcore/sample/logits_processor.py:46-54).  tests/test_plain_vs_golden.py checks the plain
implementation (tests/plain_llama.py) against these numbers.

Usage:  python tests/golden/make_golden.py /path/to/KVCore

How the numbers are made.  Weights come from ``kvcore_b200.weights.random_state_dict`` (seeded,
N(0, 0.02), norms = 1) and are loaded through the reference's ``load_weights``.  The
reference's whole stack runs (Scheduler + ModelRunner with the ``torch_paged`` backend): for
every prefix of every sequence a request with ``max_tokens=1`` is scheduled, and the logits
row the runner keeps for sampling is recorded, which gives logits at every position.
Configuration B additionally uses chunked prefill (token budget 6).

One thing is not the reference's: it has no llama3 frequency scaling, so for configuration B
each layer's ``rotary_emb.inv_freq`` buffer is overwritten with the scaled table of
tests/plain_llama.py before running.  Everything else in B (and all of A) is anchored.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))
sys.dont_write_bytecode = True

CONFIGS = {
    "A": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=256, hidden_size=64,
        intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        max_position_embeddings=128, tie_word_embeddings=False, rms_norm_eps=1e-5, rope_theta=10000.0,
        hidden_act="silu",
    ),
    "B": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=512, hidden_size=96,
        intermediate_size=160, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
        head_dim=32, max_position_embeddings=256, tie_word_embeddings=True, rms_norm_eps=1e-6,
        rope_theta=500000.0, hidden_act="silu",
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=64),
    ),
    "BIAS": dict(
        architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=300, hidden_size=80,
        intermediate_size=112, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
        max_position_embeddings=128, tie_word_embeddings=False, rms_norm_eps=1e-5, rope_theta=10000.0,
        hidden_act="silu", attention_bias=True, mlp_bias=True, logit_scale=0.25,
    ),
}
SEEDS = {"A": 0, "B": 1, "BIAS": 2}
LENGTHS = {"A": (7, 13), "B": (5, 19, 40), "BIAS": (11, 30)}
BLOCK = {"A": 16, "B": 8, "BIAS": 4}
BUDGET = {"A": 512, "B": 6, "BIAS": 9}


def state_dict_hash(tensors: dict) -> str:
    digest = hashlib.sha256()
    for name in sorted(tensors):
        digest.update(name.encode())
        digest.update(tensors[name].contiguous().view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def make_tokens(name: str) -> list[list[int]]:
    generator = torch.Generator().manual_seed(100 + SEEDS[name])
    vocab = CONFIGS[name]["vocab_size"]
    return [torch.randint(0, vocab, (n,), generator=generator).tolist() for n in LENGTHS[name]]


def reference_logits(name: str, weights: dict, sequences: list[list[int]]) -> list[torch.Tensor]:
    from transformers.models.llama.configuration_llama import LlamaConfig  # config container only

    from kvcore.config import CacheConfig, DeviceConfig, KVCoreConfig, ModelConfig, SchedulerConfig
    from kvcore.kv.kv_manager import KVManagerConfig
    from kvcore.kv.single_type_kv_manager import KVLayerSpec
    from kvcore.model.model_runner import ModelRunner
    from kvcore.model.models.llama3 import Llama3ForCausalLM
    from kvcore.sched.scheduler import Scheduler
    from kvcore.utils.request import Request
    from kvcore.utils.sampling_params import SamplingParams

    import plain_llama

    raw = CONFIGS[name]
    kwargs = {k: v for k, v in raw.items() if k not in ("architectures", "model_type", "rope_scaling", "rope_theta")}
    hf = LlamaConfig(**kwargs, rope_parameters={"rope_type": "default", "rope_theta": raw["rope_theta"]})
    layers, block = raw["num_hidden_layers"], BLOCK[name]
    head_dim = plain_llama.head_dim_of(raw)
    kv_heads = plain_llama.kv_heads_of(raw)
    max_len = raw["max_position_embeddings"]
    num_blocks = layers * (max_len // block) * 4 + 1
    config = KVCoreConfig(
        model_config=ModelConfig(model="unused", attn_backend="torch_paged", hf_config=hf,
                                 dtype=torch.float32, max_model_len=max_len),
        cache_config=CacheConfig(block_size=block, num_gpu_blocks=num_blocks, profile_kv_cache=False,
                                 enable_caching=False),
        scheduler_config=SchedulerConfig(max_num_seqs=4, max_num_scheduled_tokens=BUDGET[name],
                                         max_num_partial_prefills=4, max_long_partial_prefills=4),
        device_config=DeviceConfig(device="cpu"),
    )
    runner = ModelRunner(config)
    with torch.no_grad():
        model = Llama3ForCausalLM(config).eval()
        model.load_weights(iter(weights.items()))
        if "rope_scaling" in raw:
            table = plain_llama.rope_inv_freq(raw).to(torch.float32)
            for layer in model.model.layers:
                layer.self_attn.rotary_emb.inv_freq.copy_(table)
    runner.model = model
    specs = tuple(KVLayerSpec(layer_idx=i, block_size=block, num_kv_heads=kv_heads, head_size=head_dim,
                              dtype=torch.float32) for i in range(layers))
    kv_config = KVManagerConfig(num_gpu_blocks=num_blocks, max_model_len=max_len, layer_specs=specs,
                                enable_caching=False)
    scheduler = Scheduler(config, kv_config)
    runner.initialize_kv_cache(kv_config)

    out = []
    for seq_index, tokens in enumerate(sequences):
        rows = []
        for end in range(1, len(tokens) + 1):
            request_id = f"{name}-{seq_index}-{end}"
            scheduler.add_request(Request(request_id, tokens[:end], SamplingParams(max_tokens=1, temperature=0.0)))
            row = None
            while scheduler.has_unfinished_requests():
                so = scheduler.schedule()
                with torch.no_grad():
                    result = runner.execute_model(so)
                    state = runner.execute_model_state
                    if state is not None and state.logits is not None and state.logits.numel():
                        row = state.logits[-1].detach().to(torch.float32).clone()
                    if result is None:
                        result = runner.sample_tokens()
                sampled = {r: t[0] for r, t in zip(result.req_ids, result.sampled_token_ids) if t}
                update = scheduler.update_from_outputs(so, sampled)
                runner.remove_requests([f.request_id for f in update.finished_requests])
            rows.append(row)
        out.append(torch.stack(rows))
    return out


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    sys.path.insert(0, sys.argv[1])
    from kvcore_b200.weights import random_state_dict, write_safetensors

    record = {"configs": CONFIGS, "seeds": SEEDS, "block_sizes": BLOCK, "token_budgets": BUDGET,
              "tokens": {}, "weights_sha256": {}, "torch": torch.__version__}
    tensors = {}
    for name in CONFIGS:
        weights = random_state_dict(CONFIGS[name], SEEDS[name], 0.02, "float32")
        sequences = make_tokens(name)
        record["tokens"][name] = sequences
        record["weights_sha256"][name] = state_dict_hash(weights)
        for index, logits in enumerate(reference_logits(name, weights, sequences)):
            tensors[f"{name}/seq{index}"] = logits
            print(name, index, tuple(logits.shape), float(logits.abs().max()))
    write_safetensors(HERE / "reference_logits.safetensors", tensors)
    with (HERE / "reference_logits.json").open("w") as handle:
        json.dump(record, handle, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
