"""The path a kernel takes when one of its bounded waits runs out, exercised once by construction:
the streaming product is told (through an entry point that exists for this test) that one block shall
never ask for the copies of one of its stages, and to stop waiting after a few thousand polls.
Whoever waits for those copies, and the owners of the weight tiles that block shares, give up within
milliseconds, set the status bit and return; nothing faults, nothing waits without a limit.  The host
must then report the problem, put the hand-over scratch back into its state between launches, and the
next call must be right again."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _arm(K, block, stage, polls=4000):
    lib = K.api._lib
    lib.kvb_gemm_stream_test_give_up.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_uint]
    lib.kvb_gemm_stream_test_give_up.restype = None
    lib.kvb_gemm_stream_test_give_up(block, stage, polls)


def _scratch_is_clean(K) -> bool:
    scratch = K.api._stream_scratch[torch.device(DEV).index or 0]
    marker = int(K.api._lib.kvb_gemm_stream_scratch_marker())
    marker = marker - (1 << 32) if marker >= (1 << 31) else marker
    return bool((scratch.view(torch.int32) == marker).all())


def test_a_wait_that_runs_out_is_reported_and_leaves_the_library_usable():
    import kvcore_b200.kernels as K

    K.require_device(DEV)
    generator = torch.Generator().manual_seed(0)
    # 40 tiles x 5 stages = 200 stages dealt to the GPU's blocks: tiles are shared between neighbours
    x = (torch.randn(6, 1280, generator=generator) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2560, 1280, generator=generator) * 0.05).to(torch.bfloat16).to(DEV)
    want = x.float() @ w.float().T
    assert K.read_status() == 0
    good = K.linear_stream(x, w)
    torch.testing.assert_close(good.float(), want, rtol=2e-2, atol=2e-2)
    assert _scratch_is_clean(K)

    _arm(K, block=3, stage=0)
    broken = K.linear_stream(x, w)
    torch.cuda.synchronize()
    assert K.peek_status() & 4
    with pytest.raises(K.KernelError, match="bounded wait"):
        K.raise_on_status()
    assert K.peek_status() == 0 and _scratch_is_clean(K)
    assert not torch.allclose(broken.float(), want, rtol=2e-2, atol=2e-2)   # the tiles of that block never left

    again = K.linear_stream(x, w)                       # the hook was for one launch: this one is ordinary
    torch.testing.assert_close(again.float(), want, rtol=2e-2, atol=2e-2)
    assert torch.equal(again, good) and K.read_status() == 0


def test_a_step_whose_kernel_gave_up_raises_and_the_next_request_is_right(tmp_path):
    """The same through the step function: the replay raises after the step whose kernel gave up; a new
    request run afterwards on the same engine gets the plain implementation's logits."""
    import json

    import numpy as np

    import plain_llama
    import replay_cases as rc
    import kvcore_b200.kernels as K
    from kvcore_b200.engine.trace_replay import build_replay, replay_stream

    config = rc.TINY_CONFIGS["D"]
    folder = rc.write_model(tmp_path / "m", config, 3, "bfloat16")
    weights = plain_llama.load_weights(folder)
    vocab = config["vocab_size"]
    step_function, kv = build_replay(str(folder), "bfloat16", 512)
    first = rc.random_tokens(vocab, 40, 1)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": first[:39], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": first[39:], "want": [0]}], "end": ["a"]}]
    replay_stream(step_function, kv, [json.dumps(steps[0])], tmp_path / "o", lambda _: None)
    _arm(K, block=0, stage=0)       # the first streaming product of the decode step
    with pytest.raises(K.KernelError, match="bounded wait"):
        replay_stream(step_function, kv, [json.dumps(steps[1])], tmp_path / "o", lambda _: None)
    kv.free("a")
    assert K.peek_status() == 0
    second = rc.random_tokens(vocab, 70, 2)
    trace = rc.trace_decode_tail({"b": second}, tail=8)
    rc.run_on(step_function, kv, trace, tmp_path / "p")
    rows = rc.collect(trace, tmp_path / "p", vocab)
    reference = plain_llama.forward_logits(config, weights, second).numpy()
    for (_, pos), row in rows.items():
        assert np.abs(row - reference[pos]).max() <= 2e-2 * np.abs(reference).max()
    assert K.read_status() == 0
