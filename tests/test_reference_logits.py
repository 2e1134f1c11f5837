"""The plain implementation and the engine against logits of the reference's own forward.

``tests/golden/reference_logits.safetensors`` was written on a B200 by
``tests/golden/make_reference_logits.py``: the unmodified reference's ``Plan.prefill`` and
``Plan.decode`` (engine/model.py:284-318 of willzeng274/kernel-rush-kawk) on a seeded
two-layer model of the Qwen3-4B layer sizes, two prompts of 200 tokens, four greedy
decode steps. The tests rebuild the same folder from the same seed. The reference's
logits are bfloat16, so the comparison uses the whole-model bfloat16 tolerance.
"""

import importlib.util
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from helpers import assert_close

GOLDEN_DIR = Path(__file__).parent / "golden"
GOLDEN = GOLDEN_DIR / "reference_logits.safetensors"


def _maker():
    spec = importlib.util.spec_from_file_location("make_reference_logits", GOLDEN_DIR / "make_reference_logits.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def golden():
    from safetensors.torch import load_file

    return load_file(str(GOLDEN))


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    return _maker().reference_model_folder(tmp_path_factory.mktemp("reference_model") / "model")


def _sequences(golden):
    """For each step, each request's whole token sequence up to and including that step's input."""
    prompts = golden["prompts"].tolist()
    fed = golden["tokens"].tolist()
    steps = golden["logits"].shape[0]
    return [[prompts[b] + [fed[s][b] for s in range(step)] for b in range(len(prompts))] for step in range(steps)]


def test_golden_file_is_the_one_the_script_describes(golden):
    mk = _maker()
    assert golden["prompts"].tolist() == mk.prompts()
    assert tuple(golden["logits"].shape) == (mk.DECODE_STEPS + 1, mk.BATCH, mk.CONFIG["vocab_size"])
    # the reference fed its own greedy choice at every step
    assert torch.equal(golden["logits"][:-1].float().argmax(dim=-1).to(torch.int32), golden["tokens"])


def test_plain_implementation_matches_the_reference_forward(golden, folder):
    cfg, w = plain.read_folder(folder)
    ref = golden["logits"].float()
    for step, seqs in enumerate(_sequences(golden)):
        if step not in (0, 1, ref.shape[0] - 1):  # the prompt, the first decoded token, the last one
            continue
        for b, ids in enumerate(seqs):
            got = plain.forward_logits(cfg, w, ids, torch.float32, torch.bfloat16)[-1]
            assert_close(got[None], ref[step, b][None], "bfloat16", f"plain vs reference, step {step}, request {b}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_engine_matches_the_reference_forward(golden, folder, dtype):
    """Prefill of both prompts in one step, then one token each, as the reference ran it. The 32-bit
    path differs from the reference's bfloat16 arithmetic by rounding only, within the same tolerance."""
    from kernel_rush_kawk_b200 import Engine, StepEntry

    ref = golden["logits"].float()
    prompts = golden["prompts"].tolist()
    fed = golden["tokens"].tolist()
    engine = Engine(folder, dtype=dtype, max_tokens=2 * 256, max_slots=2)
    slots = [engine.cache.alloc() for _ in prompts]
    logits = engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    assert_close(logits, ref[0], "bfloat16", f"engine ({dtype}) vs reference, prefill")
    for step in range(1, ref.shape[0]):
        logits = engine.step([StepEntry(s, [fed[step - 1][b]], [0]) for b, s in enumerate(slots)])
        assert_close(logits, ref[step], "bfloat16", f"engine ({dtype}) vs reference, decode step {step}")
    engine.ops.check()
    for s in slots:
        engine.cache.free(s)
