"""Random weights are the same numbers wherever they are computed."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_random_weights_are_bit_equal_on_the_cpu_and_on_the_gpu():
    from kernel_rush_kawk_b200.parts import TensorSpec
    from kernel_rush_kawk_b200.weights.random_init import random_tensor, standard_normals

    a = standard_normals(300_001, 123456789, "cpu")
    b = standard_normals(300_001, 123456789, "cuda").cpu()
    assert torch.equal(a, b), "float64 draws differ between the devices"
    assert abs(a.mean().item()) < 0.01 and abs(a.std().item() - 1.0) < 0.01
    for name, spec in (("model.embed_tokens.weight", TensorSpec((301, 80), "table")),
                       ("model.layers.3.input_layernorm.weight", TensorSpec((2560,), "gain")),
                       ("model.layers.0.mlp.down_proj.weight", TensorSpec((96, 1001), "matrix"))):
        cpu = random_tensor(name, spec, 7, 0.02, "cpu")
        gpu = random_tensor(name, spec, 7, 0.02, "cuda").cpu()
        assert cpu.dtype == torch.bfloat16 and torch.equal(cpu, gpu), name


def test_an_engine_from_random_weights_equals_one_from_the_written_folder(tmp_path):
    """``Engine.from_random`` draws on the device, ``write_model_folder`` on the CPU: one model."""
    from kernel_rush_kawk_b200 import Engine, Qwen3Config, StepEntry, write_model_folder

    cfg = Qwen3Config.preset("tiny_b")
    folder = write_model_folder(tmp_path / "m", cfg, 19, std=0.05)
    prompt = list(range(3, 40))
    outs = []
    for engine in (Engine(folder, dtype="float32", max_tokens=256, max_slots=2),
                   Engine.from_random(cfg, seed=19, std=0.05, dtype="float32", max_tokens=256, max_slots=2)):
        slot = engine.cache.alloc()
        outs.append(engine.step([StepEntry(slot, prompt, [len(prompt) - 1])]))
    assert torch.equal(outs[0], outs[1])
