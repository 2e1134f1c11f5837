"""Writes tests/golden/reference_logits.safetensors: logits of the reference's own forward
passes (``Plan.prefill`` and ``Plan.decode``, engine/model.py:284-318 of
willzeng274/kernel-rush-kawk) on a random model, computed on a B200.

    python tests/golden/make_reference_logits.py /path/to/kernel-rush-kawk [output file]

It needs a CUDA device and Triton (the reference's kernels are Triton kernels). The
model is the one ``reference_model_folder`` below writes: two layers of the Qwen3-4B
layer sizes with a small vocabulary, seeded, q/k gains doubled so that attention is
sharp. Two prompts of equal length (the reference's contract) are prefilled, then
four tokens are decoded greedily; the file holds the prompts, the reference's chosen
tokens and its bfloat16 logits at each of the five steps.

The tests that read the file are ``tests/test_reference_logits.py``: they rebuild the
same folder from the same seed, and compare the plain implementation (on the CPU) and
the engine (on the GPU) with these logits.
"""

import os
import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).parent / "reference_logits.safetensors"
CONFIG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 2560, "intermediate_size": 9728,
    "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 4096,
    "rms_norm_eps": 1e-6, "rope_theta": 5000000.0, "tie_word_embeddings": True, "max_position_embeddings": 4096,
}
SEED, PROMPT_SEED = 4242, 77
BATCH, PROMPT_LEN, DECODE_STEPS = 2, 200, 4


def reference_model_folder(folder) -> Path:
    from kernel_rush_kawk_b200 import Qwen3Config, write_model_folder

    cfg = Qwen3Config.from_dict(CONFIG)
    scale = {f"model.layers.{i}.self_attn.q_norm.weight": 2.0 for i in range(cfg.num_hidden_layers)}
    return write_model_folder(folder, cfg, SEED, std=0.02, scale=scale)


def prompts() -> list:
    g = torch.Generator().manual_seed(PROMPT_SEED)
    return torch.randint(0, CONFIG["vocab_size"], (BATCH, PROMPT_LEN), generator=g).tolist()


def main(reference_root: str, target=GOLDEN) -> None:
    os.environ.setdefault("ENGINE_SELF_CHECK", "0")
    sys.path.insert(0, str(Path(reference_root) / "engine"))
    import budget as ref_budget
    import model as ref_model  # the reference's engine/model.py

    torch.backends.cuda.matmul.allow_tf32 = False
    ref_budget.start(120.0)
    ids = prompts()
    out = {"prompts": torch.tensor(ids, dtype=torch.int32)}
    with tempfile.TemporaryDirectory() as tmp:
        folder = reference_model_folder(Path(tmp) / "model")
        m = ref_model.Model(folder)
        plan = ref_model.Plan(m, BATCH, PROMPT_LEN, DECODE_STEPS + 1)
        plan.ids.copy_(torch.tensor(ids, dtype=torch.int64))
        logits = plan.prefill()
        steps, tokens = [logits.clone()], []
        for _ in range(DECODE_STEPS):
            tok = steps[-1].argmax(dim=-1)
            tokens.append(tok.clone())
            plan.tok.copy_(tok)
            steps.append(plan.decode().clone())
        torch.cuda.synchronize()
    out["logits"] = torch.stack(steps).to(torch.bfloat16).cpu()          # [steps, batch, vocab]
    out["tokens"] = torch.stack(tokens).to(torch.int32).cpu()              # [steps - 1, batch]: fed at steps 1..
    from safetensors.torch import save_file

    save_file({k: t.contiguous() for k, t in out.items()}, str(target))
    print("wrote", target, {k: tuple(t.shape) for k, t in out.items()}, "max|logit|", out["logits"].float().abs().max().item())


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        sys.exit("usage: make_reference_logits.py <checkout of willzeng274/kernel-rush-kawk> [output file]")
    main(*sys.argv[1:])
