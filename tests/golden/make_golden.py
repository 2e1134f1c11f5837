"""Writes tests/golden/golden_tiny.safetensors: outputs of the reference's own code on
a tiny random model, for the parts of it that run on a CPU.

    python tests/golden/make_golden.py /path/to/kernel-rush-kawk

What runs there without a GPU: ``Config.load``, ``Model`` (weight reading by name,
q/k/v and gate/up concatenation, tied head) with device="cpu", ``rope_tables``
(engine/model.py:25-134) and ``reference_attention`` (engine/kernels/attention.py:
255-276). Its forward passes need CUDA graphs and Triton kernels on a GPU, so logits
cannot be anchored this way; ``tests/plain_qwen3.py`` rests on the formulas for those.
The test that reads the file is ``tests/test_plain.py::test_golden_*``.
"""

import sys
import tempfile
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "engine"))
    import model as ref_model  # the reference's engine/model.py
    from kernels.attention import reference_attention

    from helpers import tiny_config
    from kernel_rush_kawk_b200 import write_model_folder

    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, seed in (("tiny_a", 101), ("tiny_b", 202)):
            folder = write_model_folder(Path(tmp) / name, tiny_config(name), seed)
            m = ref_model.Model(folder, device="cpu", max_pos=96)
            out[f"{name}.cos"] = m.cos.clone()
            out[f"{name}.sin"] = m.sin.clone()
            if name == "tiny_a":  # fused layouts: q rows, then k, then v; gate rows, then up
                out[f"{name}.layer0.wqkv"] = m.layers[0].wqkv.clone()
                out[f"{name}.layer1.wgu"] = m.layers[1].wgu.clone()
            out[f"{name}.lm_head_is_embed"] = torch.tensor([int(m.lm_head is m.embed)])
            out[f"{name}.scale"] = torch.tensor([m.scale])
    # the reference's attention oracle on a decode-like block: R new rows at pos[b]
    g = torch.Generator().manual_seed(7)
    B, HQ, HKV, D, R, cap = 2, 6, 2, 32, 3, 40
    q = torch.randn((B, HQ, R, D), generator=g)
    k = torch.randn((B, HKV, cap, D), generator=g)
    v = torch.randn((B, HKV, cap, D), generator=g)
    pos = torch.tensor([5, 30], dtype=torch.int32)
    scale = 1.0 / D ** 0.5
    out["attn.q"], out["attn.k"], out["attn.v"], out["attn.pos"] = q, k, v, pos
    out["attn.out"] = reference_attention(q, k, v, pos, R, scale).contiguous()
    from safetensors.torch import save_file

    save_file({k: t.contiguous() for k, t in out.items()}, str(Path(__file__).parent / "golden_tiny.safetensors"))
    print("wrote", len(out), "tensors")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of willzeng274/kernel-rush-kawk>")
    main(sys.argv[1])
