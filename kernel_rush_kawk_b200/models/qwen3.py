"""The Qwen3 dense decoder as a plan.

Tensor names are the checkpoint's own (engine/model.py:102-125 of
willzeng274/kernel-rush-kawk): ``model.embed_tokens.weight``, ``lm_head.weight``
(absent when tied: the head reads the embedding table, :103-107),
``model.norm.weight`` and, per layer, ``input_layernorm``,
``post_attention_layernorm``, ``self_attn.{q,k,v,o}_proj``,
``self_attn.{q,k}_norm`` and ``mlp.{gate,up,down}_proj``. The layer order is
x += Attn(norm(x)); x += MLP(norm(x)), one final norm, then the head
(engine/model.py:284-303).
"""

from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    H = cfg.hidden_size
    embed_name = "model.embed_tokens.weight"
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = lambda key: PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, {"weight": p + key + ".weight"})
        mixer = PartSpec(
            "gqa_attention",
            {"hidden": H, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
             "head_dim": cfg.head_dim, "eps": cfg.rms_norm_eps, "qk_norm": True, "window": cfg.window_of(i)},
            {k: f"{p}self_attn.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")},
        )
        ffn = PartSpec(
            "swiglu", {"hidden": H, "intermediate": cfg.intermediate_size},
            {k: f"{p}mlp.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")},
        )
        layers.append(LayerSpec("prenorm", norm("input_layernorm"), mixer, norm("post_attention_layernorm"), ffn))
    head_name = embed_name if cfg.tie_word_embeddings else "lm_head.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=H,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab": cfg.vocab_size, "hidden": H}, {"table": embed_name}),
        position=PartSpec("rope", {"theta": cfg.rope_theta, "dim": cfg.head_dim}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("output_head", {"vocab": cfg.vocab_size, "hidden": H}, {"weight": head_name}),
        max_positions=cfg.max_position_embeddings,
        stop_token_ids=cfg.eos_token_ids,
        duplicates={"lm_head.weight": embed_name} if cfg.tie_word_embeddings else {},
    )


register_architecture(Qwen3Config.architecture, Qwen3Config, qwen3_plan)
