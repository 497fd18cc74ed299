"""The Llama dense decoder as a model description.

Every layer is the same pre-norm block: RMSNorm -> GQA attention with rotary positions ->
RMSNorm -> SwiGLU feed-forward; the layers run once each in order, each with a cache of its
own (src/DotLLM.Models/Architectures/TransformerModel.cs:185-392).  Tensor names are the
HuggingFace ones; the reference resolves the same tensors under their GGUF names
(src/DotLLM.Models/Architectures/TransformerWeights.cs:186-205, 283-367).
"""
from __future__ import annotations

from dataclasses import asdict

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import ModelSpec, PartSpec, ScheduleEntry, pre_norm_layer


def build_llama_spec(cfg: LlamaConfig, norm_gain_init=("ones",)) -> ModelSpec:
    scaling = asdict(cfg.rope_scaling) if cfg.rope_scaling is not None else None
    position = {"kind": "rotary",
                "params": {"rotary_dim": cfg.head_dim, "head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                           "max_positions": cfg.max_position_embeddings, "scaling": scaling}}
    norm_params = {"eps": cfg.rms_norm_eps, "gain_init": tuple(norm_gain_init)}
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(pre_norm_layer(
            mixer=PartSpec("attention", {"n_heads": cfg.num_attention_heads,
                                         "n_kv_heads": cfg.num_key_value_heads,
                                         "head_dim": cfg.head_dim, "window": None,
                                         "position": position}, p + "self_attn."),
            feed_forward=PartSpec("gated_mlp", {"intermediate_size": cfg.intermediate_size,
                                                "activation": cfg.hidden_act}, p + "mlp."),
            mixer_norm=PartSpec("rmsnorm", norm_params, p + "input_layernorm."),
            feed_forward_norm=PartSpec("rmsnorm", norm_params, p + "post_attention_layernorm.")))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size}, "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", norm_params, "model.norm."),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size}, "lm_head."),
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id,
        # src/DotLLM.Models/Architectures/TransformerWeights.cs:213-220: no output matrix, use the embedding's
        shared_weights=(("lm_head.weight", "model.embed_tokens.weight"),) if cfg.tie_word_embeddings else ())


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec, model_types=("llama",))
