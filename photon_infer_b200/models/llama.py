"""The Llama decoder as a ``ModelSpec``: which parts each layer has, from the keys of
``config.json``.  Layer order and formulas: src/arch/llama_model.cpp:186-272 and
src/arch/transformer_block.cpp:199-296.  Tensor names are those of Hugging Face Llama
weight files; the reference's ``wq/wk/wv/wo``, ``w1/w3/w2``, ``attn_norm/ffn_norm``
(src/io/checkpoint.cpp:120-314) are ``self_attn.{q,k,v,o}_proj``,
``mlp.{gate,up,down}_proj``, ``input_layernorm/post_attention_layernorm``.
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..config.registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = lambda prefix: PartSpec("rms_norm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix)
    layers = []
    for i in range(cfg.num_hidden_layers):
        kind = cfg.layer_types[i]
        mixer_params = {
            "hidden_size": cfg.hidden_size, "n_q_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "position_encoding": "rope",
            "window": cfg.sliding_window if kind == "sliding_attention" else None,
        }
        layers.append(LayerSpec(
            block=PartSpec("pre_norm", {}),
            norm1=norm("input_layernorm."),
            mixer=PartSpec(kind, mixer_params, "self_attn."),
            norm2=norm("post_attention_layernorm."),
            feed_forward=PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                             "intermediate_size": cfg.intermediate_size}, "mlp."),
            prefix=f"model.layers.{i}.",
        ))
    rope = PartSpec("rotary", {
        "head_dim": cfg.head_dim, "theta": cfg.rope_theta,
        "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None,
        "interleaved": cfg.rope_interleaved,
    })
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        final_norm=norm("model.norm."),
        position_encodings={"rope": rope},
        layers=layers,
        run=[RunEntry(i) for i in range(cfg.num_hidden_layers)],
        eos_token_ids=tuple(cfg.eos_token_ids),
        bos_token_id=cfg.bos_token_id,
        # older exports store the rotation frequencies as a buffer of every layer; they follow from rope_theta
        ignored_tensors=("*.rotary_emb.inv_freq",),
    )


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec, replace=True)
