"""Llama 3 dense as a ModelSpec: which parts make a layer and which tensors they
read.  Tensor names: crates/ai-engine-runtime/src/name_map.rs:61-101; layer
structure: crates/ai-engine-runtime/src/arch/model.rs:104-205.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    D, V = cfg.hidden_size, cfg.vocab_size
    rope = PartSpec("rotary", dict(
        rot_dim=cfg.head_dim, theta=cfg.rope_theta,
        scaling=cfg.rope_scaling.to_dict() if cfg.rope_scaling is not None else None))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec("prenorm", {
            "mixer_norm": PartSpec("rmsnorm", dict(size=D, eps=cfg.rms_norm_eps),
                                   dict(weight=p + "input_layernorm.weight")),
            "mixer": PartSpec("gqa_attention", dict(
                hidden_size=D, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, window=0, scale=None,
                position_encoding="rope"),
                dict(q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                     v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight")),
            "ffn_norm": PartSpec("rmsnorm", dict(size=D, eps=cfg.rms_norm_eps),
                                 dict(weight=p + "post_attention_layernorm.weight")),
            "ffn": PartSpec("swiglu", dict(hidden_size=D, intermediate_size=cfg.intermediate_size),
                            dict(gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                                 down=p + "mlp.down_proj.weight")),
        }))
    embed_name, head_name = "model.embed_tokens.weight", "lm_head.weight"
    if cfg.tie_word_embeddings:
        # tied: the head is the embedding table; a file that holds only lm_head serves both
        embedding = PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D,
                                                     alternatives=(head_name,)),
                             dict(weight=embed_name))
        head = PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, alternatives=(head_name,),
                                        stored=False), dict(weight=embed_name))
    else:
        embedding = PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D),
                             dict(weight=embed_name))
        head = PartSpec("lm_head", dict(vocab_size=V, hidden_size=D), dict(weight=head_name))
    return ModelSpec(
        hidden_size=D, vocab_size=V, max_position=cfg.max_position_embeddings,
        embedding=embedding, layers=layers,
        order=[RunStep(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", dict(size=D, eps=cfg.rms_norm_eps),
                            dict(weight="model.norm.weight")),
        lm_head=head, position_encodings={"rope": rope}, eos_token_ids=cfg.eos_token_ids,
        # older exports store the rotary table's frequencies as a buffer of every layer
        ignored_tensors=("self_attn.rotary_emb.inv_freq",))


register_architecture(LlamaConfig.ARCHITECTURE, LlamaConfig, build_llama_spec)
