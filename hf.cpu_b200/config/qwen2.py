"""Qwen2 dense decoder: typed configuration from config.json and its layer plan.

Keys and defaults follow the reference's loader (src/model.c:119-145): required
layer count, width, feed-forward width and head count; optional KV-head count
(default: heads), head size (default: width / heads), eps and rope base; geometry
checks ``heads % kv_heads == 0`` and an even head size (src/model.c:141-144).
The sliding-window keys have no counterpart in the reference (its loop always
runs over keys 0..pos, src/model.c:514); they follow config.json's own meaning:
layers with index >= ``max_window_layers`` see the last ``sliding_window`` keys.

``rope_dim`` (optional, default: the head size) is how many leading dimensions of
each head the rotary encoding turns; it is what the reference reads from a GGUF
file's ``<arch>.rope.dimension_count`` (src/model.c:132-133) and must be even and
at most the head size (src/model.c:141-144).

The same class is the GGUF side of the architecture: the metadata keys under
``qwen2.`` and the ``blk.N.*`` tensor names of the reference's loader
(src/model.c:119-139, :149-180).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry,
                   UnsupportedError, take_bool, take_float, take_int)
from .registry import register_architecture


@dataclass
class Qwen2Config(ModelConfig):
    num_hidden_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rope_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    max_position_embeddings: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    hidden_act: str = "silu"
    torch_dtype: str = "bfloat16"
    eos_token_id: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Qwen2Config":
        L = take_int(d, "num_hidden_layers", lo=1, hi=1_000_000)
        E = take_int(d, "hidden_size", lo=1, hi=1_000_000)
        F = take_int(d, "intermediate_size", lo=1, hi=1_000_000)
        H = take_int(d, "num_attention_heads", lo=1, hi=1_000_000)
        G = take_int(d, "num_key_value_heads", default=H, lo=1, hi=1_000_000)
        if "head_dim" in d and d["head_dim"] is not None:
            hd = take_int(d, "head_dim", lo=2)
        else:
            if E % H:
                raise ConfigError(f"config.json: hidden_size {E} is not a multiple of "
                                  f"num_attention_heads {H} and no head_dim is given")
            hd = E // H
        V = take_int(d, "vocab_size", lo=1)
        maxpos = take_int(d, "max_position_embeddings", lo=1)
        if H % G:
            raise UnsupportedError(f"unsupported attention geometry: {H} heads over {G} key/value heads")
        if hd % 2:
            raise UnsupportedError(f"unsupported attention geometry: head_dim {hd} is odd")
        rd = take_int(d, "rope_dim", default=hd, lo=0) or hd
        if rd % 2 or rd > hd:
            raise UnsupportedError(f"unsupported attention geometry: rope_dim {rd} must be even and at most "
                                   f"head_dim {hd}")
        if H * hd > 1 << 20 or G * hd > 1 << 20:
            raise UnsupportedError("unsupported attention geometry: projection wider than 2^20")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise UnsupportedError(f"hidden_act '{act}' is not supported (only 'silu')")
        if d.get("rope_scaling") is not None:
            raise UnsupportedError("rope_scaling is not supported")
        usw = take_bool(d, "use_sliding_window", False)
        sw = take_int(d, "sliding_window", default=0, lo=0) if usw else (d.get("sliding_window") or 0)
        mwl = take_int(d, "max_window_layers", default=L, lo=0) if usw else (d.get("max_window_layers") or 0)
        if usw:
            if sw < 1:
                raise ConfigError("config.json: use_sliding_window is true but sliding_window < 1")
            if mwl > L:
                raise ConfigError(f"config.json: max_window_layers {mwl} exceeds num_hidden_layers {L}")
        eos = d.get("eos_token_id", [])
        if eos is None:
            eos = []
        if isinstance(eos, int):
            eos = [eos]
        if not isinstance(eos, list) or any(isinstance(e, bool) or not isinstance(e, int) for e in eos):
            raise ConfigError("config.json: 'eos_token_id' must be an integer or a list of integers")
        return cls(
            num_hidden_layers=L, hidden_size=E, num_attention_heads=H, num_key_value_heads=G,
            head_dim=hd, rope_dim=rd, intermediate_size=F, vocab_size=V, max_position_embeddings=maxpos,
            rms_norm_eps=take_float(d, "rms_norm_eps", 1e-5, lo=0.0),
            rope_theta=take_float(d, "rope_theta", 10000.0, lo=0.0),
            tie_word_embeddings=take_bool(d, "tie_word_embeddings", False),
            use_sliding_window=usw, sliding_window=int(sw), max_window_layers=int(mwl),
            hidden_act=act, torch_dtype=str(d.get("torch_dtype", "bfloat16")), eos_token_id=list(eos))

    def to_dict(self) -> Dict[str, Any]:
        d = super().to_dict()
        d["model_type"] = "qwen2"
        return d

    def window_of_layer(self, layer: int) -> int:
        """0 = all keys; else the number of most recent keys the layer sees."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    def plan(self) -> ModelPlan:
        E = self.hidden_size
        norm = lambda name: PartSpec("rmsnorm", {"size": E, "eps": self.rms_norm_eps, "tensor": name})
        layers = []
        for l in range(self.num_hidden_layers):
            p = f"model.layers.{l}"
            layers.append(LayerSpec(
                prefix=p,
                block=PartSpec("prenorm_residual"),
                norm1=norm(f"{p}.input_layernorm.weight"),
                mixer=PartSpec("paged_attention", {
                    "hidden_size": E, "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                    "qkv_bias": True, "out_bias": False, "window": self.window_of_layer(l),
                    "position": "rope", "prefix": f"{p}.self_attn"}),
                norm2=norm(f"{p}.post_attention_layernorm.weight"),
                ffn=PartSpec("swiglu", {"hidden_size": E, "intermediate_size": self.intermediate_size,
                                        "prefix": f"{p}.mlp"})))
        plan = ModelPlan(
            hidden_size=E, vocab_size=self.vocab_size, max_positions=self.max_position_embeddings,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab_size, "hidden_size": E,
                                             "tensor": "model.embed_tokens.weight"}),
            positions={"rope": PartSpec("rotary", {"head_dim": self.head_dim, "n_rot": self.rope_dim or self.head_dim,
                                                   "theta": self.rope_theta, "pairing": "half"})},
            layers=layers,
            schedule=[ScheduleEntry(l) for l in range(self.num_hidden_layers)],
            final_norm=norm("model.norm.weight"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab_size, "hidden_size": E,
                                          "tensor": "lm_head.weight",
                                          "tied_to": "model.embed_tokens.weight" if self.tie_word_embeddings else None}),
            eos_token_ids=list(self.eos_token_id))
        plan.validate()
        return plan


    # ---- GGUF ------------------------------------------------------------------------------------------
    gguf_architecture = "qwen2"

    _GGUF_TOP = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
                 "lm_head.weight": "output.weight"}
    _GGUF_LAYER = {
        "input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
        "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
        "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
        "self_attn.q_proj.bias": "attn_q.bias", "self_attn.k_proj.bias": "attn_k.bias",
        "self_attn.v_proj.bias": "attn_v.bias", "mlp.gate_proj.weight": "ffn_gate.weight",
        "mlp.up_proj.weight": "ffn_up.weight", "mlp.down_proj.weight": "ffn_down.weight"}

    def gguf_names(self) -> Dict[str, str]:
        names = {c: g for c, g in self._GGUF_TOP.items() if not (c == "lm_head.weight" and self.tie_word_embeddings)}
        for l in range(self.num_hidden_layers):
            for c, g in self._GGUF_LAYER.items():
                names[f"model.layers.{l}.{c}"] = f"blk.{l}.{g}"
        return names

    def gguf_left_out(self) -> List[str]:
        return ["lm_head.weight"] if self.tie_word_embeddings else []

    def gguf_metadata(self) -> List[tuple]:
        a, U32, F32 = self.gguf_architecture, 4, 6
        kv = [(f"{a}.block_count", U32, self.num_hidden_layers),
              (f"{a}.context_length", U32, self.max_position_embeddings),
              (f"{a}.embedding_length", U32, self.hidden_size),
              (f"{a}.feed_forward_length", U32, self.intermediate_size),
              (f"{a}.attention.head_count", U32, self.num_attention_heads),
              (f"{a}.attention.head_count_kv", U32, self.num_key_value_heads),
              (f"{a}.attention.key_length", U32, self.head_dim),
              (f"{a}.attention.layer_norm_rms_epsilon", F32, self.rms_norm_eps),
              (f"{a}.rope.freq_base", F32, self.rope_theta)]
        if self.rope_dim and self.rope_dim != self.head_dim:
            kv.append((f"{a}.rope.dimension_count", U32, self.rope_dim))
        if self.use_sliding_window:
            raise UnsupportedError("a sliding window has no GGUF metadata key in the reference's files")
        return kv

    @classmethod
    def from_gguf(cls, meta: Dict[str, Any], shapes: Dict[str, tuple], where: str = "") -> "Qwen2Config":
        """Keys, defaults and plausibility bounds of the reference's loader (src/model.c:119-139); the vocabulary
        is the embedding's row count (src/model.c:147-155) and the head is tied when the file has no
        ``output.weight`` (src/model.c:156-159).  Scaled rotary frequencies are not implemented: a file that asks
        for them is refused, as ``rope_scaling`` in config.json is."""
        a = cls.gguf_architecture

        def need(key):
            if f"{a}.{key}" not in meta:
                raise ConfigError(f"{where}: metadata key '{a}.{key}' is missing")
            return meta[f"{a}.{key}"]
        for key, v in meta.items():
            if key.startswith(f"{a}.rope.scaling.") or key == f"{a}.rope.scale_linear" or key == f"{a}.rope.freq_scale":
                if not (key.endswith(".type") and v in ("none", "")) and not (isinstance(v, (int, float)) and v == 1):
                    raise UnsupportedError(f"{where}: '{key}' asks for scaled rotary frequencies, which are not supported")
        E, H = need("embedding_length"), need("attention.head_count")
        if "token_embd.weight" not in shapes or len(shapes["token_embd.weight"]) != 2:
            raise ConfigError(f"{where}: token_embd.weight is missing or has an unexpected shape")
        d = {"num_hidden_layers": need("block_count"), "hidden_size": E,
             "intermediate_size": need("feed_forward_length"), "num_attention_heads": H,
             "num_key_value_heads": meta.get(f"{a}.attention.head_count_kv") or H,
             "head_dim": meta.get(f"{a}.attention.key_length") or None,
             "rope_dim": meta.get(f"{a}.rope.dimension_count") or None,
             "rms_norm_eps": float(meta.get(f"{a}.attention.layer_norm_rms_epsilon", 1e-5)),
             "rope_theta": float(meta.get(f"{a}.rope.freq_base", 10000.0)),
             "max_position_embeddings": meta.get(f"{a}.context_length", 0) or 32768,
             "vocab_size": int(shapes["token_embd.weight"][0]),
             "tie_word_embeddings": "output.weight" not in shapes}
        return cls.from_dict(d)


register_architecture("Qwen2ForCausalLM", Qwen2Config)
register_architecture("qwen2", Qwen2Config)
