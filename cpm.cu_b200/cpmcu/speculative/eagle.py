"""`LLM_with_eagle`: EAGLE drafter front end (reference cpmcu/speculative/eagle.py:15-99).
Chooses the plain EAGLE head or the MiniCPM4 variant (input norms, attention
norm, FR-Spec vocabulary, draft window) exactly as the reference does, and
splits the checkpoint's `fc` matrix into the embedding half (fc1) and the
hidden-state half (fc2)."""
import math
import types

from .. import C
from .tree_drafter import LLM_with_tree_drafter


class LLM_with_eagle(LLM_with_tree_drafter):
    def __init__(self, eagle_path, base_path, num_iter=6, topk_per_iter=10, tree_size=60, eagle_window_size=0,
                 frspec_vocab_size=0, apply_eagle_quant=False, use_rope=False, use_input_norm=False,
                 use_attn_norm=False, eagle_config=None, **kwargs):
        super().__init__("eagle", eagle_path, base_path, tree_size=tree_size, use_rope=use_rope, **kwargs)
        self.eagle_path = eagle_path
        if eagle_config is None:
            from transformers import PretrainedConfig
            eagle_config = PretrainedConfig.from_pretrained(eagle_path)
        elif isinstance(eagle_config, dict):
            eagle_config = types.SimpleNamespace(**eagle_config)
        self.eagle_config = eagle_config
        self.eagle_config.eagle_num_layers = getattr(eagle_config, "num_hidden_layers", 1)
        for attr in ("scale_depth", "dim_model_base", "scale_emb"):
            base_has, eagle_has = hasattr(self.config, attr), hasattr(self.eagle_config, attr)
            assert base_has == eagle_has, f"{attr} presence mismatch between base and eagle config"
            if base_has:
                assert getattr(self.config, attr) == getattr(self.eagle_config, attr), \
                    f"{attr} in base config and eagle config should be the same"
        scale_residual = (self.config.scale_depth / math.sqrt(self.config.num_hidden_layers + 1)
                          if hasattr(self.config, "scale_depth") else 1.0)
        self.apply_eagle_quant = apply_eagle_quant
        self.group_size = 0
        if apply_eagle_quant and hasattr(self.eagle_config, "quantization_config"):
            self.group_size = self.eagle_config.quantization_config.get("group_size", 0)
        assert self.group_size in (0, 128), "only group_size 128 is supported in quantization mode"
        self.frspec_vocab_size = frspec_vocab_size
        plain = not (use_rope or use_input_norm or use_attn_norm or apply_eagle_quant)
        if plain and frspec_vocab_size == 0 and eagle_window_size == 0:
            C.init_eagle_model(self.eagle_config.eagle_num_layers, num_iter, topk_per_iter, self.tree_size,
                               self.dtype_int)
        else:
            C.init_minicpm4_eagle_model(self.eagle_config.eagle_num_layers, num_iter, topk_per_iter, self.tree_size,
                                        self.dtype_int, apply_eagle_quant, self.group_size, eagle_window_size,
                                        frspec_vocab_size, scale_residual, use_input_norm, use_attn_norm)

    def _load(self, name, param, dtype=None, cls=None):
        if cls != self.drafter_type:
            return super()._load(name, param, dtype)
        import torch
        if name == "token_id_remap":
            param = param.contiguous().to(dtype=torch.int32)
            C.load_model(f"{cls}.{name}", param.data_ptr())
            return
        if "embed_tokens" in name:
            return  # the drafter shares the target's embedding table
        if dtype is None:
            dtype = self.dtype
        param = param.contiguous()
        if param.dtype not in (torch.int8, torch.int16, torch.int32):
            param = param.to(dtype)  # packed int4 tensors of a quantised drafter pass through untouched
        if "fc" in name:
            # the checkpoint's fc holds the embedding half and the hidden-state half side by side along the last
            # dimension: columns of the bf16 weight; for a quantised drafter the two [H -> H] linears' qweight /
            # scales tensors concatenated (reference eagle_base_w4a16_marlin_gptq.py:92-99)
            if "weight" in name or "scales" in name:
                half = param.shape[-1] // 2
                first, second = param[..., :half].contiguous(), param[..., half:].contiguous()
                C.load_model(f"{cls}.{name.replace('fc', 'fc1')}", first.data_ptr())
                C.load_model(f"{cls}.{name.replace('fc', 'fc2')}", second.data_ptr())
            else:
                C.load_model(f"{cls}.{name.replace('fc', 'fc1')}", param.data_ptr())
        else:
            C.load_model(f"{cls}.{name}", param.data_ptr())
