"""`W4A16GPTQMarlinLLM`: target with GPTQ-Marlin int4 linears (reference
cpmcu/llm_w4a16_gptq_marlin.py:24-463).  Checkpoints carry the fused tensors
`qkv_proj`, `o_proj`, `gate_up_proj`, `down_proj` as `qweight` (int32, Marlin tile
order) and `scales` (model dtype); embeddings, norms and the LM head stay bf16.

The library re-tiles the int4 tensors when they are loaded (one contiguous block
of nibbles and scales per 128-row x 256-k unit) and streams them as 4-bit through
the W4A16 GEMM, which dequantises w = (q - 8) * scale on the way into the tensor
cores (csrc/gemm_w4_umma.cu)."""
import math

import torch

from . import C
from .llm import LLM


class W4A16Mixin:
    """Overrides shared by every class whose target is W4A16 GPTQ-Marlin."""

    def _init_native(self, memory_limit, scale_embed, scale_lmhead, scale_residual, apply_sparse, sparse_args):
        cfg = self.config
        qc = getattr(cfg, "quantization_config", None) or {}
        group_size = qc.get("group_size", 128) if isinstance(qc, dict) else getattr(qc, "group_size", 128)
        assert group_size == 128, "only group_size 128 is supported in quantization mode"
        self.group_size = group_size
        common = (memory_limit, cfg.vocab_size, cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size,
                  cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, group_size,
                  self.dtype_int, self.chunk_length, scale_embed, scale_lmhead, scale_residual)
        if apply_sparse:
            C.init_w4a16_gptq_marlin_minicpm4_model(*common, *sparse_args)
        else:
            C.init_w4a16_gptq_marlin_base_model(*common)

    def _load(self, name, param, dtype=None, cls=None):
        if cls is not None and cls == getattr(self, "drafter_type", None):
            return super()._load(name, param, dtype, cls)
        if dtype is None:
            dtype = torch.float32 if "rotary_emb" in name else self.dtype
        param = param.contiguous()
        if param.dtype not in (torch.int8, torch.int16, torch.int32):
            param = param.to(dtype)  # packed integer tensors are passed through untouched
        C.load_model(name, param.data_ptr())
        if "embed_tokens" in name and getattr(self.config, "tie_word_embeddings", False):
            self._load("lm_head.weight", param)


class W4A16GPTQMarlinLLM(W4A16Mixin, LLM):
    pass
