"""EAGLE drafter (bf16) over a W4A16 GPTQ-Marlin target (reference
cpmcu/speculative/eagle_base_quant/eagle_base_w4a16_marlin_gptq.py:8-103)."""
from ...llm_w4a16_gptq_marlin import W4A16Mixin
from ..eagle import LLM_with_eagle


class W4A16GPTQMarlinLLM_with_eagle(W4A16Mixin, LLM_with_eagle):
    def __init__(self, eagle_path, base_path, use_rotation=False, **kwargs):
        if use_rotation:
            raise NotImplementedError("the rotated EAGLE variant has no native entry point")
        super().__init__(eagle_path, base_path, **kwargs)
