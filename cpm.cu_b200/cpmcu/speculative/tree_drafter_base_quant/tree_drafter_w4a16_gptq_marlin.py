"""Tree speculative decoding over a W4A16 GPTQ-Marlin target (reference
cpmcu/speculative/tree_drafter_base_quant/tree_drafter_w4a16_gptq_marlin.py)."""
from ...llm_w4a16_gptq_marlin import W4A16Mixin
from ..tree_drafter import LLM_with_tree_drafter


class W4A16GPTQMarlinLLM_with_tree_drafter(W4A16Mixin, LLM_with_tree_drafter):
    pass
