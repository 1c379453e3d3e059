"""Speculative decoding front ends (reference: cpmcu/speculative/)."""
from .eagle import LLM_with_eagle  # noqa: F401
from .tree_drafter import LLM_with_tree_drafter  # noqa: F401
