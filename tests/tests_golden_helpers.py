"""Imports the fixture generators of tests/golden/make_golden.py for the CPU tests."""
import importlib.util
import os

_spec = importlib.util.spec_from_file_location(
    "make_golden", os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_golden.py"))
_mod = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_mod)
tree_case, verify_case, generate_case = _mod.tree_case, _mod.verify_case, _mod.generate_case
