"""The C ABI library loads without a GPU and exports every symbol the header declares
(no compute calls here)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cpmcu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cpmcu_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as entry
    import cpmcu.C as C
    if not os.path.exists(C.lib_path()):
        entry.build()
    return C.load()


def test_header_declares_the_reference_entry_points():
    names = declared_symbols()
    for ref in ["init_base_model", "init_minicpm4_model", "init_w4a16_gptq_marlin_base_model",
                "init_w4a16_gptq_marlin_minicpm4_model", "init_eagle_model", "init_minicpm4_eagle_model",
                "init_w4a16_gm_spec_w4a16_gm_model", "init_hier_eagle_w4a16_gm_spec_w4a16_gm_model",
                "init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model", "init_storage", "load_model", "prefill", "decode",
                "draft", "verify_and_fix", "print_perf_summary"]:  # src/entry.cu:510-535
        assert "cpmcu_" + ref in names


def test_library_exports_every_declared_symbol(lib):
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, missing


def test_python_binding_covers_every_declared_symbol(lib):
    import cpmcu.C as C
    assert sorted(C.exported_symbols()) == declared_symbols()
    for name in ["init_base_model", "init_eagle_model", "init_minicpm4_eagle_model", "init_storage", "load_model",
                 "prefill", "decode", "draft", "verify_and_fix", "print_perf_summary"]:
        assert callable(getattr(C, name))


def test_calls_fail_loudly_without_a_model_or_gpu(lib):
    import cpmcu.C as C
    with pytest.raises(RuntimeError):
        C.init_storage()
    with pytest.raises(RuntimeError):
        C.init_w4a16_gptq_marlin_base_model(0.5, 1000, 1, 256, 704, 2, 1, 128, 1e-5, 128, 1, 128, 1.0, 1.0, 1.0)
    with pytest.raises(RuntimeError):
        C.init_hier_eagle_w4a16_gm_spec_w4a16_gm_model()
