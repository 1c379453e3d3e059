"""ctypes binding of libcpmcu_b200.so under the names of the reference's pybind
module `cpmcu.C` (src/entry.cu:510-535).  Argument order and meaning are the
reference's; pointers are passed as integers (tensor.data_ptr()).

There is no fallback: if the library is missing or no sm_100 GPU is visible,
the first call raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcpmcu_b200.so")
_lib = None

_c_int, _c_float, _c_void_p, _c_char_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p

_SIGNATURES = {
    "cpmcu_last_error": (_c_char_p, []),
    "cpmcu_init_base_model": (_c_int, [_c_float] + [_c_int] * 7 + [_c_float, _c_int, _c_int] + [_c_float] * 3),
    "cpmcu_init_minicpm4_model": (_c_int, [_c_float] + [_c_int] * 7 + [_c_float, _c_int, _c_int] + [_c_float] * 3 + [_c_int] * 5),
    "cpmcu_init_w4a16_gptq_marlin_base_model": (_c_int, [_c_float] + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_int] + [_c_float] * 3),
    "cpmcu_init_w4a16_gptq_marlin_minicpm4_model": (_c_int, [_c_float] + [_c_int] * 7 + [_c_float, _c_int, _c_int, _c_int] + [_c_float] * 3 + [_c_int] * 5),
    "cpmcu_init_eagle_model": (_c_int, [_c_int] * 5),
    "cpmcu_init_minicpm4_eagle_model": (_c_int, [_c_int] * 9 + [_c_float, _c_int, _c_int]),
    "cpmcu_init_w4a16_gm_spec_w4a16_gm_model": (_c_int, []),
    "cpmcu_init_hier_eagle_w4a16_gm_spec_w4a16_gm_model": (_c_int, []),
    "cpmcu_init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model": (_c_int, []),
    "cpmcu_init_storage": (_c_int, []),
    "cpmcu_load_model": (_c_int, [_c_char_p, _c_void_p]),
    "cpmcu_prefill": (_c_int, [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p]),
    "cpmcu_decode": (_c_int, [_c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int]),
    "cpmcu_draft": (_c_int, [_c_void_p] * 5),
    "cpmcu_verify_and_fix": (_c_int, [_c_int] + [_c_void_p] * 6),
    "cpmcu_print_perf_summary": (None, []),
    "cpmcu_begin_generation": (_c_int, [_c_int, _c_int]),
    "cpmcu_spec_step": (_c_int, [_c_void_p, _c_int]),
    "cpmcu_set_sampling": (_c_int, [ctypes.c_float, ctypes.c_ulonglong]),
    "cpmcu_sample": (_c_int, [_c_void_p, _c_int, _c_int, ctypes.c_float, ctypes.c_ulonglong, _c_int, _c_void_p]),
    "cpmcu_profile_step": (_c_int, [_c_void_p] * 3),
    "cpmcu_last_step_ms": (ctypes.c_double, []),
    "cpmcu_last_draft_ms": (ctypes.c_double, []),
    "cpmcu_last_verify_ms": (ctypes.c_double, []),
    "cpmcu_launches_per_step": (ctypes.c_long, []),
    "cpmcu_total_launches": (ctypes.c_long, []),
    "cpmcu_get_tree": (_c_int, [_c_void_p] * 6),
    "cpmcu_capture_blockmasks": (_c_int, [_c_void_p]),
    "cpmcu_release": (None, []),
    "cpmcu_linear_bf16": (_c_int, [_c_void_p] * 4 + [_c_int] * 4),
    "cpmcu_linear_w4a16": (_c_int, [_c_void_p] * 4 + [_c_int] * 4),
    "cpmcu_bench_linear": (_c_int, [_c_int] * 6 + [_c_void_p]),
    "cpmcu_bench_linear_w4": (_c_int, [_c_int] * 6 + [_c_void_p]),
    "cpmcu_bench_linear_swiglu": (_c_int, [_c_int] * 6 + [_c_void_p]),
    "cpmcu_bench_attention": (_c_int, [_c_int] * 7 + [_c_void_p]),
    "cpmcu_sparse_attention": (_c_int, [_c_void_p, _c_int, _c_void_p, _c_void_p] + [_c_int] * 4 +
                               [_c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p,
                                _c_int]),
    "cpmcu_sparse_select": (_c_int, [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_void_p] +
                            [_c_int] * 6 + [_c_void_p] * 3 + [_c_int, _c_void_p, _c_int]),
    "cpmcu_tree_attention": (_c_int, [_c_void_p, _c_int, _c_void_p, _c_void_p] + [_c_int] * 4 +
                             [_c_void_p, _c_int, _c_void_p, _c_void_p] + [_c_int] * 3 + [_c_void_p, _c_int]),
    "cpmcu_rms_norm": (_c_int, [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_float]),
    "cpmcu_rope_append": (_c_int, [_c_void_p, _c_int, _c_int, _c_int] + [_c_void_p] * 5 + [_c_int]),
    "cpmcu_silu_gate": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int]),
    "cpmcu_linear_swiglu_bf16": (_c_int, [_c_void_p] * 3 + [_c_int] * 4),
    "cpmcu_debug_linear_schedule": (_c_int, [_c_int] * 4 + [_c_void_p, _c_int]),
    "cpmcu_argmax": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p]),
    "cpmcu_argmax_noalloc": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p]),
    "cpmcu_draft_tree_from_logits": (_c_int, [_c_void_p] + [_c_int] * 4 + [_c_void_p] * 9),
    "cpmcu_verify_and_compact": (_c_int, [_c_int] + [_c_void_p] * 7 + [_c_int] * 3 + [_c_void_p]),
    "cpmcu_accept_fixup": (_c_int, [_c_int] + [_c_void_p] * 7 + [_c_int] * 5 + [_c_void_p] * 3 + [ctypes.c_float] +
                           [_c_void_p] * 3),
}


def lib_path():
    return _LIB_PATH


def load():
    """Load the shared library (raises if it has not been built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(
                "libcpmcu_b200.so is missing at %s; build it with `python cpm.cu_b200/build.py` "
                "(there is no CPU or PyTorch fallback)" % _LIB_PATH)
        lib = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def exported_symbols():
    return sorted(_SIGNATURES)


def _check(code):
    if code < 0:
        raise RuntimeError(load().cpmcu_last_error().decode())
    return code


def call(name, *args):
    """Call an extern "C" entry point by name; negative return codes raise RuntimeError."""
    fn = getattr(load(), name)
    res = fn(*args)
    if fn.restype is _c_int:
        return _check(res)
    return res


# ---------------------------------------------------------------- reference names
def init_base_model(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size, num_attention_heads,
                    num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed, scale_lmhead,
                    scale_residual):
    call("cpmcu_init_base_model", memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size,
         num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed,
         scale_lmhead, scale_residual)


def init_minicpm4_model(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size,
                        num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length,
                        scale_embed, scale_lmhead, scale_residual, sink_window_size, block_window_size, sparse_topk_k,
                        sparse_switch, apply_compress_lse):
    call("cpmcu_init_minicpm4_model", memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size,
         num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, torch_dtype, chunk_length, scale_embed,
         scale_lmhead, scale_residual, sink_window_size, block_window_size, sparse_topk_k, sparse_switch,
         int(apply_compress_lse))


def init_w4a16_gptq_marlin_base_model(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size,
                                      num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, group_size,
                                      torch_dtype, chunk_length, scale_embed, scale_lmhead, scale_residual):
    call("cpmcu_init_w4a16_gptq_marlin_base_model", memory_limit, vocab_size, num_hidden_layers, hidden_size,
         intermediate_size, num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, group_size, torch_dtype,
         chunk_length, scale_embed, scale_lmhead, scale_residual)


def init_w4a16_gptq_marlin_minicpm4_model(memory_limit, vocab_size, num_hidden_layers, hidden_size, intermediate_size,
                                          num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, group_size,
                                          torch_dtype, chunk_length, scale_embed, scale_lmhead, scale_residual,
                                          sink_window_size, block_window_size, sparse_topk_k, sparse_switch,
                                          apply_compress_lse):
    call("cpmcu_init_w4a16_gptq_marlin_minicpm4_model", memory_limit, vocab_size, num_hidden_layers, hidden_size,
         intermediate_size, num_attention_heads, num_key_value_heads, head_dim, rms_norm_eps, group_size, torch_dtype,
         chunk_length, scale_embed, scale_lmhead, scale_residual, sink_window_size, block_window_size, sparse_topk_k,
         sparse_switch, int(apply_compress_lse))


def init_eagle_model(num_layers, num_iter, topk_per_iter, tree_size, torch_dtype):
    call("cpmcu_init_eagle_model", num_layers, num_iter, topk_per_iter, tree_size, torch_dtype)


def init_minicpm4_eagle_model(num_layers, num_iter, topk_per_iter, tree_size, torch_dtype, apply_eagle_quant,
                              group_size, eagle_window_size, frspec_vocab_size, residual_scale, use_input_norm,
                              use_attn_norm):
    call("cpmcu_init_minicpm4_eagle_model", num_layers, num_iter, topk_per_iter, tree_size, torch_dtype,
         int(apply_eagle_quant), group_size, eagle_window_size, frspec_vocab_size, residual_scale,
         int(use_input_norm), int(use_attn_norm))


def init_w4a16_gm_spec_w4a16_gm_model(*args):
    call("cpmcu_init_w4a16_gm_spec_w4a16_gm_model")


def init_hier_eagle_w4a16_gm_spec_w4a16_gm_model(*args):
    call("cpmcu_init_hier_eagle_w4a16_gm_spec_w4a16_gm_model")


def init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model(*args):
    call("cpmcu_init_hier_eagle_w4a16_gm_rot_spec_w4a16_gm_model")


def init_storage():
    return call("cpmcu_init_storage")


def load_model(name, param):
    call("cpmcu_load_model", name.encode(), param)


def prefill(input_length, history_length, input, position_ids, output):
    call("cpmcu_prefill", input_length, history_length, input, position_ids, output)


def decode(input_length, padded_length, input, position_ids, cache_length, mask_2d, output, cuda_graph):
    call("cpmcu_decode", input_length, padded_length, input, position_ids, cache_length, mask_2d or None, output,
         int(cuda_graph))


def draft(tree_draft_ids, tree_position_ids, cache_length, attn_mask, tree_parent):
    call("cpmcu_draft", tree_draft_ids, tree_position_ids, cache_length, attn_mask, tree_parent)


def verify_and_fix(num_tokens, pred, gt, position_ids, cache_length, attn_mask, tree_parent):
    return call("cpmcu_verify_and_fix", num_tokens, pred, gt, position_ids, cache_length, attn_mask, tree_parent)


def print_perf_summary():
    load().cpmcu_print_perf_summary()


# ---------------------------------------------------------------- fused step (no reference counterpart)
def begin_generation(prefix_length, root_token):
    call("cpmcu_begin_generation", prefix_length, root_token)


def set_sampling(temperature, seed):
    call("cpmcu_set_sampling", float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF)


def sample(logits_ptr, rows, vocab, temperature, seed, draw, out_ptr):
    call("cpmcu_sample", logits_ptr, rows, vocab, float(temperature), int(seed) & 0xFFFFFFFFFFFFFFFF, draw, out_ptr)


def spec_step(max_tokens=16):
    """Run one captured speculative step; returns the list of emitted tokens."""
    buf = (ctypes.c_int32 * max_tokens)()
    n = call("cpmcu_spec_step", ctypes.cast(buf, _c_void_p), max_tokens)
    return list(buf[: min(n, max_tokens)])


def profile_step():
    """One eager step with per-launch CUDA events: returns ({class: (ms, launches)}, total_ms)."""
    ms = (ctypes.c_float * 3)()
    cnt = (ctypes.c_int * 3)()
    total = ctypes.c_float()
    call("cpmcu_profile_step", ctypes.cast(ms, _c_void_p), ctypes.cast(cnt, _c_void_p),
         ctypes.cast(ctypes.pointer(total), _c_void_p))
    return {"linear": (ms[0], cnt[0]), "attention": (ms[1], cnt[1]), "selection": (ms[2], cnt[2])}, total.value


def last_step_ms():
    return load().cpmcu_last_step_ms()


def last_step_split_ms():
    """(draft half, verify half) of the last spec_step in device milliseconds."""
    lib = load()
    return lib.cpmcu_last_draft_ms(), lib.cpmcu_last_verify_ms()


def launches_per_step():
    return load().cpmcu_launches_per_step()


def total_launches():
    return load().cpmcu_total_launches()


def release():
    load().cpmcu_release()
