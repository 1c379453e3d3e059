"""`LLM`: the reference's base model class (cpmcu/llm.py:22-419) over the B200
library.  Same constructor keywords, `init_storage`, `_load`, `load_from_hf`,
`prefill`, `decode` and `generate` contracts; all device work happens in
libcpmcu_b200.so through `cpmcu.C`.

Two additions that the reference does not have, both optional:
  * `config=` / `tokenizer=` let a caller pass a ready configuration object
    instead of a Hugging Face directory (used with synthetic weights);
  * `load_state_dict()` feeds tensors that are already in memory.
"""
import glob
import json
import math
import os
import time
import types

import torch
import torch.nn.functional as F

from . import C

dtype_map = {torch.float16: 0, torch.bfloat16: 1}


def dtype_to_int(dtype):
    if dtype not in dtype_map:
        raise ValueError(f"Unsupported dtype: {dtype}")
    return dtype_map[dtype]


def default_rope_inv_freq(config):
    """inv_freq of the 'default' rope type: theta^(-2i/d).  Newer `transformers` keep rope_theta inside
    config.rope_scaling / rope_parameters instead of on the config itself."""
    scaling = getattr(config, "rope_scaling", None) or {}
    theta = getattr(config, "rope_theta", None) or scaling.get("rope_theta") or 10000.0
    d = config.head_dim
    return 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))


class LLM(torch.nn.Module):
    def __init__(self, path, memory_limit=0.8, chunk_length=1024, dtype=None, cuda_graph=False, apply_sparse=False,
                 sink_window_size=1, block_window_size=32, sparse_topk_k=32, sparse_switch=8192,
                 apply_compress_lse=False, use_enter=False, use_decode_enter=False, temperature=0.0,
                 random_seed=None, minicpm4_yarn=False, config=None, tokenizer=None):
        super().__init__()
        self.path = path
        if config is None:
            from transformers import AutoConfig, AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(path, trust_remote_code=True)
            self.config = AutoConfig.from_pretrained(path, trust_remote_code=True)
        else:
            self.tokenizer = tokenizer
            self.config = config if not isinstance(config, dict) else types.SimpleNamespace(**config)
        self.dtype = dtype if dtype is not None else getattr(self.config, "torch_dtype", torch.bfloat16)
        self.dtype_int = dtype_to_int(self.dtype)
        self.cuda_graph = cuda_graph
        self.use_enter = use_enter
        self.use_decode_enter = use_decode_enter
        self.temperature = temperature
        self.chunk_length = chunk_length
        if minicpm4_yarn:
            # the reference swaps in a fixed table of 64 LongRoPE factors here (cpmcu/llm_w4a16_gptq_marlin.py:192-219);
            # give the same factors through the checkpoint's config.json (rope_scaling: rope_type "longrope") instead
            raise NotImplementedError("minicpm4_yarn=True is not supported: put the LongRoPE factors into the "
                                      "checkpoint's rope_scaling (rope_type 'longrope'), which is honoured")
        self.minicpm4_yarn = minicpm4_yarn
        self._show_prefill_progress = False
        self.generator = None
        self.sample_seed = random_seed   # seeds the device-side sampling of the fused speculative step
        if random_seed is not None:
            self.generator = torch.Generator(device="cuda")
            self.generator.manual_seed(random_seed)

        cfg = self.config
        if not hasattr(cfg, "head_dim") or cfg.head_dim is None:
            cfg.head_dim = cfg.hidden_size // cfg.num_attention_heads
        scale_embed = getattr(cfg, "scale_emb", 1.0)
        scale_lmhead = (cfg.dim_model_base / cfg.hidden_size) if hasattr(cfg, "dim_model_base") else 1.0
        scale_residual = cfg.scale_depth / math.sqrt(cfg.num_hidden_layers) if hasattr(cfg, "scale_depth") else 1.0
        self._init_native(memory_limit, scale_embed, scale_lmhead, scale_residual, apply_sparse,
                          (sink_window_size, block_window_size, sparse_topk_k, sparse_switch, apply_compress_lse))
        self.logits = torch.empty((64, cfg.vocab_size), dtype=self.dtype, device="cuda")
        self.max_total_length = 0

    def _init_native(self, memory_limit, scale_embed, scale_lmhead, scale_residual, apply_sparse, sparse_args):
        """Create the native model (bf16 target).  Quantised subclasses override this."""
        cfg = self.config
        common = (memory_limit, cfg.vocab_size, cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size,
                  cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rms_norm_eps, self.dtype_int,
                  self.chunk_length, scale_embed, scale_lmhead, scale_residual)
        if apply_sparse:
            C.init_minicpm4_model(*common, *sparse_args)
        else:
            C.init_base_model(*common)

    # ------------------------------------------------------------------ storage / weights
    def init_storage(self):
        self.max_total_length = C.init_storage()
        print("max supported length under current memory limit: ", self.max_total_length)

    def _load(self, name, param, dtype=None, cls=None):
        if dtype is None:
            dtype = torch.float32 if "rotary_emb" in name else self.dtype
        cfg = self.config
        if "gate_up_proj" in name:
            half = param.shape[0] // 2
            self._load(name.replace("gate_up_proj", "gate_proj"), param[:half], dtype)
            self._load(name.replace("gate_up_proj", "up_proj"), param[half:], dtype)
        elif "qkv_proj" in name:
            nq = cfg.num_attention_heads * cfg.head_dim
            nk = cfg.num_key_value_heads * cfg.head_dim
            self._load(name.replace("qkv_proj", "q_proj"), param[:nq], dtype)
            self._load(name.replace("qkv_proj", "k_proj"), param[nq:nq + nk], dtype)
            self._load(name.replace("qkv_proj", "v_proj"), param[nq + nk:], dtype)
        else:
            param = param.contiguous().to(dtype)
            C.load_model(name, param.data_ptr())
        if "embed_tokens" in name and getattr(cfg, "tie_word_embeddings", False):
            self._load("lm_head.weight", param)

    def _load_from_ckpt(self, path, cls=None):
        index_suffixes = ["bin.index.json", "safetensors.index.json"]
        file_suffixes = ["bin", "safetensors", "pt"]
        found = None
        for suffix in index_suffixes + file_suffixes:
            files = glob.glob(os.path.join(path, f"*.{suffix}"))
            if len(files) > 1:
                raise ValueError(f"Multiple files with suffix {suffix} found in {path}")
            if len(files) == 1:
                found = files[0]
                break
        if found is None:
            raise ValueError(f"No supported checkpoint file found in {path}, supported suffixes: "
                             f"{index_suffixes + file_suffixes}")
        if found.endswith(".index.json"):
            with open(found, "r") as f:
                names = set(json.load(f)["weight_map"].values())
            file_list = [os.path.join(path, n) for n in names]
        else:
            file_list = [found]
        for file in file_list:
            print(f"load from {file}")
            if file.endswith(".safetensors"):
                from safetensors.torch import load_file
                ckpt = load_file(file)
            else:
                ckpt = torch.load(file, map_location="cpu")
            for name, param in ckpt.items():
                self._load(name, param, cls=cls)

    def _rope_inv_freq(self):
        cfg = self.config
        scaling = getattr(cfg, "rope_scaling", None)
        rope_type = (scaling.get("rope_type", scaling.get("type")) if scaling else None) or "default"
        if rope_type != "default":
            # "llama3", or "longrope" with long_factor == short_factor, as in the reference (cpmcu/llm.py:176-186)
            from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
            inv_freq, _ = ROPE_INIT_FUNCTIONS[rope_type](cfg, "cpu", seq_len=self.max_total_length)
            return inv_freq
        return default_rope_inv_freq(cfg)

    def load_from_hf(self):
        with torch.no_grad():
            self._load_from_ckpt(self.path)
            self._load("model.rotary_emb.inv_freq", self._rope_inv_freq(), dtype=torch.float32)

    def load_state_dict_tensors(self, tensors, cls=None):
        """Load weights from an in-memory {name: tensor} mapping (host or device tensors)."""
        with torch.no_grad():
            for name, param in tensors.items():
                self._load(name, param, cls=cls)
            if cls is None:
                self._load("model.rotary_emb.inv_freq", self._rope_inv_freq(), dtype=torch.float32)

    # ------------------------------------------------------------------ forward passes
    def prefill(self, input_ids, position_ids):
        assert input_ids.dtype == torch.int32
        total = input_ids.numel()
        if total > self.max_total_length:
            raise ValueError(f"Input token count ({total}) exceeds maximum supported length "
                             f"({self.max_total_length}) under current memory limit")
        start = time.time()
        flat_ids, flat_pos = input_ids.view(-1), position_ids.view(-1)
        for i in range(0, total, self.chunk_length):
            n = min(total - i, self.chunk_length)
            C.prefill(n, i, flat_ids[i:].data_ptr(), flat_pos[i:].data_ptr(), self.logits.data_ptr())
            if self._show_prefill_progress:
                done = i + n
                rate = done / max(time.time() - start, 1e-9)
                print(f"\rPrefilling: {100.0 * done / total:.1f}% ({done}/{total} tokens) @ {rate:.1f} tokens/s",
                      end="", flush=True)
        if self._show_prefill_progress:
            print()
        self._last_prefill_time = time.time() - start
        return self.logits[:1].clone()

    def decode(self, input_ids, position_ids, cache_length, mask_2d=None):
        assert input_ids.dtype == torch.int32
        assert position_ids.dtype == torch.int32
        assert cache_length.dtype == torch.int32
        n = input_ids.numel()
        if mask_2d is not None:
            assert n == mask_2d.shape[0]
        cache_length += n  # the kernels take the length including the new rows
        padded_length = (cache_length[0].item() + 127) // 128 * 128
        C.decode(n, padded_length, input_ids.data_ptr(), position_ids.data_ptr(), cache_length.data_ptr(),
                 mask_2d.data_ptr() if mask_2d is not None else 0, self.logits.data_ptr(), self.cuda_graph)
        cache_length -= n
        return self.logits[:n].clone()

    def _pick(self, logits):
        if self.temperature > 0.0:
            probs = F.softmax(logits.float() / self.temperature, dim=-1)
            return torch.multinomial(probs, num_samples=1, generator=self.generator).squeeze(-1)
        return logits.argmax(dim=-1)

    def _text(self, token):
        return self.tokenizer.decode([token], skip_special_tokens=False) if self.tokenizer is not None else ""

    def _text_after(self, prev_token, tokens):
        """Text of `tokens` as it reads after `prev_token` (the reference decodes with one token of context)."""
        if self.tokenizer is None:
            return ""
        both = self.tokenizer.decode([prev_token] + list(tokens), skip_special_tokens=False)
        return both[len(self.tokenizer.decode([prev_token], skip_special_tokens=False)):]

    def generate(self, input_ids, generation_length=100, teminators=[], use_stream=False):
        """Greedy / sampled decoding without speculation.  Returns
        (tokens, decode_time, prefill_time), or a generator of dicts when use_stream."""
        assert input_ids.dtype == torch.int32
        prefix_length = input_ids.numel()
        if prefix_length + generation_length > self.max_total_length:
            raise ValueError(f"prompt ({prefix_length}) + generation_length ({generation_length}) exceeds the "
                             f"{self.max_total_length} tokens the KV cache holds under the current memory limit")
        position_ids = torch.arange(prefix_length, dtype=torch.int32, device="cuda")
        self._show_prefill_progress = bool(use_stream)
        torch.cuda.synchronize()
        t0 = time.time()
        logits = self.prefill(input_ids, position_ids)
        torch.cuda.synchronize()
        prefill_time = time.time() - t0
        token = self._pick(logits[0]).item()
        if not hasattr(self, "input_ids"):
            self.input_ids = torch.tensor([0], dtype=torch.int32, device="cuda")
            self.position_ids = torch.tensor([0], dtype=torch.int32, device="cuda")
            self.cache_length = torch.tensor([0], dtype=torch.int32, device="cuda")

        def steps():
            nonlocal token
            for i in range(generation_length - 1):
                self.input_ids[0] = token
                self.position_ids[0] = prefix_length + i
                self.cache_length[0] = prefix_length + i
                logits = self.decode(self.input_ids, self.position_ids, self.cache_length)
                token = self._pick(logits[0]).item()
                yield token

        if use_stream:
            # the reference's stream (cpmcu/llm.py:334-397): each token's text is decoded with the previous token as
            # context (correct spacing); decode_time counts from after the first token, which comes from prefill
            def stream():
                done = token in teminators
                yield {"token": token, "text": self._text(token), "is_finished": done or generation_length == 1,
                       "prefill_time": prefill_time, "decode_time": 0.0}
                if done:
                    return
                start = time.time()
                produced, prev = 1, token
                for tok in steps():
                    produced += 1
                    done = tok in teminators or produced == generation_length
                    yield {"token": tok, "text": self._text_after(prev, [tok]), "is_finished": done, "prefill_time": 0.0,
                           "decode_time": time.time() - start}
                    if done:
                        return
                    prev = tok
            return stream()

        tokens = [token]
        torch.cuda.synchronize()
        t0 = time.time()
        if token not in teminators:
            for tok in steps():
                tokens.append(tok)
                if tok in teminators:
                    break
        torch.cuda.synchronize()
        return tokens, time.time() - t0, prefill_time

    def print_perf_summary(self):
        C.print_perf_summary()
