"""Writes a synthetic checkpoint in the on-disk form the reference loads: a Hugging Face style directory for
the target (config.json, a tokenizer, safetensors shards with an index) and one for the EAGLE drafter
(config.json + one safetensors file).  Both the reference's classes (`load_from_hf`, cpmcu/llm.py:136-187 and
cpmcu/speculative/tree_drafter.py:49-66) and this repository's classes read these directories, so one set of
files feeds both arms of a comparison.

BENCHMARK / TEST INFRASTRUCTURE: used by bench.py's reference-CUDA arm and by the drop-in tests; the library
itself never imports it.
"""
import json
import os

import torch

SHARD_BYTES = 2 << 30


def write_tokenizer(path, vocab_size):
    """A word-level tokenizer with `vocab_size` made-up entries: the reference constructor insists on loading
    one (AutoTokenizer.from_pretrained, cpmcu/llm.py:43); token ids are fed directly, so its content is never
    used for the measurements."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    vocab = {"<unk>": 0}
    for i in range(1, vocab_size):
        vocab["t%d" % i] = i
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "<unk>"}, f)


def base_config(vocab, layers, hidden, inter, hq, hkv, head_dim=128, eps=1e-5, rope_theta=10000.0, extra=None):
    cfg = {"model_type": "llama", "architectures": ["LlamaForCausalLM"], "vocab_size": vocab, "hidden_size": hidden,
           "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": hq,
           "num_key_value_heads": hkv, "head_dim": head_dim, "rms_norm_eps": eps, "rope_theta": rope_theta,
           "torch_dtype": "bfloat16", "max_position_embeddings": 1 << 20, "tie_word_embeddings": False}
    cfg.update(extra or {})
    return cfg


class ShardWriter:
    """Collects (name, tensor) pairs and writes safetensors shards of about SHARD_BYTES each plus
    model.safetensors.index.json (one plain model.safetensors when everything fits in one shard)."""

    def __init__(self, path):
        self.path, self.cur, self.cur_bytes, self.shards, self.index = path, {}, 0, [], {}
        os.makedirs(path, exist_ok=True)

    def add(self, name, tensor):
        t = tensor.detach().to("cpu").contiguous()
        self.cur[name] = t
        self.cur_bytes += t.numel() * t.element_size()
        if self.cur_bytes >= SHARD_BYTES:
            self._flush()

    def _flush(self):
        from safetensors.torch import save_file
        if not self.cur:
            return
        fname = "model-%05d.safetensors" % (len(self.shards) + 1)
        save_file(self.cur, os.path.join(self.path, fname))
        for k in self.cur:
            self.index[k] = fname
        self.shards.append(fname)
        self.cur, self.cur_bytes = {}, 0

    def close(self):
        self._flush()
        if len(self.shards) == 1:
            os.rename(os.path.join(self.path, self.shards[0]), os.path.join(self.path, "model.safetensors"))
        else:
            with open(os.path.join(self.path, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {}, "weight_map": self.index}, f)


def write_checkpoint(base_dir, eagle_dir, config, tensors, eagle_tensors, eagle_config=None):
    """config: dict for the target's config.json; tensors / eagle_tensors: iterables of (name, tensor) with the
    reference's checkpoint names (the drafter's without the `eagle.` prefix: fc.weight, fc.bias, layers.0.*,
    input_norm1/2.weight, token_id_remap)."""
    os.makedirs(base_dir, exist_ok=True)
    with open(os.path.join(base_dir, "config.json"), "w") as f:
        json.dump(config, f)
    write_tokenizer(base_dir, min(int(config["vocab_size"]), 2048))
    w = ShardWriter(base_dir)
    for name, t in tensors:
        w.add(name, t)
    w.close()
    if eagle_dir is not None:
        os.makedirs(eagle_dir, exist_ok=True)
        ecfg = {"num_hidden_layers": 1}
        for key in ("scale_depth", "dim_model_base", "scale_emb"):
            if key in config:
                ecfg[key] = config[key]
        ecfg.update(eagle_config or {})
        with open(os.path.join(eagle_dir, "config.json"), "w") as f:
            json.dump(ecfg, f)
        ew = ShardWriter(eagle_dir)
        for name, t in eagle_tensors:
            ew.add(name, t)
        ew.close()
