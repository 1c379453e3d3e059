"""`LLM_with_tree_drafter`: the reference's tree speculative-decoding loop
(cpmcu/speculative/tree_drafter.py:27-254) over the B200 library.

`generate` keeps the reference contract: (tokens, accept_lengths, decode_time,
prefill_time) or, with use_stream, a generator of dicts.  Two loop bodies give
the same tokens:
  * the reference's three calls per step, C.draft -> C.decode -> argmax ->
    C.verify_and_fix, on tensors owned here (`fused_step=False`);
  * one captured CUDA graph per step, C.spec_step(), with the tree and the
    cache length living on the device (`fused_step=True`, the default for
    greedy decoding).
"""
import time

import torch

from .. import C
from ..llm import LLM


def pack_mask(mask_2d):
    """Pack a boolean lower-triangular [T, T] mask into one uint64 per row
    (bit j of word i = row i may attend tree node j)."""
    rows = mask_2d.shape[0]
    words = []
    for i in range(rows):
        w = 0
        for j in range(i + 1):
            if int(mask_2d[i][j]):
                w |= 1 << j
        words.append(w)
    packed = torch.tensor([[w & 0xFFFFFFFF, w >> 32] for w in words], dtype=torch.int64).to(torch.uint32)
    return packed.to("cuda").view(torch.uint64).view(-1)


class LLM_with_tree_drafter(LLM):
    def __init__(self, drafter_type, drafter_path, base_path, tree_size, use_rope=False, fused_step=True, **kwargs):
        super().__init__(base_path, **kwargs)
        self.drafter_type = drafter_type
        self.drafter_path = drafter_path
        self.base_path = base_path
        self.use_rope = use_rope
        self.fused_step = fused_step
        self.tree_size = tree_size
        self.tree_draft_ids = torch.empty((tree_size,), dtype=torch.int32, device="cuda")
        self.tree_position_ids = torch.empty((tree_size,), dtype=torch.int32, device="cuda")
        self.tree_gt_ids = torch.empty((tree_size,), dtype=torch.int32, device="cuda")
        self.tree_attn_mask = torch.empty((tree_size,), dtype=torch.uint64, device="cuda")
        self.tree_parent = torch.empty((tree_size,), dtype=torch.int32, device="cuda")
        self.cache_length = torch.tensor([0], dtype=torch.int32, device="cuda")

    def load_from_hf(self):
        with torch.no_grad():
            self._load_from_ckpt(self.drafter_path, cls=self.drafter_type)
            if self.use_rope:
                self._load(f"{self.drafter_type}.rotary_emb.inv_freq", self._rope_inv_freq(), dtype=torch.float32)
            super().load_from_hf()

    # ------------------------------------------------------------------ one step, two ways
    def _step_reference_calls(self, prefix_length, i):
        """draft -> target forward -> argmax -> verify_and_fix, as the reference loop does."""
        self.cache_length[0] = prefix_length + i
        C.draft(self.tree_draft_ids.data_ptr(), self.tree_position_ids.data_ptr(), self.cache_length.data_ptr(),
                self.tree_attn_mask.data_ptr(), self.tree_parent.data_ptr())
        logits = self.decode(self.tree_draft_ids, self.tree_position_ids, self.cache_length,
                             mask_2d=self.tree_attn_mask)
        self.tree_gt_ids.copy_(self._pick(logits))
        n = C.verify_and_fix(self.tree_draft_ids.numel(), self.tree_draft_ids.data_ptr(), self.tree_gt_ids.data_ptr(),
                             self.tree_position_ids.data_ptr(), self.cache_length.data_ptr(),
                             self.tree_attn_mask.data_ptr(), self.tree_parent.data_ptr())
        emitted = self.tree_draft_ids[:n].tolist()
        self.tree_draft_ids[0] = self.tree_draft_ids[n - 1]
        return emitted

    def _step_fused(self):
        return C.spec_step(16)

    def generate(self, input_ids, generation_length=100, teminators=[], use_stream=False):
        assert input_ids.dtype == torch.int32
        prefix_length = input_ids.numel()
        if prefix_length > self.max_total_length:
            raise ValueError(f"Input token count ({prefix_length}) exceeds maximum supported length "
                             f"({self.max_total_length}) under current memory limit")
        # every step writes the K/V rows of a whole tree behind the accepted tokens
        if prefix_length + generation_length + self.tree_size > self.max_total_length:
            raise ValueError(f"prompt ({prefix_length}) + generation_length ({generation_length}) + one draft tree "
                             f"({self.tree_size}) exceeds the {self.max_total_length} tokens the KV cache holds "
                             f"under the current memory limit")
        position_ids = torch.arange(prefix_length, dtype=torch.int32, device="cuda")
        self._show_prefill_progress = bool(use_stream)
        torch.cuda.synchronize()
        t0 = time.time()
        logits = self.prefill(input_ids, position_ids)
        torch.cuda.synchronize()
        prefill_time = time.time() - t0
        fused = self.fused_step
        if fused and self.temperature > 0.0:
            # device-side sampling inside the captured step; the whole run is a function of the seed
            seed = self.sample_seed if self.sample_seed is not None else int.from_bytes(__import__("os").urandom(8), "little")
            C.set_sampling(self.temperature, seed)
            root_t = torch.empty(1, dtype=torch.int32, device="cuda")
            C.sample(logits.data_ptr(), 1, logits.shape[-1], self.temperature, seed, 0, root_t.data_ptr())
            root = int(root_t.item())
        else:
            if fused:
                C.set_sampling(0.0, 0)
            root = self._pick(logits[0]).item()
        self.tree_draft_ids[0] = root
        if fused:
            C.begin_generation(prefix_length, root)
        self.step_device_ms = []

        def steps():
            i = 0
            while i < generation_length - 1:
                emitted = self._step_fused() if fused else self._step_reference_calls(prefix_length, i)
                if fused:
                    self.step_device_ms.append(C.last_step_ms())
                yield emitted, i
                i += len(emitted)

        if use_stream:
            # The reference's stream (cpmcu/speculative/tree_drafter.py:117-212): one dict per token; the text of a
            # step's tokens is decoded together with the previous token for correct spacing and handed to the
            # step's first token, which alone carries the step's accept_length; its last token carries decode_time.
            def stream():
                done = root in teminators
                yield {"token": root, "text": self._text(root), "is_finished": done, "accept_length": 1,
                       "prefill_time": prefill_time, "decode_time": 0.0}
                if done:
                    return
                start = time.time()
                prev = root
                for emitted, i in steps():
                    n = len(emitted)
                    new_text = self._text_after(prev, emitted)
                    for j, tok in enumerate(emitted):
                        if i + j >= generation_length - 1:
                            break
                        terminal = tok in teminators
                        yield {"token": tok, "text": new_text if j == 0 else "",
                               "is_finished": terminal or (i + j == generation_length - 2),
                               "accept_length": n if j == 0 else 0, "prefill_time": 0.0,
                               "decode_time": time.time() - start if j == n - 1 else 0.0}
                        if terminal:
                            return
                    prev = emitted[-1]
            return stream()

        tokens = [root]
        accept_lengths = []
        torch.cuda.synchronize()
        t0 = time.time()
        for emitted, i in steps():
            accept_lengths.append(len(emitted))
            tokens.extend(emitted[: generation_length - 1 - i])
            if any(t in teminators for t in emitted):
                break
        torch.cuda.synchronize()
        decode_time = time.time() - t0
        return tokens, accept_lengths, decode_time, prefill_time
