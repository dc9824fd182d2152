"""Completion-only collation: prompt tokens get label -100.

The reference uses `trl.DataCollatorForCompletionOnlyLM(response_template=...)`
(train_accelerate_fsdp2.py:98-110): labels equal input_ids, and everything up to
and including the response template is masked.  Sequences are right-padded to
the longest in the batch.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

IGNORE_INDEX = -100


def find_subsequence(seq: Sequence[int], pat: Sequence[int]) -> int:
    n, m = len(seq), len(pat)
    for i in range(n - m + 1):
        if list(seq[i:i + m]) == list(pat):
            return i
    return -1


class DataCollatorForCompletionOnlyLM:
    def __init__(self, response_template_ids: Sequence[int], pad_token_id: int = 0, ignore_index: int = IGNORE_INDEX):
        self.template = list(response_template_ids)
        self.pad, self.ignore = pad_token_id, ignore_index

    def __call__(self, examples: List[dict]) -> dict:
        L = max(len(e["input_ids"]) for e in examples)
        ids = torch.full((len(examples), L), self.pad, dtype=torch.long)
        labels = torch.full((len(examples), L), self.ignore, dtype=torch.long)
        mask = torch.zeros((len(examples), L), dtype=torch.long)
        for i, e in enumerate(examples):
            x = list(e["input_ids"])
            ids[i, :len(x)] = torch.tensor(x)
            mask[i, :len(x)] = 1
            at = find_subsequence(x, self.template)
            if at < 0:
                continue  # template missing: the whole example is ignored, as trl does
            start = at + len(self.template)
            labels[i, start:len(x)] = torch.tensor(x[start:])
        return {"input_ids": ids, "labels": labels, "attention_mask": mask}
