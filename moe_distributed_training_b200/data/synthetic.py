"""Synthetic instruction-shaped data.

Sequence lengths uniform in [min_len, max_len], token ids uniform over the
vocabulary, the first `prompt_frac` of every sequence label-masked (the prompt of
an instruction example).  One sequence per micro-batch per rank, as in the
reference's default `per_device_train_batch_size=1` (train_accelerate_fsdp2.py:52).
"""
from __future__ import annotations

from typing import Iterator, List

import torch

from .collator import IGNORE_INDEX


class SyntheticInstructionDataset:
    def __init__(self, vocab_size: int, num_examples: int, min_len: int = 128, max_len: int = 1024,
                 prompt_frac: float = 0.4, seed: int = 0, rank: int = 0, fixed_len: int = 0):
        g = torch.Generator().manual_seed(seed * 7919 + rank)
        self.examples: List[dict] = []
        for _ in range(num_examples):
            n = fixed_len or int(torch.randint(min_len, max_len + 1, (1,), generator=g))
            ids = torch.randint(0, vocab_size, (n,), generator=g)
            labels = ids.clone()
            labels[: int(prompt_frac * n)] = IGNORE_INDEX
            self.examples.append({"input_ids": ids, "labels": labels})

    def __len__(self):
        return len(self.examples)

    def __getitem__(self, i):
        return self.examples[i]

    def num_tokens(self) -> int:
        return sum(int(e["input_ids"].numel()) for e in self.examples)


def collate_packed(examples: List[dict]) -> dict:
    """Concatenate examples into one packed stream with cu_seqlens."""
    ids = torch.cat([e["input_ids"] for e in examples])
    labels = torch.cat([e["labels"] for e in examples])
    lens = torch.tensor([0] + [int(e["input_ids"].numel()) for e in examples])
    return {"input_ids": ids, "labels": labels, "cu_seqlens": torch.cumsum(lens, 0).int(),
            "max_seqlen": int(lens.max())}


def batches(ds: SyntheticInstructionDataset, batch_size: int) -> Iterator[dict]:
    for i in range(0, len(ds) - batch_size + 1, batch_size):
        yield collate_packed([ds[j] for j in range(i, i + batch_size)])
