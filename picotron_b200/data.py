"""Micro-batch data loading.

``MicroBatchDataLoader`` keeps the loader protocol the training loops and pipeline schedules
rely on (picotron/data.py:14-144): attributes ``micro_batch_size, seq_length, grad_acc_steps,
global_batch_size, num_global_micro_batches, seq_length_per_gpu`` and an endless iterator of
batches ``{"input_ids", "target_ids", "position_ids", "hidden_states"}`` where

* every rank with the same data-parallel coordinate sees the same samples
  (``DistributedSampler(num_replicas=dp, rank=dp_rank, shuffle=False)``, data.py:59-64), and
* a context-parallel rank receives its contiguous slice ``[cp_rank*s/cp, (cp_rank+1)*s/cp)`` of
  inputs, shifted-by-one targets and position ids (data.py:112-123).

``dataset_name="synthetic"`` produces seeded uniform token ids without any download — what the
benchmarks and tests use; any other name goes through Hugging Face ``datasets`` + a tokenizer
and packs documents into ``seq_length + 1`` token samples like the reference.

Batches are assembled in pinned host memory so the copy to the device is asynchronous.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import process_group_manager as pgm


class SyntheticTokens:
    """``num_samples`` rows of ``seq_length + 1`` token ids, uniform in [0, vocab), from a seed.
    Row i is a pure function of (seed, i), so any rank can materialise any sample."""

    def __init__(self, num_samples: int, seq_length: int, vocab_size: int, seed: int = 0):
        self.num_samples, self.seq_length, self.vocab_size, self.seed = num_samples, seq_length, vocab_size, seed

    def __len__(self):
        return self.num_samples

    def rows(self, indices) -> torch.Tensor:
        out = torch.empty((len(indices), self.seq_length + 1), dtype=torch.int64)
        g = torch.Generator()
        for j, i in enumerate(indices):
            g.manual_seed(self.seed * 1_000_003 + int(i))
            out[j] = torch.randint(0, self.vocab_size, (self.seq_length + 1,), generator=g)
        return out


class MicroBatchDataLoader:
    def __init__(self, micro_batch_size: int, seq_length: int, dataset_name: str = "synthetic",
                 tokenizer_name: Optional[str] = None, num_workers: int = 0, num_proc: int = 1,
                 grad_acc_steps: int = 1, device: str = "cpu", subset_name: Optional[str] = None,
                 split: str = "train", num_samples: Optional[int] = None, pin_memory: bool = True,
                 vocab_size: Optional[int] = None, seed: int = 0, dp_world_size: Optional[int] = None,
                 dp_rank: Optional[int] = None, cp_world_size: Optional[int] = None, cp_rank: Optional[int] = None,
                 cp_zigzag: bool = False):
        m = pgm.get_pgm()
        self.dp_world_size = dp_world_size if dp_world_size is not None else m.dp_world_size
        self.dp_rank = dp_rank if dp_rank is not None else m.dp_rank
        self.cp_world_size = cp_world_size if cp_world_size is not None else m.cp_world_size
        self.cp_rank = cp_rank if cp_rank is not None else m.cp_rank
        self.micro_batch_size = micro_batch_size
        self.tokenizer_name = tokenizer_name
        #: zigzag context parallelism: this rank's tokens are chunks r and 2*cp-1-r of the sequence
        self.cp_zigzag = bool(cp_zigzag) and self.cp_world_size > 1
        self.seq_length = seq_length
        self.grad_acc_steps = grad_acc_steps
        self.global_batch_size = micro_batch_size * grad_acc_steps * self.dp_world_size
        self.num_global_micro_batches = self.global_batch_size // micro_batch_size
        assert seq_length % self.cp_world_size == 0, "seq_length must be divisible by the CP size"
        self.seq_length_per_gpu = seq_length // self.cp_world_size
        self.pin_memory = pin_memory and torch.cuda.is_available()
        if dataset_name == "synthetic":
            assert vocab_size is not None, "synthetic data needs vocab_size"
            n = num_samples if num_samples is not None else 1 << 20
            self.dataset = SyntheticTokens(n, seq_length, vocab_size, seed)
        else:
            self.dataset = _HFPackedDataset(dataset_name, tokenizer_name, seq_length, subset_name, split,
                                            num_samples, num_proc)
        self.epoch = 0
        self._cursor = 0
        # DistributedSampler(shuffle=False) order: rank r takes indices r, r+dp, r+2dp, ...
        self._per_rank = len(self.dataset) // self.dp_world_size
        assert self._per_rank >= micro_batch_size, "dataset too small for one micro-batch per DP rank"

    # -- state for checkpoint/resume -------------------------------------------------------
    def state_dict(self):
        return {"epoch": self.epoch, "cursor": self._cursor}

    def load_state_dict(self, sd):
        self.epoch, self._cursor = sd["epoch"], sd["cursor"]

    def __iter__(self):
        return self

    def _next_indices(self):
        if self._cursor + self.micro_batch_size > self._per_rank:
            self.epoch += 1
            self._cursor = 0
        idx = [self.dp_rank + (self._cursor + j) * self.dp_world_size for j in range(self.micro_batch_size)]
        self._cursor += self.micro_batch_size
        return idx

    def collate(self, rows: torch.Tensor):
        """rows: [mbs, seq+1] -> this CP rank's slice of inputs / targets / positions."""
        if self.cp_zigzag:
            h = self.seq_length_per_gpu // 2
            starts = (self.cp_rank * h, (2 * self.cp_world_size - 1 - self.cp_rank) * h)
            input_ids = torch.cat([rows[:, s0:s0 + h] for s0 in starts], dim=1).contiguous()
            target_ids = torch.cat([rows[:, s0 + 1:s0 + h + 1] for s0 in starts], dim=1).contiguous()
            position_ids = torch.cat([torch.arange(s0, s0 + h, dtype=torch.long) for s0 in starts]) \
                .unsqueeze(0).expand(rows.shape[0], -1).contiguous()
        else:
            lo = self.cp_rank * self.seq_length_per_gpu
            hi = lo + self.seq_length_per_gpu
            input_ids = rows[:, lo:hi].contiguous()
            target_ids = rows[:, lo + 1:hi + 1].contiguous()
            position_ids = torch.arange(lo, hi, dtype=torch.long).unsqueeze(0).expand(rows.shape[0], -1).contiguous()
        if self.pin_memory:
            input_ids, target_ids, position_ids = (t.pin_memory() for t in (input_ids, target_ids, position_ids))
        return {"input_ids": input_ids, "target_ids": target_ids, "position_ids": position_ids,
                "hidden_states": None}

    def __next__(self):
        return self.collate(self.dataset.rows(self._next_indices()))

    # -- the reference's method names (picotron/data.py:76-123) -------------------------------------
    def collate_batch(self, batch):
        """``batch``: a list of ``{"input_ids": seq+1 tokens}`` items, as a ``torch`` ``DataLoader`` hands
        them to its ``collate_fn``."""
        return self.collate(torch.stack([torch.as_tensor(item["input_ids"]) for item in batch]))

    @staticmethod
    def tokenizer_group_text(examples, tokenizer, sequence_length: int):
        """Tokenise a list of texts, concatenate the tokens and cut them into rows of ``sequence_length + 1``
        tokens that start every ``sequence_length`` tokens (neighbouring rows share one token: the last
        target of a row is the first input of the next)."""
        encoded = tokenizer.batch_encode_plus(examples, return_attention_mask=False, return_token_type_ids=False)
        tokens = [t for doc in encoded["input_ids"] for t in doc]
        rows = max(0, (len(tokens) - 1) // sequence_length)
        return {"input_ids": [tokens[r * sequence_length:(r + 1) * sequence_length + 1] for r in range(rows)]}

    def tokenize_dataset(self, dataset, text_column_name: str, sequence_length: int, num_proc: int):
        """``dataset.map`` of ``tokenizer_group_text`` over the text column of a Hugging Face dataset."""
        from functools import partial
        tokenizer = getattr(self, "tokenizer", None)
        if tokenizer is None:
            from transformers import AutoTokenizer
            tokenizer = self.tokenizer = AutoTokenizer.from_pretrained(self.tokenizer_name)
        return dataset.map(partial(self.tokenizer_group_text, tokenizer=tokenizer, sequence_length=sequence_length),
                           input_columns=text_column_name, remove_columns=dataset.column_names, batched=True,
                           num_proc=num_proc, desc=f"Grouping texts in chunks of {sequence_length + 1}")


class _HFPackedDataset:
    """Tokenise a Hugging Face text dataset and pack it into seq+1 token rows (data.py:76-110)."""

    def __init__(self, name, tokenizer_name, seq_length, subset_name, split, num_samples, num_proc):
        from datasets import load_dataset
        from transformers import AutoTokenizer
        ds = load_dataset(name, subset_name, split=split)
        if num_samples:
            ds = ds.select(range(min(num_samples, len(ds))))
        tok = AutoTokenizer.from_pretrained(tokenizer_name)
        chunk = seq_length + 1

        def pack(batch):
            ids = [t for doc in tok(batch["text"])["input_ids"] for t in doc]
            n = len(ids) // chunk * chunk
            return {"input_ids": [ids[i:i + chunk] for i in range(0, n, chunk)]}

        self.ds = ds.map(pack, batched=True, remove_columns=ds.column_names, num_proc=num_proc)
        self.ds.set_format(type="torch", columns=["input_ids"])

    def __len__(self):
        return len(self.ds)

    def rows(self, indices):
        return torch.stack([self.ds[int(i)]["input_ids"] for i in indices])
