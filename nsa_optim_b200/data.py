"""Data sources: seeded synthetic tokens and the streaming packer.

Reference behaviour (nngabe/nsa_optim, data.py): DataConfig :17-28, TokenizedDataset :31-110,
PackedDataset :113-287 (BOS + tokens + EOS per document, greedy packing to
``max_seq_length``, ``-100`` labels on padding, per-rank shuffle seed ``seed + rank``),
create_dataloader :290-329 (collate drops ``doc_boundaries``), get_tokenizer :332-351.

Additions: :class:`SyntheticTokens` (uniform random ids; the benchmark workload), a
resumable position counter on every source, and injectable dataset / tokenizer objects so
the packer is testable without network access.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional

import torch
from torch.utils.data import DataLoader, IterableDataset


@dataclass
class DataConfig:
    dataset_name: str = "HuggingFaceFW/fineweb-edu"
    dataset_subset: str = "sample-10BT"
    tokenizer_name: str = "Qwen/Qwen3-0.6B"
    max_seq_length: int = 32768
    num_workers: int = 0
    shuffle_buffer_size: int = 10000
    seed: int = 42
    text_column: str = "text"
    pack_sequences: bool = True


class SyntheticTokens(IterableDataset):
    """Endless stream of ``(batch, seq)`` uniform-random token ids.  Batch ``i`` of rank ``r``
    depends only on ``(seed, r, i)``, so a resumed run sees the same stream."""

    def __init__(self, vocab_size: int, seq_length: int, batch_size: int = 1, seed: int = 0,
                 rank: int = 0, pin_memory: bool = False):
        self.vocab_size, self.seq_length, self.batch_size = vocab_size, seq_length, batch_size
        self.seed, self.rank, self.position = seed, rank, 0
        self.pin_memory = pin_memory and torch.cuda.is_available()

    def batch_at(self, index: int) -> Dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed((self.seed * 1_000_003 + self.rank) * 1_000_033 + index)
        ids = torch.randint(0, self.vocab_size, (self.batch_size, self.seq_length), generator=g)
        if self.pin_memory:
            ids = ids.pin_memory()
        return {"input_ids": ids, "attention_mask": torch.ones_like(ids), "labels": ids}

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        while True:
            b = self.batch_at(self.position)
            self.position += 1
            yield b

    def state_dict(self) -> Dict[str, int]:
        return {"position": self.position}

    def load_state_dict(self, st: Dict[str, int]) -> None:
        self.position = int(st.get("position", 0))


def _load_stream(cfg: DataConfig, split: str, seed: int):
    from datasets import load_dataset  # imported lazily: needs network or a local cache
    ds = load_dataset(cfg.dataset_name, cfg.dataset_subset, split=split, streaming=True)
    return ds.shuffle(seed=seed, buffer_size=cfg.shuffle_buffer_size)


class TokenizedDataset(IterableDataset):
    """One truncated/padded document per example (no packing)."""

    def __init__(self, config: DataConfig, tokenizer, split: str = "train", rank: int = 0,
                 world_size: int = 1, dataset: Optional[Iterable[Dict[str, Any]]] = None):
        self.config, self.tokenizer, self.split = config, tokenizer, split
        self.rank, self.world_size = rank, world_size
        self._dataset = dataset

    def __iter__(self):
        ds = self._dataset if self._dataset is not None else _load_stream(
            self.config, self.split, self.config.seed + self.rank)
        L = self.config.max_seq_length
        pad = self.tokenizer.pad_token_id if self.tokenizer.pad_token_id is not None else 0
        for ex in ds:
            ids = self.tokenizer.encode(ex[self.config.text_column], add_special_tokens=True)[:L]
            n = len(ids)
            ids = ids + [pad] * (L - n)
            labels = ids[:n] + [-100] * (L - n)
            yield {"input_ids": torch.tensor(ids), "attention_mask": torch.tensor([1] * n + [0] * (L - n)),
                   "labels": torch.tensor(labels)}


class PackedDataset(IterableDataset):
    """Greedy sequence packing: documents are wrapped in BOS/EOS and concatenated until the
    next one would overflow ``max_seq_length``; over-long documents are truncated; the tail is
    padded with ``-100`` labels.  ``doc_boundaries`` lists the start offset of each document."""

    def __init__(self, config: DataConfig, tokenizer, split: str = "train", rank: int = 0,
                 world_size: int = 1, dataset: Optional[Iterable[Dict[str, Any]]] = None):
        self.config, self.tokenizer, self.split = config, tokenizer, split
        self.rank, self.world_size = rank, world_size
        self._dataset = dataset
        self.documents_consumed = 0

    def _special(self, name: str) -> Optional[int]:
        return getattr(self.tokenizer, name, None)

    def _doc_tokens(self, text: str) -> List[int]:
        ids = list(self.tokenizer.encode(text, add_special_tokens=False))
        bos, eos = self._special("bos_token_id"), self._special("eos_token_id")
        if bos is not None:
            ids = [bos] + ids
        if eos is not None:
            ids = ids + [eos]
        return ids

    def _emit(self, buf: List[int], bounds: List[int]) -> Dict[str, torch.Tensor]:
        L = self.config.max_seq_length
        n = len(buf)
        pad = self._special("pad_token_id")
        pad = 0 if pad is None else pad
        ids = buf + [pad] * (L - n)
        return {"input_ids": torch.tensor(ids, dtype=torch.long),
                "attention_mask": torch.tensor([1] * n + [0] * (L - n), dtype=torch.long),
                "labels": torch.tensor(buf + [-100] * (L - n), dtype=torch.long),
                "doc_boundaries": torch.tensor(bounds, dtype=torch.long)}

    def __iter__(self):
        if not self.config.pack_sequences:
            yield from TokenizedDataset(self.config, self.tokenizer, self.split, self.rank,
                                        self.world_size, self._dataset)
            return
        ds = self._dataset if self._dataset is not None else _load_stream(
            self.config, self.split, self.config.seed + self.rank)
        L = self.config.max_seq_length
        buf: List[int] = []
        bounds: List[int] = []
        for ex in ds:
            self.documents_consumed += 1
            toks = self._doc_tokens(ex[self.config.text_column])[:L]
            if not toks:
                continue
            if len(buf) + len(toks) > L:
                yield self._emit(buf, bounds)
                buf, bounds = [], []
            bounds.append(len(buf))
            buf.extend(toks)
            if len(buf) == L:
                yield self._emit(buf, bounds)
                buf, bounds = [], []
        if buf:
            yield self._emit(buf, bounds)


def collate_fn(batch: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """Stack the model inputs; ragged ``doc_boundaries`` are dropped."""
    return {k: torch.stack([b[k] for b in batch]) for k in ("input_ids", "attention_mask", "labels")}


def create_dataloader(config: DataConfig, tokenizer, batch_size: int, split: str = "train",
                      rank: int = 0, world_size: int = 1, dataset=None) -> DataLoader:
    ds = PackedDataset(config, tokenizer, split, rank, world_size, dataset)
    return DataLoader(ds, batch_size=batch_size, num_workers=config.num_workers,
                      pin_memory=torch.cuda.is_available(), collate_fn=collate_fn)


def create_synthetic_loader(vocab_size: int, seq_length: int, batch_size: int, seed: int = 0,
                            rank: int = 0, pin_memory: bool = False) -> SyntheticTokens:
    return SyntheticTokens(vocab_size, seq_length, batch_size, seed, rank, pin_memory)


def get_tokenizer(tokenizer_path: str):
    """Hugging Face tokenizer; a missing pad token falls back to EOS."""
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(tokenizer_path, trust_remote_code=True)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    return tok
