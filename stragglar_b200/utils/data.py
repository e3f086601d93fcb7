"""Instruction-tuning data for the end-to-end run: records, prompt format, tokenizers, dataset.

The reference fine-tunes on the first 8192 examples of Alpaca, formatted as
``### Instruction: / ### Input: / ### Response:``, tokenized with the Llama tokenizer, truncated and padded to
512 tokens, batch 4 per rank behind a ``DistributedSampler`` (implementation/custom_backend/dp.py:87-119);
``motivation/load_dataset.py`` downloads the dataset beforehand.  This module provides the same pipeline without
requiring the network:

* :func:`load_records` reads a directory written by ``examples/load_dataset.py``: ``data.jsonl`` (one JSON object
  with ``instruction`` / ``input`` / ``output`` per line) or, when the Hugging Face ``datasets`` package is
  installed, a dataset saved with ``save_to_disk``;
* :func:`synthetic_records` makes Alpaca-shaped records from a seeded word list (what ``load_dataset.py`` writes when
  it cannot download);
* :class:`ByteTokenizer` (UTF-8 bytes plus BOS/EOS/PAD) stands in when no ``tokenizer.json`` is available;
  :func:`load_tokenizer` prefers a ``tokenizer.json`` found in the model directory;
* :class:`InstructionDataset` yields ``input_ids`` / ``attention_mask`` / ``labels`` (padding masked with -100, as
  ``DataCollatorForLanguageModeling(mlm=False)`` does).
"""
from __future__ import annotations

import json
import os
import random
from typing import Dict, Iterable, List, Optional, Sequence

import torch
from torch.utils.data import Dataset

Record = Dict[str, str]

_VERBS = ["Describe", "Explain", "List", "Summarize", "Compare", "Rewrite", "Classify", "Translate", "Generate", "Name"]
_TOPICS = ["the water cycle", "a binary search", "three primary colors", "the causes of inflation", "a healthy breakfast",
           "the rules of chess", "photosynthesis", "a ring network", "gradient descent", "the structure of an atom",
           "a collective operation", "the life of a star", "a persistent straggler", "tidal forces", "a haiku about rain"]
_WORDS = ("the of and to in is that it for as with was on be by this are or an from at which but not have they you "
          "one all can more when time some data model rank chunk sum wait round step send receive link fast slow "
          "light water energy number simple answer result because first then finally each every between after").split()


def format_example(ex: Record) -> str:
    """The prompt of the reference's ``format_example`` (dp.py:87-92)."""
    prompt = f"### Instruction:\n{ex['instruction']}\n\n"
    if ex.get("input"):
        prompt += f"### Input:\n{ex['input']}\n\n"
    return prompt + f"### Response:\n{ex['output']}"


def synthetic_records(n: int, seed: int = 0) -> List[Record]:
    """``n`` Alpaca-shaped records from a seeded generator (deterministic for a given ``n`` and ``seed``)."""
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        rec = {"instruction": f"{rng.choice(_VERBS)} {rng.choice(_TOPICS)}.", "input": "",
               "output": " ".join(rng.choice(_WORDS) for _ in range(rng.randint(12, 120))).capitalize() + "."}
        if rng.random() < 0.35:
            rec["input"] = " ".join(rng.choice(_WORDS) for _ in range(rng.randint(3, 25)))
        out.append(rec)
    return out


def save_records(records: Iterable[Record], directory: str) -> str:
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, "data.jsonl")
    with open(path, "w", encoding="utf-8") as f:
        for r in records:
            f.write(json.dumps({k: r.get(k, "") for k in ("instruction", "input", "output")}) + "\n")
    return path


def load_records(directory: str, limit: Optional[int] = None) -> List[Record]:
    """Records of a dataset directory (``data.jsonl``, else a Hugging Face dataset saved to disk)."""
    path = os.path.join(directory, "data.jsonl")
    if os.path.isfile(path):
        out = []
        with open(path, encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    out.append(json.loads(line))
                    if limit is not None and len(out) >= limit:
                        break
        return out
    if os.path.isdir(directory):
        try:
            from datasets import load_from_disk   # optional dependency
        except ImportError as e:
            raise FileNotFoundError(f"{directory} has no data.jsonl and the 'datasets' package is not installed") from e
        ds = load_from_disk(directory)
        if hasattr(ds, "keys") and "train" in ds:
            ds = ds["train"]
        n = len(ds) if limit is None else min(limit, len(ds))
        return [dict(ds[i]) for i in range(n)]
    raise FileNotFoundError(f"dataset directory {directory} not found")


class ByteTokenizer:
    """UTF-8 bytes as tokens: ids 0..255 are the bytes, then BOS, EOS, PAD.  Fits any vocabulary of >= 259 entries."""
    bos_id, eos_id, pad_id = 256, 257, 258
    vocab_size = 259

    def encode(self, text: str) -> List[int]:
        return [self.bos_id] + list(text.encode("utf-8")) + [self.eos_id]

    def decode(self, ids: Sequence[int]) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


class _HFTokenizer:
    """A ``tokenizer.json`` driven through the ``tokenizers`` package; EOS doubles as padding (dp.py:103)."""

    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size()
        eos = None
        for name in ("<|end_of_text|>", "</s>", "<|endoftext|>", "<eos>"):
            eos = self.tk.token_to_id(name)
            if eos is not None:
                break
        self.eos_id = self.pad_id = eos if eos is not None else 0
        self.bos_id = None

    def encode(self, text: str) -> List[int]:
        return self.tk.encode(text).ids

    def decode(self, ids: Sequence[int]) -> str:
        return self.tk.decode(list(ids))


def load_tokenizer(model_dir: Optional[str] = None):
    """The tokenizer of ``model_dir`` when it holds a ``tokenizer.json``, else the byte tokenizer."""
    if model_dir:
        path = os.path.join(model_dir, "tokenizer.json")
        if os.path.isfile(path):
            return _HFTokenizer(path)
    return ByteTokenizer()


class InstructionDataset(Dataset):
    """Records -> fixed-length ``input_ids`` / ``attention_mask`` / ``labels`` tensors (padding -> label -100)."""

    def __init__(self, records: Sequence[Record], tokenizer=None, max_length: int = 512):
        self.tok = tokenizer or ByteTokenizer()
        self.max_length = max_length
        ids = torch.full((len(records), max_length), self.tok.pad_id, dtype=torch.long)
        mask = torch.zeros((len(records), max_length), dtype=torch.long)
        for i, r in enumerate(records):
            t = self.tok.encode(format_example(r))[:max_length]
            ids[i, : len(t)] = torch.tensor(t, dtype=torch.long)
            mask[i, : len(t)] = 1
        self.input_ids, self.attention_mask = ids, mask

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int):
        ids, mask = self.input_ids[i], self.attention_mask[i]
        labels = ids.clone()
        labels[mask == 0] = -100
        return {"input_ids": ids, "attention_mask": mask, "labels": labels}
