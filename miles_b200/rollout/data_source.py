"""Prompt datasets and the rollout data source with a buffer for partial samples.

`DataSource` is the abstract contract (reference: miles/rollout/data_source.py:21-48);
`RolloutDataSource` reads JSONL / parquet prompts, applies the chat template, hands out groups of
`n_samples_per_prompt` deep copies, and saves/loads its epoch/offset state to
`<save>/rollout/global_dataset_state_dict_{rollout_id}.pt` (reference :52-231 and
miles/utils/data.py:33-277).  `SyntheticPromptSource` produces random token prompts for benchmarks.
"""
from __future__ import annotations

import abc
import copy
import json
import os
import random
from typing import Any, Callable

import torch

from ..types import Sample
from ..utils.misc import load_function


class DataSource(abc.ABC):
    @abc.abstractmethod
    def get_samples(self, num_groups: int) -> list[list[Sample]]: ...

    def add_samples(self, groups: list[list[Sample]]) -> None:
        raise NotImplementedError

    def save(self, rollout_id: int) -> None: ...

    def load(self, rollout_id: int | None = None) -> None: ...

    def __len__(self) -> int:
        return 0


def read_prompt_file(path: str) -> list[dict]:
    """`file.jsonl`, `file.json`, `file.parquet`; `path@[a:b]` selects a row slice."""
    sl = None
    if "@[" in path:
        path, rng = path.split("@[")
        a, b = rng.rstrip("]").split(":")
        sl = slice(int(a) if a else None, int(b) if b else None)
    if path.endswith(".parquet"):
        import pandas as pd

        rows = pd.read_parquet(path).to_dict("records")
    elif path.endswith(".jsonl"):
        with open(path) as f:
            rows = [json.loads(line) for line in f if line.strip()]
    else:
        with open(path) as f:
            rows = json.load(f)
    return rows[sl] if sl else rows


class Dataset:
    def __init__(self, path: str, tokenizer=None, *, input_key="input", label_key=None, metadata_key="metadata",
                 tool_key=None, apply_chat_template=False, apply_chat_template_kwargs=None, max_length=None,
                 seed=42):
        self.samples: list[Sample] = []
        for row in read_prompt_file(path):
            prompt = row[input_key]
            tools = row.get(tool_key) if tool_key else None
            if isinstance(tools, str):
                tools = json.loads(tools)
            if apply_chat_template and tokenizer is not None:
                msgs = prompt if isinstance(prompt, list) else [{"role": "user", "content": prompt}]
                prompt_text = tokenizer.apply_chat_template(msgs, tools=tools, tokenize=False, add_generation_prompt=True,
                                                            **(apply_chat_template_kwargs or {}))
            else:
                prompt_text = prompt
            if max_length is not None and tokenizer is not None and isinstance(prompt_text, str):
                if len(tokenizer(prompt_text, add_special_tokens=False)["input_ids"]) > max_length:
                    continue
            md = row.get(metadata_key) or {}
            if isinstance(md, str):
                md = json.loads(md)
            if tools is not None:
                md = {**md, "tools": tools}
            label = row.get(label_key) if label_key else None
            self.samples.append(Sample(prompt=prompt_text, label=None if label is None else str(label), metadata=md))
        self.seed = seed
        self.order = list(range(len(self.samples)))

    def shuffle(self, epoch: int):
        rng = random.Random(self.seed + epoch)
        self.order = list(range(len(self.samples)))
        rng.shuffle(self.order)

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i) -> Sample:
        return self.samples[self.order[i]]


class RolloutDataSource(DataSource):
    def __init__(self, args, tokenizer=None):
        self.args = args
        self.epoch_id = 0
        self.sample_group_index = 0
        self.sample_index = 0
        self.sample_offset = 0
        self.metadata: dict = {}
        self.tokenizer = tokenizer
        self.dataset = None
        if getattr(args, "prompt_data", None):
            self.dataset = Dataset(
                args.prompt_data, tokenizer, input_key=args.input_key, label_key=args.label_key,
                metadata_key=args.metadata_key, tool_key=args.tool_key, apply_chat_template=args.apply_chat_template,
                apply_chat_template_kwargs=args.apply_chat_template_kwargs, max_length=args.rollout_max_prompt_len,
                seed=args.rollout_seed)
            if args.rollout_shuffle:
                self.dataset.shuffle(self.epoch_id)

    def get_samples(self, num_groups: int) -> list[list[Sample]]:
        groups = []
        n = self.args.n_samples_per_prompt
        for _ in range(num_groups):
            if self.dataset is not None:
                if self.sample_offset >= len(self.dataset):
                    self.epoch_id += 1
                    self.sample_offset = 0
                    if self.args.rollout_shuffle:
                        self.dataset.shuffle(self.epoch_id)
                proto = self.dataset[self.sample_offset]
                self.sample_offset += 1
            else:
                proto = Sample()
            group = []
            for _ in range(n):
                s = copy.deepcopy(proto)
                s.group_index = self.sample_group_index
                s.index = self.sample_index
                self.sample_index += 1
                group.append(s)
            self.sample_group_index += 1
            groups.append(group)
        return groups

    def add_samples(self, groups):
        raise RuntimeError("RolloutDataSource has no buffer; use RolloutDataSourceWithBuffer")

    def _state_path(self, rollout_id):
        return os.path.join(self.args.save, "rollout", f"global_dataset_state_dict_{rollout_id}.pt")

    def state_dict(self) -> dict:
        return {"sample_offset": self.sample_offset, "epoch_id": self.epoch_id,
                "sample_group_index": self.sample_group_index, "sample_index": self.sample_index,
                "metadata": self.metadata}

    def load_state_dict(self, sd: dict):
        self.sample_offset = sd.get("sample_offset", 0)
        self.epoch_id = sd.get("epoch_id", 0)
        self.sample_group_index = sd.get("sample_group_index", 0)
        self.sample_index = sd.get("sample_index", 0)
        self.metadata = sd.get("metadata", {})
        if self.dataset is not None and self.args.rollout_shuffle:
            self.dataset.shuffle(self.epoch_id)

    def save(self, rollout_id):
        if not getattr(self.args, "save", None):
            return
        path = self._state_path(rollout_id)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        torch.save(self.state_dict(), path)

    def load(self, rollout_id=None):
        if not getattr(self.args, "load", None) or rollout_id is None:
            return
        path = os.path.join(self.args.load, "rollout", f"global_dataset_state_dict_{rollout_id}.pt")
        if os.path.exists(path):
            self.load_state_dict(torch.load(path, weights_only=False))

    def __len__(self):
        return len(self.dataset) if self.dataset is not None else 0


def pop_first(args, rollout_id, buffer: list[list[Sample]], num: int) -> list[list[Sample]]:
    out = buffer[:num]
    del buffer[:num]
    return out


class RolloutDataSourceWithBuffer(RolloutDataSource):
    """Adds a FIFO of partially generated groups (aborted by partial rollout) served before new prompts."""

    def __init__(self, args, tokenizer=None):
        super().__init__(args, tokenizer)
        self.buffer: list[list[Sample]] = []
        path = getattr(args, "buffer_filter_path", None)
        self.buffer_filter: Callable = load_function(path) if path else pop_first

    def get_samples(self, num_groups):
        out = self.buffer_filter(self.args, None, self.buffer, num_groups) if self.buffer else []
        if len(out) < num_groups:
            out += super().get_samples(num_groups - len(out))
        return out

    def add_samples(self, groups):
        for g in groups:
            assert isinstance(g, list) and len(g) == self.args.n_samples_per_prompt, "buffer takes whole groups"
        self.buffer.extend(groups)

    def state_dict(self):
        sd = super().state_dict()
        sd["buffer"] = [[s.to_dict() for s in g] for g in self.buffer]
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        self.buffer = [[Sample.from_dict(d) for d in g] for g in sd.get("buffer", [])]

    def buffer_length(self) -> int:
        return len(self.buffer)


class SyntheticPromptSource(RolloutDataSourceWithBuffer):
    """Random-token prompts: ids uniform in [low, vocab), lengths uniform in [min_len, max_len]."""

    def __init__(self, args, vocab_size: int, min_len: int, max_len: int, low: int = 3, seed: int = 0):
        super().__init__(args, None)
        self.vocab_size, self.min_len, self.max_len, self.low = vocab_size, min_len, max_len, low
        self.gen = torch.Generator().manual_seed(seed)

    def get_samples(self, num_groups):
        out = self.buffer_filter(self.args, None, self.buffer, num_groups) if self.buffer else []
        while len(out) < num_groups:
            L = int(torch.randint(self.min_len, self.max_len + 1, (1,), generator=self.gen))
            ids = torch.randint(self.low, self.vocab_size, (L,), generator=self.gen).tolist()
            group = []
            for _ in range(self.args.n_samples_per_prompt):
                s = Sample(group_index=self.sample_group_index, index=self.sample_index, tokens=list(ids), prompt=list(ids))
                self.sample_index += 1
                group.append(s)
            self.sample_group_index += 1
            out.append(group)
        return out


class SyntheticSource(SyntheticPromptSource):
    """`--data-source-path miles_b200.rollout.data_source.SyntheticSource`: random prompts sized from the model config
    and `--synthetic-prompt-len MIN MAX` (default 16 32); for smoke runs, tests and benchmarks without a dataset."""

    def __init__(self, args, tokenizer=None):
        from ..args import model_config_from_args

        lo, hi = (getattr(args, "synthetic_prompt_len", None) or (16, 32))
        super().__init__(args, model_config_from_args(args).vocab_size, int(lo), int(hi), seed=getattr(args, "seed", 0))
