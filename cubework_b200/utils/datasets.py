"""Real-data pipelines of the benchmark drivers (``--dataset_path`` / ``--tokenizer_path``).

Parity: benchmark/gpt2/gpt2.py:386-428 and benchmark/opt/opt.py:580-611 (a ``datasets`` directory saved with
``save_to_disk`` whose ``text`` column is tokenised, truncated and padded to the sequence length inside the collate
function, labels = input ids), benchmark/vit/vit.py:357-466 (CIFAR-10 with crop / flip / AutoAugment, resized to the
model's image size, mixed up inside the collate function).  Loaders are built with
:func:`cubework_b200.utils.get_dataloader`, i.e. sharded over the DATA group and pinned for the trainer's
asynchronous host-to-device copies.

Added: a token file (``.npy`` / ``.bin`` of token ids, e.g. a pre-tokenised corpus) is accepted in place of a text
dataset, so language-model runs need neither the ``datasets`` package nor a tokenizer.
"""
import os

import numpy as np
import torch
from torch.utils.data import Dataset

from .data import get_dataloader


class TokenFileDataset(Dataset):
    """Consecutive windows of ``seq_length`` tokens from a flat array of ids (``.npy``, or raw ``.bin`` of uint16 /
    int32 chosen by ``dtype``); memory-mapped."""

    def __init__(self, path, seq_length, dtype=None):
        if path.endswith(".npy"):
            self.tokens = np.load(path, mmap_mode="r")
        else:
            self.tokens = np.memmap(path, dtype=dtype or np.uint16, mode="r")
        self.seq_length = seq_length
        if len(self.tokens) < seq_length:
            raise ValueError(f"{path} holds {len(self.tokens)} tokens, fewer than one sequence of {seq_length}")

    def __len__(self):
        return len(self.tokens) // self.seq_length

    def __getitem__(self, i):
        ids = torch.from_numpy(np.asarray(self.tokens[i * self.seq_length:(i + 1) * self.seq_length]).astype(np.int64))
        return dict(input_ids=ids, attention_mask=torch.ones(self.seq_length), labels=ids.clone())


def _stack(samples):
    return {k: torch.stack([s[k] for s in samples]) for k in samples[0]}


class TextCollate:
    """Tokenise a list of ``{"text": ...}`` rows to fixed-length id / mask / label tensors."""

    def __init__(self, tokenizer, seq_length):
        self.tokenizer, self.seq_length = tokenizer, seq_length
        if self.tokenizer.pad_token is None:
            self.tokenizer.pad_token = self.tokenizer.eos_token

    def __call__(self, rows):
        enc = self.tokenizer([r["text"] for r in rows], padding="max_length", truncation=True,
                             max_length=self.seq_length, return_tensors="pt")
        ids = enc["input_ids"]
        return dict(input_ids=ids, attention_mask=enc["attention_mask"].float(), labels=ids.clone())


def language_model_loaders(dataset_path, tokenizer_path, seq_length, micro_batch_size, seed=1024, num_workers=0):
    """``(train_loader, test_loader)`` for a causal language model.

    ``dataset_path``: a token file (``.npy`` / ``.bin``; the last tenth is held out for evaluation), or a directory
    written by ``datasets.Dataset.save_to_disk`` / ``DatasetDict.save_to_disk`` with a ``text`` column (needs
    ``tokenizer_path``, a directory ``transformers.AutoTokenizer.from_pretrained`` understands)."""
    if os.path.isfile(dataset_path):
        full = TokenFileDataset(dataset_path, seq_length)
        n_test = max(1, len(full) // 10)
        train = torch.utils.data.Subset(full, range(0, len(full) - n_test))
        test = torch.utils.data.Subset(full, range(len(full) - n_test, len(full)))
        collate = _stack
    else:
        try:
            import datasets
            from transformers import AutoTokenizer
        except ImportError as e:   # noqa: PERF203
            raise RuntimeError("a text dataset directory needs the `datasets` and `transformers` packages; "
                               "pass a token file (.npy / .bin) instead") from e
        if tokenizer_path is None:
            raise ValueError("--tokenizer_path is required with a text dataset")
        data = datasets.load_from_disk(dataset_path)
        if isinstance(data, datasets.DatasetDict):
            train = data["train"]
            test = data["test"] if "test" in data else data["validation"] if "validation" in data else None
        else:
            train, test = data, None
        if test is None:
            parts = train.train_test_split(test_size=0.1, seed=seed)
            train, test = parts["train"], parts["test"]
        collate = TextCollate(AutoTokenizer.from_pretrained(tokenizer_path), seq_length)
    kw = dict(batch_size=micro_batch_size, collate_fn=collate, pin_memory=torch.cuda.is_available(),
              num_workers=num_workers, drop_last=True)
    return (get_dataloader(train, shuffle=True, seed=seed, **kw), get_dataloader(test, shuffle=False, seed=seed, **kw))


class MixupCollate:
    """Stack ``(image, label)`` samples and mix the batch with a permutation of itself (``alpha = 0`` switches the
    mixing off); yields ``pixel_values`` and ``labels = (labels, permuted labels, lambda)``."""

    def __init__(self, alpha=0.8, seed=0):
        self.alpha = alpha
        self.generator = torch.Generator().manual_seed(seed)

    def __call__(self, samples):
        from ..models.vit import mixup_collate
        images = torch.stack([s[0] for s in samples])
        labels = torch.tensor([int(s[1]) for s in samples])
        mixed, targets = mixup_collate(images, labels, self.alpha, self.generator)
        return dict(pixel_values=mixed, labels=targets)


def cifar10_loaders(dataset_path, img_size, micro_batch_size, mixup_alpha=0.8, seed=1024, num_workers=0):
    """``(train_loader, test_loader)`` over CIFAR-10 stored under ``dataset_path`` (torchvision's on-disk layout,
    never downloaded): random crop + horizontal flip + AutoAugment + resize + normalise for training, resize +
    normalise for evaluation; training batches are mixed up in the collate function."""
    try:
        from torchvision import datasets as tvd
        from torchvision import transforms as T
    except ImportError as e:
        raise RuntimeError("the CIFAR-10 pipeline needs torchvision") from e
    mean, std = (0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616)
    train_tf = T.Compose([T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.AutoAugment(T.AutoAugmentPolicy.CIFAR10),
                          T.Resize(img_size), T.ToTensor(), T.Normalize(mean, std)])
    test_tf = T.Compose([T.Resize(img_size), T.ToTensor(), T.Normalize(mean, std)])
    train = tvd.CIFAR10(dataset_path, train=True, transform=train_tf, download=False)
    test = tvd.CIFAR10(dataset_path, train=False, transform=test_tf, download=False)
    kw = dict(batch_size=micro_batch_size, pin_memory=torch.cuda.is_available(), num_workers=num_workers, drop_last=True)
    return (get_dataloader(train, shuffle=True, seed=seed, collate_fn=MixupCollate(mixup_alpha, seed), **kw),
            get_dataloader(test, shuffle=False, seed=seed, collate_fn=MixupCollate(0.0, seed), **kw))


class Cycle:
    """Endless iteration over a ``DataLoader`` (a new pass, reshuffled by the sampler's epoch, when one ends)."""

    def __init__(self, loader):
        self.loader, self.epoch, self.it = loader, 0, None

    def __iter__(self):
        return self

    def __next__(self):
        if self.it is None:
            self.it = iter(self.loader)
        try:
            return next(self.it)
        except StopIteration:
            self.epoch += 1
            sampler = getattr(self.loader, "sampler", None)
            if hasattr(sampler, "set_epoch"):
                sampler.set_epoch(self.epoch)
            self.it = iter(self.loader)
            return next(self.it)
