"""GPT-2 training entry point: ``torchrun --nproc_per_node N benchmark/gpt2/train.py -m gpt2_xl --tp 1d --tp_size N ...``

Parity: benchmark/gpt2/train.py + gpt2.py:376-469 (build model / data / criterion / optimizer / scheduler).
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

import cubework_b200 as cube  # noqa: E402
import cubework_b200.module as cube_nn  # noqa: E402
from cubework_b200 import train as driver  # noqa: E402
from cubework_b200.models import gpt2  # noqa: E402

DEFAULT_OPTIMIZER = "adamw"
SCHEDULE = "linear"
VOCAB = 50304


def build(args):
    kw = {} if args.dropout is None else dict(dropout=args.dropout, embedding_dropout=args.dropout)
    model = gpt2.build_model(args.model_name, max_position_embeddings=args.seq_length,
                             checkpoint=args.use_activation_checkpoint, init_std=0.02, **kw)

    def make_batch(g, micro):
        ids = torch.randint(0, VOCAB if args.model_name != "gpt2_tiny" else 1024, (micro, args.seq_length), generator=g)
        return dict(input_ids=ids, attention_mask=torch.ones(micro, args.seq_length), labels=ids.clone())

    return model, gpt2.GPT2LMLoss(), cube_nn.Perplexity(), make_batch, args.seq_length


def build_data(args, micro, model):
    from cubework_b200.utils.datasets import language_model_loaders
    return language_model_loaders(args.dataset_path, args.tokenizer_path, args.seq_length, micro,
                                  num_workers=args.num_workers)


def forward(model, batch):
    return model(batch["input_ids"], batch["attention_mask"]), batch["labels"]


if __name__ == "__main__":
    parser = driver.get_parser("GPT-2 on cubework_b200", "gpt2_small")
    args = cube.initialize_distributed(parser)
    driver.run(args, sys.modules[__name__])
    cube.destroy_distributed()
