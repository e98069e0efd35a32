"""ViT training entry point: ``torchrun --nproc_per_node N benchmark/vit/train.py -m vit_base --tp 2d --tp_size 4 ...``

Parity: benchmark/vit/train.py + vit.py:357-506 (mixup loss / accuracy, AdamW, cosine schedule).  Images are
synthetic N(0,1) unless a dataset path is wired in; throughput is reported in images/s.
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

import cubework_b200 as cube  # noqa: E402
from cubework_b200 import train as driver  # noqa: E402
from cubework_b200.models import vit  # noqa: E402

DEFAULT_OPTIMIZER = "adamw"
SCHEDULE = "cosine"


def build(args):
    kw = {} if args.dropout is None else dict(dropout=args.dropout)
    model = vit.build_model(args.model_name, checkpoint=args.use_activation_checkpoint, **kw)
    img = model.img_size
    classes = model.head.dense.linear.num_classes

    def make_batch(g, micro):
        return dict(pixel_values=torch.randn(micro, 3, img, img, generator=g),
                    labels=torch.randint(0, classes, (micro, ), generator=g))

    return model, vit.MixupLoss(), vit.MixupAccuracy(), make_batch, 1    # one "token" per image: throughput in images


def build_data(args, micro, model):
    from cubework_b200.utils.datasets import cifar10_loaders
    return cifar10_loaders(args.dataset_path, model.img_size, micro, num_workers=args.num_workers)


def forward(model, batch):
    return model(batch["pixel_values"]), batch["labels"]


if __name__ == "__main__":
    parser = driver.get_parser("ViT on cubework_b200", "vit_base", token_unit="images")
    args = cube.initialize_distributed(parser)
    driver.run(args, sys.modules[__name__])
    cube.destroy_distributed()
