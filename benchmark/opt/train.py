"""OPT training entry point: ``torchrun --nproc_per_node N benchmark/opt/train.py -m opt_13b --tp 3d --tp_size 8 --ckpt ...``

Parity: benchmark/opt/train.py + opt.py:536-653.  The reference optimiser for OPT is SGD (opt.py:623); ``--optimizer
adamw`` switches.  ``--fsdp`` shards parameters, gradients and optimizer state over the data-parallel group with the
package's own wrapper (``cubework_b200.parallel.fsdp``), one unit per decoder layer as in opt.py:544-562; the
reference's ``-O3`` (fairscale loss scaling) has no counterpart because bf16 needs no loss scaling.
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402

import cubework_b200 as cube  # noqa: E402
import cubework_b200.module as cube_nn  # noqa: E402
from cubework_b200 import train as driver  # noqa: E402
from cubework_b200.models import opt  # noqa: E402

DEFAULT_OPTIMIZER = "sgd"
SCHEDULE = "linear"


def build(args):
    kw = {} if args.dropout is None else dict(dropout=args.dropout)
    if getattr(args, "pure_16bit", False):      # -O3: parameters (and gradients, optimizer updates) in the AMP dtype
        kw["dtype"] = torch.bfloat16 if args.amp_dtype == "bf16" else torch.float16
    model = opt.build_model(args.model_name, max_position_embeddings=args.seq_length,
                            checkpoint=args.use_activation_checkpoint, init_std=0.02, **kw)
    vocab = model.vocab_size

    def make_batch(g, micro):
        ids = torch.randint(2, vocab, (micro, args.seq_length), generator=g)
        return dict(input_ids=ids, attention_mask=torch.ones(micro, args.seq_length), labels=ids.clone())

    return model, opt.OPTLMLoss(), cube_nn.Perplexity(), make_batch, args.seq_length


def build_data(args, micro, model):
    from cubework_b200.utils.datasets import language_model_loaders
    return language_model_loaders(args.dataset_path, args.tokenizer_path, args.seq_length, micro,
                                  num_workers=args.num_workers)


def forward(model, batch):
    return model(batch["input_ids"], batch["attention_mask"])[0], batch["labels"]


if __name__ == "__main__":
    parser = driver.get_parser("OPT on cubework_b200", "opt_125m")
    parser.add_argument("-O3", dest="pure_16bit", action="store_true",
                        help="keep the parameters themselves in the AMP dtype (no fp32 master copies)")
    args = cube.initialize_distributed(parser)
    driver.run(args, sys.modules[__name__])
    cube.destroy_distributed()
