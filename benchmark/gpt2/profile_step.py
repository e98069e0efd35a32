"""One training step of a 4-layer GPT-2 XL-shape model (same per-layer shapes as the benchmark) for kernel lists."""
import os, sys
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import torch
os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29517")
os.environ.setdefault("RANK", "0"); os.environ.setdefault("LOCAL_RANK", "0"); os.environ.setdefault("WORLD_SIZE", "1")
import cubework_b200 as cube
from cubework_b200.engine import Trainer
from cubework_b200.models import gpt2
from cubework_b200.optim import FusedAdamW
depth = int(os.environ.get("DEPTH", "4")); batch = int(os.environ.get("BATCH", "32"))
cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", "1"])
dev = torch.device("cuda", 0)
model = gpt2.GPT2(vocab_size=50304, max_position_embeddings=1024, hidden_size=1600, num_heads=int(os.environ.get("HEADS", "64")), intermediate_size=6400,
                  depth=depth, dropout=0.0, embedding_dropout=0.0, init_std=0.02).to(dev)
tr = Trainer(model, gpt2.GPT2LMLoss(), FusedAdamW(model.parameters(), lr=1e-4), amp_dtype=torch.bfloat16, clip=1.0)
ids = torch.randint(0, 50304, (batch, 1024), device=dev)
b = dict(input_ids=ids, attention_mask=torch.ones(batch, 1024, device=dev), labels=ids)
tr.step(b); tr.step(b)
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
torch.cuda.profiler.start()
e0.record(); tr.step(b); e1.record()
torch.cuda.synchronize()
torch.cuda.profiler.stop()
print("step ms", e0.elapsed_time(e1))
cube.destroy_distributed()
