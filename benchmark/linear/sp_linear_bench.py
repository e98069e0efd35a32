"""Fused products of one GPT-2 XL block under 1D tensor parallelism with row-sharded activations.

    torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmark/linear/sp_linear_bench.py [--trace]

For the forward and backward products of the attention / MLP linears (32768 tokens, hidden 1600, MLP 6400, split N
ways) the script times three things with CUDA events (median of 8 samples after 3 warm-ups; a sample is four
back-to-back calls, so that the host's launch latency hides behind the previous call as it does in a training step,
after a 200 MB scratch write and a barrier; operands and results of one call exceed L2; maximum over ranks): the
plain tcgen05 GEMM of the same per-rank shape (no exchange),
the fused all-gather -> GEMM or GEMM -> reduce-scatter kernel, and the link floor (bytes every GPU has to send,
(N-1)/N of the 105 MB activation, at the measured 770 GB/s peer-copy rate).  The roofline of a fused product is the
larger of the plain GEMM time at the measured GEMM peak and the link floor.

``--trace`` additionally runs each fused product once with the kernel's event trace switched on
(``cubework_b200.parallel.symm_impl.GGS_TRACE``) and prints, averaged over the CTAs, where the producer, the MMA
issuer and one epilogue warp spent their time.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import cubework_b200 as cube  # noqa: E402
from cubework_b200 import ops  # noqa: E402
from cubework_b200.distributed import ParallelManager as pm  # noqa: E402
from cubework_b200.ops import ext  # noqa: E402
from cubework_b200.parallel import fused, symm, symm_impl  # noqa: E402

M, H, F = 32768, 1600, 6400
LINK_GBS = 770.0


def peak_tflops():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return json.load(f)["bf16_tflops"], "measured"
    except Exception:  # noqa: BLE001
        return 1590.0, "fallback"


def timed(fn, flush, dev, iters=8, reps=4):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        flush.add_(1)
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) / reps)
    t = torch.tensor(sorted(ts)[len(ts) // 2], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item() * 1e3


def trace_summary(fn, flush, dev):
    """Average microseconds per CTA between pairs of trace events of one launch."""
    tr = torch.zeros(148 * 3, 512, 2, dtype=torch.int64, device=dev)
    symm_impl.GGS_TRACE = tr
    flush.add_(1)
    dist.barrier()
    fn()
    torch.cuda.synchronize()
    symm_impl.GGS_TRACE = None
    t = tr.cpu()

    def span(role, a, b):
        tot = []
        for cta in range(148):
            ev = t[cta * 3 + role, :510]
            ev = ev[ev[:, 1] > 0]
            s, pend = 0, None
            for code, ts in zip((ev[:, 0] >> 32).tolist(), ev[:, 1].tolist()):
                if code == a:
                    pend = ts
                elif code == b and pend is not None:
                    s += ts - pend
                    pend = None
            if len(ev):
                tot.append(s)
        return round(sum(tot) / max(1, len(tot)) / 1e3, 1)

    ent, ext_ = t[0::3, 510, 1], t[0::3, 511, 1]
    ok = (ent > 0) & (ext_ > 0)
    return {"kernel_us": round((ext_[ok].max() - ent[ok].min()).item() / 1e3, 1), "producer_flag_wait": span(0, 1, 2),
            "mma_wait_accumulator": span(2, 10, 11), "mma_main_loop": span(2, 11, 12), "epilogue_wait_mma": span(1, 3, 4),
            "epilogue_wait_flags": span(1, 4, 5), "epilogue_total": span(1, 4, 6)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--trace", action="store_true")
    args = ap.parse_args()
    n = int(os.environ["WORLD_SIZE"])
    cube.initialize_distributed(argv=["--tp", "1d", "--tp_size", str(n)])
    symm._POLICY = "1"
    mode = pm.PARALLEL_1D
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.zeros(200 << 20, dtype=torch.uint8, device=dev)
    peak, src = peak_tflops()

    def rnd(*shape):
        return (torch.randn(*shape, device=dev) * 0.05).bfloat16()

    Ml = M // n
    # name, stored A, stored B, trans_b, gather rows of A, scatter rows of the product, activation, per-rank (M, N, K)
    cases = [
        ("qkv forward: all-gather -> GEMM", rnd(Ml, H), rnd(3 * H // n, H), True, True, False, None, (M, 3 * H // n, H)),
        ("fc1 forward: all-gather -> GEMM + bias + GELU", rnd(Ml, H), rnd(F // n, H), True, True, False, "gelu", (M, F // n, H)),
        ("proj forward: GEMM -> reduce-scatter", rnd(M, H // n), rnd(H, H // n), True, False, True, None, (M, H, H // n)),
        ("fc2 forward: GEMM -> reduce-scatter", rnd(M, F // n), rnd(H, F // n), True, False, True, None, (M, H, F // n)),
        ("fc2 backward dX: all-gather -> GEMM", rnd(Ml, H), rnd(H, F // n), False, True, False, None, (M, F // n, H)),
        ("fc1 backward dX: GEMM -> reduce-scatter", rnd(M, F // n), rnd(F // n, H), False, False, True, None, (M, H, F // n)),
    ]
    link_us = (n - 1) / n * M * H * 2 / (LINK_GBS * 1e9) * 1e6
    for name, a, b, tb, gather, scatter, act, (m_, n_, k_) in cases:
        bias = torch.zeros(n_, device=dev) if act else None

        def run():
            return fused.gather_gemm_reduce(a, b, False, tb, gather_a=(mode, 0) if gather else None,
                                            scatter=(mode, 0) if scatter else None, bias=bias, act=act,
                                            pre_act_out=act is not None)

        a_loc = rnd(m_, k_)

        def plain():
            return ops.gemm(a_loc, b, False, tb, bias=bias, act=act, pre_act_out=act is not None)

        t_plain, t_fused = timed(plain, flush, dev), timed(run, flush, dev)
        roof = max(2.0 * m_ * n_ * k_ / (peak * 1e12) * 1e6, link_us)
        line = {"product": name, "ranks": n, "per_rank_MxNxK": [m_, n_, k_], "plain_gemm_us": round(t_plain, 1),
                "fused_us": round(t_fused, 1), "link_floor_us": round(link_us, 1), "roofline_us": round(roof, 1),
                "fused_fraction_of_roofline": round(roof / t_fused, 3), "peak_source": src}
        if args.trace:
            line["trace_avg_us_per_cta"] = trace_summary(run, flush, dev)
        if dist.get_rank() == 0:
            print(json.dumps(line), flush=True)
        ext.check_status()
    cube.destroy_distributed()


if __name__ == "__main__":
    main()
