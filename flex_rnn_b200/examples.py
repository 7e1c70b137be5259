"""Command line driver over the bundled step functions, in the spirit of the
reference's tests/examples.py (modes --check-flex, --benchmark-flex,
--torch-compile, --forward; the comparisons with third-party kernels are not
reproduced).

    python -m flex_rnn_b200.examples --op rwkv7 --check-flex
    python -m flex_rnn_b200.examples --op delta_rule --benchmark-flex
"""
import argparse

import torch as th

import flex_rnn_b200
from flex_rnn_b200 import workloads as W


def main(argv=None):
    ap = argparse.ArgumentParser()
    ops = list(W.STEPS) + list(W.ZOO)
    ap.add_argument("--op", default="rwkv7", choices=ops)
    ap.add_argument("--batchsz", type=int, default=8)
    ap.add_argument("--modeldim", type=int, default=None)
    ap.add_argument("--headsz", type=int, default=128)
    ap.add_argument("--seqlen", type=int, default=None)
    ap.add_argument("--benchmark-flex", action="store_true")
    ap.add_argument("--check-flex", action="store_true")
    ap.add_argument("--torch-compile", action="store_true")
    ap.add_argument("--forward", action="store_true")
    a = ap.parse_args(argv)
    check = a.check_flex or not a.benchmark_flex
    modeldim = a.modeldim or (256 if check else 4096)
    T = a.seqlen or (256 if check else 1024)
    B, C = a.batchsz, a.headsz
    H = modeldim // C
    dev = "cuda"
    print("Testing", a.op)
    print(f"Input sizes B={B}, T={T}, H={H}, C={C}")
    dtype = th.float32 if check or a.op in ("s4d", "mamba") else th.bfloat16
    if a.op in W.STEPS:
        xs, _, _ = W.synthetic(a.op, B, T, H, 64 if a.op == "mamba2" else C, C, dtype)
        step_fn, nst = W.STEPS[a.op], 1
    else:
        M, N = (modeldim, 1) if a.op in ("rwkv4", "hgrn") else (1, 1) if a.op == "mlstm_gates" else (C, 16 if a.op == "mamba" else C)
        Hh = 1 if a.op in ("rwkv4", "hgrn") else H
        ins, sts = W.zoo_case(a.op, B, T, Hh, M, N, dtype)
        xs, step_fn, nst = ins + sts, W.ZOO[a.op], len(sts)
    xs = [x.to(dev) for x in xs]
    op = flex_rnn_b200.jit(step_fn)
    flex = th.compile(lambda *z: op(*z)) if a.torch_compile else op
    if check:
        print("Verifying flex compiled kernel")
        flex_rnn_b200.check_grad(flex, op.naive_fp64, xs, backward=not a.forward)
    else:
        print("Benchmarking flex compiled kernel")
        flex_rnn_b200.benchmark(flex, xs, backward=not a.forward)


if __name__ == "__main__":
    main()
