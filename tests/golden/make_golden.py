"""Regenerates tests/golden/*.pt from the reference checkout.

Run where a checkout of the reference project is available, passing its path:

    FLEX_RNN_REFERENCE=<path to the flex_rnn checkout> python tests/golden/make_golden.py

For every benchmark step function it draws the seeded inputs of
``oracle.naive_oracle.make_inputs`` at a small shape, runs the REFERENCE's own
``flex_rnn.jit(step).naive`` (fp32 and fp64) and ``torch.autograd.grad`` on the
CPU, and stores inputs, outputs and gradients.  It also records the L2 norms of
all results at the seed-0 Delta Rule configuration B2 T64 H4 64x64 (and the
other three steps at the same shape) as known-answer values.
"""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.environ.get("FLEX_RNN_REFERENCE", os.path.join(os.sep, "root", "reference")))

import flex_rnn  # noqa: E402  (the reference project)
from oracle import naive_oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SMALL = dict(B=2, T=12, H=2, M=16, N=16)


def run_reference(op, shape, dtype, fp64):
    step = O.STEPS[op]
    xs, dy, dS = O.make_case(op, dtype=dtype, **shape)
    dys = [dy]
    ref = flex_rnn.jit(step)
    leaves = [x.clone().requires_grad_() for x in xs]
    res = (ref.naive_fp64 if fp64 else ref.naive)(*leaves)
    y, ST = res[0], res[1]
    grads = torch.autograd.grad([y, ST], leaves, [dys[0].to(y.dtype), dS.to(ST.dtype)], allow_unused=True)
    grads = [g if g is not None else torch.zeros_like(p) for g, p in zip(grads, leaves)]
    return dict(inputs=[x.clone() for x in xs], dy=dys[0], dS=dS, y=y.detach(), ST=ST.detach(),
                grads=[g.detach() for g in grads])


def main():
    for op in O.STEPS:
        for dtype, tag in ((torch.float32, "fp32"), (torch.bfloat16, "bf16")):
            out = run_reference(op, SMALL, dtype, fp64=False)
            out["fp64"] = {k: v for k, v in run_reference(op, SMALL, dtype, fp64=True).items() if k in ("y", "ST", "grads")}
            out["shape"] = SMALL
            torch.save(out, os.path.join(HERE, f"{op}_{tag}.pt"))
            print("wrote", op, tag)
    # known-answer norms at the CPU-runnable configuration
    norms = {}
    for op in O.STEPS:
        shape = dict(B=2, T=64, H=4, M=32 if op == "mamba2" else 64, N=64)
        r = run_reference(op, shape, torch.float32, fp64=False)
        norms[op] = dict(shape=shape, norms=[float(t.double().norm()) for t in [r["y"], r["ST"], *r["grads"]]])
        print(op, norms[op])
    import json
    with open(os.path.join(HERE, "norms_c0.json"), "w") as f:
        json.dump(norms, f, indent=1)


if __name__ == "__main__":
    main()
