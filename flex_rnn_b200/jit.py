"""``@flex_rnn_b200.jit``: the user-facing decorator.

Mirrors the reference front end (flex_rnn/jit.py:7-84 in the reference
project): ``jit(step)(*inputs, *initial_states)`` runs the recurrence over the
time dimension on the GPU, forward and backward, and behaves like
``jit.naive``.  Same attributes (``step``, ``apply``, ``naive``,
``naive_fp64``), same argument layout (inputs ``[B,T,H,M,N]`` with size-1 dims
broadcast, states ``[B,H,M,N]``), same PyTorch custom-op wiring so that
``torch.compile`` sees one opaque op with a fake implementation.

Differences: compiled kernels are cached per (shapes, strides, dtypes, device)
instead of once per object, so a second call with other shapes re-specialises
rather than failing an assertion.
"""
from __future__ import annotations

import inspect
import uuid
from typing import Callable, Dict, Tuple

import torch as th

from .trace import as_tuple
from .twopass import build_twopass, split_list, verify_meta

_N_PACKED_AUX = 1   # all saved row sums travel in one tensor so the op schema is fixed


def _signature(args) -> Tuple:
    if any(isinstance(s, th.SymInt) for a in args for s in tuple(a.shape) + tuple(a.stride())):
        raise RuntimeError("flex_rnn_b200 kernels are specialised for concrete shapes and strides; symbolic sizes are not "
                           "supported (under torch.compile use dynamic=False or mark the sizes static)")
    dev = args[0].device
    return tuple((tuple(a.shape), tuple(s if n > 1 else 0 for s, n in zip(a.stride(), a.shape)), a.dtype) for a in args) + \
        ((dev.type, dev.index),)


class jit:
    def __init__(self, step: Callable, n_step_args: int = None):
        self.step = step
        if n_step_args is None:
            n_step_args = len(inspect.signature(step).parameters)
        probe_out, probe_state = step(*[th.empty(1, 1, device="meta") for _ in range(n_step_args)])
        self.noutputs = len(as_tuple(probe_out))
        self.nstates = len(as_tuple(probe_state))
        self.ninputs = n_step_args - self.nstates
        self._compiled: Dict[Tuple, tuple] = {}     # signature -> (forward, backward, fw_meta, bw_meta)
        self._metas: Dict[Tuple, tuple] = {}        # signature -> (fw_meta, bw_meta)
        self.forward_func = self.backward_func = None
        self.apply = self._register_ops()

    # ------------------------------------------------------------------ public
    def __call__(self, *args):
        return self.apply(*args)

    def naive(self, *args, dtype=th.float32):
        """Plain PyTorch loop over time; defines what the compiled op computes
        (reference: flex_rnn/jit.py:23-36).  Runs on any device."""
        inputs, state0 = split_list(args, [self.ninputs, self.nstates])
        T = max(x.shape[1] for x in inputs)
        state = tuple(state0)
        outs = None
        for t in range(T):
            x_t = [x.expand(-1, T, -1, -1, -1)[:, t].to(dtype) for x in inputs]
            y_t, state = self.step(*x_t, *state)
            y_t, state = as_tuple(y_t), as_tuple(state)
            if outs is None:
                outs = tuple(th.empty(y.shape[0], T, y.shape[1], y.shape[2], dtype=y.dtype, device=y.device) for y in y_t)
            for dst, y in zip(outs, y_t):
                dst[:, t] = y.squeeze(-1)
        final = tuple(th.empty_like(s0).copy_(s) for s0, s in zip(state0, state))
        return (*outs, *final)

    def naive_fp64(self, *args):
        return self.naive(*args, dtype=th.double)

    # ----------------------------------------------------------------- internals
    def _specialise(self, inputs, state):
        key = _signature(tuple(inputs) + tuple(state))
        if key not in self._compiled:
            self._compiled[key] = build_twopass(self.step, inputs, state)
            self._metas[key] = self._compiled[key][2:]
        fwd, bwd, fw_meta, bw_meta = self._compiled[key]
        self.forward_func, self.backward_func, self.fw_meta, self.bw_meta = fwd, bwd, fw_meta, bw_meta
        return self._compiled[key]

    def _dry_metas(self, inputs, state):
        key = _signature(tuple(inputs) + tuple(state))
        if key not in self._metas:
            self._metas[key] = build_twopass(self.step, inputs, state, dryrun=True)
        return self._metas[key]

    def _register_ops(self):
        uid = uuid.uuid4().hex
        nin, nst, nout = self.ninputs, self.nstates, self.noutputs
        n_fw_out = nout + 2 * nst + _N_PACKED_AUX

        def schema(n_in, n_out):
            return "(" + ", ".join(f"Tensor x{i}" for i in range(n_in)) + ") -> (" + ", ".join(["Tensor"] * n_out) + ")"

        def materialise(meta, device):
            return tuple(th.empty_strided(s, st, dtype=dt, device=device) for s, st, dt in meta)

        @th.library.custom_op(f"flex_rnn_b200::fw_{uid}", mutates_args=(), schema=schema(nin + nst, n_fw_out))
        def fw_op(*args):
            inputs, state = split_list(args, [nin, nst])
            forward, _, fw_meta, _ = self._specialise(inputs, state)
            res = forward(inputs, state)
            verify_meta(res, materialise(fw_meta, "meta"))
            return res

        @fw_op.register_fake
        def _(*args):
            inputs, state = split_list(args, [nin, nst])
            fw_meta, _ = self._dry_metas(inputs, state)
            return materialise(fw_meta, args[0].device)

        # The backward op also receives the initial states.  Their values are never read (the kernels
        # restart from checkpoint 0); they identify the specialisation exactly: two calls with the same
        # inputs but states of other strides or dtype are different kernels.
        @th.library.custom_op(f"flex_rnn_b200::bw_{uid}", mutates_args=(),
                              schema=schema(nout + 3 * nst + nin + _N_PACKED_AUX, nin + nst))
        def bw_op(*args):
            dout, dstT, inputs, state0, store, aux = split_list(args, [nout, nst, nin, nst, nst, _N_PACKED_AUX])
            _, backward, _, bw_meta = self._lookup_for_backward(inputs, state0)
            dx, ds0 = backward(dout, dstT, inputs, store, aux)
            verify_meta(dx + ds0, materialise(bw_meta, "meta"))
            return (*dx, *ds0)

        @bw_op.register_fake
        def _(*args):
            dout, dstT, inputs, state0, store, aux = split_list(args, [nout, nst, nin, nst, nst, _N_PACKED_AUX])
            _, bw_meta = self._lookup_for_backward(inputs, state0, dry=True)
            return materialise(bw_meta, args[0].device)

        def setup_context(ctx, inputs, output):
            ctx.set_materialize_grads(False)
            ctx.save_for_backward(*inputs, *output[nout + nst:])
            ctx.out_meta = tuple(o.to("meta") for o in output[:nout + nst])

        def backward(ctx, *grads):
            # upstream gradients that autograd leaves out are zeros (reference: flex_rnn/jit.py:76-80)
            grads = list(grads[:nout + nst])
            dev = ctx.saved_tensors[0].device
            for i, m in enumerate(ctx.out_meta):
                if grads[i] is None:
                    grads[i] = th.zeros_like(m, device=dev)
            return bw_op(*grads, *ctx.saved_tensors)

        fw_op.register_autograd(backward, setup_context=setup_context)
        self._fw_op, self._bw_op = fw_op, bw_op
        return lambda *args: fw_op(*args)[:nout + nst]

    def _lookup_for_backward(self, inputs, state0, dry=False):
        """The specialisation a forward call made for exactly these inputs and
        initial states (shapes, strides, dtypes, device)."""
        key = _signature(tuple(inputs) + tuple(state0))
        table = self._metas if dry else self._compiled
        if key not in table:
            if dry:
                return self._dry_metas(inputs, state0)
            raise AssertionError("backward called for arguments that no forward call has specialised")
        return table[key]


def simplified_naive(step, *args):
    """Single-output, single-state form of ``jit.naive`` (documentation aid)."""
    inputs, state = args[:-1], args[-1]
    T = max(x.shape[1] for x in inputs)
    ys = []
    for t in range(T):
        y, state = step(*[x.expand(-1, T, -1, -1, -1)[:, t].float() for x in inputs], state)
        ys.append(y)
    return th.stack(ys, dim=1).squeeze(-1), state
