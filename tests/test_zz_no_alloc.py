"""frnn_launch_static_scratch: the launch entry point for callers that cannot
allocate device memory (an inference loop that only wants the outputs of a
forward scan, an embedding that forbids cudaMalloc after start-up).  It points
the forward kernel's training-time scratch (checkpoints, saved row sums) at a
static array inside the library.  Checked here through the C ABI against the
ordinary frnn_launch with caller-allocated scratch, on two calls in a row with
different inputs (the array is shared and keeps the previous call's contents),
plus the refusal of a request larger than the array.

Collected last on purpose (file name), so that a run that stops at the first
failure has already run every other test."""
import pytest
import torch

from flex_rnn_b200 import runtime
from flex_rnn_b200 import workloads as W
from flex_rnn_b200.twopass import generate, make_plan

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _forward_case(seed):
    B, T, H, M, N = 2, 48, 4, 64, 64
    xs, _, _ = W.synthetic("delta_rule", B, T, H, M, N, torch.float32, seed=seed)
    return (B, T, H, M, N), [x.to(DEV) for x in xs]


def test_static_scratch_matches_caller_allocated_scratch():
    (B, T, H, M, N), xs = _forward_case(0)
    plan, fw_meta, _ = make_plan(W.delta_rule, tuple(xs[:-1]), (xs[-1],))
    fw, _ = generate(plan)
    with torch.cuda.device(0):
        cubin, _ = runtime.compile_cubin(fw.source)
        mod = runtime.Module(cubin, [fw.name], [fw.smem_bytes])
        ck_bytes = B * H * fw.info["nck"] * M * N * 4
        aux_bytes = max(1, len(plan.aux)) * B * H * T * M * 4
        i_ck, i_aux = fw.params.index("ck0"), fw.params.index("aux")
        stream = torch.cuda.current_stream().cuda_stream
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        used = plan.g_fw.used_inputs()

        def tensor_maps(ptrs):
            # the kernel's TMA tensor maps embed the input addresses: encode them for this call
            return [runtime.encode_tensor_map(ptrs[tm["src_index"]] + tm["off_bytes"], tm["elt"], tm["dims"],
                                              tm["strides_bytes"], tm["box"]) for tm in fw.tmaps]

        def run(inputs, static):
            y = torch.full((B, T, H, M), float("nan"), device=DEV)
            ST = torch.full((B, H, M, N), float("nan"), device=DEV)
            ck = torch.empty(ck_bytes // 4, device=DEV)
            aux = torch.empty(aux_bytes // 4, device=DEV)
            ptrs = [x.data_ptr() for x, u in zip(inputs[:-1], used) if u]
            ptrs += [inputs[-1].data_ptr(), y.data_ptr(), ST.data_ptr()]
            ptrs += [0 if static else ck.data_ptr(), 0 if static else aux.data_ptr(), err.data_ptr()]
            ptrs += tensor_maps(ptrs)
            assert len(ptrs) == len(fw.params)
            if static:
                mod.launch_static_scratch(0, fw.grid, fw.block, fw.smem_bytes, stream, ptrs,
                                          {i_ck: ck_bytes, i_aux: aux_bytes})
            else:
                mod.launch(0, fw.grid, fw.block, fw.smem_bytes, stream, ptrs)
            torch.cuda.synchronize()
            return y, ST

        # two calls in a row through the new entry point, each against the existing one
        for seed in (0, 1):
            _, inputs = _forward_case(seed)
            y_ref, ST_ref = run(inputs, static=False)
            y, ST = run(inputs, static=True)
            assert int(err.item()) == 0
            assert torch.isfinite(y).all() and torch.isfinite(ST).all()
            assert torch.equal(y, y_ref) and torch.equal(ST, ST_ref)     # same kernel, same arithmetic: bit-exact

        # a request beyond the static array is refused with a clear message and launches nothing
        cap = runtime.lib().frnn_static_scratch_capacity()
        assert cap == 32 << 20
        ptrs = [x.data_ptr() for x, u in zip(xs[:-1], used) if u] + [xs[-1].data_ptr(), 0, 0, 0, 0, err.data_ptr()]
        ptrs += tensor_maps(ptrs)
        with pytest.raises(runtime.FrnnError, match="more scratch than the library's static buffer"):
            mod.launch_static_scratch(0, fw.grid, fw.block, fw.smem_bytes, stream, ptrs, {i_ck: cap, i_aux: 4096})

        # a scratch list longer than the parameter list, or naming a parameter twice, is refused too
        import ctypes
        n = len(ptrs)
        vals = (ctypes.c_void_p * n)(*[0 if isinstance(p, runtime.StructArg) else int(p) for p in ptrs])
        args = (ctypes.c_void_p * n)(*[p.addr if isinstance(p, runtime.StructArg) else ctypes.addressof(vals) + 8 * i
                                       for i, p in enumerate(ptrs)])
        g = (ctypes.c_uint * 3)(*fw.grid)
        b = (ctypes.c_uint * 3)(fw.block, 1, 1)
        lib = runtime.lib()
        for idx in ([i_ck, i_ck], list(range(n)) + [0]):
            sa = (ctypes.c_int * len(idx))(*idx)
            sb = (ctypes.c_size_t * len(idx))(*([256] * len(idx)))
            rc = lib.frnn_launch_static_scratch(mod._h, 0, g, b, fw.smem_bytes, ctypes.c_void_p(stream), args, n, sa, sb, len(idx))
            assert rc == 1, lib.frnn_last_error()
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        mod.close()
