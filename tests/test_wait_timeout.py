"""Every device-side wait of the generated kernels is time-bounded: when a TMA
stage never arrives the kernel records an error code and returns instead of
spinning.  Exercised here with the prelude's own wait on an mbarrier that
nothing completes and a 2 ms limit; the context stays usable afterwards.

The report reaches the caller without any debugging switch: the library's
error word lives in pinned host memory that the kernels write directly, and
the next forward or backward call looks at it before it launches and raises
(frnn_status_check of the C ABI).  For a word in device memory frnn_status
copies, waits and returns FRNN_E_KERNEL; frnn_status_post queues the copy."""
import pytest
import torch

from flex_rnn_b200 import runtime
from flex_rnn_b200.twopass import prelude

pytestmark = pytest.mark.gpu

SRC = r'''
extern "C" __global__ void wait_for_nothing(int* err, int* done) {
    __shared__ u64 bar;
    if (threadIdx.x == 0) { frnn_mbar_init(&bar, 1); frnn_mbar_init_fence(); }
    __syncthreads();
    bool ok = frnn_mbar_wait(&bar, 0, err, 7);      // no copy was ever issued on this barrier
    if (threadIdx.x == 0) done[0] = ok ? 1 : 2;
}
'''


def test_wait_runs_out_and_reports():
    src = "#define FRNN_WAIT_LIMIT_NS 2000000ull\n" + prelude().replace("#pragma once", "") + SRC
    with torch.cuda.device(0):
        cubin, _ = runtime.compile_cubin(src)
        mod = runtime.Module(cubin, ["wait_for_nothing"], [0])
        err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        done = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        mod.launch(0, (2, 1, 1), 64, 0, torch.cuda.current_stream().cuda_stream, [err.data_ptr(), done.data_ptr()])
        torch.cuda.synchronize()
        assert int(done.item()) == 2          # the wait gave up
        assert int(err.item()) == 7           # ... and said why
        # the device is still healthy
        assert float((torch.ones(8, device="cuda:0") * 2).sum().item()) == 16.0
        mod.close()


def _timed_out_kernel(err_ptr):
    src = "#define FRNN_WAIT_LIMIT_NS 2000000ull\n" + prelude().replace("#pragma once", "") + SRC
    cubin, _ = runtime.compile_cubin(src)
    mod = runtime.Module(cubin, ["wait_for_nothing"], [0])
    done = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    mod.launch(0, (1, 1, 1), 32, 0, torch.cuda.current_stream().cuda_stream, [err_ptr, done.data_ptr()])
    return mod, done


def test_status_call_returns_kernel_error():
    """frnn_status: FRNN_E_KERNEL (code 5) with the kernel's code in the message, then the word is clear."""
    with torch.cuda.device(0):
        err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        stream = torch.cuda.current_stream().cuda_stream
        runtime.status(err.data_ptr(), stream)                      # nothing reported: no error
        mod, done = _timed_out_kernel(err.data_ptr())
        with pytest.raises(runtime.FrnnError, match=r"code 5\).*reported error 7"):
            runtime.status(err.data_ptr(), stream)
        torch.cuda.synchronize()
        assert int(err.item()) == 0 and int(done.item()) == 2
        runtime.status(err.data_ptr(), stream)
        mod.close()


def test_timed_out_wait_raises_at_the_next_call():
    """A wait that ran out in a kernel of this device makes the NEXT call of a
    compiled op raise, by default (no FRNN_CHECK), and without a hang; after
    the report the word is clear and the op works again."""
    import flex_rnn_b200
    from flex_rnn_b200 import twopass
    from oracle import naive_oracle as O
    xs, _, _ = O.make_case("delta_rule", 1, 8, 2, 32, 32, torch.float32)
    xs = [x.to("cuda:0") for x in xs]
    op = flex_rnn_b200.jit(O.delta_rule)
    with torch.cuda.device(0):
        y0, S0 = op(*xs)
        st = twopass.device_status("cuda:0")
        mod, done = _timed_out_kernel(st.word.data_ptr())          # reports through the library's own word
        torch.cuda.synchronize()
        assert int(done.item()) == 2
        with pytest.raises(runtime.FrnnError, match="reported error 7"):
            op(*xs)
        y2, S2 = op(*xs)
        torch.cuda.synchronize()
        assert op.forward_func.kernel_status("cuda:0") == 0
        assert torch.equal(y0, y2) and torch.equal(S0, S2)
        mod.close()
