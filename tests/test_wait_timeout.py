"""Every device-side wait of the generated kernels is time-bounded: when a TMA
stage never arrives the kernel records an error code and returns instead of
spinning.  Exercised here with the prelude's own wait on an mbarrier that
nothing completes and a 2 ms limit; the context stays usable afterwards."""
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
