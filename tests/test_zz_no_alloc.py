"""The allocation-free Linear entry point against the regular one.

`mxq_mx_linear_static` is for callers that may not allocate device memory (a host application that hands a plugin
only input and output buffers, a serving loop with a frozen pool): its activation scratch is a fixed array inside the
library instead of a workspace argument.  The file name sorts last on purpose so that a run that stops at the first
failure has already executed every other test.
"""

import ctypes

import pytest
import torch

from mase_b200 import _lib, gemm, synthetic
from mase_b200.quantizers import _floor_tab_ptr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 1e-3
STATIC_BYTES = 40 << 20


def _run(entry, x, wp, out, workspace=None):
    lib = _lib.lib()
    M, K = x.shape
    st = gemm._status(x.device)
    stream = torch.cuda.current_stream().cuda_stream
    common = (x.data_ptr(), 1, wp.codes.data_ptr(), wp.scales.data_ptr(), out.data_ptr(), None, 1, 0, M, wp.rows, K, 4, 3,
              _floor_tab_ptr())
    if entry == "static":
        rc = lib.mxq_mx_linear_static(*common, st.data_ptr(), stream)
    else:
        rc = lib.mxq_mx_linear(*common, workspace.data_ptr(), workspace.numel(), st.data_ptr(), stream)
    return rc


def test_static_scratch_entry_matches_workspace_entry_twice():
    lib = _lib.lib()
    torch.cuda.set_device(0)
    # two calls in a row with different shapes: the second one finds the first one's leftovers in the scratch
    for M, K, N in ((384, 1024, 512), (100, 512, 768)):
        seed = M + K
        x, w = synthetic.linear_operands(M, K, N, seed=seed)
        x = x.to(DEV)
        wp = gemm.pack_mx_operand(w.to(DEV), 4, 3)
        ws = torch.empty(int(lib.mxq_mx_linear_workspace_bytes(M, K)), dtype=torch.uint8, device=DEV)
        ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert _run("workspace", x, wp, ref, ws) == 0
        before = torch.cuda.memory_allocated()
        assert _run("static", x, wp, out) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # nothing was taken from torch's allocator either
        gemm.check_status()
        assert not torch.isnan(out.float()).any()
        err = float((out.float() - ref.float()).abs().max() / ref.float().abs().max())
        assert err <= REL_TOL, f"static vs workspace entry differ by {err}"


def test_static_scratch_entry_rejects_oversized_problems():
    lib = _lib.lib()
    M, K = 16384, 4096  # needs ~66 MiB of scratch
    assert int(lib.mxq_mx_linear_workspace_bytes(M, K)) > STATIC_BYTES
    x = torch.zeros(8, 32, dtype=torch.bfloat16, device=DEV)  # never touched: the size check comes first
    st = gemm._status(x.device)
    rc = lib.mxq_mx_linear_static(x.data_ptr(), 1, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 1, 0, M, 256, K, 4, 3,
                                  _floor_tab_ptr(), st.data_ptr(), None)
    assert rc == -9
    assert b"MXQ_STATIC_SCRATCH_BYTES" in lib.mxq_error_string(rc)
