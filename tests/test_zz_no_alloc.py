"""The allocation-free Linear entry point against the regular one.

`mxq_mx_linear_static` is for callers that may not allocate device memory (a host application that hands a plugin
only input and output buffers, a serving loop with a frozen pool): its activation scratch is a fixed array inside the
library instead of a workspace argument.  The file name sorts last on purpose so that a run that stops at the first
failure has already executed every other test.
"""

import pytest
import torch

from mase_b200 import _lib, gemm, synthetic
from mase_b200.quantizers import _floor_tab_ptr
from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL_TOL = 4e-3  # bf16 output against the fp32 oracle: half an ulp is 2**-9 of the value
STATIC_BYTES = 40 << 20


def _run(entry, x, wp, out, workspace=None):
    lib = _lib.lib()
    M, K = x.shape
    st = gemm._status(x.device)
    stream = torch.cuda.current_stream().cuda_stream
    common = (x.data_ptr(), 1, wp.codes.data_ptr(), wp.scales.data_ptr(), wp.format, out.data_ptr(), None, 1, 0, M, wp.rows,
              K, 4, 3, _floor_tab_ptr())
    if entry == "static":
        rc = lib.mxq_mx_linear_static(*common, st.data_ptr(), None, stream)
    else:
        rc = lib.mxq_mx_linear(*common, workspace.data_ptr(), workspace.numel(), st.data_ptr(), None, stream)
    return rc


def test_static_scratch_entry_matches_workspace_entry_on_calls_in_a_row():
    """Calls in a row with different shapes: each one finds the previous one's leftovers in the shared array.  The
    shapes cover CTA pairs, single-CTA tiles, the transposed small-M kernel and K % 128 != 0 (whose scale region holds
    an earlier call's bytes until the pack clears it).  Results must be the bits of the workspace entry, within
    the bf16 bar of the oracle, and neither torch's allocator nor the device's free memory may move."""
    lib = _lib.lib()
    torch.cuda.set_device(0)
    # the first use of either entry point may load kernels (lazy module loading takes device memory once)
    x0, w0 = synthetic.linear_operands(8, 128, 64, seed=1)
    wp0 = gemm.pack_mx_operand(w0.to(DEV), 4, 3)
    warm = torch.empty(8, 64, dtype=torch.bfloat16, device=DEV)
    assert _run("static", x0.to(DEV), wp0, warm) == 0
    torch.cuda.synchronize()
    for M, K, N in ((640, 1024, 512), (384, 1024, 512), (100, 160, 96), (100, 512, 768), (1024, 2048, 256)):
        seed = M + K
        x, w = synthetic.linear_operands(M, K, N, seed=seed)
        xd = x.to(DEV)
        wp = gemm.pack_mx_operand(w.to(DEV), 4, 3)
        ws = torch.empty(int(lib.mxq_mx_linear_workspace_bytes(M, K)), dtype=torch.uint8, device=DEV)
        ref = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        assert _run("workspace", xd, wp, ref, ws) == 0
        assert _run("static", xd, wp, out) == 0  # lazily loads whatever this shape's kernels still need
        torch.cuda.synchronize()
        out.fill_(float("nan"))
        torch_before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        assert _run("static", xd, wp, out) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == torch_before  # nothing came from torch's allocator
        assert torch.cuda.mem_get_info()[0] >= free_before    # and nothing from the device itself
        gemm.check_status()
        assert not torch.isnan(out.float()).any()
        assert torch.equal(out, ref), f"static and workspace entry differ for {(M, K, N)}"
        oracle = O.mxfp_fake(x, 32, 4, 3).float() @ O.mxfp_fake(w, 32, 4, 3, 1).float().t()
        err = float((out.float().cpu() - oracle).abs().max() / oracle.abs().max())
        assert err <= REL_TOL, f"static entry is {err} from the oracle for {(M, K, N)}"


def test_static_scratch_entry_rejects_oversized_problems():
    lib = _lib.lib()
    M, K = 16384, 4096  # needs ~66 MiB of scratch
    assert int(lib.mxq_mx_linear_workspace_bytes(M, K)) > STATIC_BYTES
    x = torch.zeros(8, 32, dtype=torch.bfloat16, device=DEV)  # never touched: the size check comes first
    st = gemm._status(x.device)
    rc = lib.mxq_mx_linear_static(x.data_ptr(), 1, x.data_ptr(), x.data_ptr(), 0, x.data_ptr(), None, 1, 0, M, 256, K, 4, 3,
                                  _floor_tab_ptr(), st.data_ptr(), None, None)
    assert rc == -9
    assert b"MXQ_STATIC_SCRATCH_BYTES" in lib.mxq_error_string(rc)
