"""CPU-only checks: the C-ABI library loads and exports what include/mxq.h declares, host-side helpers."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import mase_b200 as mb
from mase_b200 import _lib, build, log2_tables, quantizers
from oracle import mx_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def library():
    build.build()
    return _lib.lib()


def test_library_exports_every_declared_symbol(library):
    header = open(os.path.join(ROOT, "include", "mxq.h")).read()
    declared = set(re.findall(r"\b(mxq_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in declared:
        assert hasattr(library, name), f"{name} declared in include/mxq.h but not exported"
    assert declared == set(_lib.exported_symbols()), "ctypes prototypes and header disagree"
    assert library.mxq_version() == 1
    assert library.mxq_error_string(-4) == b"pointer is not 16-byte aligned"


def test_argument_validation_without_gpu(library):
    """Bad arguments are rejected before anything is launched."""
    tab = (ctypes.c_uint8 * 256)()
    assert library.mxq_mxint_fake(None, None, 0, 0, 4, 32, 8, tab, None) == -5
    assert library.mxq_mxint_fake(16, 16, 0, 0, -1, 32, 8, tab, None) == -2
    assert library.mxq_mxint_fake(16, 16, 0, 0, 4, 32, 9, tab, None) == -3
    assert library.mxq_mxfp_fake(16, 16, 0, 0, 4, 32, 3, 3, tab, None) == -3
    assert library.mxq_mxfp_fake(16, 16, 7, 0, 4, 32, 4, 3, tab, None) == -1
    assert library.mxq_mxfp_fake(16, 16, 0, 0, 0, 32, 4, 3, tab, None) == 0  # empty: nothing to do
    assert library.mxq_bfp_fake(16, 16, 0, 4, 64, 32, 40, 8, 127, tab, None) == -3


def test_gemm_options_travel_with_the_call(library):
    """The library has no process-wide settings: options are a struct passed per call, mirrored by ctypes, and the
    Python-side `gemm.options` context is per thread."""
    import threading

    from mase_b200 import gemm

    assert library.mxq_gemm_options_size() == ctypes.sizeof(_lib.GemmOptions) == 32
    for gone in ("mxq_gemm_set_max_ctas", "mxq_gemm_set_pair_mode", "mxq_gemm_set_split_k"):
        assert not hasattr(library, gone)
    assert gemm._options_ptr() is None
    seen = {}
    barrier = threading.Barrier(2)

    def worker(name, **fields):
        with gemm.options(**fields):
            barrier.wait()  # both threads are inside their blocks at the same time
            o = _lib.GemmOptions.from_address(gemm._options_ptr())
            seen[name] = (o.max_ctas, o.tiles, o.no_split_k)
            with gemm.options(no_split_k=1):  # nested: inherits the outer fields
                o = _lib.GemmOptions.from_address(gemm._options_ptr())
                seen[name + "/inner"] = (o.max_ctas, o.tiles, o.no_split_k)
            barrier.wait()
        seen[name + "/after"] = gemm._options_ptr()

    threads = [threading.Thread(target=worker, args=("a",), kwargs={"max_ctas": 100, "tiles": _lib.TILES_SINGLE}),
               threading.Thread(target=worker, args=("b",), kwargs={"tiles": _lib.TILES_PAIRS})]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert seen["a"] == (100, 1, 0) and seen["b"] == (0, 2, 0)
    assert seen["a/inner"] == (100, 1, 1) and seen["b/inner"] == (0, 2, 1)
    assert seen["a/after"] is None and seen["b/after"] is None
    assert gemm._options_ptr() is None
    # argument validation happens before any launch, with and without options
    opts = _lib.GemmOptions(max_ctas=8)
    assert library.mxq_gemm_mxf8(None, None, None, None, 0, None, None, 1, 0, 4, 4, 32, None, ctypes.addressof(opts), None) == -5
    assert library.mxq_gemm_mxf8(32, 32, 32, 32, 7, 32, None, 1, 0, 4, 4, 32, None, None, None) == -3  # unknown codes layout
    assert library.mxq_gemm_dense(16, 16, 16, None, 5, 1, 0, 4, 4, 32, None, None, None) == -1
    assert library.mxq_mx_linear_workspace_bytes(8192, 4096) == 8192 * 4096 + 64 * 32 * 512


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_PATH", "/nonexistent/libmxq.so")
    with pytest.raises(_lib.MxqError):
        _lib.lib()


def test_cpu_tensors_are_rejected():
    for call in (
        lambda: mb.mxint_quantizer(torch.randn(2, 32), 32, 8),
        lambda: mb.mxfp_quantizer(torch.randn(2, 32), 32, 4, 3),
        lambda: mb.block_fp_quantizer(torch.randn(2, 32), 8, 8, 127, [1, 32]),
        lambda: mb.minifloat_quantizer_sim(torch.randn(2, 32), mb.MinifloatMeta(4, 3, True, "rn")),
    ):
        with pytest.raises(RuntimeError, match="CUDA"):
            call()


def test_log2_tables_reproduce_host_log2():
    """Applying the tables to the exact integer log2 equals torch.log2 + ceil/floor for random and edge values."""
    g = torch.Generator().manual_seed(0)
    ex = torch.randint(1, 255, (200000,), generator=g, dtype=torch.int32)
    near = torch.randint(0, 64, (200000,), generator=g, dtype=torch.int32)
    far = torch.randint(0, 1 << 23, (200000,), generator=g, dtype=torch.int32)
    for man in (near, (1 << 23) - 1 - near, far):
        x = ((ex << 23) | man).view(torch.float32)
        ct = torch.from_numpy(log2_tables.ceil_table(torch.float32).astype(np.int32))
        got = ex - 127 + (man > ct[ex.long()]).int()
        assert torch.equal(got, torch.log2(x).ceil().int())
        ft = torch.from_numpy(log2_tables.floor_table().astype(np.int32))
        got = ex - 127 + (((1 << 23) - 1 - man) < ft[ex.long()]).int()
        assert torch.equal(got, torch.log2(x).floor().int())
    # bf16: exhaustive over all positive normal values
    bits = torch.arange(1 << 7, 255 << 7, dtype=torch.int32)
    xb = bits.to(torch.int16).view(torch.bfloat16)
    bt = torch.from_numpy(log2_tables.ceil_table(torch.bfloat16).astype(np.int32))
    got = (bits >> 7) - 127 + ((bits & 0x7F) > bt[(bits >> 7).long()]).int()
    assert torch.equal(got, torch.log2(xb).ceil().int())


def test_permute_helpers_match_oracle():
    x = torch.arange(2 * 3 * 4 * 5).reshape(2, 3, 4, 5)
    for d in (-1, 0, 1, 2, 3, -3):
        flat = quantizers.flatten_for_quantize(x, d)
        assert torch.equal(flat, O.flatten_blocks(x, d))
        back = quantizers.permute_for_dequantize(flat, tuple(x.shape), d)
        assert torch.equal(back, x)


def test_bfp_tile_inference():
    t = quantizers._bfp_tile
    assert t((64, 128), [1, 16], True) == (1, 16)
    assert t((64, 128), [16], True) == (1, 16)          # 2-D activation: first dim is never blocked
    assert t((64, 128), [8, 16], True) == (1, 16)
    assert t((64, 128), [1, 16], False) == (1, 16)
    assert t((64, 128), [1, 256], False) == (1, 128)    # oversize tile takes the whole row
    assert t((64, 128), [16], False) == (64, 16)        # 2-D weight, one entry: whole columns of 16
    assert t((64, 128), [16, 32], False) == (16, 32)
    assert t((96,), [16], False) == (1, 16)
    assert t((4, 7, 40), [1, 16], True) == (1, 16)
    assert t((4, 7, 40), [16], True) == (7, 16)         # 3-D activation, one entry: all tokens x 16 features
    assert t((4, 7, 40), [4, 16], True) == (4, 16)
    with pytest.raises(NotImplementedError):
        t((4, 7, 40), [1, 16], False)
    with pytest.raises(RuntimeError):
        t((2, 2, 2, 2), [16], True)
    with pytest.raises(AssertionError):
        t((96,), [16], True)


def test_meta_classes_validate_like_reference():
    with pytest.raises(AssertionError):
        mb.MXFPMeta(32, 8, 3, 3, True, "rn")
    with pytest.raises(AssertionError):
        mb.MXFPMeta(32, 4, 4, 3, True, "rn")
    m = mb.MXFPMeta(32, 8, 4, 3, True, "rn")
    assert m.element_meta.n_bits == 8
    assert set(mb.quantizer_map) == {"mxfp", "mxint", "block_fp"}
    assert set(mb.quantized_module_map) == {"linear_mxfp", "linear_mxint", "linear_block_fp"}


def test_mxint_clipping_search_matches_reference_vectors(golden):
    """The calibration-time search is plain tensor code: on the CPU (through the private, device-agnostic function;
    the public entry points refuse CPU tensors) it reproduces the reference bit for bit, with and without
    activations, and so does extraction with a clipping percentile."""
    from conftest import assert_bits_equal
    from mase_b200 import quantizers as Q

    for case in (c for c in golden.cases if c["kind"] == "mxint_search"):
        dt, nbits = case["dtype"], case["bits"]
        x = golden.tensor(f"mxint_search/{dt}/x", dt)
        act = golden.tensor(f"mxint_search/{dt}/act", dt)
        meta = Q.MXIntMeta(block_size=32, scale_bits=8, element_bits=nbits)
        y = Q._mxint_clip_search(x, 1, meta, None, 32).to(x.dtype)
        assert_bits_equal(y, golden.tensor(f"mxint_search/{dt}/w{nbits}/fake", dt), f"search {dt} w{nbits}")
        y = Q._mxint_clip_search(x, 1, meta, act, 2).to(x.dtype)
        assert_bits_equal(y, golden.tensor(f"mxint_search/{dt}/w{nbits}/fake_act", dt), f"search+act {dt} w{nbits}")
        # the search picks, block by block, one of the 11 clipped quantizations
        blocks = x.flatten().reshape(-1, 32)
        cand = Q._mxint_candidates(blocks, meta, torch.tensor(Q._SEARCH_PERCENTILES, dtype=torch.float32))
        hit = (cand.view(11, -1, 32) == y.reshape(1, -1, 32)).all(dim=2).any(dim=0)
        assert bool(hit.all())


def test_gptq_checkpoints_and_layer_discovery(tmp_path):
    """Host-side parts of the GPTQ pass: Linear discovery, per-layer checkpoint files and the resume rule (only a
    consecutive run of layers starting at 0 is loaded; a damaged file ends it)."""
    import pytest
    from mase_b200 import gptq

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = torch.nn.ModuleDict({"q_proj": torch.nn.Linear(8, 8, bias=False)})
            self.mlp = torch.nn.ModuleDict({"up_proj": torch.nn.Linear(8, 16, bias=False)})
            self.norm = torch.nn.LayerNorm(8)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.model = torch.nn.Module()
            self.model.layers = torch.nn.ModuleList([Block() for _ in range(4)])

    torch.manual_seed(0)
    src, dst = Net(), Net()
    assert set(gptq.find_qlayers(src.model.layers[0])) == {"self_attn.q_proj", "mlp.up_proj"}
    ckpt = tmp_path / "c"
    for i in (0, 1, 3):  # layer 2 is missing: the resume stops after layer 1
        gptq.save_layer_checkpoint(src, i, str(ckpt))
    assert set(gptq.detect_quantized_layers(str(ckpt))) == {0, 1, 3}
    assert gptq.auto_load_quantized_layers(dst, str(ckpt)) == 1
    for i, same in ((0, True), (1, True), (3, False)):
        a, b = src.model.layers[i].mlp["up_proj"].weight, dst.model.layers[i].mlp["up_proj"].weight
        assert torch.equal(a, b) == same
    (ckpt / "quantized_model_layer_1.safetensors").write_bytes(b"not a checkpoint")
    assert gptq.auto_load_quantized_layers(Net(), str(ckpt)) == 0
    assert gptq.auto_load_quantized_layers(Net(), str(tmp_path / "absent")) == -1
    with pytest.raises(RuntimeError):
        gptq.GPTQ(torch.nn.Linear(8, 8))  # a CPU layer: no CPU path
    with pytest.raises(ValueError):
        gptq.run_gptq(Net(), {"format": "mxint", "weight_config": {}})
