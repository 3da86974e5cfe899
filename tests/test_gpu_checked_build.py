"""The kernels under the checked build (-DGACB_CHECKED=1): every gather offset, record-table slot and output index
is range-checked on the device and counted when it leaves its tensor.  The small-case, random-shape and
record-table parity tests run again through ``libgacb_checked.so``; they must pass AND leave the violation count
where it was.  Outputs and scratch buffers are also embedded between canary words that must survive.

This is the stand-in for a memory checker (none can be run on the GPU pool) and for the reference's static
guards (native/lib/DeviceLowering.cpp:251-286, native/runtime/dispatch-plan.h:609-627).
"""

from __future__ import annotations

import ctypes

import numpy as np
import pytest

import test_gpu_dcn as dcn_tests
import test_gpu_msda as msda_tests
import test_gpu_random_shapes as random_tests
from conftest import assert_fp32_gate, load_cases

pytestmark = pytest.mark.gpu


def _violations(lib):
    count, site = ctypes.c_uint(0), ctypes.c_uint(0)
    assert lib.gacb_checked_violations(ctypes.byref(count), ctypes.byref(site)) == 0
    return count.value, site.value


@pytest.fixture(scope="module")
def dev():
    import torch

    from general_ai_compiler_b200 import ops

    return torch, ops, ops.require_device(0)


@pytest.fixture()
def checked(dev):
    """Route the package's calls through the checked build for one test; no new violation may appear."""
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.build import build_variants

    if not native.CHECKED_LIB_PATH.exists():
        build_variants()
    with native.use_library(native.CHECKED_LIB_PATH) as lib:
        before, _ = _violations(lib)
        yield lib
        dev[0].cuda.synchronize()
        after, site = _violations(lib)
    assert after == before, f"{after - before} out-of-range indices inside the kernels, last at site {site}"


def test_normal_build_says_it_is_not_checked():
    from general_ai_compiler_b200 import native

    assert native.load().gacb_checked_violations(None, None) == native.GACB_ERR_UNSUPPORTED


@pytest.mark.parametrize("case", sorted(load_cases("msda_small.npz")))
def test_msda_fixture_cases(case, msda_small, dev, checked):
    msda_tests.test_small_cases_fp32(case, msda_small, dev)
    if case.startswith("cfg_") or case.startswith("dim"):
        msda_tests.test_small_cases_bf16_value(case, msda_small, dev)


@pytest.mark.parametrize("seed", range(0, 24, 2))
def test_msda_random_shapes(seed, dev, checked):
    random_tests.test_msda_random_shapes(seed, dev)


def test_msda_tile_kernel_and_query_shards(dev, checked):
    msda_tests.test_tile_kernel_is_bit_identical_to_the_rows_kernel("tiny_tsa", dev)
    msda_tests.test_tile_kernel_samples_far_from_their_cell_and_softmax_form(dev)
    msda_tests.test_query_sharding_is_bit_identical(dev)


@pytest.mark.parametrize("tensor_path", [False, True])
@pytest.mark.parametrize("seed", range(0, 14, 2))
def test_dcn_random_shapes(seed, tensor_path, dev, checked):
    random_tests.test_dcn_random_shapes(seed, tensor_path, dev)


@pytest.mark.parametrize("seed", range(0, 10, 3))
def test_conv2d_random_shapes(seed, dev, checked):
    random_tests.test_conv2d_random_shapes(seed, dev)


@pytest.mark.parametrize("seed", range(0, 12, 4))
def test_window_convolution_random_shapes(seed, dev, checked):
    random_tests.test_window_convolution_random_shapes(seed, dev)


@pytest.mark.parametrize("label,wl_args", [
    ("two_deformable_groups", dict(cin=128, cout=64, deform_groups=2)),
    ("groups_and_deformable_groups", dict(cin=256, cout=128, groups=2, deform_groups=4)),
    ("five_by_five", dict(cin=64, cout=64, kernel=(5, 5), padding=(2, 2))),
    # the shapes whose record table once overflowed: a convolution group straddling two deformable groups
    ("three_groups_two_deformable", dict(cin=384, cout=96, groups=3, deform_groups=2, kernel=(3, 1), padding=(1, 0))),
    ("straddling_groups_full_kernel", dict(cin=384, cout=96, groups=3, deform_groups=2)),
])
def test_dcn_record_table_variants(label, wl_args, dev, checked):
    dcn_tests.test_tensor_path_record_table_variants(dev, label, wl_args)


def test_dcn_shards_and_narrow_tiles(dev, checked):
    dcn_tests.test_pixel_block_sharding_is_bit_identical(dev, 64, 4)
    dcn_tests.test_row_block_sharding_is_bit_identical(dev, 64, "bf16")
    dcn_tests.test_narrow_channel_tiles_beyond_one_wave(dev, "narrow_tiles_records_once", dict(cin=64, cout=48))


def test_canaries_around_outputs_and_scratch_survive(dev, checked):
    """Outputs and the DCNv2 workspace sit between sentinel words; the kernels may write the payload only."""
    from general_ai_compiler_b200.bevformer import DcnWorkload, WORKLOADS, make_workload_inputs
    from oracle import dcnv2_c, msda_c

    torch, ops, device = dev
    pad, mark = 256, -123456.0

    def guarded(shape):
        n = int(np.prod(shape))
        buf = torch.full((n + 2 * pad,), mark, dtype=torch.float32, device=device)
        return buf, buf[pad:pad + n].view(shape)

    def intact(buf):
        return bool(torch.all(buf[:pad] == mark)) and bool(torch.all(buf[-pad:] == mark))

    w = WORKLOADS["base_sca"].with_queries(97)
    x = make_workload_inputs(w)
    t = {k: torch.from_numpy(v).to(device) for k, v in x.items()}
    for value in (t["value"], ops.cast_to_bf16(t["value"])):
        buf, out = guarded((w.batch, w.queries, w.heads * w.head_dim))
        ops.msda_forward(value, t["sampling_locations"], t["attention_weights"], w.spatial_shapes, out=out)
        torch.cuda.synchronize()
        assert intact(buf)
    assert_fp32_gate(ops.msda_forward(t["value"], t["sampling_locations"], t["attention_weights"], w.spatial_shapes).cpu().numpy(),
                     msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes), "msda")

    wl = DcnWorkload("canary", 2, 64, 21, 27, 80, seed=9)
    z = make_workload_inputs(wl)
    tz = {k: torch.from_numpy(v).to(device) for k, v in z.items()}
    ho, wo = wl.out_hw
    want = dcnv2_c(z["X"], z["offset"], z["mask"], z["W"], z["bias"], stride=wl.stride, padding=wl.padding, dilation=wl.dilation)
    for math in ("f32x3", "tf32", "bf16"):
        need = ops.dcnv2_workspace_bytes(2, 64, 21, 27, 80, 3, 3, wl.stride, wl.padding, wl.dilation, 1, 1, math)
        assert need > 0
        ws_buf = torch.full((need + 2 * 1024,), 0x5A, dtype=torch.uint8, device=device)
        ws = ws_buf[1024:1024 + need]
        assert ws.data_ptr() % 256 == 0
        buf, out = guarded((2, 80, ho, wo))
        status = torch.zeros(1, dtype=torch.int32, device=device)
        ops.dcnv2_forward(tz["X"], tz["offset"], tz["mask"], tz["W"], tz["bias"], stride=wl.stride, padding=wl.padding,
                          dilation=wl.dilation, math=math, out=out, workspace=ws, status_word=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0 and intact(buf)
        assert bool(torch.all(ws_buf[:1024] == 0x5A)) and bool(torch.all(ws_buf[-1024:] == 0x5A))
        if math == "f32x3":
            assert_fp32_gate(out.cpu().numpy(), want, "dcn f32x3")
