"""The allocation-free DCNv2 entry point, checked against the workspace-taking one through the raw C ABI.

Some hosts plan every byte of device memory before the first inference (a fixed arena, a plugin slot in another
engine, a real-time loop that cannot afford cudaMalloc's device-wide synchronisation) and so cannot supply the
scratch buffer ``gacb_dcnv2_forward`` asks for.  ``gacb_dcnv2_forward_static`` keeps that scratch inside the
library.  The test does not depend on what ran before it in the process: the first call on the device does the
one-time address lookup, whether or not other entry points were used earlier.
"""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_fp32_gate

pytestmark = pytest.mark.gpu


def _case(torch, device, batch, cin, h, w, cout, seed):
    from general_ai_compiler_b200.bevformer import DcnWorkload, make_workload_inputs

    wl = DcnWorkload("noalloc", batch, cin, h, w, cout, seed=seed)
    host = make_workload_inputs(wl)
    dev = {k: torch.from_numpy(v).to(device) for k, v in host.items()}
    return wl, host, dev


def _dims(wl):
    return (wl.batch, wl.cin, wl.height, wl.width, wl.cout, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1)


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    import torch

    from general_ai_compiler_b200 import native, ops
    from oracle import dcnv2_c

    device = ops.require_device(0)
    lib = native.load()
    stream = int(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second must not see anything the first left in the shared scratch
    for batch, cin, h, w, cout, seed in ((2, 64, 20, 24, 128, 41), (3, 128, 11, 13, 64, 42)):
        wl, host, t = _case(torch, device, batch, cin, h, w, cout, seed)
        ho, wo = wl.out_hw
        need = lib.gacb_dcnv2_workspace_bytes(*_dims(wl), native.DCN_F32X3)
        assert 0 < need <= (40 << 20)
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        y_ws = torch.zeros((batch, cout, ho, wo), device=device)
        y_static = torch.full((batch, cout, ho, wo), float("nan"), device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        ptrs = [t[k].data_ptr() for k in ("X", "offset", "mask", "W", "bias")]
        rc = lib.gacb_dcnv2_forward(*ptrs, y_ws.data_ptr(), *_dims(wl), 0, batch, native.DCN_F32X3, ws.data_ptr(),
                                    need, status.data_ptr(), stream)
        assert rc == 0, native.last_error()
        rc = lib.gacb_dcnv2_forward_static(*ptrs, y_static.data_ptr(), *_dims(wl), 0, batch, native.DCN_F32X3,
                                           status.data_ptr(), stream)
        assert rc == 0, native.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_fp32_gate(y_static.cpu().numpy(), y_ws.cpu().numpy(), "static scratch vs caller workspace")
        want = dcnv2_c(host["X"], host["offset"], host["mask"], host["W"], host["bias"], stride=wl.stride,
                       padding=wl.padding, dilation=wl.dilation)
        assert_fp32_gate(y_static.cpu().numpy(), want, "static scratch vs oracle")


def test_static_scratch_entry_rejects_oversized_calls_before_launching():
    import torch

    from general_ai_compiler_b200 import native, ops

    device = ops.require_device(0)
    lib = native.load()
    dummy = torch.zeros(64, device=device)
    # eight stage-c4 images need 49.6 MB of scratch: more than the 40 MiB built in
    dims = (8, 256, 58, 100, 256, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1)
    assert lib.gacb_dcnv2_workspace_bytes(*dims, native.DCN_F32X3) > (40 << 20)
    p = dummy.data_ptr()
    rc = lib.gacb_dcnv2_forward_static(p, p, p, p, None, p, *dims, 0, 8, native.DCN_F32X3, None, None)
    assert rc == native.GACB_ERR_UNSUPPORTED
    assert "scratch" in native.last_error()
    # the same shape restricted to six images fits
    assert lib.gacb_dcnv2_workspace_bytes(6, *dims[1:], native.DCN_F32X3) <= (40 << 20)
    torch.cuda.synchronize()
