"""A bounded wait inside the DCNv2 kernel made to run out, and what the host does with it.

``libgacb_faultinject.so`` is the same source built with a short polling limit and one extra ``math_mode`` flag
that makes the weight loader issue none of its copies.  The tensor-core thread then never sees its first weight
stage; every bounded wait gives up, the kernel unwinds (producers stop touching the pipeline, the issuing thread
commits and waits for what it issued, tensor memory is freed), sets the caller's status word and returns by
itself.  Nothing faults, traps or spins without limit, and the context stays usable: the next launches in the same
process must pass parity.  The reference reports a failed device step as a failed session that refuses further runs
(src/gac/execution/cuda.py:457-464) and a ``status: "failed"`` report (native/runtime/cuda-run.cpp:685-703).
"""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_fp32_gate

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch

    from general_ai_compiler_b200 import ops

    return torch, ops, ops.require_device(0)


@pytest.fixture()
def fault_build():
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.build import build_variants

    if not native.FAULT_LIB_PATH.exists():
        build_variants()
    with native.use_library(native.FAULT_LIB_PATH) as lib:
        yield lib


def _case(torch, device, seed=21):
    from general_ai_compiler_b200.bevformer import DcnWorkload, make_workload_inputs
    from oracle import dcnv2_c

    wl = DcnWorkload("expiry", 1, 64, 20, 24, 128, seed=seed)
    host = make_workload_inputs(wl)
    want = dcnv2_c(host["X"], host["offset"], host["mask"], host["W"], host["bias"], stride=wl.stride,
                   padding=wl.padding, dilation=wl.dilation)
    return wl, host, {k: torch.from_numpy(v).to(device) for k, v in host.items()}, want


def test_the_normal_library_refuses_the_test_flag(dev):
    torch, ops, device = dev
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.errors import EvaluationError

    wl, _, t, _ = _case(torch, device)
    with pytest.raises(EvaluationError, match="unknown flag bits"):
        ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                          dilation=wl.dilation, math="bf16", test_flags=native.DCN_TEST_DROP_WEIGHT_COPIES)


@pytest.mark.parametrize("math", ["bf16", "f32x3"])
def test_expired_wait_sets_the_status_word_and_the_gpu_stays_usable(math, dev, fault_build):
    torch, ops, device = dev
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.errors import BackendError

    wl, _, t, want = _case(torch, device)
    kw = dict(stride=wl.stride, padding=wl.padding, dilation=wl.dilation, math=math)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    out = ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], status_word=status,
                            test_flags=native.DCN_TEST_DROP_WEIGHT_COPIES, **kw)
    torch.cuda.synchronize()                      # the kernel came back by itself
    assert int(status.item()) == 1
    rc = fault_build.gacb_read_status_word(status.data_ptr(), None)
    assert rc == native.GACB_ERR_DEVICE_TIMEOUT
    with pytest.raises(BackendError, match="bounded wait"):
        native.check(rc, "status word")
    assert out.shape == want.shape                # contents are unspecified after a timeout
    # tensor memory was released and the pipeline state is gone: the same build, without the flag, is correct
    status.zero_()
    good = ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], status_word=status, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and fault_build.gacb_read_status_word(status.data_ptr(), None) == native.GACB_OK
    if math == "f32x3":
        assert_fp32_gate(good.cpu().numpy(), want, "after an expired wait")
    else:
        assert float(np.abs(good.cpu().numpy() - want).max()) <= 1e-2 * float(np.abs(want).max())


def test_expired_wait_in_the_window_kernel_of_plain_convolutions(dev, fault_build):
    """The persistent window kernel has its own pipeline (window ring, weight ring, two accumulator sets): with the
    weight copies dropped its tensor-core thread gives up on the first stage, every role unwinds, the status word is
    set, and the next call of the same kernel is correct."""
    torch, ops, device = dev
    from general_ai_compiler_b200 import native
    from oracle import conv2d_c

    rng = np.random.default_rng(31)
    x = rng.standard_normal((2, 64, 40, 30)).astype(np.float32)
    w = (rng.standard_normal((27, 64, 3, 3)) * 0.05).astype(np.float32)
    geo = native.dcnv2_launch_geometry(2, 64, 40, 30, 27, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, native.DCN_BF16, plain=True)
    assert geo.kernel == b"conv_window_kernel<bf16>"
    xd, wd = torch.from_numpy(x).to(device), torch.from_numpy(w).to(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    ops.conv2d_forward(xd, wd, None, pads=(1, 1, 1, 1), math="bf16", status_word=status,
                       test_flags=native.DCN_TEST_DROP_WEIGHT_COPIES)
    torch.cuda.synchronize()                      # the kernel came back by itself
    assert int(status.item()) == 1
    assert fault_build.gacb_read_status_word(status.data_ptr(), None) == native.GACB_ERR_DEVICE_TIMEOUT
    status.zero_()
    good = ops.conv2d_forward(xd, wd, None, pads=(1, 1, 1, 1), math="bf16", status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    rounded = [torch.from_numpy(v).to(torch.bfloat16).float().numpy() for v in (x, w)]
    assert_fp32_gate(good.cpu().numpy(), conv2d_c(rounded[0], rounded[1], None, pads=(1, 1, 1, 1)), "after an expired wait")


def test_session_raises_and_invalidates_itself_after_an_expired_wait(dev, fault_build):
    torch, ops, device = dev
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.bevformer import build_dcn_graph_for
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.errors import BackendError
    from general_ai_compiler_b200.session import CudaSession

    wl, host, _, want = _case(torch, device, seed=22)
    program = compile_cuda(build_dcn_graph_for(wl))
    program.options["dcn_test_flags"] = native.DCN_TEST_DROP_WEIGHT_COPIES
    session = CudaSession(program)
    with pytest.raises(BackendError, match="bounded wait"):
        session.run(host)
    with pytest.raises(BackendError, match="closed or failed"):       # the reference's rule: create a new session
        session.run(host)
    session.close()
    program.options.pop("dcn_test_flags")
    with CudaSession(program) as fresh:
        assert_fp32_gate(fresh.run(host).outputs["Y"], want, "fresh session after a failed one")


def test_the_normal_library_is_unaffected_afterwards(dev):
    torch, ops, device = dev
    wl, _, t, want = _case(torch, device, seed=23)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    y = ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], stride=wl.stride, padding=wl.padding,
                          dilation=wl.dilation, math="f32x3", status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_fp32_gate(y.cpu().numpy(), want, "normal library")
