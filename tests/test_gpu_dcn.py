"""DCNv2 parity on the B200 through the C ABI; the C oracle (pinned to torchvision's operator) only checks."""

from __future__ import annotations

import zlib

import numpy as np
import pytest

from conftest import assert_fp32_gate, assert_rel_gate, load_cases

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch

    from general_ai_compiler_b200 import ops

    return torch, ops, ops.require_device(0)


def _run(dev, c, math="f32x3", n_range=None, out=None, row_range=None, pixel_range=None):
    torch, ops, device = dev
    a = [int(v) for v in c["attrs"]]
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("X", "offset", "mask", "W")}
    bias = torch.from_numpy(c["bias"]).to(device) if "bias" in c else None
    status = torch.zeros(1, dtype=torch.int32, device=device)
    y = ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], bias, stride=a[0:2], padding=a[2:4], dilation=a[4:6],
                          groups=a[6], deform_groups=a[7], math=math, n_range=n_range, out=out, status_word=status,
                          row_range=row_range, pixel_range=pixel_range)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired inside the kernel"
    return y


def _workload_case(wl):
    from general_ai_compiler_b200.bevformer import make_workload_inputs

    x = make_workload_inputs(wl)
    x["attrs"] = np.asarray([*wl.stride, *wl.padding, *wl.dilation, wl.groups, wl.deform_groups], np.int32)
    return x


def test_tensor_core_path_smallest_case(dcn_small, dev):
    """First contact with the tcgen05 kernel: one 128-pixel tile row, 128 channels."""
    torch, ops, device = dev
    c = dcn_small["cfg_dcn_c5_cut"]
    assert ops.dcnv2_workspace_bytes(1, 128, 9, 11, 128, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, "f32x3") > 0
    y = _run(dev, c, "f32x3").cpu().numpy()
    assert_fp32_gate(y, c["expected"], "cfg_dcn_c5_cut f32x3")


@pytest.mark.parametrize("case", sorted(load_cases("dcn_small.npz")))
def test_reference_fixture_recipes(case, dcn_small, dev):
    c = dcn_small[case]
    y = _run(dev, c, "f32x3").cpu().numpy()
    np.testing.assert_allclose(y, c["expected"], rtol=2e-5, atol=2e-5, err_msg=case)


@pytest.mark.parametrize("math,rel", [("tf32", 1e-2), ("bf16", 1e-2)])
@pytest.mark.parametrize("case", ["cfg_dcn_c4_cut", "cfg_dcn_c5_cut"])
def test_reduced_precision_modes(case, math, rel, dcn_small, dev):
    c = dcn_small[case]
    assert_rel_gate(_run(dev, c, math).cpu().numpy(), c["expected"], rel, f"{case} {math}")


def test_zero_offsets_equal_plain_convolution(dev):
    torch, ops, device = dev
    rng = np.random.default_rng(4)
    x = torch.from_numpy(rng.standard_normal((2, 64, 17, 23)).astype(np.float32)).to(device)
    w = torch.from_numpy((rng.standard_normal((128, 64, 3, 3)) * 0.05).astype(np.float32)).to(device)
    b = torch.from_numpy(rng.standard_normal(128).astype(np.float32)).to(device)
    off = torch.zeros((2, 18, 17, 23), device=device)
    mask = torch.ones((2, 9, 17, 23), device=device)
    y = ops.dcnv2_forward(x, off, mask, w, b, padding=(1, 1), math="f32x3")
    ref = torch.nn.functional.conv2d(x.double(), w.double(), b.double(), padding=1).float()
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), ref.cpu().numpy(), "zero offsets vs conv2d")


@pytest.mark.parametrize("key", ["dcn_c4", "dcn_c5"])
def test_full_size_configurations(key, dcn_pins, dev):
    from general_ai_compiler_b200.bevformer import WORKLOADS
    from oracle import dcnv2_c

    wl = WORKLOADS[key]
    c = _workload_case(wl)
    oracle = dcnv2_c(c["X"], c["offset"], c["mask"], c["W"], c["bias"], stride=wl.stride, padding=wl.padding,
                     dilation=wl.dilation)
    pin = dcn_pins[key]
    np.testing.assert_allclose(oracle.reshape(-1)[pin["index"]], pin["expected"], rtol=2e-5, atol=2e-5)
    y = _run(dev, c, "f32x3").cpu().numpy()
    assert_fp32_gate(y, oracle, key + " f32x3")
    assert_fp32_gate(y.reshape(-1)[pin["index"]], pin["expected"], key + " pins (torchvision)")
    for math in ("tf32", "bf16"):
        assert_rel_gate(_run(dev, c, math).cpu().numpy(), oracle, 1e-2, f"{key} {math}")


def test_image_range_sharding_is_bit_identical(dev):
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import DcnWorkload

    c = _workload_case(DcnWorkload("shard", 5, 64, 19, 27, 64, seed=31))
    whole = _run(dev, c, "f32x3")
    out = torch.full_like(whole, float("nan"))
    for n0, n1 in ((0, 2), (2, 3), (3, 5)):
        _run(dev, c, "f32x3", n_range=(n0, n1), out=out)
    assert torch.equal(out, whole)
    part = torch.full_like(whole, 3.0)
    _run(dev, c, "f32x3", n_range=(1, 2), out=part)
    assert torch.all(part[0] == 3.0) and torch.all(part[2:] == 3.0) and torch.equal(part[1], whole[1])


@pytest.mark.parametrize("channels", [64, 16])   # 64: tensor-core path; 16: below its size threshold, CUDA-core path
@pytest.mark.parametrize("math", ["f32x3", "bf16"])
def test_row_block_sharding_is_bit_identical(dev, channels, math):
    """(camera, output-row block) pieces, as the balanced multi-GPU split issues them, rebuild the one-launch output
    bit for bit, and a piece writes nothing outside its rows."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import DcnWorkload
    from general_ai_compiler_b200.distributed import dcn_units

    c = _workload_case(DcnWorkload("rows", 3, channels, 19, 27, channels, seed=37))
    whole = _run(dev, c, math)
    out = torch.full_like(whole, float("nan"))
    units = dcn_units(3, 19, world=4)
    assert len(units) > 3 and {u[0] for u in units} == {0, 1, 2}
    for n, r0, r1 in units:
        _run(dev, c, math, n_range=(n, n + 1), row_range=(r0, r1), out=out)
    assert torch.equal(out, whole)
    part = torch.full_like(whole, 3.0)
    _run(dev, c, math, n_range=(0, 3), row_range=(5, 7), out=part)
    assert torch.equal(part[:, :, 5:7], whole[:, :, 5:7])
    assert torch.all(part[:, :, :5] == 3.0) and torch.all(part[:, :, 7:] == 3.0)
    _run(dev, c, math, row_range=(4, 4), out=part)                      # empty range: nothing happens
    assert torch.all(part[:, :, :5] == 3.0)
    with pytest.raises(Exception):
        _run(dev, c, math, row_range=(3, 20))


@pytest.mark.parametrize("channels", [64, 16])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_pixel_block_sharding_is_bit_identical(dev, channels, world):
    """Contiguous runs of the flattened (camera, row, column) output pixels -- one launch per rank, starting and
    ending in the middle of a camera -- rebuild the one-launch output bit for bit."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import DcnWorkload
    from general_ai_compiler_b200.distributed import dcn_pixel_block

    c = _workload_case(DcnWorkload("pixels", 3, channels, 19, 27, channels, seed=41))
    whole = _run(dev, c, "f32x3")
    out = torch.full_like(whole, float("nan"))
    blocks = [dcn_pixel_block(3, 19 * 27, world, r) for r in range(world)]
    assert blocks[0][0] == 0 and blocks[-1][1] == 3 * 19 * 27 and all(a[1] == b[0] for a, b in zip(blocks, blocks[1:]))
    for p0, p1 in blocks:
        _run(dev, c, "f32x3", pixel_range=(p0, p1), out=out)
    assert torch.equal(out, whole)
    part = torch.full_like(whole, 3.0)
    _run(dev, c, "f32x3", pixel_range=(500, 530), out=part)             # inside camera 0 (513 pixels) into camera 1
    flat_part = part.permute(0, 2, 3, 1).reshape(-1, channels)
    flat_whole = whole.permute(0, 2, 3, 1).reshape(-1, channels)
    assert torch.equal(flat_part[500:530], flat_whole[500:530])
    assert torch.all(flat_part[:500] == 3.0) and torch.all(flat_part[530:] == 3.0)
    with pytest.raises(Exception):
        _run(dev, c, "f32x3", pixel_range=(10, 3 * 19 * 27 + 1))
    with pytest.raises(Exception):
        _run(dev, c, "f32x3", pixel_range=(0, 10), n_range=(0, 1))


@pytest.mark.parametrize("label,wl_args", [
    ("two_deformable_groups", dict(cin=128, cout=64, deform_groups=2)),                  # 18 records per row: per-block records
    ("groups_and_deformable_groups", dict(cin=256, cout=128, groups=2, deform_groups=4)),  # 2 deformable groups per CTA
    ("five_by_five", dict(cin=64, cout=64, kernel=(5, 5), padding=(2, 2))),               # 25 kernel points
    ("two_by_two_strided", dict(cin=64, cout=96, kernel=(2, 2), padding=(0, 1), stride=(1, 2))),   # 4 records per row
    ("dilated", dict(cin=64, cout=64, dilation=(2, 3), padding=(2, 3))),
    # convolution groups and deformable groups that do not nest: a group's channels straddle two deformable groups
    ("three_groups_two_deformable", dict(cin=384, cout=96, groups=3, deform_groups=2, kernel=(3, 1), padding=(1, 0))),
    ("two_groups_three_deformable", dict(cin=384, cout=64, groups=2, deform_groups=3, kernel=(1, 3), padding=(0, 1))),
    ("straddling_groups_full_kernel", dict(cin=384, cout=96, groups=3, deform_groups=2)),        # 18 records: per-block path
])
def test_tensor_path_record_table_variants(dev, label, wl_args):
    """Shapes whose tap records are all made once per tile (few kernel points x deformable groups) and shapes where
    each producer group rebuilds them per K block, both against the C oracle."""
    from general_ai_compiler_b200.bevformer import DcnWorkload
    from oracle import dcnv2_c

    torch, ops, device = dev
    wl = DcnWorkload(label, 2, height=26, width=31, seed=53, **wl_args)
    c = _workload_case(wl)
    ho, wo = wl.out_hw
    assert ops.dcnv2_workspace_bytes(2, wl.cin, 26, 31, wl.cout, *wl.kernel, wl.stride, wl.padding, wl.dilation, wl.groups,
                                     wl.deform_groups, "f32x3") > 0, "meant to reach the tensor-core kernel"
    want = dcnv2_c(c["X"], c["offset"], c["mask"], c["W"], c["bias"], stride=wl.stride, padding=wl.padding,
                   dilation=wl.dilation, groups=wl.groups, deform_groups=wl.deform_groups)
    assert want.shape == (2, wl.cout, ho, wo)
    assert_fp32_gate(_run(dev, c, "f32x3").cpu().numpy(), want, label)
    for math in ("tf32", "bf16"):
        assert_rel_gate(_run(dev, c, math).cpu().numpy(), want, 1e-2, f"{label} {math}")


def test_workspace_reuse_flags(dev):
    """Packed weights and the channel-last copy left in the workspace by an earlier call can be reused: same bits;
    and the reuse really skips the step (changing W / X afterwards goes unnoticed, as documented)."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import DcnWorkload
    from general_ai_compiler_b200.errors import EvaluationError

    wl = DcnWorkload("reuse", 2, 64, 21, 28, 64, seed=61)
    c = _workload_case(wl)
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("X", "offset", "mask", "W", "bias")}
    need = ops.dcnv2_workspace_bytes(2, 64, 21, 28, 64, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, "f32x3")
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=device)

    def run(x, w, **kw):
        y = ops.dcnv2_forward(x, t["offset"], t["mask"], w, t["bias"], padding=(1, 1), workspace=ws, **kw)
        torch.cuda.synchronize()
        return y

    first = run(t["X"], t["W"])
    assert torch.equal(run(t["X"], t["W"], reuse_weights=True), first)
    assert torch.equal(run(t["X"], t["W"], reuse_weights=True, reuse_input=True), first)
    assert torch.equal(run(t["X"], t["W"] * 2, reuse_weights=True), first)              # stale weights are used
    assert torch.equal(run(t["X"] + 1, t["W"], reuse_input=True), first)                 # stale copy of X is used
    assert not torch.equal(run(t["X"], t["W"] * 2), first)
    # conv_offset on the same X and workspace leaves the copy that the deformable convolution then reuses
    w27 = torch.randn((27, 64, 3, 3), device=device) * 0.05
    ops.conv2d_forward(t["X"], w27, None, pads=(1, 1, 1, 1), workspace=ws)
    assert torch.equal(run(t["X"], t["W"], reuse_input=True), first)
    with pytest.raises(EvaluationError):
        ops.dcnv2_forward(t["X"], t["offset"], t["mask"], t["W"], t["bias"], padding=(1, 1), reuse_weights=True)
    lib = ops.native.load()
    rc = lib.gacb_dcnv2_forward(t["X"].data_ptr(), t["offset"].data_ptr(), t["mask"].data_ptr(), t["W"].data_ptr(), None,
                                first.data_ptr(), 2, 64, 21, 28, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 0, 2, 0x400, ws.data_ptr(), need,
                                None, None)
    assert rc == -1 and "flag" in ops.native.last_error()


@pytest.mark.parametrize("math", ["f32x3", "bf16"])
def test_conv_offset_and_dcn_share_one_input_copy(dev, math):
    """conv_offset and the DCNv2 it feeds read the same X: with the channel-last copy at the END of two workspaces
    that end at the same address, the first call makes the copy, the second reuses it, and both keep their own
    packed weights -- bit-identical to two calls with private workspaces, also in the steady state (nothing packed,
    one copy per block)."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import DcnWorkload

    wl = DcnWorkload("shared", 2, 64, 21, 28, 96, seed=71)
    c = _workload_case(wl)
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("X", "W", "bias")}
    w27 = (torch.randn((27, 64, 3, 3), device=device) * 0.05).contiguous()
    b27 = torch.randn(27, device=device)
    kw = dict(stride=(1, 1), padding=(1, 1), dilation=(1, 1), math=math)

    def block(x, conv_ws=None, dcn_ws=None, **flags):
        conv_flags = {k: v for k, v in flags.items() if k != "reuse_input"}
        off, mask = ops.conv2d_forward(x, w27, b27, pads=(1, 1, 1, 1), math=math, split_at=18, workspace=conv_ws, **conv_flags)
        y = ops.dcnv2_forward(x, off, mask, t["W"], t["bias"], mask_is_logits=True, workspace=dcn_ws, **kw, **flags)
        torch.cuda.synchronize()
        return off, mask, y

    want = block(t["X"])
    buf, conv_ws, dcn_ws = ops.shared_input_workspaces(t["X"], 27, 96, (3, 3), (1, 1), (1, 1), (1, 1), math=math)
    assert buf is not None and conv_ws.data_ptr() % 256 == 0 and dcn_ws.data_ptr() % 256 == 0
    assert conv_ws.data_ptr() + conv_ws.numel() == dcn_ws.data_ptr() + dcn_ws.numel()       # same end: same copy
    copy_bytes, weights = ops.workspace_parts(2, 64, 21, 28, 96, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, math)
    assert copy_bytes + weights == ops.dcnv2_workspace_bytes(2, 64, 21, 28, 96, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, math)
    buf.fill_(0xA5)
    got = block(t["X"], conv_ws, dcn_ws, input_at_end=True, reuse_input=True)
    assert all(torch.equal(g, w) for g, w in zip(got, want))
    steady = block(t["X"], conv_ws, dcn_ws, input_at_end=True, reuse_input=True, reuse_weights=True)
    assert all(torch.equal(g, w) for g, w in zip(steady, want))
    # the copy is really shared: a changed X is picked up by conv_offset's copy and seen by the DCNv2 that reuses it
    x2 = (t["X"] * 0.5 + 0.25).contiguous()
    want2 = block(x2)
    got2 = block(x2, conv_ws, dcn_ws, input_at_end=True, reuse_input=True, reuse_weights=True)
    assert all(torch.equal(g, w) for g, w in zip(got2, want2))


def test_direct_and_tensor_paths_agree(dev):
    """Cin=64 with dense weights takes the tensor-core path; the same problem viewed as 4 groups of 16 channels
    (block-diagonal weights) cannot be tiled and takes the CUDA-core path.  Both must agree to the fp32 gate."""
    torch, ops, device = dev
    rng = np.random.default_rng(9)
    x = torch.from_numpy(rng.standard_normal((1, 64, 40, 44)).astype(np.float32)).to(device)
    off = torch.from_numpy((rng.standard_normal((1, 18, 40, 44)) * 1.4).astype(np.float32)).to(device)
    mask = torch.sigmoid(torch.from_numpy(rng.standard_normal((1, 9, 40, 44)).astype(np.float32))).to(device)
    wg = torch.from_numpy((rng.standard_normal((64, 16, 3, 3)) * 0.06).astype(np.float32)).to(device)
    dense = torch.zeros((64, 64, 3, 3), device=device)
    for g in range(4):
        dense[16 * g:16 * g + 16, 16 * g:16 * g + 16] = wg[16 * g:16 * g + 16]
    assert ops.dcnv2_workspace_bytes(1, 64, 40, 44, 64, 3, 3, (1, 1), (1, 1), (1, 1), 4, 1, "f32x3") == 0
    assert ops.dcnv2_workspace_bytes(1, 64, 40, 44, 64, 3, 3, (1, 1), (1, 1), (1, 1), 1, 1, "f32x3") > 0
    y_direct = ops.dcnv2_forward(x, off, mask, wg, None, padding=(1, 1), groups=4, math="f32x3")
    y_tensor = ops.dcnv2_forward(x, off, mask, dense.contiguous(), None, padding=(1, 1), groups=1, math="f32x3")
    torch.cuda.synchronize()
    assert_fp32_gate(y_tensor.cpu().numpy(), y_direct.cpu().numpy(), "tensor vs direct")


def test_linearity_in_the_mask(dev):
    """Size-independent property at full size: halving the mask halves (y - bias)."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS

    c = _workload_case(WORKLOADS["dcn_c5"])
    y1 = _run(dev, c, "f32x3")
    c2 = dict(c, mask=(c["mask"] * np.float32(0.5)))
    y2 = _run(dev, c2, "f32x3")
    bias = torch.from_numpy(c["bias"]).to(device).reshape(1, -1, 1, 1)
    assert float(((y1 - bias) * 0.5 - (y2 - bias)).abs().max()) < 2e-5


@pytest.mark.parametrize("case", sorted(load_cases("dcn_fused.npz")))
def test_sigmoid_batchnorm_relu_folded_in(case, dcn_fused, dev):
    torch, ops, device = dev
    c = dcn_fused[case]
    use_bn, use_relu = (bool(v) for v in c["flags"])
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in c if k not in ("flags", "expected")}
    bn = (t["bn_scale"], t["bn_bias"], t["bn_mean"], t["bn_var"], 1e-5) if use_bn else None
    y = ops.dcnv2_forward(t["X"], t["offset"], t["mask_logits"], t["W"], t["bias"], padding=(1, 1), math="f32x3",
                          mask_is_logits=True, batch_norm=bn, relu=use_relu)
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), c["expected"], case)
    if use_relu:
        assert float(y.min()) >= 0.0
    # the separate route (sigmoid outside, plain kernel, BatchNorm/ReLU outside) agrees as well
    plain = ops.dcnv2_forward(t["X"], t["offset"], torch.sigmoid(t["mask_logits"]), t["W"], t["bias"], padding=(1, 1))
    if use_bn:
        shp = (1, -1, 1, 1)
        plain = (plain - t["bn_mean"].reshape(shp)) / torch.sqrt(t["bn_var"].reshape(shp) + 1e-5) * t["bn_scale"].reshape(shp) + t["bn_bias"].reshape(shp)
    if use_relu:
        plain = torch.relu(plain)
    assert float((y - plain).abs().max()) < 5e-5


def test_contract_violations(dev):
    torch, ops, device = dev
    from general_ai_compiler_b200 import native
    from general_ai_compiler_b200.errors import EvaluationError

    x = torch.zeros((1, 4, 5, 6), device=device)
    off = torch.zeros((1, 18, 5, 6), device=device)
    mask = torch.zeros((1, 9, 5, 6), device=device)
    w = torch.zeros((3, 4, 3, 3), device=device)
    with pytest.raises(EvaluationError, match="divisible"):
        ops.dcnv2_forward(x, off, mask, w, None, padding=(1, 1), groups=3)
    with pytest.raises(EvaluationError, match="offset/mask"):
        ops.dcnv2_forward(x, off[:, :-1].contiguous(), mask, w, None, padding=(1, 1))
    with pytest.raises(EvaluationError, match="exceeds"):
        ops.dcnv2_forward(torch.zeros((1, 4, 2, 2), device=device), off, mask, w, None, padding=(0, 0))
    lib = native.load()
    rc = lib.gacb_dcnv2_forward(x.data_ptr(), off.data_ptr(), mask.data_ptr(), w.data_ptr(), None, x.data_ptr(),
                                1, 4, 5, 6, 3, 3, 3, 1, 1, 1, 1, 1, 1, 3, 1, 0, 1, 0, None, 0, None, None)
    assert rc == native.GACB_ERR_SHAPE_MISMATCH
    rc = lib.gacb_dcnv2_forward(x.data_ptr(), off.data_ptr(), mask.data_ptr(), w.data_ptr(), None, x.data_ptr(),
                                1, 4, 5, 6, 3, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 0, 1, 7, None, 0, None, None)
    assert rc == native.GACB_ERR_INVALID_ARGUMENT
    # tensor-core shapes need the caller's workspace (every tensor correctly sized: nothing may be launched)
    xb = torch.zeros((1, 64, 40, 40), device=device)
    ob = torch.zeros((1, 18, 40, 40), device=device)
    mb = torch.zeros((1, 9, 40, 40), device=device)
    wb = torch.zeros((64, 64, 3, 3), device=device)
    yb = torch.zeros((1, 64, 40, 40), device=device)
    rc = lib.gacb_dcnv2_forward(xb.data_ptr(), ob.data_ptr(), mb.data_ptr(), wb.data_ptr(), None, yb.data_ptr(),
                                1, 64, 40, 40, 64, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, 0, 1, 0, None, 0, None, None)
    assert rc == native.GACB_ERR_INVALID_ARGUMENT and "workspace" in native.last_error()
    torch.cuda.synchronize()


def test_session_and_evaluate_op(dev, dcn_small):
    from general_ai_compiler_b200 import evaluate_op
    from general_ai_compiler_b200.bevformer import DcnWorkload, build_dcn_graph_for, make_workload_inputs
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.session import CudaSession
    from oracle import dcnv2_c

    wl = DcnWorkload("sess", 2, 64, 14, 18, 64, seed=12)
    x = make_workload_inputs(wl)
    want = dcnv2_c(x["X"], x["offset"], x["mask"], x["W"], x["bias"], stride=wl.stride, padding=wl.padding,
                   dilation=wl.dilation)
    (y,) = evaluate_op("DeformConv2D", (x["X"], x["offset"], x["mask"], x["W"], x["bias"]), wl.attrs())
    assert_fp32_gate(y, want, "evaluate_op DeformConv2D")
    with CudaSession(compile_cuda(build_dcn_graph_for(wl))) as session:
        res = session.run(x, profile=True)
        assert_fp32_gate(res.outputs["Y"], want, "session DeformConv2D")
        assert res.profiler.cuda_launch_profile()["launches"][0]["op"] == "DeformConv2D"
    with CudaSession(compile_cuda(build_dcn_graph_for(wl), dcn_math="bf16")) as session:
        assert_rel_gate(session.run(x).outputs["Y"], want, 1e-2, "session bf16")
    c = dcn_small["dcn_batch_grouped"]
    a = [int(v) for v in c["attrs"]]
    (y,) = evaluate_op("DeformConv2D", (c["X"], c["offset"], c["mask"], c["W"], c["bias"]),
                       {"stride": a[0:2], "padding": a[2:4], "dilation": a[4:6], "groups": a[6], "deform_groups": a[7]})
    np.testing.assert_allclose(y, c["expected"], rtol=2e-5, atol=2e-5)


# --------------------------------------------------------------------------- plain convolution (conv_offset and friends)

def _conv_attrs(c):
    a = [int(v) for v in c["attrs"]]
    return dict(strides=tuple(a[0:2]), pads=tuple(a[2:6]), dilations=tuple(a[6:8]), groups=a[8], relu=bool(a[9]))


def _run_conv(dev, c, math="f32x3", **extra):
    torch, ops, device = dev
    x, w = (torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("X", "W"))
    bias = torch.from_numpy(c["bias"]).to(device) if "bias" in c else None
    status = torch.zeros(1, dtype=torch.int32, device=device)
    y = ops.conv2d_forward(x, w, bias, math=math, status_word=status, **_conv_attrs(c), **extra)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait expired inside the kernel"
    return y


@pytest.mark.parametrize("case", sorted(load_cases("conv_small.npz")))
def test_conv2d_against_reference_evaluator_outputs(case, conv_small, dev):
    """Expected values are the reference's own NumPy Conv2D (+ReLU) outputs."""
    torch, ops, device = dev
    c = conv_small[case]
    a = _conv_attrs(c)
    n, cin, h, w = c["X"].shape
    cout, _, kh, kw = c["W"].shape
    need = ops.conv2d_workspace_bytes(n, cin, h, w, cout, kh, kw, a["strides"], a["pads"], a["dilations"], a["groups"], "f32x3")
    assert (need > 0) == case.endswith("tensor_path"), "fixture names say which kernel they are meant to reach"
    assert_fp32_gate(_run_conv(dev, c).cpu().numpy(), c["expected"], case)
    for math in ("tf32", "bf16"):
        assert_rel_gate(_run_conv(dev, c, math).cpu().numpy(), c["expected"], 1e-2, f"{case} {math}")
    (y,) = ops.evaluate_op("Conv2D", (c["X"], c["W"], c["bias"]) if "bias" in c else (c["X"], c["W"]),
                           {"strides": list(a["strides"]), "pads": list(a["pads"]), "dilations": list(a["dilations"]),
                            "groups": a["groups"], "relu": a["relu"]})
    assert_fp32_gate(y, c["expected"], f"{case} evaluate_op")


@pytest.mark.parametrize("case", ["conv_offset_small", "conv_offset_tensor_path"])
def test_conv_offset_split_feeds_dcn(case, conv_small, dev):
    """conv_offset -> (offset | mask scores) written as two tensors -> DCNv2 with the sigmoid folded in, against
    the same chain through the oracles; and the split halves equal the slices of the unsplit output bit for bit."""
    from oracle import conv2d_c, dcnv2_fused_c

    torch, ops, device = dev
    c = conv_small[case]
    whole = _run_conv(dev, c)
    offset, scores = _run_conv(dev, c, split_at=18)
    assert offset.shape[1] == 18 and scores.shape[1] == 9
    assert torch.equal(offset, whole[:, :18]) and torch.equal(scores, whole[:, 18:])
    rng = np.random.default_rng(5)
    cin = c["X"].shape[1]
    w2 = (rng.standard_normal((32, cin, 3, 3)) * np.sqrt(2.0 / (9 * cin))).astype(np.float32)
    b2 = rng.standard_normal(32).astype(np.float32)
    x = torch.from_numpy(c["X"]).to(device)
    y = ops.dcnv2_forward(x, offset, scores, torch.from_numpy(w2).to(device), torch.from_numpy(b2).to(device),
                          padding=(1, 1), mask_is_logits=True, relu=True)
    torch.cuda.synchronize()
    ref_conv = conv2d_c(c["X"], c["W"], c["bias"], pads=(1, 1, 1, 1))
    want = dcnv2_fused_c(c["X"], ref_conv[:, :18], ref_conv[:, 18:], w2, b2, relu=True, padding=(1, 1))
    # offsets that differ in the last bits move samples slightly: the chain is compared at the reduced gate
    assert_rel_gate(y.cpu().numpy(), want, 1e-3, f"{case} chain")
    # ... and so that an error of the deformable kernel cannot hide behind that gate: the same second half with
    # the ORACLE's offsets and scores fed to both sides, at the float32 gate
    y2 = ops.dcnv2_forward(x, torch.from_numpy(np.ascontiguousarray(ref_conv[:, :18])).to(device),
                           torch.from_numpy(np.ascontiguousarray(ref_conv[:, 18:])).to(device),
                           torch.from_numpy(w2).to(device), torch.from_numpy(b2).to(device), padding=(1, 1),
                           mask_is_logits=True, relu=True)
    torch.cuda.synchronize()
    assert_fp32_gate(y2.cpu().numpy(), want, f"{case} chain, oracle offsets")
    # and the first half alone at the float32 gate
    assert_fp32_gate(whole.cpu().numpy(), ref_conv, f"{case} conv_offset")


@pytest.mark.parametrize("label,wl_args", [
    ("narrow_tiles_records_once", dict(cin=64, cout=48)),
    ("narrow_tiles_records_per_block", dict(cin=128, cout=32, deform_groups=2)),
    ("narrow_tiles_two_groups", dict(cin=128, cout=96, groups=2)),
])
def test_narrow_channel_tiles_beyond_one_wave(dev, label, wl_args):
    """More CTAs than SMs with channel tiles of at most 64 columns: the kernel then runs its two-CTAs-per-SM shape
    (two producer groups, four A stages, two MMA-issuing threads).  Against the C oracle, all three math modes."""
    from general_ai_compiler_b200.bevformer import DcnWorkload
    from oracle import dcnv2_c

    torch, ops, device = dev
    wl = DcnWorkload(label, 2, height=100, width=100, seed=61, **wl_args)
    c = _workload_case(wl)
    assert (2 * 100 * 100 + 127) // 128 * wl.groups > torch.cuda.get_device_properties(device).multi_processor_count
    want = dcnv2_c(c["X"], c["offset"], c["mask"], c["W"], c["bias"], stride=wl.stride, padding=wl.padding,
                   dilation=wl.dilation, groups=wl.groups, deform_groups=wl.deform_groups)
    assert_fp32_gate(_run(dev, c, "f32x3").cpu().numpy(), want, label)
    for math in ("tf32", "bf16"):
        assert_rel_gate(_run(dev, c, math).cpu().numpy(), want, 1e-2, f"{label} {math}")


def test_conv_offset_full_size(dev):
    """The 27-channel offset/mask convolution on the six-camera C4 feature map against the C oracle, plus image-range
    sharding."""
    from oracle import conv2d_c

    torch, ops, device = dev
    rng = np.random.default_rng(77)
    x = rng.standard_normal((6, 256, 58, 100)).astype(np.float32)
    w = (rng.standard_normal((27, 256, 3, 3)) * np.sqrt(2.0 / (9 * 256))).astype(np.float32)
    b = rng.standard_normal(27).astype(np.float32)
    want = conv2d_c(x, w, b, pads=(1, 1, 1, 1))
    c = {"X": x, "W": w, "bias": b, "attrs": np.asarray([1, 1, 1, 1, 1, 1, 1, 1, 1, 0], np.int32)}
    got = _run_conv(dev, c)
    assert_fp32_gate(got.cpu().numpy(), want, "conv_offset c4")
    for math in ("tf32", "bf16"):
        assert_rel_gate(_run_conv(dev, c, math).cpu().numpy(), want, 1e-2, f"conv_offset c4 {math}")
    out = torch.full_like(got, float("nan"))
    for n0, n1 in ((0, 2), (2, 5), (5, 6)):
        _run_conv(dev, c, n_range=(n0, n1), out=out)
    assert torch.equal(out, got)


def test_conv2d_contract_violations(dev):
    torch, ops, device = dev
    from general_ai_compiler_b200.errors import BackendError, EvaluationError

    x = torch.zeros((1, 8, 6, 6), device=device)
    w = torch.zeros((4, 8, 3, 3), device=device)
    with pytest.raises(EvaluationError):
        ops.conv2d_forward(x, w, groups=3)
    with pytest.raises(EvaluationError):
        ops.conv2d_forward(x, w, pads=(1, 1))
    with pytest.raises(EvaluationError):
        ops.conv2d_forward(x, w, split_at=4)
    with pytest.raises(EvaluationError):
        ops.conv2d_forward(x, torch.zeros((4, 8, 9, 9), device=device))        # kernel larger than the padded input
    with pytest.raises(EvaluationError):
        ops.conv2d_forward(x, w, torch.zeros(5, device=device))
    lib = ops.native.load()
    # split_at without a second output, straight at the C boundary
    rc = lib.gacb_conv2d_forward(x.data_ptr(), w.data_ptr(), None, 0, x.data_ptr(), None, 2, 1, 8, 6, 6, 4, 3, 3, 1, 1,
                                 1, 1, 1, 1, 1, 1, 1, 0, 1, 0, None, 0, None, None)
    assert rc == -1 and "split_at" in ops.native.last_error()


# --------------------------------------------------------------------------- the window kernel of plain convolutions

def _bf16_round(a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).float().numpy()


@pytest.fixture
def window_path(dev):
    """Calls ``use(mode)`` to switch the window kernel on or off; the library's mode is restored afterwards."""
    _, ops, _ = dev
    lib = ops.native.load()
    before = lib.gacb_conv_window_path(-1)
    yield lib.gacb_conv_window_path
    lib.gacb_conv_window_path(before)


@pytest.mark.parametrize("label,shape", [
    # N, Cin, H, W, Cout, Kh, Kw, pads (top, left, bottom, right), relu
    ("conv_offset_c4_cut", (2, 256, 58, 100, 27, 3, 3, (1, 1, 1, 1), False)),
    ("ragged_tiles_cin192", (3, 192, 37, 45, 27, 3, 3, (1, 1, 1, 1), True)),        # three 64-channel groups, partial tiles
    ("kernel_5x5_cin64", (1, 64, 40, 44, 64, 5, 5, (2, 2, 2, 2), False)),           # two 32-column accumulator slabs
    ("uneven_pads_cin128", (2, 128, 33, 50, 16, 3, 3, (0, 2, 1, 0), False)),
    ("one_by_one_cin256", (1, 256, 64, 64, 32, 1, 1, (0, 0, 0, 0), True)),
    ("no_padding_cin384", (1, 384, 30, 41, 27, 3, 3, (0, 0, 0, 0), False)),         # three 128-channel groups
])
def test_window_kernel_matches_the_oracle_on_bf16_operands(dev, window_path, label, shape):
    """BF16 mode rounds X and W to bf16 and accumulates in float32, so the oracle on the rounded operands must agree
    at the float32 gate; the gather kernel must agree with the window kernel to the same gate."""
    from oracle import conv2d_c

    torch, ops, device = dev
    n, cin, h, w_, cout, kh, kw, pads, relu = shape
    rng = np.random.default_rng(zlib.crc32(label.encode()))
    x = rng.standard_normal((n, cin, h, w_)).astype(np.float32)
    w = (rng.standard_normal((cout, cin, kh, kw)) * np.sqrt(2.0 / (kh * kw * cin))).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    c = {"X": x, "W": w, "bias": b, "attrs": np.asarray([1, 1, *pads, 1, 1, 1, int(relu)], np.int32)}
    geo = ops.native.dcnv2_launch_geometry(n, cin, h, w_, cout, kh, kw, (1, 1), pads[:2], (1, 1), 1, 1, ops.native.DCN_BF16,
                                           plain=True)
    window_path(1)
    got = _run_conv(dev, c, "bf16").cpu().numpy()
    want = conv2d_c(_bf16_round(x), _bf16_round(w), b, pads=pads, relu=relu)
    assert_fp32_gate(got, want, f"{label} window kernel")
    window_path(0)
    gathered = _run_conv(dev, c, "bf16").cpu().numpy()
    assert_fp32_gate(gathered, want, f"{label} gather kernel")
    if pads[0] == pads[2] and pads[1] == pads[3]:      # the geometry query takes symmetric pads
        assert geo.kernel == b"conv_window_kernel<bf16>" and geo.block[0] == 320 and geo.grid[0] <= 148


def _tf32_truncate(a):
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return bits.view(np.float32)


def _tf32_round_nearest(a):
    """cvt.rna: nearest tf32, ties away from zero (the bit pattern is sign-magnitude, so adding half an ulp rounds the
    magnitude)."""
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((bits + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


@pytest.mark.parametrize("label,shape", [
    ("conv_offset_c4_cut", (2, 256, 58, 100, 27, 3, 3, (1, 1, 1, 1), False)),
    ("ragged_tiles_cin96", (3, 96, 37, 45, 27, 3, 3, (1, 1, 1, 1), True)),      # TF32: three 32-channel groups; F32X3: gather kernel
    ("kernel_5x5_cin64", (1, 64, 40, 44, 32, 5, 5, (2, 2, 2, 2), False)),
    ("uneven_pads_cin128", (2, 128, 33, 50, 16, 3, 3, (0, 2, 1, 0), False)),
])
def test_window_kernel_float32_modes(dev, window_path, label, shape):
    """F32X3 mode is the float32 product: the float32 gate against the oracle.  TF32 mode truncates the activations
    to tf32 and rounds the weights to the nearest tf32, then accumulates in float32: the float32 gate against the
    oracle on those operands.  The gather kernel must agree with each at its own gate."""
    from oracle import conv2d_c

    torch, ops, device = dev
    n, cin, h, w_, cout, kh, kw, pads, relu = shape
    rng = np.random.default_rng(zlib.crc32(label.encode()) + 1)
    x = rng.standard_normal((n, cin, h, w_)).astype(np.float32)
    w = (rng.standard_normal((cout, cin, kh, kw)) * np.sqrt(2.0 / (kh * kw * cin))).astype(np.float32)
    b = rng.standard_normal(cout).astype(np.float32)
    c = {"X": x, "W": w, "bias": b, "attrs": np.asarray([1, 1, *pads, 1, 1, 1, int(relu)], np.int32)}
    exact = conv2d_c(x, w, b, pads=pads, relu=relu)
    tf32 = conv2d_c(_tf32_truncate(x), _tf32_round_nearest(w), b, pads=pads, relu=relu)
    window_path(1)
    assert_fp32_gate(_run_conv(dev, c, "f32x3").cpu().numpy(), exact, f"{label} f32x3 window kernel")
    assert_fp32_gate(_run_conv(dev, c, "tf32").cpu().numpy(), tf32, f"{label} tf32 window kernel")
    if pads[0] == pads[2] and pads[1] == pads[3]:
        geo = ops.native.dcnv2_launch_geometry(n, cin, h, w_, cout, kh, kw, (1, 1), pads[:2], (1, 1), 1, 1,
                                               ops.native.DCN_TF32, plain=True)
        assert geo.kernel == b"conv_window_kernel<tf32>"
    window_path(0)
    assert_fp32_gate(_run_conv(dev, c, "f32x3").cpu().numpy(), exact, f"{label} f32x3 gather kernel")
    assert_rel_gate(_run_conv(dev, c, "tf32").cpu().numpy(), exact, 1e-2, f"{label} tf32 gather kernel")


def test_window_kernel_split_outputs_sharding_and_weight_reuse(dev, window_path):
    """offset/mask split outputs, image-range calls bit-identical to one call, packed weights reused across calls."""
    torch, ops, device = dev
    window_path(1)
    rng = np.random.default_rng(9)
    x = torch.from_numpy(rng.standard_normal((4, 64, 29, 36)).astype(np.float32)).to(device)
    w = torch.from_numpy((rng.standard_normal((27, 64, 3, 3)) * 0.05).astype(np.float32)).to(device)
    b = torch.from_numpy(rng.standard_normal(27).astype(np.float32)).to(device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    whole = ops.conv2d_forward(x, w, b, pads=(1, 1, 1, 1), math="bf16", status_word=status)
    off, mask = ops.conv2d_forward(x, w, b, pads=(1, 1, 1, 1), math="bf16", split_at=18, status_word=status)
    assert torch.equal(off, whole[:, :18]) and torch.equal(mask, whole[:, 18:])
    out = torch.full_like(whole, float("nan"))
    for n0, n1 in ((0, 1), (1, 4)):
        ops.conv2d_forward(x, w, b, pads=(1, 1, 1, 1), math="bf16", n_range=(n0, n1), out=out, status_word=status)
    assert torch.equal(out, whole)
    need = ops.conv2d_workspace_bytes(4, 64, 29, 36, 27, 3, 3, (1, 1), (1, 1, 1, 1), (1, 1), 1, "bf16")
    ws = torch.empty(need, dtype=torch.uint8, device=device)
    first = ops.conv2d_forward(x, w, b, pads=(1, 1, 1, 1), math="bf16", workspace=ws, status_word=status)
    again = ops.conv2d_forward(x, w, b, pads=(1, 1, 1, 1), math="bf16", workspace=ws, reuse_weights=True, reuse_input=True,
                               status_word=status)
    torch.cuda.synchronize()
    assert torch.equal(first, whole) and torch.equal(again, whole) and int(status.item()) == 0
    # a strided convolution does not qualify and still runs (another kernel)
    strided = ops.conv2d_forward(x, w, b, strides=(2, 2), pads=(1, 1, 1, 1), math="bf16", status_word=status)
    ref = torch.nn.functional.conv2d(x.double(), w.double(), b.double(), stride=2, padding=1)
    assert_rel_gate(strided.cpu().numpy(), ref.float().cpu().numpy(), 1e-2, "strided falls back")


def test_session_shares_the_channel_last_copy_between_convolutions_of_one_input(dev):
    """A graph in which a plain convolution and a DCNv2 read the same X (conv_offset and conv2 of an R101-DCN
    bottleneck): the session gives them one channel-last copy, made by the first and reused by the second; the
    results are those of the separate operators, run after run with different X."""
    from general_ai_compiler_b200 import evaluate_op
    from general_ai_compiler_b200.bevformer import DcnWorkload, make_workload_inputs
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.ir import Graph, Node, TensorSpec
    from general_ai_compiler_b200.session import CudaSession

    wl = DcnWorkload("pair", 2, 64, 40, 36, 64, seed=41)
    x = make_workload_inputs(wl)
    rng = np.random.default_rng(42)
    w27 = (rng.standard_normal((27, 64, 3, 3)) * 0.05).astype(np.float32)
    b27 = rng.standard_normal(27).astype(np.float32)
    ho, wo = wl.out_hw
    inputs = {"X": TensorSpec(x["X"].shape, "float32"), "offset": TensorSpec(x["offset"].shape, "float32"),
              "mask": TensorSpec(x["mask"].shape, "float32")}
    constants = {"W27": w27, "b27": b27, "W": x["W"], "bias": x["bias"]}
    nodes = [Node("conv_offset", "Conv2D", ("X", "W27", "b27"), ("T",), {"pads": [1, 1, 1, 1]}),
             Node("conv2", "DeformConv2D", ("X", "offset", "mask", "W", "bias"), ("Y",), wl.attrs())]
    graph = Graph("pair_of_convolutions", inputs, ("T", "Y"), nodes, constants)
    graph.validate()
    for math, check in (("f32x3", assert_fp32_gate), ("bf16", lambda a, b, what: assert_rel_gate(a, b, 1e-2, what))):
        with CudaSession(compile_cuda(graph, dcn_math=math)) as session:
            assert session._input_copy == {"conv_offset": "make", "conv2": "reuse"}
            assert session._workspaces["conv_offset"].data_ptr() < session._workspaces["conv2"].data_ptr()
            for run in range(3):                          # the second and third runs reuse the packed weights
                xr = x["X"] * np.float32(1.0 + 0.25 * run)
                res = session.run({"X": xr, "offset": x["offset"], "mask": x["mask"]})
                (t,) = evaluate_op("Conv2D", (xr, w27, b27), {"pads": [1, 1, 1, 1]})
                (y,) = evaluate_op("DeformConv2D", (xr, x["offset"], x["mask"], x["W"], x["bias"]), wl.attrs())
                check(res.outputs["T"], t, f"{math} run {run} conv_offset")
                check(res.outputs["Y"], y, f"{math} run {run} conv2")
