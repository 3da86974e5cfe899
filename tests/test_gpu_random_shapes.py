"""Seeded sweeps over the operators' contract space against the C oracle: odd extents, every head-dim path, strides,
dilations, groups, padded channel tiles, tile tails, call ranges.  Sizes stay small enough for the oracle."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_fp32_gate, assert_rel_gate

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch

    from general_ai_compiler_b200 import ops

    return torch, ops, ops.require_device(0)


def _msda_case(rng):
    levels = int(rng.integers(1, 5))
    shapes = [(int(rng.integers(1, 23)), int(rng.integers(1, 29))) for _ in range(levels)]
    head_dim = int(rng.choice([1, 3, 4, 8, 12, 16, 32, 40, 64, 128]))
    return dict(B=int(rng.integers(1, 4)), Q=int(rng.integers(1, 70)), H=int(rng.integers(1, 9)), D=head_dim,
                P=int(rng.integers(1, 9)), shapes=shapes)


@pytest.mark.parametrize("seed", range(24))
def test_msda_random_shapes(seed, dev):
    from oracle import msda_c
    from oracle.msda_numpy import msda_offsets_forward, softmax_last

    torch, ops, device = dev
    rng = np.random.default_rng(1000 + seed)
    c = _msda_case(rng)
    B, Q, H, D, P, shapes = c["B"], c["Q"], c["H"], c["D"], c["P"], c["shapes"]
    L = len(shapes)
    S = sum(h * w for h, w in shapes)
    value = rng.standard_normal((B, S, H, D)).astype(np.float32)
    loc = rng.uniform(-0.3, 1.3, (B, Q, H, L, P, 2)).astype(np.float32)
    attn = rng.random((B, Q, H, L, P)).astype(np.float32)
    t = {k: torch.from_numpy(v).to(device) for k, v in (("value", value), ("loc", loc), ("attn", attn))}
    want = msda_c(value, loc, attn, shapes)
    got = ops.msda_forward(t["value"], t["loc"], t["attn"], shapes)
    torch.cuda.synchronize()
    assert_fp32_gate(got.cpu().numpy(), want, f"msda {c}")
    # a query range writes its rows and nothing else
    if Q >= 2:
        q0, q1 = sorted(int(v) for v in rng.choice(Q + 1, 2, replace=False))
        part = torch.full_like(got, 7.0)
        ops.msda_forward(t["value"], t["loc"], t["attn"], shapes, out=part, q_range=(q0, q1))
        torch.cuda.synchronize()
        assert torch.equal(part[:, q0:q1], got[:, q0:q1])
        assert torch.all(part[:, :q0] == 7.0) and torch.all(part[:, q1:] == 7.0)
    # bf16 storage of the value
    if seed % 2 == 0:
        got16 = ops.msda_forward(ops.cast_to_bf16(t["value"]), t["loc"], t["attn"], shapes)
        torch.cuda.synchronize()
        assert_rel_gate(got16.cpu().numpy(), want, 1e-2, f"msda bf16 {c}")
    # raw scores + offsets with the softmax and the coordinate arithmetic in the kernel
    if seed % 3 == 0:
        logits = rng.standard_normal((B, Q, H, L, P)).astype(np.float32)
        norm = np.asarray([[w, h] for h, w in shapes], np.float32).reshape(1, 1, 1, L, 1, 2)
        ref = rng.uniform(0, 1, (B, Q, 1, 1, 1, 2)).astype(np.float32)
        offs = (rng.standard_normal((B, Q, H, L, P, 2)) * 2).astype(np.float32)
        weights = softmax_last(logits.reshape(B, Q, H, L * P)).reshape(B, Q, H, L, P).astype(np.float32)
        want2 = msda_offsets_forward(value, offs, weights, norm, ref, shapes, (B, Q, H, L, P, 2))
        got2 = ops.msda_offsets_forward(t["value"], torch.from_numpy(offs).to(device), torch.from_numpy(logits).to(device),
                                        torch.from_numpy(norm).to(device), torch.from_numpy(ref).to(device), shapes,
                                        (B, Q, H, L, P, 2), softmax=True)
        torch.cuda.synchronize()
        assert_fp32_gate(got2.cpu().numpy(), want2, f"msda offsets+softmax {c}")


def _dcn_case(rng, tensor_path: bool):
    kh, kw = (int(v) for v in rng.choice([1, 2, 3], 2)) if not tensor_path else (int(rng.choice([1, 3])), int(rng.choice([1, 3])))
    groups = int(rng.choice([1, 2]))
    dgroups = int(rng.choice([1, 2]))
    if tensor_path:
        cin_g = int(rng.choice([64, 128]))
        cin = cin_g * groups
        cout = int(rng.choice([16, 27, 48, 64, 96])) * groups
        h, w = int(rng.integers(16, 33)), int(rng.integers(16, 37))
    else:
        cin = int(rng.choice([2, 4, 6, 8])) * groups * dgroups
        cout = int(rng.integers(1, 6)) * groups
        h, w = int(rng.integers(3, 12)), int(rng.integers(3, 12))
    stride = (int(rng.choice([1, 2])), int(rng.choice([1, 2])))
    dilation = (int(rng.choice([1, 2])), int(rng.choice([1, 2])))
    padding = (int(rng.integers(0, 3)), int(rng.integers(0, 3)))
    return dict(N=int(rng.integers(1, 4)), cin=cin, cout=cout, h=h, w=w, kh=kh, kw=kw, stride=stride, dilation=dilation,
                padding=padding, groups=groups, dgroups=dgroups)


@pytest.mark.parametrize("tensor_path", [False, True])
@pytest.mark.parametrize("seed", range(14))
def test_dcn_random_shapes(seed, tensor_path, dev):
    from oracle import dcnv2_c

    torch, ops, device = dev
    rng = np.random.default_rng(5000 + seed + (100 if tensor_path else 0))
    for _ in range(20):
        c = _dcn_case(rng, tensor_path)
        ho = (c["h"] + 2 * c["padding"][0] - c["dilation"][0] * (c["kh"] - 1) - 1) // c["stride"][0] + 1
        wo = (c["w"] + 2 * c["padding"][1] - c["dilation"][1] * (c["kw"] - 1) - 1) // c["stride"][1] + 1
        if ho > 0 and wo > 0:
            break
    else:
        pytest.skip("no legal geometry drawn")
    K = c["kh"] * c["kw"]
    x = rng.standard_normal((c["N"], c["cin"], c["h"], c["w"])).astype(np.float32)
    off = (rng.standard_normal((c["N"], 2 * c["dgroups"] * K, ho, wo)) * 1.5).astype(np.float32)
    mask = rng.random((c["N"], c["dgroups"] * K, ho, wo)).astype(np.float32)
    wt = (rng.standard_normal((c["cout"], c["cin"] // c["groups"], c["kh"], c["kw"])) * np.sqrt(2.0 / (K * c["cin"] // c["groups"]))).astype(np.float32)
    bias = rng.standard_normal(c["cout"]).astype(np.float32) if seed % 2 else None
    kw = dict(stride=c["stride"], padding=c["padding"], dilation=c["dilation"], groups=c["groups"], deform_groups=c["dgroups"])
    want = dcnv2_c(x, off, mask, wt, bias, **kw)
    t = [torch.from_numpy(v).to(device) for v in (x, off, mask, wt)]
    tb = torch.from_numpy(bias).to(device) if bias is not None else None
    status = torch.zeros(1, dtype=torch.int32, device=device)
    got = ops.dcnv2_forward(*t, tb, math="f32x3", status_word=status, **kw)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_fp32_gate(got.cpu().numpy(), want, f"dcn {c}")
    if tensor_path:
        for math in ("tf32", "bf16"):
            g2 = ops.dcnv2_forward(*t, tb, math=math, status_word=status, **kw)
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            assert_rel_gate(g2.cpu().numpy(), want, 1e-2, f"dcn {math} {c}")
    # a run of output pixels that starts and ends anywhere
    total = c["N"] * ho * wo
    p0, p1 = sorted(int(v) for v in rng.choice(total + 1, 2, replace=False))
    part = torch.full_like(got, 5.0)
    ops.dcnv2_forward(*t, tb, math="f32x3", out=part, pixel_range=(p0, p1), status_word=status, **kw)
    torch.cuda.synchronize()
    flat_p = part.permute(0, 2, 3, 1).reshape(total, -1)
    flat_g = got.permute(0, 2, 3, 1).reshape(total, -1)
    assert torch.equal(flat_p[p0:p1], flat_g[p0:p1])
    assert torch.all(flat_p[:p0] == 5.0) and torch.all(flat_p[p1:] == 5.0)


@pytest.mark.parametrize("seed", range(10))
def test_conv2d_random_shapes(seed, dev):
    from oracle import conv2d_c

    torch, ops, device = dev
    rng = np.random.default_rng(9000 + seed)
    big = seed % 2 == 1
    groups = int(rng.choice([1, 2]))
    cin = (int(rng.choice([64, 128])) if big else int(rng.choice([3, 4, 8]))) * groups
    cout = (int(rng.choice([5, 27, 32, 80])) if big else int(rng.integers(1, 7))) * groups
    kh, kw = int(rng.choice([1, 3])), int(rng.choice([1, 3, 5] if not big else [1, 3]))
    h, w = (int(rng.integers(18, 30)), int(rng.integers(18, 34))) if big else (int(rng.integers(4, 12)), int(rng.integers(4, 12)))
    strides = (int(rng.choice([1, 2])), int(rng.choice([1, 2])))
    dil = (1, int(rng.choice([1, 2])))
    pads = tuple(int(v) for v in rng.integers(0, 3, 4))
    if h + pads[0] + pads[2] < dil[0] * (kh - 1) + 1 or w + pads[1] + pads[3] < dil[1] * (kw - 1) + 1:
        pytest.skip("kernel exceeds the padded input")
    x = rng.standard_normal((2, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin // groups, kh, kw)) * np.sqrt(2.0 / (kh * kw * cin // groups))).astype(np.float32)
    bias = rng.standard_normal(cout).astype(np.float32)
    relu = bool(seed % 3 == 0)
    want = conv2d_c(x, wt, bias, strides=strides, pads=pads, dilations=dil, groups=groups, relu=relu)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    got = ops.conv2d_forward(torch.from_numpy(x).to(device), torch.from_numpy(wt).to(device), torch.from_numpy(bias).to(device),
                             strides=strides, pads=pads, dilations=dil, groups=groups, relu=relu, status_word=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert_fp32_gate(got.cpu().numpy(), want, f"conv2d seed {seed}")
    if cout >= 2:
        cut = int(rng.integers(1, cout))
        lo, hi = ops.conv2d_forward(torch.from_numpy(x).to(device), torch.from_numpy(wt).to(device),
                                    torch.from_numpy(bias).to(device), strides=strides, pads=pads, dilations=dil,
                                    groups=groups, relu=relu, split_at=cut, status_word=status)
        torch.cuda.synchronize()
        assert torch.equal(lo, got[:, :cut]) and torch.equal(hi, got[:, cut:])


def _round_like_the_mode(x, w, math):
    """Operands as the tensor core sees them in each mode of the window kernel: bf16-rounded (BF16), activations
    truncated and weights rounded to tf32 (TF32), unchanged (F32X3: the float32 product)."""
    import torch

    if math == "bf16":
        r = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).float().numpy()
        return r(x), r(w)
    if math == "tf32":
        xb = np.ascontiguousarray(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
        wb = (np.ascontiguousarray(w, np.float32).view(np.uint32) + np.uint32(0x1000)) & np.uint32(0xFFFFE000)
        return xb.view(np.float32), wb.view(np.float32)
    return x, w


@pytest.mark.parametrize("seed", range(12))
def test_window_convolution_random_shapes(seed, dev):
    """Shapes that take the persistent window kernel (whole images, stride 1, no dilation, no groups, at most 64
    output channels, channels a multiple of 64): ragged tiles, every kernel extent, uneven pads, one to three
    images, all three math modes, each at the float32 gate against the oracle on that mode's operands."""
    from oracle import conv2d_c

    torch, ops, device = dev
    rng = np.random.default_rng(7000 + seed)
    n = int(rng.integers(1, 4))
    cin = int(rng.choice([64, 128, 192, 256]))
    cout = int(rng.choice([1, 5, 16, 27, 32, 33, 64]))
    kh, kw = int(rng.choice([1, 3, 5])), int(rng.choice([1, 3, 5]))
    h, w = int(rng.integers(17, 50)), int(rng.integers(9, 60))
    pads = tuple(int(v) for v in rng.integers(0, 3, 4))
    relu = bool(seed % 2)
    x = rng.standard_normal((n, cin, h, w)).astype(np.float32)
    wt = (rng.standard_normal((cout, cin, kh, kw)) * np.sqrt(2.0 / (kh * kw * cin))).astype(np.float32)
    bias = rng.standard_normal(cout).astype(np.float32) if seed % 3 else None
    xd, wd = torch.from_numpy(x).to(device), torch.from_numpy(wt).to(device)
    bd = torch.from_numpy(bias).to(device) if bias is not None else None
    status = torch.zeros(1, dtype=torch.int32, device=device)
    for math in ("f32x3", "tf32", "bf16"):
        xr, wr = _round_like_the_mode(x, wt, math)
        want = conv2d_c(xr, wr, bias, pads=pads, relu=relu)
        geo = ops.native.dcnv2_launch_geometry(n, cin, h, w, cout, kh, kw, (1, 1), pads[:2], (1, 1), 1, 1,
                                               ops.native.DCN_MATH_MODES[math], plain=True)
        got = ops.conv2d_forward(xd, wd, bd, pads=pads, math=math, relu=relu, status_word=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        if geo.kernel.startswith(b"conv_window_kernel") and pads[0] == pads[2] and pads[1] == pads[3]:
            assert_fp32_gate(got.cpu().numpy(), want, f"window conv seed {seed} {math}")
        elif math == "f32x3":
            assert_fp32_gate(got.cpu().numpy(), want, f"conv seed {seed} {math}")
        else:      # another kernel took it (small problems stay on the CUDA cores in float32; F32X3 beyond 32 channels)
            assert_rel_gate(got.cpu().numpy(), conv2d_c(x, wt, bias, pads=pads, relu=relu), 1e-2, f"conv seed {seed} {math}")
