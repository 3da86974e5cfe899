"""MSDA parity on the B200: every call goes through the C ABI (libgacb.so); the CPU oracle only checks."""

from __future__ import annotations

import numpy as np
import pytest

from conftest import assert_fp32_gate, assert_rel_gate, load_cases

pytestmark = pytest.mark.gpu


def _shapes(a):
    return [tuple(int(v) for v in row) for row in a]


@pytest.fixture(scope="module")
def dev():
    import torch

    from general_ai_compiler_b200 import ops

    device = ops.require_device(0)
    return torch, ops, device


def _run(dev, value, loc, attn, shapes, storage="float32", q_range=None, out=None):
    torch, ops, device = dev
    v = torch.from_numpy(np.ascontiguousarray(value)).to(device)
    if storage == "bfloat16":
        v = ops.cast_to_bf16(v)
    l = torch.from_numpy(np.ascontiguousarray(loc)).to(device)
    a = torch.from_numpy(np.ascontiguousarray(attn)).to(device)
    y = ops.msda_forward(v, l, a, shapes, q_range=q_range, out=out)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("case", sorted(load_cases("msda_small.npz")))
def test_small_cases_fp32(case, msda_small, dev):
    c = msda_small[case]
    y = _run(dev, c["value"], c["loc"], c["attn"], _shapes(c["shapes"])).cpu().numpy()
    assert_fp32_gate(y, c["expected"], case)


def test_known_answers_are_exact(msda_small, dev):
    c = msda_small["kat_center_1x1"]
    y = _run(dev, c["value"], c["loc"], c["attn"], [(1, 1)]).cpu().numpy()
    assert np.array_equal(y, np.asarray([[[7.25, -3.5]]], np.float32))
    c = msda_small["native_exact_pixel_centers"]
    y = _run(dev, c["value"], c["loc"], c["attn"], [(2, 2)]).cpu().numpy()
    assert np.array_equal(y, c["value"].reshape(1, 4, 4))
    c = msda_small["kat_2x2_bilinear_padding"]
    y = _run(dev, c["value"], c["loc"], c["attn"], [(2, 2)]).cpu().numpy()
    np.testing.assert_allclose(y[..., 0], [[1.0, 2.5, 0.25, 0.0]], rtol=0, atol=1e-7)


@pytest.mark.parametrize("case", [c for c in sorted(load_cases("msda_small.npz")) if c.startswith("cfg_") or c.startswith("dim")])
def test_small_cases_bf16_value(case, msda_small, dev):
    import torch

    c = msda_small[case]
    shapes = _shapes(c["shapes"])
    y = _run(dev, c["value"], c["loc"], c["attn"], shapes, storage="bfloat16").cpu().numpy()
    assert_rel_gate(y, c["expected"], 1e-2, case)
    # kernel error alone: oracle fed the bf16-rounded value must match to the fp32 gate
    from oracle import msda_c

    rounded = torch.from_numpy(c["value"]).to(torch.bfloat16).to(torch.float32).numpy()
    assert_fp32_gate(y, msda_c(rounded, c["loc"], c["attn"], shapes), case + " (bf16-rounded value)")


@pytest.mark.parametrize("key", ["tiny_tsa", "tiny_sca", "base_sca", "base_tsa"])
@pytest.mark.parametrize("storage", ["float32", "bfloat16"])
def test_full_size_configurations(key, storage, msda_pins, dev):
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
    from oracle import msda_c

    w = WORKLOADS[key]
    x = make_workload_inputs(w)
    y = _run(dev, x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes, storage).cpu().numpy()
    oracle = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    pin = msda_pins[key]
    assert np.array_equal(oracle.reshape(-1)[pin["index"]], pin["expected"])   # oracle == real reference here
    if storage == "float32":
        assert_fp32_gate(y, oracle, key)
        assert_fp32_gate(y.reshape(-1)[pin["index"]], pin["expected"], key + " pins")
        assert abs(float(y.astype(np.float64).sum()) - float(pin["sum64"])) <= 1e-6 * float(pin["abs_sum64"])
    else:
        assert_rel_gate(y, oracle, 1e-2, key)


def test_query_sharding_is_bit_identical(dev):
    """Concatenated query shards equal the single launch bit for bit; rows outside a shard stay untouched."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs

    w = WORKLOADS["base_sca"].with_queries(1003)
    x = make_workload_inputs(w)
    whole = _run(dev, x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    out = torch.full_like(whole, float("nan"))
    bounds = [0, 250, 251, 700, 1003]
    for q0, q1 in zip(bounds[:-1], bounds[1:]):
        _run(dev, x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes, q_range=(q0, q1), out=out)
    assert torch.equal(out, whole)
    part = torch.full_like(whole, 7.0)
    _run(dev, x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes, q_range=(10, 20), out=part)
    assert torch.all(part[:, :10] == 7.0) and torch.all(part[:, 20:] == 7.0)
    assert torch.equal(part[:, 10:20], whole[:, 10:20])
    # a rank that holds only its slice of locations/weights/output
    loc = x["sampling_locations"][:, 300:420].copy()
    attn = x["attention_weights"][:, 300:420].copy()
    local = _run(dev, x["value"], loc, attn, w.spatial_shapes)
    assert torch.equal(local, whole[:, 300:420])


def test_linearity_and_constant_field(dev):
    """Size-independent properties: the op is linear in value; a constant field with in-range samples returns
    the constant times the weight sum."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs

    w = WORKLOADS["base_tsa"].with_queries(2500)
    x = make_workload_inputs(w)
    loc, attn = x["sampling_locations"], x["attention_weights"]
    v1 = x["value"][:, : w.spatial_size]
    v2 = np.random.default_rng(3).standard_normal(v1.shape).astype(np.float32)
    y1 = _run(dev, v1, loc, attn, w.spatial_shapes)
    y2 = _run(dev, v2, loc, attn, w.spatial_shapes)
    y12 = _run(dev, (2 * v1 + v2).astype(np.float32), loc, attn, w.spatial_shapes)
    assert float((y12 - (2 * y1 + y2)).abs().max()) < 2e-5
    inner = np.clip(loc, 0.02, 0.98).astype(np.float32)        # every tap inside the 200x200 image
    const = np.full(v1.shape, 1.5, np.float32)
    yc = _run(dev, const, inner, attn, w.spatial_shapes).cpu().numpy()
    np.testing.assert_allclose(yc, 1.5, rtol=0, atol=2e-6)


def test_fully_outside_and_zero_weight_rows(dev):
    v = np.random.default_rng(0).standard_normal((1, 12, 2, 32)).astype(np.float32)
    loc = np.full((1, 5, 2, 1, 4, 2), 3.0, np.float32)          # far outside: zero padding
    attn = np.full((1, 5, 2, 1, 4), 0.25, np.float32)
    assert not _run(dev, v, loc, attn, [(3, 4)]).cpu().numpy().any()
    loc = np.random.default_rng(1).uniform(0, 1, loc.shape).astype(np.float32)
    assert not _run(dev, v, loc, np.zeros_like(attn), [(3, 4)]).cpu().numpy().any()
    # huge coordinates must not index out of bounds either
    loc[...] = 1e30
    assert not _run(dev, v, loc, attn, [(3, 4)]).cpu().numpy().any()


def test_empty_inputs(dev):
    torch, ops, device = dev
    v = torch.zeros((2, 4, 1, 32), device=device)
    y = ops.msda_forward(v, torch.zeros((2, 0, 1, 1, 3, 2), device=device), torch.zeros((2, 0, 1, 1, 3), device=device),
                         [(2, 2)])
    assert tuple(y.shape) == (2, 0, 32)


@pytest.mark.parametrize("case", sorted(load_cases("msda_offsets.npz")))
def test_fused_coordinates(case, msda_offsets, dev):
    torch, ops, device = dev
    c = msda_offsets[case]
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("value", "offsets", "weights", "normalizer", "reference")}
    y = ops.msda_offsets_forward(t["value"], t["offsets"], t["weights"], t["normalizer"], t["reference"],
                                 _shapes(c["shapes"]), tuple(int(v) for v in c["coordinate_shape"]),
                                 bool(c["reference_first"]))
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), c["expected"], case)
    np.testing.assert_allclose(y.cpu().numpy(), c["expected_grid_sample"], rtol=2e-5, atol=2e-5)


def test_fused_coordinates_equal_materialised_locations_at_scale(dev):
    torch, ops, device = dev
    rng = np.random.default_rng(11)
    B, Q, H, L, P, D = 2, 300, 8, 4, 8, 32
    shapes = [(20, 30), (10, 15), (5, 8), (3, 4)]
    S = sum(h * w for h, w in shapes)
    value = torch.from_numpy(rng.standard_normal((B, S, H, D)).astype(np.float32)).to(device)
    offsets = torch.from_numpy(rng.normal(0, 3, (B, Q, H, L, P, 2)).astype(np.float32)).to(device)
    attn = torch.softmax(torch.from_numpy(rng.standard_normal((B, Q, H, L * P)).astype(np.float32)), -1).reshape(B, Q, H, L, P).contiguous().to(device)
    norm = torch.tensor([[w, h] for h, w in shapes], dtype=torch.float32, device=device).reshape(1, 1, 1, L, 1, 2).contiguous()
    Z = 4
    ref = torch.from_numpy(rng.uniform(0, 1, (B, Q, 1, 1, 1, Z, 2)).astype(np.float32)).to(device)
    coord = (B, Q, H, L, P // Z, Z, 2)
    loc = ((offsets / norm).reshape(coord) + ref).reshape(B, Q, H, L, P, 2).contiguous()
    fused = ops.msda_offsets_forward(value, offsets, attn, norm, ref, shapes, coord, False)
    plain = ops.msda_forward(value, loc, attn, shapes)
    torch.cuda.synchronize()
    assert torch.equal(fused, plain)


@pytest.mark.parametrize("case", sorted(load_cases("msda_softmax.npz")))
def test_softmax_folded_in(case, msda_softmax, dev):
    torch, ops, device = dev
    c = msda_softmax[case]
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("value", "loc", "logits")}
    y = ops.msda_forward(t["value"], t["loc"], t["logits"], _shapes(c["shapes"]), softmax=True)
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), c["expected"], case)


def test_softmax_folded_in_at_full_size_and_with_fused_coordinates(dev):
    """base-SCA shapes: raw scores + raw offsets in one launch equal softmax and coordinate math done outside."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
    from oracle import msda_c
    from oracle.msda_numpy import softmax_last

    w = WORKLOADS["base_sca"].with_queries(1500)
    x = make_workload_inputs(w)
    rng = np.random.default_rng(77)
    B, Q, H, L, P = w.batch, w.queries, w.heads, w.levels, w.points
    logits = (rng.standard_normal((B, Q, H, L, P)) * 2).astype(np.float32)
    prob = softmax_last(logits.reshape(B, Q, H, L * P)).reshape(B, Q, H, L, P).astype(np.float32)
    want = msda_c(x["value"], x["sampling_locations"], prob, w.spatial_shapes)
    tv = torch.from_numpy(x["value"]).to(device)
    tl = torch.from_numpy(x["sampling_locations"]).to(device)
    tg = torch.from_numpy(logits).to(device)
    y = ops.msda_forward(tv, tl, tg, w.spatial_shapes, softmax=True)
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), want, "softmax folded, base-SCA shapes")
    # fused coordinates as well: offsets in pixels / (W, H) of the level + per-query reference point
    norm = torch.tensor([[ww, hh] for hh, ww in w.spatial_shapes], dtype=torch.float32, device=device).reshape(1, 1, 1, L, 1, 2).contiguous()
    ref = torch.from_numpy(rng.uniform(0, 1, (B, Q, 1, 1, 1, 2)).astype(np.float32)).to(device)
    offs = torch.from_numpy(rng.normal(0, 3, (B, Q, H, L, P, 2)).astype(np.float32)).to(device)
    loc = (offs / norm + ref).contiguous()
    both = ops.msda_offsets_forward(tv, offs, tg, norm, ref, w.spatial_shapes, tuple(offs.shape), False, softmax=True)
    plain = ops.msda_forward(tv, loc, tg, w.spatial_shapes, softmax=True)
    torch.cuda.synchronize()
    assert torch.equal(both, plain)


def test_group_reductions_match_the_reference_ops(msda_reduce, dev):
    """Camera average with visibility (spatial cross-attention) and queue mean (temporal self-attention)."""
    torch, ops, device = dev
    c = msda_reduce["sca"]
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("value", "loc", "attn", "visibility")}
    shapes, cams = _shapes(c["shapes"]), int(c["group"])
    y = ops.msda_group_forward(t["value"], t["loc"], t["attn"], shapes, group=cams, reduce="masked_average",
                               visibility=t["visibility"])
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), c["expected"], "camera average")
    assert not y[0, 0].any()
    # the same with the visible rows compacted first: identical bits, twice in a row (the list is rebuilt per call)
    compact = torch.empty(t["visibility"].numel() + 4, dtype=torch.int32, device=device)
    for _ in range(2):
        yc = ops.msda_group_forward(t["value"], t["loc"], t["attn"], shapes, group=cams, reduce="masked_average",
                                    visibility=t["visibility"], compact=compact)
        torch.cuda.synchronize()
        assert torch.equal(yc, y)
        assert int(compact[0].item()) == int((t["visibility"] != 0).sum().item())
    # rows of invisible (camera, query) pairs are skipped: their per-entry output keeps what the buffer held
    keep = torch.full((t["value"].shape[0], t["loc"].shape[1], 256), 5.0, device=device)
    ops.msda_group_forward(t["value"], t["loc"], t["attn"], shapes, visibility=t["visibility"], out=keep)
    torch.cuda.synchronize()
    vis = t["visibility"].reshape(-1, t["loc"].shape[1])
    full = ops.msda_forward(t["value"], t["loc"], t["attn"], shapes)
    assert torch.all(keep[vis == 0] == 5.0) and torch.equal(keep[vis != 0], full[vis != 0])
    c = msda_reduce["tsa"]
    t = {k: torch.from_numpy(np.ascontiguousarray(c[k])).to(device) for k in ("value", "loc", "attn")}
    y = ops.msda_group_forward(t["value"], t["loc"], t["attn"], _shapes(c["shapes"]), group=int(c["group"]), reduce="mean")
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), c["expected"], "queue mean")


def test_camera_average_at_base_size_with_sparse_visibility(dev):
    """BEVFormer-base shapes, ~25 % of (camera, query) pairs visible, raw scores: one call."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
    from oracle import msda_c
    from oracle.msda_numpy import sca_camera_average, softmax_last

    w = WORKLOADS["base_sca"].with_queries(2000)
    x = make_workload_inputs(w)
    rng = np.random.default_rng(5)
    B, Q, H, L, P = w.batch, w.queries, w.heads, w.levels, w.points
    logits = rng.standard_normal((B, Q, H, L, P)).astype(np.float32)
    vis = (rng.uniform(0, 1, (1, B, Q, 1)) < 0.25).astype(np.float32)
    prob = softmax_last(logits.reshape(B, Q, H, L * P)).reshape(B, Q, H, L, P).astype(np.float32)
    want = sca_camera_average(msda_c(x["value"], x["sampling_locations"], prob, w.spatial_shapes), vis, B)
    y = ops.msda_group_forward(torch.from_numpy(x["value"]).to(device), torch.from_numpy(x["sampling_locations"]).to(device),
                               torch.from_numpy(logits).to(device), w.spatial_shapes, group=B, reduce="masked_average",
                               visibility=torch.from_numpy(vis).to(device), softmax=True)
    yc = ops.msda_group_forward(torch.from_numpy(x["value"]).to(device), torch.from_numpy(x["sampling_locations"]).to(device),
                                torch.from_numpy(logits).to(device), w.spatial_shapes, group=B, reduce="masked_average",
                                visibility=torch.from_numpy(vis).to(device), softmax=True,
                                compact=torch.empty(B * Q + 4, dtype=torch.int32, device=device))
    torch.cuda.synchronize()
    assert_fp32_gate(y.cpu().numpy(), want, "base-size camera average")
    assert torch.equal(y, yc)
    # the same block from raw offsets (coordinates formed in the kernel), row-skip and compacted: the sampling
    # positions are those of `loc`, so both must reproduce the launch on materialised locations bit for bit
    tv, tg, tvis = (torch.from_numpy(a).to(device) for a in (x["value"], logits, vis))
    norm = torch.tensor([[ww, hh] for hh, ww in w.spatial_shapes], dtype=torch.float32,
                        device=device).reshape(1, 1, 1, L, 1, 2).contiguous()
    ref = torch.from_numpy(rng.uniform(0, 1, (B, Q, 1, 1, 1, 2)).astype(np.float32)).to(device)
    offs = torch.from_numpy(rng.normal(0, 3, (B, Q, H, L, P, 2)).astype(np.float32)).to(device)
    loc = (offs / norm + ref).contiguous()
    kw = dict(group=B, reduce="masked_average", visibility=tvis, softmax=True)
    base = ops.msda_group_forward(tv, loc, tg, w.spatial_shapes, **kw)
    fused = dict(normalizer=norm, reference=ref, coordinate_shape=tuple(offs.shape), **kw)
    skip = ops.msda_group_forward(tv, offs, tg, w.spatial_shapes, **fused)
    listed = ops.msda_group_forward(tv, offs, tg, w.spatial_shapes, **fused,
                                    compact=torch.empty(B * Q + 4, dtype=torch.int32, device=device))
    torch.cuda.synchronize()
    assert torch.equal(skip, base) and torch.equal(listed, base)


def test_contract_violations_raise_before_launch(dev):
    torch, ops, device = dev
    from general_ai_compiler_b200.errors import BackendError, EvaluationError

    v = torch.zeros((1, 6, 2, 32), device=device)
    loc = torch.zeros((1, 3, 2, 1, 4, 2), device=device)
    attn = torch.zeros((1, 3, 2, 1, 4), device=device)
    with pytest.raises(EvaluationError):
        ops.msda_forward(v, loc, attn, [(2, 2)])                 # S != sum H*W
    with pytest.raises(EvaluationError):
        ops.msda_forward(v, loc[:, :, :1].contiguous(), attn, [(2, 3)])   # head mismatch
    with pytest.raises(EvaluationError):
        ops.msda_forward(v.double(), loc, attn, [(2, 3)])
    with pytest.raises(EvaluationError):
        ops.msda_forward(v, loc, attn, [(2, 3)], q_range=(2, 9))
    # straight through the C ABI: status codes, no exception, no launch
    from general_ai_compiler_b200 import native

    lib = native.load()
    table = native.int32_table([2, 2])
    rc = lib.gacb_msda_forward(v.data_ptr(), 0, loc.data_ptr(), attn.data_ptr(), v.data_ptr(), table, 1, 1, 6, 3, 2, 32, 4, 0, 3, None)
    assert rc == native.GACB_ERR_SHAPE_MISMATCH and "sum(H*W)" in native.last_error()
    rc = lib.gacb_msda_forward(None, 0, loc.data_ptr(), attn.data_ptr(), v.data_ptr(), native.int32_table([2, 3]), 1, 1, 6, 3, 2, 32, 4, 0, 3, None)
    assert rc == native.GACB_ERR_INVALID_ARGUMENT
    rc = lib.gacb_msda_forward(v.data_ptr(), 5, loc.data_ptr(), attn.data_ptr(), v.data_ptr(), native.int32_table([2, 3]), 1, 1, 6, 3, 2, 32, 4, 0, 3, None)
    assert rc == native.GACB_ERR_INVALID_ARGUMENT
    torch.cuda.synchronize()


def test_evaluate_op_and_session_match_the_oracle(dev):
    """The reference-facing calls: evaluate_op on host arrays, and CudaSession.run (tests/test_cuda_gpu.py:39-58)."""
    from general_ai_compiler_b200 import evaluate_op
    from general_ai_compiler_b200.bevformer import build_msda_graph, make_msda_inputs
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.errors import BackendError, ValidationError
    from general_ai_compiler_b200.session import CudaSession
    from oracle import msda_c

    graph = build_msda_graph()
    inputs = make_msda_inputs(graph, seed=3070)
    expected = msda_c(inputs["value"], inputs["sampling_locations"], inputs["attention_weights"], [(15, 25)])
    (y,) = evaluate_op("MSDeformableAttention", (inputs["value"], inputs["sampling_locations"], inputs["attention_weights"]),
                       {"spatial_shapes": [[15, 25]]})
    np.testing.assert_allclose(y, expected, rtol=1e-4, atol=1e-5)
    with CudaSession(compile_cuda(graph)) as session:
        result = session.run(inputs, profile=True)
        np.testing.assert_allclose(result.outputs["output"], expected, rtol=1e-4, atol=1e-5)
        assert result.kernel_ms is not None and result.kernel_ms > 0 and result.gpu_stream_ms >= result.kernel_ms
        prof = result.profiler.cuda_launch_profile()
        assert prof["launch_count"] == 1 and prof["launches"][0]["op"] == "MSDeformableAttention"
        again = session.run(inputs)
        assert np.array_equal(again.outputs["output"], result.outputs["output"]) and again.kernel_ms is None
        with pytest.raises(ValidationError):
            session.run({"value": inputs["value"]})
        times = session.run_resident(3)
        assert len(times) == 3 and all(t > 0 for t in times)
    with pytest.raises(BackendError):
        session.run(inputs)
    with CudaSession(compile_cuda(graph, value_storage="bfloat16")) as session:
        assert_rel_gate(session.run(inputs).outputs["output"], expected, 1e-2, "bf16 session")
    # per-batch-entry copy/compute/copy pipeline: same bits as the single launch, also when run twice
    with CudaSession(compile_cuda(graph), overlap_batches=True) as session:
        first = session.run(inputs).outputs["output"]
        assert np.array_equal(first, result.outputs["output"])
        other = make_msda_inputs(graph, seed=11)
        want_other = msda_c(other["value"], other["sampling_locations"], other["attention_weights"], [(15, 25)])
        np.testing.assert_allclose(session.run(other).outputs["output"], want_other, rtol=1e-4, atol=1e-5)
        assert np.array_equal(session.run(inputs).outputs["output"], first)


def test_gather_probe_contract_and_launch():
    """The measurement helper rejects bad arguments before launching and reports the bytes one launch gathers."""
    import ctypes

    import torch

    from general_ai_compiler_b200 import native

    lib = native.load()
    dev = torch.device("cuda", 0)
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    got = ctypes.c_size_t(0)
    assert lib.gacb_gather_probe(buf.data_ptr(), buf.numel(), 8, 32, 16, 1, sink.data_ptr(), ctypes.byref(got), None) == 0
    torch.cuda.synchronize()
    assert got.value == 8 * 256 * 32 * 16 and int(sink.item()) == 0
    assert lib.gacb_gather_probe(buf.data_ptr(), buf.numel(), 8, 32, 4, 1, sink.data_ptr(), ctypes.byref(got), None) == 0
    torch.cuda.synchronize()
    assert got.value == 8 * 256 * 32 * 4 and int(sink.item()) == 0
    assert lib.gacb_gather_probe(buf.data_ptr(), buf.numel(), 8, 24, 16, 1, sink.data_ptr(), None, None) == -1     # not a multiple of 16
    assert lib.gacb_gather_probe(buf.data_ptr(), buf.numel(), 8, 32, 8, 1, sink.data_ptr(), None, None) == -1      # lane_bytes
    assert lib.gacb_gather_probe(buf.data_ptr() + 16, buf.numel() - 16, 8, 32, 16, 1, sink.data_ptr(), None, None) == -1
    assert lib.gacb_gather_probe(None, 1024, 8, 32, 16, 1, sink.data_ptr(), None, None) == -1
    assert lib.gacb_gather_probe(buf.data_ptr(), 3 * 128, 8, 32, 16, 1, sink.data_ptr(), None, None) == -1       # not a power of two
    assert "gather probe" in native.last_error()


def _tile_mode(mode):
    from general_ai_compiler_b200 import native

    return native.load().gacb_msda_tile_path(mode)


@pytest.mark.parametrize("key", ["tiny_tsa", "base_tsa"])
def test_tile_kernel_is_bit_identical_to_the_rows_kernel(key, dev):
    """Temporal self-attention shapes (one level, queries = the level's raster) run the shared-memory tile kernel;
    switching it off runs the general rows kernel on the same inputs.  The two must agree bit for bit, whole and
    sharded by query ranges that start and end inside a grid row."""
    torch, ops, device = dev
    from general_ai_compiler_b200.bevformer import WORKLOADS, make_workload_inputs
    from oracle import msda_c

    w = WORKLOADS[key]
    x = make_workload_inputs(w)
    args = (x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    previous = _tile_mode(0)
    try:
        rows = _run(dev, *args)
        _tile_mode(1)
        tile = _run(dev, *args)
        assert torch.equal(tile, rows)
        assert_fp32_gate(tile.cpu().numpy(), msda_c(*args), key)
        out = torch.full_like(rows, float("nan"))
        q = w.queries
        bounds = [0, 17, q // 3 + 5, q // 3 + 6, q - 1, q]
        for q0, q1 in zip(bounds[:-1], bounds[1:]):
            _run(dev, *args, q_range=(q0, q1), out=out)
        assert torch.equal(out, rows)
        part = torch.full_like(rows, 3.0)
        _run(dev, *args, q_range=(w.queries // 2 + 3, w.queries // 2 + 40), out=part)
        keep = torch.ones(w.queries, dtype=torch.bool, device=device)
        keep[w.queries // 2 + 3:w.queries // 2 + 40] = False
        assert torch.all(part[:, keep] == 3.0) and torch.equal(part[:, ~keep], rows[:, ~keep])
    finally:
        _tile_mode(previous)


def test_tile_kernel_samples_far_from_their_cell_and_softmax_form(dev):
    """Samples anywhere in (and outside) the map: most taps miss the staged window and come from global memory,
    level extents that are not multiples of the tile, scores with the softmax in the kernel."""
    torch, ops, device = dev
    from oracle import msda_c
    from oracle.msda_numpy import msda_logits_forward

    rng = np.random.default_rng(77)
    for (hh, ww), batch, points in (((37, 53), 2, 4), ((16, 16), 1, 8), ((61, 18), 3, 3)):
        q = hh * ww
        value = rng.standard_normal((batch, q, 8, 32)).astype(np.float32)
        near = np.stack(np.meshgrid((np.arange(ww) + 0.5) / ww, (np.arange(hh) + 0.5) / hh, indexing="xy"), -1).reshape(1, q, 1, 1, 1, 2)
        loc = (near + rng.standard_normal((batch, q, 8, 1, points, 2)) * 0.04).astype(np.float32)
        far = rng.uniform(-0.2, 1.2, loc.shape).astype(np.float32)
        loc = np.where(rng.uniform(size=(batch, q, 8, 1, points, 1)) < 0.3, far, loc).astype(np.float32)
        logits = rng.standard_normal((batch, q, 8, 1, points)).astype(np.float32)
        attn = rng.uniform(0, 1, logits.shape).astype(np.float32)
        shapes = [(hh, ww)]
        previous = _tile_mode(0)
        try:
            rows = _run(dev, value, loc, attn, shapes)
            _tile_mode(1)
            tile = _run(dev, value, loc, attn, shapes)
            assert torch.equal(tile, rows), (hh, ww)
            assert_fp32_gate(tile.cpu().numpy(), msda_c(value, loc, attn, shapes), f"tile {hh}x{ww}")
            t = [torch.from_numpy(a).to(device) for a in (value, loc, logits)]
            soft = ops.msda_forward(*t, shapes, softmax=True)
            _tile_mode(0)
            soft_rows = ops.msda_forward(*t, shapes, softmax=True)
            torch.cuda.synchronize()
            assert torch.equal(soft, soft_rows)
            assert_fp32_gate(soft.cpu().numpy(), msda_logits_forward(value, loc, logits, shapes), f"tile softmax {hh}x{ww}")
        finally:
            _tile_mode(previous)


def test_session_rejects_non_finite_inputs_on_the_staging_pass_and_stays_usable(dev):
    """The default session checks for non-finite values while it copies the inputs into its pinned buffers, slab by
    slab, before any kernel is launched: a NaN in the last camera raises ``ValidationError``, and the next run with
    clean inputs gives the oracle's result."""
    from general_ai_compiler_b200.bevformer import WORKLOADS, build_msda_graph_for, make_workload_inputs
    from general_ai_compiler_b200.compiler import compile_cuda
    from general_ai_compiler_b200.errors import ValidationError
    from general_ai_compiler_b200.session import CudaSession
    from oracle import msda_c

    w = WORKLOADS["base_sca"].with_queries(300)          # value is large enough to be staged camera by camera
    x = make_workload_inputs(w)
    want = msda_c(x["value"], x["sampling_locations"], x["attention_weights"], w.spatial_shapes)
    with CudaSession(compile_cuda(build_msda_graph_for(w))) as session:
        assert_fp32_gate(session.run(x).outputs["output"], want, "default session")
        for name in ("value", "sampling_locations", "attention_weights"):
            bad = {k: v.copy() for k, v in x.items()}
            bad[name].reshape(-1)[-3] = np.inf
            with pytest.raises(ValidationError, match=f"input '{name}' must contain finite values"):
                session.run(bad)
        assert_fp32_gate(session.run(x).outputs["output"], want, "after rejected inputs")
        pinned = session.pinned_inputs()                  # filled in place: checked where they are
        for k, v in x.items():
            np.copyto(pinned[k], v)
        assert_fp32_gate(session.run(pinned).outputs["output"], want, "pinned inputs")
        pinned["value"].reshape(-1)[5] = np.nan
        with pytest.raises(ValidationError, match="finite"):
            session.run(pinned)
