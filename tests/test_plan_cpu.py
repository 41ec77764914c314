"""CPU: the launch planner, pinned at the benchmark configurations.

Which kernel a product takes -- tile width, CTA pairing, the A operand from tensor memory, the split of the
contraction, the balanced tail, how many SMs two side-by-side products get, streaming kernels for few rows,
pieces of a long contraction -- is host arithmetic over shapes, strides and the SM count, so it is checked here
without a device through `mni_b200_plan_describe`.  The pins are the plans the measured numbers were taken
with: a change of the planner that moves one of them is a performance change and must be re-measured.  (The
reference has no counterpart: it hands every product to cuBLAS, ops/matmul.rs:145-190.)"""
import re

import pytest


@pytest.fixture(scope="module")
def plan():
    from framework_b200 import build, ops
    build.build_library()
    return ops.plan_describe


def fields(line):
    """'grad_a: tensor m=512 n=64 ...' -> ('grad_a', 'tensor', {'m': 512, ...})"""
    label, rest = line.split(": ", 1)
    kind = rest.split(" ", 1)[0]
    return label, kind, {k: int(v) for k, v in re.findall(r"(\w+)=(-?\d+)", rest)}


def by_label(lines):
    out = {}
    for line in lines:
        if ": " in line:
            label, kind, f = fields(line)
            out.setdefault(label, []).append((kind, f, line))
    return out


def tensor_plan(lines, label):
    entries = [e for e in by_label(lines)[label] if e[0] == "tensor"]
    assert len(entries) == 1, lines
    return entries[0][1]


def test_default_benchmark_shape_whole_and_as_an_eighth(plan):
    """[64,1024,768] x [768,3072]: 256-wide CTA pairs on every SM; the weight gradient folds the batches into the
    contraction and splits it two ways (72 units on 72 pairs), summed in pieces of about 1024."""
    for batches in (64, 8):
        fwd = tensor_plan(plan((batches, 1024, 768), (768, 3072)), "forward")
        assert (fwd["bn"], fwd["bk"], fwd["pair"], fwd["tmem_a"], fwd["splits"], fwd["grid"]) == (256, 16, 1, 0, 1, 148)
        assert fwd["batch"] == batches and fwd["pieces"] == 1
        bwd = plan((batches, 1024, 768), (768, 3072), backward=1)
        da, dw = tensor_plan(bwd, "grad_a"), tensor_plan(bwd, "grad_b")
        assert (da["m"], da["n"], da["k"], da["batch"], da["pieces"]) == (1024, 768, 3072, batches, 3)
        assert (dw["m"], dw["n"], dw["k"], dw["batch"], dw["fold"]) == (768, 3072, 1024, 1, batches)
        assert (dw["splits"], dw["grid"]) == (2, 144)
        assert dw["pieces"] == batches // 2                  # (batches * 1024 / 2) / 1024
        assert not any("side by side" in line for line in bwd)        # large products run one after the other
        # whole: 768 pair-tiles = 10.4 rounds, the ragged wave is left alone; an eighth: 96 tiles on 74 pairs
        # would be two rounds at 0.65 -> balanced tail
        assert da["tail"] == (1 if batches == 8 else 0) and da["grid"] == 148


def test_reserved_sms_shrink_the_grid(plan):
    """What the step driver reserves for the collective comes out of the persistent grid, in whole pairs."""
    for sms, grid in ((148, 148), (146, 146), (132, 132)):
        assert tensor_plan(plan((64, 1024, 768), (768, 3072), sm_count=sms), "forward")["grid"] == grid


def test_linear_layer(plan):
    """x[4096,1024] . W[1024,4096] + b: one round of pair tiles; the bias gradient's column sums go beside the
    products; both gradients contract over 4096 in four pieces."""
    fwd = tensor_plan(plan((4096, 1024), (1024, 4096)), "forward")
    assert (fwd["bn"], fwd["pair"], fwd["splits"], fwd["tail"], fwd["pieces"]) == (256, 1, 1, 0, 1)
    bwd = plan((4096, 1024), (1024, 4096), backward=2)
    assert any(line.startswith("grad_bias: column sums") and "side stream" in line for line in bwd)
    for label in ("grad_a", "grad_b"):
        g = tensor_plan(bwd, label)
        assert (g["bn"], g["pair"], g["splits"], g["pieces"], g["grid"]) == (256, 1, 1, 4, 128)


def test_attention_shapes_strided_key_and_narrow_outputs(plan):
    """S = Q.K^T with K read through its strides (no gather), O = S.V with 64-wide tiles and A from tensor
    memory; the two gradients of each run side by side on half of the SMs; dK^T (64 rows) is computed with
    the operands exchanged."""
    q, kt = (8, 12, 512, 64), (8, 12, 64, 512)
    s_fwd = plan(q, kt, b_strides=(393216, 32768, 1, 64))
    assert not any("gather" in line for line in s_fwd)
    f = tensor_plan(s_fwd, "forward")
    assert (f["bn"], f["pair"], f["batch"], f["k"], f["grid"]) == (256, 1, 96, 64, 148)
    s_bwd = plan(q, kt, b_strides=(393216, 32768, 1, 64), backward=1)
    assert any("side by side" in line for line in s_bwd)
    dq, dkt = tensor_plan(s_bwd, "grad_a"), tensor_plan(s_bwd, "grad_b")
    assert (dq["bn"], dq["tmem_a"], dq["grid"], dq["exchanged"]) == (64, 1, 74, 0)
    assert (dkt["bn"], dkt["tmem_a"], dkt["grid"], dkt["exchanged"]) == (64, 1, 74, 1)
    o_fwd = tensor_plan(plan((8, 12, 512, 512), (8, 12, 512, 64)), "forward")
    assert (o_fwd["bn"], o_fwd["tmem_a"], o_fwd["pair"], o_fwd["splits"], o_fwd["grid"]) == (64, 1, 0, 1, 148)
    assert o_fwd["mma_n"] == 64
    o_bwd = plan((8, 12, 512, 512), (8, 12, 512, 64), backward=1)
    ds, dv = tensor_plan(o_bwd, "grad_a"), tensor_plan(o_bwd, "grad_b")
    assert (ds["bn"], ds["pair"], ds["grid"]) == (256, 1, 74)
    assert (dv["bn"], dv["tmem_a"], dv["grid"]) == (64, 1, 74)


def test_small_square_is_split_over_the_gpu(plan):
    """512^3 has 8 tiles of 128 x 256: the cost model picks narrow tiles and a 4-way split instead."""
    f = tensor_plan(plan((512, 512), (512, 512)), "forward")
    assert (f["bn"], f["tmem_a"], f["splits"], f["grid"]) == (64, 1, 4, 128)
    bwd = plan((512, 512), (512, 512), backward=1)
    assert any("side by side" in line for line in bwd)
    for label in ("grad_a", "grad_b"):
        g = tensor_plan(bwd, label)
        assert g["splits"] * (512 // 128) * (512 // g["bn"]) == g["grid"] <= 74


def test_long_contraction_is_summed_in_pieces(plan):
    f = tensor_plan(plan((8192, 8192), (8192, 8192)), "forward")
    assert (f["bn"], f["pair"], f["splits"], f["grid"], f["pieces"]) == (256, 1, 1, 148, 8)


def test_few_rows_take_the_streaming_kernels(plan):
    """M = 1, 4 at K = N = 4096: all three products stream the weight through CUDA-core kernels; at 16 rows the
    tensor path takes over, forward and input gradient with the operands exchanged."""
    for rows in (1, 4):
        fwd = plan((rows, 4096), (4096, 4096))
        assert fwd == ["forward: streaming (skinny) forward kernel"]
        bwd = by_label(plan((rows, 4096), (4096, 4096), backward=1))
        assert bwd["grad_a"][0][0] == "streaming" and bwd["grad_b"][0][0] == "streaming"
    f = tensor_plan(plan((16, 4096), (4096, 4096)), "forward")
    assert (f["exchanged"], f["m"], f["n"], f["bn"], f["tmem_a"], f["splits"]) == (1, 4096, 16, 64, 1, 4)
    assert f["mma_n"] == 16                              # a 64-wide tile over 16 columns multiplies 16
    bwd = plan((16, 4096), (4096, 4096), backward=1)
    assert tensor_plan(bwd, "grad_a")["exchanged"] == 1
    dw = tensor_plan(bwd, "grad_b")
    assert (dw["m"], dw["n"], dw["k"], dw["bn"], dw["pair"]) == (4096, 4096, 16, 256, 1)


def test_flags_and_undescribable_views(plan):
    """The single-pass flag reaches the plan; a view whose matrix dims both have a stride other than one cannot be
    described to TMA and is gathered first; a forced split is honoured."""
    from framework_b200 import _lib
    f = tensor_plan(plan((1024, 1024), (1024, 1024), flags=_lib.PRECISION_TF32 | _lib.FORCE_TENSOR_PATH), "forward")
    assert f["single_pass"] == 1 and f["bk"] == 32
    strided = plan((256, 256), (256, 256), a_strides=(512, 2))
    assert any("gather of a strided operand" in line for line in strided)
    assert tensor_plan(plan((256, 256), (256, 256), flags=_lib.force_split_k(3)), "forward")["splits"] == 3


def test_mma_width_follows_the_output_width(plan):
    """Lone-CTA tiles wider than the output: MMAs in units of 16 columns for a K-major B (here b is given
    transposed, so its rows are contiguous along the contraction), whole 32-float chunks for an MN-major one."""
    from framework_b200 import _lib
    t = _lib.FORCE_TENSOR_PATH
    k_major = {n: tensor_plan(plan((128, 256), (256, n), b_strides=(1, 256), flags=t), "forward")["mma_n"]
               for n in (8, 16, 24, 40, 64, 100)}
    assert k_major == {8: 16, 16: 16, 24: 32, 40: 48, 64: 64, 100: 64}      # 100 columns: two 64-wide tiles
    mn_major = {n: tensor_plan(plan((128, 256), (256, n), flags=t), "forward")["mma_n"] for n in (8, 40, 64, 100)}
    assert mn_major == {8: 32, 40: 64, 64: 64, 100: 64}
    # CTA pairs keep full-width MMAs
    wide = tensor_plan(plan((32768, 256), (256, 200), flags=t), "forward")
    assert (wide["bn"], wide["pair"], wide["mma_n"]) == (256, 1, 256)


def test_errors_are_the_calls_own(plan):
    from framework_b200 import _lib
    with pytest.raises(_lib.MniError) as ei:
        plan((2, 3), (4, 2))
    assert ei.value.status == 2 and "inner dimensions must match" in ei.value.message
    with pytest.raises(_lib.MniError) as ei:
        plan((2, 3), (3, 2), sm_count=0)
    assert ei.value.status == 4
