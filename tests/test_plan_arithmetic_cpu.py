"""Host-side arithmetic of the multi-tensor launch plans, without a GPU: tile counts, tile prefix,
descriptor fields and the switch away from the 32-bit fast path for tensors of 2^31 elements or more.

The tensors are ``meta`` tensors (shapes and strides, no storage), so a 2^31-element matrix costs
nothing; the plan code only reads shapes, strides and addresses.  Model: the reference's large-tensor
coverage (``tests/test_large_tensor_paths.py``, > 2^31 elements), restated for the host part of this
package's descriptor-driven kernels.
"""
import ctypes

import pytest
import torch

from gefen_x_b200.ops import update as U

pytestmark = pytest.mark.skipif(not U.available(), reason="the descriptor layout comes from the built extension")


def _item(rows, cols, period, *, factored=True, dtype=torch.bfloat16):
    shape = (rows, cols) if cols else (rows,)
    numel = rows * (cols or 1)
    nb = numel // period
    p = torch.empty(shape, dtype=dtype, device="meta")
    st = {"m_codebook": torch.empty(nb, period, dtype=torch.uint8, device="meta"),
          "m_magnitude": torch.empty(nb, 1, dtype=torch.float32, device="meta"), "automatic_period": period}
    if factored:
        st["v_row"] = torch.empty(rows, dtype=torch.float32, device="meta")
        st["v_col"] = torch.empty(cols, dtype=torch.float32, device="meta")
    else:
        st["vmean"] = torch.empty(nb, 1, dtype=torch.float32, device="meta")
    return U.Item(p=p, grad=torch.empty(shape, dtype=dtype, device="meta"), state=st, period=period,
                  beta1=0.9, beta2=0.999, eps=1e-8)


def _descs(plan):
    raw = bytearray(plan.descs.cpu().numpy().tobytes())
    stride = len(raw) // plan.n
    return [U.TensorDesc.from_buffer_copy(bytes(raw[i * stride:(i + 1) * stride])) for i in range(plan.n)]


def test_matrix_of_two_to_the_31_elements_leaves_the_32_bit_path():
    big = _item(65536, 32768, 32768)                       # 2^31 elements
    small = _item(4096, 4096, 4096)
    plan = U.Plan("factored", [small, big], torch.device("cpu"), torch.bfloat16)
    d_small, d_big = _descs(plan)
    assert d_big.numel == 2 ** 31 and d_big.nb == 65536 and d_big.rows == 65536 and d_big.cols == 32768
    assert not plan.fast                                   # one tensor beyond 2^31 - 1 elements: general kernels
    assert U.Plan("factored", [small], torch.device("cpu"), torch.bfloat16).fast
    for d in (d_small, d_big):
        assert d.tcols * d.trows == 256 and d.vec == 1
        chunks = d.cols // 8
        assert d.n_col_tiles == -(-chunks // d.tcols)
        assert d.rows_per_tile % d.trows == 0
    start = plan.tile_start.tolist()
    tiles = [d.n_col_tiles * -(-d.rows // d.rows_per_tile) for d in (d_small, d_big)]
    assert start == [0, tiles[0], tiles[0] + tiles[1]] and plan.total_tiles == start[-1]
    # every element of the big matrix is covered exactly once by its tiles
    assert d_big.n_col_tiles * d_big.tcols * 8 >= d_big.cols
    assert -(-d_big.rows // d_big.rows_per_tile) * d_big.rows_per_tile >= d_big.rows


def test_block_path_modes_and_long_blocks():
    cases = [(1 << 20, 16, 0), (1 << 20, 256, 1), (1 << 22, 2048, 2)]
    for numel, period, mode in cases:
        it = _item(numel, 0, period, factored=False)
        plan = U.Plan("block", [it], torch.device("cpu"), torch.bfloat16)
        (d,) = _descs(plan)
        assert d.mode == mode and d.nb == numel // period and d.period == period
        want = {0: -(-d.nb // 256), 1: -(-d.nb // 8), 2: d.nb}[mode]
        assert plan.total_tiles == want
    # long blocks and few of them: routed through the two-phase kernels as a matrix whose rows tile the blocks
    assert U.two_phase_block(1 << 20, 64) and not U.two_phase_block(256, 64) and not U.two_phase_block(1 << 20, 4096)
    it = _item(1 << 26, 0, 1 << 20, factored=False)
    it.row_only = True
    plan = U.Plan("factored", [it], torch.device("cpu"), torch.bfloat16)
    (d,) = _descs(plan)
    assert d.row_only == 1 and (1 << 20) % d.cols == 0 and d.rows * d.cols == 1 << 26 and d.nb == 64


def test_state_of_the_wrong_size_is_refused_when_the_plan_is_built():
    it = _item(64, 256, 256)
    it.state["m_magnitude"] = torch.empty(63, 1, dtype=torch.float32, device="meta")
    with pytest.raises(ValueError, match="m_magnitude"):
        U.Plan("factored", [it], torch.device("cpu"), torch.bfloat16)
    it = _item(64, 256, 256)
    it.state["v_col"] = torch.empty(255, dtype=torch.float32, device="meta")
    with pytest.raises(ValueError, match="v_row / v_col"):
        U.Plan("factored", [it], torch.device("cpu"), torch.bfloat16)
    it = _item(64, 256, 128)
    it.state["m_codebook"] = torch.empty(64, 256, dtype=torch.uint8, device="meta")
    with pytest.raises(ValueError, match="m_codebook"):
        U.Plan("factored", [it], torch.device("cpu"), torch.bfloat16)


def test_crowded_bucket_tables_are_recognised_and_remembered_on_the_tensor():
    """The streamed apply kernel settles a value with one comparison, which needs at most one decision
    threshold per bucket of the search table; the host checks the table once and keeps the answer on
    the tensor, so a table that later reuses the same address cannot inherit it."""
    from gefen_x_b200.quant import codebook as C

    torch.manual_seed(5)
    cb = torch.sort(torch.rand(256) * 2 - 1).values
    cb[0], cb[-1] = -1.0, 1.0
    spread = torch.linspace(-1, 1, 256)                       # 7.8e-3 apart: one threshold per bucket at most
    lut = C.packed_search_lut(spread)
    assert U._lut_single(lut) and lut._gx_single_threshold_buckets is True
    crowded = spread.clone()
    crowded[100] = crowded[99] + 1e-6
    crowded[101] = crowded[99] + 2e-6                         # three codewords inside one bucket
    lut2 = C.packed_search_lut(torch.sort(crowded).values)
    assert not U._lut_single(lut2)
    assert int(((lut2.int() & 0xFFFF) >> 8).max()) >= 2


def test_wide_tile_prefix_follows_the_rule_the_kernels_apply():
    """Plans that may run the 16-wide streamed kernels carry a second tile prefix behind the 8-wide one;
    the kernels derive the same geometry from the descriptor (thread columns that waste the fewest
    16-element chunks, the 8-wide rows-per-thread factor)."""
    U.set_wide_chunks(True)
    try:
        items = [_item(4096, 14336, 524288), _item(2048, 1024, 2048), _item(324, 48, 1296)]
        plan = U.Plan("factored", items, torch.device("cpu"), torch.bfloat16)
    finally:
        U.set_wide_chunks(False)
    descs = _descs(plan)
    assert plan.fast == 4
    n = len(items)
    start = plan.tile_start.tolist()
    assert len(start) == 2 * (n + 1) and start[0] == 0 and start[n + 1] == 0
    for i, d in enumerate(descs):
        chunks = d.cols // 16
        tc = U._pick_tcols(chunks)
        rows_per_tile = (256 // tc) * (d.rows_per_tile // d.trows)
        tiles = ((chunks + tc - 1) // tc) * ((d.rows + rows_per_tile - 1) // rows_per_tile)
        assert start[n + 2 + i] - start[n + 1 + i] == tiles
