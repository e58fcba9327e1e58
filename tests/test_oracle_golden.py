"""Pins the CPU oracle (oracle/tiga_oracle.c) against the reference.

Two sources: literal known-answer vectors that the reference's README and
test-suite hold, and fixtures produced by running the unmodified reference
(tests/golden/make_golden.py).  Integer work must match bit for bit; float32
sums must match the reference's CPU evaluator bit for bit as well, because the
oracle keeps its summation order.
"""
import numpy as np
import pytest

GRAPHS = ("fixed16", "ragged", "hub", "empty")


def test_readme_known_answer(oracle):
    # README.md:97-111 of the reference
    row_ptr, col = [0, 2, 3, 5], [0, 2, 1, 0, 1]
    x = np.array([1.0, 2.0, 3.0], np.float32)
    w = np.array([2.0, 3.0, 4.0, 5.0, 6.0], np.float32)
    out = oracle.wsum_fwd(row_ptr, col, x, w)
    assert out.tolist() == [11.0, 8.0, 17.0]
    dy = np.ones(3, np.float32)
    assert oracle.wsum_bwd_dx(row_ptr, col, 3, dy, w).tolist() == [7.0, 10.0, 3.0]
    assert oracle.wsum_bwd_dw(row_ptr, col, dy, x).tolist() == [1.0, 3.0, 2.0, 1.0, 2.0]


def test_mean_known_answers(oracle):
    # tests/python/test_builtin_reducers.py:33-41 and :61-73 of the reference
    row_ptr, col = [0, 2, 3, 5], [0, 2, 1, 0, 1]
    x = np.array([1.0, 2.0, 4.0], np.float32)
    assert oracle.wsum_fwd(row_ptr, col, x, mean=True).tolist() == [2.5, 2.0, 1.5]
    dx = oracle.wsum_bwd_dx(row_ptr, col, 3, np.ones(3, np.float32), mean=True)
    assert dx.tolist() == [1.0, 1.5, 0.5]
    out = oracle.wsum_fwd([0, 2, 2, 4], [0, 2, 0, 1], np.array([2.0, 4.0, 8.0], np.float32), mean=True)
    assert out[0] == 5.0 and np.isnan(out[1]) and out[2] == 3.0


def test_node_epilogue_known_answer(oracle):
    # tests/python/test_torch_default.py:64-87: sum then `incoming + dst.bias`
    out = oracle.wsum_fwd([0, 2, 3, 3], [0, 1, 1], np.array([2.0, 3.0], np.float32),
                          np.array([4.0, 5.0, 2.0], np.float32))
    np.testing.assert_allclose(out + np.array([0.1, 0.2, 0.3], np.float32), [23.1, 6.2, 0.3], rtol=1e-6)
    dy = np.ones(3, np.float32)
    assert oracle.wsum_bwd_dx([0, 2, 3, 3], [0, 1, 1], 2, dy, np.array([4.0, 5.0, 2.0], np.float32)).tolist() == [4.0, 7.0]
    assert oracle.wsum_bwd_dw([0, 2, 3, 3], [0, 1, 1], dy, np.array([2.0, 3.0], np.float32)).tolist() == [2.0, 3.0, 3.0]


def test_triangular_csr_known_answer(oracle):
    # tests/python/test_reference.py:356-365: triangular(4) row_ptr [0,1,3,6,10]
    row_ptr = np.concatenate(([0], np.cumsum(np.arange(1, 5))))
    assert row_ptr.tolist() == [0, 1, 3, 6, 10]


@pytest.mark.parametrize("graph", GRAPHS)
@pytest.mark.parametrize("F", (1, 3, 64))
@pytest.mark.parametrize("tag", ("wsum", "psum", "wmean", "pmean"))
def test_sum_mean_against_reference(oracle, golden, graph, F, tag):
    key = f"{tag}_{graph}_f{F}"
    row_ptr, col, x = golden[key + "_row_ptr"], golden[key + "_col"], golden[key + "_x"]
    w = golden.get(key + "_w")
    mean = "mean" in tag
    identity = 0.5 if tag == "psum" else 0.0
    out = oracle.wsum_fwd(row_ptr, col, x, w, identity=identity, mean=mean)
    ref = golden[key + "_out"]
    assert out.shape == ref.shape
    np.testing.assert_array_equal(out, ref)  # same order => same bits (NaN == NaN here)
    if col.size == 0:
        return
    dy = golden[key + "_dy"]
    if mean:  # the fixture's loss ignores NaN rows: their cotangent is zero
        empty = np.diff(row_ptr) == 0
        dy = dy.copy()
        dy[empty] = 0
    dx = oracle.wsum_bwd_dx(row_ptr, col, x.shape[0], dy, w, mean=mean)
    np.testing.assert_allclose(dx, golden[key + "_dx"], rtol=1e-5, atol=1e-6)
    if w is not None:
        dw = oracle.wsum_bwd_dw(row_ptr, col, dy, x, mean=mean)
        np.testing.assert_allclose(dw.reshape(golden[key + "_dw"].shape), golden[key + "_dw"], rtol=1e-5, atol=2e-6)


def test_online_softmax_against_reference(oracle, golden):
    row_ptr, col = golden["softmax_row_ptr"], golden["softmax_col"]
    score, value = golden["softmax_score"], golden["softmax_value"]
    out, m, l = oracle.online_softmax_fwd(row_ptr, score, value[col])
    np.testing.assert_allclose(out, golden["softmax_out"], rtol=1e-6, atol=1e-7)
    assert np.all(out[1] == 0)  # empty row -> exact zeros
    dscore, dvalue_e = oracle.online_softmax_bwd(row_ptr, score, value[col], out, golden["softmax_dy"])
    np.testing.assert_allclose(dscore, golden["softmax_dscore"], rtol=1e-4, atol=1e-6)
    dvalue = np.zeros_like(value)
    np.add.at(dvalue, col, dvalue_e)
    np.testing.assert_allclose(dvalue, golden["softmax_dvalue"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("graph", ("fixed16", "ragged", "hub"))
def test_gat_against_reference(oracle, golden, graph):
    key = f"gat_{graph}"
    row_ptr, col = golden[key + "_row_ptr"], golden[key + "_col"]
    x, a_src, a_dst = golden[key + "_x"], golden[key + "_a_src"], golden[key + "_a_dst"]
    out, m, l, score = oracle.gat_fwd(row_ptr, col, x, x, a_src, a_dst)
    ref = oracle.bf16_to_f32(golden[key + "_out"])
    got = oracle.bf16_to_f32(out)
    # bf16 logits differ from torch's by at most an ulp of the float32 partial sums
    np.testing.assert_allclose(got, ref, rtol=2e-2, atol=2e-2)
    assert np.mean(got == ref) > 0.9
    dxs, dxd, das, dad = oracle.gat_bwd(row_ptr, col, x, x, a_src, a_dst, golden[key + "_dy"])
    ref_dx = oracle.bf16_to_f32(golden[key + "_dx"])
    err = np.abs(dxs + dxd - ref_dx)
    # the reference's own gradient runs through bf16 autograd: bf16-level noise
    assert np.median(err) < 2e-2 * np.abs(ref_dx).mean() + 1e-3
    for mine, name in ((das, "_da_src"), (dad, "_da_dst")):
        ref_a = oracle.bf16_to_f32(golden[key + name])
        scale = np.abs(ref_a).max() + 1e-6
        assert np.abs(mine - ref_a).max() / scale < 8e-2


def test_varlen_attention_against_reference(oracle, golden):
    cu = golden["attn_cu"]
    q, k, v = golden["attn_q"], golden["attn_k"], golden["attn_v"]
    scale = float(golden["attn_scale"])
    out, lse = oracle.varlen_attn_fwd(cu, q, k, v, scale, causal=True)
    np.testing.assert_allclose(out, golden["attn_out"], rtol=2e-5, atol=2e-6)
    dq, dk, dv = oracle.varlen_attn_bwd(cu, q, k, v, out, golden["attn_dy"], scale, causal=True)
    np.testing.assert_allclose(dq, golden["attn_dq"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dk, golden["attn_dk"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dv, golden["attn_dv"], rtol=1e-4, atol=1e-5)
    # the packed causal relation itself: position i of a sequence gathers [start, i]
    row_ptr, col = golden["attn_row_ptr"], golden["attn_col"]
    start = np.repeat(cu[:-1], np.diff(cu))
    deg = np.arange(cu[-1]) - start + 1
    np.testing.assert_array_equal(row_ptr, np.concatenate(([0], np.cumsum(deg))))
    np.testing.assert_array_equal(col, np.concatenate([np.arange(s, i + 1) for s, i in zip(start, np.arange(cu[-1]))]))


def test_csr_construction_bit_exact(oracle, golden):
    row_ptr, col, order = oracle.coo_to_csr(golden["coo_src"], golden["coo_dst"], 17)
    np.testing.assert_array_equal(row_ptr, golden["coo_row_ptr"])
    np.testing.assert_array_equal(col, golden["coo_col"])
    np.testing.assert_array_equal(oracle.destination_index(row_ptr), golden["coo_destination"])
    t_ptr, t_col, t_order = oracle.csr_transpose(row_ptr, col, 23)
    np.testing.assert_array_equal(t_ptr, golden["coo_t_ptr"])
    np.testing.assert_array_equal(t_col, golden["coo_t_col"])
    np.testing.assert_array_equal(t_order, golden["coo_t_order"])
    lo, hi, total = oracle.degree_stats(row_ptr)
    assert [lo, hi] == golden["coo_degree_bounds"].tolist() and total == col.size


def test_partition_and_halo_bit_exact(oracle, golden):
    for entities, world, rank, b, e in golden["owned_range_table"]:
        assert oracle.owned_range(entities, world, rank) == (b, e)
    for entity, entities, world, owner in golden["destination_owner_table"]:
        assert oracle.destination_owner(entity, entities, world) == owner
    row_ptr, col = golden["halo_row_ptr"], golden["halo_col"]
    n = row_ptr.size - 1
    for world in (2, 3, 4):
        ghosts = [oracle.derive_ghosts(row_ptr, col, n, world, r) for r in range(world)]
        for r in range(world):
            np.testing.assert_array_equal(ghosts[r], golden[f"halo_w{world}_r{r}_ghosts"])
            assert int(golden[f"halo_w{world}_r{r}_bytes"]) == ghosts[r].size * 4 * 64
            b, e = oracle.owned_range(n, world, r)
            for peer in range(world):
                recv = np.array([g for g in ghosts[r] if oracle.destination_owner(g, n, world) == peer], np.int64)
                key = f"halo_w{world}_r{r}_recv{peer}"
                np.testing.assert_array_equal(recv, golden.get(key, np.zeros(0, np.int64)))
                send = np.array([g for g in ghosts[peer] if b <= g < e], np.int64)
                key = f"halo_w{world}_r{r}_send{peer}"
                np.testing.assert_array_equal(send, golden.get(key, np.zeros(0, np.int64)))
            # local renumbering: owned first, ghosts after in ascending global id
            lp, lc = oracle.local_csr(row_ptr, col, n, world, r, ghosts[r])
            glob = np.concatenate((np.arange(b, e), ghosts[r]))
            np.testing.assert_array_equal(glob[lc], col[row_ptr[b]:row_ptr[e]])
            np.testing.assert_array_equal(lp, row_ptr[b:e + 1] - row_ptr[b])


def test_max_reducer_algebra(oracle):
    # parity unpinned by the reference; check the algebra on a hand case
    row_ptr, col = [0, 3, 3, 5], [0, 1, 2, 2, 0]
    x = np.array([[1.0, -2.0], [3.0, -2.0], [2.0, np.nan]], np.float32)
    out, arg = oracle.max_fwd(row_ptr, col, x)
    assert out[0, 0] == 3.0 and arg[0, 0] == 1
    assert np.isnan(out[0, 1]) and arg[0, 1] == 2       # NaN propagates (arith.maximumf)
    assert np.all(np.isneginf(out[1])) and np.all(arg[1] == -1)  # empty row -> identity
    assert out[2, 0] == 2.0 and arg[2, 0] == 3          # first winner kept
    dx, dw = oracle.max_bwd(row_ptr, col, 3, np.ones((3, 2), np.float32), x, arg)
    assert dx[1, 0] == 1.0 and dx[2, 0] == 1.0 and dx[0, 0] == 0.0


def test_product_reducer_known_answers_and_reference_fixtures(oracle):
    """tg.prod(): the values the reference's tests assert (tests/python/test_builtin_reducers.py:44-59,
    tests/python/test_message_passing_autograd.py:439-485) and the fixtures its Torch evaluator
    produced (tests/golden/make_golden_programs.py): forward bit for bit (same left fold from 1),
    cotangents within float32 rounding (Torch divides the row product by the message, the oracle
    multiplies the other messages)."""
    import os

    row_ptr, col = np.array([0, 2, 2, 5]), np.array([0, 1, 0, 1, 2])
    x = np.array([2.0, 3.0, 5.0], np.float32)
    out = oracle.product_fwd(row_ptr, x[col])
    assert out.tolist() == [6.0, 1.0, 30.0]
    d_message = oracle.product_vjp(row_ptr, x[col], np.ones(3, np.float32))
    assert np.bincount(col, weights=d_message, minlength=3).tolist() == [18.0, 12.0, 6.0]
    edge = np.array([2.0, 0.0, 3.0, 4.0, 5.0], np.float32)
    assert oracle.product_fwd([0, 3, 5], edge).tolist() == [0.0, 20.0]
    assert oracle.product_vjp([0, 3, 5], edge, np.array([7.0, 11.0], np.float32)).tolist() == [0.0, 42.0, 0.0, 55.0, 44.0]

    cases = dict(np.load(os.path.join(os.path.dirname(__file__), "golden", "program_cases.npz")))
    row_ptr, col = cases["row_ptr"], cases["col"]
    message = cases["prod_edge_in_x"]
    np.testing.assert_array_equal(oracle.product_fwd(row_ptr, message), cases["prod_edge_out"])
    np.testing.assert_allclose(oracle.product_vjp(row_ptr, message, cases["prod_edge_dy"]), cases["prod_edge_d_x"],
                               rtol=2e-5, atol=1e-7)
    x = cases["prod_src_in_x"]
    np.testing.assert_array_equal(oracle.product_fwd(row_ptr, x[col]), cases["prod_src_out"])
    d_message = oracle.product_vjp(row_ptr, x[col], cases["prod_src_dy"])
    d_x = np.zeros_like(x)
    np.add.at(d_x, col, d_message)
    np.testing.assert_allclose(d_x, cases["prod_src_d_x"], rtol=1e-4, atol=1e-6)
