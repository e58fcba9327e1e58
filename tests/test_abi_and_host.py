"""CPU-side checks: the C-ABI library loads and exports every declared symbol,
and the host-side mirror of the reference API behaves like the reference
(golden fixtures made by the reference itself)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import tiga as tg
from tiga import _native
from tiga import capture as cap
from tiga.distributed import model as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tiga_b200.h")).read()
    return sorted(set(re.findall(r"TGB_API[^;]*?\b(tgb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    declared = _declared_symbols()
    assert len(declared) >= 12
    handle = ctypes.CDLL(_native.library_path())
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in include/tiga_b200.h but not exported"
    assert set(declared) == set(_native.exported_symbols())


def test_status_strings_follow_reference_codes():
    lib = _native.lib()
    assert lib.tgb_status_string(0) == b"ok"
    assert lib.tgb_status_string(1) == b"invalid argument"
    assert lib.tgb_status_string(2) == b"unsupported"
    assert lib.tgb_status_string(3) == b"out of memory"
    assert lib.tgb_status_string(4) == b"internal error"
    assert b"sm_100a" in lib.tgb_version()


def test_argument_errors_without_gpu():
    lib = _native.lib()
    size = ctypes.c_uint64()
    assert lib.tgb_csr_plan_sizes(4, 4, 4, 16, 1, ctypes.byref(size), ctypes.byref(size)) == _native.INVALID_ARGUMENT
    assert b"index_bits" in lib.tgb_last_error()
    assert lib.tgb_csr_plan_sizes(1 << 31, 4, 4, 64, 1, ctypes.byref(size), ctypes.byref(size)) == _native.UNSUPPORTED
    assert lib.tgb_csr_reduce_fwd(None, 0, None, None, None, None, 4, 0, 0.0, 0, None, 0, 0) == _native.INVALID_ARGUMENT
    with pytest.raises(ValueError):
        _native.check(_native.INVALID_ARGUMENT, "probe")


def test_cpu_call_is_refused_not_emulated():
    class WeightedSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    g = tg.Graph.from_csr(torch.tensor([0, 2, 3, 5]), torch.tensor([0, 2, 1, 0, 1]), num_src=3)
    with pytest.raises(NotImplementedError):
        WeightedSum()(graph=g, src={"x": torch.ones(3)}, dst={}, edge={"weight": torch.ones(5)})


def test_reference_evaluator_matches_readme():
    class WeightedSum(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge):
            return edge.weight * src.x

    g = tg.Graph.from_csr(torch.tensor([0, 2, 3, 5]), torch.tensor([0, 2, 1, 0, 1]), num_src=3)
    x = torch.tensor([1.0, 2.0, 3.0], requires_grad=True)
    w = torch.tensor([2.0, 3.0, 4.0, 5.0, 6.0], requires_grad=True)
    out = WeightedSum().reference(graph=g, src={"x": x}, dst={}, edge={"weight": w})
    dx, dw = torch.autograd.grad(out.sum(), (x, w))
    assert out.tolist() == [11.0, 8.0, 17.0] and dx.tolist() == [7.0, 10.0, 3.0]
    assert dw.tolist() == [1.0, 3.0, 2.0, 1.0, 2.0]


def test_capture_recognisers():
    class Plain(tg.MessagePassing):
        def edge(self, src, dst, edge):
            return src.h

    class Weighted(tg.MessagePassing):
        def edge(self, src, dst, edge):
            return src.x * edge.w

    class GAT(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, a_src, a_dst):
            s = (src.x * a_src).sum(dim=-1) + (a_dst * dst.x).sum(dim=-1)
            return self.reducer(tg.math.maximum(s, 0.2 * s), src.x)

    class Attention(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge, scale):
            return self.reducer((src.key * dst.query).sum(dim=-1) * scale, src.value)

    class Opaque(tg.MessagePassing):
        def edge(self, src, dst, edge):
            return torch.relu(src.x)

    assert cap.recognize_weighted_sum(cap.capture_edge(Plain().edge, {})) == cap.WeightedSumPattern("h", None)
    assert cap.recognize_weighted_sum(cap.capture_edge(Weighted().edge, {})) == cap.WeightedSumPattern("x", "w")
    gat = cap.recognize_gat(cap.capture_edge(GAT().edge, {"a_src": torch.zeros(2), "a_dst": torch.zeros(2)}))
    assert gat == cap.GATPattern("x", "x", "a_src", "a_dst", 0.2)
    dense = cap.recognize_dense_attention(cap.capture_edge(Attention().edge, {"scale": 0.25}))
    assert dense == cap.DenseAttentionPattern("key", "query", "value", 0.25)
    assert cap.capture_edge(Opaque().edge, {}) is None

    class UserMax(tg.Reducer):
        associative = commutative = True

        def identity(self):
            return float("-inf")

        def combine(self, left, right):
            return tg.math.maximum(left, right)

    assert cap.reducer_algebra(UserMax()) == "max"
    assert cap.reducer_algebra(tg.sum()) == "sum"
    assert cap.reducer_algebra(tg.prod()) == "prod"

    class UserProduct(tg.Reducer):
        name = "user_product"
        associative = commutative = True

        def identity(self):
            return 1.0

        def combine(self, left, right):
            return right * left

    assert cap.reducer_algebra(UserProduct()) == "prod"

    # float keyword parameters of edge() are read at every call, unless Python itself consumed the value
    from tiga import edge_program as ep

    class Scaled(tg.MessagePassing):
        def edge(self, src, dst, edge, scale, shift):
            return (src.u - dst.u) * scale + shift * 2.0 + 0.25

    consumed = set()
    staged = cap.capture_edge(Scaled().edge, {"scale": 0.25, "shift": 0.25}, consumed)
    assert consumed == {"shift"}                                  # shift * 2.0 happened in Python
    program = ep.compile_expression(staged).literalised(frozenset(consumed))
    assert program.constant_names == ("scale", None, None) and program.constants == (0.25, 0.5, 0.25)
    assert program.rebound({"scale": 0.75}).constants == (0.75, 0.5, 0.25)
    assert program.rebound({"scale": 0.75}).key() == program.key()

    # the same program as generated CUDA source, compiled for sm_100a by the runtime compiler (no GPU needed)
    from tiga import edge_jit

    source = edge_jit.generate_source(program, 4, (0, 0), ep.REDUCE_SUM)
    assert "value[2] = __fsub_rn(value[0], value[1]);" in source and "a.constants[0]" in source
    try:
        module = edge_jit.Module(source)
    except edge_jit.CompilerUnavailable:
        module = None
    if module is not None:
        import ctypes

        size = ctypes.c_int64()
        assert _native.lib().tgb_jit_image_bytes(module.handle, ctypes.byref(size)) == 0 and size.value > 1000
        with pytest.raises(RuntimeError, match="did not compile"):
            edge_jit.Module("this is not CUDA")

    # anything else is staged into step / combine / finalize register programs
    from tiga import algebra as alg

    class AffineComposition(tg.Reducer):
        associative = True

        def identity(self):
            return 1.0, 0.0

        def lift(self, scale, bias):
            return scale, bias

        def combine(self, left, right):
            return right[0] * left[0], right[0] * left[1] + right[1]

        def finalize(self, state):
            return state[1]

    assert cap.reducer_algebra(AffineComposition()) is None
    rules = alg.capture_algebra(AffineComposition(), 2)
    assert rules.arity == 2 and rules.identity == (1.0, 0.0) and len(rules.finalize.ops) == 1
    assert rules.step.ops.count(0) == 4 and rules.combine.ops.count(0) == 4       # four argument loads each
    struct = alg.make_struct(rules, (0, 1))
    assert struct.step.num_instructions == len(rules.step.ops) and struct.finalize.out[0] == rules.finalize.outs[0]
    AffineComposition.associative = False
    assert alg.capture_algebra(AffineComposition(), 2) is None
    # tuple states whose components add independently, lifts that are monomials of the message
    mean = cap.capture_reducer(tg.mean())
    assert (mean.kind, mean.components, mean.scalar) == ("additive", ((1.0, 1), (1.0, 0)), False)

    class Moments(tg.Reducer):
        associative = commutative = True

        def identity(self):
            return 0.0, 0.0, 0.0

        def lift(self, message):
            return message, 0.5 * message * message, 1.0

        def combine(self, left, right):
            return left[0] + right[0], right[1] + left[1], left[2] + right[2]

        def finalize(self, state):
            return state[1] / state[2]

    moments = cap.capture_reducer(Moments())
    assert (moments.kind, moments.components) == ("additive", ((1.0, 1), (0.5, 2), (1.0, 0)))

    class Crossed(Moments):          # component 0 mixes in component 1: not independent
        def combine(self, left, right):
            return left[0] + right[1], left[1] + right[1], left[2] + right[2]

    assert cap.capture_reducer(Crossed()) is None

    class FieldSoftmax(tg.MessagePassing):
        reducer = tg.online_softmax()

        def edge(self, src, dst, edge):
            return self.reducer(edge.score, src.value)

    assert cap.recognize_field_softmax(cap.capture_edge(FieldSoftmax().edge, {})) == \
        cap.FieldSoftmaxPattern("score", "value")


def test_graph_constructors_match_reference(golden):
    src = torch.from_numpy(golden["coo_src"])
    dst = torch.from_numpy(golden["coo_dst"])
    g = tg.Graph.from_coo(src, dst, num_src=23, num_dst=17)
    row_ptr, col = g.resolve_csr()
    assert np.array_equal(row_ptr.numpy(), golden["coo_row_ptr"])
    assert np.array_equal(col.numpy(), golden["coo_col"])
    assert np.array_equal(g.destination_index().numpy(), golden["coo_destination"])
    assert list(g.degree_bounds()) == golden["coo_degree_bounds"].tolist()
    t = g.transpose()
    t_ptr, t_col = t.resolve_csr()
    assert np.array_equal(t_ptr.numpy(), golden["coo_t_ptr"])
    assert np.array_equal(t_col.numpy(), golden["coo_t_col"])
    # packed causal relation: cu_seqlens == cat of triangular blocks
    cu = torch.from_numpy(golden["attn_cu"])
    a = tg.Graph.cu_seqlens(cu, causal=True)
    b = tg.Graph.cat([tg.Graph.triangular(int(n)) for n in cu.diff()])
    for graph in (a, b):
        rp, ci = graph.resolve_csr()
        assert np.array_equal(rp.numpy(), golden["attn_row_ptr"])
        assert np.array_equal(ci.numpy(), golden["attn_col"])
    assert tg.Graph.triangular(4).resolve_csr()[0].tolist() == [0, 1, 3, 6, 10]
    r = tg.Graph.regular(5, 2)
    assert r.resolve_csr()[1].tolist() == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4]
    with pytest.raises(ValueError):
        tg.Graph.from_csr(torch.tensor([0, 2]), torch.tensor([0, 5]), num_src=3, validate="full")
    with pytest.raises(TypeError):
        tg.Graph.from_csr(torch.tensor([0.0, 1.0]), torch.tensor([0]))


def test_partition_model_matches_reference(golden):
    for entities, world, rank, b, e in golden["owned_range_table"].tolist():
        assert dist.owned_range(entities, world, rank) == (b, e)
    for entity, entities, world, owner in golden["destination_owner_table"].tolist():
        assert dist.destination_owner(entity, entities, world) == owner
    row_ptr, col = golden["halo_row_ptr"], golden["halo_col"]
    n = row_ptr.size - 1
    for world in (2, 3, 4):
        maps = [dist.derive_halo_map(row_ptr, col, num_entities=n, world_size=world, rank=r) for r in range(world)]
        for r, m in enumerate(maps):
            requests = [[i for i in maps[p].ghost_ids if m.owned_begin <= i < m.owned_end] for p in range(world)]
            full = dist.derive_halo_map(row_ptr, col, num_entities=n, world_size=world, rank=r,
                                        peer_requests=requests)
            assert list(full.ghost_ids) == golden[f"halo_w{world}_r{r}_ghosts"].tolist()
            assert [full.owned_begin, full.owned_end] == golden[f"halo_w{world}_r{r}_range"].tolist()
            assert full.bytes_for(4, 64) == int(golden[f"halo_w{world}_r{r}_bytes"])
            for peer, ids in full.receive_from:
                assert list(ids) == golden[f"halo_w{world}_r{r}_recv{peer}"].tolist()
            for peer, ids in full.send_to:
                assert list(ids) == golden[f"halo_w{world}_r{r}_send{peer}"].tolist()
            assert len(full.receive_from) == sum(f"halo_w{world}_r{r}_recv{p}" in golden for p in range(world))
    assert dist.partition_bounds(10, 3) == [0, 4, 7, 10]
    rp = torch.tensor([0, 90, 95, 96, 98, 100])
    assert dist.partition_bounds(5, 2, row_ptr=rp, balance="edges") == [0, 1, 5]


def test_synthetic_rmat_is_deterministic():
    from baseline import synthetic as syn

    a = syn.rmat_csr(10, 8, seed=7)
    b = syn.rmat_csr(10, 8, seed=7)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    row_ptr, col = a
    dst = torch.repeat_interleave(torch.arange(1024), row_ptr.diff())
    key = dst * 1024 + col
    assert torch.equal(key, torch.unique(key))            # sorted by (dst, src), no duplicates
    rev = col * 1024 + dst
    assert torch.equal(torch.sort(rev).values, key)        # symmetric


def test_degree_histogram_and_locality_signal():
    # ragged CSR with empty rows: degrees 2, 0, 3, 1, 0
    row_ptr = torch.tensor([0, 2, 2, 5, 6, 6])
    col = torch.tensor([0, 4, 1, 2, 3, 3])
    g = tg.Graph.from_csr(row_ptr, col, num_src=5)
    assert g.degree_histogram() == (2, 1, 1, 1)
    assert sum(d * c for d, c in enumerate(g.degree_histogram())) == col.numel()
    # every sampled slot: |col - row| = 0, 4, 1, 0, 1, 0 -> mean 1.0, over 5 endpoints
    assert abs(g.source_index_span_ratio() - 1.0 / 5) < 1e-12
    assert tg.Graph.triangular(4).degree_histogram() == (0, 1, 1, 1, 1)
    assert tg.Graph.dense(3, 2).degree_histogram() == (0, 0, 0, 2)
    rows = torch.arange(1000).repeat_interleave(3)
    banded = (rows + torch.arange(3).repeat(1000)).clamp(max=999)      # row i reads i, i+1, i+2: index-local
    local = tg.Graph.from_csr(torch.arange(0, 3001, 3), banded, num_src=1000)
    assert local.source_index_span_ratio() < 0.01
    gen = torch.Generator().manual_seed(0)
    random_col = torch.randint(0, 4096, (4096 * 8,), generator=gen)
    scattered = tg.Graph.from_csr(torch.arange(0, 4096 * 8 + 1, 8), random_col, num_src=4096)
    assert 0.28 < scattered.source_index_span_ratio() < 0.39    # random numbering approaches one third
    hub = tg.Graph.from_csr(torch.tensor([0, 5000]), torch.zeros(5000, dtype=torch.int64), num_src=1)
    with pytest.raises(ValueError):
        hub.degree_histogram()


def test_b200_native_codegen_provider_is_registered():
    from tiga import _native, codegen

    assert "b200-native" in codegen.discover_providers()
    provider = codegen.get_provider("b200-native")
    report = codegen.provider_conformance(provider)
    assert report == {"abi_version": 1, "name": "b200-native", "target_family": "cuda-sm100a", "devices": ("cuda",),
                      "input_ir": "vendor-ir", "artifacts": ("shared-library",), "supports_async": True,
                      "supports_distributed": True}
    # every lowering name resolves to entry points the header declares
    for lowering, entries in codegen.LOWERINGS.items():
        compiled = provider.compile(lowering, target="sm_100a", options={})
        assert compiled.entry_points == entries and all(name in _native.exported_symbols() for name in entries)
    with pytest.raises(NotImplementedError):
        provider.compile("gf-kernel-to-ttir-fixed-csr-weighted-sum", target=None, options={})
    with pytest.raises(NotImplementedError):
        provider.compile("b200-csr-weighted-sum-degree-bucket", target="sm_90a", options={})
    with pytest.raises(ValueError):
        codegen.ProviderCapabilities("x", "y", ("cuda",), "ptx", (), False, False)
    with pytest.raises(LookupError):
        codegen.get_provider("triton")
    with pytest.raises(ValueError):
        codegen.register_provider("b200-native", codegen.provider_factory)


def test_gfg_reader_and_writer_match_the_reference_files(tmp_path):
    """tests/golden/gfg_case/ was written by the unmodified reference's tg.save: this package must
    read it, report what the reference's tg.load reports, and write the same bytes."""
    import filecmp
    import json

    case = os.path.join(ROOT, "tests", "golden", "gfg_case")
    expected = json.load(open(os.path.join(case, "expected.json")))
    row_ptr = [0, 2, 2, 5, 6, 6, 9]
    col_idx = [0, 4, 1, 2, 3, 3, 0, 2, 4]
    for name, dtype in (("plain_i32.gfg", torch.int32), ("fields_i64.gfg", torch.int64)):
        graph = tg.load(os.path.join(case, name))
        want = expected[name]
        assert (graph.schema.realization, graph.schema.origin) == (want["realization"], want["origin"])
        assert (graph.num_src, graph.num_dst, graph.num_edges) == (want["num_src"], want["num_dst"], want["num_edges"])
        assert [list(part) for part in graph.paged_rows(2, 5)] == want["paged_rows_2_5"]
        rows, cols, first = graph.paged_page(3, 6)
        assert [list(rows), list(cols), first] == want["paged_page_3_6"]
        assert "backing=nvme:" in graph.explain() and graph.schema.index_dtype == dtype
        loaded_rows, loaded_cols = graph.resolve_csr()
        assert loaded_rows.tolist() == row_ptr and loaded_cols.tolist() == col_idx and loaded_rows.dtype == dtype
    stored = tg.load(os.path.join(case, "fields_i64.gfg"))
    fields = {role: stored.fields(role) for role in ("src", "dst", "edge")}
    assert fields["src"]["x"].shape == (5, 3) and fields["src"]["x"][2].tolist() == [1.0, 2.0, 3.0]
    assert fields["edge"]["weight"].tolist() == [1.0 + 0.125 * e for e in range(9)]
    # writer: same files, byte for byte (manifest text included)
    plain = tg.Graph.from_csr(torch.tensor(row_ptr, dtype=torch.int32), torch.tensor(col_idx, dtype=torch.int32),
                              num_src=5, validate="full")
    tg.save(plain, tmp_path / "plain_i32.gfg")
    wide = tg.Graph.from_csr(torch.tensor(row_ptr), torch.tensor(col_idx), num_src=5)
    tg.save(wide, tmp_path / "fields_i64.gfg", fields=fields)
    for name in ("plain_i32.gfg", "fields_i64.gfg"):
        listing = filecmp.dircmp(os.path.join(case, name), tmp_path / name)
        assert not listing.left_only and not listing.right_only and not listing.diff_files, listing.report()
        sub = filecmp.dircmp(os.path.join(case, name, "fields"), tmp_path / name / "fields") if name.startswith("fields") else None
        assert sub is None or (not sub.diff_files and not sub.left_only and not sub.right_only)
    # a paged graph is copied without materialising it; overwriting and corrupt files are refused
    tg.save(tg.load(tmp_path / "plain_i32.gfg"), tmp_path / "copy.gfg")
    assert tg.load(tmp_path / "copy.gfg").paged_rows(2, 5) == tg.load(tmp_path / "plain_i32.gfg").paged_rows(2, 5)
    with pytest.raises(FileExistsError):
        tg.save(plain, tmp_path / "copy.gfg")
    (tmp_path / "copy.gfg" / "col_idx.bin").write_bytes(b"")
    with pytest.raises(ValueError, match="col_idx size"):
        tg.load(tmp_path / "copy.gfg")
    with pytest.raises(ValueError):
        tg.save(plain, tmp_path / "again.gfg", overwrite=True)


def test_edge_expression_compiles_to_a_register_program():
    from tiga import capture as cap, edge_program as ep

    class Flux(tg.MessagePassing):
        reducer = tg.sum()

        def edge(self, src, dst, edge, k, gain):
            s = edge.weight * (src.u - dst.u) * gain
            return tg.math.maximum(s, k * s) / 2.0 + (-src.u).exp()

    staged = cap.capture_edge(Flux().edge, {"k": 0.2, "gain": torch.ones(4)})
    program = ep.compile_expression(staged)
    assert [o.role for o in program.operands] == ["edge", "src", "dst", "param"]
    assert program.ops.count(ep.OP_LOAD) == 4            # `s` and src.u are used twice, loaded once
    assert program.constants == (0.2, 2.0)
    for i, op in enumerate(program.ops):                 # operands are earlier instructions
        if op not in (ep.OP_LOAD, ep.OP_CONST):
            assert program.lhs[i] < i and program.rhs[i] <= i
    # shapes: fields share a rank, tensor parameters broadcast from the right
    shape, moduli = ep.bind(program, [torch.zeros(7, 1), torch.zeros(5, 4), torch.zeros(5, 4), torch.ones(4)])
    assert shape == (4,) and moduli == (1, 0, 0, 0)
    shape, moduli = ep.bind(program, [torch.zeros(7, 1, 1), torch.zeros(5, 3, 4), torch.zeros(5, 3, 4), torch.ones(4)])
    assert shape == (3, 4) and moduli == (1, 0, 0, 4)
    with pytest.raises(NotImplementedError, match="same number of dimensions"):
        ep.bind(program, [torch.zeros(7), torch.zeros(5, 4), torch.zeros(5, 4), torch.ones(4)])
    struct = ep.make_struct(program, 4, (1, 0, 0, 0))
    assert struct.num_instructions == len(program.ops) and struct.width == 4
    # a reduction over features is not element-wise: no program
    assert ep.compile_expression(cap.capture_edge(lambda src, dst, edge: (src.x * dst.x).sum(-1), {})) is None


def test_repeat_write_back_stages_values_that_alias_the_carried_buffers():
    from tiga import control

    a, b = torch.arange(4.0), torch.arange(4.0) * 10
    static = (a.clone(), b.clone())
    control._write_back(static, (static[1], static[0]))                 # a swap hands back the inputs themselves
    assert torch.equal(static[0], b) and torch.equal(static[1], a)
    control._write_back(static, (static[0][:], static[0] + 1))           # a view of a carried buffer
    assert torch.equal(static[0], b) and torch.equal(static[1], b + 1)
    # the host loop (no CUDA graph) gives the same swap semantics
    x, y = tg.repeat((a, b), lambda p, q: (q, p), iterations=5)
    assert torch.equal(x, b) and torch.equal(y, a)
