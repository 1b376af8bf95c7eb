"""Unit tests of the tensor and core layers on the CPU, one behaviour per test, in the spirit of the
reference's in-module tests (crates/axonml-tensor/src/{ops,creation,view,sparse,shape}.rs,
crates/axonml-core/src/{storage,dtype,device,error,allocator}.rs)."""
import math

import pytest
import torch

import axonml_b200.tensor as T
from axonml_b200 import core
from axonml_b200.core import DType, Device, Storage
from axonml_b200.tensor import ops, shape as SH, view as V
from axonml_b200.tensor.sparse import SparseCOO, SparseCSR, SparseFormat, SparseTensor


# ------------------------------------------------------------------------------------------- ops
def test_softmax_rows_sum_to_one_and_keep_order():
    x = T.from_vec([1.0, 2.0, 3.0, 1.0, 1.0, 1.0], [2, 3])
    y = ops.softmax(x, -1)
    assert torch.allclose(y.sum(-1), torch.ones(2))
    assert y[0, 2] > y[0, 1] > y[0, 0]
    assert torch.allclose(y[1], torch.full((3,), 1 / 3))


def test_log_softmax_is_log_of_softmax():
    x = torch.randn(4, 7)
    assert torch.allclose(ops.log_softmax(x, -1), ops.softmax(x, -1).log(), atol=1e-6)


def test_clamp_and_one_sided_clamps():
    x = T.from_vec([-2.0, -0.5, 0.5, 2.0])
    assert ops.clamp(x, -1.0, 1.0).tolist() == [-1.0, -0.5, 0.5, 1.0]
    assert ops.clamp_min(x, 0.0).tolist() == [0.0, 0.0, 0.5, 2.0]
    assert ops.clamp_max(x, 0.0).tolist() == [-2.0, -0.5, 0.0, 0.0]


def test_leaky_relu_and_elu_negative_branch():
    x = T.from_vec([-2.0, 0.0, 3.0])
    assert ops.leaky_relu(x, 0.1).tolist() == pytest.approx([-0.2, 0.0, 3.0])
    assert ops.elu(x, 1.0).tolist() == pytest.approx([math.exp(-2) - 1, 0.0, 3.0])


@pytest.mark.parametrize("name,ref", [
    ("neg", torch.neg), ("abs", torch.abs), ("exp", torch.exp), ("tanh", torch.tanh), ("sigmoid", torch.sigmoid),
    ("relu", torch.relu), ("square", torch.square), ("silu", torch.nn.functional.silu)])
def test_unary_ops_match_torch(name, ref):
    x = torch.randn(33)
    assert torch.allclose(getattr(ops, name)(x), ref(x), atol=1e-6)


def test_sqrt_ln_pow_on_positive_values():
    x = torch.rand(17) + 0.5
    assert torch.allclose(ops.sqrt(x), x.sqrt())
    assert torch.allclose(ops.ln(x), x.log()) and torch.allclose(ops.log(x), x.log())
    assert torch.allclose(ops.pow(x, 3.0), x ** 3, atol=1e-6)
    assert torch.allclose(ops.pow(x, torch.full_like(x, 0.5)), x.sqrt(), atol=1e-6)


def test_gelu_matches_one_of_the_two_usual_forms():
    x = torch.linspace(-3, 3, 25)
    y = ops.gelu(x)
    exact, tanh = torch.nn.functional.gelu(x), torch.nn.functional.gelu(x, approximate="tanh")
    assert min(float((y - exact).abs().max()), float((y - tanh).abs().max())) < 1e-5


def test_comparisons_return_boolean_masks():
    a, b = T.from_vec([1.0, 2.0, 3.0]), T.from_vec([3.0, 2.0, 1.0])
    assert ops.eq(a, b).tolist() == [False, True, False]
    assert ops.lt(a, b).tolist() == [True, False, False]
    assert ops.gt(a, b).tolist() == [False, False, True]
    assert ops.where_cond(ops.gt(a, b), a, b).tolist() == [3.0, 2.0, 3.0]


def test_binary_ops_broadcast():
    a, b = T.ones(2, 3), T.from_vec([1.0, 2.0, 3.0])
    assert ops.add(a, b).tolist() == [[2, 3, 4], [2, 3, 4]]
    assert ops.sub(a, b).tolist() == [[0, -1, -2], [0, -1, -2]]
    assert ops.mul(a, b.unsqueeze(0)).shape == (2, 3)
    assert ops.div(a, T.full([2, 1], 2.0)).tolist() == [[0.5] * 3] * 2
    assert ops.add_scalar(a, 2.0).sum().item() == 18 and ops.mul_scalar(a, -1.0).sum().item() == -6


def test_topk_largest_and_smallest():
    x = T.from_vec([3.0, 1.0, 4.0, 1.5, 9.0])
    v, i = ops.topk(x, 2)
    assert v.tolist() == [9.0, 4.0] and i.tolist() == [4, 2]
    v, i = ops.topk(x, 2, largest=False)
    assert v.tolist() == [1.0, 1.5] and i.tolist() == [1, 3]


def test_sort_and_argsort_both_directions():
    x = T.from_vec([3.0, 1.0, 2.0])
    v, i = ops.sort(x)
    assert v.tolist() == [1.0, 2.0, 3.0] and i.tolist() == [1, 2, 0]
    v, _ = ops.sort(x, descending=True)
    assert v.tolist() == [3.0, 2.0, 1.0]
    assert ops.argsort(x, descending=True).tolist() == [0, 2, 1]


def test_nonzero_one_and_two_dimensions():
    assert ops.nonzero(T.from_vec([0.0, 1.0, 0.0, 2.0])).flatten().tolist() == [1, 3]
    assert ops.nonzero(T.from_vec([0.0, 1.0, 2.0, 0.0], [2, 2])).tolist() == [[0, 1], [1, 0]]


def test_unique_is_sorted_and_deduplicated():
    assert ops.unique(T.from_vec([3.0, 1.0, 3.0, 2.0, 1.0])).tolist() == [1.0, 2.0, 3.0]


def test_flip_and_roll():
    x = T.from_vec([1.0, 2.0, 3.0, 4.0], [2, 2])
    assert ops.flip(x, [0]).tolist() == [[3, 4], [1, 2]] and ops.flip(x, [0, 1]).tolist() == [[4, 3], [2, 1]]
    v = T.arange(5)
    assert ops.roll(v, 2, 0).tolist() == [3, 4, 0, 1, 2] and ops.roll(v, -1, 0).tolist() == [1, 2, 3, 4, 0]


def test_scatter_gather_masked():
    src = T.from_vec([1.0, 2.0, 3.0], [1, 3])
    idx = torch.tensor([[2, 0, 1]])
    out = ops.scatter(T.zeros(1, 3), 1, idx, src)
    assert out.tolist() == [[2.0, 3.0, 1.0]]
    assert ops.gather(out, 1, idx).tolist() == [[1.0, 2.0, 3.0]]
    m = torch.tensor([[True, False, True]])
    assert ops.masked_select(out, m).tolist() == [2.0, 1.0]
    assert ops.masked_fill(out, m, -1.0).tolist() == [[-1.0, 3.0, -1.0]]


def test_reductions():
    x = T.from_vec([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3])
    assert ops.sum(x).item() == 21 and ops.sum(x, 0).tolist() == [5, 7, 9] and ops.sum(x, 1, True).shape == (2, 1)
    assert ops.mean(x).item() == 3.5 and ops.prod(x).item() == 720
    assert ops.max(x).item() == 6 and ops.min(x).item() == 1
    assert ops.argmax(x).item() == 5 and ops.argmin(x, 1).tolist() == [0, 0]
    assert ops.var_dim(x, 1).tolist() == pytest.approx([2 / 3, 2 / 3])


def test_matmul_shapes_vector_matrix_batched():
    a, b = torch.randn(3, 4), torch.randn(4, 5)
    assert torch.allclose(ops.matmul(a, b), a @ b, atol=1e-5)
    assert ops.matmul(torch.randn(2, 3, 4), torch.randn(2, 4, 6)).shape == (2, 3, 6)
    assert ops.matmul(a, torch.randn(4)).shape == (3,)
    assert ops.dot(T.from_vec([1.0, 2.0, 3.0]), T.from_vec([4.0, 5.0, 6.0])).item() == 32


def test_cat_and_stack():
    a, b = T.ones(2, 3), T.zeros(2, 3)
    assert ops.cat([a, b], 0).shape == (4, 3) and ops.cat([a, b], 1).shape == (2, 6)
    s = ops.stack([a, b], 0)
    assert s.shape == (2, 2, 3) and s[1].sum().item() == 0


# -------------------------------------------------------------------------------------- creation
def test_zeros_ones_full_shapes_and_values():
    assert T.zeros(2, 3).tolist() == [[0.0] * 3] * 2 and T.ones(4).sum().item() == 4
    f = T.full([2, 2], 7.5)
    assert f.shape == (2, 2) and f.unique().tolist() == [7.5]
    assert T.zeros(2, dtype=DType.I64).dtype == torch.int64


def test_eye_and_diag():
    assert T.eye(3).tolist() == [[1, 0, 0], [0, 1, 0], [0, 0, 1]]
    assert T.diag([1.0, 2.0]).tolist() == [[1, 0], [0, 2]]


def test_rand_is_in_unit_interval_and_randn_is_centred():
    torch.manual_seed(0)
    r = T.rand(10000)
    assert 0.0 <= float(r.min()) and float(r.max()) < 1.0
    n = T.randn(20000)
    assert abs(float(n.mean())) < 0.05 and abs(float(n.std()) - 1.0) < 0.05
    u = T.uniform([5000], -2.0, 3.0)
    assert -2.0 <= float(u.min()) and float(u.max()) <= 3.0
    k = T.randint(3, 7, [1000])
    assert int(k.min()) >= 3 and int(k.max()) < 7


def test_arange_linspace_logspace():
    assert T.arange(5).tolist() == [0, 1, 2, 3, 4] and T.arange(1, 7, 2).tolist() == [1, 3, 5]
    assert T.linspace(0.0, 1.0, 5).tolist() == pytest.approx([0, 0.25, 0.5, 0.75, 1.0])
    assert T.logspace(0.0, 2.0, 3).tolist() == pytest.approx([1, 10, 100])


def test_like_constructors_copy_shape_and_dtype():
    x = torch.randn(3, 2, dtype=torch.float64)
    for t, v in ((T.zeros_like(x), 0.0), (T.ones_like(x), 1.0), (T.full_like(x, 4.0), 4.0)):
        assert t.shape == x.shape and t.dtype == x.dtype and t.unique().tolist() == [v]


def test_from_vec_rejects_a_wrong_shape():
    assert T.from_vec([1.0, 2.0, 3.0, 4.0], [2, 2])[1, 0].item() == 3.0
    with pytest.raises(RuntimeError):
        T.from_vec([1.0, 2.0, 3.0], [2, 2])


# ----------------------------------------------------------------------------------------- views
def test_slice_select_narrow_are_views():
    x = T.arange(12).reshape(3, 4)
    assert V.slice_dim0(x, 1, 3).tolist() == [[4, 5, 6, 7], [8, 9, 10, 11]]
    assert V.select(x, 1, 2).tolist() == [2, 6, 10]
    n = V.narrow(x, 1, 1, 2)
    assert n.tolist() == [[1, 2], [5, 6], [9, 10]]
    assert n.data_ptr() == x.data_ptr() + x.element_size()


def test_chunk_and_split_cover_the_tensor():
    x = T.arange(10)
    parts = V.chunk(x, 3)
    assert [len(p) for p in parts] == [4, 4, 2] and torch.cat(parts).equal(x)
    assert [p.tolist() for p in V.split(x, 4)] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]


def test_reshape_transpose_permute_squeeze():
    x = T.arange(6).reshape(2, 3)
    assert V.reshape(x, [3, 2]).tolist() == [[0, 1], [2, 3], [4, 5]]
    assert V.transpose(x, 0, 1).tolist() == [[0, 3], [1, 4], [2, 5]] and V.t(x).shape == (3, 2)
    assert V.permute(torch.zeros(2, 3, 4), [2, 0, 1]).shape == (4, 2, 3)
    assert V.squeeze(torch.zeros(1, 3, 1)).shape == (3,) and V.squeeze(torch.zeros(1, 3, 1), 0).shape == (3, 1)
    assert V.unsqueeze(x, 0).shape == (1, 2, 3) and V.flatten(torch.zeros(2, 3, 4), 1).shape == (2, 12)
    assert not V.transpose(x, 0, 1).is_contiguous() and V.contiguous(V.transpose(x, 0, 1)).is_contiguous()
    assert V.expand(torch.ones(1, 3), [4, 3]).shape == (4, 3)


def test_slice_specs_index_range_all_newaxis():
    x = T.arange(24).reshape(2, 3, 4)
    S = T.SliceSpec
    assert T.slice_with(x, [S.Index(1), S.All, S.range(1, 3)]).tolist() == x[1, :, 1:3].tolist()
    assert T.slice_with(x, [S.All, S.Index(-1)]).tolist() == x[:, -1].tolist()
    assert T.slice_with(x, [S.NewAxis, S.Index(0)]).shape == (1, 3, 4)
    assert T.slice_with(x, [S.All, S.All, S.range_step(0, 4, 2)]).tolist() == x[:, :, 0:4:2].tolist()
    assert T.slice_with(x, [S.from_(1)]).shape == (1, 3, 4) and T.slice_with(x, [S.All, S.to(2)]).shape == (2, 2, 4)


# ------------------------------------------------------------------------------ shape arithmetic
def test_numel_and_contiguous_strides():
    assert SH.numel([2, 3, 4]) == 24 and SH.numel([]) == 1 and SH.numel([5, 0]) == 0
    assert list(SH.contiguous_strides([2, 3, 4])) == [12, 4, 1] and list(SH.contiguous_strides([])) == []
    assert SH.is_contiguous([2, 3], [3, 1]) and not SH.is_contiguous([2, 3], [1, 2])


def test_broadcast_shape_rules():
    assert list(SH.broadcast_shape([2, 1, 4], [3, 1])) == [2, 3, 4]
    assert list(SH.broadcast_shape([5], [])) == [5]
    assert SH.can_broadcast([4, 1], [1, 6]) and not SH.can_broadcast([2, 3], [4, 3])
    with pytest.raises(core.BroadcastError):
        SH.broadcast_shape([2, 3], [4, 3])
    assert list(SH.broadcast_strides([3, 1], [1, 1], [2, 3, 4])) == [0, 1, 0]


def test_reshape_infers_one_dimension_and_checks_the_count():
    assert list(SH.reshape([2, 6], [3, -1])) == [3, 4] and list(SH.reshape([4], [2, 2])) == [2, 2]
    with pytest.raises(core.InvalidOperation):
        SH.reshape([2, 6], [5, -1])
    with pytest.raises(core.InvalidOperation):
        SH.reshape([2, 6], [-1, -1])
    with pytest.raises(core.ShapeMismatch):
        SH.reshape([2, 6], [5, 2])


def test_squeeze_unsqueeze_transpose_of_shapes():
    assert list(SH.squeeze([1, 3, 1])) == [3] and list(SH.squeeze([1, 3, 1], 2)) == [1, 3]
    assert list(SH.squeeze([2, 3], 0)) == [2, 3]
    assert list(SH.unsqueeze([2, 3], 1)) == [2, 1, 3] and list(SH.unsqueeze([2, 3], 2)) == [2, 3, 1]
    with pytest.raises(core.InvalidDimension):
        SH.unsqueeze([2, 3], 3)
    assert list(SH.transpose_shape([2, 3, 4], 0, 2)) == [4, 3, 2] and list(SH.transpose_strides([12, 4, 1], 0, 2)) == [1, 4, 12]


def test_normalize_dim_and_index_round_trip():
    assert SH.normalize_dim(-1, 3) == 2 and SH.normalize_dim(1, 3) == 1
    with pytest.raises(core.InvalidDimension):
        SH.normalize_dim(3, 3)
    strides = SH.contiguous_strides([2, 3, 4])
    for lin in (0, 5, 17, 23):
        idx = SH.unravel_index(lin, [2, 3, 4])
        assert SH.linear_index(idx, strides) == lin
    SH.validate_indices([1, 2, 3], [2, 3, 4])
    with pytest.raises(core.IndexOutOfBounds):
        SH.validate_indices([1, 3, 0], [2, 3, 4])


# ---------------------------------------------------------------------------------------- sparse
def _coo():
    return SparseCOO.from_coo_2d([0, 1, 2, 0], [0, 2, 1, 2], [1.0, 2.0, 3.0, 4.0], [3, 3])


def test_sparse_coo_creation_and_dense_form():
    c = _coo()
    assert c.nnz() == 4 and c.density() == pytest.approx(4 / 9)
    assert c.to_dense().tolist() == [[1, 0, 4], [0, 0, 2], [0, 3, 0]]
    assert c.transpose().to_dense().equal(c.to_dense().t())


def test_sparse_coo_coalesce_adds_duplicates():
    c = SparseCOO.from_coo_2d([0, 0, 1], [1, 1, 0], [1.0, 2.0, 5.0], [2, 2]).coalesce()
    assert c.nnz() == 2 and c.to_dense().tolist() == [[0, 3], [5, 0]]


def test_sparse_csr_rows_matvec_and_conversion():
    d = torch.tensor([[1.0, 0, 4], [0, 0, 2], [0, 3, 0]])
    r = SparseCSR.from_dense(d)
    assert r.nnz() == 4 and r.nrows() == 3 and r.ncols() == 3 and r.crow.tolist() == [0, 2, 3, 4]
    x = torch.tensor([1.0, 2.0, 3.0])
    assert torch.allclose(r.matvec(x), d @ x) and torch.allclose(_coo().matvec(x), d @ x)
    assert _coo().to_csr().to_dense().equal(d) and r.to_coo().to_dense().equal(d)
    b = torch.randn(3, 5)
    assert torch.allclose(r.matmul_dense(b), d @ b, atol=1e-6) and torch.allclose(_coo().matmul_dense(b), d @ b, atol=1e-6)


def test_sparse_tensor_constructors_and_scalar_product():
    d = torch.tensor([[0.0, 2.0], [0.05, 0.0]])
    s = SparseTensor.from_dense(d, 0.1)
    assert s.nnz() == 1 and s.shape() == (2, 2) and s.density() == 0.25
    assert SparseTensor.eye(3).to_dense().equal(torch.eye(3))
    assert SparseTensor.diag([1.0, 2.0]).to_dense().tolist() == [[1, 0], [0, 2]]
    assert s.mul_scalar(3.0).to_dense().tolist() == [[0, 6], [0, 0]]
    m = SparseTensor.from_dense(torch.tensor([[1.0, 0], [0, 2.0]]))
    assert m.matmul(torch.ones(2, 2)).tolist() == [[1, 1], [2, 2]] and m.matvec(torch.ones(2)).tolist() == [1, 2]
    assert m.as_format(SparseFormat.CSR).format() == SparseFormat.CSR and m.as_format(SparseFormat.COO).format() == SparseFormat.COO


# --------------------------------------------------------------------------------------- storage
def test_storage_zeros_from_vec_len_and_bytes():
    z = Storage.zeros(5)
    assert z.len() == 5 and not z.is_empty() and z.size_bytes() == 20 and z.as_slice().tolist() == [0.0] * 5
    s = Storage.from_vec([1.0, 2.0, 3.0])
    assert s.as_slice().tolist() == [1.0, 2.0, 3.0] and s.device().is_cpu()
    assert Storage.zeros(0).is_empty()


def test_storage_slice_shares_memory_and_checks_bounds():
    s = Storage.from_vec([1.0, 2.0, 3.0, 4.0, 5.0])
    v = s.slice(1, 3)
    assert v.len() == 3 and v.offset() == 1 and v.as_slice().tolist() == [2.0, 3.0, 4.0]
    v.as_slice_mut()[0] = 9.0
    assert s.as_slice()[1].item() == 9.0
    with pytest.raises((core.IndexOutOfBounds, IndexError, ValueError)):
        s.slice(3, 5)


def test_storage_deep_copy_and_copy_from():
    s = Storage.from_vec([1.0, 2.0])
    d = s.deep_copy()
    d.as_slice_mut()[0] = 7.0
    assert s.as_slice()[0].item() == 1.0 and d.is_unique()
    t = Storage.zeros(2)
    t.copy_from(s)
    assert t.as_slice().tolist() == [1.0, 2.0]
    with pytest.raises(core.Error):
        Storage.zeros(3).copy_from(s)


def test_storage_guards_release_on_drop():
    s = Storage.from_vec([1.0, 2.0])
    with s.write() as w:
        w[1] = 5.0
    with s.read() as r:
        assert r.tensor().tolist() == [1.0, 5.0]


# ------------------------------------------------------------------------- dtype, device, errors
def test_dtype_sizes_and_groups():
    assert DType.F32.size_of() == 4 and DType.F64.size_of() == 8 and DType.BF16.size_of() == 2 and DType.Bool.size_of() == 1
    assert DType.F16.is_float() and not DType.I32.is_float() and DType.I32.is_integer() and DType.I8.is_signed()
    assert not DType.U8.is_signed() and not DType.Bool.is_integer()
    assert DType.default_float() == DType.F32 and DType.default_int() == DType.I64
    for dt in DType:
        assert DType.from_torch(dt.to_torch()) == dt
    assert core.as_torch_dtype("bf16") == torch.bfloat16 and str(DType.F32) == "f32"


def test_scalar_tower_constants():
    assert core.Scalar.of(DType.Bool).dtype() == DType.Bool and core.Scalar.accepts(torch.int8)
    assert core.Numeric.accepts(DType.I32) and not core.Numeric.accepts(DType.Bool)
    assert core.Float.accepts(DType.BF16) and not core.Float.accepts(DType.I64)
    with pytest.raises(TypeError):
        core.Float.of(DType.I32)
    i8 = core.Numeric.of(DType.I8)
    assert (i8.ZERO, i8.ONE, i8.min_value(), i8.max_value()) == (0, 1, -128, 127)
    f32 = core.Float.of(torch.float32)
    assert f32.EPSILON == pytest.approx(2 ** -23) and f32.INFINITY == float("inf") and math.isnan(f32.NAN)
    assert f32.max_value() == pytest.approx(3.4028235e38) and 0 < f32.MIN_POSITIVE < 1e-37


def test_device_parse_display_and_defaults():
    assert Device.Cpu().is_cpu() and not Device.Cpu().is_gpu() and Device.Cpu().is_available()
    assert Device.parse("cuda:1") == Device.Cuda(1) and Device.parse("cpu") == Device.Cpu()
    assert Device.Cuda(2).device_index() == 2 and Device.Cuda(0).is_gpu()
    assert str(Device.Cuda(1).to_torch()) == "cuda:1" and Device.from_torch(torch.device("cpu")) == Device.Cpu()
    caps = Device.Cpu().capabilities()
    assert caps.supports_f64 and caps.total_memory > 0 and caps.name
    for unavailable in (Device.Metal(), Device.Vulkan(), Device.Wgpu()):
        assert not unavailable.is_available()
    assert core.vulkan_device_count() == 0 and core.default_device() in (Device.Cpu(), Device.Cuda(0))


def test_error_variants_carry_their_fields_and_compare():
    e = core.ShapeMismatch([2, 3], [3, 2])
    assert isinstance(e, core.Error) and "[2, 3]" in str(e) and "[3, 2]" in str(e)
    assert "3" in str(core.InvalidDimension(3, 2)) and "cuda" in str(core.DeviceNotAvailable("cuda:7")).lower()
    assert isinstance(core.Error.shape_mismatch([1], [2]), core.ShapeMismatch)
    assert isinstance(core.Error.invalid_operation("x"), core.InvalidOperation) and "x" in str(core.Error.internal("x"))
    assert str(core.ShapeMismatch([1], [2])) == str(core.ShapeMismatch([1], [2]))


def test_default_allocator_allocates_zeroed_host_memory():
    a = core.DefaultAllocator()
    t = a.allocate(16)
    assert t.numel() == 16 and t.dtype == torch.float32
    a.deallocate(t)
    assert a.total_memory() > 0 and 0 < a.free_memory() <= a.total_memory()


def test_cpu_backend_elementwise_gemm_and_reductions():
    B = core.CpuBackend
    a, b = torch.tensor([1.0, -2.0, 3.0]), torch.tensor([4.0, 5.0, -6.0])
    assert B.add(a, b).tolist() == [5, 3, -3] and B.mul(a, b).tolist() == [4, -10, -18] and B.relu(a).tolist() == [1, 0, 3]
    assert float(B.sum(a)) == 2 and float(B.max(a)) == 3 and float(B.min(a)) == -2 and int(B.argmax(a)) == 2
    assert float(B.dot(a, b)) == -24
    x, y = torch.randn(4, 6), torch.randn(6, 5)
    c = torch.zeros(4, 5)
    B.sgemm(c, x, y, 4, 5, 6)
    assert torch.allclose(c, x @ y, atol=1e-5)
    c2 = torch.ones(4, 5)
    B.sgemm(c2, x, y, 4, 5, 6, alpha=2.0, beta=3.0)
    assert torch.allclose(c2, 2 * (x @ y) + 3, atol=1e-5)
    d = torch.empty(3)
    B.fill(d, 2.5)
    assert d.tolist() == [2.5] * 3
    B.fill_zeros(d)
    assert d.sum().item() == 0
    assert B.transpose(x).shape == (6, 4) and B().name() and B().backend_type() == core.BackendType.Cpu


def test_launch_config_covers_every_element():
    for n in (1, 255, 256, 257, 10 ** 6):
        cfg = core.launch_config(n)
        assert cfg.block_dim == (core.BLOCK_SIZE, 1, 1) and cfg.grid_dim[0] * core.BLOCK_SIZE >= n > (cfg.grid_dim[0] - 1) * core.BLOCK_SIZE
